"""Worker for the expert-parallel equivalence test: SFT of the tiny Qwen3-MoE config, with the experts replicated
(world 1) or split over the ranks (``ep_size`` = world).  Rank 0 writes the loss / grad-norm trajectory and, after a
save, checks that the checkpoint holds every expert."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

from trl_b200.parallel import dist as D
from trl_b200.testing import make_tiny_model, synthetic_token_batches
from trl_b200.trainer.sft_config import SFTConfig
from trl_b200.trainer.sft_trainer import SFTTrainer


class Tok:
    pad_token, eos_token, pad_token_id, eos_token_id, chat_template = "<pad>", "<eos>", 0, 1, None

    def save_pretrained(self, p):
        pass

    def convert_tokens_to_ids(self, t):
        return 1


def main():
    out, mode, steps = sys.argv[1], sys.argv[2], int(sys.argv[3])
    D.init_process_group(use_cpu=True)
    world = D.world_size()
    torch.manual_seed(0)
    model = make_tiny_model("tiny-qwen3-moe", seed=0)
    rows = synthetic_token_batches(1024, 4 * steps, 128, seed=3)
    args = SFTConfig(output_dir=out + "_o", per_device_train_batch_size=4 // world, max_steps=steps, logging_steps=1,
                     learning_rate=1e-4, use_cpu=True, save_strategy="no", padding_free=True, shard_mode=mode,
                     ep_size=world, weight_decay=0.01, lr_scheduler_type="constant", train_sampling_strategy="sequential",
                     completion_only_loss=True, dataset_kwargs={"skip_prepare_dataset": True}, max_length=None)
    tr = SFTTrainer(model, args, train_dataset=rows, processing_class=Tok())
    tr.train()
    if world > 1:
        l0 = model.layers[0]
        assert l0.experts_gate_up.shape[0] == model.config.num_experts // world and l0.ep is not None
    tr.save_model(out + "_ckpt")
    if D.is_main():
        from trl_b200.models.hf_io import load_state_dict_dir

        sd = load_state_dict_dir(out + "_ckpt")
        n_exp = len([k for k in sd if k.startswith("model.layers.0.mlp.experts.") and k.endswith("gate_proj.weight")])
        assert n_exp == model.config.num_experts, n_exp
        hist = [{"loss": h["loss"], "grad_norm": h["grad_norm"]} for h in tr.state.log_history if "grad_norm" in h]
        digest = {k: float(v.double().sum()) for k, v in sd.items() if "experts.3." in k or "experts.0." in k or "gate.weight" in k}
        with open(out, "w") as f:
            json.dump({"hist": hist, "digest": digest}, f)
    D.barrier()


if __name__ == "__main__":
    main()
