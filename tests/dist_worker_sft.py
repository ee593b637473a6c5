"""Worker for the distributed SFT equivalence test: trains the tiny Qwen2 config on packed synthetic
token batches and writes the loss / grad-norm trajectory as JSON (rank 0)."""
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
    model = make_tiny_model("tiny-qwen2", seed=0)
    rows = synthetic_token_batches(1024, 4 * steps, 128, seed=3)
    # "sp2": Ulysses sequence parallelism over both ranks; "cp2": context parallel (gathered K/V); plain DP engine
    optim = "adamw_torch_fused"
    if mode.endswith("+sgd"):  # another update rule on the engine's master slices (sharded under zero2)
        mode, optim = mode[:-4], "sgd"
    sp = 2 if mode in ("sp2", "cp2") else 1
    pc = {"sp_size" if mode == "sp2" else "cp_size": sp} if sp > 1 else None
    mode = "ddp" if sp > 1 else mode
    args = SFTConfig(output_dir=out + "_o", per_device_train_batch_size=4 // (world // sp), max_steps=steps, logging_steps=1,
                     learning_rate=1e-4 if optim != "sgd" else 0.05, optim=optim, optim_args="momentum=0.9", use_cpu=True, save_strategy="no", padding_free=True, shard_mode=mode,
                     parallelism_config=pc,
                     lr_scheduler_type="constant", train_sampling_strategy="sequential", completion_only_loss=True,
                     dataset_kwargs={"skip_prepare_dataset": True}, gradient_checkpointing=mode == "full_shard_stream",
                     max_length=None)
    tr = SFTTrainer(model, args, train_dataset=rows, processing_class=Tok())
    tr.train()
    if D.is_main():
        hist = [{"loss": h["loss"], "grad_norm": h["grad_norm"]} for h in tr.state.log_history if "grad_norm" in h]
        with open(out, "w") as f:
            json.dump(hist, f)
    D.barrier()


if __name__ == "__main__":
    main()
