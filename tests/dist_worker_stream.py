"""Worker for the streamed full-shard checkpoint test (gloo): trains 3 steps either straight through or with a
checkpoint after step 2 and a resume in a fresh trainer, and saves the final model (rank 0)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

from trl_b200.parallel import dist as D
from trl_b200.testing import make_tiny_model, synthetic_token_batches
from trl_b200.trainer.sft_config import SFTConfig
from trl_b200.trainer.sft_trainer import SFTTrainer

from dist_worker_sft import Tok


def make(out, mode, steps, save_steps=None):
    torch.manual_seed(0)
    model = make_tiny_model("tiny-qwen2", seed=0)
    rows = synthetic_token_batches(1024, 4 * 3, 128, seed=3)
    args = SFTConfig(output_dir=out, per_device_train_batch_size=4 // D.world_size(), max_steps=steps, logging_steps=1,
                     learning_rate=1e-3, weight_decay=0.1, use_cpu=True, padding_free=True, shard_mode=mode,
                     save_strategy="steps" if save_steps else "no", save_steps=save_steps or 500,
                     lr_scheduler_type="constant", train_sampling_strategy="sequential", completion_only_loss=True,
                     dataset_kwargs={"skip_prepare_dataset": True}, gradient_checkpointing=True, max_length=None,
                     report_to="none")
    return SFTTrainer(model, args, train_dataset=rows, processing_class=Tok())


def main():
    out, mode, variant = sys.argv[1], sys.argv[2], sys.argv[3]
    D.init_process_group(use_cpu=True)
    if variant == "straight":
        tr = make(out, mode, 3)
        tr.train()
    elif variant == "phase1":  # elastic resume, first half: two steps, checkpoint, stop
        tr = make(out, mode, 2, save_steps=2)
        tr.train()
        D.barrier()
        return
    elif variant == "phase2":  # second half, possibly with another world size / shard mode
        tr = make(out, mode, 3)
        tr.train(resume_from_checkpoint=os.path.join(out, "checkpoint-2"))
    else:
        tr = make(out, mode, 2, save_steps=2)
        tr.train()
        D.barrier()
        tr = make(out, mode, 3)
        tr.train(resume_from_checkpoint=os.path.join(out, "checkpoint-2"))
    tr.save_model(os.path.join(out, "final"))
    D.barrier()


if __name__ == "__main__":
    main()
