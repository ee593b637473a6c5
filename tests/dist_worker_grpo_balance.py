"""2 gloo ranks: GRPO with completions dealt to the ranks by length after scoring.  Checks that the exchange keeps
the job's multiset of (completion, advantage) pairs, evens out the token counts, and that training still works."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

from trl_b200 import GRPOConfig, GRPOTrainer
from trl_b200.parallel import dist as D
from trl_b200.testing import make_dataset, make_tiny_model, make_tiny_tokenizer


def reward(completions, completion_ids=None, **kw):
    return [float(sum(ids) % 11) / 11 + 0.01 * len(ids) for ids in completion_ids]


def main():
    out_path, balance = sys.argv[1], sys.argv[2] == "1"
    D.init_process_group()
    tok = make_tiny_tokenizer()
    model = make_tiny_model()
    args = GRPOConfig(output_dir=os.path.join(os.path.dirname(out_path), f"o{D.rank()}"), per_device_train_batch_size=4,
                      gradient_accumulation_steps=2, num_generations=4, max_completion_length=24, max_steps=2,
                      logging_steps=1, learning_rate=1e-3, use_cpu=True, save_strategy="no", report_to="none",
                      loss_type="dapo", beta=0.04, eos_prob_floor=0.08, balance_completions=balance, seed=5)
    tr = GRPOTrainer(model, reward, args, train_dataset=make_dataset("standard_prompt_only", 32), processing_class=tok)
    seen = []
    orig = tr._rebalance_across_ranks

    def spy(p, c, slp, tm, adv, std):
        before = sorted((tuple(ci), round(float(a), 6)) for ci, a in zip(c, adv.tolist()))
        res = orig(p, c, slp, tm, adv, std)
        after = sorted((tuple(ci), round(float(a), 6)) for ci, a in zip(res[1], res[4].tolist()))
        seen.append({"before": before, "after": after, "tok_before": sum(len(x) + len(y) for x, y in zip(p, c)),
                     "tok_after": sum(len(x) + len(y) for x, y in zip(res[0], res[1]))})
        return res

    tr._rebalance_across_ranks = spy
    tr.train()
    allseen = D.gather_object([seen])
    if D.rank() == 0:
        with open(out_path, "w") as f:
            json.dump({"calls": allseen, "log": [h for h in tr.state.log_history if "loss" in h]}, f)
    D.barrier()


if __name__ == "__main__":
    main()
