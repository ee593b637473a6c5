"""2-GPU worker: TP weight buffers filled straight from full-shard parameter shards equal slices of the full model."""
import copy
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
os.environ["TRL_B200_FULLSHARD_POISON"] = "1"
import torch
import torch.distributed as td

from trl_b200.ops import cuda as K
from trl_b200.parallel import dist as D
from trl_b200.parallel.fullshard import FullShardEngine
from trl_b200.parallel.reshard import WeightResharder
from trl_b200.rollout.tp_engine import TPRolloutEngine
from trl_b200.testing import make_tiny_model


sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _dist_util import Deadline  # noqa: E402


def main():
    D.init_process_group()
    DL = Deadline()  # the ranks leave on their own, between steps, before the parent's limit
    rank = D.rank()
    dev = torch.device("cuda", D.local_rank())
    model = make_tiny_model("tiny-qwen2", dtype=torch.bfloat16, device=dev, hidden_size=512, num_attention_heads=4,
                            num_key_value_heads=2, head_dim=128, intermediate_size=1024, num_hidden_layers=3, seed=0)
    full = copy.deepcopy(model)  # complete reference copy (same seed on both ranks)
    group = td.new_group([0, 1])
    tp = TPRolloutEngine(model, group, max_num_seqs=4, max_model_len=128)
    eng = FullShardEngine(model, copiers=4)  # from here on, remote slices of the layer buckets are NaN
    DL.check()
    for w in tp.w:
        for t in w.values():
            if t is not None:
                t.fill_(float("nan"))
    rs = WeightResharder(eng, tp)
    rs.run()
    torch.cuda.synchronize()
    K.check_status(dev)
    ref_tp = TPRolloutEngine(full, group, max_num_seqs=4, max_model_len=128)  # sliced from the complete copy
    DL.check()
    for a, b in zip(tp.w, ref_tp.w):
        for k in a:
            if a[k] is not None:
                assert torch.equal(a[k], b[k]), (rank, k)
    total = sum(p.numel() * 2 for n, p in full.named_parameters() if n.startswith("layers.") and p.ndim == 2)
    assert abs(rs.bytes - total / 2) < 1e-6 * total  # exactly 1/tp of the layer matrices crossed into this rank
    td.barrier()
    if rank == 0:
        print("RESHARD_OK", rs.n, rs.bytes)
    DL.check()
    td.destroy_process_group()


if __name__ == "__main__":
    main()
