"""2-GPU worker: full-shard engine (AG fused into the QKV GEMM, stale remote slices poisoned) vs zero2."""
import copy
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
os.environ["TRL_B200_FULLSHARD_POISON"] = "1"
import torch
import torch.distributed as td

from trl_b200.models.decoder import SeqCtx
from trl_b200.ops import cuda as K
from trl_b200.ops import functional as ops
from trl_b200.parallel import dist as D
from trl_b200.parallel.engine import TrainEngine
from trl_b200.parallel.fullshard import FullShardEngine
from trl_b200.testing import make_tiny_model


def run(model, engine, rank, steps=3):
    dev = model.device
    losses = []
    for s in range(steps):
        engine.zero_grad()
        g = torch.Generator().manual_seed(1000 * s + rank)
        ids = torch.randint(0, 1024, (300,), generator=g).to(dev)
        ctx = SeqCtx.from_lengths([120, 180], dev)
        h = model.forward_hidden(ids, ctx)
        tgt = torch.roll(ids, -1)
        loss_sum, _, _, n = ops.lm_head_ce(h, model.lm_head_weight, tgt)
        loss = loss_sum / n
        loss.backward()
        norm = engine.step(1e-3, 1.0)
        losses.append((float(loss), float(norm)))
    return losses


sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _dist_util import Deadline  # noqa: E402


def main():
    D.init_process_group()
    DL = Deadline()  # the ranks leave on their own, between steps, before the parent's limit
    rank = D.rank()
    dev = torch.device("cuda", D.local_rank())
    base = make_tiny_model("tiny-qwen2", dtype=torch.bfloat16, device=dev, hidden_size=512, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=128, intermediate_size=1024, num_hidden_layers=3, seed=0)
    m_fs, m_z2 = copy.deepcopy(base), copy.deepcopy(base)
    e_fs = FullShardEngine(m_fs, copiers=4)
    e_z2 = TrainEngine(m_z2, mode="zero2", use_symm_kernels=True)
    m_fs.train()
    m_z2.train()
    a = run(m_fs, e_fs, rank)
    b = run(m_z2, e_z2, rank)
    torch.cuda.synchronize()
    K.check_status(dev)
    DL.check()
    for (la, na), (lb, nb) in zip(a, b):
        assert abs(la - lb) < 5e-2 and abs(na - nb) < 5e-2 * max(1.0, nb), (a, b)
    e_fs.gather_full_params()
    torch.cuda.synchronize()
    DL.check()
    for (n, p), (_, q) in zip(m_fs.named_parameters(), m_z2.named_parameters()):
        assert torch.isfinite(p.float()).all(), n
        assert torch.allclose(p.float(), q.float(), atol=3e-2, rtol=3e-2), n
    td.barrier()
    if rank == 0:
        print("FULLSHARD_OK", a)
    DL.check()
    td.destroy_process_group()


if __name__ == "__main__":
    main()
