"""2-GPU worker: a mixture-of-experts model with its experts split over the ranks (``shard_experts``: fused dispatch /
grouped GEMM / combine kernels inside every layer, expert buckets local to their owner in the zero-2 engine) against
the same model with every expert on every rank, over three optimizer steps."""
import copy
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as td

from trl_b200.models.decoder import SeqCtx
from trl_b200.ops import cuda as K
from trl_b200.ops import functional as ops
from trl_b200.parallel import dist as D
from trl_b200.parallel.engine import TrainEngine
from trl_b200.parallel.expert_parallel import ExpertParallelMoE, ep_hf_state_dict, shard_experts
from trl_b200.testing import make_tiny_model

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _dist_util import Deadline  # noqa: E402


def run(model, engine, rank, steps=3):
    dev = model.device
    out = []
    for s in range(steps):
        engine.zero_grad()
        for micro in range(2):
            g = torch.Generator().manual_seed(1000 * s + 10 * micro + rank)
            n = 260 + 40 * rank  # the ranks hold different numbers of tokens
            ids = torch.randint(0, 1024, (n,), generator=g).to(dev)
            ctx = SeqCtx.from_lengths([100, n - 100], dev)
            h = model.forward_hidden(ids, ctx)
            loss_sum, _, _, cnt = ops.lm_head_ce(h, model.lm_head_weight, torch.roll(ids, -1))
            loss = loss_sum / cnt / 2 + 0.01 * model.aux_loss(ctx)
            engine.backward(loss)
        out.append((float(loss.detach()), float(engine.step(1e-3, 1.0))))
    return out


def main():
    D.init_process_group()
    DL = Deadline()
    rank, world = D.rank(), D.world_size()
    dev = torch.device("cuda", D.local_rank())
    base = make_tiny_model("tiny-qwen3-moe", dtype=torch.bfloat16, device=dev, hidden_size=256, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=64, num_experts=8, num_experts_per_tok=2,
                           moe_intermediate_size=128, num_hidden_layers=2, seed=0)
    m_ep, m_rep = copy.deepcopy(base), copy.deepcopy(base)
    shard_experts(m_ep, max_tokens=1024)
    assert isinstance(m_ep.layers[0].ep, ExpertParallelMoE) and m_ep.layers[0].experts_gate_up.shape[0] == 8 // world
    for m in (m_ep, m_rep):
        m.train()
    e_ep = TrainEngine(m_ep, mode="zero2", weight_decay=0.01)
    e_rep = TrainEngine(m_rep, mode="zero2", weight_decay=0.01)
    assert e_ep.use_symm and any(b.local for b in e_ep.buckets) and e_ep.per_rank_state
    DL.check()
    a = run(m_ep, e_ep, rank)
    b = run(m_rep, e_rep, rank)
    torch.cuda.synchronize()
    K.check_status(dev)
    DL.check()
    for (la, na), (lb, nb) in zip(a, b):
        assert abs(la - lb) < 5e-2 and abs(na - nb) < 5e-2 * max(1.0, nb), (a, b)
    sd = ep_hf_state_dict(m_ep, to_cpu=True)  # collective: every rank gathers
    ref = m_rep.state_dict_hf()
    assert set(sd) == set(ref)
    for k, v in ref.items():
        assert torch.isfinite(sd[k].float()).all(), k
        assert torch.allclose(sd[k].float().cpu(), v.float().cpu(), atol=3e-2, rtol=3e-2), k
    td.barrier()
    if rank == 0:
        print("EP_MODEL_OK", a, b)
    DL.check()
    td.destroy_process_group()


if __name__ == "__main__":
    main()
