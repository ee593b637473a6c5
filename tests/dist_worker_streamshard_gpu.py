"""2-GPU worker: streamed full-shard engine (bf16; own peer-memory kernels or the backend's collectives) vs zero2."""
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
from trl_b200.parallel.streamshard import StreamShardEngine
from trl_b200.testing import make_tiny_model


def run(model, engine, rank, steps=3):
    dev = model.device
    out = []
    for s in range(steps):
        engine.zero_grad()
        for micro in range(2):  # gradient accumulation: the per-layer reduce-scatter adds into the fp32 slice
            g = torch.Generator().manual_seed(1000 * s + 10 * micro + rank)
            ids = torch.randint(0, 1024, (300,), generator=g).to(dev)
            ctx = SeqCtx.from_lengths([120, 180], dev)
            h = model.forward_hidden(ids, ctx)
            loss_sum, _, _, n = ops.lm_head_ce(h, model.lm_head_weight, torch.roll(ids, -1))
            loss = loss_sum / n / 2
            engine.backward(loss)
        out.append((float(loss.detach()), float(engine.step(1e-3, 1.0))))
    return out


sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _dist_util import Deadline  # noqa: E402


def main():
    D.init_process_group()
    DL = Deadline()  # the ranks leave on their own, between steps, before the parent's limit
    rank = D.rank()
    dev = torch.device("cuda", D.local_rank())
    base = make_tiny_model("tiny-qwen2", dtype=torch.bfloat16, device=dev, hidden_size=512, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=128, intermediate_size=1024, num_hidden_layers=3, seed=0)
    m_st, m_z2 = copy.deepcopy(base), copy.deepcopy(base)
    DL.check()
    for m in (m_st, m_z2):
        m.gradient_checkpointing_enable()
        m.train()
    e_st = StreamShardEngine(m_st)
    assert e_st.fused == (os.environ.get("TRL_B200_STREAM_FUSED", "1") != "0")
    e_z2 = TrainEngine(m_z2, mode="zero2", use_symm_kernels=False)
    a = run(m_st, e_st, rank)
    b = run(m_z2, e_z2, rank)
    torch.cuda.synchronize()
    K.check_status(dev)
    DL.check()
    for (la, na), (lb, nb) in zip(a, b):
        assert abs(la - lb) < 5e-2 and abs(na - nb) < 5e-2 * max(1.0, nb), (a, b)
    sd = e_st.streamed_hf_state_dict(to_cpu=True)
    ref = m_z2.state_dict_hf()
    DL.check()
    for k, v in ref.items():
        assert torch.isfinite(sd[k].float()).all(), k
        assert torch.allclose(sd[k].float().cpu(), v.float().cpu(), atol=3e-2, rtol=3e-2), k
    # parameter memory: one slice per layer + two slots, not the whole model
    held = sum(l.master.numel() for l in e_st.layers) + sum(s.numel() for s in e_st.slots)
    whole = sum(l.numel for l in e_st.layers)
    assert held < 0.5 * whole + 2 * e_st.slots[0].numel() + 1
    td.barrier()
    if rank == 0:
        print("STREAMSHARD_OK", a, b)
    DL.check()
    td.destroy_process_group()


if __name__ == "__main__":
    main()
