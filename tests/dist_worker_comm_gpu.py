"""2+ GPU worker: comm kernels (csrc/comm.cu) against NCCL + PyTorch references."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import copy

import torch
import torch.distributed as td

from trl_b200.ops import cuda as K
from trl_b200.oracle import ops as ref
from trl_b200.parallel import dist as D
from trl_b200.parallel.engine import TrainEngine
from trl_b200.parallel.symm import SymmArena, SyncWords
from trl_b200.testing import make_tiny_model


sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _dist_util import Deadline  # noqa: E402


def main():
    D.init_process_group()
    DL = Deadline()  # the ranks leave on their own, between steps, before the parent's limit
    rank, world = D.rank(), D.world_size()
    dev = torch.device("cuda", D.local_rank())
    torch.manual_seed(0)
    DL.check()
    # ---- fused optimizer step vs NCCL reduce-scatter + AdamW + all-gather -------------------------------
    base = make_tiny_model("tiny-qwen2", dtype=torch.bfloat16, device=dev, hidden_size=256, intermediate_size=512,
                           num_attention_heads=2, num_key_value_heads=1, head_dim=128)
    m_fused, m_nccl = copy.deepcopy(base), copy.deepcopy(base)
    e_fused = TrainEngine(m_fused, mode="zero2", use_symm_kernels=True)
    e_nccl = TrainEngine(m_nccl, mode="zero2", use_symm_kernels=False)
    assert e_fused.use_symm and not e_nccl.use_symm
    for variant in ("p2p", "multimem"):
        if variant == "multimem" and not e_fused._arenas["param"].multicast_ptr:
            continue
        e_fused.use_multimem = variant == "multimem"
        for step in range(2):
            g = torch.Generator(device=dev).manual_seed(100 * rank + step)
            for bf, bn in zip(e_fused.buckets, e_nccl.buckets):
                r = torch.randn(bf.flat_grad.shape, device=dev, generator=g)
                bf.flat_grad.copy_(r)
                bn.flat_grad.copy_(r)
            n1 = e_fused.step(1e-2, 1.0)
            n2 = e_nccl.step(1e-2, 1.0)
            torch.cuda.synchronize()
            K.check_status(dev)
            assert torch.allclose(n1, n2, rtol=1e-4), (variant, float(n1), float(n2))
            for (na, pa), (_, pb) in zip(m_fused.named_parameters(), m_nccl.named_parameters()):
                assert torch.allclose(pa.float(), pb.float(), atol=2e-2, rtol=2e-2), (variant, na)
            for bf, bn in zip(e_fused.buckets, e_nccl.buckets):
                assert torch.allclose(bf.master, bn.master, atol=1e-5, rtol=1e-5)
        td.barrier()
    # replicas identical on every rank after the broadcast stores
    flat = torch.cat([b.flat_param.float() for b in e_fused.buckets])
    ref0 = flat.clone()
    td.broadcast(ref0, 0)
    assert torch.equal(flat, ref0)
    DL.check()
    # ---- shard all-gather: pull and multimem push ---------------------------------------------------------
    per = 1 << 16
    arena = SymmArena(world * per * 2 + 4096, dev)
    buf, off = arena.carve(world * per, torch.bfloat16)
    sync = SyncWords(dev, channel=1)
    for mm in (False, True):
        if mm and not arena.multicast_ptr:
            continue
        buf.zero_()
        buf[rank * per:(rank + 1) * per] = torch.arange(per, device=dev).to(torch.bfloat16) + rank
        torch.cuda.synchronize()
        td.barrier()
        K.shard_allgather(arena, off, per, sync, use_multimem=mm)
        torch.cuda.synchronize()
        K.check_status(dev)
        for r in range(world):
            want = torch.arange(per, device=dev).to(torch.bfloat16) + r
            assert torch.equal(buf[r * per:(r + 1) * per], want), (mm, r)
        td.barrier()
    DL.check()
    # ---- TP decode: all-reduce + residual add + RMSNorm ----------------------------------------------------
    T, H = 64, 3584
    arena2 = SymmArena(2 * T * H * 2 + 4096, dev)
    parts, off2 = arena2.carve(2 * T * H, torch.bfloat16)
    sync2 = SyncWords(dev, channel=2)
    w = (1 + 0.1 * torch.randn(H, device=dev)).to(torch.bfloat16)
    td.broadcast(w, 0)
    res = torch.randn(T, H, device=dev).to(torch.bfloat16)
    td.broadcast(res, 0)
    for it in range(3):
        epoch = it + 1
        mine = torch.randn(T, H, device=dev, generator=torch.Generator(device=dev).manual_seed(7 * rank + it)).to(torch.bfloat16)
        parts[(epoch & 1) * T * H:((epoch & 1) + 1) * T * H].copy_(mine.reshape(-1))
        tot = mine.float().clone()
        td.all_reduce(tot)
        want_res = (res.float() + tot.to(torch.bfloat16).float()).to(torch.bfloat16)
        want_y = ref.rms_norm(want_res, w, 1e-6)
        y = K.allreduce_add_rmsnorm(arena2, off2, T * H, res, w, 1e-6, sync2)
        torch.cuda.synchronize()
        K.check_status(dev)
        assert torch.allclose(res.float(), want_res.float(), atol=3e-2, rtol=2e-2), it
        assert torch.allclose(y.float(), want_y.float(), atol=5e-2, rtol=3e-2), it
        g = res.clone()
        td.broadcast(g, 0)
        assert torch.equal(g, res)  # bit-identical residual stream on all ranks
    DL.check()
    # ---- all-gather fused into the GEMM ------------------------------------------------------------------
    from trl_b200.ops.cuda_comm import AgGemmState, ag_gemm

    for (M, N, Kd, extra) in [(512, 1024, 512, 4096), (300, 1536 + 256, 256, 0)]:
        total = N * Kd + extra
        total = (total + world * 256 - 1) // (world * 256) * (world * 256)
        per = total // world
        ar = SymmArena(total * 2 + 4096, dev)
        buf, off = ar.carve(total, torch.bfloat16)
        full = (torch.randn(total, device=dev, generator=torch.Generator(device=dev).manual_seed(42)) * 0.1).to(torch.bfloat16)
        buf.zero_()
        buf[rank * per:(rank + 1) * per] = full[rank * per:(rank + 1) * per]  # only the own shard is valid
        x = torch.randn(M, Kd, device=dev, generator=torch.Generator(device=dev).manual_seed(9)).to(torch.bfloat16)
        w_off = extra // 2 // 8 * 8
        st = AgGemmState(dev)
        torch.cuda.synchronize()
        td.barrier()
        for call in range(2):
            if call == 1:  # second call on the same buffer: remote parts wiped again
                td.barrier()
                keep = buf[rank * per:(rank + 1) * per].clone()
                buf.zero_()
                buf[rank * per:(rank + 1) * per] = keep
                torch.cuda.synchronize()
                td.barrier()
            y = ag_gemm(x, ar, off, per, total, w_off, N, st)
            torch.cuda.synchronize()
            K.check_status(dev)
            W = full[w_off:w_off + N * Kd].view(N, Kd)
            want = x.float() @ W.float().t()
            assert torch.allclose(y.float(), want, atol=3e-2 * want.abs().max().item() + 1e-2, rtol=2e-2), (M, N, Kd, call)
            assert torch.equal(buf, full), "local buffer not completed by the kernel"
        td.barrier()
    td.barrier()
    if rank == 0:
        print("COMM_OK multicast=%d" % int(bool(arena.multicast_ptr)))
    td.destroy_process_group()


if __name__ == "__main__":
    main()
