"""Multi-GPU micro-benchmarks of the fused compute+collective kernels against their NCCL(+cuBLAS) baselines.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29533 \
        -m trl_b200.benchmarks.comm [--model llama-3-8b] [--tokens 4096]

Device-timed with CUDA events, max over ranks; rank 0 prints one JSON object.  Roofline per fused kernel =
max(FLOPs / measured cuBLAS rate, bytes that must cross NVLink into this GPU / 770 GB/s).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as td

from ..models.configuration import preset
from ..ops import cuda as K
from ..ops.cuda_comm import AgGemmState, ag_gemm
from ..parallel import dist as D
from ..parallel.symm import SymmArena, SyncWords

NVLINK_GBS = 770.0


def timed(fn, iters=5, warmup=2, pre=None):
    ts = []
    for i in range(warmup + iters):
        if pre is not None:
            pre()
        torch.cuda.synchronize()
        td.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        if i >= warmup:
            ts.append(a.elapsed_time(b))
    t = torch.tensor([sorted(ts)[len(ts) // 2]], device="cuda")
    td.all_reduce(t, td.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--copiers", type=int, default=16)
    ap.add_argument("--moe-tokens", type=int, default=8192, help="tokens per rank for the expert-parallel MoE block")
    ap.add_argument("--copiers-sweep", default="", help="comma-separated copier-CTA counts: time only the fused "
                                                        "all-gather + GEMM for each and exit")
    a = ap.parse_args()
    D.init_process_group()
    rank, world = D.rank(), D.world_size()
    dev = torch.device("cuda", D.local_rank())
    cfg = preset(a.model)
    H, I = cfg.hidden_size, cfg.intermediate_size
    nqkv = cfg.q_size + 2 * cfg.kv_size
    layer_elems = nqkv * H + cfg.q_size * H + 3 * I * H + 2 * H
    total = (layer_elems + world * 256 - 1) // (world * 256) * (world * 256)
    per = total // world
    peaks = {}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    tfl = json.load(open(pk)).get("bf16_tflops", 1590.0) if os.path.exists(pk) else 1590.0
    out = {"world": world, "model": a.model, "tokens": a.tokens, "layer_MB": round(total * 2 / 1e6, 1)}
    # ---- AG -> GEMM (QKV of one layer; the kernel gathers the whole layer bucket) ----------------------
    arena = SymmArena(total * 2 + 4096, dev)
    buf, off = arena.carve(total, torch.bfloat16)
    buf.normal_(0, 0.02)
    x = torch.randn(a.tokens, H, device=dev, dtype=torch.bfloat16)
    y = torch.empty(a.tokens, nqkv, device=dev, dtype=torch.bfloat16)
    if a.copiers_sweep:
        sweep = {}
        for c in [int(v) for v in a.copiers_sweep.split(",")]:
            st_c = AgGemmState(dev, copiers=c)
            sweep[str(c)] = timed(lambda: ag_gemm(x, arena, off, per, total, 0, nqkv, st_c, out=y))
        K.check_status(dev)
        full = torch.empty(total, device=dev, dtype=torch.bfloat16)
        shard = buf[rank * per:(rank + 1) * per]

        def nccl_ref():
            td.all_gather_into_tensor(full, shard)
            torch.matmul(x, full[:nqkv * H].view(nqkv, H).t(), out=y)
        out["ag_gemm_copier_sweep_ms"] = sweep
        out["nccl_allgather_then_cublas_ms"] = timed(nccl_ref)
        if rank == 0:
            print(json.dumps(out))
        td.barrier()
        td.destroy_process_group()
        return
    st = AgGemmState(dev, copiers=a.copiers)
    t_fused = timed(lambda: ag_gemm(x, arena, off, per, total, 0, nqkv, st, out=y))
    full = torch.empty(total, device=dev, dtype=torch.bfloat16)
    shard = buf[rank * per:(rank + 1) * per]

    def nccl_path():
        td.all_gather_into_tensor(full, shard)
        torch.matmul(x, full[:nqkv * H].view(nqkv, H).t(), out=y)
    t_nccl = timed(nccl_path)
    t_ag_only = timed(lambda: td.all_gather_into_tensor(full, shard))
    t_gemm_only = timed(lambda: torch.matmul(x, full[:nqkv * H].view(nqkv, H).t(), out=y))
    flops = 2.0 * a.tokens * nqkv * H
    link_bytes = total * 2 * (world - 1) / world
    roof_ms = max(flops / (tfl * 1e9), link_bytes / (NVLINK_GBS * 1e6))
    out["ag_gemm"] = {"fused_ms": t_fused, "nccl_allgather_then_cublas_ms": t_nccl, "nccl_allgather_ms": t_ag_only,
                      "cublas_gemm_ms": t_gemm_only, "roofline_ms": roof_ms, "fraction_of_roofline": roof_ms / t_fused,
                      "bytes_over_nvlink_MB": link_bytes / 1e6}
    K.check_status(dev)
    # ---- shard all-gather alone: pull, multimem push, NCCL -------------------------------------------------
    sync = SyncWords(dev, channel=3)
    out["allgather"] = {"pull_ms": timed(lambda: K.shard_allgather(arena, off, per, sync, False)), "nccl_ms": t_ag_only,
                        "link_floor_ms": link_bytes / (NVLINK_GBS * 1e6)}
    if arena.multicast_ptr:
        out["allgather"]["multimem_push_ms"] = timed(lambda: K.shard_allgather(arena, off, per, sync, True))
    K.check_status(dev)
    # ---- reduce-scatter + AdamW + parameter broadcast for one layer bucket -----------------------------------
    ga = SymmArena(total * 4 + 4096, dev)
    grad, goff = ga.carve(total, torch.float32)
    grad.normal_()
    master, m, v = torch.randn(per, device=dev), torch.zeros(per, device=dev), torch.zeros(per, device=dev)
    red, ss = torch.empty(per, device=dev), torch.zeros(1, device=dev)
    clip = torch.ones(1, device=dev)
    sync2 = SyncWords(dev, channel=4)
    for mm in ([False, True] if arena.multicast_ptr else [False]):
        def fused():
            K.rs_reduce(ga, goff, False, rank * per, per, red, ss, sync2, use_multimem=mm)
            K.adamw_bcast(arena, off, rank * per, per, master, red, m, v, 1, 1e-4, 0.9, 0.999, 1e-8, 0.0, clip, sync2,
                          use_multimem=mm)
        out.setdefault("rs_adamw", {})["multimem_ms" if mm else "p2p_ms"] = timed(fused)
    gshard = torch.empty(per, device=dev)
    pshard = torch.empty(per, device=dev, dtype=torch.bfloat16)

    def nccl_opt():
        td.reduce_scatter_tensor(gshard, grad, op=td.ReduceOp.AVG)
        K.adamw_flat(master, gshard, m, v, 1, 1e-4, 0.9, 0.999, 1e-8, 0.0, 1.0, pshard)
        td.all_gather_into_tensor(full, pshard)
    out["rs_adamw"]["nccl_rs_fused_adamw_nccl_ag_ms"] = timed(nccl_opt)
    rs_bytes = total * 4 * (world - 1) / world + total * 2 * (world - 1) / world
    out["rs_adamw"]["link_floor_ms"] = rs_bytes / (NVLINK_GBS * 1e6)
    if rank == 0:  # the sections above are complete: keep them even if the next one fails
        print(json.dumps({**out, "partial": "before ep_moe"}), flush=True)
    # ---- expert-parallel MoE block (Qwen3-30B-A3B expert shapes): dispatch/combine fused into the grouped GEMMs ----
    E, Hm, Im, k = 128, 2048, 768, 8
    if E % world == 0:
        from ..parallel.expert_parallel import ExpertParallelMoE

        Tm = a.moe_tokens
        e_loc = E // world
        gu = (torch.randn(e_loc, 2 * Im, Hm, device=dev) / Hm ** 0.5).to(torch.bfloat16)
        dn = (torch.randn(e_loc, Hm, Im, device=dev) / Im ** 0.5).to(torch.bfloat16)
        xh = (torch.randn(Tm, Hm, device=dev) * 0.5).to(torch.bfloat16)
        tw, ti = torch.softmax(torch.randn(Tm, E, device=dev), -1).topk(k, -1)
        ep = ExpertParallelMoE(None, E, Hm, Im, k, max_tokens=Tm, device=dev)
        with torch.no_grad():
            t_ep = timed(lambda: ep(xh, gu, dn, tw, ti))

        def nccl_ep():  # all-to-all rows out, local grouped GEMMs, all-to-all rows back, combine
            flat = ti.reshape(-1)
            order = torch.argsort(flat, stable=True)
            cnt = torch.bincount(flat, minlength=E)
            send = cnt.view(world, e_loc).sum(1)
            recv = torch.empty_like(send)
            td.all_to_all_single(recv, send)
            cnt_in = torch.empty(world, e_loc, dtype=cnt.dtype, device=dev)
            td.all_to_all_single(cnt_in.view(-1), cnt)
            sl, rl = send.tolist(), recv.tolist()
            xp = xh[order // k]
            xin = torch.empty(sum(rl), Hm, dtype=xh.dtype, device=dev)
            td.all_to_all_single(xin, xp, rl, sl)
            # received rows are source-major; sort them by local expert for the grouped GEMM
            eid = torch.repeat_interleave(torch.arange(e_loc, device=dev).repeat(world), cnt_in.reshape(-1))
            o2 = torch.argsort(eid, stable=True)
            offs = torch.zeros(e_loc + 1, dtype=torch.int32, device=dev)
            offs[1:] = torch.bincount(eid, minlength=e_loc).cumsum(0)
            act = K.grouped_gemm(xin[o2], gu, offs, Im, swiglu=True)
            yin = torch.empty_like(xin)
            yin[o2] = K.grouped_gemm(act, dn, offs, Hm)
            yp = torch.empty_like(xp)
            td.all_to_all_single(yp, yin, sl, rl)
            inv = torch.empty_like(order)
            inv[order] = torch.arange(order.numel(), device=dev)
            return (yp[inv].view(Tm, k, Hm).float() * tw[..., None]).sum(1).to(xh.dtype)
        with torch.no_grad():
            t_nccl = timed(nccl_ep)
        flops = 2.0 * Tm * k * Hm * 3 * Im
        link_bytes = 2.0 * Tm * k * Hm * 2 * (world - 1) / world  # rows in + rows out
        roof = max(flops / (tfl * 1e9), link_bytes / (NVLINK_GBS * 1e6))
        out["ep_moe"] = {"tokens_per_rank": Tm, "fused_ms": t_ep, "nccl_all_to_all_plus_grouped_gemm_ms": t_nccl,
                         "roofline_ms": roof, "frac_of_roofline": roof / t_ep}
    K.check_status(dev)
    if rank == 0:
        print(json.dumps(out))
    td.barrier()
    td.destroy_process_group()


if __name__ == "__main__":
    main()
