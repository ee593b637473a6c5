"""Kernel micro-benchmarks (CUDA-event timing, L2 flushed between iterations).

    python -m trl_b200.benchmarks.kernels gemm --m 8192 --n 4608 --k 3584
    python -m trl_b200.benchmarks.kernels lmhead --m 8192 --v 152064 --k 3584
    python -m trl_b200.benchmarks.kernels decode_attn --batch 64 --ctx 1024
    python -m trl_b200.benchmarks.kernels rmsnorm --t 16384 --h 3584
    python -m trl_b200.benchmarks.kernels adamw --n 268435456

Each prints one JSON line with the achieved rate and, when ``MEASURED_PEAKS.json`` sits at the
repository root, the fraction of the measured copy bandwidth / cuBLAS bf16 throughput.  ``--iters 1
--warmup 1`` gives a run small enough to sit under ``ncu``.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def timeit(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "lmhead", "lmhead_bwd", "decode_attn", "rmsnorm", "adamw", "grpo_loss", "moe", "decode_gemm", "fa"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4608)
    ap.add_argument("--k", type=int, default=3584)
    ap.add_argument("--v", type=int, default=152064)
    ap.add_argument("--t", type=int, default=16384)
    ap.add_argument("--h", type=int, default=3584)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--baseline", action="store_true", help="also time the library (cuBLAS / eager) path")
    ap.add_argument("--tp", type=int, default=1, help="decode_gemm: the shapes of one rank of a tensor-parallel group of "
                    "this size; the row-parallel GEMMs then run their fused all-reduce form against a local stand-in "
                    "for the peer's accumulator")
    a = ap.parse_args()
    from ..ops import cuda as K

    hbm, tfl, src = _peaks()
    dev = "cuda"
    out = {"kernel": a.kernel, "peaks": src}
    if a.kernel == "gemm":
        A = torch.randn(a.m, a.k, device=dev, dtype=torch.bfloat16)
        B = torch.randn(a.n, a.k, device=dev, dtype=torch.bfloat16)
        C = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
        ms = timeit(lambda: K.gemm_bf16_tn(A, B, out=C), a.iters, a.warmup)
        fl = 2.0 * a.m * a.n * a.k
        out.update(shape=[a.m, a.n, a.k], ms=ms, tflops=fl / ms / 1e9, frac_of_cublas_peak=fl / ms / 1e9 / tfl)
        # the two gradient products of the same linear layer: dX = dY W (W read MN-major), dW = dY^T x (both MN-major)
        dY = torch.randn(a.m, a.n, device=dev, dtype=torch.bfloat16)
        dX = torch.empty(a.m, a.k, device=dev, dtype=torch.bfloat16)
        dW = torch.empty(a.n, a.k, device=dev, dtype=torch.bfloat16)
        ms_dx = timeit(lambda: K.gemm_bf16(dY, B, b_mn=True, out=dX), a.iters, a.warmup)
        ms_dw = timeit(lambda: K.gemm_bf16(dY, A, a_mn=True, b_mn=True, out=dW), a.iters, a.warmup)
        out.update(dgrad_ms=ms_dx, dgrad_tflops=fl / ms_dx / 1e9, wgrad_ms=ms_dw, wgrad_tflops=fl / ms_dw / 1e9)
        # the same three products on the CTA-pair kernel (cta_group::2, 256 x 256 tile per pair of SMs)
        ms_p = timeit(lambda: K.gemm_pair_bf16(A, B, out=C), a.iters, a.warmup)
        ms_pdx = timeit(lambda: K.gemm_pair_bf16(dY, B, b_mn=True, out=dX), a.iters, a.warmup)
        ms_pdw = timeit(lambda: K.gemm_pair_bf16(dY, A, a_mn=True, b_mn=True, out=dW), a.iters, a.warmup)
        out.update(pair_ms=ms_p, pair_tflops=fl / ms_p / 1e9, pair_dgrad_ms=ms_pdx, pair_wgrad_ms=ms_pdw)
        if a.baseline:
            ms2 = timeit(lambda: torch.matmul(A, B.t(), out=C), a.iters, a.warmup)
            ms3 = timeit(lambda: torch.matmul(dY, B, out=dX), a.iters, a.warmup)
            ms4 = timeit(lambda: torch.matmul(dY.t(), A, out=dW), a.iters, a.warmup)
            out.update(cublas_ms=ms2, cublas_tflops=fl / ms2 / 1e9, cublas_dgrad_ms=ms3, cublas_wgrad_ms=ms4,
                       fwd_vs_cublas=ms2 / ms, dgrad_vs_cublas=ms3 / ms_dx, wgrad_vs_cublas=ms4 / ms_dw,
                       pair_fwd_vs_cublas=ms2 / ms_p, pair_dgrad_vs_cublas=ms3 / ms_pdx, pair_wgrad_vs_cublas=ms4 / ms_pdw)
    elif a.kernel in ("lmhead", "lmhead_bwd"):
        H = torch.randn(a.m, a.k, device=dev, dtype=torch.bfloat16)
        W = (torch.randn(a.v, a.k, device=dev) * 0.02).to(torch.bfloat16)
        y = torch.randint(0, a.v, (a.m,), device=dev)
        fl = 2.0 * a.m * a.v * a.k
        if a.kernel == "lmhead":
            ms = timeit(lambda: K.lmhead_forward(H, W, y, 1.0, True, True), a.iters, a.warmup)
        else:
            _, _, lse, _ = K.lmhead_forward(H, W, y, 1.0, False, False)
            g = torch.ones(a.m, device=dev)
            dz = torch.empty(a.m, a.v, device=dev, dtype=torch.bfloat16)
            ms = timeit(lambda: K.lmhead_dz(H, W, y, lse, g, 1.0, out=dz), a.iters, a.warmup)
        out.update(shape=[a.m, a.v, a.k], ms=ms, tflops=fl / ms / 1e9, frac_of_cublas_peak=fl / ms / 1e9 / tfl)
        if a.baseline and a.kernel == "lmhead":
            def eager():
                for hc, yc in zip(H.split(2048), y.split(2048)):
                    lg = (hc @ W.t()).float()
                    torch.log_softmax(lg, -1).gather(-1, yc[:, None])
            out["eager_chunked_ms"] = timeit(eager, max(2, a.iters // 3), 1)
    elif a.kernel == "decode_attn":
        Hq, Hk, D, bs = 28, 4, 128, 16
        nb = a.batch * ((a.ctx + bs) // bs + 1)
        kc = torch.randn(nb, bs, Hk, D, device=dev, dtype=torch.bfloat16)
        vc = torch.randn(nb, bs, Hk, D, device=dev, dtype=torch.bfloat16)
        mb = nb // a.batch
        table = torch.randperm(nb, device=dev).reshape(a.batch, mb).to(torch.int32)
        q = torch.randn(a.batch, Hq, D, device=dev, dtype=torch.bfloat16)
        lens = torch.full((a.batch,), a.ctx - 1, device=dev, dtype=torch.int32)
        splits = max(1, min(8, -(-(4 * 148) // (a.batch * Hk))))
        po = torch.empty(a.batch * Hq * splits * D, device=dev)
        pml = torch.empty(a.batch * Hq * splits * 2, device=dev)
        o = torch.empty(a.batch, Hq, D, device=dev, dtype=torch.bfloat16)
        ms = timeit(lambda: K.paged_decode_attn(q, kc, vc, lens, None, table, bs, 1 / math.sqrt(D), splits, po, pml, o),
                    a.iters, a.warmup)
        byt = 2.0 * a.batch * a.ctx * Hk * D * 2
        out.update(batch=a.batch, ctx=a.ctx, splits=splits, cuda_core_ms=ms, cuda_core_frac_of_copy_bw=byt / ms / 1e6 / hbm)
        # tensor-core kernel: 64-token pages, V transposed inside a page
        bs2 = 64
        nb2 = a.batch * ((a.ctx + bs2) // bs2 + 1)
        kc2 = torch.randn(nb2, bs2, Hk, D, device=dev, dtype=torch.bfloat16)
        vt2 = torch.randn(nb2, Hk, D, bs2, device=dev, dtype=torch.bfloat16)
        table2 = torch.randperm(nb2, device=dev).reshape(a.batch, nb2 // a.batch).to(torch.int32)
        for sp in sorted({1, 2, splits}):
            po2 = torch.empty(a.batch * Hq * sp * D, device=dev)
            pml2 = torch.empty(a.batch * Hq * sp * 2, device=dev)
            ms2 = timeit(lambda: K.paged_decode_attn_tc(q, kc2, vt2, lens, None, table2, 1 / math.sqrt(D), sp, po2, pml2, o),
                         a.iters, a.warmup)
            out[f"tcgen05_splits{sp}_ms"] = ms2
            out[f"tcgen05_splits{sp}_frac_of_copy_bw"] = byt / ms2 / 1e6 / hbm
            ms3 = timeit(lambda: K.paged_decode_attn_tc(q, kc2, vt2, lens, None, table2, 1 / math.sqrt(D), sp, po2, pml2, o,
                                                        groups=2), a.iters, a.warmup)
            out[f"tcgen05_2groups_splits{sp}_ms"] = ms3
            out[f"tcgen05_2groups_splits{sp}_frac_of_copy_bw"] = byt / ms3 / 1e6 / hbm
        K.check_status(dev)
    elif a.kernel == "decode_gemm":
        # the weight-streaming GEMMs of one Qwen2.5-7B decode step at batch a.batch: cuBLAS vs the stream-K kernel,
        # each alone with a cold L2, then the four back to back (as in a layer) with and without dependent launch
        rows = []
        tp = a.tp
        shapes = (("qkv", 4608 // tp, 3584, "acc"), ("o_proj", 3584, 3584 // tp, "acc" if tp == 1 else "allreduce"),
                  ("gate_up", 37888 // tp, 3584, "swiglu"), ("down", 3584, 18944 // tp, "acc" if tp == 1 else "allreduce"),
                  ("lm_head", a.v, 3584, "store"))
        bufs = []
        for name, N, Kd, kind in shapes:
            x = (torch.randn(a.batch, Kd, device=dev) * 0.5).to(torch.bfloat16)
            w = (torch.randn(N, Kd, device=dev) / Kd ** 0.5).to(torch.bfloat16)
            if kind == "allreduce":
                y32, peer = torch.zeros(a.batch, N, device=dev), torch.zeros(a.batch, N, device=dev)
                stage = torch.zeros(a.batch, N, device=dev)
                ctr = torch.zeros(4 * ((N + 127) // 128), dtype=torch.int32, device=dev)
                arr = torch.zeros(32, dtype=torch.int32, device=dev)
                own = lambda x=x, w=w, y32=y32, peer=peer, stage=stage, ctr=ctr, arr=arr: K.decode_gemm(
                    x, w, y32=y32, peers=([peer.data_ptr()] * (tp - 1), [arr.data_ptr()] + [arr[16:].data_ptr()] * (tp - 1),
                                          stage, ctr))
            elif kind == "acc":
                y32 = torch.zeros(a.batch, N, device=dev)
                own = lambda x=x, w=w, y32=y32: K.decode_gemm(x, w, y32=y32)
            elif kind == "swiglu":
                ob = torch.empty(a.batch, N // 2, device=dev, dtype=torch.bfloat16)
                own = lambda x=x, w=w, ob=ob: K.decode_gemm(x, w, out=ob, swiglu=True)
            else:
                ob = torch.empty(a.batch, N, device=dev, dtype=torch.bfloat16)
                own = lambda x=x, w=w, ob=ob: K.decode_gemm(x, w, out=ob)
            lib_fn = lambda x=x, w=w: torch.nn.functional.linear(x, w)
            t_lib = timeit(lib_fn, a.iters, a.warmup)
            t_own = timeit(own, a.iters, a.warmup)
            byt = N * Kd * 2.0
            rows.append({"gemm": name, "weight_MB": round(byt / 1e6, 1), "cublas_us": round(t_lib * 1e3, 1),
                         "own_us": round(t_own * 1e3, 1), "floor_us": round(byt / hbm / 1e3, 1),
                         "own_frac_of_copy_bw": round(byt / t_own / 1e6 / hbm, 3)})
            if name != "lm_head":
                bufs.append((own, lib_fn, byt))

        def chain(fns, reps=28):
            for _ in range(reps):
                for f in fns:
                    f()

        total = 28 * sum(b for _, _, b in bufs)
        res = {}
        for label, fns, pdl in (("cublas", [b[1] for b in bufs], False), ("own", [b[0] for b in bufs], False),
                                ("own_pdl", [b[0] for b in bufs], True)):
            was = K.set_pdl(pdl)
            g = torch.cuda.CUDAGraph()
            chain(fns, 1)
            torch.cuda.synchronize()
            with torch.cuda.graph(g):
                chain(fns)
            ms = timeit(g.replay, a.iters, a.warmup)
            K.set_pdl(was)
            res[label + "_28_layers_ms"] = round(ms, 3)
            res[label + "_frac_of_copy_bw"] = round(total / ms / 1e6 / hbm, 3)
        out.update(batch=a.batch, tp=tp, gemms=rows, chain=res)
    elif a.kernel == "fa":
        # varlen attention, forward and forward + backward: this library's tcgen05 kernels against flash-attn's
        # flash_attn_varlen_func (when importable) on two packings: one 8192-token pack of documents with log-uniform
        # lengths in [128, 8192], and 8 sequences of 1280 tokens (the GRPO micro-batch shape)
        import random

        rows = []
        rng = random.Random(0)
        docs, left = [], 8192
        while left > 0:
            L = min(left, int(math.exp(rng.uniform(math.log(128), math.log(8192)))))
            docs.append(L)
            left -= L
        for label, lens, Hq, Hk in (("pack8192_loguniform", docs, 32, 8), ("8x1280", [1280] * 8, 28, 4),
                                    ("1x8192", [8192], 32, 8)):
            T = sum(lens)
            q = torch.randn(T, Hq, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
            k = torch.randn(T, Hk, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
            v = torch.randn(T, Hk, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
            cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
            g = torch.randn(T, Hq, 128, device=dev, dtype=torch.bfloat16)
            flops = sum(4.0 * Hq * 128 * L * (L + 1) / 2 for L in lens)  # causal: QK^T and PV over the visible half

            def own_fwd():
                with torch.no_grad():
                    return K.attention_varlen(q, k, v, cu, max(lens), True, None)

            def own_fb():
                o = K.attention_varlen(q, k, v, cu, max(lens), True, None)
                torch.autograd.grad(o, (q, k, v), g)

            rec = {"case": label, "tokens": T, "docs": len(lens), "heads": [Hq, Hk]}
            t = timeit(own_fwd, a.iters, a.warmup)
            rec.update(own_fwd_ms=round(t, 4), own_fwd_tflops=round(flops / t / 1e9, 1))
            t = timeit(own_fb, a.iters, a.warmup)
            rec.update(own_fwd_bwd_ms=round(t, 4), own_fwd_bwd_tflops=round(3.5 * flops / t / 1e9, 1))
            if a.baseline:
                try:
                    from flash_attn import flash_attn_varlen_func

                    def lib_fwd():
                        with torch.no_grad():
                            return flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True)

                    def lib_fb():
                        o = flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True)
                        torch.autograd.grad(o, (q, k, v), g)

                    t = timeit(lib_fwd, a.iters, a.warmup)
                    rec.update(flash_attn_fwd_ms=round(t, 4), flash_attn_fwd_tflops=round(flops / t / 1e9, 1))
                    t = timeit(lib_fb, a.iters, a.warmup)
                    rec.update(flash_attn_fwd_bwd_ms=round(t, 4), flash_attn_fwd_bwd_tflops=round(3.5 * flops / t / 1e9, 1))
                except Exception as e:  # noqa: BLE001
                    rec["flash_attn"] = f"unavailable: {type(e).__name__}: {str(e)[:80]}"
            rows.append(rec)
        out.update(cases=rows)
    elif a.kernel == "moe":
        # Qwen3-30B-A3B expert shapes: 128 experts, hidden 2048, expert FFN 768, top-8; a.t tokens
        E, H, I, k = 128, 2048, 768, 8
        x = (torch.randn(a.t, H, device=dev) * 0.5).to(torch.bfloat16)
        gu = (torch.randn(E, 2 * I, H, device=dev) / H ** 0.5).to(torch.bfloat16)
        dw = (torch.randn(E, H, I, device=dev) / I ** 0.5).to(torch.bfloat16)
        tw, ti = torch.softmax(torch.randn(a.t, E, device=dev), -1).topk(k, -1)
        with torch.no_grad():
            ms = timeit(lambda: K.moe_experts(x, gu, dw, tw, ti), a.iters, a.warmup)
        flops = 2.0 * a.t * k * H * 3 * I
        out.update(tokens=a.t, experts=E, top_k=k, moe_block_ms=ms, tflops=flops / ms / 1e9,
                   frac_of_cublas_burst=flops / ms / 1e9 / tfl)
        flat = ti.reshape(-1)
        order = torch.argsort(flat, stable=True)
        offsets = torch.zeros(E + 1, dtype=torch.int32, device=dev)
        offsets[1:] = torch.bincount(flat, minlength=E).cumsum(0)
        xp = x[order // k]
        ms1 = timeit(lambda: K.grouped_gemm(xp, gu, offsets, I, swiglu=True), a.iters, a.warmup)
        out.update(gate_up_swiglu_ms=ms1, gate_up_tflops=2.0 * a.t * k * H * 2 * I / ms1 / 1e9)
        # backward: the block's forward + backward, and the two grouped gradient kernels on the gate/up shapes
        xg, gug, dwg = (t.clone().requires_grad_(True) for t in (x, gu, dw))

        def fwd_bwd():
            K.moe_experts(xg, gug, dwg, tw, ti).backward(x)
            xg.grad = gug.grad = dwg.grad = None
        ms_fb = timeit(fwd_bwd, a.iters, a.warmup)
        d_gu = (torch.randn(xp.shape[0], 2 * I, device=dev) * 0.1).to(torch.bfloat16)
        ms_dx = timeit(lambda: K.grouped_gemm(d_gu, gu, offsets, H, w_transposed=True), a.iters, a.warmup)
        dwo = torch.empty_like(gu)
        ms_dw = timeit(lambda: K.grouped_wgrad(d_gu, xp, offsets, E, out=dwo), a.iters, a.warmup)
        f_gu = 2.0 * a.t * k * H * 2 * I
        out.update(moe_block_fwd_bwd_ms=ms_fb, gate_up_dgrad_ms=ms_dx, gate_up_dgrad_tflops=f_gu / ms_dx / 1e9,
                   gate_up_wgrad_ms=ms_dw, gate_up_wgrad_tflops=f_gu / ms_dw / 1e9)
        if a.baseline:
            from trl_b200.oracle.ops import moe_experts as loop

            offs_h = offsets.tolist()

            def lib_grads():  # what the backward did before: one library GEMM per expert and product
                for e in range(E):
                    s0, s1 = offs_h[e], offs_h[e + 1]
                    if s1 > s0:
                        torch.matmul(d_gu[s0:s1], gu[e])
                        torch.matmul(d_gu[s0:s1].t(), xp[s0:s1])
            out["gate_up_dgrad_wgrad_library_loop_ms"] = timeit(lib_grads, max(2, a.iters // 3), 1)

            with torch.no_grad():
                out["expert_loop_ms"] = timeit(lambda: loop(x, gu, dw, tw, ti), max(2, a.iters // 3), 1)
            if hasattr(torch, "_grouped_mm"):
                try:
                    offs = offsets[1:].contiguous()
                    gut = gu.transpose(1, 2)
                    out["torch_grouped_mm_gate_up_ms"] = timeit(lambda: torch._grouped_mm(xp, gut, offs=offs), a.iters, a.warmup)
                except Exception as e:  # library kernel not built for this GPU
                    out["torch_grouped_mm"] = f"unavailable: {type(e).__name__}"
    elif a.kernel == "rmsnorm":
        x = torch.randn(a.t, a.h, device=dev, dtype=torch.bfloat16)
        w = torch.ones(a.h, device=dev, dtype=torch.bfloat16)
        y = torch.empty_like(x)
        ms = timeit(lambda: K.rmsnorm_infer(x, w, 1e-6, out=y), a.iters, a.warmup)
        byt = 2.0 * a.t * a.h * 2
        out.update(shape=[a.t, a.h], ms=ms, gbs=byt / ms / 1e6, frac_of_copy_bw=byt / ms / 1e6 / hbm)
    elif a.kernel == "adamw":
        n = a.n if a.n > 1 << 20 else 1 << 28
        p, g = torch.randn(n, device=dev), torch.randn(n, device=dev)
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        sh = torch.empty(n, device=dev, dtype=torch.bfloat16)
        ms = timeit(lambda: K.adamw_flat(p, g, m, v, 1, 1e-4, 0.9, 0.999, 1e-8, 0.0, 1.0, sh), a.iters, a.warmup)
        byt = n * (4 * 4 + 3 * 4 + 2.0)
        out.update(n=n, ms=ms, gbs=byt / ms / 1e6, frac_of_copy_bw=byt / ms / 1e6 / hbm)
    elif a.kernel == "grpo_loss":
        B, T = a.batch, a.ctx
        lp = -torch.rand(B, T, device=dev)
        old, ref = lp + 0.1 * torch.randn_like(lp), lp + 0.1 * torch.randn_like(lp)
        adv, mask = torch.randn(B, device=dev), torch.ones(B, T, device=dev)
        rs = torch.full((B,), 1.0 / (B * T), device=dev)
        ms = timeit(lambda: K.grpo_loss(lp, old, ref, adv, mask, rs, lp, 0.2, 0.2, 0.04, None), a.iters, a.warmup)
        byt = B * T * 4 * 6.0
        out.update(shape=[B, T], ms=ms, gbs=byt / ms / 1e6)
    K.check_status()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
