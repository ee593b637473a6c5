"""ctypes bindings + autograd wrappers for the sm_100a kernel library.

Kernels are launched on the caller's current CUDA stream, so they compose with torch ops,
side streams and CUDA-graph capture.  Every kernel that can wait takes a per-device status
buffer; :func:`check_status` reads it (one host sync) and raises if a bounded wait ran out.
"""
from __future__ import annotations

import os

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .._native import kernels

_status: dict[int, torch.Tensor] = {}


def lib():
    return kernels(required=True)


def _p(t):
    return None if t is None else c_void_p(t.data_ptr())


def _s():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def status_buffer(device=None) -> torch.Tensor:
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if idx not in _status:
        _status[idx] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_status(device=None, reset: bool = True):
    """Raise if any kernel recorded an error (timeout, bad shape) since the last check."""
    st = status_buffer(device)
    vals = st.tolist()
    if vals[0] != 0:
        if reset:
            st.zero_()
        raise RuntimeError(f"trl_b200 kernel error: code={vals[0]} site={vals[1]} block={vals[2]} extra={vals[3]}")


def bounded_wait_selftest(flag: torch.Tensor, expect: int, budget_ms: int = 50):
    """Launches the one-thread bounded wait on ``flag`` (uint32/int32 tensor); the outcome is read with check_status."""
    _chk(lib().trlb_bounded_wait_selftest(_p(flag), ctypes.c_uint(expect), c_int(budget_ms), _p(status_buffer(flag.device)),
                                          _s()), "bounded_wait_selftest")


LAUNCHES = [0]  # kernels of this library launched (or captured into a graph) from Python


def _chk(rc: int, what: str):
    LAUNCHES[0] += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


# -------------------------------------------------------------------------------------------
# tcgen05 GEMM family
# -------------------------------------------------------------------------------------------
def gemm_bf16_tn(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor | None = None, out: torch.Tensor | None = None):
    """out[M,N] = a[M,K] @ b[N,K]^T (+ bias) on the tcgen05 kernel.  bf16 in/out, fp32 accumulate."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_cuda
    assert a.stride(-1) == 1 and b.stride(-1) == 1
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    rc = lib().trlb_gemm_bf16_tn(_p(a), _p(b), _p(out), _p(bias), c_int(M), c_int(N), c_int(K),
                                 c_longlong(a.stride(0)), c_longlong(b.stride(0)), c_longlong(out.stride(0)),
                                 _p(status_buffer(a.device)), _s())
    _chk(rc, "trlb_gemm_bf16_tn")
    return out


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, bias=None, *, a_mn: bool = False, b_mn: bool = False, out=None):
    """``out[M, N] = op(a) @ op(b)^T (+ bias)`` on the tcgen05 kernel with either operand given transposed:
    ``a`` is ``[M, K]`` (``a_mn=False``) or ``[K, M]`` (``a_mn=True``), ``b`` is ``[N, K]`` or ``[K, N]``.  The
    transposed forms are read as MN-major tensor-core operands straight from their TMA tiles: nothing is transposed
    in memory.  This is what makes ``dX = dY @ W`` and ``dW = dY^T @ x`` run on the same kernel as ``y = x @ W^T``."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_cuda and a.stride(-1) == 1 and b.stride(-1) == 1
    K_, M = (a.shape if a_mn else a.shape[::-1])
    Kb, N = (b.shape if b_mn else b.shape[::-1])
    assert K_ == Kb, (a.shape, b.shape, a_mn, b_mn)
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    rc = lib().trlb_gemm_bf16(_p(a), _p(b), _p(out), _p(bias), c_int(M), c_int(N), c_int(K_), c_longlong(a.stride(0)),
                              c_longlong(b.stride(0)), c_longlong(out.stride(0)), c_int(int(a_mn)), c_int(int(b_mn)),
                              _p(status_buffer(a.device)), _s())
    _chk(rc, "trlb_gemm_bf16")
    return out


def gemm_pair_bf16(a: torch.Tensor, b: torch.Tensor, bias=None, *, a_mn: bool = False, b_mn: bool = False, out=None):
    """Same contract as :func:`gemm_bf16` on the CTA-pair kernel (``tcgen05`` ``cta_group::2``: two SMs per 256 x 256
    tile, each staging its own rows of ``a`` and half of the ``b`` tile).  Plain store epilogue (+ bias)."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_cuda and a.stride(-1) == 1 and b.stride(-1) == 1
    K_, M = (a.shape if a_mn else a.shape[::-1])
    Kb, N = (b.shape if b_mn else b.shape[::-1])
    assert K_ == Kb, (a.shape, b.shape, a_mn, b_mn)
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    rc = lib().trlb_gemm_pair_bf16(_p(a), _p(b), _p(out), _p(bias), c_int(M), c_int(N), c_int(K_), c_longlong(a.stride(0)),
                                   c_longlong(b.stride(0)), c_longlong(out.stride(0)), c_int(int(a_mn)), c_int(int(b_mn)),
                                   _p(status_buffer(a.device)), _s())
    _chk(rc, "trlb_gemm_pair_bf16")
    return out


def _linear_gemm(*a, **kw):
    """The GEMM of :class:`LinearFn`: the CTA-pair kernel (faster of the two own kernels); ``TRL_B200_GEMM_PAIR=0``
    selects the one-CTA kernel."""
    return (gemm_pair_bf16 if os.environ.get("TRL_B200_GEMM_PAIR", "1") != "0" else gemm_bf16)(*a, **kw)


class LinearFn(torch.autograd.Function):
    """``y = x W^T (+ b)`` with forward, input gradient and weight gradient all on the tcgen05 GEMM (no operand is
    transposed in memory; the bias gradient is a column sum)."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, weight)
        ctx.has_bias, ctx.shape = bias is not None, x.shape
        return _linear_gemm(x2, weight, bias).view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, weight = ctx.saved_tensors
        g2 = gy.reshape(-1, gy.shape[-1])
        if g2.stride(-1) != 1 or g2.stride(0) % 8:
            g2 = g2.contiguous()
        dx = _linear_gemm(g2, weight, b_mn=True).view(ctx.shape) if ctx.needs_input_grad[0] else None
        dw = _linear_gemm(g2, x2, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None
        db = g2.sum(0).to(gy.dtype) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        return dx, dw, db


def linear_own_ok(x, weight) -> bool:
    """Shapes the tcgen05 GEMM takes for all three products of a linear layer (16-byte TMA stride rule)."""
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.stride(-1) == 1
            and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0 and weight.stride(0) % 8 == 0 and x.numel() > 0
            and (x.numel() // x.shape[-1]) % 8 == 0)


_scratch: dict = {}


def _scratch_buf(key, nbytes, device):
    buf = _scratch.get((key, device))
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _scratch[(key, device)] = buf
    return buf


def lmhead_forward(hidden, weight, labels, inv_temp: float, want_entropy=True, want_argmax=False):
    """Fused lm_head GEMM + online softmax.  Returns (logp, entropy|None, lse, argmax|None), fp32 [M]."""
    M, K = hidden.shape
    V = weight.shape[0]
    dev = hidden.device
    L = lib()
    ns = L.trlb_lmhead_num_splits(c_int(M), c_int(V))
    stats = _scratch_buf("lmh_stats", ns * M * 16, dev)
    args = _scratch_buf("lmh_arg", ns * M * 4, dev)
    logp = torch.empty(M, dtype=torch.float32, device=dev)
    lse = torch.empty(M, dtype=torch.float32, device=dev)
    ent = torch.empty(M, dtype=torch.float32, device=dev) if want_entropy else None
    amax = torch.empty(M, dtype=torch.int32, device=dev) if want_argmax else None
    labels = labels.to(torch.int64).contiguous()
    rc = L.trlb_lmhead_fwd(_p(hidden), _p(weight), _p(labels), c_int(M), c_int(V), c_int(K),
                           c_longlong(hidden.stride(0)), c_longlong(weight.stride(0)), c_float(inv_temp),
                           _p(stats), _p(args), c_int(ns), _p(logp), _p(ent), _p(lse), _p(amax),
                           _p(status_buffer(dev)), _s())
    _chk(rc, "trlb_lmhead_fwd")
    return logp, ent, lse, amax


def lmhead_dz(hidden, weight, labels, lse, grow, inv_temp: float, out=None, ent=None, gent=None):
    """dZ[M,V] = grow * (1[label] - softmax(z/T)) / T as bf16 (stage 1 of the lm_head backward); with ``ent`` and
    ``gent`` (entropy and its incoming gradient per row) the entropy's gradient -gent * p (log p + H) / T is added."""
    M, K = hidden.shape
    V = weight.shape[0]
    if out is None:
        out = torch.empty(M, V, dtype=torch.bfloat16, device=hidden.device)
    rc = lib().trlb_lmhead_dz(_p(hidden), _p(weight), _p(labels), _p(lse), _p(grow), _p(ent), _p(gent), _p(out), c_int(M), c_int(V),
                              c_int(K), c_longlong(hidden.stride(0)), c_longlong(weight.stride(0)),
                              c_longlong(out.stride(0)), c_float(inv_temp), _p(status_buffer(hidden.device)), _s())
    _chk(rc, "trlb_lmhead_dz")
    return out


class _LmHeadLogprobFn(torch.autograd.Function):
    """log p(label) (+ entropy) from hidden @ W^T without materialising fp32 logits.

    Backward recomputes the logits tile by tile inside the dZ kernel (bf16 dZ in token chunks),
    then dH = dZ @ W and dW += dZ^T @ H.  The entropy carries a gradient only with ``entropy_grad``
    (the GRPO entropy bonus); otherwise it is a statistic, as in trl/trainer/utils.py:1291-1424.
    """

    CHUNK = 8192

    @staticmethod
    def forward(ctx, hidden, weight, labels, inv_temp, want_entropy, want_argmax, entropy_grad=False):
        hidden = hidden.contiguous()
        labels = labels.to(torch.int64).contiguous()
        logp, ent, lse, amax = lmhead_forward(hidden, weight, labels, inv_temp, want_entropy, want_argmax)
        ctx.entropy_grad = bool(entropy_grad and ent is not None)
        ctx.save_for_backward(hidden, weight, labels, lse, ent if ctx.entropy_grad else None)
        ctx.inv_temp = inv_temp
        ctx.mark_non_differentiable(*[t for t in ((None if ctx.entropy_grad else ent), amax) if t is not None])
        return logp, ent, amax

    @staticmethod
    def backward(ctx, g_logp, g_ent, _ga):
        hidden, weight, labels, lse, ent = ctx.saved_tensors
        M, K = hidden.shape
        V = weight.shape[0]
        g = g_logp.float().contiguous() if g_logp is not None else torch.zeros(M, device=hidden.device)
        ge = g_ent.float().contiguous() if (ctx.entropy_grad and g_ent is not None) else None
        dH = torch.empty_like(hidden) if ctx.needs_input_grad[0] else None
        dW = torch.zeros(V, K, dtype=torch.float32, device=hidden.device) if ctx.needs_input_grad[1] else None
        ck = _LmHeadLogprobFn.CHUNK
        buf = _scratch_buf("lmh_dz", min(ck, M) * V * 2, hidden.device)
        for s in range(0, M, ck):
            e = min(M, s + ck)
            dz = buf[: (e - s) * V * 2].view(torch.bfloat16).view(e - s, V)
            lmhead_dz(hidden[s:e], weight, labels[s:e], lse[s:e], g[s:e], ctx.inv_temp, out=dz,
                      ent=None if ge is None else ent[s:e], gent=None if ge is None else ge[s:e])
            if dH is not None:
                torch.matmul(dz, weight, out=dH[s:e])
            if dW is not None:
                dW += torch.matmul(dz.t(), hidden[s:e]).float()
        return dH, (dW.to(weight.dtype) if dW is not None else None), None, None, None, None, None


def lm_head_logprobs(hidden, weight, labels, temperature=1.0, compute_entropy=True, entropy_grad=False):
    logp, ent, _ = _LmHeadLogprobFn.apply(hidden, weight, labels.clamp_min(0), 1.0 / float(temperature),
                                          compute_entropy, False, entropy_grad)
    return logp, ent


def lm_head_ce(hidden, weight, labels, ignore_index=-100):
    valid = labels != ignore_index
    logp, ent, amax = _LmHeadLogprobFn.apply(hidden, weight, labels.masked_fill(~valid, -1), 1.0, True, True)
    vf = valid.float()
    loss_sum = -(logp * vf).sum()
    with torch.no_grad():
        correct = ((amax.long() == labels) & valid).sum()
        ent_sum = (ent * vf).sum()
    return loss_sum, correct, ent_sum, valid.sum()


# -------------------------------------------------------------------------------------------
# memory-bound fused ops
# -------------------------------------------------------------------------------------------
class RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        shp = x.shape
        H = shp[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        w = weight if weight.dtype == torch.bfloat16 else weight.to(torch.bfloat16)
        _chk(lib().trlb_rmsnorm_fwd(_p(x2), _p(w), _p(y), _p(rstd), c_int(T), c_int(H), c_float(eps), _s()), "rmsnorm_fwd")
        ctx.save_for_backward(x2, w, rstd)
        ctx.shp = shp
        ctx.wdtype = weight.dtype
        return y.view(shp)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        T, H = x2.shape
        dy2 = dy.reshape(T, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        L = lib()
        parts = L.trlb_rmsnorm_bwd_parts(c_int(T))
        scratch = _scratch_buf("rms_dw", parts * H * 4, x2.device)
        dw = torch.empty(H, dtype=torch.float32, device=x2.device)
        _chk(L.trlb_rmsnorm_bwd(_p(dy2), _p(x2), _p(w), _p(rstd), _p(dx), _p(scratch), _p(dw), None, c_int(T), c_int(H),
                                _s()), "rmsnorm_bwd")
        return dx.view(ctx.shp), dw.to(ctx.wdtype), None


class RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, positions, theta):
        T, Hq, D = q.shape
        Hk = k.shape[1]
        assert q.stride(2) == 1 and q.stride(1) == D and k.stride(2) == 1 and k.stride(1) == D
        pos = positions if positions.dtype == torch.int32 else positions.to(torch.int32)
        qo = torch.empty(T, Hq, D, dtype=q.dtype, device=q.device)
        ko = torch.empty(T, Hk, D, dtype=k.dtype, device=k.device)
        _chk(lib().trlb_rope(_p(q), _p(k), c_longlong(q.stride(0)), c_longlong(k.stride(0)), _p(pos), _p(qo), _p(ko),
                             c_int(T), c_int(Hq), c_int(Hk), c_int(D), c_float(theta), c_float(1.0), _s()), "rope")
        ctx.save_for_backward(pos)
        ctx.theta = theta
        return qo, ko

    @staticmethod
    def backward(ctx, dq, dk):
        (pos,) = ctx.saved_tensors
        dq, dk = dq.contiguous(), dk.contiguous()
        T, Hq, D = dq.shape
        Hk = dk.shape[1]
        gq, gk = torch.empty_like(dq), torch.empty_like(dk)
        _chk(lib().trlb_rope(_p(dq), _p(dk), c_longlong(dq.stride(0)), c_longlong(dk.stride(0)), _p(pos), _p(gq), _p(gk),
                             c_int(T), c_int(Hq), c_int(Hk), c_int(D), c_float(ctx.theta), c_float(-1.0), _s()), "rope_bwd")
        return gq, gk, None, None


_ROW_OF_FREQ: dict = {}


class MRopeFn(torch.autograd.Function):
    """Multimodal RoPE on q and k in one kernel: ``positions3`` [3, T] and the frequency sections pick, per rotary
    frequency, which position row turns it; the backward pass is the inverse rotation."""

    @staticmethod
    def forward(ctx, q, k, positions3, theta, sections):
        T, Hq, D = q.shape
        Hk = k.shape[1]
        assert q.stride(2) == 1 and q.stride(1) == D and k.stride(2) == 1 and k.stride(1) == D
        if sum(sections) != D // 2:
            raise ValueError(f"mrope_section {list(sections)} must sum to head_dim / 2 = {D // 2}")
        key = (q.device, tuple(sections))
        rof = _ROW_OF_FREQ.get(key)
        if rof is None:
            rof = _ROW_OF_FREQ[key] = torch.tensor([i % 3 for i, n in enumerate(sections) for _ in range(n)],
                                                   dtype=torch.int32, device=q.device)
        pos = positions3.to(torch.int32).contiguous()
        qo = torch.empty(T, Hq, D, dtype=q.dtype, device=q.device)
        ko = torch.empty(T, Hk, D, dtype=k.dtype, device=k.device)
        _chk(lib().trlb_rope_multi(_p(q), _p(k), c_longlong(q.stride(0)), c_longlong(k.stride(0)), _p(pos), _p(rof), _p(qo),
                                   _p(ko), c_int(T), c_int(Hq), c_int(Hk), c_int(D), c_float(theta), c_float(1.0), _s()),
             "rope_multi")
        ctx.save_for_backward(pos, rof)
        ctx.theta = theta
        return qo, ko

    @staticmethod
    def backward(ctx, dq, dk):
        pos, rof = ctx.saved_tensors
        dq, dk = dq.contiguous(), dk.contiguous()
        T, Hq, D = dq.shape
        Hk = dk.shape[1]
        gq, gk = torch.empty_like(dq), torch.empty_like(dk)
        _chk(lib().trlb_rope_multi(_p(dq), _p(dk), c_longlong(dq.stride(0)), c_longlong(dk.stride(0)), _p(pos), _p(rof),
                                   _p(gq), _p(gk), c_int(T), c_int(Hq), c_int(Hk), c_int(D), c_float(ctx.theta),
                                   c_float(-1.0), _s()), "rope_multi_bwd")
        return gq, gk, None, None, None


class SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        shp = gate_up.shape
        I = shp[-1] // 2
        gu = gate_up.reshape(-1, 2 * I)
        if not gu.is_contiguous():
            gu = gu.contiguous()
        out = torch.empty(gu.shape[0], I, dtype=gu.dtype, device=gu.device)
        _chk(lib().trlb_swiglu_fwd(_p(gu), _p(out), c_longlong(gu.shape[0]), c_int(I), _s()), "swiglu_fwd")
        ctx.save_for_backward(gu)
        ctx.shp = shp
        return out.view(shp[:-1] + (I,))

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        I = gu.shape[1] // 2
        d = dout.reshape(-1, I)
        if not d.is_contiguous():
            d = d.contiguous()
        dgu = torch.empty_like(gu)
        _chk(lib().trlb_swiglu_bwd(_p(d), _p(gu), _p(dgu), c_longlong(gu.shape[0]), c_int(I), _s()), "swiglu_bwd")
        return dgu.view(ctx.shp)


def adamw_flat(master, grad, m, v, step, lr, b1, b2, eps, wd, grad_scale=1.0, shadow=None):
    """Fused AdamW over a flat fp32 shard; ``grad_scale`` may be a 0-dim CUDA tensor (no host sync)."""
    gs_ptr, gs = None, 1.0
    if torch.is_tensor(grad_scale):
        gs_t = grad_scale.reshape(1).float()
        gs_ptr = gs_t
    else:
        gs = float(grad_scale)
    assert grad.dtype in (torch.float32, torch.bfloat16) and master.dtype == torch.float32
    _chk(lib().trlb_adamw(_p(master), _p(grad), c_int(int(grad.dtype == torch.bfloat16)), _p(m), _p(v), _p(shadow),
                          c_longlong(master.numel()), c_int(step), c_float(lr), c_float(b1), c_float(b2), c_float(eps),
                          c_float(wd), c_float(gs), _p(gs_ptr), _s()), "adamw")


def sumsq(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    _chk(lib().trlb_sumsq(_p(x), c_int(int(x.dtype == torch.bfloat16)), c_longlong(x.numel()), _p(out), _s()), "sumsq")
    return out


# -------------------------------------------------------------------------------------------
# attention
# -------------------------------------------------------------------------------------------
def fa_varlen_fwd(q, k, v, cu_q, cu_k, causal=True, window=None, scale=None):
    """Forward of the tcgen05 varlen attention.  q [Tq, Hq, 128], k / v [Tk, Hk, 128] bf16 (any row stride; the last
    two dimensions dense), cu_q / cu_k int32 device tensors.  Returns (out [Tq, Hq, 128] bf16, lse [Hq, Tq] fp32)."""
    Tq, Hq, Dh = q.shape
    Tk, Hk, _ = k.shape
    for t in (q, k, v):
        assert t.dtype == torch.bfloat16 and t.stride(2) == 1 and t.stride(1) == Dh
    out = torch.empty(Tq, Hq, Dh, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(Hq, Tq, dtype=torch.float32, device=q.device)
    sc = float(scale) if scale is not None else 1.0 / Dh ** 0.5
    _chk(lib().trlb_fa_varlen_fwd(_p(q), _p(k), _p(v), c_longlong(q.stride(0)), c_longlong(k.stride(0)),
                                  c_longlong(v.stride(0)), _p(cu_q), _p(cu_k), c_int(cu_q.numel() - 1), c_int(Tq), c_int(Tk),
                                  c_int(Hq), c_int(Hk), c_int(Dh), c_float(sc), c_int(int(bool(causal))),
                                  c_int(int(window or 0)), _p(out), c_longlong(out.stride(0)), _p(lse),
                                  _p(status_buffer(q.device)), _s()), "fa_varlen_fwd")
    return out, lse


def fa_varlen_bwd(q, k, v, out, dout, lse, cu_q, cu_k, causal=True, window=None, scale=None):
    """Backward of :func:`fa_varlen_fwd`: returns (dq, dk, dv) bf16, shaped like q / k / v (contiguous)."""
    Tq, Hq, Dh = q.shape
    Tk, Hk, _ = k.shape
    dout = dout if (dout.stride(2) == 1 and dout.stride(1) == Dh) else dout.contiguous()
    dq = torch.empty(Tq, Hq, Dh, dtype=torch.bfloat16, device=q.device)
    dk = torch.empty(Tk, Hk, Dh, dtype=torch.bfloat16, device=q.device)
    dv = torch.empty(Tk, Hk, Dh, dtype=torch.bfloat16, device=q.device)
    delta = torch.empty(Hq, Tq, dtype=torch.float32, device=q.device)
    sc = float(scale) if scale is not None else 1.0 / Dh ** 0.5
    _chk(lib().trlb_fa_varlen_bwd(_p(q), _p(k), _p(v), _p(out), _p(dout), c_longlong(q.stride(0)), c_longlong(k.stride(0)),
                                  c_longlong(v.stride(0)), c_longlong(out.stride(0)), c_longlong(dout.stride(0)), _p(cu_q),
                                  _p(cu_k), c_int(cu_q.numel() - 1), c_int(Tq), c_int(Tk), c_int(Hq), c_int(Hk), c_int(Dh),
                                  c_float(sc), c_int(int(bool(causal))), c_int(int(window or 0)), _p(lse), _p(delta), _p(dq),
                                  _p(dk), _p(dv), c_longlong(dq.stride(0)), c_longlong(dk.stride(0)), c_longlong(dv.stride(0)),
                                  _p(status_buffer(q.device)), _s()), "fa_varlen_bwd")
    LAUNCHES[0] += 2  # delta + two gradient kernels behind one entry point
    return dq, dk, dv


class AttnKeep:
    """Attention outputs kept across the recompute of activation checkpointing.

    A checkpointed layer runs its forward twice: once when the model is evaluated and once more, inside backward, to
    rebuild what autograd needs.  Everything in the layer is cheap to rebuild except attention, whose cost grows
    with the square of the sequence length, while its output is one [tokens, hidden] tensor.  The decoder therefore
    names every checkpointed layer call (``with AttnKeep.scope((forward_id, layer)):``): the first attention call
    under a name stores its output and log-sum-exp, the second one (the recompute) takes them back instead of
    launching the kernel.  A new forward pass drops whatever an abandoned one left behind."""

    store: dict = {}
    current = None
    forward_id = 0
    enabled = os.environ.get("TRL_B200_KEEP_ATTN", "1") != "0"

    @classmethod
    def new_forward(cls) -> int:
        cls.forward_id += 1
        cls.store.clear()  # whatever a forward pass without a backward pass left behind
        return cls.forward_id

    class scope:
        def __init__(self, key):
            self.key = key

        def __enter__(self):
            self.prev, AttnKeep.current = AttnKeep.current, (self.key if AttnKeep.enabled else None)

        def __exit__(self, *exc):
            AttnKeep.current = self.prev


class _FaVarlenFn(torch.autograd.Function):
    """Varlen attention on the tcgen05 kernels (csrc/fa_varlen_tcgen05.cu): grouped-query heads are indexed, never
    expanded; the backward recomputes the probabilities from the saved log-sum-exp."""

    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, causal, window):
        key = AttnKeep.current
        kept = AttnKeep.store.pop(key, None) if key is not None else None
        if kept is not None and kept[0].shape == q.shape:
            out, lse = kept  # the recompute of a checkpointed layer: same inputs, same result
        else:
            out, lse = fa_varlen_fwd(q, k, v, cu_q, cu_k, causal, window)
            if key is not None:
                AttnKeep.store[key] = (out.detach(), lse)
        ctx.save_for_backward(q, k, v, out, lse, cu_q, cu_k)
        ctx.causal, ctx.window = causal, window
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
        dq, dk, dv = fa_varlen_bwd(q, k, v, out, dout, lse, cu_q, cu_k, ctx.causal, ctx.window)
        return dq, dk, dv, None, None, None, None


def _fa_ok(q, k, v) -> bool:
    def dense_heads(t):
        return t.stride(2) == 1 and t.stride(1) == t.shape[2] and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0

    return (q.dtype == torch.bfloat16 and q.shape[2] == 128 and k.shape[2] == 128 and q.shape[1] % k.shape[1] == 0
            and all(dense_heads(t) for t in (q, k, v)))


def _i32(cu, device):
    return cu if (cu.dtype == torch.int32 and cu.device == device) else cu.to(device=device, dtype=torch.int32)


def attention_varlen(q, k, v, cu_seqlens, max_seqlen, causal=True, window=None):
    """Causal GQA attention over packed documents [T, H, D]; ``window`` = sliding-window size or None.  head_dim 128
    in bf16 runs on this library's tcgen05 kernels (forward and backward); other shapes use the library kernel."""
    if _fa_ok(q, k, v) and (causal or not window):
        cu = _i32(cu_seqlens, q.device)
        return _FaVarlenFn.apply(q, k, v, cu, cu, bool(causal), int(window) if window else None)
    from torch.nn.attention.varlen import varlen_attn

    cu = cu_seqlens.to(torch.int32)
    Hq, Hk = q.shape[1], k.shape[1]
    if Hq != Hk:
        rep = Hq // Hk
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
    left = int(window) - 1 if window else -1
    return varlen_attn(q.contiguous(), k.contiguous(), v.contiguous(), cu, cu, int(max_seqlen), int(max_seqlen),
                       window_size=(left, 0) if causal else (left, left))


def attention_varlen_qk(q, k, v, cu_q, cu_k, max_q, max_k):
    """Causal GQA attention with separate query / key segments [Tq, H, D] x [Tk, Hk, D]; the causal mask is aligned to
    the end of each key segment (query i sees keys up to i + len_k - len_q)."""
    if _fa_ok(q, k, v):
        return _FaVarlenFn.apply(q, k, v, _i32(cu_q, q.device), _i32(cu_k, q.device), True, None)
    from torch.nn.attention.varlen import varlen_attn

    Hq, Hk = q.shape[1], k.shape[1]
    if Hq != Hk:
        rep = Hq // Hk
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
    return varlen_attn(q.contiguous(), k.contiguous(), v.contiguous(), cu_q.to(torch.int32), cu_k.to(torch.int32),
                       int(max_q), int(max_k), window_size=(-1, 0))


def grouped_gemm(a, w, offsets, n_out, swiglu=False, out=None, w_transposed=False):
    """Per-expert GEMM on tcgen05: rows of ``a`` [R, K] are sorted by expert, ``offsets`` [E + 1] int32 on the device,
    ``w`` [E, n_out (or 2 * n_out with swiglu), K].  Returns [R, n_out]; with ``swiglu`` the gate / up halves are
    combined in the epilogue.  ``w_transposed``: ``w`` is [E, K, n_out] and is read as it lies (the input gradient of
    a layer whose forward weight is ``w``)."""
    R, Kd = a.shape
    E = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and a.stride(1) == 1
    if w_transposed:
        assert not swiglu and w.shape[1] == Kd and w.shape[2] == n_out
    else:
        assert w.shape[1] == (2 * n_out if swiglu else n_out) and w.shape[2] == Kd
    if out is None:
        out = torch.empty(R, n_out, dtype=torch.bfloat16, device=a.device)
    _chk(lib().trlb_grouped_gemm_bf16(_p(a), _p(w), _p(offsets), _p(out), c_longlong(R), c_int(E), c_int(n_out), c_int(Kd),
                                      c_longlong(a.stride(0)), c_longlong(out.stride(0)), c_int(int(swiglu)),
                                      c_int(int(w_transposed)), _p(status_buffer(a.device)), _s()), "grouped_gemm")
    return out


def grouped_wgrad(g, x, offsets, num_experts, out=None):
    """Per-expert weight gradient on tcgen05: ``out[e] = g[rows of e]^T @ x[rows of e]`` with ``g`` [R, N], ``x``
    [R, K] sorted by expert and ``offsets`` [E + 1] int32 on the device; returns [E, N, K] bf16 (zeros for an expert
    without rows).  Neither operand is transposed in memory and nothing is read back to the host."""
    R, N = g.shape
    Kd = x.shape[1]
    assert g.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and g.stride(1) == 1 and x.stride(1) == 1
    assert x.shape[0] == R
    if out is None:
        out = torch.empty(num_experts, N, Kd, dtype=torch.bfloat16, device=g.device)
    _chk(lib().trlb_grouped_wgrad_bf16(_p(g), _p(x), _p(offsets), _p(out), c_longlong(R), c_int(num_experts), c_int(N),
                                       c_int(Kd), c_longlong(g.stride(0)), c_longlong(x.stride(0)),
                                       _p(status_buffer(g.device)), _s()), "grouped_wgrad")
    return out


def moe_combine_bwd(d_out, y_perm, order, topk_w, d_y=None):
    """Backward of the weighted combine in one pass: ``d_y[r] = w[order[r]] * d_out[order[r] // k]`` (bf16, written to
    ``d_y`` when given) and ``d_w[order[r]] = <d_out[order[r] // k], y_perm[r]>`` (fp32, shaped like ``topk_w``)."""
    rows, H = y_perm.shape
    k = topk_w.shape[1]
    d_y = torch.empty(rows, H, dtype=torch.bfloat16, device=d_out.device) if d_y is None else d_y
    d_w = torch.empty(topk_w.numel(), dtype=torch.float32, device=d_out.device)
    assert d_out.dtype == torch.bfloat16 and y_perm.dtype == torch.bfloat16 and order.dtype == torch.int64
    assert d_y.is_contiguous() and y_perm.is_contiguous()
    _chk(lib().trlb_moe_combine_bwd(_p(d_out.contiguous()), _p(y_perm), _p(order), _p(topk_w.float().contiguous()),
                                    _p(d_y), _p(d_w), c_longlong(rows), c_int(k), c_int(H), _s()), "moe_combine_bwd")
    return d_y, d_w.view_as(topk_w)


def moe_gather_sum(rows, inv, T, k):
    """``out[t] = sum_j rows[inv[t, j]]`` (bf16): the scatter-add of permuted rows back to tokens, as a gather."""
    H = rows.shape[1]
    out = torch.empty(T, H, dtype=torch.bfloat16, device=rows.device)
    ones = torch.ones(T * k, dtype=torch.float32, device=rows.device)
    _chk(lib().trlb_moe_combine(_p(rows), _p(inv), _p(ones), _p(out), c_int(T), c_int(k), c_int(H), _s()), "moe_combine")
    return out


class _MoeExpertsFn(torch.autograd.Function):
    """Sort tokens by expert, gate/up grouped GEMM with SwiGLU epilogue, down grouped GEMM, weighted combine.
    Backward recomputes the gate/up pre-activations with the same kernel; input gradients read the forward weights
    transposed through the grouped kernel and weight gradients come from the grouped weight-gradient kernel, so the
    backward has no per-expert loop and never reads the token counts back to the host."""

    @staticmethod
    def forward(ctx, hidden, gate_up_w, down_w, topk_w, topk_idx):
        T, H = hidden.shape
        k = topk_idx.shape[1]
        E, I2, _ = gate_up_w.shape
        I = I2 // 2
        flat_e = topk_idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        counts = torch.zeros(E, dtype=torch.int32, device=hidden.device)
        counts.scatter_add_(0, flat_e, torch.ones_like(flat_e, dtype=torch.int32))  # no host sync: graph-capturable
        offsets = torch.zeros(E + 1, dtype=torch.int32, device=hidden.device)
        offsets[1:] = counts.cumsum(0)
        tok = order // k
        x_perm = hidden.index_select(0, tok)
        act = grouped_gemm(x_perm, gate_up_w, offsets, I, swiglu=True)
        y_perm = grouped_gemm(act, down_w, offsets, H)
        inv = torch.empty(T * k, dtype=torch.int32, device=hidden.device)
        inv[order] = torch.arange(T * k, dtype=torch.int32, device=hidden.device)
        out = torch.empty(T, H, dtype=torch.bfloat16, device=hidden.device)
        _chk(lib().trlb_moe_combine(_p(y_perm), _p(inv), _p(topk_w.float().contiguous()), _p(out), c_int(T), c_int(k),
                                    c_int(H), _s()), "moe_combine")
        ctx.save_for_backward(hidden, gate_up_w, down_w, topk_w, order, offsets, act, y_perm, inv)
        ctx.k = k
        return out

    @staticmethod
    def backward(ctx, d_out):
        hidden, gate_up_w, down_w, topk_w, order, offsets, act, y_perm, inv = ctx.saved_tensors
        k = ctx.k
        E, I2, H = gate_up_w.shape
        I = I2 // 2
        T = hidden.shape[0]
        d_y, d_topk_w = moe_combine_bwd(d_out, y_perm, order, topk_w)
        # down projection: y = act @ Wd[e]^T with Wd[e] [H, I]  ->  d_act = d_y @ Wd[e],  dWd[e] = d_y^T @ act
        d_act = grouped_gemm(d_y, down_w, offsets, I, w_transposed=True)
        d_down = grouped_wgrad(d_y, act, offsets, E)
        x_perm = hidden.index_select(0, order // k)
        gu = grouped_gemm(x_perm, gate_up_w, offsets, I2, swiglu=False)  # recompute the pre-activations
        d_gu = torch.empty_like(gu)
        _chk(lib().trlb_swiglu_bwd(_p(d_act), _p(gu), _p(d_gu), c_longlong(gu.shape[0]), c_int(I), _s()), "swiglu_bwd")
        # gate/up projection: gu = x @ Wgu[e]^T with Wgu[e] [2I, H]  ->  d_x = d_gu @ Wgu[e],  dWgu[e] = d_gu^T @ x
        d_x = grouped_gemm(d_gu, gate_up_w, offsets, H, w_transposed=True)
        d_gate_up = grouped_wgrad(d_gu, x_perm, offsets, E)
        d_hidden = moe_gather_sum(d_x, inv, T, k)
        return d_hidden, d_gate_up, d_down, d_topk_w.to(topk_w.dtype), None


def moe_experts(hidden, gate_up_w, down_w, topk_w, topk_idx):
    if hidden.dtype != torch.bfloat16 or hidden.shape[1] % 8 or (gate_up_w.shape[1] // 2) % 8:
        from ..oracle.ops import moe_experts as ref

        return ref(hidden, gate_up_w, down_w, topk_w, topk_idx)
    return _MoeExpertsFn.apply(hidden.contiguous(), gate_up_w, down_w, topk_w, topk_idx)


# -------------------------------------------------------------------------------------------
# fused losses
# -------------------------------------------------------------------------------------------
_AUX_SCRATCH: dict = {}


class _MoeAuxLossFn(torch.autograd.Function):
    """Router load-balancing loss ``E * sum_e f_e P_e`` in one reduction kernel (csrc/moe.cu); the gradient reaches the
    router probabilities only (f counts hard assignments): ``dL/dP[n, e] = E f_e mask_n / valid``."""

    @staticmethod
    def forward(ctx, probs, idx, num_experts, mask):
        N, E = probs.shape
        K = idx.shape[1]
        dev = probs.device
        key = (dev, E)
        acc = _AUX_SCRATCH.get(key)
        if acc is None:
            acc = _AUX_SCRATCH[key] = torch.zeros(2 * E + 2, dtype=torch.float32, device=dev)
        out = torch.empty(E + 2, dtype=torch.float32, device=dev)  # [loss, valid, f_0 .. f_{E-1}]
        p = probs if probs.dtype in (torch.float32, torch.bfloat16) else probs.float()
        p = p.contiguous()
        m = None if mask is None else mask.reshape(-1).float().contiguous()
        _chk(lib().trlb_moe_aux_loss(_p(p), c_int(int(p.dtype == torch.bfloat16)), _p(idx.to(torch.int64).contiguous()),
                                     _p(m), c_int(N), c_int(E), c_int(K), _p(acc), _p(out[0:1]), _p(out[2:]), _p(out[1:2]),
                                     _s()), "moe_aux_loss")
        ctx.save_for_backward(out, m)
        ctx.E, ctx.dtype = E, probs.dtype
        return out[0].clone()

    @staticmethod
    def backward(ctx, g):
        out, m = ctx.saved_tensors
        row = (g * ctx.E / out[1]) * out[2:]
        return (m[:, None] * row[None, :]).to(ctx.dtype), None, None, None


def moe_aux_loss(probs, idx, num_experts, mask=None):
    if mask is None:  # the backward needs the row count: give it an explicit all-ones mask
        mask = torch.ones(probs.shape[0], dtype=torch.float32, device=probs.device)
    return _MoeAuxLossFn.apply(probs, idx, num_experts, mask)


class GrpoLossFn(torch.autograd.Function):
    """Clipped-ratio + KL token loss, reduced with per-row scales; returns (loss, stats[8])."""

    @staticmethod
    def forward(ctx, logp, old_logp, ref_logp, adv, mask, row_scale, entropy, eps_low, eps_high, beta, delta):
        B, T = logp.shape
        dev = logp.device
        f = lambda t: None if t is None else t.float().contiguous()
        logp_c = f(logp)
        dlogp = torch.empty(B, T, dtype=torch.float32, device=dev)
        stats = torch.zeros(8, dtype=torch.float32, device=dev)
        _chk(lib().trlb_grpo_loss(_p(logp_c), _p(f(old_logp)), _p(f(ref_logp)), _p(f(adv)), _p(f(mask)), _p(f(row_scale)),
                                  _p(f(entropy)), _p(dlogp), None, _p(stats), c_int(B), c_int(T), c_float(eps_low),
                                  c_float(eps_high), c_float(beta), c_float(delta if delta else 0.0), c_float(1.0), _s()),
             "grpo_loss")
        ctx.save_for_backward(dlogp)
        ctx.mark_non_differentiable(stats)
        return stats[0].clone(), stats

    @staticmethod
    def backward(ctx, g_loss, _g_stats):
        (dlogp,) = ctx.saved_tensors
        return (dlogp * g_loss,) + (None,) * 10


def grpo_loss(logp, old_logp, ref_logp, adv, mask, row_scale, entropy, eps_low, eps_high, beta, delta=None):
    return GrpoLossFn.apply(logp, old_logp, ref_logp, adv, mask, row_scale, entropy, eps_low, eps_high, beta, delta)


class DpoLossFn(torch.autograd.Function):
    """Sigmoid DPO over a packed token stream; returns (mean loss, per-pair metrics [P, 8])."""

    @staticmethod
    def forward(ctx, pol_logp, ref_logp, mask, cu_seqlens, beta, label_smoothing):
        P = (cu_seqlens.numel() - 1) // 2
        dev = pol_logp.device
        pol = pol_logp.float().contiguous()
        dpol = torch.empty_like(pol)
        out = torch.empty(P, 8, dtype=torch.float32, device=dev)
        _chk(lib().trlb_dpo_loss(_p(pol), _p(ref_logp.float().contiguous()), _p(mask.float().contiguous()),
                                 _p(cu_seqlens.to(torch.int32).contiguous()), c_int(P), c_float(beta),
                                 c_float(label_smoothing), c_float(1.0 / max(P, 1)), _p(dpol), _p(out), _s()), "dpo_loss")
        ctx.save_for_backward(dpol)
        ctx.mark_non_differentiable(out)
        return out[:, 0].mean(), out

    @staticmethod
    def backward(ctx, g, _go):
        (dpol,) = ctx.saved_tensors
        return dpol * g, None, None, None, None, None


def dpo_loss(pol_logp, ref_logp, mask, cu_seqlens, beta, label_smoothing=0.0):
    return DpoLossFn.apply(pol_logp, ref_logp, mask, cu_seqlens, beta, label_smoothing)


# -------------------------------------------------------------------------------------------
# rollout-engine decode kernels (no autograd)
# -------------------------------------------------------------------------------------------
def rmsnorm_infer(x, w, eps, out=None):
    T, H = x.shape
    out = torch.empty_like(x) if out is None else out
    _chk(lib().trlb_rmsnorm_fwd(_p(x), _p(w), _p(out), None, c_int(T), c_int(H), c_float(eps), _s()), "rmsnorm_fwd")
    return out


def add_rmsnorm_infer(res, delta, w, eps, out=None):
    """res += delta (in place); returns rmsnorm(res) * w."""
    T, H = res.shape
    out = torch.empty_like(res) if out is None else out
    _chk(lib().trlb_add_rmsnorm(_p(res), _p(delta), _p(w), _p(out), c_int(T), c_int(H), c_float(eps), _s()), "add_rmsnorm")
    return out


def add_rmsnorm_f32_infer(res, delta32, w, eps, out=None):
    """res += delta32 (fp32 partial sums of the split-K decode GEMM, cleared here); returns rmsnorm(res) * w."""
    T, H = res.shape
    assert delta32.dtype == torch.float32 and delta32.is_contiguous()
    out = torch.empty_like(res) if out is None else out
    _chk(lib().trlb_add_rmsnorm_f32(_p(res), _p(delta32), _p(w), _p(out), c_int(T), c_int(H), c_float(eps), _s()),
         "add_rmsnorm_f32")
    return out


def add_rmsnorm_f32_wait(res, delta32, w, eps, arrive_ptr: int, target: int, done_ptr: int, out=None):
    """Consumer of a row-parallel :func:`decode_gemm` fused with its all-reduce: waits (bounded) until the arrival
    counter at ``arrive_ptr`` has reached ``target`` (ranks x GEMM CTAs), then ``res += delta32`` (cleared) and returns
    ``rmsnorm(res) * w``; the counter is taken back down by ``target`` when the last row is done."""
    T, H = res.shape
    assert delta32.dtype == torch.float32 and delta32.is_contiguous()
    out = torch.empty_like(res) if out is None else out
    _chk(lib().trlb_add_rmsnorm_f32_wait(_p(res), _p(delta32), _p(w), _p(out), c_int(T), c_int(H), c_float(eps),
                                         c_void_p(arrive_ptr), ctypes.c_uint(target), c_void_p(done_ptr),
                                         _p(status_buffer(res.device)), _s()), "add_rmsnorm_f32_wait")
    return out


def tp_token_sync(mail_ptrs, flag_ptrs, rank: int, world: int, tok, logp, epoch_word):
    """Rank 0's sampled tokens and log-probs replace those of the other ranks of a tensor-parallel decode group
    (``mail_ptrs`` / ``flag_ptrs``: every rank's mailbox and flag address in symmetric memory)."""
    B = tok.shape[0]
    mails = (ctypes.c_ulonglong * world)(*mail_ptrs)
    flags = (ctypes.c_ulonglong * world)(*flag_ptrs)
    _chk(lib().trlb_tp_token_sync(mails, flags, c_int(rank), c_int(world), _p(tok), _p(logp), c_int(B), _p(epoch_word),
                                  _p(status_buffer(tok.device)), _s()), "tp_token_sync")


def accum_grad(dst32, src_bf16):
    """dst32 (fp32 main gradient, contiguous) += src (bf16 gradient of one micro-batch)."""
    _chk(lib().trlb_accum_bf16_f32(_p(dst32), _p(src_bf16), c_longlong(dst32.numel()), _s()), "accum_grad")


def set_pdl(on: bool) -> bool:
    """Programmatic dependent launch for the decode-path kernels (their prologues and the first ring of weight tiles
    overlap the tail of the kernel before them).  Returns the previous setting.  Choose before a CUDA graph is captured."""
    return bool(lib().trlb_set_pdl(c_int(int(bool(on)))))


def decode_gemm(x, w, bias=None, *, y32=None, out=None, swiglu=False, max_ctas: int = 0, tiled_shape=None,
                peers=None):
    """Weight-streaming tcgen05 GEMM for decode batches (at most 128 rows of ``x``).

    ``y32`` given: ``y32[B, N] (fp32) += x @ w^T (+ bias)``, work split stream-K style over every SM; the caller passes
    zeros (the consumer kernels clear the buffer after reading it).  Otherwise bf16 ``out[B, N] = x @ w^T (+ bias)``;
    with ``swiglu`` ``w`` is ``[2N, K]`` (gate rows, then up rows) and ``out = silu(x Wg^T) * (x Wu^T)``.

    ``tiled_shape=(rows, K)``: ``w`` is the flat tile-major copy made by :func:`tile_weights` of a ``[rows, K]`` weight.
    ``peers=(peer_y32_ptrs, arrive_ptrs, stage, slab_ctr)``: row-parallel GEMM fused with its all-reduce: partial sums
    are collected in the local fp32 ``stage`` (shaped like ``y32``, zeros; left zeroed) and every finished 32-feature
    quarter of a slab is added once into ``y32`` and the peers' buffers (device addresses), bumping every rank's
    arrival counter (``arrive_ptrs[0]`` is this rank's own); ``slab_ctr``: zeroed int32 words, four per 128 features.
    A consumer waits for ``ranks * decode_gemm_arrivals(N)``."""
    B, Kd = x.shape
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1
    if tiled_shape is not None:
        rows, kw = tiled_shape
        assert kw == Kd and w.is_contiguous()
        ldw = 0
    else:
        assert w.stride(1) == 1 and w.shape[1] == Kd
        rows, ldw = w.shape[0], w.stride(0)
    N = rows // 2 if swiglu else rows
    if y32 is not None:
        assert y32.dtype == torch.float32 and y32.stride(1) == 1 and tuple(y32.shape) == (B, N) and not swiglu
        mode, ldy, dst32, dstb, ret = 0, y32.stride(0), y32, None, y32
    else:
        if out is None:
            out = torch.empty(B, N, dtype=torch.bfloat16, device=x.device)
        assert out.dtype == torch.bfloat16 and out.stride(1) == 1 and tuple(out.shape) == (B, N)
        mode, ldy, dst32, dstb, ret = (2 if swiglu else 1), out.stride(0), None, out, out
    n_peers, peer_arr, arrive_arr, stage, slab_ctr = 0, None, None, None, None
    if peers is not None:
        peer_ptrs, arrive_ptrs, stage, slab_ctr = peers
        n_peers = len(peer_ptrs)
        assert mode == 0 and len(arrive_ptrs) == n_peers + 1
        if n_peers:
            assert stage.dtype == torch.float32 and stage.stride() == y32.stride() and slab_ctr.numel() * 32 >= N
        peer_arr = (c_void_p * max(1, n_peers))(*peer_ptrs) if n_peers else None
        arrive_arr = (c_void_p * (n_peers + 1))(*arrive_ptrs)
    _chk(lib().trlb_decode_gemm(_p(x), _p(w), _p(bias), _p(dst32), _p(dstb), c_int(B), c_int(N), c_int(Kd),
                                c_longlong(x.stride(0)), c_longlong(ldw), c_longlong(ldy), c_int(mode),
                                c_int(int(tiled_shape is not None)), c_int(max_ctas), c_int(n_peers), peer_arr, arrive_arr,
                                _p(stage), _p(slab_ctr), _p(status_buffer(x.device)), _s()), "decode_gemm")
    return ret


def decode_gemm_ctas(B: int, N: int, K: int, mode: int = 0, max_ctas: int = 0) -> int:
    """Grid size :func:`decode_gemm` uses for ``B`` rows and an ``[N, K]`` weight (mode 0: fp32 sums, 1: bf16 store,
    2: SwiGLU)."""
    return int(lib().trlb_decode_gemm_ctas(c_int(B), c_int(N), c_int(K), c_int(mode), c_int(max_ctas)))


def decode_gemm_arrivals(N: int) -> int:
    """Arrival-counter increments per rank of one fused all-reduce :func:`decode_gemm` with ``N`` output features."""
    return int(lib().trlb_decode_gemm_arrivals(c_int(N)))


def tile_weights(w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Tile-major copy of a row-major ``[rows, K]`` bf16 weight for :func:`decode_gemm` (``tiled_shape=(rows, K)``):
    ``[ceil(rows/128)][ceil(K/64)][128][64]``, every 16 KB tile contiguous, zero padded."""
    rows, Kd = w.shape
    assert w.dtype == torch.bfloat16 and w.stride(1) == 1
    L = lib()
    L.trlb_tiled_elems.restype = c_longlong
    n = int(L.trlb_tiled_elems(c_int(rows), c_int(Kd)))
    if out is None:
        out = torch.empty(n, dtype=torch.bfloat16, device=w.device)
    assert out.numel() == n and out.is_contiguous() and out.dtype == torch.bfloat16
    _chk(L.trlb_tile_weights(_p(w), c_longlong(w.stride(0)), _p(out), c_int(rows), c_int(Kd), _s()), "tile_weights")
    return out


def swiglu_infer(gu, out=None):
    T, I2 = gu.shape
    out = torch.empty(T, I2 // 2, dtype=gu.dtype, device=gu.device) if out is None else out
    _chk(lib().trlb_swiglu_fwd(_p(gu), _p(out), c_longlong(T), c_int(I2 // 2), _s()), "swiglu_fwd")
    return out


def rope_kv_write(qkv, seq_lens, slot_ids, block_table, block_size, q_out, k_cache, v_cache, Hq, Hk, D, theta,
                  v_transposed=False, pos_delta=None):
    """RoPE on q/k of the new tokens, q -> q_out, k/v appended to the paged cache.  ``v_transposed``: the V cache is
    [block, head, dim, token] (layout of the tensor-core decode attention) instead of [block, token, head, dim].
    ``pos_delta`` (int32 per slot, optional): rotary position = cache position + delta (multimodal RoPE, where an
    image of many tokens advances the position by less than its token count)."""
    B = qkv.shape[0]
    _chk(lib().trlb_rope_kv_write(_p(qkv), c_longlong(qkv.stride(0)), _p(seq_lens), _p(slot_ids), _p(block_table),
                                  c_int(block_table.shape[1]), c_int(block_size), _p(q_out), _p(k_cache), _p(v_cache),
                                  c_int(B), c_int(Hq), c_int(Hk), c_int(D), c_float(theta), c_int(int(v_transposed)),
                                  _p(pos_delta), _s()),
         "rope_kv_write")


def rope_kv_write_f32(acc, bias, q_norm, k_norm, norm_eps, seq_lens, slot_ids, block_table, block_size, q_out, k_cache,
                      v_cache, Hq, Hk, D, theta, v_transposed=False, pos_delta=None):
    """Like :func:`rope_kv_write` for the fp32 sums of the stream-K QKV GEMM: adds ``bias``, applies the per-head
    RMSNorm of q / k when ``q_norm`` / ``k_norm`` are given, rotates, appends, and clears ``acc``."""
    B = acc.shape[0]
    assert acc.dtype == torch.float32 and acc.stride(1) == 1
    _chk(lib().trlb_rope_kv_write_f32(_p(acc), c_longlong(acc.stride(0)), _p(bias), _p(q_norm), _p(k_norm),
                                      c_float(norm_eps), _p(seq_lens), _p(slot_ids), _p(block_table),
                                      c_int(block_table.shape[1]), c_int(block_size), _p(q_out), _p(k_cache), _p(v_cache),
                                      c_int(B), c_int(Hq), c_int(Hk), c_int(D), c_float(theta), c_int(int(v_transposed)),
                                      _p(pos_delta), _s()), "rope_kv_write_f32")


def kv_write_prefill(k, v, tok_slot, tok_pos, block_table, block_size, k_cache, v_cache, v_transposed=False):
    T, Hk, D = k.shape
    _chk(lib().trlb_kv_write_prefill(_p(k), _p(v), c_longlong(k.stride(0)), c_longlong(v.stride(0)), _p(tok_slot),
                                     _p(tok_pos), _p(block_table), c_int(block_table.shape[1]), c_int(block_size),
                                     _p(k_cache), _p(v_cache), c_int(T), c_int(Hk), c_int(D), c_int(int(v_transposed)), _s()),
         "kv_write_prefill")


def paged_decode_attn(q, k_cache, v_cache, seq_lens, slot_ids, block_table, block_size, scale, splits, part_o, part_ml,
                      out):
    B, Hq, D = q.shape
    Hk = k_cache.shape[2]
    _chk(lib().trlb_paged_decode_attn(_p(q), _p(k_cache), _p(v_cache), _p(seq_lens), _p(slot_ids), _p(block_table),
                                      c_int(block_table.shape[1]), c_int(block_size), c_int(B), c_int(Hq), c_int(Hk),
                                      c_int(D), c_float(scale), c_int(splits), _p(part_o), _p(part_ml), _p(out), _s()),
         "paged_decode_attn")
    return out


def paged_decode_attn_tc(q, k_cache, v_cache_t, seq_lens, slot_ids, block_table, scale, splits, part_o, part_ml, out,
                         groups: int = 1):
    """Tensor-core (tcgen05) decode attention.  k_cache [blocks, 64, Hk, 128]; v_cache_t [blocks, Hk, 128, 64].
    ``groups=2`` runs the variant with two softmax warp groups per CTA that take alternate 128-token tiles."""
    B, Hq, D = q.shape
    nb, bs, Hk, Dk = k_cache.shape
    if D != 128 or Dk != 128 or bs != 64 or tuple(v_cache_t.shape) != (nb, Hk, 128, 64):
        raise ValueError("paged_decode_attn_tc needs head_dim 128, 64-token pages and a transposed V cache")
    fn = lib().trlb_paged_decode_attn_tc2 if groups == 2 else lib().trlb_paged_decode_attn_tc
    _chk(fn(_p(q), _p(k_cache), _p(v_cache_t), _p(seq_lens), _p(slot_ids), _p(block_table),
                                         c_int(block_table.shape[1]), c_int(nb), c_int(B), c_int(Hq), c_int(Hk),
                                         c_float(scale), c_int(splits), _p(part_o), _p(part_ml), _p(out),
                                         _p(status_buffer(q.device)), _s()), "paged_decode_attn_tc")
    return out


_SAMPLE_SCRATCH: dict = {}


def _sample_scratch(device, B):
    """Row counters + per-slice partials of the split sampler; zeroed once, the kernel leaves the counters at zero.
    One buffer per device: sampler calls of one process are expected on one stream."""
    need = 4096 * (4 + 8 * 16 + 8 * 4)  # fixed layout for up to 4096 rows (see trlb_sample)
    buf = _SAMPLE_SCRATCH.get(device)
    if buf is None:
        if torch.cuda.is_current_stream_capturing():
            return None  # no allocation during capture: the one-CTA-per-row kernel is used instead
        buf = torch.zeros(need, dtype=torch.uint8, device=device)
        _SAMPLE_SCRATCH[device] = buf
    return buf


def sample_tokens(logits, inv_temp, min_p, eos_id, eos_floor, seed, step_ptr, greedy, out_tok, out_logp):
    B, V = logits.shape
    scratch = _sample_scratch(logits.device, B)
    _chk(lib().trlb_sample(_p(logits), c_int(int(logits.dtype == torch.bfloat16)), c_longlong(logits.stride(0)), c_int(B),
                           c_int(V), c_float(inv_temp), c_float(min_p or 0.0), c_int(-1 if eos_id is None else eos_id),
                           c_float(eos_floor or 0.0), ctypes.c_uint(seed & 0xFFFFFFFF), _p(step_ptr), c_int(int(greedy)),
                           _p(out_tok), _p(out_logp), _p(scratch), c_longlong(0 if scratch is None else scratch.numel()),
                           _s()), "sample")


def advance(tok, logp, slot_ids, seq_lens, n_gen, finished, out_tokens, out_logps, eos_id, max_total_len, next_input,
            step_counter, bump_len=1):
    B = tok.shape[0]
    _chk(lib().trlb_advance(_p(tok), _p(logp), _p(slot_ids), c_int(B), _p(seq_lens), _p(n_gen), _p(finished),
                            _p(out_tokens), _p(out_logps), c_int(out_tokens.shape[1]),
                            c_int(-1 if eos_id is None else eos_id), c_int(max_total_len), _p(next_input),
                            _p(step_counter), c_int(bump_len), _s()), "advance")


# -------------------------------------------------------------------------------------------
# collectives fused with compute (csrc/comm.cu); `arena` is a parallel.symm.SymmArena
# -------------------------------------------------------------------------------------------
def rs_reduce(arena, byte_offset, grad_is_bf16, lo, n, out, sumsq, sync, use_multimem=False):
    """out[n] (fp32) = mean over ranks of grad[lo:lo+n]; sumsq += |out|^2.  Reads peers' buffers in place."""
    mc = arena.mc(byte_offset) if (use_multimem and not grad_is_bf16) else None
    _chk(lib().trlb_rs_reduce(arena.peers(byte_offset), arena.pads(), c_int(arena.rank), c_int(arena.world), mc,
                              c_int(int(grad_is_bf16)), c_longlong(lo), c_longlong(n), _p(out), _p(sumsq),
                              sync.epoch_ptr, sync.gate_ptr, c_int(sync.channel), _p(status_buffer(out.device)), _s()),
         "rs_reduce")


def rs_reduce_accum(arena, byte_offset, grad_is_bf16, lo, n, out, sumsq, sync, max_ctas: int = 0):
    """out[n] (fp32) += mean over ranks of grad[lo:lo+n], read in place from every rank's buffer at ``byte_offset`` of
    the arena; ``max_ctas`` bounds the grid so that the kernel can run beside other work."""
    _chk(lib().trlb_rs_reduce_accum(arena.peers(byte_offset), arena.pads(), c_int(arena.rank), c_int(arena.world),
                                    c_int(int(grad_is_bf16)), c_longlong(lo), c_longlong(n), _p(out), _p(sumsq),
                                    sync.epoch_ptr, sync.gate_ptr, c_int(sync.channel), c_int(max_ctas),
                                    _p(status_buffer(out.device)), _s()), "rs_reduce_accum")


def shard_pull(arena, byte_offset, per, dst, ctas: int = 32):
    """``dst[p * per:(p + 1) * per] = `` rank p's ``per`` bf16 elements at ``byte_offset`` of the arena, for every p
    (peer loads; no barrier: the caller orders the launch after the slices became final)."""
    assert dst.dtype == torch.bfloat16 and dst.numel() >= per * arena.world
    _chk(lib().trlb_shard_pull(arena.peers(byte_offset), c_int(arena.rank), c_int(arena.world), _p(dst), c_longlong(per),
                               c_int(ctas), _s()), "shard_pull")


def norm_allreduce(arena, byte_offset, my_sumsq, max_norm, norm_out, clip_out, sync):
    _chk(lib().trlb_norm_allreduce(arena.peers(byte_offset), arena.pads(), c_int(arena.rank), c_int(arena.world),
                                   _p(my_sumsq), c_float(max_norm or 0.0), _p(norm_out), _p(clip_out), sync.epoch_ptr,
                                   sync.gate_ptr, c_int(sync.channel), _p(status_buffer(norm_out.device)), _s()),
         "norm_allreduce")


def adamw_bcast(arena, byte_offset, lo, n, master, grad, m, v, step, lr, b1, b2, eps, wd, clip, sync, use_multimem=False,
                no_decay_ranges=()):
    """AdamW on the shard; refreshed bf16 parameters are stored into every rank's replica at [lo, lo+n).
    ``no_decay_ranges``: up to 16 ``(lo, hi)`` element ranges of the bucket (biases, norm weights) exempt from decay."""
    mc = arena.mc(byte_offset) if use_multimem else None
    flat = [int(x) for r in no_decay_ranges for x in r]
    nd = (c_longlong * max(1, len(flat)))(*flat) if flat else None
    _chk(lib().trlb_adamw_bcast(arena.peers(byte_offset), arena.pads(), c_int(arena.rank), c_int(arena.world), mc,
                                c_longlong(lo), c_longlong(n), _p(master), _p(grad), _p(m), _p(v), c_int(step), c_float(lr),
                                c_float(b1), c_float(b2), c_float(eps), c_float(wd), _p(clip), sync.epoch_ptr, sync.gate_ptr,
                                c_int(sync.channel), _p(status_buffer(master.device)), nd, c_int(len(flat) // 2), _s()),
         "adamw_bcast")


def shard_allgather(arena, byte_offset, per, sync, use_multimem=False):
    mc = arena.mc(byte_offset) if use_multimem else None
    _chk(lib().trlb_shard_allgather(arena.peers(byte_offset), arena.pads(), c_int(arena.rank), c_int(arena.world), mc,
                                    c_longlong(per), sync.epoch_ptr, sync.gate_ptr, c_int(sync.channel),
                                    _p(status_buffer(arena.buf.device)), _s()), "shard_allgather")


def allreduce_add_rmsnorm(arena, byte_offset, buf_elems, res, w, eps, sync, out=None):
    """res += sum over ranks of their partial [T,H] (in the arena, double-buffered); returns rmsnorm(res) * w."""
    T, H = res.shape
    out = torch.empty_like(res) if out is None else out
    _chk(lib().trlb_allreduce_add_rmsnorm(arena.peers(byte_offset), arena.pads(), c_int(arena.rank), c_int(arena.world),
                                          c_longlong(buf_elems), _p(res), _p(w), _p(out), c_int(T), c_int(H), c_float(eps),
                                          sync.epoch_ptr, sync.gate_ptr, c_int(sync.channel),
                                          _p(status_buffer(res.device)), _s()), "allreduce_add_rmsnorm")
    return out
