"""ctypes bindings + autograd wrappers for the sm_100a kernel library.

Kernels are launched on the caller's current CUDA stream, so they compose with torch ops,
side streams and CUDA-graph capture.  Every kernel that can wait takes a per-device status
buffer; :func:`check_status` reads it (one host sync) and raises if a bounded wait ran out.
"""
from __future__ import annotations

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


def _chk(rc: int, what: str):
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


def lmhead_dz(hidden, weight, labels, lse, grow, inv_temp: float, out=None):
    """dZ[M,V] = grow * (1[label] - softmax(z/T)) / T as bf16 (stage 1 of the lm_head backward)."""
    M, K = hidden.shape
    V = weight.shape[0]
    if out is None:
        out = torch.empty(M, V, dtype=torch.bfloat16, device=hidden.device)
    rc = lib().trlb_lmhead_dz(_p(hidden), _p(weight), _p(labels), _p(lse), _p(grow), _p(out), c_int(M), c_int(V),
                              c_int(K), c_longlong(hidden.stride(0)), c_longlong(weight.stride(0)),
                              c_longlong(out.stride(0)), c_float(inv_temp), _p(status_buffer(hidden.device)), _s())
    _chk(rc, "trlb_lmhead_dz")
    return out


class _LmHeadLogprobFn(torch.autograd.Function):
    """log p(label) (+ entropy, no grad) from hidden @ W^T without materialising fp32 logits.

    Backward recomputes the logits tile by tile inside the dZ kernel (bf16 dZ in token chunks),
    then dH = dZ @ W and dW += dZ^T @ H are plain library GEMMs.
    """

    CHUNK = 8192

    @staticmethod
    def forward(ctx, hidden, weight, labels, inv_temp, want_entropy, want_argmax):
        hidden = hidden.contiguous()
        labels = labels.to(torch.int64).contiguous()
        logp, ent, lse, amax = lmhead_forward(hidden, weight, labels, inv_temp, want_entropy, want_argmax)
        ctx.save_for_backward(hidden, weight, labels, lse)
        ctx.inv_temp = inv_temp
        ctx.mark_non_differentiable(*[t for t in (ent, amax) if t is not None])
        return logp, ent, amax

    @staticmethod
    def backward(ctx, g_logp, _ge, _ga):
        hidden, weight, labels, lse = ctx.saved_tensors
        M, K = hidden.shape
        V = weight.shape[0]
        g = g_logp.float().contiguous()
        dH = torch.empty_like(hidden) if ctx.needs_input_grad[0] else None
        dW = torch.zeros(V, K, dtype=torch.float32, device=hidden.device) if ctx.needs_input_grad[1] else None
        ck = _LmHeadLogprobFn.CHUNK
        buf = _scratch_buf("lmh_dz", min(ck, M) * V * 2, hidden.device)
        for s in range(0, M, ck):
            e = min(M, s + ck)
            dz = buf[: (e - s) * V * 2].view(torch.bfloat16).view(e - s, V)
            lmhead_dz(hidden[s:e], weight, labels[s:e], lse[s:e], g[s:e], ctx.inv_temp, out=dz)
            if dH is not None:
                torch.matmul(dz, weight, out=dH[s:e])
            if dW is not None:
                dW += torch.matmul(dz.t(), hidden[s:e]).float()
        return dH, (dW.to(weight.dtype) if dW is not None else None), None, None, None, None


def lm_head_logprobs(hidden, weight, labels, temperature=1.0, compute_entropy=True):
    valid = labels >= 0
    logp, ent, _ = _LmHeadLogprobFn.apply(hidden, weight, labels.clamp_min(0), 1.0 / float(temperature),
                                          compute_entropy, False)
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
