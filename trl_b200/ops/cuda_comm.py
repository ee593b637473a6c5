"""Bindings of the all-gather-fused GEMM (``trlb_ag_gemm_bf16_tn`` in csrc/gemm_tcgen05.cu)."""
from __future__ import annotations

from ctypes import c_int, c_longlong

import torch

from .cuda import _chk, _p, _s, lib, status_buffer


class AgGemmState:
    """Per-buffer bookkeeping: arrival counters per 256-row weight tile and the call number."""

    def __init__(self, device, max_tiles: int = 4096, copiers: int = 16):
        self.count = torch.zeros(max_tiles, dtype=torch.int32, device=device)
        self.calls = 0
        self.copiers = copiers


def ag_gemm(x: torch.Tensor, arena, byte_offset: int, per: int, total: int, w_off: int, N: int, state: AgGemmState,
            bias: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[M,N] = x[M,K] @ W[N,K]^T where W starts ``w_off`` elements into a symmetric bf16 buffer of ``total``
    elements (rank r holds [r*per, (r+1)*per)).  The copier CTAs of the same kernel pull the missing parts of the
    *whole* buffer over NVLink while the tensor-core CTAs start on the locally owned tiles; when the kernel has
    finished, the local buffer is complete for the layer's other GEMMs."""
    M, K = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    if (N + 255) // 256 > state.count.numel():
        raise ValueError("weight has more 256-row tiles than the counter array")
    state.calls += 1
    # every buffer/weight pair needs its own counters or a zeroed array: the target grows per call
    _chk(lib().trlb_ag_gemm_bf16_tn(_p(x), _p(out), _p(bias), c_int(M), c_int(N), c_int(K), c_longlong(x.stride(0)),
                                    c_longlong(out.stride(0)), arena.peers(byte_offset), c_int(arena.rank),
                                    c_int(arena.world), c_longlong(per), c_longlong(w_off), c_longlong(total),
                                    _p(state.count), c_int(state.calls), c_int(state.copiers),
                                    _p(status_buffer(x.device)), _s()), "ag_gemm")
    return out
