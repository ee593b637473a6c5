"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at the moment they launch: a serving
loop whose memory was fully committed at start-up, a C program that links the library without PyTorch's
allocator.  ``trlb_paged_decode_attn_noalloc`` keeps its split-KV scratch in a fixed device array inside
the library.  This test checks it against the ordinary entry point (caller-provided scratch) on two
consecutive calls with different inputs, because the shared array keeps the previous call's contents.
The file is named so that pytest collects it last.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, B, Hq, Hk, bs, max_blocks):
    g = torch.Generator(device="cuda").manual_seed(seed)
    D = 128
    nblocks = B * max_blocks
    kc = torch.randn(nblocks, bs, Hk, D, device="cuda", dtype=torch.bfloat16, generator=g)
    vc = torch.randn(nblocks, bs, Hk, D, device="cuda", dtype=torch.bfloat16, generator=g)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16, generator=g)
    table = torch.randperm(nblocks, device="cuda", generator=g).reshape(B, max_blocks).to(torch.int32)
    lens = torch.randint(0, bs * max_blocks - 1, (B,), device="cuda", generator=g).to(torch.int32)
    return q, kc, vc, lens, table


def _compare(fn, seed, B, Hq, Hk, splits, bs=16, max_blocks=24, permute_slots=False):
    from trl_b200.ops import cuda as K

    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    q, kc, vc, lens, table = _inputs(seed, B, Hq, Hk, bs, max_blocks)
    slots = torch.randperm(B, device="cuda").to(torch.int32) if permute_slots else None
    D = 128
    scale = 1.0 / math.sqrt(D)
    ref = torch.empty(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    part_o = torch.empty(B * Hq * splits * D, device="cuda")
    part_ml = torch.empty(B * Hq * splits * 2, device="cuda")
    K.paged_decode_attn(q, kc, vc, lens, slots, table, bs, scale, splits, part_o, part_ml, ref)
    out = torch.full_like(ref, float("nan"))
    rc = fn(c_void_p(q.data_ptr()), c_void_p(kc.data_ptr()), c_void_p(vc.data_ptr()), c_void_p(lens.data_ptr()),
            None if slots is None else c_void_p(slots.data_ptr()), c_void_p(table.data_ptr()), c_int(max_blocks),
            c_int(bs), c_int(B), c_int(Hq), c_int(Hk), c_int(D), c_float(scale), c_int(splits), c_void_p(out.data_ptr()),
            stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert torch.allclose(out.float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_noalloc_entry_matches_regular_entry_twice():
    from trl_b200._native import kernels

    fn = kernels().trlb_paged_decode_attn_noalloc
    fn.restype = c_int
    for seed, (B, Hq, Hk, splits) in enumerate([(6, 8, 2, 3), (9, 28, 4, 2)]):
        _compare(fn, seed, B, Hq, Hk, splits)


def test_noalloc_entry_at_the_exact_limit_and_with_permuted_slots():
    from trl_b200._native import kernels

    fn = kernels().trlb_paged_decode_attn_noalloc
    fn.restype = c_int
    _compare(fn, 7, 64, 32, 8, 4, max_blocks=6)           # 64 * 32 * 4 = 8192 partial rows: the whole array
    _compare(fn, 8, 12, 16, 4, 2, permute_slots=True)     # rows read the cache slots a permutation names


def test_noalloc_entry_rejects_unsupported_shapes():
    from trl_b200._native import kernels

    fn = kernels().trlb_paged_decode_attn_noalloc
    fn.restype = c_int
    dummy = torch.zeros(8, device="cuda")
    p = c_void_p(dummy.data_ptr())
    st = c_void_p(torch.cuda.current_stream().cuda_stream)
    # head_dim 64, and query heads that the KV heads do not divide: refused before anything is launched
    assert fn(p, p, p, p, None, p, c_int(1), c_int(16), c_int(2), c_int(8), c_int(2), c_int(64), c_float(1.0), c_int(1), p,
              st) == -71
    assert fn(p, p, p, p, None, p, c_int(1), c_int(16), c_int(2), c_int(7), c_int(2), c_int(128), c_float(1.0), c_int(1), p,
              st) == -71
    torch.cuda.synchronize()


def test_noalloc_entry_rejects_oversized_request():
    from trl_b200._native import kernels

    lib = kernels()
    fn = lib.trlb_paged_decode_attn_noalloc
    fn.restype = c_int
    dummy = torch.zeros(8, device="cuda")
    p = c_void_p(dummy.data_ptr())
    # 64 * 64 * 4 = 16384 partials > 8192: must refuse without launching anything
    rc = fn(p, p, p, p, None, p, c_int(1), c_int(16), c_int(64), c_int(64), c_int(8), c_int(128), c_float(1.0), c_int(4),
            p, c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -70
    torch.cuda.synchronize()
