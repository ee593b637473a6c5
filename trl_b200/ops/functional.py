"""Op entry points used by the models, the trainers and the rollout engine.

Every function has two implementations behind one signature:

* CUDA tensors run the hand-written sm_100a kernels from ``trl_b200/csrc``
  (``ops/cuda.py`` wraps them in ``torch.autograd.Function``).  If the native
  library is missing on a machine that has a GPU the call raises; there is no
  silent eager fallback for the kernels this module owns.
* CPU tensors run the fp32 PyTorch oracle (``trl_b200/oracle/ops.py``), which
  is also what the kernels are tested against.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..oracle import ops as _ref


def _cuda():
    from . import cuda as _c

    return _c


def _use_kernel(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.bfloat16,)


import os as _os

# which GEMM the decoder's plain linears run on: "own" = this library's tcgen05 kernel for the forward, the input
# gradient and the weight gradient (operands read transposed in place), "cublas" = the library GEMM through torch.
# The default follows the measurements in benchmarks/kernels.py gemm: the library where it is faster.
_LINEAR_IMPL = _os.environ.get("TRL_B200_LINEAR", "cublas")


def set_linear_impl(name: str) -> str:
    """Selects the GEMM of :func:`linear` ("own" or "cublas"); returns the previous choice."""
    global _LINEAR_IMPL
    if name not in ("own", "cublas"):
        raise ValueError(name)
    was, _LINEAR_IMPL = _LINEAR_IMPL, name
    return was


def linear(x, weight, bias=None):
    """``x @ weight^T (+ bias)``.  With ``TRL_B200_LINEAR=own`` (or :func:`set_linear_impl`) bf16 CUDA inputs run
    forward, dgrad and wgrad on the tcgen05 GEMM under autograd; otherwise the library GEMM."""
    if _LINEAR_IMPL == "own" and x.is_cuda:
        c = _cuda()
        if c.linear_own_ok(x, weight):
            return c.LinearFn.apply(x, weight, bias)
    return F.linear(x, weight, bias)


def rms_norm(x, weight, eps):
    if _use_kernel(x):
        return _cuda().RMSNormFn.apply(x, weight, eps)
    return _ref.rms_norm(x, weight, eps)


def apply_rope_qk(q, k, positions, theta):
    """RoPE on q [T,Hq,D] and k [T,Hkv,D]; returns new tensors."""
    if _use_kernel(q):
        return _cuda().RopeFn.apply(q, k, positions, theta)
    return _ref.apply_rope(q, positions, theta), _ref.apply_rope(k, positions, theta)


def swiglu(gate_up):
    if _use_kernel(gate_up):
        return _cuda().SwigluFn.apply(gate_up)
    return _ref.swiglu(gate_up)


def attention_varlen(q, k, v, cu_seqlens, max_seqlen, causal=True, window=None):
    """``window``: sliding-window size (a token sees itself and the window - 1 tokens before it); None = full."""
    if q.is_cuda:
        return _cuda().attention_varlen(q, k, v, cu_seqlens, max_seqlen, causal, window)
    return _ref.attention_varlen(q, k, v, cu_seqlens, max_seqlen, causal, window=window)


def attention_varlen_qk(q, k, v, cu_q, cu_k, max_q, max_k):
    """Causal varlen attention with separate query / key segmentation; the mask is aligned to the END of each key
    segment (a query segment is the tail of its key segment).  Used by context parallelism."""
    if q.is_cuda:
        return _cuda().attention_varlen_qk(q, k, v, cu_q, cu_k, max_q, max_k)
    return _ref.attention_varlen_qk(q, k, v, cu_q, cu_k)


def lm_head_logprobs(hidden, weight, labels, temperature=1.0, bias=None, softcap=None,
                     compute_entropy=True, chunk_tokens: int = 4096, entropy_grad: bool = False):
    """Fused lm_head GEMM + log-softmax gather (+entropy); logits never materialise.  ``entropy_grad``: the entropy
    is differentiable too (GRPO entropy bonus); by default it is a statistic without gradient."""
    from ..models.activation_offloading import no_offload

    with no_offload():  # the head's input is used again at once: it stays on the device
        return _lm_head_logprobs(hidden, weight, labels, temperature, bias, softcap, compute_entropy, chunk_tokens,
                                 entropy_grad)


def _lm_head_logprobs(hidden, weight, labels, temperature, bias, softcap, compute_entropy, chunk_tokens, entropy_grad):
    if _use_kernel(hidden) and bias is None and not softcap:
        return _cuda().lm_head_logprobs(hidden, weight, labels, temperature, compute_entropy, entropy_grad)
    if hidden.shape[0] <= chunk_tokens or not torch.is_grad_enabled():
        outs = [
            _ref.lm_head_logprobs(h, weight, y, temperature, bias, softcap, compute_entropy, entropy_grad)
            for h, y in zip(hidden.split(chunk_tokens), labels.split(chunk_tokens))
        ] or [(hidden.new_zeros(0, dtype=torch.float32), hidden.new_zeros(0, dtype=torch.float32))]
        lp = torch.cat([o[0] for o in outs])
        en = torch.cat([o[1] for o in outs]) if compute_entropy else None
        return lp, en
    # token-chunked with recompute so the [chunk, V] logits tile is the peak
    from torch.utils.checkpoint import checkpoint

    lps, ens = [], []
    for h, y in zip(hidden.split(chunk_tokens), labels.split(chunk_tokens)):
        lp, en = checkpoint(_ref.lm_head_logprobs, h, weight, y, temperature, bias, softcap,
                            compute_entropy, entropy_grad, use_reentrant=False)
        lps.append(lp)
        ens.append(en)
    return torch.cat(lps), (torch.cat(ens) if compute_entropy else None)


def lm_head_ce(hidden, weight, labels, ignore_index=-100, bias=None):
    """Sum NLL + (correct, entropy_sum, n_valid) without a full logits tensor."""
    from ..models.activation_offloading import no_offload

    with no_offload():
        if _use_kernel(hidden) and bias is None:
            return _cuda().lm_head_ce(hidden, weight, labels, ignore_index)
        return _ref.lm_head_ce(hidden, weight, labels, ignore_index, bias)


def moe_mlp(hidden, router_w, gate_up_w, down_w, top_k, norm_topk_prob):
    """Router + experts.  Returns (out, router_probs, topk_idx)."""
    w, idx, probs = _ref.moe_router(hidden, router_w, top_k, norm_topk_prob)
    if hidden.is_cuda:
        out = _cuda().moe_experts(hidden, gate_up_w, down_w, w, idx)
    else:
        out = _ref.moe_experts(hidden, gate_up_w, down_w, w, idx)
    return out, probs, idx


def apply_mrope_qk(q, k, positions3, theta, sections):
    """Multimodal rotary embedding of q and k: one kernel on bf16 CUDA tensors, the PyTorch oracle elsewhere."""
    if _use_kernel(q) and q.shape[-1] % 4 == 0:
        return _cuda().MRopeFn.apply(q, k, positions3, theta, tuple(sections))
    return _ref.apply_mrope(q, positions3, theta, sections), _ref.apply_mrope(k, positions3, theta, sections)


moe_router = _ref.moe_router
selective_log_softmax = _ref.selective_log_softmax
entropy_from_logits = _ref.entropy_from_logits


def load_balancing_loss(router_probs, topk_idx, num_experts, top_k, token_mask=None):
    """Router aux loss ``E * sum_e f_e P_e``: one reduction kernel on CUDA tensors, the dense oracle on CPU."""
    if router_probs.is_cuda and num_experts <= 1024:
        return _cuda().moe_aux_loss(router_probs, topk_idx, num_experts, token_mask)
    return _ref.load_balancing_loss(router_probs, topk_idx, num_experts, top_k, token_mask)
