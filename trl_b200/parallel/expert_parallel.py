"""Expert-parallel MoE block: experts are split over the ranks of a group, tokens stay where they are.

Forward on every rank, for its local experts and every source rank s (a *segment*):

    x_perm  this rank's tokens, sorted by global expert, in a symmetric buffer
    pull    x_in[segment rows] = x_perm_of_rank_s[rows of expert e]                           peer loads, each row once
    GEMM 1  act = swiglu(x_in . W_gate_up[e]^T)                                               local grouped GEMM
    GEMM 2  y_perm_of_rank_s[rows of expert e] = act[segment rows] . W_down[e]^T              C rows: stored to rank s
    combine out[t] = sum_j w[t, j] * y_perm[position of (t, j)]                               local

The combine all-to-all is the stores of the second grouped GEMM (``trlb_grouped_gemm_seg_bf16``).  The dispatch can
ride on the loads of the first one too (``fused_dispatch=True``: A tiles by TMA from rank s), but every N tile of the
gate/up projection then re-reads its rows over NVLink (6x for I = 768), so the default pulls the rows once with a copy
kernel and runs the first GEMM on the local copy.  Only the per-expert row offsets travel through NCCL.
The reference reaches expert parallelism through DeepSpeed / accelerate sharding of transformers MoE blocks
(trl/accelerate_configs/*.yaml); it has no fused path.

Backward (training) moves rows the same way: x and d_y rows are pulled from the source ranks, the local experts'
input and weight gradients run on the grouped kernels (forward weights read transposed; ``grouped_wgrad``), and the
stores of the last grouped GEMM return the d_x rows to their source ranks.  The gate/up pre-activations are
recomputed.

``shard_experts(model, group)`` wires the block into a model (expert slices as parameters flagged ``_ep_local``,
``layer.ep`` called by ``DecoderLayer.mlp_block``); ``HostExpertParallelMoE`` is the same block over the backend's
all-to-all for CPU / gloo runs and shapes outside the kernels; ``ep_hf_state_dict`` gathers the experts for saving."""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong

import torch
import torch.distributed as td

from .symm import SymmArena


class ExpertParallelMoE:
    def __init__(self, group, num_experts: int, hidden: int, intermediate: int, top_k: int, max_tokens: int, device,
                 fused_dispatch: bool = False):
        self.fused_dispatch = fused_dispatch
        self.group = group if group is not None else td.group.WORLD
        self.world, self.rank = td.get_world_size(self.group), td.get_rank(self.group)
        if num_experts % self.world:
            raise ValueError("the number of experts must be divisible by the expert-parallel size")
        self.E, self.E_loc, self.H, self.I, self.k = num_experts, num_experts // self.world, hidden, intermediate, top_k
        self.max_rows = max_tokens * top_k
        self.dev = device
        row_bytes = hidden * 2
        self.arena = SymmArena(2 * (self.max_rows * row_bytes + 256) + 4096, device, self.group)
        self.x_buf, self.x_off = self.arena.carve(self.max_rows * hidden, torch.bfloat16)
        self.y_buf, self.y_off = self.arena.carve(self.max_rows * hidden, torch.bfloat16)
        self.x_buf, self.y_buf = self.x_buf.view(self.max_rows, hidden), self.y_buf.view(self.max_rows, hidden)
        self.act = torch.empty(self.world * self.max_rows, intermediate, dtype=torch.bfloat16, device=device)
        self.x_in = None if fused_dispatch else torch.empty(self.world * self.max_rows, hidden, dtype=torch.bfloat16,
                                                            device=device)
        self._sync = torch.zeros(1, dtype=torch.float32, device=device)
        self._a_x = (ctypes.c_ulonglong * self.world)(*[p + self.x_off for p in self.arena.peer_ptrs])
        self._c_y = (ctypes.c_ulonglong * self.world)(*[p + self.y_off for p in self.arena.peer_ptrs])
        # indexed with up to `world` buffer ids by the segment GEMM's host code: one entry per rank, all the local buffer
        self._self_act = (ctypes.c_ulonglong * self.world)(*([self.act.data_ptr()] * self.world))

    # ---- routing tables ---------------------------------------------------------------------------------------------
    def _route(self, topk_idx):
        T, k = topk_idx.shape
        flat = topk_idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        counts = torch.zeros(self.E, dtype=torch.int32, device=self.dev)
        counts.scatter_add_(0, flat, torch.ones_like(flat, dtype=torch.int32))
        offsets = torch.zeros(self.E + 1, dtype=torch.int32, device=self.dev)
        offsets[1:] = counts.cumsum(0)
        all_off = torch.empty(self.world, self.E + 1, dtype=torch.int32, device=self.dev)
        td.all_gather_into_tensor(all_off, offsets, group=self.group)
        e0 = self.rank * self.E_loc
        loc = all_off[:, e0:e0 + self.E_loc + 1]                         # [W, E_loc + 1]
        cnt = (loc[:, 1:] - loc[:, :-1]).t().contiguous()                # [E_loc, W] segment order: expert-major
        seg_rows = cnt.reshape(-1)
        seg_act_row = (seg_rows.cumsum(0) - seg_rows).to(torch.int32)    # compact local layout of act
        seg_src = torch.arange(self.world, dtype=torch.int32, device=self.dev).repeat(self.E_loc)
        seg_src_row = loc[:, :-1].t().contiguous().reshape(-1)           # first row of the segment in the source's buffers
        seg_w = torch.arange(self.E_loc, dtype=torch.int32, device=self.dev).repeat_interleave(self.world)
        zeros = torch.zeros_like(seg_src)
        loc_off = torch.zeros(self.E_loc + 1, dtype=torch.int32, device=self.dev)  # rows per local expert, all sources
        loc_off[1:] = cnt.sum(1).cumsum(0)
        return order, offsets, all_off, dict(rows=seg_rows.contiguous(), act_row=seg_act_row, src=seg_src,
                                             src_row=seg_src_row, w=seg_w, zeros=zeros, loc_off=loc_off)

    def _seg_gemm(self, a_bases, c_bases, n_bufs, a_rows, w, seg, a_src, a_row, c_dst, c_row, n_out, k_dim, lda, ldc, swiglu,
                  w_transposed=False):
        from ..ops.cuda import _chk, _p, _s, lib, status_buffer

        _chk(lib().trlb_grouped_gemm_seg_bf16(a_bases, c_bases, c_int(n_bufs), c_longlong(a_rows), _p(w), c_int(w.shape[0]),
                                              c_int(seg["rows"].numel()), _p(seg["rows"]), _p(a_src), _p(a_row), _p(c_dst),
                                              _p(c_row), _p(seg["w"]), c_longlong(self.world * self.max_rows), c_int(n_out),
                                              c_int(k_dim), c_longlong(lda), c_longlong(ldc), c_int(int(swiglu)),
                                              c_int(int(w_transposed)), _p(status_buffer(self.dev)), _s()),
             "grouped_gemm_seg")

    def _pull_rows(self, bases, seg, dst):
        """dst[segment rows] = rows of the source ranks' symmetric buffer (each row crosses NVLink once)."""
        from ..ops.cuda import _chk, _p, _s, lib

        _chk(lib().trlb_moe_pull_rows(bases, c_int(self.world), _p(seg["rows"]), _p(seg["src"]), _p(seg["src_row"]),
                                      _p(seg["act_row"]), c_int(seg["rows"].numel()), _p(dst), c_int(self.H), _s()),
             "moe_pull_rows")

    def _bwd_buffer(self, name):
        buf = getattr(self, name, None)
        if buf is None:
            buf = torch.empty(self.world * self.max_rows, self.H, dtype=torch.bfloat16, device=self.dev)
            setattr(self, name, buf)
        return buf

    def _device_barrier(self):
        td.all_reduce(self._sync, group=self.group)  # stream-ordered: completes when every rank has reached it

    # ---- forward ----------------------------------------------------------------------------------------------------------
    def forward_nograd(self, hidden, gate_up_local, down_local, topk_w, topk_idx, keep=None):
        from ..ops.cuda import _chk, _p, _s, lib

        T, H = hidden.shape
        k = topk_idx.shape[1]
        if T * k > self.max_rows:
            raise ValueError(f"{T} tokens x top-{k} exceeds the expert-parallel buffers ({self.max_rows} rows)")
        order, offsets, all_off, seg = self._route(topk_idx)
        tok = order // k
        torch.index_select(hidden, 0, tok, out=self.x_buf[:T * k])
        self._device_barrier()  # every rank's x rows are in place (and nobody still reads the previous layer's)
        if self.fused_dispatch:
            self._seg_gemm(self._a_x, self._self_act, self.world, self.max_rows, gate_up_local, seg, seg["src"],
                           seg["src_row"], seg["zeros"], seg["act_row"], self.I, H, H, self.I, True)
        else:
            from ..ops.cuda import grouped_gemm

            self._pull_rows(self._a_x, seg, self.x_in)
            grouped_gemm(self.x_in, gate_up_local, seg["loc_off"], self.I, swiglu=True, out=self.act)
        self._seg_gemm(self._self_act, self._c_y, self.world, self.world * self.max_rows, down_local, seg, seg["zeros"],
                       seg["act_row"], seg["src"], seg["src_row"], H, self.I, self.I, H, False)
        self._device_barrier()  # all peers have stored my y rows
        inv = torch.empty(T * k, dtype=torch.int32, device=self.dev)
        inv[order] = torch.arange(T * k, dtype=torch.int32, device=self.dev)
        out = torch.empty(T, H, dtype=torch.bfloat16, device=self.dev)
        _chk(lib().trlb_moe_combine(_p(self.y_buf), _p(inv), _p(topk_w.float().contiguous()), _p(out), c_int(T), c_int(k),
                                    c_int(H), _s()), "moe_combine")
        if keep is not None:
            keep.update(order=order, offsets=offsets, all_off=all_off, seg=seg, y_perm=self.y_buf[:T * k].clone())
        return out

    def __call__(self, hidden, gate_up_local, down_local, topk_w, topk_idx):
        if not torch.is_grad_enabled() or not (hidden.requires_grad or gate_up_local.requires_grad):
            return self.forward_nograd(hidden, gate_up_local, down_local, topk_w, topk_idx)
        return _EpMoeFn.apply(hidden, gate_up_local, down_local, topk_w, topk_idx, self)


class _EpMoeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, gate_up_local, down_local, topk_w, topk_idx, ep: ExpertParallelMoE):
        keep: dict = {}
        out = ep.forward_nograd(hidden, gate_up_local, down_local, topk_w, topk_idx, keep)
        ctx.ep, ctx.keep, ctx.k = ep, keep, topk_idx.shape[1]
        ctx.save_for_backward(hidden, gate_up_local, down_local, topk_w)
        return out

    @staticmethod
    def backward(ctx, d_out):
        """Rows travel as in the forward pass: x and d_y rows are pulled from the source ranks' symmetric buffers into
        the expert-sorted local layout, the local experts' gradients run on the grouped kernels, and the stores of the
        last grouped GEMM put every d_x row back into its source rank's buffer.  One scalar (the number of rows this
        rank's experts received) is read back to size the element-wise work."""
        from ..ops.cuda import _chk, _p, _s, grouped_gemm, grouped_wgrad, lib, moe_combine_bwd, moe_gather_sum

        ep, keep, k = ctx.ep, ctx.keep, ctx.k
        hidden, gu_w, dn_w, topk_w = ctx.saved_tensors
        W, E_loc, I, H = ep.world, ep.E_loc, ep.I, ep.H
        order, seg = keep["order"], keep["seg"]
        tok = order // k
        Tk = order.numel()
        torch.index_select(hidden, 0, tok, out=ep.x_buf[:Tk])
        _, d_topk = moe_combine_bwd(d_out, keep["y_perm"], order, topk_w, d_y=ep.y_buf[:Tk])
        ep._device_barrier()  # every rank's x and d_y rows are in place
        x_full = ep.x_in if ep.x_in is not None else ep._bwd_buffer("_x_in_bwd")
        dy_full = ep._bwd_buffer("_dy_in_bwd")
        ep._pull_rows(ep._a_x, seg, x_full)
        ep._pull_rows(ep._c_y, seg, dy_full)
        ep._device_barrier()  # every rank has pulled: x_buf is free to receive the d_x rows
        off = seg["loc_off"]
        n = int(off[-1])
        if n > 0:
            x_in, dy_in = x_full[:n], dy_full[:n]
            gu = grouped_gemm(x_in, gu_w, off, 2 * I)  # recompute the pre-activations
            act = torch.empty(n, I, dtype=gu.dtype, device=gu.device)
            _chk(lib().trlb_swiglu_fwd(_p(gu), _p(act), c_longlong(n), c_int(I), _s()), "swiglu_fwd")
            d_dn_w = grouped_wgrad(dy_in, act, off, E_loc)
            d_act = grouped_gemm(dy_in, dn_w, off, I, w_transposed=True)
            d_gu = torch.empty_like(gu)
            _chk(lib().trlb_swiglu_bwd(_p(d_act), _p(gu), _p(d_gu), c_longlong(n), c_int(I), _s()), "swiglu_bwd")
            d_gu_w = grouped_wgrad(d_gu, x_in, off, E_loc)
            bases = (ctypes.c_ulonglong * W)(*([d_gu.data_ptr()] * W))
            ep._seg_gemm(bases, ep._a_x, W, n, gu_w, seg, seg["zeros"], seg["act_row"], seg["src"], seg["src_row"], H,
                         2 * I, 2 * I, H, False, w_transposed=True)
        else:
            d_gu_w, d_dn_w = torch.zeros_like(gu_w), torch.zeros_like(dn_w)
        ep._device_barrier()  # all peers have stored my d_x rows
        inv = torch.empty(Tk, dtype=torch.int32, device=d_out.device)
        inv[order] = torch.arange(Tk, dtype=torch.int32, device=d_out.device)
        d_hidden = moe_gather_sum(ep.x_buf, inv, hidden.shape[0], k)
        return d_hidden, d_gu_w, d_dn_w, d_topk.to(topk_w.dtype), None, None


# ---------------------------------------------------------------------------------------------------------------------
# Host path: the same block through the backend's all-to-all (gloo on CPU, NCCL where the symmetric kernels do not
# apply: fp32, tiny hidden sizes).  Everything is ordinary autograd, so it is also the oracle of the fused path.
# ---------------------------------------------------------------------------------------------------------------------
class _AllToAllRows(torch.autograd.Function):
    """Rows exchanged with per-rank counts; the backward pass sends the gradients the other way."""

    @staticmethod
    def forward(ctx, x, send, recv, group):
        ctx.send, ctx.recv, ctx.group = send, recv, group
        out = torch.empty((sum(recv),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        td.all_to_all_single(out, x.contiguous(), list(recv), list(send), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        d = torch.empty((sum(ctx.send),) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        td.all_to_all_single(d, g.contiguous(), list(ctx.send), list(ctx.recv), group=ctx.group)
        return d, None, None, None


class HostExpertParallelMoE:
    """Expert parallelism over ``all_to_all_single``: tokens sorted by expert, sent to the expert's owner, run through
    the local experts, sent back and combined with the routing weights."""

    def __init__(self, group, num_experts: int, top_k: int):
        self.group = group if group is not None else td.group.WORLD
        self.world, self.rank = td.get_world_size(self.group), td.get_rank(self.group)
        if num_experts % self.world:
            raise ValueError("the number of experts must be divisible by the expert-parallel size")
        self.E, self.E_loc, self.k = num_experts, num_experts // self.world, top_k

    def __call__(self, hidden, gate_up_local, down_local, topk_w, topk_idx):
        W, E_loc = self.world, self.E_loc
        T, k = topk_idx.shape
        flat = topk_idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        tok = order // k
        counts = torch.bincount(flat, minlength=self.E)
        all_cnt = torch.empty(W * self.E, dtype=counts.dtype, device=counts.device)
        td.all_gather_into_tensor(all_cnt, counts, group=self.group)
        all_cnt = all_cnt.view(W, self.E).cpu()
        e0 = self.rank * E_loc
        send = [int(all_cnt[self.rank, r * E_loc:(r + 1) * E_loc].sum()) for r in range(W)]
        recv = [int(all_cnt[s, e0:e0 + E_loc].sum()) for s in range(W)]
        x_in = _AllToAllRows.apply(hidden.index_select(0, tok), send, recv, self.group)  # source-major, expert-minor
        # rows of local expert e: one run per source
        base = [sum(recv[:s]) for s in range(W)]
        within = all_cnt[:, e0:e0 + E_loc].cumsum(1) - all_cnt[:, e0:e0 + E_loc]
        y_in = torch.zeros_like(x_in)
        I = gate_up_local.shape[1] // 2
        for e in range(E_loc):
            idx = torch.cat([torch.arange(base[s] + int(within[s, e]), base[s] + int(within[s, e]) + int(all_cnt[s, e0 + e]),
                                          device=hidden.device) for s in range(W)])
            if idx.numel() == 0:
                continue
            xe = x_in.index_select(0, idx)
            gu = xe @ gate_up_local[e].t()
            act = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
            y_in = y_in.index_copy(0, idx, (act @ down_local[e].t()).to(y_in.dtype))
        y_perm = _AllToAllRows.apply(y_in, recv, send, self.group)
        w_perm = topk_w.reshape(-1).index_select(0, order)
        out = torch.zeros(T, hidden.shape[1], dtype=torch.float32, device=hidden.device)
        out = out.index_add(0, tok, y_perm.float() * w_perm.float()[:, None])
        return out.to(hidden.dtype)


def shard_experts(model, group=None, max_tokens: int = 16384, fused: bool | None = None):
    """Turns a replicated MoE model into an expert-parallel one, in place (collective over ``group``).

    Every MoE layer keeps experts ``[rank * E / world, (rank + 1) * E / world)`` of ``experts_gate_up`` /
    ``experts_down``; the new parameters carry ``_ep_local = True`` so that the training engines leave their gradients
    unreduced (each expert receives the tokens of every rank through the dispatch; the gradients are scaled by 1 / world
    like an averaged data-parallel gradient) and keep their optimizer state whole on the owner.  ``layer.ep`` runs
    the block: the fused kernels over symmetric memory on bf16 CUDA models (pull dispatch, grouped tcgen05 GEMMs,
    peer-store combine), the backend's all-to-all elsewhere.  ``max_tokens``: most tokens of one forward call on a
    rank (sizes the symmetric buffers of the fused path)."""
    import torch.nn as nn

    lm = getattr(model, "language_model", model)
    cfg = lm.config
    if not cfg.is_moe:
        raise ValueError("shard_experts needs a mixture-of-experts model")
    group = group if group is not None else td.group.WORLD
    world, rank = td.get_world_size(group), td.get_rank(group)
    if cfg.num_experts % world:
        raise ValueError(f"{cfg.num_experts} experts cannot be split over {world} ranks")
    e_loc = cfg.num_experts // world
    first = lm.layers[0].experts_gate_up
    if fused is None:
        from .symm import symmetric_available

        fused = (first.is_cuda and first.dtype == torch.bfloat16 and world > 1 and symmetric_available()
                 and cfg.hidden_size % 64 == 0 and cfg.moe_intermediate_size % 64 == 0)
    ep = (ExpertParallelMoE(group, cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts_per_tok,
                            max_tokens, first.device) if fused
          else HostExpertParallelMoE(group, cfg.num_experts, cfg.num_experts_per_tok))
    for l in lm.layers:
        for name in ("experts_gate_up", "experts_down"):
            full = getattr(l, name)
            p = nn.Parameter(full.detach()[rank * e_loc:(rank + 1) * e_loc].clone(), requires_grad=full.requires_grad)
            p._ep_local = True
            setattr(l, name, p)
        l.ep, l.ep_first_expert = ep, rank * e_loc
    lm.ep_group, lm.ep_world, lm.ep_rank = group, world, rank
    return model


@torch.no_grad()
def ep_hf_state_dict(model, to_cpu: bool = True) -> dict:
    """Complete checkpoint tensors of an expert-parallel model (collective): the experts of one layer at a time are
    all-gathered, exported and (with ``to_cpu``) copied to host memory before the next layer's are gathered; ranks
    that do not save pass False and get an empty dict."""
    from ..models.hf_io import to_hf_state_dict

    lm = getattr(model, "language_model", model)
    group, world = lm.ep_group, lm.ep_world
    state = {"prev": None}

    def gather(i):
        if state["prev"] is not None:
            state["prev"]._ep_full = None
        l = lm.layers[i]
        full = []
        for t in (l.experts_gate_up.detach(), l.experts_down.detach()):
            out = torch.empty(world * t.numel(), dtype=t.dtype, device=t.device)
            td.all_gather_into_tensor(out, t.contiguous().view(-1), group=group)
            full.append(out.view((world * t.shape[0],) + tuple(t.shape[1:])))
        l._ep_full, state["prev"] = tuple(full), l

    sd = to_hf_state_dict(lm, before_layer=gather, copy_to="cpu" if to_cpu else None)
    if state["prev"] is not None:
        state["prev"]._ep_full = None
    return sd
