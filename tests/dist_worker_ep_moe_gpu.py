"""2-GPU worker: expert-parallel MoE block (dispatch / combine fused into the grouped GEMMs) vs the local expert loop."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as td

from trl_b200.ops import cuda as K
from trl_b200.oracle import ops as ref
from trl_b200.parallel import dist as D
from trl_b200.parallel.expert_parallel import ExpertParallelMoE


sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _dist_util import Deadline  # noqa: E402


def main():
    D.init_process_group()
    DL = Deadline()  # the ranks leave on their own, between steps, before the parent's limit
    rank, world = D.rank(), D.world_size()
    dev = torch.device("cuda", D.local_rank())
    E, I, H, k = 8, 256, 512, 2
    g = torch.Generator().manual_seed(0)  # same weights everywhere
    gu = (torch.randn(E, 2 * I, H, generator=g) / H ** 0.5).to(torch.bfloat16).to(dev)
    dw = (torch.randn(E, H, I, generator=g) / I ** 0.5).to(torch.bfloat16).to(dev)
    e_loc = E // world
    gu_loc = gu[rank * e_loc:(rank + 1) * e_loc].clone().requires_grad_(True)
    dw_loc = dw[rank * e_loc:(rank + 1) * e_loc].clone().requires_grad_(True)
    ep = ExpertParallelMoE(None, E, H, I, k, max_tokens=1024, device=dev)
    for step, T in enumerate((700, 333)):  # different token counts per call and per rank
        gl = torch.Generator().manual_seed(100 + 10 * step + rank)
        T = T + 17 * rank
        hidden = (torch.randn(T, H, generator=gl) * 0.5).to(torch.bfloat16).to(dev).requires_grad_(True)
        logits = torch.randn(T, E, generator=gl).to(dev)
        logits[:, 3] = -1e9
        tw, ti = torch.softmax(logits, -1).topk(k, -1)
        tw = (tw / tw.sum(-1, keepdim=True)).requires_grad_(True)
        out = ep(hidden, gu_loc, dw_loc, tw, ti)
        out.float().square().sum().backward()
        torch.cuda.synchronize()
        K.check_status(dev)
        h32 = hidden.detach().float().requires_grad_(True)
        g32, d32 = gu.float().requires_grad_(True), dw.float().requires_grad_(True)
        w32 = tw.detach().clone().requires_grad_(True)
        want = ref.moe_experts(h32, g32, d32, w32, ti).float()
        want.square().sum().backward()
        scale = max(1.0, want.abs().max().item())
        assert (out.float() - want).abs().max().item() < 0.05 * scale, (step, rank)
        assert (hidden.grad.float() - h32.grad).abs().max().item() < 0.08 * (h32.grad.abs().max().item() + 1e-6)
        assert (tw.grad - w32.grad).abs().max().item() < 0.08 * (w32.grad.abs().max().item() + 1e-6)
        # expert weight gradients: the local slice holds the contributions of every rank's tokens
        full = g32.grad.clone()
        td.all_reduce(full)
        got = gu_loc.grad.float()
        assert (got - full[rank * e_loc:(rank + 1) * e_loc]).abs().max().item() < 0.08 * (full.abs().max().item() + 1e-6)
        hidden.grad = None
        gu_loc.grad = None
        dw_loc.grad = None
        with torch.no_grad():  # inference path
            out2 = ep(hidden.detach(), gu_loc, dw_loc, tw.detach(), ti)
        assert (out2.float() - want).abs().max().item() < 0.05 * scale
    torch.cuda.synchronize()
    K.check_status(dev)
    td.barrier()
    if rank == 0:
        print("EP_MOE_OK")
    DL.check()
    td.destroy_process_group()


if __name__ == "__main__":
    main()
