"""2-GPU worker: Ulysses sequence parallelism and context parallelism (gathered K/V) on GPUs, bf16, with the tcgen05
attention kernels: the two ranks split one packed stream; the summed loss and the summed gradients must equal those
of one rank that runs the whole stream."""
import copy
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as td

from trl_b200.models.decoder import SeqCtx
from trl_b200.ops import cuda as K
from trl_b200.ops import functional as ops
from trl_b200.parallel import dist as D
from trl_b200.parallel.ulysses import SpInfo, shard_sequence
from trl_b200.testing import make_tiny_model

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _dist_util import Deadline  # noqa: E402


def loss_and_grads(model, ids, tgt, ctx):
    for p in model.parameters():
        p.grad = None
    h = model.forward_hidden(ids, ctx)
    loss_sum, _, _, n = ops.lm_head_ce(h, model.lm_head_weight, tgt)
    loss_sum.backward()
    return loss_sum.detach().float(), n, {k: p.grad.detach().float().clone() for k, p in model.named_parameters()}


def main():
    D.init_process_group()
    DL = Deadline()
    rank = D.rank()
    dev = torch.device("cuda", D.local_rank())
    base = make_tiny_model("tiny-qwen2", dtype=torch.bfloat16, device=dev, hidden_size=512, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=128, intermediate_size=1024, num_hidden_layers=2, seed=0)
    g = torch.Generator().manual_seed(11)  # the same stream on both ranks
    lens = [301, 77, 190, 1, 64]           # 633 tokens: odd total, so the stream is padded to a multiple of 2
    ids = torch.randint(0, 1024, (sum(lens),), generator=g).to(dev)
    tgt = torch.roll(ids, -1)
    ends = torch.tensor(lens).cumsum(0) - 1
    tgt[ends.to(dev)] = -100
    ctx = SeqCtx.from_lengths(lens, dev)
    ref_loss, ref_n, ref_g = loss_and_grads(copy.deepcopy(base), ids, tgt, ctx)
    group = td.new_group([0, 1])
    for mode in ("ulysses", "allgather_kv"):
        DL.check()
        model = copy.deepcopy(base)
        sp = SpInfo(group, 2, rank, mode)
        l_ids, l_tgt, l_ctx = shard_sequence(ids, tgt, SeqCtx.from_lengths(lens, dev), sp, 0)
        loss, n, grads = loss_and_grads(model, l_ids, l_tgt, l_ctx)
        tot = torch.stack([loss, n.float() if torch.is_tensor(n) else torch.tensor(float(n), device=dev)])
        td.all_reduce(tot)
        assert int(tot[1]) == int(ref_n), (mode, tot, ref_n)
        assert abs(float(tot[0]) - float(ref_loss)) < 2e-2 * abs(float(ref_loss)), (mode, float(tot[0]), float(ref_loss))
        for k, gr in grads.items():
            td.all_reduce(gr)
            want = ref_g[k]
            err = (gr - want).abs().max().item()
            assert err < 0.05 * (want.abs().max().item() + 1e-3), (mode, k, err, want.abs().max().item())
    torch.cuda.synchronize()
    K.check_status(dev)
    td.barrier()
    if rank == 0:
        print("SPCP_OK")
    DL.check()
    td.destroy_process_group()


if __name__ == "__main__":
    main()
