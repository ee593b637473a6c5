"""tcgen05 paged decode attention and the transposed-V cache writers vs fp32 PyTorch references (B200)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(q, kc, vct, lens, table, scale):
    """q [B,Hq,D]; kc [nb,64,Hk,D]; vct [nb,Hk,D,64]; attends over lens[b] tokens."""
    B, Hq, D = q.shape
    Hk = kc.shape[2]
    G = Hq // Hk
    out = torch.zeros(B, Hq, D, dtype=torch.float32, device=q.device)
    for b in range(B):
        n = int(lens[b])
        if n <= 0:
            continue
        pages = table[b, : (n + 63) // 64].long()
        k = kc[pages].float().reshape(-1, Hk, D)[:n]                       # [n, Hk, D]
        v = vct[pages].float().permute(0, 3, 1, 2).reshape(-1, Hk, D)[:n]  # [n, Hk, D]
        for h in range(Hq):
            s = (k[:, h // G] @ q[b, h].float()) * scale
            out[b, h] = torch.softmax(s, 0) @ v[:, h // G]
    return out


@pytest.mark.parametrize("groups", [1, 2])
@pytest.mark.parametrize("Hq,Hk,splits", [(28, 4, 3), (8, 2, 1), (14, 2, 2)])
def test_decode_attention_tc_matches_reference(Hq, Hk, splits, groups):
    from trl_b200.ops import cuda as K

    torch.manual_seed(0)
    D, bs = 128, 64
    lens = torch.tensor([1, 64, 65, 300, 129, 1280, 0, 777], dtype=torch.int32)
    B = lens.numel()
    max_blocks = 24
    nb = B * max_blocks + 3
    kc = torch.randn(nb, bs, Hk, D, device="cuda", dtype=torch.bfloat16)
    vct = torch.randn(nb, Hk, D, bs, device="cuda", dtype=torch.bfloat16)
    table = torch.randperm(nb)[: B * max_blocks].reshape(B, max_blocks).to(torch.int32).cuda()
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    part_o = torch.empty(B * Hq * splits * D, device="cuda")
    part_ml = torch.empty(B * Hq * splits * 2, device="cuda")
    out = torch.full((B, Hq, D), 7.0, device="cuda", dtype=torch.bfloat16)
    seq_lens = (lens - 1).cuda()  # the kernel attends over seq_lens + 1 tokens; -1 marks an inactive slot
    scale = 1 / math.sqrt(D)
    for _ in range(2):  # second call: barriers, TMEM and partial buffers are reusable
        K.paged_decode_attn_tc(q, kc, vct, seq_lens, None, table, scale, splits, part_o, part_ml, out, groups=groups)
    torch.cuda.synchronize()
    K.check_status(q.device)
    ref = _reference(q, kc, vct, lens, table, scale)
    err = (out.float() - ref).abs().max().item()
    assert err < 2e-2, err
    assert out[6].abs().max().item() == 0.0  # inactive slot


def test_transposed_v_cache_writers():
    from trl_b200.ops import cuda as K

    torch.manual_seed(1)
    Hq, Hk, D, bs = 8, 2, 128, 64
    B, max_blocks = 3, 4
    nb = B * max_blocks
    table = torch.randperm(nb).reshape(B, max_blocks).to(torch.int32).cuda()
    kc = torch.zeros(nb, bs, Hk, D, device="cuda", dtype=torch.bfloat16)
    vct = torch.zeros(nb, Hk, D, bs, device="cuda", dtype=torch.bfloat16)
    # prefill: 70 tokens of sequence 1, 5 tokens of sequence 2
    T = 75
    k = torch.randn(T, Hk, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(T, Hk, D, device="cuda", dtype=torch.bfloat16)
    tok_slot = torch.tensor([1] * 70 + [2] * 5, dtype=torch.int32, device="cuda")
    tok_pos = torch.tensor(list(range(70)) + list(range(5)), dtype=torch.int32, device="cuda")
    K.kv_write_prefill(k, v, tok_slot, tok_pos, table, bs, kc, vct, v_transposed=True)
    for t in (0, 63, 64, 69, 70, 74):
        slot, pos = int(tok_slot[t]), int(tok_pos[t])
        blk = int(table[slot, pos // bs])
        assert torch.equal(kc[blk, pos % bs], k[t])
        assert torch.equal(vct[blk, :, :, pos % bs], v[t])
    # decode append: one new token per sequence at positions (0, 70, 5)
    qkv = torch.randn(B, (Hq + 2 * Hk) * D, device="cuda", dtype=torch.bfloat16)
    seq_lens = torch.tensor([0, 70, 5], dtype=torch.int32, device="cuda")
    q_out = torch.empty(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    K.rope_kv_write(qkv, seq_lens, None, table, bs, q_out, kc, vct, Hq, Hk, D, 10000.0, v_transposed=True)
    vnew = qkv[:, (Hq + Hk) * D:].view(B, Hk, D)
    for b, pos in enumerate((0, 70, 5)):
        blk = int(table[b, pos // bs])
        assert torch.equal(vct[blk, :, :, pos % bs], vnew[b])
