"""Rollout engine: decode kernels vs PyTorch references, engine vs the eager generator (B200)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_paged_decode_attention_matches_reference():
    from trl_b200.ops import cuda as K

    torch.manual_seed(0)
    B, Hq, Hk, D, bs = 5, 8, 2, 128, 16
    lens = torch.tensor([1, 17, 300, 129, 64], dtype=torch.int32)
    max_blocks = 32
    nblocks = B * max_blocks
    kc = torch.randn(nblocks, bs, Hk, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(nblocks, bs, Hk, D, device="cuda", dtype=torch.bfloat16)
    perm = torch.randperm(nblocks)[: B * max_blocks].reshape(B, max_blocks).to(torch.int32).cuda()
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    splits = 3
    part_o = torch.empty(B * Hq * splits * D, device="cuda")
    part_ml = torch.empty(B * Hq * splits * 2, device="cuda")
    out = torch.empty(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    seq_lens = (lens - 1).cuda()  # kernel attends over seq_lens + 1 tokens
    K.paged_decode_attn(q, kc, vc, seq_lens, None, perm, bs, 1 / math.sqrt(D), splits, part_o, part_ml, out)
    for b in range(B):
        n = int(lens[b])
        blocks = perm[b, : (n + bs - 1) // bs].long()
        k = kc[blocks].reshape(-1, Hk, D)[:n].float()
        v = vc[blocks].reshape(-1, Hk, D)[:n].float()
        k = k.repeat_interleave(Hq // Hk, dim=1)
        v = v.repeat_interleave(Hq // Hk, dim=1)
        s = torch.einsum("hd,thd->ht", q[b].float(), k) / math.sqrt(D)
        o = torch.einsum("ht,thd->hd", torch.softmax(s, -1), v)
        assert torch.allclose(out[b].float(), o, atol=2e-2, rtol=2e-2), (b, (out[b].float() - o).abs().max())


def test_sampler_matches_distribution_and_logprob():
    from trl_b200.ops import cuda as K
    from trl_b200.rollout.sampling import SamplingParams, process_logits

    torch.manual_seed(0)
    V, B = 50, 4096
    row = torch.randn(V, device="cuda") * 2
    logits = row[None].repeat(B, 1).contiguous()
    sp = SamplingParams(temperature=0.8, eos_token_id=3, eos_prob_floor=0.2, min_p=0.01)
    tok = torch.empty(B, dtype=torch.int32, device="cuda")
    lp = torch.empty(B, dtype=torch.float32, device="cuda")
    step = torch.zeros(1, dtype=torch.int32, device="cuda")
    K.sample_tokens(logits, 1 / sp.temperature, sp.min_p, sp.eos_token_id, sp.eos_prob_floor, 123, step, False, tok, lp)
    ref_logp = torch.log_softmax(process_logits(row[None], sp), -1)[0]
    assert torch.allclose(lp, ref_logp[tok.long()], atol=1e-4)
    freq = torch.bincount(tok.long(), minlength=V).float() / B
    assert (freq - ref_logp.exp()).abs().max() < 0.03
    assert abs(freq[3].item() - max(0.2, ref_logp.exp()[3].item())) < 0.03
    # greedy
    K.sample_tokens(logits, 1.0, 0.0, None, 0.0, 0, step, True, tok, lp)
    assert (tok.long() == row.argmax()).all()


@pytest.mark.parametrize("block_size", [16, None])  # None: 64-token pages + tensor-core decode attention
def test_engine_greedy_matches_eager_generator(block_size):
    from trl_b200.rollout.engine import EagerGenerator, RolloutEngine
    from trl_b200.rollout.sampling import SamplingParams
    from trl_b200.testing import make_tiny_model

    model = make_tiny_model("tiny-qwen2", dtype=torch.bfloat16, device="cuda", hidden_size=256, num_attention_heads=2,
                            num_key_value_heads=1, head_dim=128, intermediate_size=512)
    torch.manual_seed(0)
    prompts = [torch.randint(5, 1000, (n,)).tolist() for n in (5, 70, 16, 130)]
    sp = SamplingParams(n=2, max_tokens=12, greedy=True, temperature=1.0, eos_token_id=2)
    eng = RolloutEngine(model, max_num_seqs=4, max_model_len=192, block_size=block_size, poll_every=4)
    assert eng.attn_tc == (block_size is None)
    outs = eng.generate(prompts, sp)
    ref = EagerGenerator(model).generate(prompts, sp)
    assert len(outs) == 8
    agree = sum(o.token_ids[:4] == r.token_ids[:4] for o, r in zip(outs, ref))
    assert agree >= 6, [(o.token_ids, r.token_ids) for o, r in zip(outs, ref)]
    for o, r in zip(outs, ref):
        if o.token_ids == r.token_ids:
            assert max(abs(a - b) for a, b in zip(o.logprobs, r.logprobs)) < 0.15


@pytest.mark.parametrize("block_size", [16, None])
def test_engine_sampling_with_shared_prefix_and_continuous_batching(block_size):
    from trl_b200.rollout.engine import RolloutEngine
    from trl_b200.rollout.sampling import SamplingParams
    from trl_b200.testing import make_tiny_model

    model = make_tiny_model("tiny-qwen2", dtype=torch.bfloat16, device="cuda", hidden_size=256, num_attention_heads=2,
                            num_key_value_heads=1, head_dim=128, intermediate_size=512)
    prompts = [list(range(10, 10 + n)) for n in (7, 16, 33 if block_size else 90)]
    sp = SamplingParams(n=4, max_tokens=20, temperature=1.0, eos_token_id=2, eos_prob_floor=0.1, seed=5)
    eng = RolloutEngine(model, max_num_seqs=5, max_model_len=128, block_size=block_size, poll_every=4)  # 12 requests > 5 slots
    outs = eng.generate(prompts, sp)
    assert len(outs) == 12 and all(o is not None for o in outs)
    assert all(1 <= len(o.token_ids) <= 20 and len(o.logprobs) == len(o.token_ids) for o in outs)
    assert any(o.finish_reason == "stop" for o in outs)
    assert eng.sched.num_free_blocks == eng.num_blocks  # everything released
    assert len({tuple(o.token_ids) for o in outs[:4]}) > 1  # samples of one prompt differ


def test_a_new_seed_changes_the_samples_but_not_the_captured_graph():
    """The seed reaches the sampler through the device-side step counter: same seed, same completions; another seed,
    other completions, with the decode graph of the first call replayed."""
    from trl_b200.rollout.engine import RolloutEngine
    from trl_b200.rollout.sampling import SamplingParams
    from trl_b200.testing import make_tiny_model

    model = make_tiny_model("tiny-qwen2", dtype=torch.bfloat16, device="cuda", hidden_size=256, num_attention_heads=2,
                            num_key_value_heads=1, head_dim=128, intermediate_size=512)
    prompts = [list(range(10, 10 + n)) for n in (7, 16)]
    eng = RolloutEngine(model, max_num_seqs=4, max_model_len=64, poll_every=4)

    def run(seed):
        sp = SamplingParams(n=2, max_tokens=12, temperature=1.0, eos_token_id=2, seed=seed)
        return [tuple(o.token_ids) for o in eng.generate(prompts, sp)]
    a = run(5)
    graph = eng._graph
    assert graph is not None
    b, c = run(6), run(5)
    assert eng._graph is graph          # no new capture for a new seed
    assert a == c and a != b


@pytest.mark.parametrize("B", [64, 16])  # 2 and 8 CTAs per row
def test_split_sampler_matches_distribution_and_logprob(B):
    from trl_b200.ops import cuda as K
    from trl_b200.rollout.sampling import SamplingParams, process_logits

    torch.manual_seed(0)
    V = 1024
    row = (torch.randn(V, device="cuda") * 3).to(torch.bfloat16)
    logits = row[None].repeat(B, 1).contiguous()
    sp = SamplingParams(temperature=0.7, eos_token_id=5, eos_prob_floor=0.1)
    ref_logp = torch.log_softmax(process_logits(row[None].float(), sp), -1)[0]
    tok = torch.full((B,), -1, dtype=torch.int32, device="cuda")
    lp = torch.empty(B, dtype=torch.float32, device="cuda")
    step = torch.zeros(1, dtype=torch.int32, device="cuda")
    counts = torch.zeros(V, device="cuda")
    n_calls = 4096 // B
    for i in range(n_calls):
        step.fill_(i)
        K.sample_tokens(logits, 1 / sp.temperature, 0.0, sp.eos_token_id, sp.eos_prob_floor, 77, step, False, tok, lp)
        assert 0 <= int(tok.min()) and int(tok.max()) < V  # checked on the host before it is used as an index
        assert torch.allclose(lp, ref_logp[tok.long()], atol=2e-3)
        counts += torch.bincount(tok.long(), minlength=V).float()
    freq = counts / (B * n_calls)
    assert (freq - ref_logp.exp()).abs().max() < 0.03
    assert abs(freq[5].item() - max(0.1, ref_logp.exp()[5].item())) < 0.03
    K.sample_tokens(logits, 1.0, 0.0, None, 0.0, 0, step, True, tok, lp)
    assert (tok.long() == row.float().argmax()).all()


def test_engine_moe_decode_under_cuda_graph_matches_eager():
    from trl_b200.rollout.engine import EagerGenerator, RolloutEngine
    from trl_b200.rollout.sampling import SamplingParams
    from trl_b200.testing import make_tiny_model

    model = make_tiny_model("tiny-qwen3-moe", dtype=torch.bfloat16, device="cuda", hidden_size=256, num_attention_heads=2,
                            num_key_value_heads=1, head_dim=128, moe_intermediate_size=128, num_experts=8)
    torch.manual_seed(0)
    prompts = [torch.randint(5, 1000, (n,)).tolist() for n in (9, 70, 33)]
    sp = SamplingParams(n=2, max_tokens=10, greedy=True, eos_token_id=2)
    eng = RolloutEngine(model, max_num_seqs=6, max_model_len=128, poll_every=4)
    assert eng.use_graph
    outs = eng.generate(prompts, sp)
    ref = EagerGenerator(model).generate(prompts, sp)
    agree = sum(o.token_ids[:3] == r.token_ids[:3] for o, r in zip(outs, ref))
    assert agree >= 4, [(o.token_ids, r.token_ids) for o, r in zip(outs, ref)]


def test_engine_generates_from_image_prompts_like_the_eager_generator():
    """Vision-language model: image features are spliced into the prefill embeddings; decode is the text path."""
    from trl_b200.models.configuration import preset
    from trl_b200.models.vision import VisionArch, VisionLanguageModel, VlmArch
    from trl_b200.rollout.engine import EagerGenerator, RolloutEngine
    from trl_b200.rollout.sampling import SamplingParams

    torch.manual_seed(0)
    text = preset("tiny-qwen2", hidden_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                  intermediate_size=512)
    vis = VisionArch(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2, image_size=28,
                     patch_size=14)
    cfg = VlmArch(text=text, vision=vis, image_token_index=7)
    model = VisionLanguageModel(cfg, dtype=torch.bfloat16, device="cuda")
    n_img_tok = cfg.image_seq_length
    prompts, images = [], []
    for n_img, tail in ((1, 9), (2, 40), (0, 12)):
        p = [11, 12]
        for _ in range(n_img):
            p += [7] * n_img_tok + [13]
        p += torch.randint(20, 1000, (tail,)).tolist()
        prompts.append(p)
        images.append(torch.randn(n_img, 3, 28, 28) if n_img else None)
    sp = SamplingParams(n=2, max_tokens=8, greedy=True, temperature=1.0, eos_token_id=2)
    eng = RolloutEngine(model, max_num_seqs=6, max_model_len=128, poll_every=4)
    outs = eng.generate(prompts, sp, images=images)
    ref = EagerGenerator(model).generate(prompts, sp, images=images)
    assert len(outs) == 6
    agree = sum(o.token_ids[:3] == r.token_ids[:3] for o, r in zip(outs, ref))
    assert agree >= 4, [(o.token_ids, r.token_ids) for o, r in zip(outs, ref)]
    # the images matter: other pixels, other continuation for at least one image prompt
    other = [None if x is None else torch.randn_like(x) * 3 for x in images]
    outs2 = eng.generate(prompts, sp, images=other)
    assert any(a.token_ids != b.token_ids for a, b in zip(outs[:4], outs2[:4]))


def test_engine_generates_with_multimodal_rope_like_the_eager_generator():
    """Qwen2-VL layout: images of different sizes as flat patches, three rotary position rows in the prefill, and a
    per-slot rotary lead in the decode kernels (an image advances the position by less than its token count)."""
    from trl_b200.models.configuration import preset
    from trl_b200.models.vision_qwen import Qwen2VLArch, Qwen2VLModel, QwenVisionArch, patchify
    from trl_b200.rollout.engine import EagerGenerator, RolloutEngine
    from trl_b200.rollout.sampling import SamplingParams

    torch.manual_seed(0)
    text = preset("tiny-qwen2", hidden_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                  intermediate_size=512)
    text.extra["mrope_section"] = [16, 24, 24]
    vis = QwenVisionArch(depth=2, embed_dim=64, hidden_size=256, num_heads=2, mlp_ratio=2)
    cfg = Qwen2VLArch(text, vis, image_token_id=7)
    model = Qwen2VLModel(cfg, dtype=torch.bfloat16, device="cuda")
    prompts, images = [], []
    for sizes, tail in (((56, 112),), 9), (((28, 28), (84, 56)), 40), ((), 12):
        p, pv, grids = [11, 12], [], []
        for h, w in sizes:
            a, g = patchify(torch.randn(1, 3, h, w), vis)
            pv.append(a)
            grids.append(g)
            p += [7] * (a.shape[0] // 4) + [13]
        p += torch.randint(20, 1000, (tail,)).tolist()
        prompts.append(p)
        images.append((torch.cat(pv), torch.cat(grids)) if sizes else None)
    sp = SamplingParams(n=2, max_tokens=8, greedy=True, temperature=1.0, eos_token_id=2)
    eng = RolloutEngine(model, max_num_seqs=6, max_model_len=128, poll_every=4)
    assert eng.rope_delta is not None
    outs = eng.generate(prompts, sp, images=images)
    # 56 x 112 -> 2 x 4 merged tokens that advance the position by 4 (lead -4); 28 x 28 -> one token (0) and
    # 84 x 56 -> 3 x 2 tokens that advance it by 3 (-3); no lead for the text prompt
    assert sorted(eng.rope_delta.tolist()) == [-4, -4, -3, -3, 0, 0]
    ref = EagerGenerator(model).generate(prompts, sp, images=images)
    agree = sum(o.token_ids[:3] == r.token_ids[:3] for o, r in zip(outs, ref))
    assert agree >= 4, [(o.token_ids, r.token_ids) for o, r in zip(outs, ref)]
    outs_text = eng.generate(prompts[2:], sp)  # the slots are reused: the lead of a text prompt is zero again
    assert sorted(eng.rope_delta.tolist())[-2:] == [0, 0] and len(outs_text) == 2
    assert [o.token_ids[:3] for o in outs_text] == [o.token_ids[:3] for o in outs[4:]]
