"""Tensor / sampler / bookkeeping utilities shared by the trainers.

Same names and results as trl/trainer/utils.py (line references in each
docstring); the heavy ones (``selective_log_softmax``, ``entropy_from_logits``,
chunked lm-head log-probs) delegate to :mod:`trl_b200.ops`.
"""
from __future__ import annotations

import asyncio
import contextlib
import hashlib
import threading
from typing import Any, Iterable, Sequence

import numpy as np
import torch
import torch.nn as nn

from ..ops.functional import entropy_from_logits, selective_log_softmax  # noqa: F401  (re-exported)
from ..parallel.dist import ensure_master_addr_port  # noqa: F401  (re-exported)


def pad(tensors: list[torch.Tensor], padding_value: int = 0, padding_side: str = "right",
        pad_to_multiple_of: int | None = None) -> torch.Tensor:
    """Stack tensors of different leading sizes (utils.py:116-179)."""
    shape = np.max([t.shape for t in tensors], 0).tolist()
    if pad_to_multiple_of is not None:
        r = shape[0] % pad_to_multiple_of
        if r:
            shape[0] += pad_to_multiple_of - r
    out = torch.full((len(tensors), *shape), padding_value, dtype=tensors[0].dtype, device=tensors[0].device)
    for i, t in enumerate(tensors):
        n = t.shape[0]
        if padding_side == "left":
            sl = slice(shape[0] - n, shape[0])
        elif padding_side == "right":
            sl = slice(0, n)
        else:
            raise ValueError("padding_side must be 'left' or 'right'")
        out[(i, sl) + tuple(slice(0, s) for s in t.shape[1:])] = t
    return out


def disable_dropout_in_model(model: nn.Module) -> None:
    for m in model.modules():
        if isinstance(m, nn.Dropout):
            m.p = 0


def flush_left(mask: torch.Tensor, *tensors: torch.Tensor):
    """Shift every row left so its first non-zero mask entry sits in column 0, then drop
    trailing all-zero columns (utils.py:414-476)."""
    _, M = mask.shape
    first = mask.argmax(dim=1)
    pos = torch.arange(M, device=mask.device)[None]
    idx = (pos + first[:, None]).clamp(max=M - 1)
    valid_src = (pos + first[:, None]) < M
    mask_r = mask.gather(1, idx) * valid_src
    outs = [t.gather(1, idx) * valid_src.to(t.dtype) if t.ndim == 2 else t for t in tensors]
    keep = mask_r.sum(0) != 0
    last = int(keep.nonzero().max()) + 1 if keep.any() else 0
    mask_r = mask_r[:, :last]
    outs = [t[:, :last] for t in outs]
    return (mask_r, *outs) if tensors else mask_r


def flush_right(mask: torch.Tensor, *tensors: torch.Tensor):
    m = mask.flip(1)
    res = flush_left(m, *[t.flip(1) for t in tensors])
    if not tensors:
        return res.flip(1)
    return tuple(r.flip(1) for r in res)


class RepeatSampler:
    """Index sampler for online RL (utils.py:695-788): permute, cut into chunks of
    ``batch_size`` (incomplete tail dropped), emit every chunk ``repeat_count`` times and every
    index ``mini_repeat_count`` times."""

    def __init__(self, data_source, mini_repeat_count: int, batch_size: int = 1, repeat_count: int = 1,
                 shuffle: bool = True, seed: int | None = None):
        self.data_source, self.mini_repeat_count = data_source, mini_repeat_count
        self.batch_size, self.repeat_count, self.shuffle, self.seed = batch_size, repeat_count, shuffle, seed
        self.num_samples = len(data_source)
        self.generator = torch.Generator()
        if seed is not None:
            self.generator.manual_seed(seed)

    def __iter__(self):
        order = (torch.randperm(self.num_samples, generator=self.generator).tolist() if self.shuffle
                 else list(range(self.num_samples)))
        chunks = [order[i:i + self.batch_size] for i in range(0, len(order), self.batch_size)]
        for chunk in chunks:
            if len(chunk) != self.batch_size:
                continue
            for _ in range(self.repeat_count):
                for idx in chunk:
                    for _ in range(self.mini_repeat_count):
                        yield idx

    def __len__(self) -> int:
        return (self.num_samples // self.batch_size) * self.batch_size * self.mini_repeat_count * self.repeat_count


RepeatRandomSampler = RepeatSampler


class _RepeatedIterable:
    """Re-iterable view produced by :func:`repeat_iterable_dataset`; stays chained to its source so that ``set_epoch``
    reaches an upstream shuffle."""

    def __init__(self, rows, mini_repeat_count, batch_size, repeat_count):
        self.rows, self.mini_repeat_count, self.batch_size, self.repeat_count = rows, mini_repeat_count, batch_size, repeat_count

    def set_epoch(self, epoch: int):
        if hasattr(self.rows, "set_epoch"):
            self.rows.set_epoch(epoch)

    def __iter__(self):
        import copy

        buf = []
        for r in self.rows:
            buf.append(r)
            if len(buf) == self.batch_size:
                for _ in range(self.repeat_count):
                    for x in buf:
                        for _ in range(self.mini_repeat_count):
                            yield copy.deepcopy(x)  # every repeat is its own object, like a fresh dataset access
                buf = []
        # an incomplete last chunk is dropped, like RepeatSampler does


def repeat_iterable_dataset(rows: Iterable, mini_repeat_count: int, batch_size: int = 1, repeat_count: int = 1):
    """Streaming counterpart of :class:`RepeatSampler` (trl/trainer/utils.py:791-853): rows come out in the order in
    which the unshuffled sampler would emit their indices."""
    return _RepeatedIterable(rows, mini_repeat_count, batch_size, repeat_count)


def get_callable_name(func) -> str:
    """Display name of a reward callable: functions by ``__name__``, ``functools.partial`` objects by the function
    they wrap (however deeply nested), callable instances by their class (trl/trainer/utils.py:224-232)."""
    import functools

    while isinstance(func, functools.partial):
        func = func.func
    return getattr(func, "__name__", type(func).__name__)


def nanstd(t: torch.Tensor, dim=None, keepdim: bool = False) -> torch.Tensor:
    """Bessel-corrected std ignoring NaNs; NaN where fewer than two values (utils.py:857-890)."""
    if dim is None:
        v = t[~torch.isnan(t)]
        n = v.numel()
        if n <= 1:
            return t.new_tensor(float("nan"))
        return ((v - v.mean()) ** 2).sum().div(n - 1).sqrt()
    valid = ~torch.isnan(t)
    cnt = valid.sum(dim, keepdim=True)
    mean = torch.nansum(t, dim=dim, keepdim=True) / cnt.clamp_min(1)
    sq = torch.where(valid, (t - mean) ** 2, torch.zeros_like(t)).sum(dim, keepdim=True)
    out = (sq / (cnt - 1).clamp_min(1)).sqrt()
    out = torch.where(cnt > 1, out, torch.full_like(out, float("nan")))
    return out if keepdim else out.squeeze(dim)


def nanmin(t: torch.Tensor) -> torch.Tensor:
    v = t[~torch.isnan(t)]
    return v.min() if v.numel() else t.new_tensor(float("nan"))


def nanmax(t: torch.Tensor) -> torch.Tensor:
    v = t[~torch.isnan(t)]
    return v.max() if v.numel() else t.new_tensor(float("nan"))


def balanced_partition(costs: Sequence[float], parts: int, per_part: int) -> list[list[int]]:
    """Indices of ``costs`` dealt into ``parts`` lists of exactly ``per_part`` entries with near-equal cost sums:
    longest first, each to the least loaded part that still has room (ties: lowest part, then lowest index), so every
    rank that runs it on the same costs gets the same answer.  Each list comes back in ascending index order."""
    if len(costs) != parts * per_part:
        raise ValueError(f"{len(costs)} items cannot fill {parts} parts of {per_part}")
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    load, out = [0.0] * parts, [[] for _ in range(parts)]
    for i in order:
        p = min((q for q in range(parts) if len(out[q]) < per_part), key=lambda q: (load[q], q))
        out[p].append(i)
        load[p] += costs[i]
    return [sorted(x) for x in out]


class DeferredMetric:
    """A metric value whose cross-rank reduction waits for the next ``log`` call.

    The reference reduces every metric in the micro-batch that produced it (``accelerator.reduce`` /
    ``gather`` inside ``compute_loss``, e.g. trl/trainer/grpo_trainer.py:3226-3235), which makes every
    micro-batch a synchronisation point between ranks with different sequence lengths.  Here a micro-batch only
    records its local partial sums on the device; :func:`resolve_deferred_metrics` reduces all of them with ONE
    collective (and one host read) per logging step and yields the same numbers: ``ratio`` entries become
    ``sum_over_ranks(num) / max(sum_over_ranks(den), 1)``, ``mean`` entries the mean over ranks, ``sum`` entries
    the sum over ranks.
    """

    __slots__ = ("local", "kind")

    def __init__(self, local: torch.Tensor, kind: str):
        self.local, self.kind = local, kind


def defer_ratio(num: torch.Tensor, den: torch.Tensor) -> DeferredMetric:
    return DeferredMetric(torch.stack([num.detach().float().reshape(()), den.detach().float().reshape(())]), "ratio")


def defer_mean(value: torch.Tensor) -> DeferredMetric:
    return DeferredMetric(value.detach().float().reshape(1), "mean")


def resolve_deferred_metrics(metrics: dict) -> None:
    """Replace every :class:`DeferredMetric` in ``metrics`` (name -> list) by its globally reduced float.
    Every rank must hold the same entries in the same order (they do: the entries follow the code path, not the data)."""
    from ..parallel import dist as D

    pend = [(k, i) for k in sorted(metrics) for i, e in enumerate(metrics[k]) if isinstance(e, DeferredMetric)]
    if not pend:
        return
    flat = torch.cat([metrics[k][i].local for k, i in pend])
    world = D.world_size()
    if world > 1:
        D.all_reduce(flat, "sum")
    vals = flat.tolist()
    o = 0
    for k, i in pend:
        e = metrics[k][i]
        if e.kind == "ratio":
            metrics[k][i] = vals[o] / max(vals[o + 1], 1.0)
            o += 2
        else:
            metrics[k][i] = vals[o] / (world if e.kind == "mean" else 1)
            o += 1


def split_tensor_dict(d: dict[str, Any], num_chunks: int) -> list[dict[str, Any]]:
    """Equal dim-0 chunks; 0-dim tensors / scalars replicated, ``None`` preserved (utils.py:893-927)."""
    first = next(v for v in d.values() if torch.is_tensor(v) and v.ndim > 0)
    n = first.shape[0] // num_chunks
    out = []
    for i in range(num_chunks):
        c = {}
        for k, v in d.items():
            if torch.is_tensor(v) and v.ndim > 0:
                c[k] = v[i * n:(i + 1) * n]
            elif isinstance(v, list) and len(v) == first.shape[0]:
                c[k] = v[i * n:(i + 1) * n]
            else:
                c[k] = v
        out.append(c)
    return out


def shuffle_sequence_dict(d: dict[str, Any], generator: torch.Generator | None = None) -> dict[str, Any]:
    """One random permutation applied to every tensor / list along dim 0 (utils.py:930-957)."""
    first = next(v for v in d.values() if (torch.is_tensor(v) and v.ndim > 0) or isinstance(v, list))
    n = len(first)
    perm = torch.randperm(n, generator=generator)

    def p(v):
        if v is None:
            return None
        if torch.is_tensor(v) and v.ndim == 0:
            return v
        if torch.is_tensor(v):
            return v[perm.to(v.device)]
        if isinstance(v, list):
            return [v[i] for i in perm.tolist()]
        return v
    return {k: p(v) for k, v in d.items()}


# keys of a vision batch that travel with ``pixel_values`` and are split / merged with it, per layout
_VISION_COMPANIONS = ("image_grid_thw", "image_position_ids", "pixel_attention_mask", "spatial_shapes")


def split_pixel_values_by_grid(batch: dict) -> dict:
    """One ``pixel_values`` entry per sample instead of one flat tensor (``batch["num_images"]`` images per sample), so
    that samples can be shuffled or re-dealt between ranks (trl/trainer/utils.py:995-1043).  Three layouts:

    * ``image_grid_thw`` (Qwen2-VL family): ``pixel_values`` holds patches, image i owns ``prod(grid[i])`` rows;
    * ``image_position_ids`` (Gemma family): one ``pixel_values`` row per image;
    * ``spatial_shapes`` (LFM2-VL family): rows are tiles, ``batch["num_tiles"]`` of them per sample, with
      ``pixel_attention_mask`` and ``spatial_shapes`` split the same way.
    """
    if "pixel_values" not in batch or "num_images" not in batch:
        return batch
    pv, counts = batch["pixel_values"], [int(n) for n in batch["num_images"]]
    if "image_grid_thw" in batch:
        grid = batch["image_grid_thw"]
        per_image = grid.prod(-1).tolist()
        if sum(per_image) != pv.shape[0]:
            raise ValueError(f"image_grid_thw describes {sum(per_image)} patches, pixel_values has {pv.shape[0]} rows")
        rows, o = [], 0
        for n in counts:
            rows.append(sum(per_image[o:o + n]))
            o += n
        return {**batch, "pixel_values": list(torch.split(pv, rows, 0)), "image_grid_thw": list(torch.split(grid, counts, 0))}
    if "image_position_ids" in batch:
        return {**batch, "pixel_values": list(torch.split(pv, counts, 0)),
                "image_position_ids": list(torch.split(batch["image_position_ids"], counts, 0))}
    if "spatial_shapes" in batch:
        tiles = [int(n) for n in batch["num_tiles"]]
        return {**batch, "pixel_values": list(torch.split(pv, tiles, 0)),
                "pixel_attention_mask": list(torch.split(batch["pixel_attention_mask"], tiles, 0)),
                "spatial_shapes": list(torch.split(batch["spatial_shapes"], tiles, 0))}
    return batch


def unsplit_pixel_values_by_grid(batch: dict) -> dict:
    """Inverse of :func:`split_pixel_values_by_grid`: per-sample lists back to flat tensors."""
    out = dict(batch)
    for k in ("pixel_values",) + _VISION_COMPANIONS:
        if isinstance(out.get(k), list):
            out[k] = torch.cat(out[k], 0)
    return out


def hash_module(module: nn.Module) -> str:
    """sha256 over the sorted state dict: cache key for precomputed reference log-probs (utils.py:1173-1181)."""
    h = hashlib.sha256()
    for k, v in sorted(module.state_dict().items()):
        h.update(k.encode())
        h.update(str(v.dtype).encode())
        t = v.detach().cpu()
        if t.dtype in (torch.bfloat16,) or "float8" in str(t.dtype):
            t = t.float()
        h.update(t.contiguous().numpy().tobytes())
    return h.hexdigest()


@contextlib.contextmanager
def use_adapter(model, adapter_name: str | None):
    """``None`` disables LoRA inside the block (frozen reference policy); a name activates that
    adapter and restores the previous one afterwards (utils.py:1199-1236)."""
    if not hasattr(model, "set_adapter_enabled") and not hasattr(model, "active_adapter"):
        yield
        return
    if adapter_name is None:
        model.set_adapter_enabled(False)
        try:
            yield
        finally:
            model.set_adapter_enabled(True)
    else:
        prev = getattr(model, "active_adapter", "default")
        if adapter_name == prev and not hasattr(model, "set_adapter"):
            yield  # the model's one adapter is the active one already
            return
        if not hasattr(model, "set_adapter"):
            raise NotImplementedError(f"adapter {adapter_name!r}: native models carry one adapter ({prev!r}); a second set "
                                      "of adapter weights (for example a separate reference adapter) is not supported")
        model.set_adapter(adapter_name)
        try:
            yield
        finally:
            model.set_adapter(prev)


# ---- a daemon asyncio loop for async reward functions / tools (utils.py:1239-1288) ----
_loop = None
_loop_lock = threading.Lock()


def get_daemon_loop() -> asyncio.AbstractEventLoop:
    global _loop
    with _loop_lock:
        if _loop is None or _loop.is_closed():
            _loop = asyncio.new_event_loop()
            threading.Thread(target=_loop.run_forever, daemon=True, name="trl-b200-async").start()
    return _loop


def run_coroutine_sync(coro):
    return asyncio.run_coroutine_threadsafe(coro, get_daemon_loop()).result()


# ---- FLOP accounting (utils.py:1520-1630) --------------------------------------------
B200_PEAK_BF16_FLOPS = 2.25e15
H100_PEAK_BF16_FLOPS = 989.5e12


def compute_flops_per_token(config, seq_len: int) -> int:
    """Training FLOPs per token of a causal decoder: 3 x the forward pass (backward counted as twice the forward), two
    FLOPs per multiply-add.  Attention scores are counted against the whole ``seq_len`` (the non-causal convention of
    PaLM / Megatron; :func:`adjusted_mfu` removes the masked half).  Mixture-of-experts layers count the router and
    the ``num_experts_per_tok`` active experts; the embedding lookup is counted like a ``V x h`` product and the
    lm_head only when it is not tied to it (trl/trainer/utils.py:1520-1574)."""
    c = config
    h, L, V = c.hidden_size, c.num_hidden_layers, c.vocab_size
    hd = getattr(c, "head_dim", None) or h // c.num_attention_heads
    q, kv = c.num_attention_heads * hd, c.num_key_value_heads * hd
    attn = 2 * h * (q + 2 * kv) + 2 * q * h + 2 * 2 * q * seq_len
    dense_mlp = 2 * 3 * h * c.intermediate_size
    k = getattr(c, "num_experts_per_tok", None) or 0
    n_exp = getattr(c, "num_experts", None) or getattr(c, "num_local_experts", None) or 0
    if k and n_exp:
        sparse = k * 2 * 3 * h * c.moe_intermediate_size + 2 * h * n_exp
        step = getattr(c, "decoder_sparse_step", 1) or 1
        layers = sum(attn + (sparse if li % step == 0 else dense_mlp) for li in range(L))
    else:
        layers = L * (attn + dense_mlp)
    head = 0 if getattr(c, "tie_word_embeddings", False) else 2 * V * h
    return int(3 * (layers + 2 * V * h + head))


def compute_mfu(flops_per_token, tokens_per_second: float, world_size: int = 1,
                peak_flops_per_device: float = B200_PEAK_BF16_FLOPS) -> float:
    """Model FLOPs utilisation in percent: ``flops_per_token`` (from :func:`compute_flops_per_token`) times the job's
    tokens per second over the peak of ``world_size`` devices (default peak: B200 dense bf16; the reference defaults to
    an H100's 989.5e12).  Tokens that several ranks see together (sequence / context / tensor parallel groups) are to
    be counted once by the caller."""
    return 100.0 * float(flops_per_token) * tokens_per_second / (peak_flops_per_device * world_size)


def adjusted_mfu(mfu: float, config, seq_len: int) -> float:
    """``mfu`` corrected for causal masking: half of the attention-score FLOPs (``Q K^T`` and ``P V``) that
    :func:`compute_flops_per_token` counts are never done."""
    c = config
    hd = getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads
    full = compute_flops_per_token(c, seq_len)
    half_scores = c.num_hidden_layers * 3 * 2 * c.num_attention_heads * hd * seq_len
    return mfu * (full - half_scores) / full


def print_prompt_completions_sample(prompts: list, completions: list, rewards: dict[str, list[float]],
                                    advantages: list[float], step: int, num_samples: int | None = None,
                                    extra: dict[str, list] | None = None) -> None:
    """Rich table of sampled rollouts (utils.py:563-692); plain text when rich is unavailable."""
    n = len(prompts)
    idx = list(range(n))
    if num_samples is not None and 0 < num_samples < n:
        import random

        idx = random.sample(idx, num_samples)

    def text(x):
        if not isinstance(x, list):
            return str(x)
        parts = []
        for m in x:  # one block per message: the role on a line of its own, reasoning before the answer
            if m.get("role") == "tool" and "name" in m:
                body = f"{m['name']}({m.get('args')})"
            else:
                think = m.get("reasoning_content") or m.get("thinking")
                body = (str(think) + "\n" if think else "") + str(m.get("content", ""))
            parts.append(f"{str(m.get('role', '?')).upper()}\n{body}")
        return "\n\n".join(parts)
    try:
        from rich.console import Console
        from rich.panel import Panel
        from rich.table import Table
        from rich.text import Text

        table = Table(show_header=True, header_style="bold white", expand=True)
        table.add_column("Prompt", style="bright_yellow")
        table.add_column("Completion", style="bright_green")
        for k in rewards:
            table.add_column(k, style="bold cyan", justify="right")
        table.add_column("Advantage", style="bold magenta", justify="right")
        for k in (extra or {}):  # columns logged by reward functions come last
            table.add_column(k, style="magenta")
        for i in idx:
            table.add_row(Text(text(prompts[i])), Text(text(completions[i])), *[f"{rewards[k][i]:.2f}" for k in rewards],
                          f"{advantages[i]:.2f}", *[str(v[i]) for v in (extra or {}).values()])
            table.add_section()
        Console().print(Panel(table, expand=False, title=f"Step {step}", border_style="bold white"))
    except Exception:
        for i in idx:
            print(f"[step {step}] prompt={text(prompts[i])!r} completion={text(completions[i])!r} "
                  f"rewards={ {k: v[i] for k, v in rewards.items()} } adv={advantages[i]:.3f}")


def get_peft_config(model_args):
    """ModelConfig -> LoraConfig (utils.py:254-277)."""
    if not getattr(model_args, "use_peft", False):
        return None
    from ..models.lora import LoraConfig

    return LoraConfig(task_type=model_args.lora_task_type, r=model_args.lora_r,
                      target_modules=model_args.lora_target_modules, target_parameters=model_args.lora_target_parameters,
                      lora_alpha=model_args.lora_alpha, lora_dropout=model_args.lora_dropout, bias="none",
                      use_rslora=model_args.use_rslora, use_dora=model_args.use_dora,
                      modules_to_save=model_args.lora_modules_to_save)


def get_quantization_config(model_args):
    """4/8-bit loading needs bitsandbytes kernels, which this build does not carry."""
    if getattr(model_args, "load_in_4bit", False) or getattr(model_args, "load_in_8bit", False):
        raise NotImplementedError("load_in_4bit / load_in_8bit: no quantised-weight kernels in this build")
    return None


def create_model_from_path(model_id: str, architecture=None, **kwargs):
    """dtype defaults to float32 (utils.py:1123-1170); ``model_id`` is a local directory or a preset name."""
    from ..models.hf_io import load_model

    dtype = kwargs.pop("dtype", kwargs.pop("torch_dtype", "float32"))
    kwargs.pop("device_map", None)
    kwargs.pop("trust_remote_code", None)
    kwargs.pop("attn_implementation", None)
    kwargs.pop("revision", None)
    return load_model(model_id, dtype=dtype, **kwargs)


def maybe_gather_lm_head_ctx(model, engine=None):
    """Fused lm-head losses read the weight directly: under full-shard the head bucket must be
    materialised first (utils.py:188-221)."""
    if engine is not None and hasattr(engine, "gathered"):
        return engine.gathered(["lm_head", "embed_tokens"])
    return contextlib.nullcontext()


def generate_model_card(base_model=None, model_name="model", hub_model_id=None, dataset_name=None, tags=None,
                        trainer_name="Trainer", trainer_citation=None, template_file="lm_model_card.md", paper_title=None,
                        paper_id=None, wandb_url=None, comet_url=None, trackio_url=None, **_):
    """Renders ``trl_b200/templates/<template_file>`` (counterpart of trl/trainer/utils.py:280-411); returns the text."""
    import os
    import sys

    import jinja2

    import torch

    from .. import __version__

    here = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "templates", template_file)
    with open(here) as f:
        template = jinja2.Template(f.read())
    tags = list(dict.fromkeys((tags or []) + ["generated_from_trainer", "trl_b200"]))
    card = [f"base_model: {base_model}" if base_model else None, f"datasets: {dataset_name}" if dataset_name else None,
            "library_name: transformers", f"model_name: {model_name}", "tags:"] + [f"- {t}" for t in tags] + ["licence: license"]
    versions = "\n".join([f"- trl_b200: {__version__}", f"- PyTorch: {torch.__version__}",
                           f"- Python: {sys.version.split()[0]}"])
    return template.render(card_data="\n".join(c for c in card if c), model_name=model_name, base_model=base_model,
                           hub_model_id=hub_model_id or model_name, dataset_name=dataset_name, trainer_name=trainer_name,
                           trainer_citation=trainer_citation, paper_title=paper_title, paper_id=paper_id,
                           versions=versions, wandb_url=wandb_url, comet_url=comet_url, trackio_url=trackio_url)


# ---- small helpers kept for API compatibility (trl/trainer/utils.py) ----------------------------------------------------
def identity(x):
    return x


def remove_none_values(example):
    """``None`` entries removed from nested lists / mappings (a dataset transform: Arrow fills missing keys of
    heterogeneous rows with ``None``; trl/trainer/utils.py:1088-1131)."""
    from collections.abc import Mapping

    if isinstance(example, list):
        return [remove_none_values(v) if isinstance(v, (Mapping, list)) else v for v in example]
    if isinstance(example, Mapping):
        return {k: (remove_none_values(v) if isinstance(v, (Mapping, list)) else v) for k, v in example.items()
                if v is not None}
    raise TypeError("Input must be a list or a dictionary.")


def get_config_model_id(config) -> str:
    return getattr(config, "_name_or_path", "")


def start_event_loop_in_daemon(name: str | None = None):
    """New asyncio loop running forever in a daemon thread; returns (thread, loop, ready event)."""
    import threading

    loop = asyncio.new_event_loop()
    ready = threading.Event()

    def run():
        asyncio.set_event_loop(loop)
        loop.call_soon(ready.set)
        loop.run_forever()

    t = threading.Thread(target=run, name=name, daemon=True)
    t.start()
    return t, loop, ready


def shutdown_event_loop_in_daemon(thread, loop) -> None:
    if loop is None or thread is None:
        return
    loop.call_soon_threadsafe(loop.stop)
    thread.join(timeout=5)


def get_comet_experiment_url():
    """URL of the running Comet experiment, or None (comet_ml is optional and absent from offline images)."""
    try:
        import comet_ml
    except ImportError:
        return None
    exp = comet_ml.get_running_experiment()
    return exp.url if exp is not None else None


def get_trackio_space_url():
    try:
        from trackio import context_vars
    except ImportError:
        return None
    run = context_vars.current_run.get()
    if run is None or getattr(run, "_space_id", None) is None:
        return None
    return f"https://{run._space_id.replace('/', '-')}.hf.space?project={run.project}&runs={run.name}&sidebar=collapsed"


def log_table_to_comet_experiment(name: str, table) -> None:
    try:
        import comet_ml
    except ImportError as e:
        raise ModuleNotFoundError("The comet-ml is not installed. Please install it first: pip install comet-ml") from e
    exp = comet_ml.get_running_experiment()
    if exp is not None:
        exp.log_table(tabular_data=table, filename=name)


def __getattr__(name):  # names that live in the ops / parallel packages here, under the reference's module path
    if name in ("selective_log_softmax", "entropy_from_logits"):
        from ..oracle import ops as _o

        return getattr(_o, name)
    if name == "patch_chunked_lm_head":
        from ..ops.chunked_lm_head import patch_chunked_lm_head

        return patch_chunked_lm_head
    if name == "ensure_master_addr_port":
        from ..parallel.dist import ensure_master_addr_port

        return ensure_master_addr_port
    raise AttributeError(name)
