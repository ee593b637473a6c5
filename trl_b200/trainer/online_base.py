"""Shared machinery of the online-RL trainers (GRPO, RLOO): prompt sampling schedule,
generation through the rollout engine, reward evaluation, per-token log-probabilities.

Follows the skeleton of trl/trainer/grpo_trainer.py (dataloader/sampler :1213-1271,
``_prepare_inputs`` buffering :1555-1584, ``_generate`` :2143-2258, ``_calculate_rewards``
:1612-1703, ``_get_per_token_logps_and_entropies`` :1435-1541) with the forward kept
padding-free and the lm_head fused with the log-softmax gather.
"""
from __future__ import annotations

import asyncio
import copy
import inspect
import itertools
import os
import warnings
from collections import defaultdict, deque
from typing import Any, Callable, Optional

import numpy as np
import torch
import torch.nn as nn

from ..data_utils import apply_chat_template, is_conversational, maybe_apply_chat_template
from ..loop.trainer import Trainer
from ..models.decoder import CausalLM, SeqCtx
from ..models.vision import merge_vision_entries, same_vision_entry
from ..ops import functional as ops
from ..parallel import dist as D
from ..rollout.sampling import SamplingParams
from .utils import (RepeatSampler, get_callable_name, create_model_from_path, disable_dropout_in_model, nanmax, nanmin, nanstd, pad,
                    print_prompt_completions_sample, resolve_deferred_metrics, run_coroutine_sync, shuffle_sequence_dict, split_tensor_dict,
                    use_adapter)

RewardFunc = Any


def _identity(x):
    return x


class OnlineTrainer(Trainer):
    _name = "Online"

    def __init__(self, model, reward_funcs, args, train_dataset=None, eval_dataset=None, processing_class=None,
                 reward_processing_classes=None, callbacks=None, optimizers=(None, None), peft_config=None,
                 tools=None, rollout_func=None, environment_factory=None):
        if isinstance(model, str):
            kw = dict(args.model_init_kwargs or {})
            model_id = model
            model = create_model_from_path(model, **kw)
        else:
            model_id = getattr(model, "name_or_path", "")
        if peft_config is not None:
            from ..models.lora import get_peft_model

            model = get_peft_model(model, peft_config)
        if processing_class is None:
            from transformers import AutoTokenizer

            processing_class = AutoTokenizer.from_pretrained(model_id, padding_side="left")
        tok = processing_class
        if tok.pad_token is None:
            tok.pad_token = tok.eos_token
        self.pad_token_id, self.eos_token_id = tok.pad_token_id, tok.eos_token_id
        # ---- reward functions -------------------------------------------------------------------
        if not isinstance(reward_funcs, list):
            reward_funcs = [reward_funcs]
        self.reward_func_names = []
        for i, rf in enumerate(reward_funcs):
            if isinstance(rf, str):
                reward_funcs[i] = create_model_from_path(rf, num_labels=1, **dict(args.model_init_kwargs or {}))
                reward_funcs[i].name_or_path = rf
            if isinstance(reward_funcs[i], nn.Module):
                self.reward_func_names.append(os.path.basename(str(getattr(reward_funcs[i], "name_or_path", f"reward_model_{i}"))) or f"reward_model_{i}")
            else:
                self.reward_func_names.append(get_callable_name(reward_funcs[i]))
        self.reward_funcs = reward_funcs
        if args.reward_weights is not None:
            if len(args.reward_weights) != len(reward_funcs):
                raise ValueError(f"Number of reward weights ({len(args.reward_weights)}) must match number of reward "
                                 f"functions ({len(reward_funcs)})")
            self.reward_weights = torch.tensor(args.reward_weights, dtype=torch.float32)
        else:
            self.reward_weights = torch.ones(len(reward_funcs), dtype=torch.float32)
        if reward_processing_classes is None:
            reward_processing_classes = [None] * len(reward_funcs)
        elif not isinstance(reward_processing_classes, list):
            reward_processing_classes = [reward_processing_classes]
        if len(reward_processing_classes) != len(reward_funcs):
            raise ValueError("The number of reward processing classes must match the number of reward functions.")
        for i, rf in enumerate(reward_funcs):
            if isinstance(rf, nn.Module) and reward_processing_classes[i] is None:
                reward_processing_classes[i] = tok
        self.reward_processing_classes = reward_processing_classes
        # ---- generation settings -------------------------------------------------------------------
        self.tools, self.rollout_func, self.environment_factory = tools or [], rollout_func, environment_factory
        self.max_completion_length = args.max_completion_length
        self.num_generations = args.num_generations
        self.num_generations_eval = args.num_generations_eval or args.num_generations
        self.temperature, self.top_p, self.top_k, self.min_p = args.temperature, args.top_p, args.top_k, args.min_p
        self.repetition_penalty = args.repetition_penalty
        self.chat_template_kwargs = args.chat_template_kwargs or {}
        self.num_iterations, self.beta = args.num_iterations, args.beta
        self.epsilon_low = args.epsilon
        self.epsilon_high = args.epsilon_high if args.epsilon_high is not None else args.epsilon
        self.mask_truncated_completions = args.mask_truncated_completions
        self.shuffle_dataset = args.shuffle_dataset
        self.use_vllm = args.use_vllm
        self._step = 0
        self._buffered_inputs = None
        self._last_loaded_step = -1
        self.num_completions_to_print = args.num_completions_to_print
        self.log_completions = args.log_completions
        self._logs = {"prompt": deque(), "completion": deque(), "rewards": defaultdict(deque), "advantages": deque(),
                      "extra": defaultdict(deque)}
        self._total_train_tokens = 0
        if args.disable_dropout:
            disable_dropout_in_model(model)
        super().__init__(optimizers=optimizers, model=model, args=args, data_collator=_identity, train_dataset=train_dataset,
                         eval_dataset=eval_dataset, processing_class=tok, callbacks=callbacks)
        self.model_accepts_loss_kwargs = False
        self.compute_loss_func = "non-None: the trainer divides by the accumulation steps itself"
        # ---- reference policy ---------------------------------------------------------------------------
        self.ref_model = None
        self._ref_is_adapter_off = False
        if self.beta != 0.0 or getattr(args, "_needs_ref", False):
            if getattr(self.model, "peft_config", None) is not None:
                self._ref_is_adapter_off = True
            else:
                self.ref_model = copy.deepcopy(self.model).eval().requires_grad_(False)
        for i, rf in enumerate(self.reward_funcs):
            if isinstance(rf, nn.Module):
                self.reward_funcs[i] = rf.to(self.args.device).eval().requires_grad_(False)
        if args.sync_ref_model and self.ref_model is not None:
            from .callbacks import SyncRefModelCallback

            self.add_callback(SyncRefModelCallback(ref_model=self.ref_model))
        self._rollout = None

    # ---- sampling schedule --------------------------------------------------------------------------------
    def _get_train_sampler(self, dataset=None):
        ds = dataset if dataset is not None else self.train_dataset
        a = self.args
        return RepeatSampler(ds, mini_repeat_count=self.num_generations,
                             batch_size=a.generation_batch_size // self.num_generations,
                             repeat_count=self.num_iterations * a.steps_per_generation, shuffle=self.shuffle_dataset,
                             seed=a.seed)

    def _get_eval_sampler(self, dataset):
        return RepeatSampler(dataset, mini_repeat_count=self.num_generations_eval, seed=self.args.seed, shuffle=False)

    def get_train_dataloader(self):
        self._train_batch_size = self.args.per_device_train_batch_size * self.args.steps_per_generation
        ds = self.train_dataset
        if ds is not None and (not hasattr(ds, "__len__") or not hasattr(ds, "__getitem__")):
            # streaming dataset: the same repetition pattern as RepeatSampler, applied to the stream (needs max_steps)
            from .utils import repeat_iterable_dataset

            a = self.args
            held, self.train_dataset = ds, repeat_iterable_dataset(
                ds, self.num_generations, a.generation_batch_size // self.num_generations,
                self.num_iterations * a.steps_per_generation)
            try:
                return super().get_train_dataloader()
            finally:
                self.train_dataset = held
        return super().get_train_dataloader()

    def _count_items(self, batches):
        return None

    def _prepare_inputs(self, generation_batch):
        """Generate once per ``steps_per_generation * num_iterations`` calls; serve slices in between."""
        mode = "train" if self.model.training else "eval"
        if mode == "train":
            a = self.args
            generate_every = a.steps_per_generation * self.num_iterations
            if self._step % generate_every == 0 or self._buffered_inputs is None:
                batch = self._generate_and_score_completions(generation_batch)
                batch = shuffle_sequence_dict(batch)
                self._buffered_inputs = split_tensor_dict(batch, a.steps_per_generation)
            inputs = self._buffered_inputs[self._step % a.steps_per_generation]
        else:
            inputs = self._generate_and_score_completions(generation_batch)
        return inputs

    def training_step(self, model, inputs, num_items_in_batch=None):
        import time

        t0 = time.perf_counter()
        out = super().training_step(model, inputs, num_items_in_batch)
        self._step += 1
        self._metrics["train"]["step_time"].append(time.perf_counter() - t0)
        return out

    # ---- generation ---------------------------------------------------------------------------------------------
    def _sampling_params(self, n: int = 1) -> SamplingParams:
        a = self.args
        return SamplingParams(n=n, temperature=self.temperature, top_p=self.top_p, top_k=self.top_k or 0,
                              min_p=self.min_p or 0.0, repetition_penalty=self.repetition_penalty,
                              max_tokens=self.max_completion_length, eos_token_id=self.eos_token_id,
                              eos_prob_floor=a.eos_prob_floor, seed=a.seed + 7919 * self.state.global_step + D.rank(),
                              **(a.generation_kwargs or {}))

    def _get_rollout(self):
        a0 = self.args
        if a0.use_vllm and a0.vllm_mode == "server":  # generation lives in another process: `trl vllm-serve`
            if self._rollout is None:
                from ..generation.server_rollout import ServerRollout

                self._rollout = ServerRollout(self.model, base_url=a0.vllm_server_base_url, host=a0.vllm_server_host,
                                              port=a0.vllm_server_port, timeout=a0.vllm_server_timeout,
                                              client=getattr(self, "_rollout_client", None))
            return self._rollout
        gen_model = self.model
        if getattr(getattr(self, "engine", None), "mode", "") == "full_shard_stream":
            # the training side holds one layer at a time: generation gets its own whole replica, refreshed from the
            # slices before every generation batch (`export_weights`)
            if getattr(self.model, "is_vlm", False):
                raise NotImplementedError("streamed full shard with a vision-language generation replica")
            if getattr(self, "_gen_model", None) is None:
                self._gen_model = CausalLM(self.model.config, dtype=self.model.dtype, device=self.args.device, init=False)
                self._gen_model.eval().requires_grad_(False)
            gen_model = self._gen_model
        elif (getattr(self.model, "peft_config", None) is not None and self.args.device.type == "cuda"
              and any(len(l.lora) for l in self.model.layers)):
            # adapters: the decode kernels read plain weight matrices, so generation gets a replica with the adapters
            # folded in, refreshed before every generation batch (`export_merged_weights`); the eager generator on
            # CPU runs the adapted model itself
            if getattr(self.model, "is_vlm", False):
                raise NotImplementedError("adapters with a vision-language generation replica")
            if getattr(self, "_gen_model", None) is None:
                self._gen_model = CausalLM(self.model.config, dtype=self.model.dtype, device=self.args.device, init=False)
                self._gen_model.eval().requires_grad_(False)
                self._gen_merged = True
            gen_model = self._gen_model
        if self._rollout is None:
            if self.args.device.type == "cuda":
                from ..rollout.engine import RolloutEngine

                a = self.args
                max_len = a.vllm_max_model_length or (self._max_prompt_len_seen + self.max_completion_length + 8)
                bs = a.rollout_block_size or None  # None: the engine picks the page size
                max_len = (max_len + 63) // 64 * 64
                tp = int(a.vllm_tensor_parallel_size or 1)
                nseq = a.per_device_train_batch_size * a.steps_per_generation
                if tp > 1 and D.world_size() > 1:
                    from ..rollout.tp_engine import TPRolloutEngine

                    if D.world_size() % tp != 0:
                        raise ValueError(f"vllm_tensor_parallel_size ({tp}) must divide the world size ({D.world_size()})")
                    groups = [list(range(i, i + tp)) for i in range(0, D.world_size(), tp)]
                    self._tp_group = D.new_subgroups_by_enumeration(groups)
                    self._rollout = TPRolloutEngine(gen_model, self._tp_group, max_num_seqs=nseq, max_model_len=max_len,
                                                    block_size=bs, poll_every=a.rollout_poll_every)
                else:
                    try:
                        self._rollout = RolloutEngine(gen_model, max_num_seqs=nseq, max_model_len=max_len, block_size=bs,
                                                      poll_every=a.rollout_poll_every)
                    except NotImplementedError as e:  # e.g. GeGLU models: correct but slow eager generation
                        import warnings

                        from ..rollout.engine import EagerGenerator

                        warnings.warn(f"{e}; falling back to the eager generator")
                        self._rollout = EagerGenerator(gen_model)
            else:
                from ..rollout.engine import EagerGenerator

                self._rollout = EagerGenerator(gen_model)
        return self._rollout

    def _tokenize_prompts_with_images(self, prompts: list, images: list):
        """Vision-language prompts: the processor expands every image placeholder and converts the images.
        Returns (prompt ids, per-prompt image entries: pixel tensors [n_images_i, C, S, S], or (patches, grid) pairs
        for towers that take images of any size)."""
        from ..data_utils import prepare_multimodal_messages

        proc = self.processing_class
        if not hasattr(proc, "tokenizer"):
            raise ValueError("prompts with images need a processor (image processor + tokenizer) as processing_class")
        imgs = [list(i) if i is not None else [] for i in images]
        if prompts and is_conversational({"prompt": prompts[0]}):
            msgs = [prepare_multimodal_messages(p, images=i) for p, i in zip(prompts, imgs)]
            texts = proc.apply_chat_template(msgs, tools=self.tools or None, add_generation_prompt=True, tokenize=False,
                                             **self.chat_template_kwargs)
        else:
            texts = list(prompts)
        enc = proc(images=imgs if any(imgs) else None, text=texts, add_special_tokens=False, return_tensors=None)
        ids = [list(x) for x in enc["input_ids"]]
        from ..models.vision import split_vision_batch

        return ids, split_vision_batch(enc, [len(i) for i in imgs])

    def _tokenize_prompts(self, prompts: list):
        tok = self.processing_class
        if prompts and is_conversational({"prompt": prompts[0]}):
            ids = [tok.apply_chat_template(p, tools=self.tools or None, add_generation_prompt=True, tokenize=True,
                                           return_dict=True, **self.chat_template_kwargs)["input_ids"] for p in prompts]
            ids = [i[0] if i and isinstance(i[0], list) else i for i in ids]
        else:
            ids = tok(text=list(prompts), add_special_tokens=False)["input_ids"] if not getattr(
                tok, "add_bos_token", False) else tok(text=list(prompts))["input_ids"]
        return ids

    def _generate(self, prompts: list, images: list | None = None):
        """Returns (prompt_ids, completion_ids, sampling logprobs | None, extras).  ``images``: per prompt a list of
        images (vision-language models); their pixel tensors come back in ``extras["pixel_values_list"]``."""
        extras = {}
        if self.rollout_func is not None:
            out = self.rollout_func(prompts, self)
            for k in ("prompt_ids", "completion_ids", "logprobs"):
                if k not in out:
                    raise ValueError(f"rollout_func must return {k!r}")
            extras = {k: v for k, v in out.items() if k not in ("prompt_ids", "completion_ids", "logprobs")}
            return out["prompt_ids"], out["completion_ids"], out["logprobs"], extras
        pixels = None
        if images is not None and any(i for i in images):
            if self.rollout_func is not None:
                raise ValueError("rollout_func and image prompts cannot be combined")
            prompt_ids, pixels = self._tokenize_prompts_with_images(prompts, images)
            extras["pixel_values_list"] = pixels
        elif prompts and isinstance(prompts[0], (list, tuple)) and prompts[0] and isinstance(prompts[0][0], int):
            prompt_ids = [list(p) for p in prompts]  # pre-tokenised prompts (synthetic benchmarks, custom pipelines)
        else:
            prompt_ids = self._tokenize_prompts(prompts)
        self._max_prompt_len_seen = max([len(p) for p in prompt_ids] + [getattr(self, "_max_prompt_len_seen", 0)])
        # identical consecutive prompts (the num_generations copies) are sent once with n>1 so that
        # the engine shares their prompt KV blocks
        uniq, counts, uniq_px = [], [], []
        for j, p in enumerate(prompt_ids):
            px = pixels[j] if pixels is not None else None
            same_px = px is None or (bool(uniq_px) and same_vision_entry(uniq_px[-1], px))
            if uniq and uniq[-1] == p and same_px and counts[-1] < self.num_generations:
                counts[-1] += 1
            else:
                uniq.append(p)
                uniq_px.append(px)
                counts.append(1)
        gen_kw = {"images": uniq_px} if pixels is not None else {}
        eng = self._get_rollout()
        if self.state.global_step != self._last_loaded_step and getattr(self, "_gen_model", None) is not None:
            with self._profile("sync_weights"):  # slices of the streamed engine -> the whole generation replica
                if getattr(self, "_gen_merged", False):  # adapters folded into the replica, the policy left as it is
                    from ..models.lora import export_merged_weights

                    export_merged_weights(self.model, self._gen_model)
                else:
                    self.engine.export_weights(self._gen_model)
                if hasattr(eng, "sync_weights"):
                    eng.sync_weights()
            self._last_loaded_step = self.state.global_step
        elif self.state.global_step != self._last_loaded_step and hasattr(eng, "sync_weights"):
            with self._profile("sync_weights"):  # trainer -> generator weights (no-op when storage is shared)
                sharded = getattr(self, "engine", None) is not None and hasattr(self.engine, "gather_full_params")
                if sharded and hasattr(eng, "w") and getattr(eng, "tp", 1) > 1:
                    # full shard -> TP layout: every TP rank pulls exactly its slices from the owners' shards
                    if getattr(self, "_resharder", None) is None:
                        from ..parallel.reshard import WeightResharder

                        self._resharder = WeightResharder(self.engine, eng)
                    self._resharder.run()
                else:
                    if sharded:
                        self.engine.gather_full_params()  # the generator reads the policy's buffers directly
                    eng.sync_weights()
            self._last_loaded_step = self.state.global_step
        with self._profile("rollout.generate"):
            if len(set(counts)) == 1:
                outs = eng.generate(uniq, self._sampling_params(counts[0]), **gen_kw)
            else:
                outs = []
                for j, (p, c) in enumerate(zip(uniq, counts)):
                    kw1 = {"images": [uniq_px[j]]} if pixels is not None else {}
                    outs.extend(eng.generate([p], self._sampling_params(c), **kw1))
        completion_ids = [o.token_ids for o in outs]
        logprobs = [o.logprobs for o in outs]
        return prompt_ids, completion_ids, logprobs, extras

    def _profile(self, name):
        from ..extras.profiling import profiling_context

        return profiling_context(self, name)

    # ---- rewards ---------------------------------------------------------------------------------------------------
    def _calculate_rewards(self, inputs, prompts, completions, completion_ids_list):
        dev = self.args.device
        rewards = torch.zeros(len(prompts), len(self.reward_funcs), device=dev)
        keys = [k for k in inputs[0] if k not in ("prompt", "completion", "completion_ids")]
        kwargs = {k: [ex[k] for ex in inputs] for k in keys}
        kwargs["trainer_state"] = self.state
        extra_cols, extra_metrics = defaultdict(list), defaultdict(list)
        kwargs["log_extra"] = lambda name, values: extra_cols[name].extend(values)
        kwargs["log_metric"] = lambda name, value: extra_metrics[name].append(float(value))
        for i, (rf, rpc, name) in enumerate(zip(self.reward_funcs, self.reward_processing_classes, self.reward_func_names)):
            with self._profile(name):
                if isinstance(rf, nn.Module):
                    if is_conversational(inputs[0]):
                        texts = [apply_chat_template({"messages": p + c}, rpc)["text"] for p, c in zip(prompts, completions)]
                    else:
                        texts = [p + c for p, c in zip(prompts, completions)]
                    enc = rpc(text=texts, return_tensors="pt", padding=True, padding_side="right", add_special_tokens=False)
                    with torch.inference_mode():
                        out = rf(input_ids=enc["input_ids"].to(dev), attention_mask=enc["attention_mask"].to(dev))
                    rewards[:, i] = out.logits[:, 0].float()
                else:
                    sig_kwargs = dict(prompts=prompts, completions=completions, completion_ids=completion_ids_list, **kwargs)
                    try:
                        params = inspect.signature(rf).parameters
                        if not any(p.kind == p.VAR_KEYWORD for p in params.values()):
                            sig_kwargs = {k: v for k, v in sig_kwargs.items() if k in params}
                    except (TypeError, ValueError):
                        pass
                    res = rf(**sig_kwargs)
                    if asyncio.iscoroutine(res):
                        res = run_coroutine_sync(res)
                    res = [r if r is not None else float("nan") for r in res]
                    rewards[:, i] = torch.tensor(res, dtype=torch.float32, device=dev)
        if torch.isnan(rewards).all(dim=1).any():
            idx = int(torch.isnan(rewards).all(dim=1).nonzero()[0])
            warnings.warn(f"All reward functions returned None for prompt={prompts[idx]!r}; it carries no signal.")
        self._extra_cols, self._extra_metrics = extra_cols, extra_metrics
        return D.gather(rewards)

    # ---- log-probabilities --------------------------------------------------------------------------------------------
    def _get_per_token_logps_and_entropies(self, model, prompt_ids, completion_ids, batch_size=None,
                                           compute_entropy=False, temperature=None, pixel_values_list=None,
                                           entropy_grad=False):
        """prompt_ids / completion_ids: lists of id lists.  Returns padded [B, Tc] log-probs (and entropies).
        ``pixel_values_list``: per sequence the pixel tensor of its images (vision-language models).
        ``entropy_grad``: the entropies are differentiable (entropy bonus) instead of detached statistics."""
        temperature = self.temperature if temperature is None else temperature
        dev = self.args.device
        B = len(prompt_ids)
        Tc = max(1, max(len(c) for c in completion_ids))
        bs = batch_size or B
        logps = torch.zeros(B, Tc, dtype=torch.float32, device=dev)
        ents = torch.zeros(B, Tc, dtype=torch.float32, device=dev) if compute_entropy else None
        aux_total = None
        for s in range(0, B, bs):
            # all index vectors of the micro-batch are built on the host with numpy and travel in ONE pinned buffer
            # (asynchronous copy), so the host prepares the next micro-batch while the GPU is still on this one
            P, C = prompt_ids[s:s + bs], completion_ids[s:s + bs]
            lp_ = np.fromiter((len(x) for x in P), dtype=np.int64, count=len(P))
            lc_ = np.fromiter((len(x) for x in C), dtype=np.int64, count=len(C))
            lens = lp_ + lc_
            total, n_sel = int(lens.sum()), int(lc_.sum())
            if n_sel == 0:
                continue
            starts = np.concatenate([[0], np.cumsum(lens)])
            c_starts = np.concatenate([[0], np.cumsum(lc_)])[:-1]
            k = len(P)
            packed = np.empty(2 * total + (k + 1) + 3 * n_sel, dtype=np.int64)
            o_pos, o_cu, o_sel, o_row, o_col = total, 2 * total, 2 * total + k + 1, 2 * total + k + 1 + n_sel, \
                2 * total + k + 1 + 2 * n_sel
            packed[:total] = np.fromiter(itertools.chain.from_iterable(itertools.chain.from_iterable(zip(P, C))),
                                         dtype=np.int64, count=total)
            packed[o_pos:o_cu] = np.arange(total) - np.repeat(starts[:-1], lens)
            packed[o_cu:o_sel] = starts
            within = np.arange(n_sel) - np.repeat(c_starts, lc_)
            # rows that predict completion tokens: positions p-1 .. p+c-2 of every sequence
            packed[o_sel:o_row] = np.repeat(starts[:-1] + lp_ - 1, lc_) + within
            packed[o_row:o_col] = np.repeat(np.arange(s, s + k), lc_)
            packed[o_col:] = within
            host = torch.from_numpy(packed)
            if dev.type == "cuda":
                host = host.pin_memory()
            buf = host.to(dev, non_blocking=True)
            flat, sel_t, r, c_ = buf[:total], buf[o_sel:o_row], buf[o_row:o_col], buf[o_col:]
            ctx = SeqCtx(buf[o_pos:o_cu].to(torch.int32), buf[o_cu:o_sel].to(torch.int32), int(lens.max()))
            fwd_kw = {}
            if pixel_values_list is not None and getattr(model, "is_vlm", False):
                fwd_kw = merge_vision_entries(pixel_values_list[s:s + bs], dev)
            hidden = model.forward_hidden(flat, ctx, **fwd_kw)
            tgt = flat[sel_t + 1]
            lp, en = ops.lm_head_logprobs(hidden[sel_t], model.lm_head_weight, tgt, temperature,
                                          softcap=model.config.final_logit_softcapping, compute_entropy=compute_entropy,
                                          entropy_grad=entropy_grad and compute_entropy)
            if getattr(self, "_keep_selected_hidden", False):  # value heads read the same rows (PPO)
                self._selected_hidden = (hidden[sel_t], r, c_, flat, ctx, sel_t)
            logps = logps.index_put((r, c_), lp)
            if compute_entropy:
                ents = ents.index_put((r, c_), en)
            if model.config.is_moe and torch.is_grad_enabled():
                a = model.aux_loss(ctx)
                aux_total = a if aux_total is None else aux_total + a
        self._last_aux_loss = aux_total
        return logps, ents

    def _ref_logps(self, prompt_ids, completion_ids, batch_size, pixel_values_list=None):
        kw = {"pixel_values_list": pixel_values_list}
        if (self.ref_model is not None and getattr(self, "_ref_stream", None) is None
                and getattr(getattr(self, "engine", None), "mode", "") == "full_shard_stream"):
            # the policy is trained on streamed slices because the whole model is too large to keep around: the frozen
            # reference gets the same treatment (one slice per layer and rank, layers gathered as the forward reaches them)
            from ..parallel.streamshard import StreamShardEngine

            if getattr(self.args, "sync_ref_model", False):
                raise NotImplementedError("sync_ref_model copies whole parameters; it is not available with "
                                          "shard_mode='full_shard_stream'")
            self._ref_stream = StreamShardEngine(self.ref_model, frozen=True, device=self.args.device,
                                                    init_seed=self.args.seed)
        with torch.no_grad():
            if self.ref_model is not None:
                return self._get_per_token_logps_and_entropies(self.ref_model, prompt_ids, completion_ids, batch_size,
                                                               **kw)[0]
            with use_adapter(self.model, None):
                return self._get_per_token_logps_and_entropies(self.model, prompt_ids, completion_ids, batch_size, **kw)[0]

    # ---- logging --------------------------------------------------------------------------------------------------------
    def log(self, logs: dict, start_time: float | None = None):
        mode = "train" if self.model.training else "eval"
        m = self._metrics[mode]
        resolve_deferred_metrics(m)
        for k in list(m.keys()):
            vals = [float(v) for v in m[k]]
            vals = [v for v in vals if v == v]  # drop NaN
            if vals:
                m[k] = vals
            else:
                del m[k]
        super().log(logs, start_time)
        if self.log_completions and D.is_main() and self._logs["prompt"]:
            print_prompt_completions_sample(list(self._logs["prompt"]), list(self._logs["completion"]),
                                            {k: list(v) for k, v in self._logs["rewards"].items()},
                                            list(self._logs["advantages"]), self.state.global_step,
                                            self.num_completions_to_print,
                                            {k: list(v) for k, v in self._logs["extra"].items()})
            try:
                import pandas as pd

                d = os.path.join(self.args.output_dir, "completions")
                os.makedirs(d, exist_ok=True)
                table = {"step": [self.state.global_step] * len(self._logs["prompt"]),
                         "prompt": [str(p) for p in self._logs["prompt"]],
                         "completion": [str(c) for c in self._logs["completion"]],
                         **{k: list(v) for k, v in self._logs["rewards"].items()},
                         "advantage": list(self._logs["advantages"])}
                df = pd.DataFrame(table)
                if getattr(self.args, "log_unique_prompts", False):  # one row per prompt: the first completion seen
                    df = df.drop_duplicates(subset=["prompt"])
                df.to_parquet(os.path.join(d, f"completions_{self.state.global_step:05d}.parquet"))
            except Exception:
                pass
            for v in (self._logs["prompt"], self._logs["completion"], self._logs["advantages"]):
                v.clear()
            self._logs["rewards"].clear()
            self._logs["extra"].clear()
