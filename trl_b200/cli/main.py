"""``trl`` command line (console entry ``trl_b200.cli:main``).

Sub-commands ``dpo, env, grpo, kto, reward, rloo, sft, skills, vllm-serve`` like trl/cli/main.py:22-51.
Training commands take the script's own arguments plus launcher arguments: ``--num_processes N`` and
``--accelerate_config <profile|path.yaml>`` (profiles: single_gpu, multi_gpu, zero1, zero2, zero3, fsdp1, fsdp2).
The reference forwards unknown arguments to ``accelerate launch`` (trl/cli/commands/training.py:34-72); here the
launcher is ``torch.distributed.run`` with one process per GPU and the profile selects the engine's shard mode.
"""
from __future__ import annotations

import argparse
import importlib
import os
import subprocess
import sys

TRAINING = ("dpo", "grpo", "kto", "reward", "rloo", "sft")
PROFILE_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "accelerate_configs")


def resolve_profile(name_or_path: str) -> dict:
    """A packaged profile name or a YAML path -> {"num_processes": int, "shard_mode": str, ...}."""
    import yaml

    path = name_or_path
    if not os.path.isfile(path):
        cand = os.path.join(PROFILE_DIR, f"{name_or_path}.yaml")
        if not os.path.isfile(cand):
            names = sorted(f[:-5] for f in os.listdir(PROFILE_DIR) if f.endswith(".yaml"))
            raise ValueError(f"Accelerate config {name_or_path!r} is neither a file nor a predefined config ({names})")
        path = cand
    with open(path) as f:
        cfg = yaml.safe_load(f) or {}
    if "shard_mode" not in cfg:  # a genuine accelerate YAML: map its distributed_type onto an engine mode
        dt = str(cfg.get("distributed_type", "")).upper()
        ds = cfg.get("deepspeed_config", {}) or {}
        if dt == "DEEPSPEED":
            cfg["shard_mode"] = {1: "zero1", 2: "zero2", 3: "full_shard"}.get(int(ds.get("zero_stage", 2)), "zero2")
        elif dt == "FSDP":
            cfg["shard_mode"] = "full_shard"
        else:
            cfg["shard_mode"] = "ddp"
    # sequence sharding: our own keys (sp_size / cp_size) or accelerate's parallelism_config_* keys
    pc = dict(cfg.get("parallelism_config") or {})
    for ours, theirs in (("sp_size", "parallelism_config_sp_size"), ("cp_size", "parallelism_config_cp_size")):
        v = cfg.get(ours, cfg.get(theirs))
        if v is not None and int(v) > 1:
            pc[ours] = int(v)
    if pc:
        cfg["parallelism_config"] = pc
    return cfg


def _pop_launcher_args(argv: list[str]) -> tuple[list[str], dict]:
    out, launch = [], {}
    i = 0
    while i < len(argv):
        a = argv[i]
        if a in ("--num_processes", "--accelerate_config", "--main_process_port", "--mixed_precision"):
            launch[a[2:]] = argv[i + 1]
            i += 2
        elif a.startswith(("--num_processes=", "--accelerate_config=", "--main_process_port=")):
            k, v = a[2:].split("=", 1)
            launch[k] = v
            i += 1
        else:
            out.append(a)
            i += 1
    return out, launch


def run_training(name: str, argv: list[str]) -> int:
    script_argv, launch = _pop_launcher_args(argv)
    mod = importlib.import_module(f"trl_b200.scripts.{name}")
    parser = mod.make_parser()
    # validate early (also surfaces --help); unknown keys of a YAML config are launcher arguments
    *parsed, remaining, cfg_remaining = parser.parse_args_and_config(script_argv, return_remaining_strings=True,
                                                                     separate_remaining_strings=True)
    extra, launch2 = _pop_launcher_args(cfg_remaining)
    launch = {**launch2, **launch}
    if remaining or extra:
        raise SystemExit(f"trl {name}: unknown arguments {remaining + extra} (launcher arguments are "
                         "--num_processes and --accelerate_config)")
    prof = resolve_profile(launch["accelerate_config"]) if "accelerate_config" in launch else {}
    nproc = int(launch.get("num_processes", prof.get("num_processes", 1) if "accelerate_config" in launch else 1))
    import torch

    if torch.cuda.is_available():
        nproc = min(nproc, torch.cuda.device_count())
    if "shard_mode" in prof and "--shard_mode" not in script_argv:
        script_argv += ["--shard_mode", prof["shard_mode"]]
    if prof.get("parallelism_config") and "--parallelism_config" not in script_argv:
        import json

        script_argv += ["--parallelism_config", json.dumps(prof["parallelism_config"])]
    if nproc <= 1:
        script_args, training_args, model_args, dataset_args = parser.parse_args_and_config(script_argv)[:4]
        mod.main(script_args, training_args, model_args, dataset_args)
        return 0
    port = launch.get("main_process_port", "29500")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), mod.__file__] + script_argv
    return subprocess.call(cmd)


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    ap = argparse.ArgumentParser(prog="trl", description="B200-native post-training CLI")
    ap.add_argument("command", choices=list(TRAINING) + ["env", "skills", "vllm-serve", "rollout-serve"])
    if not argv or argv[0] in ("-h", "--help"):
        ap.print_help()
        return 0
    from .commands import CommandContext, EnvCommand, SkillsCommand, TrainingCommand, VllmServeCommand

    cmd = argv[0]
    commands = {n: TrainingCommand(n) for n in TRAINING}
    commands.update({"env": EnvCommand(), "skills": SkillsCommand(), "vllm-serve": VllmServeCommand()})
    serve = VllmServeCommand()
    serve.name = "rollout-serve"
    commands["rollout-serve"] = serve
    if cmd not in commands:
        ap.parse_args([cmd])
        return 2
    return commands[cmd].run(None, CommandContext(argv))


if __name__ == "__main__":
    sys.exit(main())
