"""Every example script runs end to end in its offline smoke mode; the tiny-model generator writes loadable checkpoints."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPTS = os.path.join(ROOT, "examples", "scripts")


def _run(args, tmp_path, timeout=600):
    env = dict(os.environ, PYTHONPATH=ROOT, TRL_EXPERIMENTAL_SILENCE="1", OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable] + args, env=env, cwd=SCRIPTS, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    return r.stdout


EXAMPLES = ["kto", "reward_modeling", "rloo", "sft_lora", "gkd", "dpo_vlm", "grpo_vlm", "cpo_simpo", "orpo", "prm", "ppo", "bco",
            "xpo_nash_md", "gold_distillation", "sft_expert_parallel", "online_dpo"]

_RUNNER = """
import runpy, sys, os
names, out = sys.argv[1].split(","), sys.argv[2]
for n in names:
    print("EXAMPLE", n, flush=True)
    sys.argv = [n + ".py", "--smoke", "--out", os.path.join(out, n)]
    runpy.run_path(n + ".py", run_name="__main__")
    print("EXAMPLE_DONE", n, flush=True)
"""


def test_examples_smoke(tmp_path):
    """All example scripts in their offline smoke mode, one after the other in ONE interpreter (start-up dominates)."""
    out = _run(["-c", _RUNNER, ",".join(EXAMPLES), str(tmp_path)], tmp_path, timeout=900)
    for name in EXAMPLES:
        assert f"EXAMPLE_DONE {name}" in out, (name, out[-1500:])
        saved = os.listdir(tmp_path / name)
        assert any(f.endswith(".safetensors") for f in saved), (name, saved)
    assert out.count("train_runtime") >= len(EXAMPLES)


def test_sft_vlm_example_smoke(tmp_path):
    out = _run(["sft_vlm.py", "--steps", "2", "--out", str(tmp_path / "v")], tmp_path)
    assert "train_runtime" in out and os.path.exists(tmp_path / "v" / "preprocessor_config.json")
    out = _run(["sft_vlm.py", "--steps", "2", "--family", "qwen2_vl", "--out", str(tmp_path / "q")], tmp_path)
    assert "train_runtime" in out
    import json

    assert json.load(open(tmp_path / "q" / "config.json"))["model_type"] == "qwen2_vl"
    assert json.load(open(tmp_path / "q" / "preprocessor_config.json"))["processor_class"] == "DynamicResolutionProcessor"


def test_generate_tiny_models_are_loadable(tmp_path):
    _run(["generate_tiny_models.py", "--out", str(tmp_path), "--families", "tiny-qwen2", "tiny-qwen3-moe",
          "--reward-heads"], tmp_path)
    import transformers as tf

    from trl_b200.models.hf_io import load_model
    from trl_b200.scripts.utils import load_processing_class

    m = load_model(str(tmp_path / "tiny-qwen2"))
    hf = tf.AutoModelForCausalLM.from_pretrained(str(tmp_path / "tiny-qwen2"))
    assert sum(p.numel() for p in hf.parameters()) == sum(p.numel() for p in m.parameters())
    assert load_model(str(tmp_path / "tiny-qwen2-reward")).config.num_labels == 1
    assert load_model(str(tmp_path / "tiny-qwen3-moe")).config.is_moe
    vlm = load_model(str(tmp_path / "tiny-llava"))
    proc = load_processing_class(str(tmp_path / "tiny-llava"))
    assert vlm.config.image_token_index == proc.image_token_id
