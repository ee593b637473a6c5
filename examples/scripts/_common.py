"""Shared by the example scripts: JSON-lines loading and the offline smoke set-up (tiny random model, word-level
tokenizer, synthetic rows), so that every example can be run end to end without checkpoints or datasets:

    python examples/scripts/<name>.py --smoke
"""
import argparse
import json


def parser(doc: str, out: str) -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=doc, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default=None, help="local checkpoint directory")
    ap.add_argument("--data", default=None, help="JSON-lines file")
    ap.add_argument("--out", default=out)
    ap.add_argument("--smoke", action="store_true", help="tiny random model + synthetic data on CPU, 2 steps")
    return ap


def load_rows(path: str) -> list[dict]:
    return [json.loads(line) for line in open(path)]


def smoke(kind: str, n: int = 16):
    """(model, tokenizer, rows, config overrides) for a CPU smoke run on one of the dataset formats."""
    from trl_b200.testing import make_dataset, make_tiny_model, make_tiny_tokenizer

    over = dict(use_cpu=True, bf16=False, max_steps=2, logging_steps=1, save_strategy="no", report_to="none",
                per_device_train_batch_size=4, gradient_accumulation_steps=1, learning_rate=1e-3)
    return make_tiny_model("tiny-qwen2"), make_tiny_tokenizer(), make_dataset(kind, n), over


def pick(a, kind: str, **defaults):
    """Model, tokenizer (None = loaded from the checkpoint by the trainer), rows and config keywords for either mode."""
    if a.smoke:
        model, tok, rows, over = smoke(kind)
        return model, tok, rows, {**defaults, **over}
    if not a.model or not a.data:
        raise SystemExit("--model and --data are required (or pass --smoke)")
    return a.model, None, load_rows(a.data), defaults
