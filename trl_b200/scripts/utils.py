"""Script plumbing: dataclass-driven argument parsing with YAML configs, dataset (mixture) loading.

Behaviour of trl/scripts/utils.py: ``ScriptArguments`` (:145-202), ``DatasetConfig`` /
``DatasetMixtureConfig`` / ``get_dataset`` (:39-142, :412-488), ``init_zero_verbose`` (:205-231) and
``TrlParser`` (:234-386): ``--config file.yaml`` values become argparse *defaults* (the command line
wins), an ``env:`` block is exported to ``os.environ``, unknown keys are returned as leftover
``--key value`` strings (launcher arguments) or rejected.
"""
from __future__ import annotations

import argparse
import dataclasses
import importlib
import json
import logging
import os
import sys
import types
import typing
import warnings
from dataclasses import dataclass, field
from typing import Any, Optional, Union


@dataclass
class DatasetConfig:
    path: str = ""
    name: Optional[str] = None
    data_dir: Optional[str] = None
    data_files: Optional[Any] = None
    split: str = "train"
    columns: Optional[list] = None


@dataclass
class DatasetMixtureConfig:
    datasets: list = field(default_factory=list, metadata={"help": "List of dataset configs (dicts) to mix."})
    streaming: bool = False
    test_split_size: Optional[float] = None

    def __post_init__(self):
        self.datasets = [DatasetConfig(**d) if isinstance(d, dict) else d for d in (self.datasets or [])]


@dataclass
class ScriptArguments:
    dataset_name: Optional[str] = field(default=None, metadata={"help": "Dataset path (local directory / file) or name."})
    dataset_config: Optional[str] = None
    dataset_train_split: str = "train"
    dataset_test_split: str = "test"
    dataset_streaming: bool = False
    ignore_bias_buffers: bool = False


def init_zero_verbose():
    """Route logging and warnings through rich at ERROR level (quiet scripts)."""
    fmt = "%(message)s"
    try:
        from rich.logging import RichHandler

        logging.basicConfig(format=fmt, datefmt="[%X]", handlers=[RichHandler()], level=logging.ERROR)
    except Exception:
        logging.basicConfig(format=fmt, level=logging.ERROR)

    def warning_handler(message, category, filename, lineno, file=None, line=None):
        logging.warning(f"{filename}:{lineno}: {category.__name__}: {message}")

    warnings.showwarning = warning_handler


def _load_local_dataset(path: str, name=None, split=None, streaming=False, data_files=None):
    """No network: ``path`` is a directory saved with ``save_to_disk``, a json/jsonl/csv/parquet file, a
    directory of such files, or ``synthetic:<kind>[:n]`` (fixtures of :mod:`trl_b200.testing`)."""
    import datasets as hfds

    if path.startswith("synthetic:"):
        from ..testing import make_dataset

        parts = path.split(":")
        ds = make_dataset(parts[1], int(parts[2]) if len(parts) > 2 else 64)
        return hfds.DatasetDict({"train": ds, "test": ds.select(range(min(8, len(ds))))})
    if os.path.isdir(path) and (os.path.exists(os.path.join(path, "dataset_dict.json"))
                                or os.path.exists(os.path.join(path, "state.json"))):
        ds = hfds.load_from_disk(path)
        return ds if isinstance(ds, hfds.DatasetDict) else hfds.DatasetDict({"train": ds})
    ext = {".json": "json", ".jsonl": "json", ".csv": "csv", ".parquet": "parquet", ".txt": "text"}
    if os.path.isfile(path):
        return hfds.load_dataset(ext[os.path.splitext(path)[1]], data_files=path, streaming=streaming)
    if os.path.isdir(path):
        return hfds.load_dataset(path, name=name, data_files=data_files, streaming=streaming)
    raise FileNotFoundError(f"dataset {path!r} is not a local path; Hub datasets need network access")


def get_dataset(mixture_config: DatasetMixtureConfig):
    """Concatenate the configured datasets (optionally keeping only some columns) into a DatasetDict."""
    import datasets as hfds

    parts = []
    for c in mixture_config.datasets:
        dd = _load_local_dataset(c.path, c.name, c.split, mixture_config.streaming, c.data_files)
        ds = dd[c.split] if isinstance(dd, (dict, hfds.DatasetDict)) else dd
        if c.columns:
            ds = ds.select_columns(c.columns)
        parts.append(ds)
    if not parts:
        raise ValueError("No datasets were loaded from the mixture configuration")
    combined = hfds.concatenate_datasets(parts) if len(parts) > 1 else parts[0]
    if mixture_config.test_split_size is not None:
        return combined.train_test_split(test_size=mixture_config.test_split_size)
    return hfds.DatasetDict({"train": combined})


def load_script_dataset(script_args: ScriptArguments, dataset_args: DatasetMixtureConfig | None = None):
    if dataset_args is not None and dataset_args.datasets:
        if script_args.dataset_name:
            warnings.warn("Both `datasets` and `dataset_name` are provided; `datasets` takes precedence.")
        return get_dataset(dataset_args)
    if not script_args.dataset_name:
        raise ValueError("Either `datasets` or `dataset_name` must be provided.")
    return _load_local_dataset(script_args.dataset_name, script_args.dataset_config, streaming=script_args.dataset_streaming)


# ---------------------------------------------------------------------------------------------------
# dataclass -> argparse
# ---------------------------------------------------------------------------------------------------
def load_processing_class(path, **tokenizer_kwargs):
    """Tokenizer for a text checkpoint directory; for a vision-language checkpoint (``model_type: llava`` or
    ``qwen2_vl``) a processor: the framework's ``VisionProcessor`` / ``DynamicResolutionProcessor`` when one was saved
    next to the model, else ``transformers.AutoProcessor``.
    Presets (no files on disk) get the offline ChatML fixture tokenizer."""
    import json
    import os

    path = str(path)
    if not os.path.isdir(path):
        from ..testing import make_tiny_tokenizer

        return make_tiny_tokenizer()
    from transformers import AutoTokenizer

    cfg = os.path.join(path, "config.json")
    is_vlm = False
    if os.path.exists(cfg):
        with open(cfg) as f:
            is_vlm = json.load(f).get("model_type") in ("llava", "qwen2_vl")
    if is_vlm:
        pre = os.path.join(path, "preprocessor_config.json")
        if os.path.exists(pre):
            with open(pre) as f:
                kind = json.load(f).get("processor_class")
            if kind in ("VisionProcessor", "DynamicResolutionProcessor"):
                from ..models import vision_processing

                return getattr(vision_processing, kind).from_pretrained(path)
        from transformers import AutoProcessor

        return AutoProcessor.from_pretrained(path)
    return AutoTokenizer.from_pretrained(path, **tokenizer_kwargs)


def _str2bool(v):
    if isinstance(v, bool):
        return v
    s = str(v).lower()
    if s in ("yes", "true", "t", "y", "1"):
        return True
    if s in ("no", "false", "f", "n", "0"):
        return False
    raise argparse.ArgumentTypeError(f"Truthy value expected, got {v!r}")


def _json_or_str(v):
    if isinstance(v, str) and v.strip()[:1] in "[{":
        try:
            return json.loads(v)
        except json.JSONDecodeError:
            return v
    return v


def _unwrap(tp):
    origin = typing.get_origin(tp)
    if origin in (Union, types.UnionType):
        args = [a for a in typing.get_args(tp) if a is not type(None)]
        return _unwrap(args[0]) if args else (str, None)
    if origin in (list, typing.List):
        args = typing.get_args(tp)
        return (list, args[0] if args else str)
    if tp in (list,):
        return (list, str)
    return (tp, None)


class TrlParser(argparse.ArgumentParser):
    def __init__(self, dataclass_types=None, **kwargs):
        kwargs.setdefault("formatter_class", argparse.ArgumentDefaultsHelpFormatter)
        super().__init__(**kwargs)
        if dataclass_types is None:
            dataclass_types = []
        elif dataclasses.is_dataclass(dataclass_types):
            dataclass_types = [dataclass_types]
        self.dataclass_types = list(dataclass_types)
        for dt in self.dataclass_types:
            if "config" in {f.name for f in dataclasses.fields(dt)}:
                raise ValueError(f"Dataclass {dt.__name__} has a field named 'config'. This field is reserved for the "
                                 "config file path and should not be used in the dataclass.")
            self._add_dataclass(dt)

    def _add_dataclass(self, dt):
        hints = typing.get_type_hints(dt)
        seen = {a.dest for a in self._actions}
        for f in dataclasses.fields(dt):
            if not f.init or f.name in seen or f.name.startswith("_"):
                continue
            tp, elem = _unwrap(hints.get(f.name, str))
            kw: dict[str, Any] = {"help": (f.metadata or {}).get("help")}
            default = f.default if f.default is not dataclasses.MISSING else (
                f.default_factory() if f.default_factory is not dataclasses.MISSING else None)
            kw["default"] = default
            if tp is bool:
                kw.update(type=_str2bool, nargs="?", const=True)
            elif tp is list:
                kw.update(nargs="+", type=elem if elem in (int, float, str) else _json_or_str)
            elif tp in (int, float, str):
                kw["type"] = tp
            else:
                kw["type"] = _json_or_str
            self.add_argument(f"--{f.name}", **kw)
            if tp is bool and default is True:
                self.add_argument(f"--no_{f.name}", dest=f.name, action="store_false", help=argparse.SUPPRESS)

    def parse_args_into_dataclasses(self, args=None, return_remaining_strings=False):
        ns, remaining = self.parse_known_args(args)
        outs = []
        for dt in self.dataclass_types:
            names = {f.name for f in dataclasses.fields(dt) if f.init}
            kw = {k: v for k, v in vars(ns).items() if k in names}
            for k, v in list(kw.items()):
                if isinstance(v, list) and len(v) == 1 and isinstance(v[0], (list, dict)):
                    kw[k] = v[0]
            outs.append(dt(**kw))
        if return_remaining_strings:
            return (*outs, remaining)
        if remaining:
            raise ValueError(f"Some specified arguments are not used by the TrlParser: {remaining}")
        return tuple(outs)

    def parse_args_and_config(self, args=None, return_remaining_strings=False, fail_with_unknown_args=True,
                              separate_remaining_strings=False):
        args = list(args) if args is not None else sys.argv[1:]
        config_remaining: list[str] = []
        if "--config" in args:
            import yaml

            i = args.index("--config")
            path = args[i + 1]
            del args[i:i + 2]
            with open(path) as f:
                cfg = yaml.safe_load(f) or {}
            env = cfg.pop("env", {})
            if not isinstance(env, dict):
                raise ValueError("`env` field should be a dict in the YAML file.")
            for k, v in env.items():
                os.environ[k] = str(v)
            config_remaining = self.set_defaults_with_config(**cfg)
        out = self.parse_args_into_dataclasses(args, return_remaining_strings=return_remaining_strings)
        if return_remaining_strings:
            *dcs, rem = out
            if separate_remaining_strings:
                return (*dcs, rem, config_remaining)
            return (*dcs, config_remaining + rem)
        if config_remaining and fail_with_unknown_args:
            raise ValueError(f"Unknown keys in the config file: {config_remaining}")
        return out

    def set_defaults_with_config(self, **kwargs) -> list[str]:
        known = {a.dest: a for a in self._actions}
        leftover = []
        for k, v in kwargs.items():
            if k in known:
                known[k].default = v
                known[k].required = False
            else:
                leftover += [f"--{k}", str(v)]
        return leftover


def get_git_commit_hash(package_name: str):
    try:
        mod = importlib.import_module(package_name)
        root = os.path.dirname(os.path.dirname(mod.__file__))
        import subprocess

        return subprocess.check_output(["git", "-C", root, "rev-parse", "HEAD"], stderr=subprocess.DEVNULL).decode().strip()
    except Exception:
        return None
