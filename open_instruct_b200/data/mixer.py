"""Dataset mixing, transform chains and the tokenised-dataset cache.

Contract of the reference (``open_instruct/dataset_transformation.py:1861-2455``):

* mix grammar ``[name, amount, name, amount, ...]``: an amount containing ``.`` is a fraction of the
  dataset (``"1.0"`` = all of it, ``"2.5"`` = two full copies plus a seeded random half), one without is
  an absolute number of samples; names may be local ``.jsonl`` / ``.parquet`` files or hub datasets;
  either one split for all datasets or one split per dataset;
* every dataset runs through its transform chain (``TRANSFORM_FNS`` names, each with its own kwargs)
  with deterministic fingerprints, then the mix is concatenated and gets an ``index`` column;
* the result is cached on local disk under a key that hashes dataset configs, tokenizer config and
  chat template, together with per-dataset statistics.
"""

from __future__ import annotations

import hashlib
import json
import logging
import multiprocessing
import os
from dataclasses import asdict, dataclass, field
from typing import Any

import numpy as np

from .tokenize import (
    DATASET_ORIGIN_KEY,
    ENV_CONFIG_KEY,
    SFT_TOKENIZE_FNS,
    TOOLS_COLUMN_KEY,
    TRANSFORM_FNS,
    TokenizerConfig,
)

logger = logging.getLogger(__name__)

DATASET_CACHE_VERSION = "b200-v1"
# planning constants used to decide how many worker processes a map/filter deserves
APPLY_CHAT_TEMPLATE_EXAMPLE_PER_SECOND_PER_CPU = 400
FILTER_EXAMPLE_PER_SECOND_PER_CPU = 1130


def max_num_processes() -> int:
    return int(float(os.environ.get("BEAKER_ASSIGNED_CPU_COUNT", multiprocessing.cpu_count())))


def get_num_proc(dataset_len: int, num_available_cpus: int, example_per_second_per_cpu: int) -> int:
    """Enough workers to finish in about a second each, never more than the CPUs we have."""
    return max(1, min(num_available_cpus, dataset_len // max(1, example_per_second_per_cpu)))


def _load_any(name: str, split: str, revision: str | None):
    from datasets import Dataset, load_dataset

    if os.path.exists(name) and name.endswith((".jsonl", ".json")):
        if split != "train":
            raise ValueError("Only train split is supported for local jsonl files.")
        ds = load_dataset("json", data_files=name, split="train")
    elif os.path.exists(name) and name.endswith(".parquet"):
        if split != "train":
            raise ValueError("Only train split is supported for local parquet files.")
        ds = load_dataset("parquet", data_files=name, split="train")
    elif os.path.isdir(name) and os.path.exists(os.path.join(name, "dataset_info.json")):
        from datasets import load_from_disk

        ds = load_from_disk(name)
    else:
        ds = load_dataset(name, split=split, revision=revision)
    if not isinstance(ds, Dataset):
        raise TypeError(f"expected a Dataset for {name}, got {type(ds)}")
    return ds


@dataclass
class DatasetConfig:
    dataset_name: str
    dataset_split: str = "train"
    dataset_revision: str = "main"
    dataset_range: int | None = None
    transform_fn: list[str] = field(default_factory=list)
    transform_fn_args: list[dict[str, Any]] = field(default_factory=list)
    target_columns: list[str] | None = None
    dataset_config_seed: int = 42
    dataset_commit_hash: str | None = None
    frac_or_num_samples: int | float | None = None
    original_dataset_size: int | None = None
    is_upsampled: bool = False
    dataset: Any = field(init=False, default=None, repr=False, compare=False)

    def __post_init__(self):
        self.dataset = _load_any(self.dataset_name, self.dataset_split, self.dataset_revision)
        if self.dataset_range is None:
            self.update_range(len(self.dataset))

    def update_range(self, dataset_range: int) -> None:
        self.dataset_range = dataset_range
        self.original_dataset_size = len(self.dataset)
        self.dataset = self.select_samples(dataset_range)
        self.is_upsampled = dataset_range > self.original_dataset_size

    def select_samples(self, target_size: int):
        """First ``target_size`` rows; beyond the dataset size: whole copies plus a seeded random remainder."""
        n = len(self.dataset)
        reps, extra = divmod(target_size, n)
        idx = list(range(n)) * reps
        if extra:
            if reps == 0:
                idx = list(range(extra))
            else:
                rng = np.random.RandomState(self.dataset_config_seed)
                idx += rng.choice(n, size=extra, replace=False).tolist()
        return self.dataset.select(idx)


def _template_hash(tokenizer) -> str:
    tpl = getattr(tokenizer, "chat_template", None)
    try:
        s = json.dumps(tpl, sort_keys=True)
    except TypeError:
        s = str(tpl)
    return hashlib.sha256(s.encode()).hexdigest()


def _keep(col: str, dataset, cols: list[str]) -> list[str]:
    return cols + [col] if col in dataset.column_names and col not in cols else cols


def get_dataset_v1(dc: DatasetConfig, tc: TokenizerConfig):
    """Run one dataset through its transform chain."""
    if len(dc.transform_fn) != len(dc.transform_fn_args):
        raise ValueError(f"transform_fn and transform_fn_args must have the same length: {dc.transform_fn} vs {dc.transform_fn_args}")
    cpus = max_num_processes()
    tokenizer = tc.tokenizer
    ds = dc.dataset
    name = dc.dataset_name
    ds = ds.map(lambda ex: {**ex, DATASET_ORIGIN_KEY: name}, desc=f"tagging source {name}")
    tc_json = json.dumps({k: v for k, v in asdict(tc).items() if v is not None}, sort_keys=True)
    tpl_hash = _template_hash(tokenizer)[:16]
    for fn_name, fn_args in zip(dc.transform_fn, dc.transform_fn_args):
        fn, kind = TRANSFORM_FNS[fn_name]
        kwargs = {"tokenizer": tokenizer, **fn_args}
        fp = hashlib.sha256(f"{DATASET_CACHE_VERSION}:{fn_name}:{ds._fingerprint}:{json.dumps(fn_args, sort_keys=True)}:"
                            f"{tc_json}:{tpl_hash}".encode()).hexdigest()[:16]
        cols = ds.column_names if dc.target_columns is None else list(dc.target_columns)
        cols = _keep(DATASET_ORIGIN_KEY, ds, cols)
        if fn_name in SFT_TOKENIZE_FNS:
            cols = [c for c in cols if c != TOOLS_COLUMN_KEY]  # consumed by the template, never persisted
        else:
            cols = _keep(TOOLS_COLUMN_KEY, ds, cols)
        cols = _keep(ENV_CONFIG_KEY, ds, cols)
        if kind == "map":
            nproc = get_num_proc(len(ds), cpus, APPLY_CHAT_TEMPLATE_EXAMPLE_PER_SECOND_PER_CPU)
            ds = ds.map(fn, fn_kwargs=kwargs, remove_columns=[c for c in ds.column_names if c not in cols],
                        num_proc=nproc if nproc > 1 else None, new_fingerprint=fp)
        elif kind == "filter":
            nproc = get_num_proc(len(ds), cpus, FILTER_EXAMPLE_PER_SECOND_PER_CPU)
            ds = ds.filter(fn, fn_kwargs=kwargs, num_proc=nproc if nproc > 1 else None, new_fingerprint=fp)
        else:
            raise ValueError(f"Unknown transform function type: {kind}")
    if len(ds) == 0:
        raise ValueError("No examples left after transformation")
    return ds


def _dc_dict(dc: DatasetConfig, drop_none: bool) -> dict:
    d = asdict(dc)
    d.pop("dataset", None)
    return {k: v for k, v in d.items() if v is not None} if drop_none else d


def compute_config_hash(dcs: list[DatasetConfig], tc: TokenizerConfig) -> str:
    blob = {
        "cache_version": DATASET_CACHE_VERSION,
        "dataset_configs": [_dc_dict(dc, True) for dc in dcs],
        "tokenizer_config": {k: v for k, v in asdict(tc).items() if v is not None},
        "chat_template_hash": _template_hash(tc.tokenizer),
    }
    return hashlib.sha256(json.dumps(blob, sort_keys=True).encode()).hexdigest()[:10]


def load_dataset_configs(dataset_mixer_list: list[str], dataset_mixer_list_splits: list[str],
                         dataset_transform_fn: list[str], transform_fn_args: list[dict[str, Any]],
                         target_columns: list[str] | None = None, dataset_config_seed: int = 42) -> list[DatasetConfig]:
    if len(dataset_mixer_list) % 2:
        raise ValueError(f"Data mixer list length is not even: {dataset_mixer_list}")
    n = len(dataset_mixer_list) // 2
    splits = list(dataset_mixer_list_splits)
    if len(splits) == 1:
        splits = splits * n
    if len(splits) != n:
        raise ValueError(f"dataset_mixer_list_splits length must be 1 or {n}: {dataset_mixer_list_splits}")
    dcs = []
    for i in range(n):
        name, amount = dataset_mixer_list[2 * i], str(dataset_mixer_list[2 * i + 1])
        frac_or_num = float(amount) if "." in amount else int(amount)
        dc = DatasetConfig(dataset_name=name, dataset_split=splits[i], transform_fn=list(dataset_transform_fn),
                           transform_fn_args=[dict(a) for a in transform_fn_args], target_columns=target_columns,
                           frac_or_num_samples=frac_or_num, dataset_config_seed=dataset_config_seed)
        size = len(dc.dataset)
        new_range = int(frac_or_num * size) if isinstance(frac_or_num, float) else int(frac_or_num)
        if new_range <= 0:
            raise ValueError(f"dataset {name}: requested {amount} -> {new_range} samples")
        dc.update_range(new_range)
        dcs.append(dc)
    return dcs


def _statistics(dcs: list[DatasetConfig], transformed: list) -> dict:
    per = []
    for dc, ds in zip(dcs, transformed):
        row = {"dataset_name": dc.dataset_name, "dataset_split": dc.dataset_split, "initial_instances": dc.dataset_range,
               "final_instances": len(ds), "instances_filtered": (dc.dataset_range or 0) - len(ds),
               "frac_or_num_samples": dc.frac_or_num_samples, "original_dataset_size": dc.original_dataset_size,
               "is_upsampled": dc.is_upsampled, "upsampling_factor": (dc.dataset_range or 0) / max(1, dc.original_dataset_size or 1)}
        for key in ("input_ids", "chosen_input_ids", "input_ids_prompt"):
            if key in ds.column_names:
                lens = [len(x) for x in ds[key]]
                row.update(total_tokens=int(sum(lens)), avg_tokens_per_instance=float(np.mean(lens)), max_tokens=int(max(lens)))
                break
        if "labels" in ds.column_names:
            row["trainable_tokens"] = int(sum(sum(1 for t in lab if t != -100) for lab in ds["labels"]))
        per.append(row)
    return {"per_dataset_stats": per, "dataset_order": [dc.dataset_name for dc in dcs]}


class LocalDatasetTransformationCache:
    """Disk cache keyed by ``compute_config_hash``: ``<dir>/<hash>/`` holds the dataset and its statistics."""

    def __init__(self, config_hash: str | None = None, dataset_local_cache_dir: str = "local_dataset_cache"):
        self.config_hash = config_hash
        self.root = dataset_local_cache_dir
        os.makedirs(self.root, exist_ok=True)

    def path(self, config_hash: str | None = None) -> str:
        return os.path.join(self.root, config_hash or self.config_hash)

    def load_or_transform_dataset(self, dcs: list[DatasetConfig], tc: TokenizerConfig, dataset_skip_cache: bool = False,
                                  return_statistics: bool = False):
        from datasets import concatenate_datasets, load_from_disk

        h = self.config_hash or compute_config_hash(dcs, tc)
        path = self.path(h)
        stats_path = os.path.join(path, "dataset_statistics.json")
        if os.path.exists(path) and os.path.exists(os.path.join(path, "dataset_info.json")) and not dataset_skip_cache:
            logger.info("found cached dataset at %s", path)
            ds = load_from_disk(path, keep_in_memory=True)
            stats = json.load(open(stats_path)) if os.path.exists(stats_path) else {}
            return (ds, stats) if return_statistics else ds
        transformed = [get_dataset_v1(dc, tc) for dc in dcs]
        stats = _statistics(dcs, transformed)
        ds = concatenate_datasets(transformed)
        if dataset_skip_cache:
            return (ds, stats) if return_statistics else ds
        ds.save_to_disk(path)
        with open(os.path.join(path, "config.json"), "w") as fh:
            json.dump({"tokenizer_config": asdict(tc), "dataset_configs": [_dc_dict(dc, False) for dc in dcs],
                       "config_hash": h}, fh, indent=2, default=str)
        with open(stats_path, "w") as fh:
            json.dump(stats, fh, indent=2)
        ds = load_from_disk(path, keep_in_memory=True)
        return (ds, stats) if return_statistics else ds


def get_cached_dataset_tulu_with_statistics(dataset_mixer_list: list[str], dataset_mixer_list_splits: list[str],
                                            tc: TokenizerConfig, dataset_transform_fn: list[str],
                                            transform_fn_args: list[dict[str, Any]], target_columns: list[str] | None = None,
                                            dataset_cache_mode: str = "local", dataset_config_hash: str | None = None,
                                            hf_entity: str | None = None, dataset_local_cache_dir: str = "local_dataset_cache",
                                            dataset_skip_cache: bool = False, drop_dataset_source: bool = True,
                                            dataset_config_seed: int = 42, system_prompt_override: str | None = None):
    """Mixed, transformed, cached dataset with an ``index`` column, plus its statistics."""
    if dataset_cache_mode not in ("local", "hf"):
        raise ValueError("dataset_cache_mode must be 'local' or 'hf'")
    if dataset_cache_mode == "hf":
        logger.warning("hub-backed dataset cache needs network access; using the local cache directory instead")
    if system_prompt_override is not None:
        transform_fn_args = [dict(a) for a in transform_fn_args]
        for name, a in zip(dataset_transform_fn, transform_fn_args):
            if name == "rlvr_tokenize_v1":
                a["system_prompt_override"] = system_prompt_override
    dcs = []
    if dataset_config_hash is None:
        dcs = load_dataset_configs(dataset_mixer_list, dataset_mixer_list_splits, dataset_transform_fn, transform_fn_args,
                                   target_columns, dataset_config_seed)
        dataset_config_hash = compute_config_hash(dcs, tc)
    cache = LocalDatasetTransformationCache(dataset_config_hash, dataset_local_cache_dir)
    ds, stats = cache.load_or_transform_dataset(dcs, tc, dataset_skip_cache, return_statistics=True)
    if drop_dataset_source and DATASET_ORIGIN_KEY in ds.column_names:
        ds = ds.remove_columns([DATASET_ORIGIN_KEY])
    if "index" not in ds.column_names:
        ds = ds.add_column("index", list(range(len(ds))))
    return ds, stats


def get_cached_dataset_tulu(*args, **kwargs):
    return get_cached_dataset_tulu_with_statistics(*args, **kwargs)[0]
