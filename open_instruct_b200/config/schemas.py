"""Config dataclasses shared by the DPO / GRPO / reward-model entry points.

Field names and defaults follow the reference's shared config blocks
(``open_instruct/olmo_core_utils.py:40-241``), from which its ``DPOExperimentConfig`` and
``GRPOExperimentConfig`` inherit (``dpo_utils.py:198-210``, ``grpo_utils.py:74-80``).  Everything has a
default so that the blocks compose through multiple inheritance.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Literal


@dataclass
class ExperimentConfig:
    exp_name: str = "experiment"
    run_name: str | None = None
    seed: int = 42
    data_loader_seed: int | None = None


@dataclass
class ModelConfig:
    model_name_or_path: str | None = None
    config_name: str | None = None
    attn_implementation: str | None = field(default=None, metadata={"help": "Accepted for recipe compatibility; attention is this package's varlen kernel"})
    loss_implementation: str = "default"
    model_revision: str | None = None
    low_cpu_mem_usage: bool = False
    rope_scaling_factor: float | None = None
    rope_scaling_beta_fast: float = 32
    rope_scaling_beta_slow: float = 1
    rope_scaling_old_context_len: int = 8192
    dtype: str = "bfloat16"
    gradient_checkpointing: bool = False
    use_cache: bool | None = None
    use_peft: bool = False
    lora_r: int = 16
    lora_alpha: int = 32
    lora_dropout: float = 0.05
    lora_target_modules: list[str] | None = None
    lora_modules_to_save: list[str] | None = None
    lora_task_type: str = "CAUSAL_LM"
    # quantised base weights (bitsandbytes in the reference, ``open_instruct/model_utils.py:209-216``): accepted on the
    # command line so that recipes parse, refused at start-up when switched on - this framework trains bf16 + fp32 master
    load_in_8bit: bool = False
    load_in_4bit: bool = False
    bnb_4bit_quant_type: str | None = "nf4"
    use_bnb_nested_quant: bool = False

    def __post_init__(self):
        check_model_config(self)


def spec_with_rope_flags(spec, cfg):
    """``--rope_scaling_factor`` (with ``--rope_scaling_beta_fast / _beta_slow / _old_context_len``): train the model with its
    context extended by YaRN, as the reference's olmo-core path does (``open_instruct/olmo_core_utils.py:448-456``).  Returns the
    spec with that scaling rule (and a ``max_position_embeddings`` that covers the extended context); unchanged without the flag."""
    factor = getattr(cfg, "rope_scaling_factor", None)
    if factor is None:
        return spec
    old = int(getattr(cfg, "rope_scaling_old_context_len", 8192))
    rule = {"rope_type": "yarn", "factor": float(factor), "beta_fast": float(getattr(cfg, "rope_scaling_beta_fast", 32)),
            "beta_slow": float(getattr(cfg, "rope_scaling_beta_slow", 1)), "original_max_position_embeddings": old}
    return spec.replace(rope_scaling=rule, max_position_embeddings=max(spec.max_position_embeddings, int(old * factor)))


def check_model_config(cfg) -> None:
    """Refuse switches that would otherwise parse and do nothing."""
    if getattr(cfg, "load_in_8bit", False) or getattr(cfg, "load_in_4bit", False) or getattr(cfg, "use_bnb_nested_quant", False):
        raise ValueError("load_in_8bit / load_in_4bit / use_bnb_nested_quant: quantised base weights are not available in this "
                         "framework (no bitsandbytes); train bf16 with fp32 master weights, optionally with use_lora")
    if getattr(cfg, "gradient_checkpointing", False) and getattr(cfg, "use_cache", None):
        cfg.use_cache = False  # a KV cache is incompatible with activation checkpointing (``open_instruct/model_utils.py:222-226``)
    mods = getattr(cfg, "lora_target_modules", None)
    if mods:
        known = {"q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj", "all-linear"}
        bad = [m for m in mods if m not in known]
        if bad:
            raise ValueError(f"lora_target_modules {bad}: adapters are built for {sorted(known)}")


def check_context_parallel(cp_degree, cp_strategy: str, world: int | None = None) -> int:
    """Sequence-parallel degree that realises a context-parallel request (``open_instruct/olmo_core_utils.py:151-181``).
    ``ulysses`` is what ``parallel/ulysses.py`` implements (heads are exchanged for sequence around attention); the ring
    strategies ``llama3`` (all-gather K/V) and ``zig_zag`` are refused with a pointer to it: inside one NVSwitch domain the
    head exchange moves less data than a K/V ring, and no ring kernel is built."""
    if not cp_degree or cp_degree <= 1:
        return 1
    if cp_strategy != "ulysses":
        raise ValueError(f"cp_strategy {cp_strategy!r} (ring attention) is not built; use cp_strategy ulysses "
                         f"(heads must divide by cp_degree {cp_degree})")
    if world is not None and world % cp_degree:
        raise ValueError(f"cp_degree {cp_degree} must divide the number of ranks {world}")
    return int(cp_degree)


@dataclass
class TrainingConfig:
    num_epochs: int = 1
    per_device_train_batch_size: int = 8
    gradient_accumulation_steps: int = 1
    learning_rate: float = 2e-5
    warmup_ratio: float = 0.1
    weight_decay: float = 0.0
    max_grad_norm: float | None = None
    max_seq_length: int = 4096
    lr_scheduler_type: str = "linear"
    max_train_steps: int | None = None
    activation_memory_budget: float = 1.0
    activation_checkpointing_mode: Literal["budget", "selected_modules"] = "budget"
    activation_checkpointing_modules: list[str] = field(default_factory=list)
    compile_model: bool = False
    fused_optimizer: bool = True
    cp_degree: int | None = None
    cp_strategy: Literal["llama3", "zig_zag", "ulysses"] = "llama3"


@dataclass
class DatasetMixConfig:
    mixer_list: list[str] = field(default_factory=list)
    mixer_list_splits: list[str] = field(default_factory=lambda: ["train"])
    transform_fn: list[str] = field(default_factory=list)
    target_columns: list[str] = field(default_factory=list)
    cache_mode: Literal["hf", "local"] = "local"
    local_cache_dir: str = "local_dataset_cache"
    skip_cache: bool = False
    cache_dataset_only: bool = False
    config_hash: str | None = None
    hf_entity: str | None = None


@dataclass
class LoggingConfig:
    logging_steps: int = 1
    with_tracking: bool = False
    wandb_project: str = "open_instruct_internal"
    wandb_entity: str | None = None
    report_to: str | list[str] = "all"
    wandb_group_name: str | None = None


@dataclass
class CheckpointConfig:
    output_dir: str = "output/"
    checkpointing_steps: int = 500
    ephemeral_save_interval: int | None = None
    keep_last_n_checkpoints: int = 3
    resume_from_checkpoint: str | None = None


@dataclass
class LoRAConfig:
    use_lora: bool = False
    lora_rank: int = 64
    lora_alpha: float = 16
    lora_dropout: float = 0.1


@dataclass
class HubConfig:
    push_to_hub: bool = False
    hf_repo_id: str | None = None
    hf_repo_revision: str | None = None
    hf_repo_url: str | None = None


@dataclass
class EvalConfig:
    try_launch_beaker_eval_jobs: bool = False
    try_auto_save_to_beaker: bool = False
    gs_bucket_path: str | None = None
    oe_eval_tasks: list[str] | None = None
    oe_eval_max_length: int = 4096
    oe_eval_gpu_multiplier: int | None = None
    eval_workspace: str | None = None
    eval_priority: str | None = "high"
