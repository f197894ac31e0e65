"""``python -m open_instruct_b200.dpo recipe.yaml`` - DPO through the same trainer as ``dpo_tune_cache``.

The reference has two DPO entry points that share one config dataclass: ``dpo_tune_cache.py`` (accelerate + DeepSpeed) and
``dpo.py`` (olmo-core FSDP/HSDP + TP, ``open_instruct/dpo.py:141-342``).  Here one sharded-optimizer runtime serves both
names; the olmo-core-only switches (``tensor_parallel_degree``, ``shard_degree``, ``num_replicas``) are accepted by the
config and have no effect, because parameters are resident on every GPU and the optimizer is always sharded over all ranks.
"""

from .dpo_tune_cache import main  # noqa: F401

if __name__ == "__main__":
    from .config.argparser import ArgumentParserPlus
    from .data.tokenize import TokenizerConfig
    from .dpo_utils import DPOExperimentConfig

    main(*ArgumentParserPlus((DPOExperimentConfig, TokenizerConfig)).parse())
