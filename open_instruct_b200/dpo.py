"""``python -m open_instruct_b200.dpo recipe.yaml`` - DPO through the same trainer as ``dpo_tune_cache``.

The reference has two DPO entry points that share one config dataclass: ``dpo_tune_cache.py`` (accelerate + DeepSpeed) and
``dpo.py`` (olmo-core FSDP/HSDP + TP, ``open_instruct/dpo.py:141-342``).  Here one sharded-optimizer runtime serves both
names.  ``tensor_parallel_degree`` splits every layer over groups of that many ranks (``parallel/tp.py:TrainTP``), with
data parallelism across the groups; ``fsdp_shard_degree`` sets the size of the parameter-sharding groups when the
parameters are sharded (``parallel/zero3.py``), replicas across them.
"""

from .dpo_tune_cache import main  # noqa: F401

if __name__ == "__main__":
    from .config.argparser import ArgumentParserPlus
    from .data.tokenize import TokenizerConfig
    from .dpo_utils import DPOExperimentConfig

    main(*ArgumentParserPlus((DPOExperimentConfig, TokenizerConfig)).parse())
