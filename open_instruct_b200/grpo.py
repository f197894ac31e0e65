"""``python -m open_instruct_b200.grpo recipe.yaml`` - GRPO through the same actors as ``grpo_fast``.

The reference's second GRPO entry point (``open_instruct/grpo.py:103-343`` + ``grpo_olmo_core_actor.py``) keeps the Ray topology
of ``grpo_fast`` and swaps the learner for an olmo-core FSDP2 train module with callbacks for weight sync, evaluation and
reference-policy updates.  Those three happen inside this framework's driver loop (``grpo_fast.main``), so both names run
the same code.
"""

from .grpo_fast import main  # noqa: F401

if __name__ == "__main__":
    from .config.argparser import ArgumentParserPlus
    from .config.schemas import ModelConfig
    from .data.tokenize import TokenizerConfig
    from .environments.tools.utils import EnvsConfig
    from .grpo_utils import GRPOExperimentConfig
    from .streaming import StreamingDataLoaderConfig, VLLMConfig

    parser = ArgumentParserPlus((GRPOExperimentConfig, TokenizerConfig, ModelConfig, StreamingDataLoaderConfig, VLLMConfig, EnvsConfig))
    parser.set_defaults(exp_name="grpo", warmup_ratio=0.0, max_grad_norm=1.0, per_device_train_batch_size=1)
    main(*parser.parse())
