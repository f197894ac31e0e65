"""GRPO driven by a ``Trainer`` with callbacks (the ``grpo`` API).

    python -m open_instruct_b200.grpo recipe.yaml [--flag value ...]

The reference's second GRPO entry point (``open_instruct/grpo.py:103-343`` + ``grpo_olmo_core_actor.py`` + ``grpo_callbacks.py``)
keeps the actor topology of ``grpo_fast`` - learner ranks, rollout engines, the data-preparation actor, the actor manager -
and moves what happens around a training step into callbacks: weight sync, reference-policy update, evaluation,
checkpoints, step timing.  Same here: ``grpo_fast.GRPORun`` builds the topology and offers the pieces of a step;
this file wires them as callbacks around a ``Trainer`` in the driver, where ``grpo_fast.main`` runs them as a plain loop.
Both accept the same six config dataclasses.
"""

from __future__ import annotations

from .config.schemas import ModelConfig
from .data.tokenize import TokenizerConfig
from .grpo_callbacks import (
    DataPreparationActorCheckpointCallback,
    DriverGRPOModule,
    EvalCallback,
    RefPolicyUpdateCallback,
    StepLogCallback,
    StepSource,
    VLLMWeightSyncCallback,
)
from .grpo_fast import GRPORun
from .grpo_utils import GRPOExperimentConfig
from .streaming import StreamingDataLoaderConfig, VLLMConfig
from .trainer import StepTimingCallback, Trainer


def main(args: GRPOExperimentConfig, tc: TokenizerConfig, model_config: ModelConfig, streaming: StreamingDataLoaderConfig,
         vllm: VLLMConfig, tools_config=None) -> dict:
    run = GRPORun(args, tc, model_config, streaming, vllm, tools_config)
    if run.cached_only is not None:
        return run.cached_only
    run.ref_update_in_step = False  # RefPolicyUpdateCallback does it
    try:
        start = run.begin()
        callbacks = [StepTimingCallback(), VLLMWeightSyncCallback(run), RefPolicyUpdateCallback(run), EvalCallback(run), StepLogCallback(run),
                     DataPreparationActorCheckpointCallback(run)]
        trainer = Trainer(DriverGRPOModule(run), StepSource(start + 1, args.num_training_steps), max_steps=args.num_training_steps,
                          callbacks=callbacks, tracker=None, start_step=start)
        trainer.fit()
    finally:
        run.close()
    out = dict(run.last)
    out["num_training_steps"] = args.num_training_steps
    return out


if __name__ == "__main__":
    from .config.argparser import ArgumentParserPlus
    from .environments.tools.utils import EnvsConfig

    parser = ArgumentParserPlus((GRPOExperimentConfig, TokenizerConfig, ModelConfig, StreamingDataLoaderConfig, VLLMConfig, EnvsConfig))
    parser.set_defaults(exp_name="grpo", warmup_ratio=0.0, max_grad_norm=1.0, per_device_train_batch_size=1)
    main(*parser.parse())
