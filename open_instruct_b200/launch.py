"""Job launcher: one rank per GPU through ``torch.distributed.run``, with the dataset cache filled first.

    python -m open_instruct_b200.launch --num_gpus 8 -- python -m open_instruct_b200.finetune recipe.yaml --learning_rate 5e-6

What it takes over from the reference's cluster launcher (``mason.py``):

* *auto dataset caching* (``mason.py:395-470``): before any GPU process starts, the training command is run once
  with ``--cache_dataset_only`` (arguments that do not influence the cache are stripped) so that N ranks do not
  tokenise the same mix N times;
* *process-count rewriting* (``mason.py:533-546``): the launcher owns ``--nnodes / --nproc-per-node / --node-rank``
  and the rendezvous address, the user command stays free of them;
* *auto output directory* (``mason.py:472-508``): ``--output_dir`` is filled in as
  ``<auto_output_dir_path>/<exp_name>_<timestamp>`` when the command does not set one;
* *experiment spec*: ``--dry_run`` prints the resolved spec (commands, environment, resources) as JSON instead of
  running; ``--experiment_spec out.yaml`` writes the same job in the task format of the reference's scheduler
  (``mason.py:600-690`` builds a Beaker ``ExperimentSpec``): one task per job with image, cluster constraints, priority,
  preemptibility, GPU count, replicas + leader selection + host networking for several nodes, environment variables and
  named secrets, mounted datasets, retries.  Writing the file needs no scheduler client; submitting it is the scheduler's
  own CLI (``beaker experiment create out.yaml``).

Image builds and site-specific storage mounts of the reference have no counterpart here.
"""

from __future__ import annotations

import argparse
import json
import os
import shlex
import subprocess
import sys
import time

TRAINING_MODULES = ("open_instruct_b200.finetune", "open_instruct_b200.dpo_tune_cache", "open_instruct_b200.grpo_fast",
                    "open_instruct_b200.reward_modeling", "open_instruct_b200.finetune_numpy", "open_instruct_b200.dpo", "open_instruct_b200.grpo")
# arguments that do not change what gets tokenised: dropped from the caching run so it starts fast and never touches a GPU
CACHE_EXCLUDED_ARGS = {"--with_tracking": False, "--checkpoint_state_freq": True, "--checkpoint_state_dir": True, "--gs_checkpoint_state_dir": True,
                       "--push_to_hub": False, "--try_launch_beaker_eval_jobs": False, "--wandb_entity": True, "--hf_entity": True}
SINGLE_PROCESS_MODULES = ("open_instruct_b200.grpo_fast", "open_instruct_b200.grpo")  # start their own learner / engine processes


def split_command(argv: list[str]) -> tuple[list[str], list[str]]:
    if "--" not in argv:
        raise SystemExit("usage: launch.py [launcher options] -- <training command>")
    i = argv.index("--")
    return argv[:i], argv[i + 1:]


def training_module(command: list[str]) -> str | None:
    for tok in command:
        for m in TRAINING_MODULES:
            if tok == m or tok.endswith(m.rsplit(".", 1)[-1] + ".py"):
                return m
    return None


def without_args(command: list[str], excluded: dict[str, bool]) -> list[str]:
    out, skip = [], False
    for tok in command:
        if skip:
            skip = False
            continue
        if tok in excluded:
            skip = excluded[tok]
            continue
        if "=" in tok and tok.split("=", 1)[0] in excluded:
            continue
        out.append(tok)
    return out


def has_arg(command: list[str], name: str) -> bool:
    return any(t == name or t.startswith(name + "=") for t in command)


def caching_command(command: list[str]) -> list[str]:
    return without_args(command, CACHE_EXCLUDED_ARGS) + ["--cache_dataset_only"]


def distributed_command(command: list[str], num_gpus: int, num_nodes: int, node_rank: int, master_addr: str, master_port: int) -> list[str]:
    """``python [-m mod | script.py] args`` -> ``python -m torch.distributed.run ... [-m mod | script.py] args``."""
    if not command or "python" not in os.path.basename(command[0]):
        raise SystemExit("the training command must start with a python interpreter")
    head = [command[0], "-m", "torch.distributed.run", f"--nnodes={num_nodes}", f"--nproc-per-node={num_gpus}", f"--node-rank={node_rank}",
            "--master-addr", master_addr, "--master-port", str(master_port)]
    return head + command[1:]


def build_spec(opts, command: list[str]) -> dict:
    module = training_module(command)
    cmd = list(command)
    if module and opts.auto_output_dir_path and not has_arg(cmd, "--output_dir") and not has_arg(cmd, "--save_folder"):
        exp = next((cmd[i + 1] for i, t in enumerate(cmd[:-1]) if t == "--exp_name"), module.rsplit(".", 1)[-1])
        cmd += ["--output_dir", os.path.join(opts.auto_output_dir_path, f"{exp}_{int(time.time())}")]
    steps = []
    if module and not opts.no_auto_dataset_cache and module != "open_instruct_b200.finetune_numpy":
        steps.append({"name": "cache_dataset", "command": caching_command(cmd), "gpus": 0})
    if module in SINGLE_PROCESS_MODULES or opts.num_gpus * opts.num_nodes == 1:
        run = cmd
    else:
        run = distributed_command(cmd, opts.num_gpus, opts.num_nodes, opts.node_rank, opts.master_addr, opts.master_port)
    steps.append({"name": "train", "command": run, "gpus": opts.num_gpus})
    env = {k: v for k, v in (e.split("=", 1) for e in opts.env)}
    env.setdefault("MASTER_ADDR", opts.master_addr)
    env.setdefault("TOKENIZERS_PARALLELISM", "false")
    return {"steps": steps, "env": env, "resources": {"gpus_per_node": opts.num_gpus, "nodes": opts.num_nodes}, "description": opts.description}


def experiment_spec(opts, spec: dict) -> dict:
    """The job of ``build_spec`` as a scheduler experiment (Beaker v2 field names): the steps become one shell command, the
    caching step runs on the first replica only."""
    nodes = opts.num_nodes
    lines = []
    for st in spec["steps"]:
        cmd = " ".join(shlex.quote(c) for c in st["command"])
        if nodes > 1 and st["name"] == "train":
            # every replica learns its rank and the leader's address from the scheduler
            cmd = cmd.replace(f"--node-rank={opts.node_rank}", "--node-rank=$BEAKER_REPLICA_RANK").replace(
                f"--master-addr {shlex.quote(opts.master_addr)}", "--master-addr $BEAKER_LEADER_REPLICA_HOSTNAME")
        if st["gpus"] == 0:
            cmd = f"if [ \"${{BEAKER_REPLICA_RANK:-0}}\" = \"0\" ]; then CUDA_VISIBLE_DEVICES= {cmd}; fi"
        lines.append(cmd)
    env = [{"name": k, "value": v} for k, v in sorted(spec["env"].items())]
    env += [{"name": e.split("=", 1)[1] if "=" in e else e, "secret": e.split("=", 1)[0]} for e in opts.secret]
    task = {"name": opts.task_name or "train", "image": {"beaker": opts.image} if opts.image else {"docker": "nvcr.io/nvidia/pytorch:latest"},
            "command": ["/bin/bash", "-c", " && ".join(lines)], "envVars": env,
            "resources": {"gpuCount": opts.num_gpus, **({"sharedMemory": opts.shared_memory} if opts.shared_memory else {})},
            "context": {"priority": opts.priority, "preemptible": bool(opts.preemptible)},
            "constraints": {"cluster": list(opts.cluster)} if opts.cluster else {},
            "datasets": [{"mountPath": m.split(":", 1)[1], "source": {"beaker": m.split(":", 1)[0]}} for m in opts.mount],
            "result": {"path": "/output"}}
    if nodes > 1:
        task.update({"replicas": nodes, "leaderSelection": True, "hostNetworking": True, "propagateFailure": True, "propagatePreemption": True,
                     "synchronizedStartTimeout": "48h"})
    exp = {"version": "v2", "description": spec.get("description") or "", "budget": opts.budget, "tasks": [task]}
    if opts.max_retries:
        exp["retry"] = {"allowedTaskRetries": opts.max_retries}
    return exp


def run_spec(spec: dict) -> int:
    env = {**os.environ, **spec["env"]}
    for step in spec["steps"]:
        print(f"[launch] {step['name']}: {' '.join(shlex.quote(c) for c in step['command'])}", flush=True)
        step_env = dict(env)
        if step["gpus"] == 0:
            step_env["CUDA_VISIBLE_DEVICES"] = ""
        rc = subprocess.call(step["command"], env=step_env)
        if rc != 0:
            print(f"[launch] step {step['name']} exited with {rc}", file=sys.stderr)
            return rc
    return 0


def main(argv: list[str] | None = None) -> int:
    own, command = split_command(list(sys.argv[1:] if argv is None else argv))
    ap = argparse.ArgumentParser()
    ap.add_argument("--num_gpus", type=int, default=1)
    ap.add_argument("--num_nodes", type=int, default=1)
    ap.add_argument("--node_rank", type=int, default=0)
    ap.add_argument("--master_addr", default="127.0.0.1")
    ap.add_argument("--master_port", type=int, default=29400)
    ap.add_argument("--env", action="append", default=[], help="NAME=VALUE, repeatable")
    ap.add_argument("--no_auto_dataset_cache", action="store_true")
    ap.add_argument("--auto_output_dir_path", default="")
    ap.add_argument("--description", default="")
    ap.add_argument("--dry_run", action="store_true")
    # scheduler experiment file (written, never submitted from here)
    ap.add_argument("--experiment_spec", default="", help="write the job as a scheduler experiment YAML and exit")
    ap.add_argument("--cluster", action="append", default=[])
    ap.add_argument("--image", default="")
    ap.add_argument("--priority", default="normal", choices=["low", "normal", "high", "urgent"])
    ap.add_argument("--preemptible", action="store_true")
    ap.add_argument("--budget", default="")
    ap.add_argument("--task_name", default="")
    ap.add_argument("--shared_memory", default="")
    ap.add_argument("--secret", action="append", default=[], help="SECRET_NAME=ENV_NAME, repeatable")
    ap.add_argument("--mount", action="append", default=[], help="dataset:/mount/path, repeatable")
    ap.add_argument("--max_retries", type=int, default=0)
    opts = ap.parse_args(own)
    spec = build_spec(opts, command)
    if opts.experiment_spec:
        import yaml

        with open(opts.experiment_spec, "w") as fh:
            yaml.safe_dump(experiment_spec(opts, spec), fh, sort_keys=False)
        print(f"[launch] wrote {opts.experiment_spec}")
        return 0
    if opts.dry_run:
        print(json.dumps(spec, indent=2))
        return 0
    return run_spec(spec)


if __name__ == "__main__":
    sys.exit(main())
