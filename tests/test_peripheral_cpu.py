"""CPU tests for offline tooling: code execution, numpy shards, model merging, LoRA, legacy mixer."""

import gzip
import json
import os

import numpy as np
import pytest
import torch

from open_instruct_b200.models.spec import get_spec


def test_code_exec_assert_and_stdio():
    from open_instruct_b200.code_utils.code_utils import get_successful_tests_fast, get_successful_tests_stdio

    prog = "def add(a, b):\n    return a + b\n"
    res, times = get_successful_tests_fast(prog, ["assert add(1, 2) == 3", "assert add(1, 2) == 4", "import time; time.sleep(5)"], 1.0)
    assert res == [1, 0, 0] and len(times) == 3
    res, _ = get_successful_tests_stdio("print(int(input()) * 2)", [{"input": "4\n", "output": "8"}, {"input": "4\n", "output": "9"}], 1.0)
    assert res == [1, 0]
    # the guard makes destructive calls unusable inside the child, and the parent is untouched
    res, _ = get_successful_tests_fast("import os\nos.remove('x')", ["assert True"], 1.0)
    assert res == [0] and os.remove is not None
    assert get_successful_tests_fast("import subprocess", ["assert True"], 1.0)[0] == [0]


def test_code_api_routes():
    from fastapi.testclient import TestClient

    from open_instruct_b200.code_utils.api import app

    try:
        c = TestClient(app)
    except Exception as e:  # httpx missing
        pytest.skip(str(e))
    assert c.get("/health").json() == {"status": "healthy"}
    r = c.post("/test_program", json={"program": "x = 1", "tests": ["assert x == 1", "assert x == 2"], "max_execution_time": 1.0}).json()
    assert r["results"] == [1, 0]


def test_shard_writer_resume_and_reader(tmp_path):
    from open_instruct_b200.data.numpy_dataset_conversion import NumpyPackedFSLDataset, ShardWriter, select_token_dtype

    assert select_token_dtype(256) is np.uint8 and select_token_dtype(257) is np.uint16 and select_token_dtype(70000) is np.uint32
    rng = np.random.default_rng(0)
    docs = [rng.integers(0, 1000, size=int(n)) for n in rng.integers(3, 40, size=30)]
    w = ShardWriter(tmp_path, 1000, sync_every=1)
    for d in docs[:10]:
        w.append(d, np.where(np.arange(len(d)) < 2, -100, d))
    w.sync()
    for f in w.fh.values():
        f.close()
    # simulate a crash in the middle of a sample: data written, commit record cut in half
    with open(tmp_path / "_tokens.partial.bin", "ab") as f:
        f.write(b"\x01\x02\x03\x04\x05\x06")
    with open(tmp_path / "_boundaries.partial.bin", "ab") as f:
        f.write(b"\x00" * 7)
    w = ShardWriter(tmp_path, 1000, resume=True)
    assert w.num_samples == 10 and w.position == sum(len(d) for d in docs[:10])
    for d in docs[10:]:
        w.append(d, np.where(np.arange(len(d)) < 2, -100, d))
    chunks = w.finalize(max_shard_gb=200 * 2 / 1024**3)  # 200 tokens of uint16 per shard
    total = sum(len(d) for d in docs)
    assert chunks[-1][1] == total and len(chunks) == -(-total // 200)
    flat = np.concatenate(docs)
    got = np.concatenate([np.memmap(tmp_path / f"token_ids_part_{i:04d}.npy", mode="r", dtype=np.uint16) for i in range(len(chunks))])
    assert np.array_equal(got, flat)
    with gzip.open(tmp_path / "token_ids_part_0000.csv.gz", "rt") as f:
        first = [tuple(map(int, ln.split(","))) for ln in f]
    assert first[0] == (0, len(docs[0])) and first[-1][1] == 200
    ds = NumpyPackedFSLDataset(tmp_path, 64, 1000)
    assert len(ds) == sum((e - s) // 64 for s, e in chunks)
    win = ds[1]
    assert np.array_equal(win.input_ids, flat[64:128]) and win.cu_seqlens[0] == 0 and win.cu_seqlens[-1] == 64
    assert not win.label_mask[win.cu_seqlens[1]:win.cu_seqlens[1] + 2].any()


def _tiny_ckpt(path, seed):
    from open_instruct_b200.ckpt.hf_io import save_hf_checkpoint
    from open_instruct_b200.models.llama import LlamaModel

    m = LlamaModel(get_spec("tiny"), seed=seed)
    save_hf_checkpoint(m.flat, m.spec, str(path), dtype=torch.float32)
    return m


def test_merge_models(tmp_path):
    from safetensors.torch import load_file

    from open_instruct_b200.ckpt.merge_models import merge_models

    a, b = _tiny_ckpt(tmp_path / "a", 1), _tiny_ckpt(tmp_path / "b", 2)
    merge_models([str(tmp_path / "a"), str(tmp_path / "b")], str(tmp_path / "m"), [1.0, 3.0], dtype="float32")
    sd = load_file(str(tmp_path / "m" / "model.safetensors"))
    exp = 0.25 * a.p["l0.wo"] + 0.75 * b.p["l0.wo"]
    assert torch.allclose(sd["model.layers.0.self_attn.o_proj.weight"], exp.detach(), atol=1e-6)
    assert (tmp_path / "m" / "config.json").exists()
    with pytest.raises(ValueError):
        merge_models([str(tmp_path / "a")], str(tmp_path / "x"), [1.0, 2.0])


def test_lora_ref_grads_match_merged_contraction(tmp_path):
    from safetensors.torch import load_file

    from open_instruct_b200.models.llama import LlamaModel
    from open_instruct_b200.models.lora import LoRAAdapters, merge_lora_checkpoint

    spec = get_spec("tiny")
    m = _tiny_ckpt(tmp_path / "base", 3)
    lora = LoRAAdapters(spec, m.layout, rank=4, alpha=8.0, seed=1)
    with torch.no_grad():
        for k in lora.B:
            lora.B[k].normal_(0, 0.05)
    base = m.flat.detach().clone()
    ids = torch.randint(0, spec.vocab_size, (24,))
    pos = torch.cat([torch.arange(10), torch.arange(14)])
    cu = torch.tensor([0, 10, 24], dtype=torch.int32)
    labels = torch.roll(ids, -1)
    # (1) autograd through the adapters
    lora.apply_ref(m, base)
    loss = -m.token_logprobs(ids, pos, cu, labels)[0].mean()
    loss.backward()
    g_auto = lora.flat.grad.clone()
    # (2) merged weights -> dL/dW_eff -> contraction (what the fused path does)
    m2 = LlamaModel(spec, flat=base.clone())
    lora.merge_into(m2, base)
    m2.flat.requires_grad_(True)
    m2.p = m2.layout.views(m2.flat)
    loss2 = -m2.token_logprobs(ids, pos, cu, labels)[0].mean()
    loss2.backward()
    assert abs(loss.item() - loss2.item()) < 1e-5
    m2.main_grad = m2.flat.grad.float()
    g_merged = lora.pull_grads(m2)
    assert torch.allclose(g_auto, g_merged, atol=1e-5, rtol=1e-4)
    # (3) adapter files fold into the checkpoint
    lora.save(str(tmp_path / "adapter"))
    n = merge_lora_checkpoint(str(tmp_path / "base"), str(tmp_path / "adapter"), str(tmp_path / "merged"), dtype=torch.float32)
    assert n == len(lora.slots)
    sd = load_file(str(tmp_path / "merged" / "model.safetensors"))
    k = "model.layers.1.mlp.up_proj.weight"
    assert torch.allclose(sd[k], m2.layout.views(m2.flat.detach())["l1.w_gate_up"][spec.intermediate_size:], atol=1e-6)


def test_legacy_get_datasets(tmp_path):
    from open_instruct_b200.data.legacy_mix import get_datasets

    a, b = tmp_path / "a.jsonl", tmp_path / "b.jsonl"
    a.write_text("\n".join(json.dumps({"messages": [{"role": "user", "content": f"q{i}"}, {"role": "assistant", "content": "a"}]}) for i in range(10)))
    b.write_text("\n".join(json.dumps({"instruction": f"do {i}", "input": "", "output": "ok"}) for i in range(8)))
    out = get_datasets({str(a): 0.5, str(b): 1.0}, splits=["train"], columns_to_keep=["messages"], add_source_col=True, keep_ids=True)
    assert len(out["train"]) == 5 + 8 and set(out["train"].column_names) == {"messages", "id", "source"}
    assert out["train"][12]["messages"][1]["content"] == "ok"
    out = get_datasets([str(a), "3", str(b), "2"], splits=["train"], columns_to_keep=["messages"])
    assert len(out["train"]) == 5
    with pytest.raises(NotImplementedError):
        get_datasets({str(a): 0.5, str(b): 3}, splits=["train"])


def _completions():
    rows = []
    for p in range(3):
        for c in range(2):
            rows.append({"messages": [{"role": "user", "content": f"q{p}"}, {"role": "assistant", "content": f"a{p}{c}"}],
                         "model_completion": f"a{p}{c}", "reference_completion": f"ref{p}"})
    return rows


def test_rejection_sampling_select_and_vote():
    from open_instruct_b200.rejection_sampling.rejection_sampling import majority_vote, select

    length = lambda convs: [float(len(c[-1]["content"])) + (0.5 if c[-1]["content"].endswith("1") else 0.0) for c in convs]
    neg = lambda convs: [-x for x in length(convs)]
    table, per = select(_completions(), {"len": length, "len2": length, "neg": neg}, num_completions=2)
    # reference ("refP", 4 chars) is the longest, "aP0" the shortest
    assert [c[-1]["content"] for c in table["chosen"]] == ["ref0", "ref1", "ref2"]
    assert [c[-1]["content"] for c in table["rejected"]] == ["a00", "a10", "a20"]
    assert len(per["messages"]) == 9 and set(table["chosen_score"][0]) == {"len", "len2", "neg"}
    table, per = select(_completions(), {"len": length}, num_completions=2, include_reference=False)
    assert [c[-1]["content"] for c in table["chosen"]] == ["a01", "a11", "a21"] and len(per["messages"]) == 6
    v = majority_vote({"a": torch.tensor([1, 2]), "b": torch.tensor([1, 3]), "c": torch.tensor([0, 3])})
    assert v.tolist() == [1, 3]


def test_synthetic_preferences_with_fake_judge(tmp_path):
    from open_instruct_b200.rejection_sampling import synthetic_preference_dataset as spd

    src = tmp_path / "c.jsonl"
    src.write_text("\n".join(json.dumps(r) for r in _completions()))

    async def judge(messages):
        # prefers whichever shown response is the reference answer, else response 0
        text = messages[0]["content"]
        r1 = text.split("Response 1:")[1]
        return "Comparison: ok\nPreferred: " + ("1" if "'ref" in r1 else "0")

    out = spd.main(spd.Args(input_filename=str(src), save_filename=str(tmp_path / "o.jsonl"), num_completions=2), judge=judge)
    assert len(out["chosen"]) == 9  # 3 prompts x C(3, 2)
    for ch, rj in zip(out["chosen"], out["rejected"]):
        assert not rj[-1]["content"].startswith("ref") and ch[:-1] == rj[:-1]
    assert sum(c[-1]["content"].startswith("ref") for c in out["chosen"]) == 6


def test_launcher_spec():
    import argparse

    from open_instruct_b200 import launch

    own, cmd = launch.split_command(["--num_gpus", "4", "--", "python", "-m", "open_instruct_b200.finetune", "r.yaml", "--with_tracking",
                                     "--wandb_entity", "x", "--learning_rate", "1e-5"])
    assert own == ["--num_gpus", "4"] and launch.training_module(cmd) == "open_instruct_b200.finetune"
    c = launch.caching_command(cmd)
    assert c[-1] == "--cache_dataset_only" and "--with_tracking" not in c and "x" not in c and "1e-5" in c
    opts = argparse.Namespace(num_gpus=4, num_nodes=2, node_rank=1, master_addr="10.0.0.1", master_port=1234, env=["A=b"], no_auto_dataset_cache=False,
                              auto_output_dir_path="/out", description="")
    spec = launch.build_spec(opts, cmd)
    assert [s["name"] for s in spec["steps"]] == ["cache_dataset", "train"] and spec["env"]["A"] == "b"
    train = spec["steps"][1]["command"]
    assert train[1:3] == ["-m", "torch.distributed.run"] and "--nproc-per-node=4" in train and "--node-rank=1" in train
    assert "--output_dir" in train and train[train.index("--output_dir") + 1].startswith("/out/finetune_")
    spec = launch.build_spec(opts, ["python", "-m", "open_instruct_b200.grpo_fast", "--output_dir", "o"])
    assert spec["steps"][1]["command"][1:3] == ["-m", "open_instruct_b200.grpo_fast"]


def test_resource_plan():
    from open_instruct_b200.grpo_fast_resource_plan import build_plan, check_or_raise

    plan = build_plan([6], False, 2, 1)
    assert plan.min_gpus == 8 and plan.min_cpus == 60 + 2 + 2 + 1
    assert plan.shortfalls({"GPU": 8, "CPU": 100}) == []
    assert "learner group requires GPU=6" in plan.shortfalls({"GPU": 4, "CPU": 100})[0]
    assert "full topology requires at least GPU=8" in plan.shortfalls({"GPU": 7, "CPU": 100})[0]
    with pytest.raises(RuntimeError):
        check_or_raise(plan, {"GPU": 7, "CPU": 100})
    assert len(check_or_raise(plan, {"GPU": 8, "CPU": 10})) == 1
    assert build_plan([1], True, 1, 1).min_gpus == 1


def test_finetune_numpy_end_to_end(tmp_path):
    from open_instruct_b200 import finetune_numpy as fn
    from open_instruct_b200.data.numpy_dataset_conversion import NumpyPackedFSLDataset, ShardWriter

    spec = get_spec("tiny")
    rng = np.random.default_rng(1)
    w = ShardWriter(tmp_path / "data", spec.vocab_size)
    for _ in range(40):
        d = rng.integers(1, spec.vocab_size, size=int(rng.integers(5, 30)))
        w.append(d, np.where(np.arange(len(d)) < 2, -100, d))
    w.finalize()
    ds = NumpyPackedFSLDataset(tmp_path / "data", 32, spec.vocab_size)
    b = fn.window_to_batch([ds[0], ds[1]])
    cu = b["cu_seq_lens_q"]
    assert cu[-1] == 64 and 32 in cu.tolist() and (b["position_ids"][cu[:-1].long()] == 0).all()
    assert (b["labels_shifted"][cu[1:].long() - 1] == -100).all()
    args = fn.Args(model_name_or_path="tiny", dataset_path=str(tmp_path / "data"), sequence_length=32, global_batch_size=128,
                   rank_microbatch_size=64, max_train_steps=3, save_folder=str(tmp_path / "out"), save_interval=2, learning_rate=1e-3)
    m = fn.main(args)
    assert m["completed_steps"] == 3 and np.isfinite(m["train_loss"])
    assert (tmp_path / "out" / "hf" / "config.json").exists() and (tmp_path / "out" / "step_2").exists()
    args.max_train_steps = 4
    assert fn.main(args)["completed_steps"] == 4  # resumed from step_2, ran 2 more


def test_distill_compression_roundtrip_and_sampler(tmp_path):
    from open_instruct_b200.distill.compression import QuantizationConfig, compress_logprobs, decompress_logprobs, pack_bits, unpack_bits
    from open_instruct_b200.distill.sample_logits import Args, ParquetShardWriter, process_dataset
    from open_instruct_b200.models.llama import LlamaModel

    ids = torch.randint(0, 128256, (5, 7, 64))
    assert torch.equal(unpack_bits(pack_bits(ids, 17), 17, 64), ids)
    assert pack_bits(ids, 17).shape[-1] == 64 * 17 // 8
    cfg = QuantizationConfig(k=64, exact_k=8, vocab_size=128256)
    logits = torch.randn(40, 1000) * 3
    lp = torch.log_softmax(logits, -1).topk(64, -1).values
    comp = compress_logprobs(lp, cfg)
    assert comp.dtype == torch.uint8 and comp.shape == (40, cfg.logprob_bytes()) and cfg.logprob_bytes() < 64 * 2 // 2
    back = decompress_logprobs(comp, cfg)
    assert torch.allclose(back[:, :8], lp[:, :8], atol=5e-3)
    assert (back - lp).abs().max() < 0.25 and (back - lp).abs().mean() < 0.03
    # teacher sampling end to end on the tiny model
    spec = get_spec("tiny")
    m = LlamaModel(spec, seed=0)
    rows = [{"input_ids": torch.randint(1, spec.vocab_size, (n,)).tolist()} for n in (9, 17, 5)]
    qc = QuantizationConfig(k=16, exact_k=4, residual_bins=[], polynomial_degree=2, vocab_size=spec.vocab_size)
    n = process_dataset(m, rows, qc, Args(top_k=16, max_batch_tokens=20), ParquetShardWriter(str(tmp_path / "t"), 2))
    import pyarrow.parquet as pq

    files = sorted((tmp_path / "t").glob("*.parquet"))
    assert n == 3 and len(files) == 2
    t = pq.read_table(files[0]).to_pylist()
    assert t[0]["num_positions"] == 9 and len(t[0]["compressed_logprobs"]) == 9 * qc.logprob_bytes()


def test_decontamination_and_oai_generate(tmp_path):
    import asyncio

    from open_instruct_b200.decontamination.search import find_contamination
    from open_instruct_b200.experimental import oai_generate as og

    leak = "what is the capital of the country whose flag is a red circle on white background answer tokyo"
    train = [{"messages": [{"role": "user", "content": "hello there"}, {"role": "assistant", "content": "hi"}]},
             {"messages": [{"role": "user", "content": "Quiz: " + leak.upper()}, {"role": "assistant", "content": "Tokyo"}]}]
    ev = [{"text": leak}, {"text": "a completely unrelated question about prime numbers and their distribution over the integers today"}]
    rep = find_contamination(train, ev, ["messages"], ["text"], n=8, threshold=0.5)
    assert rep["eval_contaminated"] == 1 and rep["train_contaminated"] == [1]
    assert find_contamination(train, ev, ["messages"], ["text"], mode="exact")["eval_contaminated"] == 0

    calls = []

    async def post(url, payload, headers):
        calls.append(payload)
        if len(calls) == 1:
            raise RuntimeError("transient")
        return {"choices": [{"message": {"content": "ok:" + payload["messages"][0]["content"]}}], "usage": {"total_tokens": 3}}

    rows = [{"custom_id": "a", "body": {"messages": [{"role": "user", "content": "x"}]}}, {"custom_id": "b", "body": {"messages": [{"role": "user", "content": "y"}]}}]
    out = asyncio.run(og.run_chat(rows, og.Args(max_parallel_requests=1), post=post))
    assert [o["response"] for o in out] == ["ok:x", "ok:y"] and len(calls) == 3

    state = {"polls": 0}

    def http(method, url, **kw):
        if url.endswith("/files"):
            state["lines"] = kw["files"]["file"][1].decode().splitlines()
            return {"id": "file-1"}
        if url.endswith("/batches"):
            return {"id": "b1", "status": "validating"}
        if url.endswith("/batches/b1"):
            state["polls"] += 1
            return {"id": "b1", "status": "completed", "output_file_id": "file-2"}
        if url.endswith("/content"):
            return "\n".join(json.dumps({"custom_id": json.loads(l)["custom_id"], "response": {"body": {"choices": [{"message": {"content": "r"}}]}}})
                             for l in state["lines"]).encode()
        raise AssertionError(url)

    out = og.run_batch(rows, og.Args(poll_seconds=0.0), http=http)
    assert [o["response"] for o in out] == ["r", "r"] and state["polls"] == 1


def test_recipes_parse():
    from open_instruct_b200.config.argparser import ArgumentParserPlus
    from open_instruct_b200.config.schemas import ModelConfig
    from open_instruct_b200.data.tokenize import TokenizerConfig
    from open_instruct_b200.dpo_utils import DPOExperimentConfig
    from open_instruct_b200.finetune import FlatArguments
    from open_instruct_b200.grpo_utils import GRPOExperimentConfig
    from open_instruct_b200.streaming import StreamingDataLoaderConfig, VLLMConfig

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs", "train_configs")
    a, _ = ArgumentParserPlus((FlatArguments, TokenizerConfig)).parse([os.path.join(root, "tulu3_sft_8b.yaml"), "--learning_rate", "1e-5"])
    assert a.learning_rate == 1e-5 and a.gradient_accumulation_steps == 16 and a.packing
    d, _ = ArgumentParserPlus((DPOExperimentConfig, TokenizerConfig)).parse([os.path.join(root, "tulu3_dpo_8b.yaml")])
    assert str(getattr(d.loss_type, "value", d.loss_type)) == "dpo_norm" and d.beta == 5.0
    g = ArgumentParserPlus((GRPOExperimentConfig, TokenizerConfig, ModelConfig, StreamingDataLoaderConfig, VLLMConfig)).parse(
        [os.path.join(root, "tulu3_grpo_8b.yaml")])
    assert g[0].num_learners_per_node == [6] and g[3].num_samples_per_prompt_rollout == 16 and g[4].vllm_num_engines == 2


@pytest.mark.parametrize("module", ["finetune", "dpo_tune_cache", "reward_modeling", "grpo_fast", "finetune_numpy"])
def test_entry_point_help(module):
    """Every trainer builds its command line (no duplicate fields across its config dataclasses)."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-m", f"open_instruct_b200.{module}", "--help"], capture_output=True, text=True, timeout=180, cwd=root)
    assert res.returncode == 0 and "--" in res.stdout, res.stderr[-1500:]


def test_human_eval_app_and_metrics(tmp_path):
    from fastapi.testclient import TestClient

    from open_instruct_b200.human_eval.app import create_app, export_records
    from open_instruct_b200.human_eval.metrics import comparison_results

    inst = [{"id": f"q{i}", "prompt": f"prompt {i}", "completions": [{"model": "m1", "completion": f"a{i}"}, {"model": "m2", "completion": f"b{i}"}]}
            for i in range(3)]
    db = str(tmp_path / "he.sqlite3")
    c = TestClient(create_app(inst, db, seed=0))
    assert c.get("/summary").status_code == 401
    assert c.post("/signup", json={"username": "ann", "password": "pw"}).status_code == 200
    assert c.post("/signup", json={"username": "ann", "password": "x"}).status_code == 409
    assert c.post("/login", json={"username": "ann", "password": "bad"}).status_code == 401
    out = c.get("/api/model-outputs/1").json()
    assert out["prompt"] == "prompt 1" and {x["model"] for x in out["completions"]} == {"m1", "m2"}
    assert "error" in c.get("/api/model-outputs/9").json()
    assert "Instance 2" in c.get("/instances/2").text

    def judge(i, a, b, pref, acc_a="yes", acc_b="no"):
        r = c.post("/api/submit-evaluation", json={"index": i, "prompt": inst[i]["prompt"], "model_a": a, "model_b": b, "completion_a": "x",
                                                   "completion_b": "y", "completion_a_is_acceptable": acc_a, "completion_b_is_acceptable": acc_b,
                                                   "preference": pref})
        assert r.status_code == 200

    judge(0, "m1", "m2", "a-is-better")
    judge(0, "m2", "m1", "b-is-slightly-better", "no", "yes")   # second annotation of q0, sides swapped: m1 again
    judge(1, "m1", "m2", "tie")
    judge(1, "m1", "m2", "b-is-better")                         # tie vs preference: half an agreement
    judge(2, "m2", "m1", "a-is-better", "yes", "yes")
    assert c.post("/api/submit-feedback", json={"index": 2, "prompt": "p", "model_a": "m1", "model_b": "m2", "completion_a": "x",
                                                "completion_b": "y", "instance_quality": "bad", "comment": "unclear"}).status_code == 200
    s = c.get("/summary").json()
    assert s["user_contributions"] == {"ann": 5, "all": 5} and s["progress"]["missing_indices"] == []
    res = s["results"]["m1_vs_m2"]
    cmp_ = res["comparison_results"]
    assert cmp_["m1_wins"] == pytest.approx(1 / 3) and cmp_["m2_wins"] == pytest.approx(2 / 3)
    assert cmp_["agreement"] == {"num_instances_with_multiple_annotations": 2, "comparison_agreement": 0.5, "relaxed_comparison_agreement": 0.75}
    assert res["acceptance_results"]["m1"] == pytest.approx(1.0) and res["acceptance_results"]["m2"] == pytest.approx(1 / 3)
    assert res["feedback_records"] == {"bad": [2]}
    assert comparison_results([], "m1", "m2")["m1_wins"] == 0
    assert export_records(db, str(tmp_path / "out.jsonl")) == 6 and export_records(db, str(tmp_path / "out.csv")) == 6


def test_dataset_builders(tmp_path):
    from open_instruct_b200.data import builders
    from open_instruct_b200.data.synthetic import make_byte_tokenizer
    from transformers import AutoTokenizer

    rows = [{"question": "2+2?", "answer": "It is 4.\n#### 4"}, {"question": "big?", "answer": "a lot\n#### 1,234.5"}]
    assert builders.qa_to_messages(rows)[0]["messages"][1] == {"role": "assistant", "content": "It is 4.\n#### 4"}
    rl = builders.gsm8k_to_rlvr(rows)
    assert [r["ground_truth"] for r in rl] == ["4", "1234.5"] and rl[0]["dataset"] == "gsm8k" and len(rl[0]["messages"]) == 1
    c = builders.counter_env_samples(12)
    assert c[10]["ground_truth"] == "1" and c[9]["env_config"] == {"env_configs": [{"env_name": "counter", "target": "10"}]}
    g = builders.guess_number_env_samples(3, nothink=True)
    assert g[2]["env_config"]["env_configs"][0] == {"env_name": "guess_number", "number": "3"} and g[0]["messages"][1]["content"].endswith("/nothink")
    tok = AutoTokenizer.from_pretrained(make_byte_tokenizer(str(tmp_path / "tok")))
    data = [{"id": f"r{i}", "messages": [{"role": "system", "content": "s"}, {"role": "user", "content": "u" * (10 * (i + 1))},
                                         {"role": "assistant", "content": "a" * 5}]} for i in range(4)]
    st = builders.messages_statistics(data, tok)
    assert st["num_instances"] == 4 and st["turns_summary"]["mean"] == 2.0 and st["assistant_response_lengths_summary"]["max"] == 5.0
    assert st["total_lengths_summary"]["max"] == 45.0 and st["top_100_longest_instances"][0] == "r3"
    assert st["num_instances_with_total_length_gt_512"] == 0
    h = builders.token_length_histogram([{"text": "x" * n} for n in (3, 9, 17)], tok, "text", bucket=8)
    assert h["counts"] == [1, 1, 1] and h["edges"] == [0, 8, 16, 24]
    builders.main(["env", "--kind", "counter", "--num", "5", "--out", str(tmp_path / "c.jsonl")])
    assert len(builders.read_jsonl(str(tmp_path / "c.jsonl"))) == 5


def test_legacy_dataset_processors(tmp_path):
    """First-generation processors: column contract, prompt masking, length filters (the prompt limit wins for preferences)."""
    import datasets

    from helpers import make_tokenizer
    from open_instruct_b200.data import dataset_processor as dp
    from open_instruct_b200.data.templates import CHAT_TEMPLATES
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(make_tokenizer(str(tmp_path / "tok")))
    tok.chat_template = CHAT_TEMPLATES["tulu"]
    tok.add_special_tokens({"pad_token": "<pad>"})
    u = lambda t: {"role": "user", "content": t}
    a = lambda t: {"role": "assistant", "content": t}
    pref = datasets.Dataset.from_list([{"chosen": [u("say hi"), a("hi there friend")], "rejected": [u("say hi"), a("no")]},
                                       {"chosen": [u("count to twenty " * 40), a("one two")], "rejected": [u("count to twenty " * 40), a("three")]}])
    cfg = dp.DatasetConfig(max_prompt_token_length=30, max_token_length=5, num_proc=1)
    proc = dp.PreferenceDatasetProcessor(tok, cfg)
    out = proc.tokenize(pref)
    assert set(dp.TOKENIZED_PREFERENCE_DATASET_KEYS) <= set(out.column_names)
    assert out[0][dp.INPUT_IDS_CHOSEN_KEY][: len(out[0][dp.INPUT_IDS_PROMPT_KEY])] == out[0][dp.INPUT_IDS_PROMPT_KEY]
    assert len(proc.filter(out)) == 1  # the prompt limit is the only rule when it is given: row 0 stays although it exceeds max_token_length
    assert len(dp.PreferenceDatasetProcessor(tok, dp.DatasetConfig(max_token_length=5, num_proc=1)).filter(out)) == 0

    sft = datasets.Dataset.from_list([{"messages": [u("what is 2 plus 2"), a("four")], "ground_truth": "4", "dataset": "gsm8k"},
                                      {"messages": [u("only a question")], "ground_truth": "", "dataset": "gsm8k"}])
    p2 = dp.SFTGroundTruthDatasetProcessor(tok, dp.DatasetConfig(train_only_on_prompt=True, num_proc=1))
    t2 = p2.tokenize(sft)
    n = len(t2[0][dp.INPUT_IDS_PROMPT_KEY])
    assert t2[0][dp.LABELS_KEY][:n] == [-100] * n and t2[0][dp.LABELS_KEY][n:] == t2[0][dp.INPUT_IDS_KEY][n:] and t2[0][dp.GROUND_TRUTHS_KEY] == "4"
    assert len(p2.filter(t2)) == 1 and len(p2.filter(t2, need_contain_labels=False)) == 2  # a lone prompt has no trainable token
    assert dp.get_num_proc(10, 64, 400) == 1 and dp.get_num_proc(100000, 8, 400) == 8
    import pytest

    with pytest.raises(ValueError):
        dp.DatasetConfig(chat_template="no_such_template")


def test_notifications_progress_and_tracker_gates(tmp_path, monkeypatch):
    """Slack alerts, scheduler progress lines, run tags, disk warnings - and the tracker's optional back ends: every one of
    them works against a fake service and degrades to nothing when its service is missing."""
    import sys
    import types

    from open_instruct_b200.utils import notify
    from open_instruct_b200.utils.common import Tracker

    assert notify.format_eta(59) == "0m" and notify.format_eta(3700) == "1h 1m" and notify.format_eta(90061) == "1d 1h 1m"
    assert notify.progress_text(0, 40, 5.0) == "[0.0% complete (step 0/40), eta calculating...]"
    assert notify.progress_text(10, 40, 600.0) == "[25.0% complete (step 10/40), eta 30m]"
    assert notify.progress_text(40, 40, 7200.0) == "[100.0% complete (step 40/40), finished in 2h 0m]"

    class Sink(notify.DescriptionSink):
        text = "my run git_commit: old git_branch: old [50% ...]"

        def get(self):
            return self.text

        def set(self, t):
            self.text = t

        def url(self):
            return "https://jobs.example/1"

    monkeypatch.setenv("GIT_COMMIT", "abc123")
    monkeypatch.setenv("GIT_BRANCH", "main")
    sink = Sink()
    rep = notify.ProgressReporter(40, sink, wandb_url="https://wandb.example/run")
    out = rep.update(10)
    assert out.startswith("my run git_commit: abc123 git_branch: main https://wandb.example/run [25.0% complete (step 10/40), eta ")
    assert rep.update(40).count("git_commit:") == 1 and "finished in" in sink.text
    assert notify.ProgressReporter(40, sink=None).update(1) is None or True  # no scheduler: nothing happens

    sent = []

    class R:
        ok, status_code, text = True, 200, "ok"

    monkeypatch.delenv("SLACK_WEBHOOK_URL", raising=False)
    assert notify.send_slack_message("x", post=lambda *a, **k: sent.append((a, k)) or R()) is False and not sent
    monkeypatch.setenv("SLACK_WEBHOOK_URL", "https://hooks.example/T/B")
    assert notify.send_slack_message("job died", sink=sink, post=lambda *a, **k: sent.append((a, k)) or R()) is True
    assert sent[0][0][0] == "https://hooks.example/T/B" and sent[0][1]["json"]["text"] == "job died Check it out: https://jobs.example/1"

    def boom(*a, **k):
        raise OSError("no network")

    assert notify.send_slack_message("x", post=boom) is False

    class A:
        send_slack_alerts = True

    calls = []
    monkeypatch.setattr(notify, "send_slack_message", lambda m, **k: calls.append(m))

    @notify.alert_on_failure
    def main(args):
        raise RuntimeError("out of cheese")

    import pytest

    with pytest.raises(RuntimeError):
        main(A())
    assert calls and "RuntimeError: out of cheese" in calls[0]

    monkeypatch.setenv("WANDB_TAGS", "a,b")
    assert notify.get_wandb_tags()[:3] == ["a", "b", "commit: abc123"] and "branch: main" in notify.get_wandb_tags()
    assert notify.warn_if_low_disk_space("gs://bucket/x") is None
    assert "Disk usage near capacity" in notify.warn_if_low_disk_space(str(tmp_path / "not" / "yet"), threshold=0.0)
    assert notify.warn_if_low_disk_space(str(tmp_path), threshold=1.1) is None

    # tracker back ends: a fake wandb module receives init / log / finish; tensorboard writes event files; both are optional
    logged = []
    fake = types.SimpleNamespace(init=lambda **k: logged.append(("init", k["project"], k["name"])), log=lambda m, step: logged.append(("log", step, dict(m))),
                                 finish=lambda: logged.append(("finish",)))
    monkeypatch.setitem(sys.modules, "wandb", fake)
    t = Tracker(str(tmp_path / "run"), "r1", {"lr": 1.0}, report_to=("wandb", "tensorboard"), wandb_project="proj")
    t.log({"loss": 0.5, "note": "text"}, 3)
    t.close()
    assert logged[0] == ("init", "proj", "r1") and logged[1][:2] == ("log", 3) and logged[-1] == ("finish",)
    assert os.path.exists(tmp_path / "run" / "metrics.jsonl") and os.path.exists(tmp_path / "run" / "run_config.json")
    tb = tmp_path / "run" / "tb" / "r1"
    assert (not tb.exists()) or any(f.name.startswith("events") for f in tb.iterdir())  # written when tensorboard is installed
    monkeypatch.setitem(sys.modules, "wandb", None)  # import fails: the tracker carries on with the jsonl file alone
    t2 = Tracker(str(tmp_path / "run2"), "r2", None, report_to=("wandb",))
    t2.log({"loss": 1.0}, 1)
    t2.close()
    assert os.path.exists(tmp_path / "run2" / "metrics.jsonl")


def test_launcher_writes_a_scheduler_experiment(tmp_path):
    import yaml

    from open_instruct_b200 import launch

    out = tmp_path / "exp.yaml"
    rc = launch.main(["--num_gpus", "8", "--num_nodes", "2", "--cluster", "big-cluster", "--priority", "high", "--preemptible", "--budget", "team/x",
                      "--image", "me/img", "--secret", "MY_HF_TOKEN=HF_TOKEN", "--mount", "ds123:/data", "--env", "A=b", "--max_retries", "2",
                      "--experiment_spec", str(out), "--", "python", "-m", "open_instruct_b200.finetune", "recipe.yaml", "--with_tracking"])
    assert rc == 0
    exp = yaml.safe_load(open(out))
    task = exp["tasks"][0]
    assert exp["version"] == "v2" and exp["budget"] == "team/x" and exp["retry"] == {"allowedTaskRetries": 2}
    assert task["replicas"] == 2 and task["leaderSelection"] and task["hostNetworking"] and task["resources"]["gpuCount"] == 8
    assert task["context"] == {"priority": "high", "preemptible": True} and task["constraints"] == {"cluster": ["big-cluster"]}
    script = task["command"][2]
    assert "--cache_dataset_only" in script.split(" && ")[0] and "BEAKER_REPLICA_RANK" in script.split(" && ")[0]  # cached once, on replica 0
    assert "--with_tracking" not in script.split(" && ")[0] and "--with_tracking" in script.split(" && ")[1]
    assert "--nnodes=2" in script and "--node-rank=$BEAKER_REPLICA_RANK" in script and "--master-addr $BEAKER_LEADER_REPLICA_HOSTNAME" in script
    assert {"name": "HF_TOKEN", "secret": "MY_HF_TOKEN"} in task["envVars"] and {"name": "A", "value": "b"} in task["envVars"]
    assert task["datasets"] == [{"mountPath": "/data", "source": {"beaker": "ds123"}}]


def _recipe_files():
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs", "train_configs")
    return sorted(os.path.join(root, f) for f in os.listdir(root) if f.endswith(".yaml"))


@pytest.mark.parametrize("path", _recipe_files(), ids=os.path.basename)
def test_every_recipe_parses_with_its_entry_point(path):
    """Each recipe names its trainer in the first line; all its keys are flags of that trainer and pass its validation."""
    from open_instruct_b200.config.argparser import ArgumentParserPlus
    from open_instruct_b200.config.schemas import ModelConfig
    from open_instruct_b200.data.tokenize import TokenizerConfig
    from open_instruct_b200.dpo_utils import DPOExperimentConfig
    from open_instruct_b200.environments.tools.utils import EnvsConfig
    from open_instruct_b200.finetune import FlatArguments
    from open_instruct_b200.finetune_numpy import Args as NumpyArgs
    from open_instruct_b200.grpo_utils import GRPOExperimentConfig
    from open_instruct_b200.reward_modeling import Args as RMArgs
    from open_instruct_b200.streaming import StreamingDataLoaderConfig, VLLMConfig

    grpo = (GRPOExperimentConfig, TokenizerConfig, ModelConfig, StreamingDataLoaderConfig, VLLMConfig, EnvsConfig)
    parsers = {"finetune": (FlatArguments, TokenizerConfig), "dpo_tune_cache": (DPOExperimentConfig, TokenizerConfig), "dpo": (DPOExperimentConfig, TokenizerConfig),
               "grpo_fast": grpo, "grpo": grpo, "reward_modeling": (RMArgs, TokenizerConfig, ModelConfig), "finetune_numpy": (NumpyArgs,)}
    first = open(path).readline()
    assert first.startswith("# entry: "), f"{path} must start with '# entry: <trainer module>'"
    entry = first.split(":", 1)[1].strip()
    out = ArgumentParserPlus(parsers[entry]).parse([path])
    assert out is not None


def test_decontamination_through_an_elasticsearch_index(tmp_path):
    """Index the user turns of a training file into (a fake of) Elasticsearch, query it with evaluation examples, drop the
    contaminated rows; an interrupted indexing run resumes from the index's document count."""
    import json

    from helpers import FakeElasticsearch
    from open_instruct_b200.decontamination import es as es_mod
    from open_instruct_b200.decontamination import index as index_cli
    from open_instruct_b200.decontamination import search as search_cli

    leaked = "What is the sum of the first ten positive odd integers, and why is x^2+y^2=z^2 relevant?"
    train = [{"messages": [{"role": "user", "content": "Tell me a story about a dragon who learns to bake bread."}, {"role": "assistant", "content": "Once..."}]},
             {"messages": [{"role": "user", "content": f"Please answer carefully. {leaked} Thanks!"}, {"role": "assistant", "content": "100"}]},
             {"messages": [{"role": "user", "content": "Summarise the plot of Hamlet in two sentences."}, {"role": "assistant", "content": "..."}]}]
    tp, ep = tmp_path / "train.jsonl", tmp_path / "eval.jsonl"
    tp.write_text("".join(json.dumps(r) + "\n" for r in train))
    ep.write_text("".join(json.dumps(r) + "\n" for r in [{"text": leaked}, {"text": "Name three rivers in South America and the countries they cross."}]))
    fake = FakeElasticsearch()
    try:
        added = index_cli.main(["--es_url", fake.url, "--dataset", str(tp), "--text_batch_size", "2"])
        index = es_mod.index_name_for(str(tp))
        assert added == {index: 3} and len(fake.indices[index]["docs"]) == 3
        assert [r for r in fake.requests if r[0] == "BULK"] == [("BULK", 2), ("BULK", 1)]
        assert index_cli.main(["--es_url", fake.url, "--dataset", str(tp)]) == {index: 0}          # nothing left to add
        # the analyzer keeps operators together: "x^2+y^2=z^2" is one token on both sides
        assert "x^2+y^2=z^2" in es_mod.tokenize(leaked)
        rep = search_cli.main(["--es_url", fake.url, "--train", str(tp), "--eval", str(ep), "--field", "text", "--ngram_size", "8",
                               "--threshold", "0.5", "--output_dir", str(tmp_path / "out"), "--decontaminate"])
        assert rep["eval_contaminated"] == 1 and rep["eval_total"] == 2 and rep["train_contaminated"] == [1]
        assert rep["matches"][0]["score"] == 1.0            # every token of the leaked question lies inside a matching 8-gram
        kept = [json.loads(l) for l in open(tmp_path / "out" / "train_decontaminated.jsonl")]
        assert [r["messages"][0]["content"][:4] for r in kept] == ["Tell", "Summ"]
        rep = search_cli.main(["--es_url", fake.url, "--train", str(tp), "--eval", str(ep), "--field", "text", "--index_type", "exact",
                               "--output_dir", str(tmp_path / "out2")])
        assert rep["train_contaminated"] == [1] and rep["eval_contaminated"] == 1
    finally:
        fake.close()


def test_numa_node_of_a_gpu_and_binding(tmp_path):
    """The node comes from the GPU's PCI device in sysfs, else from the rank formula; binding goes through the host runtime and
    leaves the process on that node's CPUs."""
    import os

    from open_instruct_b200.utils import numa

    root = tmp_path / "sys"
    for n in (0, 1):
        (root / f"devices/system/node/node{n}").mkdir(parents=True)
    dev = root / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    unknown = root / "bus/pci/devices/0000:9d:00.0"
    unknown.mkdir(parents=True)
    (unknown / "numa_node").write_text("-1\n")
    s = str(root)
    assert numa.numa_node_count(s) == 2
    assert numa.pci_numa_node("00000000:1B:00.0", s) == 1          # the driver's spelling: 8-digit domain, upper case
    assert numa.node_for_gpu(0, "0000:1b:00.0", 8, s) == 1
    assert numa.node_for_gpu(5, "0000:9d:00.0", 8, s) == 1          # sysfs does not say: ranks 4-7 of 8 sit on the second node
    assert numa.node_for_gpu(2, None, 8, s) == 0
    assert numa.bind_to_gpu("cpu") is None
    before = os.sched_getaffinity(0)
    try:
        n = numa.bind_to_node(0)
        if n > 0:   # this machine exposes node 0
            assert len(os.sched_getaffinity(0)) <= n
        assert numa.bind_to_node(4096) == 0
    finally:
        os.sched_setaffinity(0, before)


def test_dataset_filters_and_rewrites(tmp_path):
    """The pre-mix row filters: each predicate on text that should and should not trip it, then the command over a file."""
    import json

    from open_instruct_b200.data import filters as F

    assert F.cjk_ratio("你好世界 hi") > 0.4 and F.cjk_ratio("plain text") == 0.0
    for yes in ("As of my last update in 2023, the tallest building is...", "My knowledge cutoff is September 2021.",
                "I don't have access to real-time information, but", "I was trained on data up to early 2022 so"):
        assert F.mentions_cutoff(yes), yes
    for no in ("The cutoff for applications is Friday.", "Update the training data loader."):
        assert not F.mentions_cutoff(no), no
    for yes in ("I am ChatGPT, a large language model.", "I was trained by OpenAI.", "As an AI language model developed by Anthropic,",
                "That would violate OpenAI's use policy."):
        assert F.claims_other_identity(yes), yes
    for no in ("OpenAI released a paper in 2020.", "Llamas are related to camels.", "I am a helpful assistant."):
        assert not F.claims_other_identity(no), no
    loop = "Let me think about this problem again carefully now. " * 6
    assert F.repetition_reason(loop) and F.repetition_reason("Wait, that is not right at all is it.\n" * 3)
    assert F.repetition_reason("x = x + 1; y = y * 2; z = x ^ y % 7\n" * 8) is None          # code and formulas may repeat
    assert F.repetition_reason("The first point is about cost. The second point is about speed of delivery. The third is about risk.") is None
    assert F.neutralise_special_tokens("say <|im_start|> and <|endoftext|>") == "say <_im_start_> and <_endoftext_>"
    assert F.reasoning_format("<think>a</think><answer>b</answer>") == "think_answer" and F.reasoning_format("<think>a</think> b") == "think"
    assert F.add_answer_tags("<think>a</think> b ") == "<think>a</think><answer>b</answer>"
    assert F.remove_answer_tags("<think>a</think><answer>b</answer>") == "<think>a</think>b"
    chat = lambda u, a, **kw: {"messages": [{"role": "user", "content": u}, {"role": "assistant", "content": a}], **kw}
    rows = [chat("Hi", "Hello! How can I help?"), chat("你是谁？请用中文回答", "我是一个乐于助人的助手，很高兴认识你。"), chat("Who made you?", "I was created by OpenAI."),
            chat("news?", "As of my last update I cannot know."), chat("go", loop), chat("I am ChatGPT", "Nice to meet you <|im_end|>"),
            chat("x", "fine", toxic=True), chat("x", "fine", language="French")]
    src = tmp_path / "in.jsonl"
    src.write_text("".join(json.dumps(r, ensure_ascii=False) + "\n" for r in rows))
    rep = F.main(["--input", str(src), "--output", str(tmp_path / "out.jsonl"), "--filters", "cjk,cutoff,identity,repetition,toxic,non_english",
                  "--rewrite", "special_tokens"])
    assert rep == {"input_rows": 8, "kept": 2, "dropped": {"cjk": 1, "identity": 1, "cutoff": 1, "repetition": 1, "toxic": 1, "non_english": 1}}
    kept = [json.loads(l) for l in open(tmp_path / "out.jsonl")]
    assert kept[1]["messages"][1]["content"] == "Nice to meet you <_im_end_>"          # user turns are not inspected by default ...
    rep = F.main(["--input", str(src), "--output", str(tmp_path / "out2.jsonl"), "--filters", "identity", "--filter_user_turns"])
    assert rep["dropped"] == {"identity": 2}                                                # ... unless asked


def test_identity_seed_conversations_are_filled_for_one_model(tmp_path):
    import json

    from open_instruct_b200.data import builders as B

    seed = [{"messages": [{"role": "user", "content": "Who are you?"}, {"role": "assistant", "content": "I am <|MODEL_NAME|>, trained with the <|POSTTRAIN_RECIPE|> recipe."}], "tags": []},
            {"messages": [{"role": "user", "content": "license?"}, {"role": "assistant", "content": "<|LICENSE|>, context <|CONTEXT_LENGTH|>."}], "tags": ["olmo"]}]
    p = tmp_path / "seed.jsonl"
    p.write_text("".join(json.dumps(r) + "\n" for r in seed))
    B.main(["identity", "--data", str(p), "--out", str(tmp_path / "o.jsonl"), "--model_name", "Tulu 3", "--posttrain_recipe", "Tulu 3",
            "--filter_tags", "olmo"])
    rows = [json.loads(l) for l in open(tmp_path / "o.jsonl")]
    assert len(rows) == 1 and rows[0]["messages"][1]["content"] == "I am Tulu 3, trained with the Tulu 3 recipe."
    with pytest.raises(ValueError, match="LICENSE"):
        B.fill_identity_placeholders(seed, {"model_name": "X", "posttrain_recipe": "Y"})
    full = B.fill_identity_placeholders(seed, {"model_name": "X", "posttrain_recipe": "Y", "license": "Apache 2.0", "context_length": 4096})
    assert full[1]["messages"][1]["content"] == "Apache 2.0, context 4096."


def test_decontamination_by_embedding_search(tmp_path):
    """Vector index: messages embedded by a local model (mean-pooled, normalised), kNN search through (a fake of) Elasticsearch; the
    leaked question's nearest neighbour is its own training row with similarity 1."""
    import json

    transformers = pytest.importorskip("transformers")
    import torch

    from helpers import FakeElasticsearch, make_tokenizer
    from open_instruct_b200.decontamination import es as es_mod
    from open_instruct_b200.decontamination import index as index_cli
    from open_instruct_b200.decontamination import search as search_cli

    tok_dir = make_tokenizer(str(tmp_path / "enc"))
    tok = transformers.AutoTokenizer.from_pretrained(tok_dir)
    torch.manual_seed(0)
    transformers.LlamaModel(transformers.LlamaConfig(vocab_size=len(tok) + 8, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                                                     num_attention_heads=2, num_key_value_heads=2)).save_pretrained(tok_dir)
    leaked = "What is the sum of the first ten positive odd integers?"
    train = [{"messages": [{"role": "user", "content": "Tell me a story about a dragon who bakes bread."}, {"role": "assistant", "content": "Once"}]},
             {"messages": [{"role": "user", "content": leaked}, {"role": "assistant", "content": "100"}]},
             {"messages": [{"role": "user", "content": "Summarise Hamlet in two sentences."}, {"role": "assistant", "content": "..."}]}]
    tp, ep = tmp_path / "train.jsonl", tmp_path / "eval.jsonl"
    tp.write_text("".join(json.dumps(r) + "\n" for r in train))
    ep.write_text(json.dumps({"text": leaked}) + "\n")
    fake = FakeElasticsearch()
    try:
        added = index_cli.main(["--es_url", fake.url, "--dataset", str(tp), "--index_type", "vector", "--model", tok_dir])
        index = es_mod.index_name_for(str(tp), "vector")
        assert added == {index: 3} and fake.indices[index]["dims"] == 32
        v = fake.indices[index]["docs"][0]["_source"]["vector"]
        assert abs(sum(x * x for x in v) - 1.0) < 1e-4
        rep = search_cli.main(["--es_url", fake.url, "--train", str(tp), "--eval", str(ep), "--field", "text", "--index_type", "vector",
                               "--model", tok_dir, "--threshold", "0.999", "--output_dir", str(tmp_path / "out")])
        assert rep["train_contaminated"] == [1] and rep["eval_contaminated"] == 1
        assert rep["matches"][0]["results"][0]["original_id"] == 1 and abs(rep["matches"][0]["results"][0]["score"] - 1.0) < 1e-4
        emb = es_mod.Embedder(tok_dir, max_batch_tokens=4)
        assert emb(["a much longer text than four tokens allow for sure", "hi"])[0] is None     # too long for the budget: skipped
    finally:
        fake.close()
