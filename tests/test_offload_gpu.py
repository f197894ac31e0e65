"""Optimizer-state offload on the GPU: streamed AdamW over pinned host state equals the resident optimizer."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_offloaded_optimizer_matches_resident_on_gpu():
    from open_instruct_b200.data.collate import to_device
    from open_instruct_b200.data.synthetic import sft_step_batches
    from open_instruct_b200.learner import Learner, LearnerConfig
    from open_instruct_b200.models import get_spec

    spec = get_spec("tiny128")
    dev = torch.device("cuda:0")
    outs = []
    for offload in (False, True):
        cfg = LearnerConfig(ops="fused", comm="none", learning_rate=1e-3, weight_decay=0.1, max_grad_norm=1.0, total_steps=10, seed=1,
                            offload_optimizer=offload)
        L = Learner(spec, cfg, device=dev)
        if offload:
            L.opt.offload_chunk = 100_000  # several chunks, both staging sets in use
            assert L.opt.master.device.type == "cpu" and L.opt.master.is_pinned()
        for s in range(3):
            mbs = [to_device(b, dev) for b in sft_step_batches(2, 256, spec.vocab_size, seed=s)]
            out = L.sft_step(mbs)
        torch.cuda.synchronize()
        outs.append((L.model.flat.detach().float().cpu(), L.opt.m.cpu().clone(), float(out["loss"])))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1]) and outs[0][2] == outs[1][2]


def test_learner_state_parks_on_the_host_between_steps():
    from open_instruct_b200.data.collate import to_device
    from open_instruct_b200.data.synthetic import sft_step_batches
    from open_instruct_b200.learner import Learner, LearnerConfig
    from open_instruct_b200.models import get_spec

    spec = get_spec("tiny128")
    dev = torch.device("cuda:0")
    mk = lambda: Learner(spec, LearnerConfig(ops="fused", comm="none", learning_rate=1e-3, total_steps=10, seed=4), device=dev)
    a, b = mk(), mk()
    for s in range(3):
        mbs = [to_device(x, dev) for x in sft_step_batches(2, 256, spec.vocab_size, seed=s)]
        a.sft_step(mbs)
        freed = b.offload_to_cpu()
        assert freed > 0 and not b.opt.master.is_cuda and b.model.main_grad is None
        b.backload_to_gpu()
        assert b.opt.master.is_cuda
        b.sft_step(mbs)
    torch.cuda.synchronize()
    assert torch.equal(a.model.flat.detach(), b.model.flat.detach())
