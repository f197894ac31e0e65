"""Worker for the multi-rank optimizer tests (launched under torchrun by the test files).

Every rank trains the same tiny model for a few steps on its own synthetic micro-batches with the
requested communication back ends and checks that they agree with each other and, on rank 0,
with a single-process run over the union of the data.
"""

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from open_instruct_b200.data.collate import to_device  # noqa: E402
from open_instruct_b200.data.synthetic import sft_step_batches  # noqa: E402
from open_instruct_b200.learner import Learner, LearnerConfig  # noqa: E402
from open_instruct_b200.models import get_spec  # noqa: E402
from open_instruct_b200.parallel import dist as pdist  # noqa: E402


def run(learner, rank_ids, steps, device, spec, seq):
    out = []
    for s in range(steps):
        mbs = []
        for r in rank_ids:
            mbs += [to_device(b, device) for b in sft_step_batches(2, seq, spec.vocab_size, seed=100 * s + r)]
        out.append(learner.sft_step(mbs))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--comms", default="nccl")
    ap.add_argument("--steps", type=int, default=3)
    args = ap.parse_args()
    rank, world, device = pdist.init_distributed()
    if args.device == "cpu":
        device = torch.device("cpu")
    cuda = device.type == "cuda"
    spec = get_spec("tiny128" if cuda else "tiny")
    seq = 384 if cuda else 96
    base = dict(learning_rate=1e-3, lr_scheduler_type="constant", max_grad_norm=1.0, weight_decay=0.01, seed=7,
                ops="fused" if cuda else "ref")
    flats = {}
    for name in args.comms.split(","):
        comm = name.split("+")[0]
        # "fused+overlap": the gradient exchange starts under the last micro-batch's backward (opt-in, read when the optimizer is built)
        os.environ["B200_OVERLAP_GRADS"] = "1" if name.endswith("+overlap") else "0"
        lr_ = Learner(spec, LearnerConfig(comm=comm, **base), device=device)
        os.environ.pop("B200_OVERLAP_GRADS", None)
        outs = run(lr_, [rank], args.steps, device, spec, seq)
        if cuda:
            from open_instruct_b200.ops import lib

            lib.check_status()
        flats[name] = (lr_.model.flat.detach().float().cpu().clone(), float(outs[-1]["grad_norm"].item()))
        del lr_
    names = list(flats)
    for other in names[1:]:
        a, b = flats[names[0]][0], flats[other][0]
        err = (a - b).abs().max().item()
        assert err < (2e-2 if cuda else 1e-6), f"{names[0]} vs {other}: max param diff {err}"
        assert abs(flats[names[0]][1] - flats[other][1]) < 1e-3 * max(1.0, flats[names[0]][1])
    # every rank holds the same parameters
    mine = flats[names[0]][0].to(device)
    ref = mine.clone()
    torch.distributed.broadcast(ref, src=0)
    assert torch.equal(mine, ref), "ranks diverged"
    if rank == 0 and not cuda:
        # single-process oracle over the union of all ranks' micro-batches
        single = Learner(spec, LearnerConfig(comm="none", **base), device=device, group=pdist.SOLO)
        outs = run(single, list(range(world)), args.steps, device, spec, seq)
        n = single.model.layout.total
        err = (single.model.flat.detach()[:n] - flats[names[0]][0][:n]).abs().max().item()
        assert err < 1e-5, f"multi-rank vs single-process: {err}"
    if cuda and "fused" in names and world == 2:
        # A peer that never arrives: rank 0 runs one device barrier with a 50 ms limit while rank 1 skips that call.  The
        # kernel must return by itself, leave ST_TIMEOUT_PEER in the status word, and the host check must raise; nothing
        # hangs or faults, and the context stays usable.
        from open_instruct_b200.ops import lib
        from open_instruct_b200.parallel.symm import SymmetricState

        st = SymmetricState(4096, device, peer_timeout_ms=50)
        # the small-vector all-reduce of the logging path, three in a row (the exchange slots alternate), against NCCL
        from open_instruct_b200.utils.common import MetricsTracker

        for k in range(3):
            v = torch.arange(100, device=device, dtype=torch.float32) * (rank + 1) + k
            want = v.clone()
            torch.distributed.all_reduce(want)
            assert torch.equal(st.allreduce_vector_(v), want)
        mt = MetricsTracker(device=device)
        mt["loss"] = float(rank + 1)
        mt.reduce_(average=True)  # goes through the same kernel (a symmetric state exists for the default group)
        assert abs(mt.get_metrics_list()["loss"] - 1.5) < 1e-6
        st.barrier()  # both ranks: a normal barrier passes
        torch.cuda.synchronize()
        lib.check_status()
        if rank == 0:
            st.barrier()
            torch.cuda.synchronize()
            assert int(lib.status_word(device).item()) == 5, "expected ST_TIMEOUT_PEER"
            try:
                lib.check_status()
                raise AssertionError("check_status did not raise after a timed-out peer wait")
            except lib.KernelError:
                pass
            assert int(lib.status_word(device).item()) == 0  # cleared by the raise; the context is still usable
            x = torch.ones(8, device=device)
            assert float((x * 2).sum().item()) == 16.0
        else:
            st._barrier_epoch += 1  # keep the epoch counters of the two ranks aligned
    pdist.barrier()
    if rank == 0:
        print("ZERO_WORKER_OK", {k: v[1] for k, v in flats.items()})
    pdist.destroy()


if __name__ == "__main__":
    main()
