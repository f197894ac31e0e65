"""The C++ host runtime (paged-KV block manager, continuous-batching scheduler, packer) under AddressSanitizer +
UndefinedBehaviorSanitizer and under ThreadSanitizer.

``ops/csrc/host/tests/host_stress.cpp`` drives one engine from a scheduling thread, three producer threads and an observer, with a
roomy and with a tiny cache (which forces preemption-by-recompute), and packs ragged examples into exactly sized buffers
from four threads.  It is compiled together with ``host_runtime.cpp`` once per sanitizer and must finish with no report.
Also a regression case for what the stress test found: a sequence that was already given its decode slot in a step must not
be preempted later in the same step."""

import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "open_instruct_b200", "ops", "csrc", "host")


@pytest.mark.parametrize("name,flags", [("asan_ubsan", ["-fsanitize=address,undefined", "-fno-omit-frame-pointer"]), ("tsan", ["-fsanitize=thread"])])
def test_host_runtime_is_clean_under_sanitizers(tmp_path, name, flags):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no C++ compiler")
    exe = str(tmp_path / f"host_stress_{name}")
    build = subprocess.run([cxx, "-std=c++17", "-O1", "-g", *flags, "-pthread", os.path.join(HOST, "host_runtime.cpp"),
                            os.path.join(HOST, "tests", "host_stress.cpp"), "-o", exe], capture_output=True, text=True, timeout=600)
    if build.returncode != 0 and "sanitizer" in (build.stderr + build.stdout).lower() and "cannot find" in build.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    env = {**os.environ, "ASAN_OPTIONS": "detect_leaks=1:halt_on_error=1", "UBSAN_OPTIONS": "halt_on_error=1:print_stacktrace=1",
           "TSAN_OPTIONS": "halt_on_error=1"}
    run = subprocess.run([exe], capture_output=True, text=True, timeout=900, env=env)
    out = run.stdout + run.stderr
    assert run.returncode == 0 and "HOST_STRESS_OK" in run.stdout, out[-4000:]
    for bad in ("ERROR: AddressSanitizer", "WARNING: ThreadSanitizer", "runtime error:", "ERROR: LeakSanitizer"):
        assert bad not in out, out[-4000:]
    assert "preemptions" in run.stdout


def test_scheduler_never_preempts_a_sequence_it_already_scheduled():
    from open_instruct_b200.rollout.engine import KV_BLOCK, _Host

    host = _Host(num_blocks=6, max_running=8)  # 6 blocks of 64 tokens: three sequences fit until they cross a block boundary
    for sid in range(3):
        host.add(sid, sid, KV_BLOCK - 2, 4 * KV_BLOCK)  # different groups: nothing shared
    produced = {sid: 0 for sid in range(3)}
    preempted_total = 0
    for _ in range(400):
        pre, dec, pmt = host.schedule()
        preempted_total += len(pmt)
        assert not (set(pre + dec) & set(pmt)), (pre, dec, pmt)      # nobody is both scheduled and taken apart
        assert len(set(pre + dec)) == len(pre + dec)
        for sid in pre + dec:
            blocks, _ = host.blocks(sid)
            assert blocks, f"sequence {sid} was scheduled without cache blocks"
            host.advance(sid, 1)
            produced[sid] += 1
            if produced[sid] >= 3 * KV_BLOCK:
                host.finish(sid)
        if all(v >= 3 * KV_BLOCK for v in produced.values()):
            break
    assert all(v >= 3 * KV_BLOCK for v in produced.values()) and preempted_total > 0
    assert host.free_blocks() == 6
