"""The flag protocols of the peer-memory kernels (`csrc/flag_protocol.h`: epoch exchange, parity slots,
"parameters ready" words) run as a host program: one thread per rank, randomised arrival orders and delays, the
same template code the CUDA kernels instantiate with system-scope loads and stores. This is the stand-in for a
race detector on the device side: the properties (nobody passes an exchange early, no slot is overwritten before
it has been read, a consumer that sees the ready words sees every store) are checked on every round, including
across the wrap of the 32-bit epoch counters."""
import os
import shutil
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def binary():
    if shutil.which("g++") is None:
        pytest.skip("no host compiler")
    out = os.path.join(tempfile.mkdtemp(prefix="tlm_proto_"), "flag_protocol_host_test")
    cmd = ["g++", "-O2", "-std=c++17", "-pthread", "-I", os.path.join(ROOT, "train_large_model_from_scratch_b200", "csrc"),
           "-o", out, os.path.join(ROOT, "tests", "flag_protocol_host_test.cpp")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return out


@pytest.mark.parametrize("ranks,rounds,seed,start", [(2, 1500, 1, 0), (4, 800, 2, 0), (8, 400, 3, 0),
                                                     (8, 400, 4, 2147483500), (3, 600, 5, -300)])
def test_protocol_properties_hold_under_random_arrival_orders(binary, ranks, rounds, seed, start):
    r = subprocess.run([binary, str(ranks), str(rounds), str(seed), str(start)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.startswith("ok:")


def test_attention_block_order_is_a_heavy_first_bijection():
    """`csrc/tile_order.h` (the decode the attention kernels apply to their linear block id) as a host program."""
    if shutil.which("g++") is None:
        pytest.skip("no host compiler")
    out = os.path.join(tempfile.mkdtemp(prefix="tlm_order_"), "tile_order_host_test")
    cmd = ["g++", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "train_large_model_from_scratch_b200", "csrc"),
           "-o", out, os.path.join(ROOT, "tests", "tile_order_host_test.cpp")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([out], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stdout + r.stderr
