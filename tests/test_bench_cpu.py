"""Host side of `bench.py`: configuration selection, the flags it hands to the real CLI, the JSON line."""
import importlib.util
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("name,n,sep,seq", [("B", 8, 1, 4096), ("C", 8, 8, 32768), ("C", 2, 2, 8192), ("D", 8, 8, 4096),
                                            ("E", 8, 2, 4096), ("E", 1, 1, 4096), ("S", 1, 1, 4096)])
def test_config_selection_and_flags_parse(name, n, sep, seq, tmp_path):
    from train_large_model_from_scratch_b200.training import build_config, parse_args
    b = _load_bench()
    b._select_config(name, n)
    assert (b.SEP_SIZE, b.SEQ_LEN) == (sep, seq)
    cfg = build_config(parse_args(b._flags(n, 10, str(tmp_path))))
    assert cfg.parallel.sep_size == sep and cfg.train.seq_len == seq
    assert cfg.train.total_batch_size == seq * b.MICRO_BATCH * b.GRAD_ACCUM * (n // sep)
    assert cfg.model.block_size >= seq and cfg.model.use_moe == (name == "D")


def test_result_line_has_the_contract_keys():
    b = _load_bench()
    out = b._result("ours", 2, 4, 3, 800.0, 131072, {"sm_mhz": 1500.0, "sm_max_mhz": 1965.0, "reasons": []},
                    {"gpu_launches": 10, "e2e": {"value": 1.0, "unit": "tokens/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 4}})
    for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
              "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches"):
        assert k in out, k
    assert out["ms_per_step"] == 200.0 and abs(out["value"] - 131072 / 0.2) < 1e-6
    assert out["n_gpus"] == 2 and out["higher_is_better"] is True and out["scaling"] == "weak"
    json.dumps(out)


def test_reference_arm_reports_unavailable_without_cuda():
    import torch
    if torch.cuda.is_available():
        pytest.skip("needs a box without CUDA")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-500:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line


def test_extra_configurations_run_as_child_jobs_and_failures_stay_contained(tmp_path, monkeypatch):
    """`run_extras` starts one child job per extra configuration with the launcher's rank variables removed, keeps
    the keys of the child's JSON line, and reports a child that fails or hangs as `unavailable` without raising."""
    bench = _load_bench()
    fake = tmp_path / "fake_bench.py"
    fake.write_text(
        "import json, os, sys, time\n"
        "cfg = sys.argv[sys.argv.index('--config') + 1]\n"
        "assert 'RANK' not in os.environ and os.environ.get('MASTER_PORT') != '1234', 'launcher variables leaked'\n"
        "assert '--no-extras' in sys.argv\n"
        "if cfg == 'C':\n"
        "    mode = os.environ.get('FAKE_MODE', 'ok')\n"
        "    if mode == 'fail':\n"
        "        print('boom', file=sys.stderr); sys.exit(3)\n"
        "    if mode == 'hang':\n"
        "        time.sleep(60)\n"
        "print('noise before the result')\n"
        "print(json.dumps({'metric': 'm', 'value': 1.5, 'unit': 'tokens/s', 'ms_per_step': 2.0, 'steps': 20,\n"
        "                  'config': {'model': cfg}, 'e2e': {'value': 1.25}, 'clocks': {'sm_mhz': 1500}}))\n")
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    os.rename(fake, tmp_path / "bench.py")
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("MASTER_PORT", "1234")

    class Args:
        gpus, steps, warmup, impl, ref_compile, moe_fallback, extra_timeout = 1, 50, 3, "ours", 1, 1, 20

    out = bench.run_extras(Args)
    assert set(out) == {k for k, _ in bench.EXTRAS}
    assert out["moe"]["value"] == 1.5 and out["moe"]["config"]["model"] == "D" and out["moe"]["steps"] == 20
    assert out["ulysses"]["e2e"]["value"] == 1.25 and "wall_s" in out["ulysses"]

    monkeypatch.setenv("FAKE_MODE", "fail")
    out = bench.run_extras(Args)
    assert "unavailable" in out["ulysses"] and "exit code 3" in out["ulysses"]["unavailable"] and "boom" in out["ulysses"]["unavailable"]
    assert out["moe"]["value"] == 1.5

    monkeypatch.setenv("FAKE_MODE", "hang")
    Args.extra_timeout = 2
    out = bench.run_extras(Args)
    assert "no result within 2 s" in out["ulysses"]["unavailable"] and out["moe"]["value"] == 1.5


def test_fused_path_rooflines_count_the_bytes_that_leave_a_gpu():
    """benchmarks/fused_paths.py: FLOPs and NVLink bytes per call of the fused exchange kernels, from the configuration."""
    sys.path.insert(0, ROOT)
    try:
        from benchmarks import fused_paths
    finally:
        sys.path.remove(ROOT)
    bench = _load_bench()
    bench._select_config("C", 8)                        # Ulysses over 8 ranks, 4096 tokens per rank, micro-batch 1
    roofs = {label: (flops, nbytes) for _, label, flops, nbytes in fused_paths._rooflines(bench, 8)}
    qkv = roofs["QKV GEMM + RoPE + seq->head scatter"]
    assert qkv[0] == 2.0 * 4096 * 2048 * 1024 and qkv[1] == 4096 * 2048 * 2 * 7 / 8
    o = roofs["attention forward + head->seq scatter of O"]
    assert o[0] == 4.0 * 1 * 2 * 32768 * 32768 * 64 / 2 and o[1] == 32768 * 2 * 64 * 2 * 7 / 8
    bench = _load_bench()
    bench._select_config("D", 8)
    moe = fused_paths._rooflines(bench, 8)
    assert len(moe) == 2 and all(nbytes == 4 * 4096 // 8 * 2 * 1024 * 2 * 7 / 8 for _, _, _, nbytes in moe)
