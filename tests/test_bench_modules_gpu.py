"""The measurement modules named in profiles/ stay runnable: tiny shapes, one JSON line per
record, sane fields."""
import json
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def run_module(mod, *args):
    res = subprocess.run([sys.executable, "-m", mod, *args], capture_output=True, text=True,
                         timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    return [json.loads(line) for line in res.stdout.splitlines() if line.startswith("{")]


def test_prefill_bench_small():
    recs = run_module("sparser_faster_llms_b200.prefill_bench", "--tokens", "512", "--d-model",
                      "512", "--d-ff", "2048", "--reps", "2", "--warmup", "1")
    assert [r["mode"] for r in recs] == ["gather", "routed", "dense_all", "cublas"]
    by = {r["mode"]: r for r in recs}
    assert by["routed"]["rel_l2_vs_dense_formula"] < 1.5e-2
    assert by["dense_all"]["rel_l2_vs_dense_formula"] < 1.5e-2
    assert by["routed"]["dense_rows"] > 0 and by["routed"]["wait_status"] == [0, 0]
    assert all(r["ms"] > 0 for r in recs)


def test_sweep_bench_small():
    recs = run_module("sparser_faster_llms_b200.sweep_bench", "--d-model", "512", "--d-ff", "2048",
                      "--tokens", "4,256", "--densities", "0.02,0.3", "--skews", "0")
    assert len(recs) == 4
    for r in recs:
        assert r["us"]["sparse"] > 0 and r["us"]["cublas"] > 0
        if r["tokens"] >= 128:
            assert r["rel_l2_vs_cublas"]["dense_all"] < 2e-2
        if r["density"] <= 0.05:
            assert r["rel_l2_vs_cublas"]["sparse"] < 2e-2 and r["best_exact_path"] is not None
        else:  # 30 %: the 31-entry slabs overflow, the gather path is lossy by design
            assert r["overflowed_rows"] > 0


def test_training_bench_small():
    recs = run_module("sparser_faster_llms_b200.training_bench", "--batch", "2", "--seq", "256",
                      "--d-model", "512", "--d-ff", "1024", "--density", "0.03", "--reps", "3",
                      "--warmup", "4")  # the warm-up also loads the tail GEMMs' library kernels
    assert len(recs) == 1
    r = recs[0]
    assert r["tokens"] == 512 and r["l0_per_token"] > 0
    assert r["sparse"]["forward_backward_ms"] > r["sparse"]["forward_ms"] > 0
    assert r["sparse"]["dead_neuron_bookkeeping_ms"] > 0 and r["dense"]["forward_ms"] > 0


def test_decode_model_cli_small():
    recs = run_module("sparser_faster_llms_b200.decode_model", "--batch", "2", "--prompt", "32",
                      "--generate", "24", "--layers", "2")
    assert len(recs) == 1
    r = recs[0]
    assert r["twell"]["ms_per_token"] > 0 and r["dense"]["ms_per_token"] > 0
