"""bench.py's reference arm runs on the host cores alone: one JSON line with the contract's keys."""
import json
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_json_line_on_cpu():
    res = subprocess.run([sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--steps",
                          "3", "--warmup", "1"], capture_output=True, text=True, timeout=600,
                         cwd=REPO)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and rec["higher_is_better"] is True
    assert rec["metric"] == "sparse_ffn_decode_tokens_per_s" and rec["unit"] == "tokens/s"
    assert rec["value"] > 0 and rec["n_gpus"] == 1 and rec["steps"] == 3 and rec["warmup"] == 1
    assert rec["cpu_baseline"]["kind"] in ("port", "reference")
    assert rec["cpu_baseline"]["cores"] >= 1 and rec["cpu_baseline"]["value"] == rec["value"]
    assert rec["e2e"] == {"value": rec["value"], "unit": rec["unit"], "h2d_bytes_per_step": 0,
                          "d2h_bytes_per_step": 0}
    assert "workload" in rec["config"]


def test_reference_arm_on_other_ranks_exits_quietly():
    import os
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    res = subprocess.run([sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--gpus",
                          "2", "--steps", "3", "--warmup", "1"], capture_output=True, text=True,
                         timeout=600, cwd=REPO, env=env)
    assert res.returncode == 0
    assert not [l for l in res.stdout.splitlines() if l.startswith("{")]
