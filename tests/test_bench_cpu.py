"""The legs of bench.py that need no GPU: the reference arm (CPU oracle port of the train step,
with the reference's shipped `--cpu` codec as a side record) and the tokenizer mode.  Each must
print exactly one JSON line on stdout."""
import json
import os
import subprocess
import sys

from conftest import ROOT


def _run(*args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                       timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, r.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_prints_one_line_with_the_contract_keys():
    d = _run("--impl", "reference", "--config", "c0", "--steps", "2", "--warmup", "1")
    assert d["impl"] == "reference" and d["unit"] == "symbols/s" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"] == {"value": d["value"], "unit": "symbols/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and d["higher_is_better"] is True
    side = d["shipped_cpu_codec"]          # None where oracle/_ref was never built
    if side is not None:
        assert side["round_trip_exact"] and abs(side["ratio"] - 1.0) < 1e-3 and side["cores"] == 1


def test_tokenizer_mode_round_trips_and_matches_the_reference_tool():
    d = _run("--mode", "words", "--steps", "1")
    assert d["round_trip_exact"] and d["value"] > 0 and d["config"]["entries"] > 256
    if d["cpu_baseline"] is not None:      # oracle/_ref/preprocess_ref present
        assert d["cpu_baseline"]["same_output"] and d["cpu_baseline"]["kind"] == "reference"
