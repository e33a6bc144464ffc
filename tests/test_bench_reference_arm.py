"""`bench.py --impl reference` on the CPU: the line the contract asks for, on the tiny
configuration (the oracle port timed on the host cores; no GPU involved)."""
import json
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent


def _run(*extra):
    out = subprocess.run([sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--workload",
                          "tiny", *extra], capture_output=True, text=True, timeout=600, cwd=REPO)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_prints_one_contract_line():
    d = _run("--steps", "3", "--warmup", "1", "--cpu-sample-tokens", "256")
    assert d["impl"] == "reference" and d["metric"] == "moe_layer_tokens_per_s"
    assert d["unit"] == "tokens/s" and d["higher_is_better"] is True and d["n_gpus"] == 1
    assert d["steps"] == 3 and d["warmup"] == 1            # K timed passes after W warm-up passes
    assert d["value"] > 0 and abs(d["value"] - 256 / (d["ms_per_step"] * 1e-3)) < 1e-6 * d["value"]
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"]
    assert "256 tokens" in cb["sample"] and "3 timed passes" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}
    assert d["config"]["workload"].startswith("tiny:") and d["vs_baseline"] is None
    assert "fit the 126 MB L2" in d["config"]["l2"]        # the tiny case is the one that fits


def test_other_ranks_of_the_reference_arm_do_nothing(monkeypatch):
    monkeypatch.setenv("RANK", "1")
    out = subprocess.run([sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--workload", "tiny"], capture_output=True, text=True, timeout=120, cwd=REPO)
    assert out.returncode == 0 and not [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
