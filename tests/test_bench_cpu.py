"""The reference arm of bench.py on the host: it needs no GPU, so its JSON line can be checked here."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(
    not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "diff_gpt")),
    reason="the unmodified reference is not installed under baseline/_ref (it is not part of the history)",
)
def test_reference_arm_prints_one_line_of_the_agreed_shape():
    """`bench.py --impl reference` times the unmodified reference's Engine on the host cores and prints ONE JSON line with
    the keys the own arm prints, `impl: "reference"`, a `cpu_baseline` that names the sample it ran, and an `e2e` equal
    to its value; it does not map the CUDA library into the process."""
    out = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
        cwd=ROOT, capture_output=True, text=True, timeout=600,
    )
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, lines
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and "unavailable" not in d
    assert d["metric"] == "mc_decode_tokens_per_s" and d["unit"] == "tokens/s" and d["higher_is_better"] is True
    assert d["n_gpus"] == 1 and d["steps"] == 1 and d["warmup"] == 0 and d["value"] > 0 and d["ms_per_step"] > 0
    assert d["config"]["workload"].startswith("BASELINE config 4")
    cb = d["cpu_baseline"]
    assert cb["kind"] == "reference" and cb["cores"] >= 1 and cb["value"] == d["value"] and "trajectories" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["native_library_loaded"] is False
