"""The benchmark's reference arm runs on the host only: one short invocation checks that it
prints a single JSON line with the keys the benchmark contract names."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    from oracle.oracle import Reference
    if not Reference.available():
        pytest.skip("reference loops not built (oracle/build.py)")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "img/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["steps"] == 1 and d["n_gpus"] == 1
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["value"] == d["value"] and d["e2e"]["h2d_bytes_per_step"] == 0
    assert "workload" in d["config"]


def test_case_names_parse():
    """`bench.py --case` names: <op>_<dtype>_<H>x<W>x<C>."""
    for name in ("fprop_f32_56x56x96", "wgrad2_bf16_224x224x64", "ln_bf16_28x28x192", "pw_f32_224x224x64"):
        op, tag, shape = name.split("_")
        assert tag in ("f32", "bf16") and len(shape.split("x")) == 3 and op
