"""The fp32 oracles of this repo against the UNMODIFIED reference engine (``baseline/_ref``, its torch
backend on the CPU): every device tolerance in the GPU tests is relative to these oracles, so their
agreement with the reference is pinned here.  Skipped when the reference is not installed."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"

pytestmark = pytest.mark.skipif(not (REF / "engine_api.py").exists(), reason="the reference is not installed under baseline/_ref")


def _run(which: str) -> dict:
    r = subprocess.run([sys.executable, str(ROOT / "tests" / "ref_cross.py"), which], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])


def test_qwen35_oracle_matches_the_reference_engine():
    """Config 1 of the benchmark plan: prompt 64, 24 teacher-forced decode steps through the reference's
    paged engine (bf16 weights, int8 KV); the oracle computes in fp32 from the same bf16 weights."""
    d = _run("qwen35")
    assert d["worst_abs"] < 0.08 * max(1.0, d["scale"]), d     # the reference computes in bf16
    assert d["argmax_agree"] >= d["steps"] - 2, d


def test_qwen4_oracle_matches_the_reference_model():
    """fp32 on both sides: decode agrees to rounding; prefill rows differ only where the reference's
    ``relu`` block scores tie (few visible blocks), never at the sampling row."""
    d = _run("qwen4")
    assert d["decode_worst_abs"] < 1e-3, d
    assert d["prefill_last_row_abs"] < 1e-3, d
