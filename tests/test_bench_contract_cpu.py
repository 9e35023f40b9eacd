"""The benchmark's CPU-side contract: the reference arm (the oracle port on the host cores) prints one
JSON line with the agreed keys, and the product arm refuses to run without a GPU instead of falling
back to anything."""

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.timeout(600)
def test_reference_arm_prints_the_contract_line():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "c1",
                        "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=550, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "moe_layer_tokens_per_s"
    assert line["unit"] == "tokens/s" and line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["steps"] == 2 and line["warmup"] == 1 and line["value"] > 0 and line["ms_per_step"] > 0
    assert line["config"]["workload"].startswith("c1")
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}


@pytest.mark.timeout(300)
def test_product_arm_needs_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--steps", "1", "--warmup", "1", "--sub", "none"],
                       capture_output=True, text=True, timeout=280, cwd=str(ROOT))
    assert r.returncode != 0
    assert "no fallback" in (r.stderr + r.stdout) or "CUDA" in (r.stderr + r.stdout)


def test_operator_headers_import_without_torch():
    code = ("import sys; from b12x_b200.moe import fused_moe, ep_moe; "
            "assert 'torch' not in sys.modules; print(fused_moe.META.qualname, ep_moe.META.qualname, "
            "len(fused_moe.META.entry_points))")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-1000:]
    assert r.stdout.split()[:2] == ["moe.fused_moe", "moe.ep_moe"]
