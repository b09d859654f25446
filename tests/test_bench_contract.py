"""bench.py's output contract: one JSON line with the keys the measurement protocol names.  CPU: the reference arm (the
oracle port on the host cores) and the workload table; GPU: the smallest workload through the native arm."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
             "dtype", "data", "config", "e2e"}


def run_bench(*flags, timeout=600):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *flags], capture_output=True, text=True, timeout=timeout, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_line():
    d = run_bench("--impl", "reference", "--workload", "tiny", "--steps", "1", "--warmup", "0")
    assert BASE_KEYS <= set(d) and d["impl"] == "reference"
    assert d["metric"] == "fused_block_tflops" and d["unit"] == "TFLOP/s" and d["value"] > 0
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert d["config"]["workload"] == "tiny" and "model" not in d["config"]


@pytest.mark.parametrize("workload,metric", [("llama3_8b_swiglu_ffn_m64", "fused_block_tflops"), ("llama3_8b_vanilla_decode_m16_p1024", "fused_block_tflops"),
                                             ("llama3_8b_kv_evict_b4_l4096_k1024", "kv_evict_gbs"), ("rmsnorm_32768x4096", "rmsnorm_gbs")])
def test_reference_arm_covers_every_kind_of_workload(workload, metric):
    d = run_bench("--impl", "reference", "--workload", workload, "--steps", "1", "--warmup", "0")
    assert d["impl"] == "reference" and d["metric"] == metric and d["value"] > 0
    assert d["config"]["workload"] == workload and d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["sample"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0


def test_both_arms_print_the_same_config():
    sys.path.insert(0, ROOT)
    import bench
    for name, w in bench.WORKLOADS.items():
        c = bench.workload_config(name, w)
        assert c["workload"] == name and "model" not in c and "recorded_ms" not in c


def test_workload_table():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.DEFAULT in bench.WORKLOADS and bench.WORKLOADS[bench.DEFAULT].get("kind") is None
    kinds = {w.get("kind", "attention") for w in bench.WORKLOADS.values()}
    assert kinds == {"attention", "ffn", "evict", "decode", "rmsnorm"}
    for name, w in bench.WORKLOADS.items():
        if w.get("kind") is None:
            assert w["Hq"] % w["Hkv"] == 0 and w["D"] in (64, 128) and w["N"] % 8 == 0, name
            assert w["variant"] in ("vanilla", "prenorm", "qknorm", "roco", "keyformer"), name
        elif w["kind"] == "evict":
            assert w["topk"] * w.get("group", 1) + w["recent"] > 0 and w["L"] <= 262144, name
        elif w["kind"] == "decode":
            assert w["H"] * w["D"] == w["N"] and w["M"] <= 16, name   # the reference's points are MHA with N = H * D


@pytest.mark.gpu
def test_native_arm_line_on_the_smallest_workload():
    d = run_bench("--workload", "tiny", "--steps", "3", "--warmup", "3", "--no-cpu-baseline")
    assert BASE_KEYS | {"roofline", "clocks", "gpu_launches", "timed_region_s", "burst", "passes_per_step"} <= set(d)
    assert d["e2e"]["api"].startswith("generated-module forward(")
    assert d["gpu_launches"] > 0 and d["value"] > 0 and d["e2e"]["value"] > 0
    assert d["e2e"]["h2d_bytes_per_step"] > 0 and d["e2e"]["d2h_bytes_per_step"] > 0
    r = d["roofline"]
    assert r["bound"] in ("hbm", "tensor") and r["peak"] > 0 and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    assert d["warmup"] >= 3 and d["n_gpus"] == 1
