"""The sweep harness (trinity_b200/sweep.py) against the reference's harnesses (benchmark/*_benchmark.py): tensor
tables and zero lists from fixtures recorded off the reference's own classes, IR-file parsing, candidate selection, the
result-record schema (benchmark/vanilla_llama_benchmark.py:388-401); on a GPU, a sweep over the recorded IR candidates
of every family."""
import json
import math
import os

import pytest

from trinity_b200 import sweep


def test_tensor_tables_match_the_reference_harnesses(golden_dir):
    tables = json.load(open(os.path.join(golden_dir, "sweep_tables.json")))
    assert len(tables) == 12
    for t in tables:
        mine = sweep.tensor_shapes(t["family"], t["config"])
        assert {k: list(v) for k, v in mine.items()} == t["shapes"], t["harness"]
        zero = sweep._FFN_ZERO if t["family"] in sweep.FFN_FAMILIES else sweep._ATTN_ZERO
        assert sorted(k for k in mine if k in zero) == t["zeros"], t["harness"]
        assert t["dtype"] == "torch.float16"
        scale = 0.001 if t["family"] in sweep.FFN_FAMILIES else 0.01
        assert t["input_abs_max"] == pytest.approx(scale, rel=1e-2)


def test_parse_ir_file_and_select(tmp_path):
    p = tmp_path / "ir.txt"
    p.write_text("# header\n0: (seq a b)\n\n3: (ploop 0 N tile_n n dummydata)\nnot an id: (x)\n7:(store (output O2) x y)\n12 : (z)\nplain line\n")
    got = sweep.parse_ir_file(str(p))
    assert got == [(0, "(seq a b)"), (7, "(store (output O2) x y)"), (12, "(z)")]
    assert sweep.select(got, 5, None) == got[1:]
    assert sweep.select(got, 0, 2) == got[:2]
    assert sweep.select(got, None, 1) == got
    assert sweep.select(got, 100, 5) == []


def test_record_schema_and_ranking():
    cfg = {"M": 16, "N": 4096}
    rows = [sweep.record(1, "(a)", 0.5, cfg), sweep.record(2, "(b)", math.inf, cfg, "boom"), sweep.record(3, "(c)", 0.25, cfg),
            {"tensor_config": cfg, "error": "whole configuration failed", "results": []}]
    assert list(rows[0]) == ["ir_id", "ir_expression", "execution_time_ms", "tensor_config", "error"]
    assert [r["ir_id"] for r in sweep.best(rows, 5)] == [3, 1]
    back = json.loads(json.dumps(rows))      # Python's json writes and reads Infinity, as the reference's files hold it
    assert back[1]["execution_time_ms"] == math.inf and back[1]["error"] == "boom"
    assert "2 valid" in sweep.report(rows, 1) and "IR 3" in sweep.report(rows, 1)


def test_unknown_family_and_missing_device():
    import torch
    with pytest.raises(ValueError):
        sweep.tensor_shapes("mamba", {"M": 1, "N": 8})
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            sweep.BlockSweep("vanilla", {"M": 16, "D": 128, "N": 4096, "P": 1024, "H": 32})


@pytest.mark.gpu
def test_sweep_over_recorded_candidates(golden_dir, tmp_path):
    """Every recorded candidate of every family runs under the harness protocol at its own configuration, binds the
    tensors its parameter list names, and lands in the result file with a finite time and no error; a candidate that
    names a tensor outside the table becomes an error row."""
    import torch
    from trinity_b200 import ops
    fixtures = json.load(open(os.path.join(golden_dir, "ir_modules.json")))
    for family in sweep.FAMILIES:
        mine = [f for f in fixtures if f["family"] == family]
        assert mine, family
        cfg = mine[0]["constants"]
        ir = tmp_path / f"{family}.txt"
        ir.write_text("".join(f"{f['ir_id']}: {f['ir']}\n" for f in mine) + "99999: (store (output Z) (load (input X) (index fulltile)) (index fulltile))\n")
        out = tmp_path / f"{family}.json"
        rc = sweep.main(["--family", family, "--ir", str(ir), "--configs", _write(tmp_path / f"{family}_cfg.json", [cfg]),
                         "--output", str(out), "--all"])
        assert rc == 0
        ops.device_status()
        rows = json.load(open(out))
        assert [r["ir_id"] for r in rows] == sorted(f["ir_id"] for f in mine) + [99999] or \
            [r["ir_id"] for r in rows] == [f["ir_id"] for f in mine] + [99999]
        for r in rows[:-1]:
            assert r["error"] is None and 0 < r["execution_time_ms"] < 5.0, (family, r["ir_id"], r["error"])
            assert r["tensor_config"] == cfg
        assert rows[-1]["error"] and rows[-1]["execution_time_ms"] == math.inf
        times = [r["execution_time_ms"] for r in rows[:-1]]
        print(f"\n{family}: {min(times) * 1e3:.1f} .. {max(times) * 1e3:.1f} us over {len(times)} candidates")
    torch.cuda.synchronize()


def _write(path, obj):
    path.write_text(json.dumps(obj))
    return str(path)
