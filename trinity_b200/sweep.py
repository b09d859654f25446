"""The sweep harness around the generated modules: time every IR candidate of a file under the reference's protocol
and write the reference's result records.

Mirrors ``benchmark/*_benchmark.py`` of the reference (one script per block family and model there, one class here):

* IR files hold one candidate per line, ``<id>: <expression>``; lines without a numeric id and expressions containing
  ``dummydata`` are skipped (``benchmark/vanilla_llama_benchmark.py:141-162``).
* Tensors are fp16; inputs are ``randn.clamp(-1, 1) * scale`` (scale 0.01 for the attention families, 0.001 for the FFN
  families), outputs and intermediates are zeros (``benchmark/vanilla_llama_benchmark.py:131-138``,
  ``benchmark/ffn_llama_benchmark.py:97-110``).  A parameter a candidate lists that the table lacks is an error of that
  candidate, recorded in its row, as in the reference.
* Timing: one call outside capture, ten warm-ups on a side stream, CUDA-graph capture of ``forward(*args)``, a hundred
  replays between CUDA events (``benchmark/vanilla_llama_benchmark.py:223-301``).
* Records: ``{ir_id, ir_expression, execution_time_ms, tensor_config, error}`` written after every configuration
  (``benchmark/vanilla_llama_benchmark.py:388-401,517-546``); a failed candidate has ``execution_time_ms = inf``
  (JSON ``Infinity``, as Python's ``json`` writes it) and the exception text in ``error``.

    python -m trinity_b200.sweep --family roco --configs evaluation/llama_configs.json \\
        --ir evaluation/roco/roco_llama_cost6_kern1.txt --output roco_llama.json --all
"""
from __future__ import annotations

import argparse
import json
import math
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .codegen import convert_ir_to_triton

ATTN_FAMILIES = ("vanilla", "prenorm", "qknorm", "keyformer", "roco")
FFN_FAMILIES = ("ffn_llama", "ffn_falcon")
FAMILIES = ATTN_FAMILIES + FFN_FAMILIES

# tensors the harness creates as zeros (outputs, accumulators, scratch); every other table entry is a random input
_ATTN_ZERO = {"C", "C_exp", "C_sum", "K", "K1", "K2", "O", "O1", "Q", "Q1", "Q2", "V", "V1", "V2"}
_FFN_ZERO = {"attn_O1", "attn_O2", "attn_O3", "attn_O_norm", "FF1a", "FF1b", "FF1b_silu", "FF1", "FF2", "O_FF", "O_FF1",
             "O_FF_norm"}
# tensors zeroed again before each candidate is timed (``benchmark/vanilla_llama_benchmark.py:236-240``)
_ATTN_RESET = ("O2", "Q1", "K1", "V1", "Q2", "K2", "V2", "Q", "K", "V", "C", "C_exp", "C_sum", "C_div", "O", "O1", "X2",
               "X_norm")


def tensor_shapes(family: str, cfg: Dict[str, int]) -> Dict[str, Tuple[int, ...]]:
    """The name -> shape table of one family's harness for a ``{M, N, D, H, P}`` configuration."""
    if family not in FAMILIES:
        raise ValueError(f"unknown block family {family!r}")
    M, N = int(cfg["M"]), int(cfg["N"])
    if family in FFN_FAMILIES:
        # the Llama FFN harness takes the hidden width from P, the Falcon one uses N for every width
        F = int(cfg["P"]) if family == "ffn_llama" else N
        return {
            "O2": (M, N), "WO": (N, N), "attn_O1": (M, N), "X": (M, N), "attn_O2": (M, N), "attn_O3": (M,),
            "attn_O_norm": (M, N), "WFF1a": (N, F), "WFF1b": (N, F), "FF1a": (M, F), "FF1b": (M, F), "FF1b_silu": (M, F),
            "FF1": (M, F), "FF2": (M, N), "WFF2": (F, N), "O_FF": (M, N), "O_FF1": (M,), "O_FF_norm": (M, N),
        }
    D, H, P = int(cfg["D"]), int(cfg["H"]), int(cfg["P"])
    t = {
        "X": (M, N), "X2": (M,), "X_norm": (M, N), "WQ": (N, N), "WK": (N, N), "WV": (N, N),
        "Q": (H, M, D), "K": (H, M, D), "V": (H, M, D), "Q1": (M, N), "K1": (M, N), "V1": (M, N),
        "Q2": (M, H, D), "K2": (M, H, D), "V2": (M, H, D), "K_cache": (H, P + M, D), "V_cache": (H, P + M, D),
        "O": (H, M, D), "O1": (M, H, D), "O2": (M, N),
        "C": (H, M, P), "C_exp": (H, M, P + M), "C_div": (H, M, P + M), "C_sum": (H, M),
    }
    if family == "qknorm":
        t.update({"Q_norm": (H, M, D), "K_norm": (H, M, D)})
    elif family == "keyformer":
        t.update({"noise": (H, M, P + M), "C_perturb": (H, M, P + M), "C_exp_perturb": (H, M, P + M), "C_sum_perturb": (H, M),
                  "C_div_perturb": (H, M, P + M), "C_out": (H, P + M)})
    elif family == "roco":
        t.update({"C_out1": (H, P + M), "C_out2": (H, P + M)})
    return t


def parse_ir_file(path: str) -> List[Tuple[int, str]]:
    out: List[Tuple[int, str]] = []
    with open(path) as f:
        for line in f:
            head, sep, expr = line.strip().partition(":")
            if not sep:
                continue
            try:
                ir_id = int(head)
            except ValueError:
                continue
            expr = expr.strip()
            if expr and "dummydata" not in expr:
                out.append((ir_id, expr))
    return out


def select(expressions: List[Tuple[int, str]], start: Optional[int], num: Optional[int]) -> List[Tuple[int, str]]:
    """Candidates with id >= start, at most ``num`` of them (``None``: no limit)."""
    if start is None:
        return expressions
    picked = [(i, e) for i, e in expressions if i >= start]
    return picked[:num] if num else picked


def record(ir_id: int, expr: str, ms: float, cfg: Dict[str, int], error: Optional[str] = None) -> Dict:
    return {"ir_id": ir_id, "ir_expression": expr, "execution_time_ms": ms, "tensor_config": cfg, "error": error}


def best(records: Iterable[Dict], top_k: int) -> List[Dict]:
    ok = [r for r in records if r.get("error") is None and math.isfinite(r.get("execution_time_ms", math.inf))]
    return sorted(ok, key=lambda r: r["execution_time_ms"])[:top_k]


class BlockSweep:
    """One family at one tensor configuration: owns the tensors, times candidates."""

    def __init__(self, family: str, tensor_config: Dict[str, int], device: Optional[torch.device] = None, seed: int = 42):
        if not torch.cuda.is_available():
            raise RuntimeError("the sweep times CUDA kernels: no CUDA device is visible")
        self.family = family
        self.tensor_config = dict(tensor_config)
        self.shapes = tensor_shapes(family, tensor_config)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.seed = seed
        self.tensors: Dict[str, torch.Tensor] = {}
        self.create_test_tensors()

    def create_test_tensors(self) -> None:
        ffn = self.family in FFN_FAMILIES
        zero, scale = (_FFN_ZERO, 0.001) if ffn else (_ATTN_ZERO, 0.01)
        gen = torch.Generator(device=self.device)
        gen.manual_seed(self.seed)
        self.tensors = {}
        for name, shape in self.shapes.items():
            if name in zero:
                self.tensors[name] = torch.zeros(shape, dtype=torch.float16, device=self.device)
            else:
                r = torch.randn(shape, dtype=torch.float16, device=self.device, generator=gen)
                self.tensors[name] = r.clamp_(-1, 1).mul_(scale)

    def load(self, ir_expr: str) -> Dict:
        """Generate the module for one candidate and execute its text, as the harness's import of a temp file does."""
        ns: Dict = {}
        exec(compile(convert_ir_to_triton(ir_expr, None, self.tensor_config), "<generated module>", "exec"), ns)
        if "forward" not in ns:
            raise RuntimeError("generated module defines no forward")
        return ns

    def arguments(self, module: Dict) -> List[torch.Tensor]:
        args = []
        for name in module["TENSOR_PARAMS"]:
            if name not in self.tensors:
                if name not in self.shapes:
                    raise ValueError(f"Unknown tensor parameter: {name}")
                self.tensors[name] = torch.zeros(self.shapes[name], dtype=torch.float16, device=self.device)
            args.append(self.tensors[name])
        return args

    def time_module(self, module: Dict, warmup_runs: int = 10, benchmark_runs: int = 100) -> float:
        if self.family in ATTN_FAMILIES:
            for name in _ATTN_RESET:
                if name in self.tensors:
                    self.tensors[name].zero_()
        args = self.arguments(module)
        forward = module["forward"]
        with torch.cuda.device(self.device):
            stream = torch.cuda.Stream(self.device)
            forward(*args)  # outside capture: sizes the workspace, creates per-device state
            torch.cuda.synchronize(self.device)
            with torch.cuda.stream(stream):
                for _ in range(warmup_runs):
                    forward(*args)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                with torch.cuda.graph(graph, stream=stream):
                    forward(*args)
            stream.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(stream):
                t0.record()
                for _ in range(benchmark_runs):
                    graph.replay()
                t1.record()
            stream.synchronize()
        out = "O2" if self.family in ATTN_FAMILIES else ("O_FF_norm" if self.family == "ffn_falcon" else "FF2")
        if out in self.tensors and bool(torch.isnan(self.tensors[out]).any()):
            print(f"WARNING: NaN values detected in {out}")
        return t0.elapsed_time(t1) / benchmark_runs

    def run_single(self, ir_id: int, ir_expr: str, **timing) -> Dict:
        try:
            ms = self.time_module(self.load(ir_expr), **timing)
            return record(ir_id, ir_expr, ms, self.tensor_config)
        except Exception as e:  # a candidate that cannot be generated, bound or run is a row, not the end of the sweep
            return record(ir_id, ir_expr, math.inf, self.tensor_config, str(e) or type(e).__name__)

    def run_all(self, expressions: List[Tuple[int, str]], **timing) -> List[Dict]:
        return [self.run_single(i, e, **timing) for i, e in expressions]


def run_sweep(family: str, tensor_configs: List[Dict[str, int]], expressions: List[Tuple[int, str]], output: Optional[str],
              **timing) -> List[Dict]:
    """Every configuration over every candidate; the output file is rewritten after each configuration."""
    rows: List[Dict] = []
    if output:
        with open(output, "w") as f:
            json.dump([], f)
    for cfg in tensor_configs:
        try:
            rows.extend(BlockSweep(family, cfg).run_all(expressions, **timing))
        except Exception as e:
            rows.append({"tensor_config": cfg, "error": str(e), "results": []})
        if output:
            with open(output, "w") as f:
                json.dump(rows, f, indent=2)
    return rows


def report(rows: List[Dict], top_k: int) -> str:
    lines = [f"{len(rows)} records, {sum(1 for r in rows if r.get('error') is None)} valid"]
    for n, r in enumerate(best(rows, top_k), 1):
        c = r["tensor_config"]
        lines.append(f"{n}. IR {r['ir_id']}: {r['execution_time_ms']:.4f} ms  (M={c['M']}, N={c['N']})  {r['ir_expression'][:80]}...")
    return "\n".join(lines)


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="Time IR candidates of one block family on the B200 back end")
    ap.add_argument("--family", required=True, choices=FAMILIES)
    ap.add_argument("--ir", required=True, help="IR file, one '<id>: <expression>' per line")
    ap.add_argument("--configs", required=True, help="JSON list of {M, D, N, P, H} tensor configurations")
    ap.add_argument("--output", required=True)
    ap.add_argument("--start", type=int, default=0, help="first candidate id")
    ap.add_argument("--num", type=int, default=10, help="number of candidates")
    ap.add_argument("--end", action="store_true", help="from --start to the last candidate")
    ap.add_argument("--all", action="store_true", help="every candidate of the file")
    ap.add_argument("--topk", type=int, default=5)
    a = ap.parse_args(argv)
    if a.end and a.num != 10:
        ap.error("--end and --num exclude each other")
    with open(a.configs) as f:
        configs = json.load(f)
    expressions = parse_ir_file(a.ir)
    expressions = select(expressions, a.start, None if (a.all or a.end) else a.num)
    rows = run_sweep(a.family, configs, expressions, a.output)
    print(report(rows, a.topk))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
