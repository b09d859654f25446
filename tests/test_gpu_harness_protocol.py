"""The reference harness's calling protocol, replayed on a generated module: one call outside capture, ten warm-ups on
a side stream, CUDA-graph capture of forward(*args), a hundred replays between CUDA events, NaN check on O2
(benchmark/vanilla_llama_benchmark.py:223-301; FFN: benchmark/ffn_llama_benchmark.py:194-267)."""
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import close, dev
from tests.test_codegen import FFN, KEYFORMER, PRENORM, ROCO, VANILLA

pytestmark = pytest.mark.gpu


def harness_time(module, tensors, warmup_runs=10, benchmark_runs=100):
    args = [tensors[p] for p in module["TENSOR_PARAMS"]]
    forward = module["forward"]
    stream = torch.cuda.Stream(dev())
    forward(*args)                       # the harness's "autotune" call: outside capture
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        for _ in range(warmup_runs):
            forward(*args)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            forward(*args)
    stream.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        start.record()
        for _ in range(benchmark_runs):
            graph.replay()
        end.record()
    stream.synchronize()
    return start.elapsed_time(end) / benchmark_runs


def load(ir_text, constants):
    from trinity_b200.codegen import convert_ir_to_triton
    ns = {}
    exec(compile(convert_ir_to_triton(ir_text, None, constants), "<module>", "exec"), ns)
    return ns


@pytest.mark.parametrize("ir_text,flagkw", [(VANILLA, {}), (PRENORM, {"prenorm": True}), (KEYFORMER, {"keyformer": True}), (ROCO, {"roco": True})])
def test_attention_module_under_graph_replay(ir_text, flagkw):
    """Llama reference shape (M16 N4096 D128 P1024 H32, fp16, inputs * 0.01 as the harness does)."""
    M, N, D, P, H = 16, 4096, 128, 1024, 32
    inp = orc.ref_attention_inputs(M, N, D, P, seed=42)
    t = {k: v.to(torch.float16).to(dev()) for k, v in inp.items()}
    t["O2"] = torch.zeros(M, N, dtype=torch.float16, device=dev())
    for name in ("C_out", "C_out1", "C_out2"):
        t[name] = torch.zeros(H, P + M, dtype=torch.float16, device=dev())
    m = load(ir_text, {"M": M, "D": D, "N": N, "P": P, "H": H})
    ms = harness_time(m, t)
    from trinity_b200 import ops
    ops.device_status()
    assert ms > 0 and not torch.isnan(t["O2"]).any()
    kw = dict(flagkw)
    noise = inp["noise"] if kw.pop("keyformer", False) else None
    f16 = lambda v: v.to(torch.float16).float()
    ref = orc.attention_block(f16(inp["X"]), f16(inp["WQ"]), f16(inp["WK"]), f16(inp["WV"]), f16(inp["K_cache"]), f16(inp["V_cache"]),
                              past=P, head_dim=D, noise=None if noise is None else f16(noise), **kw)
    # after 111 identical calls the result is still the single-call result (outputs are overwritten, not accumulated)
    close(t["O2"], ref["O2"], rtol=2e-2, atol=2e-2 * float(ref["O2"].abs().max()), msg="O2 after graph replays")
    close(t["K_cache"][:, P:], ref["K_new"], rtol=2e-2, atol=2e-2 * float(ref["K_new"].abs().max()), msg="appended K rows")
    print(f"\n{m['KIND']}: {ms * 1e3:.1f} us per replay")


def test_ffn_module_under_graph_replay():
    M, N, P = 16, 4096, 14336
    inp = orc.ref_ffn_inputs(M, N, P, seed=42)
    t = {k: v.to(torch.float16).to(dev()) for k, v in inp.items()}
    t.update(FF1=torch.zeros(M, P, dtype=torch.float16, device=dev()), FF2=torch.zeros(M, N, dtype=torch.float16, device=dev()),
             attn_O2=torch.zeros(M, N, dtype=torch.float16, device=dev()))
    m = load(FFN, {"M": M, "N": N, "P": P})
    ms = harness_time(m, t)
    from trinity_b200 import ops
    ops.device_status()
    f16 = lambda v: v.to(torch.float16).float()
    ref = orc.ffn_block(f16(inp["O2"]), f16(inp["WFF1b"]), f16(inp["WFF1a"]), f16(inp["WFF2"]), wo=f16(inp["WO"]), residual=f16(inp["X"]), norm=True)
    close(t["FF2"], ref["FF2"], rtol=2e-2, atol=2e-2 * float(ref["FF2"].abs().max()), msg="FF2 after graph replays")
    print(f"\nffn_llama block: {ms * 1e3:.1f} us per replay")
