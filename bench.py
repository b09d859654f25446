#!/usr/bin/env python
"""Benchmark of the fused attention block on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Workload (default): Llama-3-8B Vanilla attention block, prefill -- batch 8, seq 2048, hidden 4096,
GQA 32/8 heads, head_dim 128, causal, scale 1/sqrt(128), bf16; synthetic seeded inputs (x ~ N(0,1),
weights ~ N(0,0.02)).  One step = one forward of the block (QKV projection + cache append + causal
attention) over one batch.  At N GPUs every rank runs its own batch (batch-sharded, no collective).

Prints ONE JSON line.  `value` is TFLOP/s from the algorithmic FLOPs of the block
(2*T*N*(Hq+2Hkv)*D for the projection + 4*B*Hq*S^2*D/2 for causal attention) with inputs resident in
HBM; `e2e` is the same through the generated-module forward() with pinned HOST buffers copied in and the
result copied out inside the timed region.  `--impl reference` times the CPU oracle (the fp32
restatement of the reference's eager PyTorch classes) on the host cores on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    # name: B, S, N, Hq, Hkv, D, variant
    "llama3_8b_vanilla_prefill_b8_s2048": dict(B=8, S=2048, N=4096, Hq=32, Hkv=8, D=128, variant="vanilla"),
    "llama3_8b_qknorm_prefill_b8_s2048": dict(B=8, S=2048, N=4096, Hq=32, Hkv=8, D=128, variant="qknorm"),
    "llama3_8b_prenorm_b8_s4096": dict(B=8, S=4096, N=4096, Hq=32, Hkv=8, D=128, variant="prenorm"),
    "falcon_7b_vanilla_b16_s2048": dict(B=16, S=2048, N=4544, Hq=71, Hkv=1, D=64, variant="vanilla"),
    "falcon_7b_prenorm_b16_s2048": dict(B=16, S=2048, N=4544, Hq=71, Hkv=1, D=64, variant="prenorm"),
    "falcon_7b_qknorm_b16_s2048": dict(B=16, S=2048, N=4544, Hq=71, Hkv=1, D=64, variant="qknorm"),
    "falcon_7b_roco_b16_s2048": dict(B=16, S=2048, N=4544, Hq=71, Hkv=1, D=64, variant="roco", topk=1024),
    "falcon_7b_keyformer_b16_s2048": dict(B=16, S=2048, N=4544, Hq=71, Hkv=1, D=64, variant="keyformer", topk=1024),
    "llama3_8b_roco_b4_s4096": dict(B=4, S=4096, N=4096, Hq=32, Hkv=8, D=128, variant="roco", topk=1024),
    "llama3_8b_keyformer_b4_s4096": dict(B=4, S=4096, N=4096, Hq=32, Hkv=8, D=128, variant="keyformer", topk=1024),
    "llama3_8b_keyformer_b1_s4096": dict(B=1, S=4096, N=4096, Hq=32, Hkv=8, D=128, variant="keyformer", topk=1024),   # profiling size
    "llama3_8b_vanilla_prefill_b2_s2048": dict(B=2, S=2048, N=4096, Hq=32, Hkv=8, D=128, variant="vanilla"),   # profiling size
    "tiny": dict(B=2, S=256, N=512, Hq=4, Hkv=2, D=128, variant="vanilla"),
    # FFN blocks: M tokens, N hidden, P inner
    # the reference's own benchmark points (evaluation/llama_configs.json, falcon_configs.json)
    "llama3_8b_vanilla_decode_m16_p1024": dict(kind="decode", family="vanilla", M=16, D=128, N=4096, P=1024, H=32,
                                               recorded_ms=0.2070),   # evaluation/vanilla/vanilla_llama.json, best candidate
    "falcon_7b_vanilla_decode_m16_p1024": dict(kind="decode", family="vanilla", M=16, D=64, N=4544, P=1024, H=71),
    "llama3_8b_kv_evict_b16_l8192_k4096": dict(kind="evict", B=16, Hkv=32, L=8192, D=128, topk=4096, recent=0),
    "llama3_8b_kv_evict_b4_l4096_k1024": dict(kind="evict", B=4, Hkv=32, L=4096, D=128, topk=1024, recent=64),   # after cfg 4
    # grouped-query caches: a cache row keeps what any of the 4 q heads of its group selected (4 lists per row)
    "llama3_8b_gqa_kv_evict_b16_l8192_k2048": dict(kind="evict", B=16, Hkv=8, group=4, L=8192, D=128, topk=2048, recent=128),
    "falcon_7b_kv_evict_b16_l2048_k1024": dict(kind="evict", B=16, Hkv=71, L=2048, D=64, topk=1024, recent=0),
    "llama3_8b_swiglu_ffn_m64": dict(kind="ffn", M=64, N=4096, P=14336, act="swiglu", dtype="fp16"),
    "llama3_8b_swiglu_ffn_m16384": dict(kind="ffn", M=16384, N=4096, P=14336, act="swiglu", dtype="bf16"),
    "falcon_7b_gelu_ffn_m32768": dict(kind="ffn", M=32768, N=4544, P=18176, act="gelu", dtype="bf16"),
}
DEFAULT = "llama3_8b_vanilla_prefill_b8_s2048"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from an ncu capture of this very
# command at full size (profiles/traffic_llama_b8_s2048.md); null where no capture has been taken.
NCU_TRAFFIC = {"llama3_8b_vanilla_prefill_b8_s2048": 613_224_192}


def block_flops(w, batch=None):
    B = w["B"] if batch is None else batch
    T = B * w["S"]
    proj = 2.0 * T * w["N"] * (w["Hq"] + 2 * w["Hkv"]) * w["D"]
    attn = 4.0 * B * w["Hq"] * w["S"] * w["S"] * w["D"] / 2.0
    return proj, attn


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            if len(s) < 6:
                continue
            try:
                mhz.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz)}


def make_inputs(w, dtype, seed):
    from oracle import oracle as orc
    t = orc.bench_attention_inputs(w["B"], w["S"], w["N"], w["Hq"], w["Hkv"], w["D"], seed=seed,
                                   norm_weights=w["variant"] in ("qknorm", "prenorm"))
    return {k: v.to(dtype) for k, v in t.items()}


def oracle_step(w, t, batch_slice):
    """The CPU oracle on `batch_slice` sequences of the workload (fp32, all host threads)."""
    from oracle import oracle as orc
    B = batch_slice
    x = t["X"][:B].float()
    kc = torch.zeros(B, w["Hkv"], w["S"], w["D"])
    vc = torch.zeros(B, w["Hkv"], w["S"], w["D"])
    kw = {}
    if w["variant"] == "qknorm":
        kw = dict(qknorm=True, q_norm_weight=t["q_norm_weight"].float(), k_norm_weight=t["k_norm_weight"].float(), qk_eps=1e-6)
    if w["variant"] == "prenorm":
        kw = dict(prenorm=True, norm_weight=t["norm_weight"].float(), norm_eps=1e-5)
    return orc.attention_block(x, t["WQ"].float(), t["WK"].float(), t["WV"].float(), kc, vc, past=0, head_dim=w["D"],
                               causal=True, sm_scale=w["D"] ** -0.5, **kw)


def time_cpu(w, t, steps, warmup, batch_slice):
    torch.set_num_threads(os.cpu_count())
    for _ in range(warmup):
        oracle_step(w, t, batch_slice)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle_step(w, t, batch_slice)
    dt = (time.perf_counter() - t0) / steps
    proj, attn = block_flops(w, batch_slice)
    return dt, (proj + attn) / dt / 1e12


def run_reference(args, w, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t = make_inputs(w, torch.float32, seed=0)
    dt, tflops = time_cpu(w, t, args.steps, min(args.warmup, 1), batch_slice=1)
    cores = os.cpu_count()
    line = {
        "impl": "reference", "metric": "fused_block_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "sample": "1 sequence (batch 1) of the workload per step"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": "1 sequence (batch 1, seq %d) per step, fp32 oracle port of the reference's eager classes" % w["S"]},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_ffn(args, w, name):
    """FFN block: act(x @ W_gate [, x @ W_up]) @ W_down.  One GPU: tb200_ffn_forward.  N GPUs: tensor-parallel
    (column-parallel up, row-parallel down, one NCCL all-reduce), total work fixed -> strong scaling."""
    import torch.distributed as dist
    from oracle import oracle as orc
    from trinity_b200 import _lib as L
    from trinity_b200 import ops, shard

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    dtype = torch.float16 if w["dtype"] == "fp16" else torch.bfloat16
    M, N, P = w["M"], w["N"], w["P"]
    gated = w["act"] == "swiglu"
    host = {k: v.to(dtype) for k, v in orc.bench_ffn_inputs(M, N, P, seed=0, gated=gated).items()}
    x = host["X"].to(dev)
    weight_bytes = (3 if gated else 2) * N * P * 2
    copies = 2 if weight_bytes < 1.5e9 else 1        # rotate weight copies so that no step finds its weights in L2
    sets = []
    for _ in range(copies):
        sh = shard.shard_ffn_weights(host["W_gate"], host.get("W_up"), host["W_down"], None, rank, world)
        sets.append(shard.FfnShard(sh.w_gate.to(dev), None if sh.w_up is None else sh.w_up.to(dev), sh.w_down.to(dev), None))
    ff2 = torch.zeros(M, N, dtype=dtype, device=dev)
    act = L.FFN_SWIGLU if gated else L.FFN_GELU
    it = [0]

    def step():
        s_ = sets[it[0] % copies]
        it[0] += 1
        if world == 1:
            ops.ffn_forward(x, s_.w_gate, s_.w_up, s_.w_down, ff2, act=act)
            return ff2
        return shard.tensor_parallel_ffn(x, s_, act=w["act"])["FF2"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    ops.device_status()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # The reference times CUDA-graph replays of forward() (benchmark/ffn_llama_benchmark.py:194-267): with tens of
    # microseconds per call, Python launch overhead would otherwise be what is measured.  One graph holds one step
    # per weight set; a step of the timed region is one replayed forward.
    use_graph = world == 1 and M <= 1024
    if use_graph:
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for _ in range(copies):
                    step()
            graph.replay()
        torch.cuda.synchronize()
        reps = max(1, args.steps // copies)
        with torch.cuda.stream(side):
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / (reps * copies)
    else:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / args.steps
    # stage split with the building-block GEMMs (same kernels the block chains)
    ff1 = torch.empty(M, P // world, dtype=dtype, device=dev)

    def up(s_):
        ops.gemm(x, s_.w_gate, b2=s_.w_up, act=0 if gated else 1, split_k=0, out=ff1)

    def down(s_):
        ops.gemm(ff1, s_.w_down, split_k=0, out=ff2)

    def time_stage(fn):
        for s_ in sets:
            fn(s_)
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if use_graph:
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g_, stream=side):
                    for s_ in sets:
                        fn(s_)
                g_.replay()
                a0.record()
                for _ in range(reps):
                    g_.replay()
                a1.record()
            torch.cuda.synchronize()
            return a0.elapsed_time(a1) / (reps * copies)
        a0.record()
        for i in range(args.steps):
            fn(sets[i % copies])
        a1.record()
        torch.cuda.synchronize()
        return a0.elapsed_time(a1) / args.steps

    st_ms = [time_stage(up), time_stage(down)]
    # end to end: pinned host x in, ff2 out
    x_host = host["X"].pin_memory()
    o_host = torch.empty(M, N, dtype=dtype).pin_memory()

    def e2e_step():
        x.copy_(x_host, non_blocking=True)
        o_host.copy_(step(), non_blocking=True)

    for _ in range(3):
        e2e_step()
    barrier()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    ops.device_status()
    if world > 1:
        tt = torch.tensor([ms, ms_e2e], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ms_e2e = tt.tolist()
    flops = 2.0 * M * N * P * (3 if gated else 2)
    algo_bytes = weight_bytes + 2 * M * N * 2
    peaks = load_peaks()
    if rank == 0:
        ai = flops / algo_bytes
        hbm_bound = ai < peaks["bf16_tflops"] * 1e12 / (peaks["hbm_gbs"] * 1e9)
        up_bytes = (2 if gated else 1) * N * P * 2 / world + M * N * 2 + M * P * 2 / world
        up_flops = 2.0 * M * N * P * (2 if gated else 1) / world
        if hbm_bound:
            roof = {"bound": "hbm", "kernel": "gemm_kernel (gate/up projection, K-sliced) + splitk_finish", "achieved": up_bytes / (st_ms[0] * 1e-3) / 1e9,
                    "peak": peaks["hbm_gbs"], "unit": "GB/s", "bytes_per_launch": up_bytes}
        else:
            roof = {"bound": "tensor", "kernel": "gemm_kernel (gate/up projection)", "achieved": up_flops / (st_ms[0] * 1e-3) / 1e12,
                    "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "flops_per_launch": up_flops}
        roof.update(frac=roof["achieved"] / roof["peak"], peak_source=peaks["source"], traffic=None, ms_per_launch=st_ms[0])
        line = {
            "metric": "fused_block_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "us_per_call": ms * 1e3, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": name, "tokens": M, "hidden": N, "inner": P, "act": w["act"],
                       "parallelism": "single GPU" if world == 1 else f"tensor-parallel x{world}, one NCCL all-reduce",
                       "l2": f"{copies} rotating weight sets of {weight_bytes / 1e6:.0f} MB each (> 126 MB L2)",
                       "timing": "CUDA-graph replay, as the reference harness" if use_graph else "stream launches"},
            "block_hbm_gbs": algo_bytes / world / (ms * 1e-3) / 1e9, "block_frac_of_hbm": algo_bytes / world / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "block_frac_of_tensor_peak": flops / world / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
            "e2e": {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": M * N * 2,
                    "d2h_bytes_per_step": M * N * 2, "api": "ops.ffn_forward / shard.tensor_parallel_ffn"},
            "gpu_launches": None, "roofline": roof,
            "stages": {"up_ms": st_ms[0], "down_ms": st_ms[1]}, "clocks": clocks,
        }
        if not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count())
            rows = min(M, 256)
            t0 = time.perf_counter()
            orc.ffn_block(host["X"][:rows].float(), host["W_gate"].float(), host["W_up"].float() if gated else None, host["W_down"].float(), act=w["act"])
            dt = time.perf_counter() - t0
            line["cpu_baseline"] = {"value": flops * rows / M / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port", "seconds": dt,
                                    "sample": f"{rows} of {M} tokens, 1 pass, fp32 oracle port of baseline/ffn_ref.py"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_decode(args, w, name):
    """The reference's own benchmark point (evaluation/llama_configs.json / falcon_configs.json: 16 new tokens on 1024
    cached keys, fp16, MHA, no mask, scale 1), called the way its harness calls a generated module: tensors from
    trinity_b200.sweep's table, forward(*TENSOR_PARAMS) under CUDA-graph replay.  A decode step streams the projection
    weights once: the block is HBM-bound, bytes = WQ, WK, WV + both caches + X + O2."""
    from trinity_b200 import ops, sweep
    from trinity_b200 import _lib as L
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        raise SystemExit("the decode workloads are single-sequence: run them on one GPU")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    cfg = dict(M=w["M"], D=w["D"], N=w["N"], P=w["P"], H=w["H"])
    M, D, N, P, H = (cfg[k] for k in "MDNPH")
    family = w["family"]
    ir_text = ("(ploop 0 %d %d n (seq (store (input K_cache,V_cache) (load (input X) (index fulltile)) (index fulltile)) "
               "(store (output O2) (* (load (input X) (index fulltile)) (load (input WQ,WK,WV) (index fulltile))) (index fulltile))))" % (N, D))
    bs = sweep.BlockSweep(family, cfg, device=dev)
    module = bs.load(ir_text)
    warmup = max(args.warmup, 3)
    sampler = ClockSampler(0)
    sampler.start()
    ms = bs.time_module(module, warmup_runs=max(warmup, 10), benchmark_runs=max(args.steps, 100))
    ops.device_status()
    t = bs.tensors
    # stage split (CUDA events inside the call, stream launches: each stage carries about 2.7 us of event cost)
    stage = [0.0] * 4
    reps = 20
    for _ in range(reps):
        st = ops.attn_forward(t["X"].unsqueeze(0), t["WQ"], t["WK"], t["WV"], t["K_cache"].unsqueeze(0), t["V_cache"].unsqueeze(0),
                              t["O2"].unsqueeze(0), past=P, head_dim=D, flags=0, sm_scale=1.0, timed=True)
        stage = [a + b / reps for a, b in zip(stage, st)]
    empty = stage[0]  # the norm stage of a block without a norm: two event records and nothing between them
    # end to end: X from pinned host memory, O2 back, through the generated module, every step
    x_host, o_host = t["X"].cpu().pin_memory(), torch.empty(M, N, dtype=torch.float16).pin_memory()
    args_list = bs.arguments(module)

    def e2e_step():
        t["X"].copy_(x_host, non_blocking=True)
        module["forward"](*args_list)
        o_host.copy_(t["O2"], non_blocking=True)

    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop()
    flops = 2.0 * M * N * 3 * H * D + 4.0 * H * M * (P + M) * D
    w_bytes = 3 * N * H * D * 2
    algo_bytes = w_bytes + 2 * H * (P + M) * D * 2 + 2 * M * N * 2
    qkv_ms = max(stage[1] - empty, 1e-6)
    qkv_bytes = w_bytes + M * N * 2 + 3 * M * H * D * 2
    peaks = load_peaks()
    line = {
        "metric": "fused_block_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1, "steps": max(args.steps, 100),
        "warmup": max(warmup, 10) + 1, "ms_per_step": ms, "us_per_call": ms * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
        "config": {"workload": name, "family": family, **cfg, "timing": "CUDA-graph replay of forward(*TENSOR_PARAMS), the reference harness's protocol",
                   "l2": "the 100 MB of projection weights stay partly in the 126 MB L2 between replays, as they do for the reference's own numbers"},
        "block_hbm_gbs": algo_bytes / (ms * 1e-3) / 1e9, "block_frac_of_hbm": algo_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "e2e": {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": M * N * 2,
                "d2h_bytes_per_step": M * N * 2, "api": "generated-module forward(*TENSOR_PARAMS), stream launches"},
        "gpu_launches": 4 * max(args.steps, 100),
        "roofline": {"bound": "hbm", "kernel": "gemm_kernel<PARTIAL> + qkv_finish_kernel (QKV projection, K-sliced)",
                     "achieved": qkv_bytes / (qkv_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": qkv_bytes / (qkv_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "peak_source": peaks["source"],
                     "bytes_per_launch": qkv_bytes, "traffic": None, "ms_per_launch": qkv_ms,
                     "note": "stage time between CUDA events inside the call, minus the cost of an empty stage"},
        "stages": {"qkv_ms": qkv_ms, "attention_ms": max(stage[2] - empty, 0.0), "event_cost_ms": empty}, "clocks": clocks,
    }
    if w.get("recorded_ms"):
        # the best candidate time in the reference's own result file: its Triton kernel on its GPU (model not recorded)
        line["reference_recorded"] = {"ms_per_call": w["recorded_ms"], "ratio": w["recorded_ms"] / ms, "hardware": "not recorded"}
    if not args.no_cpu_baseline:
        from oracle import oracle as orc
        torch.set_num_threads(os.cpu_count())
        c = {k: t[k].float().cpu() for k in ("X", "WQ", "WK", "WV", "K_cache", "V_cache")}
        orc.attention_block(c["X"], c["WQ"], c["WK"], c["WV"], c["K_cache"], c["V_cache"], past=P, head_dim=D)
        t0 = time.perf_counter()
        for _ in range(5):
            orc.attention_block(c["X"], c["WQ"], c["WK"], c["WV"], c["K_cache"], c["V_cache"], past=P, head_dim=D)
        dt = (time.perf_counter() - t0) / 5
        line["cpu_baseline"] = {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port", "seconds": dt,
                                "sample": "the whole workload (one sequence), 5 passes, fp32 oracle port of baseline/ref_rms.py"}
    print(json.dumps(line), flush=True)


def run_evict(args, w, name):
    """KV-cache eviction (top-k index lists -> packed caches), an HBM-bound step: every rank packs the caches of its own
    batch (no collective, weak scaling).  Algorithmic bytes = kept positions x head_dim x 2 B x (K, V) x (read + write)."""
    import torch.distributed as dist
    from oracle import oracle as orc
    from trinity_b200 import ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B, H, Lc, D, topk, recent = (w[k] for k in ("B", "Hkv", "L", "D", "topk", "recent"))
    group = w.get("group", 1)
    gen = torch.Generator(device=dev).manual_seed(rank)
    k = torch.randn(B, H, Lc, D, generator=gen, device=dev).to(torch.bfloat16)
    v = torch.randn(B, H, Lc, D, generator=gen, device=dev).to(torch.bfloat16)
    # one top-k list per q head (distinct positions, score order); the lists of a group lie one after the other
    idx = ops.topk(torch.randn(B, H * group, Lc, generator=gen, device=dev), topk).view(B, H, group * topk)
    k_dst, v_dst, pos, n = ops.kv_compact(k, v, idx, Lc, recent)
    kept = int(n.sum())
    algo_bytes = kept * D * 2 * 2 * 2

    def step():
        ops.kv_compact(k, v, idx, Lc, recent, k_dst=k_dst, v_dst=v_dst, kept_pos=pos, new_len=n)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    ops.device_status()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    # end to end: the index lists come from pinned host memory, the kept positions and counts go back
    idx_host = idx.cpu().pin_memory()
    pos_host, n_host = torch.empty(pos.shape, dtype=torch.int32).pin_memory(), torch.empty(n.shape, dtype=torch.int32).pin_memory()

    def e2e_step():
        idx.copy_(idx_host, non_blocking=True)
        step()
        pos_host.copy_(pos, non_blocking=True)
        n_host.copy_(n, non_blocking=True)

    for _ in range(3):
        e2e_step()
    barrier()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    ops.device_status()
    if world > 1:
        tt = torch.tensor([ms, ms_e2e], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ms_e2e = tt.tolist()
    if rank == 0:
        peaks = load_peaks()
        gbs = algo_bytes / (ms * 1e-3) / 1e9
        line = {
            "metric": "kv_evict_gbs", "value": gbs * world, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16 (bf16 moved as bits)",
            "data": "synthetic",
            "config": {"workload": name, "batch_per_gpu": B, "kv_heads": H, "q_heads_per_kv_head": group, "cache_len": Lc, "head_dim": D, "topk": topk,
                       "keep_recent": recent, "kept_positions": kept,
                       "l2": f"source caches {2 * B * H * Lc * D * 2 / 1e6:.0f} MB + destination {algo_bytes / 2e6:.0f} MB (> 126 MB L2)"},
            "e2e": {"value": algo_bytes * world / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": idx.numel() * 4, "d2h_bytes_per_step": (pos.numel() + n.numel()) * 4, "api": "ops.kv_compact"},
            "gpu_launches": args.steps,
            "roofline": {"bound": "hbm", "kernel": "kv_compact_kernel", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "peak_source": peaks["source"], "bytes_per_launch": algo_bytes,
                         "traffic": None, "ms_per_launch": ms},
            "clocks": clocks,
        }
        if not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count())
            kc, vc, ic = k[0].cpu(), v[0].cpu(), idx[0].cpu()
            t0 = time.perf_counter()
            _, _, _, nc = orc.kv_compact(kc, vc, ic, Lc, recent)
            dt = time.perf_counter() - t0
            line["cpu_baseline"] = {"value": int(nc.sum()) * D * 8 / dt / 1e9, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
                                    "seconds": dt, "sample": f"1 of {B} sequences ({H} cache rows), 1 pass, oracle port"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shard", default="batch", choices=["batch", "heads"],
                    help="attention at N > 1 GPUs: 'batch' = every rank its own batch (weak scaling), 'heads' = one batch, "
                         "KV-head groups dealt out over the ranks (strong scaling)")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if w.get("kind") == "decode":
        if args.impl == "reference":
            raise SystemExit("--impl reference is defined for the attention workloads")
        return run_decode(args, w, args.workload)
    if w.get("kind") == "evict":
        if args.impl == "reference":
            raise SystemExit("--impl reference is defined for the attention workloads")
        return run_evict(args, w, args.workload)
    if w.get("kind") == "ffn":
        if args.impl == "reference":
            raise SystemExit("--impl reference is defined for the attention workloads")
        return run_ffn(args, w, args.workload)
    if args.impl == "reference":
        return run_reference(args, w, args.workload)
    if args.warmup < 3:
        args.warmup = 3

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: trinity_b200 has no CPU path (use --impl reference for the CPU oracle)")
    import torch.distributed as dist
    from trinity_b200 import _lib as L
    from trinity_b200 import ops
    from trinity_b200.codegen import convert_ir_to_triton

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    dtype = torch.bfloat16
    head_sharded = args.shard == "heads" and world > 1
    host = make_inputs(w, dtype, seed=0 if head_sharded else rank)   # batch-sharded: every rank its own batch
    B, S, N, Hq, Hkv, D = (w[k] for k in ("B", "S", "N", "Hq", "Hkv", "D"))
    if head_sharded:   # KV-head groups: x replicated, column slices of the weights, O2 comes out column-sharded
        from trinity_b200 import shard
        host["WQ"], host["WK"], host["WV"] = shard.shard_attention_weights(host["WQ"], host["WK"], host["WV"], D, rank, world)
        Hq, Hkv = Hq // world, Hkv // world
    flags = L.ATTN_CAUSAL | {"vanilla": 0, "qknorm": L.ATTN_QKNORM, "prenorm": L.ATTN_PRENORM, "roco": L.ATTN_ROCO,
                             "keyformer": L.ATTN_KEYFORMER}[w["variant"]]
    x = host["X"].to(dev)
    wq, wk, wv = host["WQ"].to(dev), host["WK"].to(dev), host["WV"].to(dev)
    nw = host.get("norm_weight")
    qw, kw_ = host.get("q_norm_weight"), host.get("k_norm_weight")
    nw, qw, kw_ = (None if v is None else v.to(dev) for v in (nw, qw, kw_))
    k_cache = torch.zeros(B, Hkv, S, D, dtype=dtype, device=dev)
    v_cache = torch.zeros(B, Hkv, S, D, dtype=dtype, device=dev)
    o2 = torch.zeros(B, S, Hq * D, dtype=dtype, device=dev)
    kwargs = dict(past=0, head_dim=D, flags=flags, sm_scale=D ** -0.5, norm_weight=nw if flags & L.ATTN_PRENORM else None,
                  norm_eps=1e-5, q_norm_weight=qw if flags & L.ATTN_QKNORM else None,
                  k_norm_weight=kw_ if flags & L.ATTN_QKNORM else None, qk_eps=1e-6)
    if flags & (L.ATTN_ROCO | L.ATTN_KEYFORMER):
        topk = w.get("topk", 0)
        kwargs.update(topk=topk, topk_idx=torch.zeros(B, Hq, topk, dtype=torch.int32, device=dev), tau=1.0)
        if flags & L.ATTN_ROCO:
            kwargs.update(c_out1=torch.zeros(B, Hq, S, dtype=torch.float32, device=dev),
                          c_out2=torch.zeros(B, Hq, S, dtype=torch.float32, device=dev))
        else:   # Gumbel(0,1) noise, generated on the device (4.3 GB at B4 S4096): -log(-log(U))
            gen = torch.Generator(device=dev).manual_seed(rank)
            u = torch.rand(B, Hq, S, S, generator=gen, device=dev, dtype=torch.float32).clamp_(1e-9, 1 - 1e-9)
            kwargs.update(noise=(-torch.log(-torch.log(u))).to(dtype), c_out=torch.zeros(B, Hq, S, dtype=torch.float32, device=dev))
            del u

    def step():
        ops.attn_forward(x, wq, wk, wv, k_cache, v_cache, o2, **kwargs)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    ops.device_status()

    # ---- device-resident timing: K steps between CUDA events on the launching stream
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps

    # ---- per-stage times (CUDA events between the stages, same stream, same inputs)
    stage = [0.0, 0.0, 0.0, 0.0]
    for _ in range(args.steps):
        s_ms = ops.attn_forward(x, wq, wk, wv, k_cache, v_cache, o2, timed=True, **kwargs)
        stage = [a + b / args.steps for a, b in zip(stage, s_ms)]

    # ---- end to end through the generated module: pinned host X in, O2 out, every step
    ir_text = "(ploop 0 %d %d n (seq (store (input K_cache,V_cache) (load (input X) (index fulltile)) (index fulltile)) " \
              "(store (output O2) (* (load (input X) (index fulltile)) (load (input WQ,WK,WV) (index fulltile))) (index fulltile))))" % (N, D)
    constants = {"M": S, "D": D, "N": N, "P": 0, "H": Hq, "H_KV": Hkv, "CAUSAL": 1, "SM_SCALE": D ** -0.5,
                 "NORM_EPS": 1e-5, "QK_EPS": 1e-6}
    if w["variant"] == "vanilla":
        src = convert_ir_to_triton(ir_text, None, constants)
        ns = {}
        exec(compile(src, "<generated module>", "exec"), ns)
        forward, params = ns["forward"], ns["TENSOR_PARAMS"]
        named = {"K_cache": k_cache, "O2": o2, "V_cache": v_cache, "WK": wk, "WQ": wq, "WV": wv, "X": x}

        def api_step(x_in, o_out):
            named["X"], named["O2"] = x_in, o_out
            forward(*[named[p] for p in params])
    else:
        def api_step(x_in, o_out):
            ops.attn_forward(x_in, wq, wk, wv, k_cache, v_cache, o_out, **kwargs)
    # Every step copies its own input from pinned host memory and its own result back.  The three legs run on three
    # streams over two device buffers, so that step i+1's upload and step i-1's download overlap step i's kernels
    # (PCIe is full duplex); every copy and every kernel of the K steps lies inside the timed region.
    x_host = host["X"].pin_memory()
    o_host = [torch.empty(B, S, Hq * D, dtype=dtype).pin_memory() for _ in range(2)]
    x_dev = [x, torch.empty_like(x)]
    o_dev = [o2, torch.empty_like(o2)]
    s_in, s_out, s_run = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()

    def e2e_run(n):
        up = [torch.cuda.Event() for _ in range(n)]
        ran = [torch.cuda.Event() for _ in range(n)]
        down = [torch.cuda.Event() for _ in range(n)]
        for i in range(n):
            k = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ran[i - 2])          # the kernels that read this x buffer have finished
                x_dev[k].copy_(x_host, non_blocking=True)
                up[i].record(s_in)
            s_run.wait_event(up[i])
            if i >= 2:
                s_run.wait_event(down[i - 2])            # this o2 buffer has been downloaded
            api_step(x_dev[k], o_dev[k])
            ran[i].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ran[i])
                o_host[k].copy_(o_dev[k], non_blocking=True)
                down[i].record(s_out)
        s_run.wait_event(down[n - 1])
        if n >= 2:
            s_run.wait_event(down[n - 2])

    e2e_run(3)
    barrier()
    e0.record()
    e2e_run(args.steps)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    ops.device_status()

    if world > 1:
        tt = torch.tensor([ms, ms_e2e], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ms_e2e = tt.tolist()

    proj, attn = block_flops(w)
    second_pass = attn / 2 if flags & (L.ATTN_ROCO | L.ATTN_KEYFORMER) else 0.0    # Q K^T recomputed for the per-key sums
    total = (proj + attn + second_pass) * (1 if head_sharded else world)
    peaks = load_peaks()
    if rank == 0:
        share = world if head_sharded else 1          # this rank's part of the block's work
        gemm_tflops = proj / share / (stage[1] * 1e-3) / 1e12 if stage[1] > 0 else None
        attn_tflops = attn / share / (stage[2] * 1e-3) / 1e12 if stage[2] > 0 else None
        peak = peaks["bf16_tflops"]
        line = {
            "metric": "fused_block_tflops", "value": total / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "us_per_call": ms * 1e3,
            "higher_is_better": True, "scaling": "strong" if head_sharded else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": B, "seq_len": S, "hidden": N, "q_heads": Hq, "kv_heads": Hkv,
                       "head_dim": D, "causal": True, "parallelism": (f"KV-head groups over {world} GPUs, no collective" if head_sharded else f"batch-sharded x{world}, no collective"),
                       "l2": "working set (x, weights, q, caches, o2 > 400 MB) exceeds the 126 MB L2"},
            "e2e": {"value": total / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": o_host[0].numel() * 2,
                    "api": "generated-module forward(*TENSOR_PARAMS)", "overlap": "upload / kernels / download on three streams, two buffers"},
            "gpu_launches": args.steps * (2 + (1 if flags & L.ATTN_PRENORM else 0) + (2 if flags & (L.ATTN_ROCO | L.ATTN_KEYFORMER) else 0)),
            "roofline": {"bound": "tensor", "kernel": "gemm_kernel<bf16, QKV> (tcgen05 QKV projection)",
                         "achieved": gemm_tflops, "peak": peak, "unit": "TFLOP/s",
                         "frac": (gemm_tflops / peak) if gemm_tflops else None, "peak_source": peaks["source"] + " burst cuBLAS bf16",
                         "traffic": NCU_TRAFFIC.get(args.workload) if world == 1 else None, "flops_per_launch": proj / share,
                         "ms_per_launch": stage[1]},
            "stages": {"rmsnorm_ms": stage[0], "qkv_gemm_ms": stage[1], "attention_ms": stage[2], "scores_ms": stage[3],
                       "qkv_gemm_tflops": gemm_tflops, "attention_tflops": attn_tflops,
                       "attention_frac_of_peak": (attn_tflops / peak) if attn_tflops else None},
            "block_frac_of_peak": total / world / (ms * 1e-3) / 1e12 / peak,
            "clocks": clocks,
        }
        if not args.no_cpu_baseline:
            cpu_t = {k: v.float() for k, v in host.items()}
            dt, tf = time_cpu(w, cpu_t, steps=1, warmup=0, batch_slice=1)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port", "seconds": dt,
                                    "sample": "1 of %d sequences (seq %d), 1 timed pass, fp32 oracle port of the reference's eager classes" % (B, S)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
