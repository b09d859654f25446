#!/usr/bin/env python
"""Benchmark of the fused transformer blocks on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference|torch_sdpa|cudnn|flashinfer] [--workload NAME]

Workload (default): Llama-3-8B Vanilla attention block, prefill -- batch 8, seq 2048, hidden 4096, GQA 32/8 heads,
head_dim 128, causal, scale 1/sqrt(128), bf16; synthetic seeded inputs (x ~ N(0,1), weights ~ N(0,0.02)).  One PASS = one
forward of the block (QKV projection + cache append + causal attention) over one batch.  A STEP is `passes_per_step`
passes back to back, chosen so that the K timed steps last at least a second of device time (the steady, power-capped
regime); a burst figure (20 passes after an idle gap) is printed beside it.  At N GPUs every rank runs its own batch
(batch-sharded, no collective) and the line also carries the two partitions that do exchange or split work: the same
block cut by KV-head groups, and the tensor-parallel SwiGLU FFN with its NCCL all-reduce.

Prints ONE JSON line.  `value` is TFLOP/s from the algorithmic FLOPs of the block (2*T*N*(Hq+2Hkv)*D for the projection
+ 4*B*Hq*S^2*D/2 for causal attention) with inputs resident in HBM; `e2e` is the same through the generated-module
forward() with pinned HOST buffers copied in and the result copied out inside the timed region.  `--impl reference`
times the CPU oracle (the fp32 restatement of the reference's eager PyTorch classes) on the host cores on a bounded
sample; the other `--impl` values time library attention kernels on the same shapes, for context.
"""
from __future__ import annotations

import argparse
import hashlib
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
    # attention blocks: B, S, N, Hq, Hkv, D, variant
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
    # the reference's own benchmark points (evaluation/llama_configs.json, falcon_configs.json)
    "llama3_8b_vanilla_decode_m16_p1024": dict(kind="decode", family="vanilla", M=16, D=128, N=4096, P=1024, H=32,
                                               recorded_ms=0.2070,   # evaluation/vanilla/vanilla_llama.json, best candidate
                                               ffn_inner=14336, ffn_act="swiglu"),
    "falcon_7b_vanilla_decode_m16_p1024": dict(kind="decode", family="vanilla", M=16, D=64, N=4544, P=1024, H=71,
                                               ffn_inner=18176, ffn_act="gelu"),
    "llama3_8b_kv_evict_b16_l8192_k4096": dict(kind="evict", B=16, Hkv=32, L=8192, D=128, topk=4096, recent=0),
    "llama3_8b_kv_evict_b4_l4096_k1024": dict(kind="evict", B=4, Hkv=32, L=4096, D=128, topk=1024, recent=64),
    # grouped-query caches: a cache row keeps what any of the 4 q heads of its group selected (4 lists per row)
    "llama3_8b_gqa_kv_evict_b16_l8192_k2048": dict(kind="evict", B=16, Hkv=8, group=4, L=8192, D=128, topk=2048, recent=128),
    "falcon_7b_kv_evict_b16_l2048_k1024": dict(kind="evict", B=16, Hkv=71, L=2048, D=64, topk=1024, recent=0),
    # FFN blocks: M tokens, N hidden, P inner
    "llama3_8b_swiglu_ffn_m64": dict(kind="ffn", M=64, N=4096, P=14336, act="swiglu", dtype="fp16"),
    "llama3_8b_swiglu_ffn_m16384": dict(kind="ffn", M=16384, N=4096, P=14336, act="swiglu", dtype="bf16"),
    "falcon_7b_gelu_ffn_m32768": dict(kind="ffn", M=32768, N=4544, P=18176, act="gelu", dtype="bf16"),
    # standalone RMSNorm with a weight: rows x cols, one read and one write per element
    "rmsnorm_32768x4096": dict(kind="rmsnorm", rows=32768, cols=4096),
    "rmsnorm_32768x4544": dict(kind="rmsnorm", rows=32768, cols=4544),
}
DEFAULT = "llama3_8b_vanilla_prefill_b8_s2048"
MIN_REGION_S = 1.0        # the K timed steps last at least this long
BURST_PASSES = 20
TP_FFN_LEG = "llama3_8b_swiglu_ffn_m16384"


def block_flops(w, batch=None):
    B = w["B"] if batch is None else batch
    T = B * w["S"]
    proj = 2.0 * T * w["N"] * (w["Hq"] + 2 * w["Hkv"]) * w["D"]
    attn = 4.0 * B * w["Hq"] * w["S"] * w["S"] * w["D"] / 2.0
    return proj, attn


def workload_config(name, w):
    """What both arms (native and reference) print under `config`: the workload, nothing about how an arm runs it."""
    c = {"workload": name}
    c.update({k: v for k, v in w.items() if k != "recorded_ms"})
    return c


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained") or p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def recorded_dram_traffic(kernel, workload):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the tracked table of ncu captures (one line per
    kernel and workload, with a hash of the kernel's source at capture time).  None when there is no capture of this
    pair or when the source has changed since: a stale figure is worse than none."""
    path = os.path.join(ROOT, "profiles", "dram_traffic_per_launch.txt")
    if not os.path.exists(path):
        return None
    for line in open(path):
        f = line.split()
        if len(f) >= 5 and not line.startswith("#") and f[0] == kernel and f[1] == workload:
            src = os.path.join(ROOT, "trinity_b200", "csrc", f[3])
            if os.path.exists(src) and hashlib.sha256(open(src, "rb").read()).hexdigest()[:16] == f[4]:
                return int(f[2])
    return None


class ClockSampler:
    """SM clock and throttle reasons every few milliseconds while the timed regions run (NVML in this process; the
    nvidia-smi loop of the measurement protocol when NVML cannot be loaded).  Every sample carries a host time, so a
    region's samples are the ones that fall between the host times taken around it."""

    BAD = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown")

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period, self.samples = index, period_s, []
        self.stop_flag, self.thread, self.proc, self.max_mhz = threading.Event(), None, None, None

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            # NVML counts physical devices: follow CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [v for v in vis.split(",") if v.strip().isdigit()]
            phys = int(ids[self.index]) if self.index < len(ids) else self.index
            h = nv.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                     "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}

            def loop():
                while not self.stop_flag.is_set():
                    try:
                        mhz = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                        mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                        self.samples.append((time.time(), mhz, [n for n, bit in names.items() if mask & bit]))
                    except Exception:
                        pass
                    time.sleep(self.period)
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception:
            self._start_smi()

    def _start_smi(self):
        fields = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                  "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={fields}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

        def read():
            for line in self.proc.stdout:
                s = [c.strip() for c in line.split(",")]
                try:
                    self.max_mhz = float(s[1])
                    self.samples.append((time.time(), float(s[0]), [n for n, v in zip(names, s[2:6]) if v.lower().startswith("active")]))
                except (ValueError, IndexError):
                    continue
        self.thread = threading.Thread(target=read, daemon=True)
        self.thread.start()

    def stop(self):
        self.stop_flag.set()
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def window(self, t0: float, t1: float):
        """Median SM clock and the reasons seen between two host times."""
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        mhz = sorted(s[1] for s in inside)
        reasons = sorted({r for s in inside for r in s[2]})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(mhz),
                "rejected": any(r in self.BAD for r in reasons)}


def bind_to_gpu_numa_node(local: int):
    """Run this process (and so first-touch its pinned host buffers) on the CPUs next to its GPU.  With all ranks on one
    NUMA node, eight ranks' host copies share one socket's memory controllers and cross the socket link.  The CPU set is
    NVML's "ideal CPU affinity" of the device, else the cpulist of the PCI device's NUMA node.  Returns what was done."""
    try:
        allowed = os.sched_getaffinity(0)
        cpus, how = set(), None
        try:
            import pynvml as nv
            nv.nvmlInit()
            vis = [v for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v.strip().isdigit()]
            h = nv.nvmlDeviceGetHandleByIndex(int(vis[local]) if local < len(vis) else local)
            words = (max(allowed) // 64) + 1
            mask = nv.nvmlDeviceGetCpuAffinity(h, words)
            cpus = {64 * i + b for i, wd in enumerate(mask) for b in range(64) if (wd >> b) & 1}
            how = "nvml cpu affinity"
        except Exception:
            pr = torch.cuda.get_device_properties(local)
            path = "/sys/bus/pci/devices/%04x:%02x:%02x.0/numa_node" % (getattr(pr, "pci_domain_id", 0), pr.pci_bus_id, getattr(pr, "pci_device_id", 0))
            node = int(open(path).read().strip())
            if node >= 0:
                for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
                    a_, _, b_ = part.partition("-")
                    cpus.update(range(int(a_), int(b_ or a_) + 1))
                how = f"numa node {node}"
        use = cpus & allowed
        if not use or use == allowed:
            return None if not use else f"{how}: already there ({len(use)} cpus)"
        os.sched_setaffinity(0, use)
        return f"{how}: {len(use)} of {len(allowed)} cpus"
    except Exception:
        return None


class Dist:
    """The launcher's environment: one process per GPU; NCCL only when there is more than one."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.numa_node = bind_to_gpu_numa_node(self.local) if self.world > 1 else None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max(self, *values):
        if self.world == 1:
            return list(values)
        import torch.distributed as dist
        t = torch.tensor(values, dtype=torch.float64, device=self.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def close(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


def measure(step, steps, warmup, d: Dist, min_region_s=MIN_REGION_S, burst_passes=BURST_PASSES):
    """W warm-up passes, a burst figure (a few passes after an idle gap), then EXACTLY `steps` timed steps of
    `passes_per_step` passes each, between CUDA events on the launching stream with a barrier and a device
    synchronisation on both sides; times are the maximum over the ranks."""
    for _ in range(warmup):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    d.barrier()
    e0.record()
    for _ in range(3):
        step()
    e1.record()
    torch.cuda.synchronize()
    est_ms, = d.max(e0.elapsed_time(e1) / 3)
    time.sleep(0.25)                                   # let the clocks come back up: the burst figure starts from idle
    d.barrier()
    tb0 = time.time()
    e0.record()
    for _ in range(burst_passes):
        step()
    e1.record()
    d.barrier()
    tb1 = time.time()
    burst_ms, = d.max(e0.elapsed_time(e1) / burst_passes)
    passes = max(1, math.ceil(min_region_s * 1e3 / (steps * est_ms)))
    d.barrier()
    t0 = time.time()
    e0.record()
    for _ in range(steps * passes):
        step()
    e1.record()
    d.barrier()
    t1 = time.time()
    total_ms, = d.max(e0.elapsed_time(e1))
    return {"ms_per_pass": total_ms / (steps * passes), "ms_per_step": total_ms / steps, "passes_per_step": passes,
            "region_s": total_ms / 1e3, "burst_ms_per_pass": burst_ms, "burst_window": (tb0, tb1), "window": (t0, t1)}


def regime_fields(m, sampler, value_of):
    """The keys every native line carries about WHICH regime was measured: the steady figure is the line's value, the
    burst figure sits beside it, each with the clocks sampled while it ran."""
    out = {"timed_region_s": m["region_s"], "passes_per_step": m["passes_per_step"], "ms_per_pass": m["ms_per_pass"]}
    if sampler is not None:
        out["clocks"] = sampler.window(*m["window"])
        out["burst"] = {"value": value_of(m["burst_ms_per_pass"]), "ms_per_pass": m["burst_ms_per_pass"], "passes": BURST_PASSES,
                        "clocks": sampler.window(*m["burst_window"])}
    return out


# =============================================================================================== attention blocks
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
    if w["variant"] == "roco":
        kw = dict(roco=True, topk=w.get("topk", 0))
    return orc.attention_block(x, t["WQ"].float(), t["WK"].float(), t["WV"].float(), kc, vc, past=0, head_dim=w["D"],
                               causal=True, sm_scale=w["D"] ** -0.5, **kw)


def time_cpu(fn, steps, warmup):
    torch.set_num_threads(os.cpu_count())
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    return (time.perf_counter() - t0) / steps


ATTN_IR = {
    "vanilla": "{o2}",
    "prenorm": "(seq (store (tensor X2) (rsum (sqr (load (input X) (index fulltile))) 1) (index fulltile)) {o2})",
    "qknorm": "(seq (store (tensor Q_norm,K_norm) (load (input X) (index fulltile)) (index fulltile)) {o2})",
    "keyformer": "(seq (store (output C_out) (load (input noise) (index fulltile)) (index fulltile)) {o2})",
    "roco": "(seq (store (output C_out1) (load (input X) (index fulltile)) (index fulltile)) (seq (store (output C_out2) (load (input X) "
            "(index fulltile)) (index fulltile)) {o2}))",
}


def generated_module(variant, N, D, constants):
    """The block as a user of the reference's operator API gets it: module text from convert_ir_to_triton, executed."""
    from trinity_b200.codegen import convert_ir_to_triton
    o2 = "(store (output O2) (* (load (input X) (index fulltile)) (load (input WQ,WK,WV) (index fulltile))) (index fulltile))"
    body = ATTN_IR[variant].format(o2=o2)
    ir_text = "(ploop 0 %d %d n (seq (store (input K_cache,V_cache) (load (input X) (index fulltile)) (index fulltile)) %s))" % (N, D, body)
    ns = {}
    exec(compile(convert_ir_to_triton(ir_text, None, constants), "<generated module>", "exec"), ns)
    assert ns["KIND"] == variant, (ns["KIND"], variant)
    return ns


class AttentionBlock:
    """Device tensors of one attention workload on this rank and the two ways to run it."""

    def __init__(self, w, d: Dist, seed, head_sharded=False):
        from trinity_b200 import _lib as L
        from trinity_b200 import shard
        self.w, self.d = w, d
        dtype = torch.bfloat16
        host = make_inputs(w, dtype, seed=seed)
        B, S, N, Hq, Hkv, D = (w[k] for k in ("B", "S", "N", "Hq", "Hkv", "D"))
        if head_sharded:   # KV-head groups: x replicated, column slices of the weights, O2 comes out column-sharded
            host["WQ"], host["WK"], host["WV"] = shard.shard_attention_weights(host["WQ"], host["WK"], host["WV"], D, d.rank, d.world)
            Hq, Hkv = Hq // d.world, Hkv // d.world
        self.B, self.S, self.N, self.Hq, self.Hkv, self.D = B, S, N, Hq, Hkv, D
        self.host = host
        dev = d.dev
        self.flags = L.ATTN_CAUSAL | {"vanilla": 0, "qknorm": L.ATTN_QKNORM, "prenorm": L.ATTN_PRENORM, "roco": L.ATTN_ROCO,
                                      "keyformer": L.ATTN_KEYFORMER}[w["variant"]]
        flags = self.flags
        self.x = host["X"].to(dev)
        self.wq, self.wk, self.wv = host["WQ"].to(dev), host["WK"].to(dev), host["WV"].to(dev)
        nw, qw, kw_ = (None if host.get(k) is None else host[k].to(dev) for k in ("norm_weight", "q_norm_weight", "k_norm_weight"))
        self.k_cache = torch.zeros(B, Hkv, S, D, dtype=dtype, device=dev)
        self.v_cache = torch.zeros(B, Hkv, S, D, dtype=dtype, device=dev)
        self.o2 = torch.zeros(B, S, Hq * D, dtype=dtype, device=dev)
        self.kwargs = dict(past=0, head_dim=D, flags=flags, sm_scale=D ** -0.5, norm_weight=nw if flags & L.ATTN_PRENORM else None,
                           norm_eps=1e-5, q_norm_weight=qw if flags & L.ATTN_QKNORM else None,
                           k_norm_weight=kw_ if flags & L.ATTN_QKNORM else None, qk_eps=1e-6)
        self.extra = {}                       # the module's keyword-only tensors
        if flags & L.ATTN_PRENORM:
            self.extra["norm_weight"] = nw
        if flags & L.ATTN_QKNORM:
            self.extra.update(q_norm_weight=qw, k_norm_weight=kw_)
        self.named = {"K_cache": self.k_cache, "O2": self.o2, "V_cache": self.v_cache, "WK": self.wk, "WQ": self.wq, "WV": self.wv, "X": self.x}
        self.topk = 0
        if flags & (L.ATTN_ROCO | L.ATTN_KEYFORMER):
            self.topk = w.get("topk", 0)
            idx = torch.zeros(B, Hq, self.topk, dtype=torch.int32, device=dev)
            self.kwargs.update(topk=self.topk, topk_idx=idx, tau=1.0)
            self.extra["topk_idx"] = idx
            if flags & L.ATTN_ROCO:
                c1, c2 = (torch.zeros(B, Hq, S, dtype=torch.float32, device=dev) for _ in range(2))
                self.kwargs.update(c_out1=c1, c_out2=c2)
                self.named.update(C_out1=c1, C_out2=c2)
            else:   # Gumbel(0,1) noise, generated on the device (4.3 GB at B4 S4096): -log(-log(U))
                gen = torch.Generator(device=dev).manual_seed(d.rank)
                noise = torch.empty(B, Hq, S, S, dtype=dtype, device=dev)
                for b in range(B):
                    u = torch.rand(Hq, S, S, generator=gen, device=dev, dtype=torch.float32).clamp_(1e-9, 1 - 1e-9)
                    noise[b] = (-torch.log(-torch.log(u))).to(dtype)
                    del u
                c = torch.zeros(B, Hq, S, dtype=torch.float32, device=dev)
                self.kwargs.update(noise=noise, c_out=c)
                self.named.update(noise=noise, C_out=c)
        constants = {"M": S, "D": D, "N": N, "P": 0, "H": Hq, "H_KV": Hkv, "CAUSAL": 1, "SM_SCALE": D ** -0.5, "NORM_EPS": 1e-5,
                     "QK_EPS": 1e-6, "TAU": 1.0, "TOPK": self.topk}
        self.module = generated_module(w["variant"], N, D, constants)

    def step(self):
        from trinity_b200 import ops
        ops.attn_forward(self.x, self.wq, self.wk, self.wv, self.k_cache, self.v_cache, self.o2, **self.kwargs)

    def timed_step(self):
        from trinity_b200 import ops
        return ops.attn_forward(self.x, self.wq, self.wk, self.wv, self.k_cache, self.v_cache, self.o2, timed=True, **self.kwargs)

    def api_step(self, x_in, o_out):
        """forward(*TENSOR_PARAMS, **optional tensors) of the generated module: the call a user of the operator API makes."""
        named = dict(self.named, X=x_in, O2=o_out)
        self.module["forward"](*[named[p] for p in self.module["TENSOR_PARAMS"]], **self.extra)

    def launches_per_pass(self):
        from trinity_b200 import _lib as L
        f = self.flags
        return 2 + (1 if f & L.ATTN_PRENORM else 0) + (2 if f & (L.ATTN_ROCO | L.ATTN_KEYFORMER) else 0)


def stage_times(blk: AttentionBlock, passes):
    """Per-stage device times (CUDA events the library records between its stages, on the launching stream)."""
    acc = [0.0] * 4
    for _ in range(passes):
        acc = [a + b / passes for a, b in zip(acc, blk.timed_step())]
    return acc


def e2e_pipeline(blk: AttentionBlock, d: Dist, passes):
    """Every pass copies its own input from pinned host memory and its own result back.  The three legs run on three
    streams over two device buffers, so that pass i+1's upload and pass i-1's download overlap pass i's kernels (PCIe
    is full duplex); every copy and every kernel of the passes lies inside the timed region."""
    x_host = blk.host["X"].pin_memory()
    o_host = [torch.empty(blk.o2.shape, dtype=blk.o2.dtype).pin_memory() for _ in range(2)]
    x_dev = [blk.x, torch.empty_like(blk.x)]
    o_dev = [blk.o2, torch.empty_like(blk.o2)]
    s_in, s_out, s_run = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()

    def run(n):
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
            blk.api_step(x_dev[k], o_dev[k])
            ran[i].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ran[i])
                o_host[k].copy_(o_dev[k], non_blocking=True)
                down[i].record(s_out)
        s_run.wait_event(down[n - 1])
        if n >= 2:
            s_run.wait_event(down[n - 2])

    run(3)
    d.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run(passes)
    e1.record()
    d.barrier()
    ms, = d.max(e0.elapsed_time(e1) / passes)
    return ms, x_host.numel() * x_host.element_size(), o_host[0].numel() * o_host[0].element_size()


def partition_legs(args, d: Dist):
    """The two partitions of the block family that are more than replicas, measured at N > 1 GPUs inside the default run:
    (i) the default attention block cut by KV-head groups -- one batch for all ranks, no collective, strong scaling;
    (ii) the Llama SwiGLU FFN tensor-parallel -- column-parallel gate/up, row-parallel down, one NCCL all-reduce."""
    import torch.distributed as dist
    from trinity_b200 import shard
    from oracle import oracle as orc
    out = {}
    w = WORKLOADS[DEFAULT]
    if w["Hkv"] % d.world == 0:
        blk = AttentionBlock(w, d, seed=0, head_sharded=True)
        m = measure(blk.step, max(4, args.steps // 2), 3, d, min_region_s=0.4, burst_passes=10)
        proj, attn = block_flops(w)
        out["kv_head_groups"] = {
            "workload": DEFAULT, "scaling": "strong", "collective": None, "ms_per_pass": m["ms_per_pass"],
            "value": (proj + attn) / (m["ms_per_pass"] * 1e-3) / 1e12, "unit": "TFLOP/s (whole job)", "timed_region_s": m["region_s"],
            "burst_ms_per_pass": m["burst_ms_per_pass"], "kv_heads_per_gpu": w["Hkv"] // d.world,
            "note": "x and the norm are replicated, the weights' columns and the caches' heads are dealt out; O2 comes out column-sharded"}
        del blk
        torch.cuda.empty_cache()
    fw = WORKLOADS[TP_FFN_LEG]
    M, N, P = fw["M"], fw["N"], fw["P"]
    if P % (8 * d.world) == 0:
        dtype = torch.bfloat16
        host = {k: v.to(dtype) for k, v in orc.bench_ffn_inputs(M, N, P, seed=0, gated=True).items()}
        sh = shard.shard_ffn_weights(host["W_gate"], host["W_up"], host["W_down"], None, d.rank, d.world)
        sets = [shard.FfnShard(sh.w_gate.to(d.dev), sh.w_up.to(d.dev), sh.w_down.to(d.dev), None) for _ in range(2)]
        x = host["X"].to(d.dev)
        it = [0]

        def step():
            it[0] += 1
            return shard.tensor_parallel_ffn(x, sets[it[0] & 1], act="swiglu")["FF2"]

        from trinity_b200.peer import PeerReduce
        comm = PeerReduce(M, N, dtype, d.dev)

        def fused_step():
            it[0] += 1
            return shard.tensor_parallel_ffn(x, sets[it[0] & 1], act="swiglu", peer=comm)["FF2"]

        m = measure(fused_step, max(4, args.steps // 2), 3, d, min_region_s=0.4, burst_passes=10)
        m_nccl = measure(step, max(4, args.steps // 2), 3, d, min_region_s=0.4, burst_passes=10)
        buf = step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            dist.all_reduce(buf)
        d.barrier()
        e0.record()
        for _ in range(20):
            dist.all_reduce(buf)
        e1.record()
        d.barrier()
        ar_ms, = d.max(e0.elapsed_time(e1) / 20)
        comm.close()
        flops = 2.0 * M * N * P * 3
        out["tensor_parallel_ffn"] = {
            "workload": TP_FFN_LEG, "scaling": "strong",
            "collective": "the down projection's epilogue sends its tiles to their owner rank over NVLink (TMA stores to peer memory), a second "
                          "kernel sums in rank order and writes every rank's result (tb200_gemm_peer_reduce); no NCCL call in the block",
            "ms_per_pass": m["ms_per_pass"], "value": flops / (m["ms_per_pass"] * 1e-3) / 1e12, "unit": "TFLOP/s (whole job)",
            "timed_region_s": m["region_s"], "burst_ms_per_pass": m["burst_ms_per_pass"],
            "with_nccl_allreduce": {"ms_per_pass": m_nccl["ms_per_pass"], "value": flops / (m_nccl["ms_per_pass"] * 1e-3) / 1e12,
                                    "burst_ms_per_pass": m_nccl["burst_ms_per_pass"], "allreduce_ms": ar_ms, "allreduce_bytes": M * N * 2,
                                    "allreduce_busbw_gbs": M * N * 2 * 2 * (d.world - 1) / d.world / (ar_ms * 1e-3) / 1e9,
                                    "allreduce_share_of_pass": ar_ms / m_nccl["ms_per_pass"],
                                    "note": "the same block with GEMM, then one NCCL all-reduce (sum) of (tokens, hidden) bf16"}}
    return out


def run_attention(args, w, name):
    from trinity_b200 import _lib as L
    from trinity_b200 import ops
    d = Dist()
    args.warmup = max(args.warmup, 3)
    head_sharded = args.shard == "heads" and d.world > 1
    blk = AttentionBlock(w, d, seed=0 if head_sharded else d.rank, head_sharded=head_sharded)   # batch-sharded: every rank its own batch
    sampler = ClockSampler(d.local)
    if d.rank == 0:
        sampler.start()
    m = measure(blk.step, args.steps, args.warmup, d)
    ops.device_status()
    # per-stage times: a burst sample (after an idle gap) and a steady one (back to back for a few tenths of a second)
    time.sleep(0.25)
    burst_stage = stage_times(blk, 10)
    steady_stage = stage_times(blk, max(10, min(400, int(0.4e3 / m["ms_per_pass"]))))
    e2e_passes = max(args.steps, min(400, int(0.5e3 / (3.5 * m["ms_per_pass"]))))
    ms_e2e, h2d, d2h = e2e_pipeline(blk, d, e2e_passes)
    ops.device_status()
    parts = partition_legs(args, d) if (d.world > 1 and name == DEFAULT and not head_sharded) else None
    sampler.stop()

    proj, attn = block_flops(w)
    flags = blk.flags
    second_pass = attn / 2 if flags & (L.ATTN_ROCO | L.ATTN_KEYFORMER) else 0.0    # Q K^T recomputed for the per-key sums
    total = (proj + attn + second_pass) * (1 if head_sharded else d.world)
    peaks = load_peaks()
    if d.rank == 0:
        share = d.world if head_sharded else 1          # this rank's part of the block's work
        tf = lambda fl, ms: fl / share / (ms * 1e-3) / 1e12 if ms > 0 else None
        value_of = lambda ms: total / (ms * 1e-3) / 1e12
        line = {
            "metric": "fused_block_tflops", "value": value_of(m["ms_per_pass"]), "unit": "TFLOP/s", "n_gpus": d.world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": m["ms_per_step"], "us_per_call": m["ms_per_pass"] * 1e3,
            "higher_is_better": True, "scaling": "strong" if head_sharded else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(name, w),
            "protocol": {"parallelism": (f"KV-head groups over {d.world} GPUs, no collective" if head_sharded else f"batch-sharded x{d.world}, no collective"),
                         "step": "passes_per_step forwards of the block back to back; value and us_per_call are per forward",
                         "l2": "working set (x, weights, q, caches, o2 > 400 MB) exceeds the 126 MB L2", "causal": True},
        }
        line.update(regime_fields(m, sampler, value_of))
        line["e2e"] = {"value": total / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_pass": ms_e2e, "passes": e2e_passes,
                       "h2d_bytes_per_step": h2d * m["passes_per_step"], "d2h_bytes_per_step": d2h * m["passes_per_step"],
                       "h2d_bytes_per_pass": h2d, "d2h_bytes_per_pass": d2h,
                       "h2d_gbs_per_rank": h2d / (ms_e2e * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (ms_e2e * 1e-3) / 1e9,
                       "host_cpu_binding_rank0": d.numa_node,
                       "api": "generated-module forward(*TENSOR_PARAMS" + (", **" + "/".join(sorted(blk.extra)) + ")" if blk.extra else ")"),
                       "overlap": "upload / kernels / download on three streams, two buffers",
                       "resident": "noise tensor generated and kept on the device" if flags & L.ATTN_KEYFORMER else None}
        line["gpu_launches"] = (args.steps * m["passes_per_step"]) * blk.launches_per_pass()
        gemm_tf, gemm_tf_burst = tf(proj, steady_stage[1]), tf(proj, burst_stage[1])
        line["roofline"] = {
            "bound": "tensor", "kernel": "gemm_kernel<bf16, QKV> (tcgen05 QKV projection, head split and cache append in the epilogue)",
            "regime": "steady: timed inside a loop of whole blocks lasting tenths of a second", "achieved": gemm_tf,
            "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": gemm_tf / peaks["bf16_tflops_sustained"] if gemm_tf else None,
            "peak_source": peaks["source"] + ", cuBLAS bf16 sustained", "flops_per_launch": proj / share, "ms_per_launch": steady_stage[1],
            "traffic": recorded_dram_traffic("gemm_kernel_qkv", name) if d.world == 1 else None,
            "burst": {"achieved": gemm_tf_burst, "peak": peaks["bf16_tflops"], "frac": gemm_tf_burst / peaks["bf16_tflops"] if gemm_tf_burst else None,
                      "ms_per_launch": burst_stage[1], "peak_source": peaks["source"] + ", cuBLAS bf16 burst"}}
        attn_tf, attn_tf_burst = tf(attn, steady_stage[2]), tf(attn, burst_stage[2])
        line["stages"] = {
            "rmsnorm_ms": steady_stage[0], "qkv_gemm_ms": steady_stage[1], "attention_ms": steady_stage[2], "scores_ms": steady_stage[3],
            "qkv_gemm_tflops": gemm_tf, "attention_tflops": attn_tf,
            "attention_frac_of_peak": attn_tf / peaks["bf16_tflops_sustained"] if attn_tf else None,
            "burst": {"rmsnorm_ms": burst_stage[0], "qkv_gemm_ms": burst_stage[1], "attention_ms": burst_stage[2], "scores_ms": burst_stage[3],
                      "attention_tflops": attn_tf_burst, "attention_frac_of_peak": attn_tf_burst / peaks["bf16_tflops"] if attn_tf_burst else None}}
        if flags & L.ATTN_PRENORM and steady_stage[0] > 0:
            # The norm weight is folded into the projection weights (ops.FoldedWeights): the stage is the row statistic, one
            # read of x.  Inside the block it is the first launch after the host has waited for the previous call, so the
            # event interval also holds the host's launch latency; the kernel is therefore timed back to back as well.
            inv = torch.empty(blk.B * blk.S, dtype=torch.float32, device=d.dev)
            for _ in range(3):
                ops.row_inv_rms(blk.x, 1e-5, out=inv)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(50):
                ops.row_inv_rms(blk.x, 1e-5, out=inv)
            e1.record()
            torch.cuda.synchronize()
            alone_ms = e0.elapsed_time(e1) / 50
            norm_bytes = blk.B * blk.S * blk.N * 2
            line["stages"]["rmsnorm_kernel_alone_ms"] = alone_ms
            line["stages"]["rmsnorm_hbm_gbs"] = norm_bytes / (alone_ms * 1e-3) / 1e9
            line["stages"]["rmsnorm_frac_of_hbm"] = line["stages"]["rmsnorm_hbm_gbs"] / peaks["hbm_gbs"]
            line["stages"]["rmsnorm_note"] = "row statistic only (x read once, 268 MB > L2 at this size); the scale is applied in the projection's epilogue"
        if flags & (L.ATTN_ROCO | L.ATTN_KEYFORMER):
            line["stages"].update(score_stage_split(blk, steady_stage[3], peaks))
        line["block_frac_of_peak"] = total / d.world / (m["ms_per_pass"] * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"]
        if parts is not None:
            line["partitions"] = parts
        if not args.no_cpu_baseline:
            cpu_t = {k: v.float() for k, v in blk.host.items()}
            dt = time_cpu(lambda: oracle_step(w, cpu_t, 1), steps=1, warmup=0)
            p1, a1 = block_flops(w, 1)
            line["cpu_baseline"] = {"value": (p1 + a1) / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port", "seconds": dt,
                                    "sample": "1 of %d sequences (seq %d), 1 timed pass, fp32 oracle port of the reference's eager classes" % (blk.B, blk.S)}
        print(json.dumps(line), flush=True)
    d.close()


def score_stage_split(blk, scores_ms, peaks):
    """The per-key reduction pass and the top-k inside the block's last stage, each against HBM: top-k is timed alone on
    the block's own scores, the reduction pass is the rest of the stage."""
    from trinity_b200 import ops
    key = blk.kwargs.get("c_out") if blk.kwargs.get("c_out") is not None else blk.kwargs["c_out1"]
    idx = blk.kwargs["topk_idx"]
    for _ in range(3):
        ops.topk(key, blk.topk, out=idx)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        ops.topk(key, blk.topk, out=idx)
    e1.record()
    torch.cuda.synchronize()
    topk_ms = e0.elapsed_time(e1) / 20
    topk_bytes = key.numel() * 4 + idx.numel() * 4
    score_ms = max(scores_ms - topk_ms, 1e-6)
    rows = blk.B * blk.Hq * blk.S
    # what the pass must move: q (once per key tile it is L2-resident), k, the row statistics, the fp32 outputs
    score_bytes = rows * blk.D * 2 + blk.B * blk.Hkv * blk.S * blk.D * 2 + rows * 4 + key.numel() * 4 * (1 if blk.kwargs.get("c_out") is not None else 2)
    if blk.kwargs.get("noise") is not None:
        score_bytes += blk.kwargs["noise"].numel() * 2 // 2 + rows * 4      # the causal half of the noise tensor, second statistic
    return {"topk_ms": topk_ms, "topk_hbm_gbs": topk_bytes / (topk_ms * 1e-3) / 1e9, "topk_frac_of_hbm": topk_bytes / (topk_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "topk_note": "one CTA per row sorts 64-bit keys in shared memory: bound by shared-memory traffic, not HBM",
            "score_pass_ms": score_ms, "score_pass_hbm_gbs": score_bytes / (score_ms * 1e-3) / 1e9,
            "score_pass_frac_of_hbm": score_bytes / (score_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "score_pass_note": "recomputes Q K^T on the tensor core (one ex2 per score): bound by the special-function unit"
                               + (" and the noise stream" if blk.kwargs.get("noise") is not None else "")}


# =============================================================================================== FFN blocks
def run_ffn(args, w, name):
    """FFN block: act(x @ W_gate [, x @ W_up]) @ W_down.  One GPU: tb200_ffn_forward.  N GPUs: tensor-parallel
    (column-parallel up, row-parallel down, one NCCL all-reduce), total work fixed -> strong scaling."""
    from oracle import oracle as orc
    from trinity_b200 import _lib as L
    from trinity_b200 import ops, shard

    d = Dist()
    rank, world, dev = d.rank, d.world, d.dev
    args.warmup = max(args.warmup, 3)
    dtype = torch.float16 if w["dtype"] == "fp16" else torch.bfloat16
    M, N, P = w["M"], w["N"], w["P"]
    gated = w["act"] == "swiglu"
    host = {k: v.to(dtype) for k, v in orc.bench_ffn_inputs(M, N, P, seed=0, gated=gated).items()}
    x = host["X"].to(dev)
    weight_bytes = (3 if gated else 2) * N * P * 2
    copies = 2 if weight_bytes < 1.5e9 else 1        # rotate weight copies so that no pass finds its weights in L2
    sets = []
    for _ in range(copies):
        sh = shard.shard_ffn_weights(host["W_gate"], host.get("W_up"), host["W_down"], None, rank, world)
        sets.append(shard.FfnShard(sh.w_gate.to(dev), None if sh.w_up is None else sh.w_up.to(dev), sh.w_down.to(dev), None))
    ff2 = torch.zeros(M, N, dtype=dtype, device=dev)
    act = L.FFN_SWIGLU if gated else L.FFN_GELU
    it = [0]

    comm = None
    if world > 1 and M % (128 * world) == 0:
        from trinity_b200.peer import PeerReduce
        comm = PeerReduce(M, N, dtype, dev)

    def step():
        s_ = sets[it[0] % copies]
        it[0] += 1
        if world == 1:
            ops.ffn_forward(x, s_.w_gate, s_.w_up, s_.w_down, ff2, act=act)
            return ff2
        return shard.tensor_parallel_ffn(x, s_, act=w["act"], peer=comm)["FF2"]

    def nccl_step():
        s_ = sets[it[0] % copies]
        it[0] += 1
        return shard.tensor_parallel_ffn(x, s_, act=w["act"])["FF2"]

    sampler = ClockSampler(d.local)
    if rank == 0:
        sampler.start()
    # The reference times CUDA-graph replays of forward() (benchmark/ffn_llama_benchmark.py:194-267): with tens of
    # microseconds per call, Python launch overhead would otherwise be what is measured.  One graph holds one pass
    # per weight set; a pass of the timed region is one replayed forward.
    use_graph = world == 1 and M <= 1024
    side = torch.cuda.Stream()

    def graphed(fn):
        """fn() once per weight set inside one CUDA graph; returns a callable that replays it (= `copies` passes)."""
        for _ in range(copies):
            fn()
        torch.cuda.synchronize()
        g_ = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for _ in range(copies):
                fn()
            side.synchronize()
            with torch.cuda.graph(g_, stream=side):
                for _ in range(copies):
                    fn()
        torch.cuda.synchronize()
        return g_.replay

    if use_graph:
        replay = graphed(step)
        with torch.cuda.stream(side):
            m = measure(replay, args.steps, args.warmup, d)
        for k in ("ms_per_pass", "burst_ms_per_pass"):
            m[k] /= copies
        m["passes_per_step"] *= copies
    else:
        m = measure(step, args.steps, args.warmup, d)
    m_nccl = measure(nccl_step, max(4, args.steps // 2), 3, d, min_region_s=0.4, burst_passes=10) if comm is not None else None
    ops.device_status()
    ms = m["ms_per_pass"]
    # stage split with the building-block GEMMs (same kernels the block chains)
    ff1 = torch.empty(M, P // world, dtype=dtype, device=dev)
    jt = [0]

    def up():
        s_ = sets[jt[0] % copies]
        jt[0] += 1
        ops.gemm(x, s_.w_gate, b2=s_.w_up, act=0 if gated else 1, split_k=0, out=ff1)

    def down():
        s_ = sets[jt[0] % copies]
        jt[0] += 1
        ops.gemm(ff1, s_.w_down, split_k=0, out=ff2)

    def time_stage(fn):
        n = max(10, min(2000, int(0.3e3 / max(ms, 1e-3))))
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if use_graph:
            rp = graphed(fn)
            with torch.cuda.stream(side):
                rp()
                a0.record()
                for _ in range(n // copies + 1):
                    rp()
                a1.record()
            torch.cuda.synchronize()
            return a0.elapsed_time(a1) / ((n // copies + 1) * copies)
        for _ in range(3):
            fn()
        a0.record()
        for _ in range(n):
            fn()
        a1.record()
        torch.cuda.synchronize()
        return a0.elapsed_time(a1) / n

    st_ms = [time_stage(up), time_stage(down)]
    # end to end: pinned host x in, ff2 out, every pass; upload, kernels and download on three streams, two buffers
    x_host = host["X"].pin_memory()
    o_host = [torch.empty(M, N, dtype=dtype).pin_memory() for _ in range(2)]
    x_dev, o_dev = [x, torch.empty_like(x)], [ff2, torch.empty_like(ff2)]
    s_in, s_out, s_run = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()

    def e2e_run(n):
        up_e, ran, down_e = ([torch.cuda.Event() for _ in range(n)] for _ in range(3))
        for i in range(n):
            k = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ran[i - 2])
                x_dev[k].copy_(x_host, non_blocking=True)
                up_e[i].record(s_in)
            s_run.wait_event(up_e[i])
            if i >= 2:
                s_run.wait_event(down_e[i - 2])
            s_ = sets[i % copies]
            if world == 1:
                ops.ffn_forward(x_dev[k], s_.w_gate, s_.w_up, s_.w_down, o_dev[k], act=act)
                res = o_dev[k]
            else:
                res = shard.tensor_parallel_ffn(x_dev[k], s_, act=w["act"], peer=comm)["FF2"]
            ran[i].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ran[i])
                o_host[k].copy_(res, non_blocking=True)
                down_e[i].record(s_out)
        s_run.wait_event(down_e[n - 1])
        if n >= 2:
            s_run.wait_event(down_e[n - 2])

    e2e_passes = max(args.steps, min(400, int(0.4e3 / max(2 * ms, 0.05))))
    e2e_run(3)
    d.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_run(e2e_passes)
    e1.record()
    d.barrier()
    ms_e2e, = d.max(e0.elapsed_time(e1) / e2e_passes)
    sampler.stop()
    ops.device_status()
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
                    "peak": peaks["hbm_gbs"], "unit": "GB/s", "bytes_per_launch": up_bytes, "peak_source": peaks["source"] + ", stream copy"}
        else:
            roof = {"bound": "tensor", "kernel": "gemm_kernel (gate/up projection)", "achieved": up_flops / (st_ms[0] * 1e-3) / 1e12,
                    "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s", "flops_per_launch": up_flops,
                    "regime": "steady: timed in a loop of tenths of a second", "peak_source": peaks["source"] + ", cuBLAS bf16 sustained"}
        roof.update(frac=roof["achieved"] / roof["peak"], traffic=None, ms_per_launch=st_ms[0])
        value_of = lambda t: flops / (t * 1e-3) / 1e12
        launches_per_pass = 2 if not hbm_bound else 4
        line = {
            "metric": "fused_block_tflops", "value": value_of(ms), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": m["ms_per_step"], "us_per_call": ms * 1e3, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": workload_config(name, w),
            "protocol": {"parallelism": "single GPU" if world == 1 else (f"tensor-parallel x{world}, all-reduce inside the down projection's kernels over peer memory "
                                                                         "(tb200_gemm_peer_reduce)" if comm is not None else f"tensor-parallel x{world}, one NCCL all-reduce"),
                         "l2": f"{copies} rotating weight sets of {weight_bytes / 1e6:.0f} MB each (> 126 MB L2)",
                         "timing": "CUDA-graph replay, as the reference harness" if use_graph else "stream launches"},
            "block_hbm_gbs": algo_bytes / world / (ms * 1e-3) / 1e9, "block_frac_of_hbm": algo_bytes / world / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "block_frac_of_tensor_peak": flops / world / (ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"],
            "e2e": {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_pass": ms_e2e, "passes": e2e_passes,
                    "h2d_bytes_per_step": M * N * 2 * m["passes_per_step"], "d2h_bytes_per_step": M * N * 2 * m["passes_per_step"],
                    "h2d_bytes_per_pass": M * N * 2, "d2h_bytes_per_pass": M * N * 2,
                    "api": "ops.ffn_forward (tb200_ffn_forward)" if world == 1 else "shard.tensor_parallel_ffn",
                    "overlap": "upload / kernels / download on three streams, two buffers"},
            "gpu_launches": args.steps * m["passes_per_step"] * launches_per_pass, "roofline": roof,
            "stages": {"up_ms": st_ms[0], "down_ms": st_ms[1]},
        }
        line.update(regime_fields(m, sampler, value_of))
        if m_nccl is not None:
            line["with_nccl_allreduce"] = {"ms_per_pass": m_nccl["ms_per_pass"], "value": value_of(m_nccl["ms_per_pass"]),
                                           "note": "the same block with GEMM, then one NCCL all-reduce of (tokens, hidden)"}
        if not args.no_cpu_baseline:
            rows = min(M, 256)
            dt = time_cpu(lambda: orc.ffn_block(host["X"][:rows].float(), host["W_gate"].float(), host["W_up"].float() if gated else None,
                                                host["W_down"].float(), act=w["act"]), 1, 0)
            line["cpu_baseline"] = {"value": flops * rows / M / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port", "seconds": dt,
                                    "sample": f"{rows} of {M} tokens, 1 pass, fp32 oracle port of baseline/ffn_ref.py"}
        print(json.dumps(line), flush=True)
    if comm is not None:
        comm.close()
    d.close()


# =============================================================================================== reference decode point
def run_decode(args, w, name):
    """The reference's own benchmark point (evaluation/llama_configs.json / falcon_configs.json: 16 new tokens on 1024
    cached keys, fp16, MHA, no mask, scale 1), called the way its harness calls a generated module: tensors from
    trinity_b200.sweep's table, forward(*TENSOR_PARAMS) under CUDA-graph replay.  A decode step streams the projection
    weights once: the block is HBM-bound, bytes = WQ, WK, WV + both caches + X + O2."""
    from trinity_b200 import ops, sweep
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
    replays = max(args.steps, 100, int(1.0e3 / 0.045))          # at least a second of replays
    t0 = time.time()
    ms = bs.time_module(module, warmup_runs=max(warmup, 10), benchmark_runs=replays)
    t1 = time.time()
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
    n_e2e = max(args.steps, 200)
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1) / n_e2e
    sampler.stop()
    flops = 2.0 * M * N * 3 * H * D + 4.0 * H * M * (P + M) * D
    w_bytes = 3 * N * H * D * 2
    algo_bytes = w_bytes + 2 * H * (P + M) * D * 2 + 2 * M * N * 2
    qkv_ms = max(stage[1] - empty, 1e-6)
    qkv_bytes = w_bytes + M * N * 2 + 3 * M * H * D * 2
    peaks = load_peaks()
    line = {
        "metric": "fused_block_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(warmup, 10) + 1, "ms_per_step": ms * replays / args.steps, "us_per_call": ms * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16", "data": "synthetic", "config": workload_config(name, w),
        "protocol": {"timing": "CUDA-graph replay of forward(*TENSOR_PARAMS), the reference harness's protocol",
                     "l2": "the 100 MB of projection weights stay partly in the 126 MB L2 between replays, as they do for the reference's own numbers"},
        "timed_region_s": ms * replays / 1e3, "passes_per_step": replays / args.steps, "ms_per_pass": ms, "clocks": sampler.window(t0, t1),
        "block_hbm_gbs": algo_bytes / (ms * 1e-3) / 1e9, "block_frac_of_hbm": algo_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "e2e": {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_pass": ms_e2e, "h2d_bytes_per_step": M * N * 2,
                "d2h_bytes_per_step": M * N * 2, "api": "generated-module forward(*TENSOR_PARAMS), stream launches"},
        "gpu_launches": 4 * replays,
        "roofline": {"bound": "hbm", "kernel": "gemm_kernel<PARTIAL> (QKV projection, K-sliced; its slices are summed by attn_decode_kernel)",
                     "achieved": qkv_bytes / (qkv_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": qkv_bytes / (qkv_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "peak_source": peaks["source"] + ", stream copy",
                     "bytes_per_launch": qkv_bytes, "traffic": None, "ms_per_launch": qkv_ms,
                     "note": "stage time between CUDA events inside the call, minus the cost of an empty stage"},
        "stages": {"qkv_ms": qkv_ms, "attention_ms": max(stage[2] - empty, 0.0), "event_cost_ms": empty},
    }
    line["gpu_launches"] = 2 * replays     # sliced QKV projection + the one-kernel decode attention
    if w.get("ffn_inner"):
        line["layer"] = decode_layer_leg(w, t, dev, peaks)
    if w.get("recorded_ms"):
        # the best candidate time in the reference's own result file: its Triton kernel on its GPU (model not recorded)
        line["reference_recorded"] = {"ms_per_call": w["recorded_ms"], "ratio": w["recorded_ms"] / ms, "hardware": "not recorded"}
    if not args.no_cpu_baseline:
        from oracle import oracle as orc
        c = {k: t[k].float().cpu() for k in ("X", "WQ", "WK", "WV", "K_cache", "V_cache")}
        dt = time_cpu(lambda: orc.attention_block(c["X"], c["WQ"], c["WK"], c["WV"], c["K_cache"], c["V_cache"], past=P, head_dim=D), 5, 1)
        line["cpu_baseline"] = {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port", "seconds": dt,
                                "sample": "the whole workload (one sequence), 5 passes, fp32 oracle port of baseline/ref_rms.py"}
    print(json.dumps(line), flush=True)


def decode_layer_leg(w, t, dev, peaks):
    """The decode step of a whole layer: the attention block and the FFN block that consumes its O2 (output projection,
    residual, RMSNorm, MLP), as one tb200_layer_forward call and as the two block calls, both under CUDA-graph replay.
    HBM-bound on the weights: bytes = WQ, WK, WV, WO, the MLP weights, both caches."""
    from trinity_b200 import _lib as L
    from trinity_b200 import ops
    M, D, N, P, H, inner = w["M"], w["D"], w["N"], w["P"], w["H"], w["ffn_inner"]
    gated = w["ffn_act"] == "swiglu"
    g = torch.Generator(device="cpu").manual_seed(3)
    mk = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(torch.float16).to(dev)
    wo, wg, wd = mk(H * D, N), mk(N, inner), mk(inner, N)
    wu = mk(N, inner) if gated else None
    ff2 = torch.zeros(M, N, dtype=torch.float16, device=dev)
    x3, o2 = t["X"].unsqueeze(0), t["O2"].unsqueeze(0)
    attn = lambda: dict(tensors=(x3, t["WQ"], t["WK"], t["WV"], t["K_cache"].unsqueeze(0), t["V_cache"].unsqueeze(0), o2),
                        past=P, head_dim=D, flags=0, sm_scale=1.0)
    ffn = lambda: dict(tensors=(t["X"], wg, wu, wd, ff2), act=L.FFN_SWIGLU if gated else L.FFN_GELU, flags=L.FFN_NORM,
                       o2=t["O2"], wo=wo)

    def one_call():
        ops.layer_forward(attn(), ffn())

    def two_calls():
        a, f = attn(), ffn()
        ops.attn_forward(*a.pop("tensors"), **a)
        ops.ffn_forward(*f.pop("tensors"), **f)

    def replay_ms(fn, reps=300):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                fn()
            for _ in range(10):
                graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    ms_one, ms_two = replay_ms(one_call), replay_ms(two_calls)
    ops.device_status()
    w_bytes = (3 * N * H * D + H * D * N + (3 if gated else 2) * N * inner) * 2
    algo = w_bytes + 2 * H * (P + M) * D * 2
    return {"api": "tb200_layer_forward (attention block + FFN block with WO, residual, RMSNorm), CUDA-graph replay",
            "ms_per_call": ms_one, "ms_as_two_calls": ms_two, "algorithmic_bytes": algo,
            "hbm_gbs": algo / (ms_one * 1e-3) / 1e9, "frac_of_hbm": algo / (ms_one * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "l2": "486 MB (Llama) / 640 MB (Falcon) of weights per call: nothing survives in the 126 MB L2 between replays"}


# =============================================================================================== KV eviction
def run_evict(args, w, name):
    """KV-cache eviction (top-k index lists -> packed caches), an HBM-bound step: every rank packs the caches of its own
    batch (no collective, weak scaling).  Algorithmic bytes = kept positions x head_dim x 2 B x (K, V) x (read + write)."""
    from oracle import oracle as orc
    from trinity_b200 import ops

    d = Dist()
    rank, world, dev = d.rank, d.world, d.dev
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

    args.warmup = max(args.warmup, 3)
    sampler = ClockSampler(d.local)
    if rank == 0:
        sampler.start()
    m = measure(step, args.steps, args.warmup, d)
    ms = m["ms_per_pass"]
    ops.device_status()
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
    n_e2e = max(args.steps, min(1000, int(0.3e3 / max(ms, 1e-3))))
    d.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    d.barrier()
    ms_e2e, = d.max(e0.elapsed_time(e1) / n_e2e)
    sampler.stop()
    ops.device_status()
    if rank == 0:
        peaks = load_peaks()
        value_of = lambda t: algo_bytes * world / (t * 1e-3) / 1e9
        gbs = algo_bytes / (ms * 1e-3) / 1e9
        line = {
            "metric": "kv_evict_gbs", "value": value_of(ms), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": m["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16 (bf16 moved as bits)",
            "data": "synthetic", "config": workload_config(name, w),
            "protocol": {"kept_positions": kept,
                         "l2": f"source caches {2 * B * H * Lc * D * 2 / 1e6:.0f} MB + destination {algo_bytes / 2e6:.0f} MB (> 126 MB L2)"},
            "e2e": {"value": algo_bytes * world / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_pass": ms_e2e,
                    "h2d_bytes_per_step": idx.numel() * 4 * m["passes_per_step"], "d2h_bytes_per_step": (pos.numel() + n.numel()) * 4 * m["passes_per_step"],
                    "api": "ops.kv_compact (tb200_kv_compact)"},
            "gpu_launches": args.steps * m["passes_per_step"],
            "roofline": {"bound": "hbm", "kernel": "kv_compact_kernel", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "peak_source": peaks["source"] + ", stream copy", "bytes_per_launch": algo_bytes,
                         "traffic": recorded_dram_traffic("kv_compact_kernel", name) if world == 1 else None, "ms_per_launch": ms},
        }
        line.update(regime_fields(m, sampler, value_of))
        if not args.no_cpu_baseline:
            kc, vc, ic = k[0].cpu(), v[0].cpu(), idx[0].cpu()
            torch.set_num_threads(os.cpu_count())
            t0 = time.perf_counter()
            _, _, _, nc = orc.kv_compact(kc, vc, ic, Lc, recent)
            dt = time.perf_counter() - t0
            line["cpu_baseline"] = {"value": int(nc.sum()) * D * 8 / dt / 1e9, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
                                    "seconds": dt, "sample": f"1 of {B} sequences ({H} cache rows), 1 pass, oracle port"}
        print(json.dumps(line), flush=True)
    d.close()


# =============================================================================================== standalone RMSNorm
def run_rmsnorm(args, w, name):
    """y = x * rsqrt(mean(x^2) + eps) * weight over (rows, cols) bf16: one read and one write per element, nothing else."""
    from oracle import oracle as orc
    from trinity_b200 import ops
    d = Dist()
    rows, cols = w["rows"], w["cols"]
    gen = torch.Generator(device=d.dev).manual_seed(d.rank)
    # two input/output pairs (2 x 537 MB at 32768 x 4096), alternated: no pass finds its rows in the 126 MB L2
    xs = [torch.randn(rows, cols, generator=gen, device=d.dev).to(torch.bfloat16) for _ in range(2)]
    ys = [torch.empty_like(xs[0]) for _ in range(2)]
    wt = (1 + 0.02 * torch.randn(cols, generator=gen, device=d.dev)).to(torch.bfloat16)
    it = [0]

    def step():
        it[0] += 1
        ops.rmsnorm(xs[it[0] & 1], wt, 1e-5, out=ys[it[0] & 1])

    args.warmup = max(args.warmup, 3)
    sampler = ClockSampler(d.local)
    if d.rank == 0:
        sampler.start()
    m = measure(step, args.steps, args.warmup, d)
    ms = m["ms_per_pass"]
    ops.device_status()
    x_host = xs[0].cpu().pin_memory()
    y_host = torch.empty(rows, cols, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        xs[0].copy_(x_host, non_blocking=True)
        ops.rmsnorm(xs[0], wt, 1e-5, out=ys[0])
        y_host.copy_(ys[0], non_blocking=True)

    for _ in range(2):
        e2e_step()
    n_e2e = max(args.steps, 20)
    d.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    d.barrier()
    ms_e2e, = d.max(e0.elapsed_time(e1) / n_e2e)
    sampler.stop()
    if d.rank == 0:
        peaks = load_peaks()
        algo_bytes = 2 * rows * cols * 2
        value_of = lambda t: algo_bytes * d.world / (t * 1e-3) / 1e9
        gbs = algo_bytes / (ms * 1e-3) / 1e9
        line = {
            "metric": "rmsnorm_gbs", "value": value_of(ms), "unit": "GB/s", "n_gpus": d.world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": m["ms_per_step"], "us_per_call": ms * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 in and out, fp32 statistic", "data": "synthetic", "config": workload_config(name, w),
            "protocol": {"l2": f"two alternating input/output pairs of {algo_bytes / 1e6:.0f} MB each (> 126 MB L2)", "rows_per_rank": rows},
            "e2e": {"value": algo_bytes * d.world / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_pass": ms_e2e,
                    "h2d_bytes_per_step": rows * cols * 2 * m["passes_per_step"], "d2h_bytes_per_step": rows * cols * 2 * m["passes_per_step"],
                    "api": "ops.rmsnorm (tb200_rmsnorm)"},
            "gpu_launches": args.steps * m["passes_per_step"],
            "roofline": {"bound": "hbm", "kernel": "rmsnorm_kernel<bf16>", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "peak_source": peaks["source"] + ", stream copy", "bytes_per_launch": algo_bytes,
                         "traffic": recorded_dram_traffic("rmsnorm_kernel", name) if d.world == 1 else None, "ms_per_launch": ms},
        }
        line.update(regime_fields(m, sampler, value_of))
        if not args.no_cpu_baseline:
            xc, wc = xs[0][:4096].float().cpu(), wt.float().cpu()
            dt = time_cpu(lambda: orc.rmsnorm(xc, wc, 1e-5), 3, 1)
            line["cpu_baseline"] = {"value": 2 * 4096 * cols * 2 / dt / 1e9, "unit": "GB/s (16-bit bytes the GPU kernel would move)", "cores": os.cpu_count(),
                                    "kind": "port", "seconds": dt, "sample": f"4096 of {rows} rows, 3 passes, fp32 oracle port of baseline/ref_rms.py:101-102"}
        print(json.dumps(line), flush=True)
    d.close()


# =============================================================================================== the reference arm (CPU)
def run_reference(args, w, name):
    """The reference's own arithmetic for the workload -- the fp32 oracle port of its eager PyTorch classes -- on the host
    cores of the box, all threads, on a bounded sample per step.  Rank 0 alone runs it."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import oracle as orc
    kind = w.get("kind", "attention")
    cores = os.cpu_count()
    metric, unit = "fused_block_tflops", "TFLOP/s"
    if kind == "attention":
        t = make_inputs(w, torch.float32, seed=0)
        fn = lambda: oracle_step(w, t, 1)
        proj, attn = block_flops(w, 1)
        units = (proj + attn + (attn / 2 if w["variant"] in ("roco", "keyformer") else 0)) / 1e12
        sample = "1 sequence (batch 1, seq %d) per step, fp32 oracle port of the reference's eager classes" % w["S"]
        if w["variant"] == "keyformer":
            sample += "; without the noise statistic (a 4096 x 4096 noise tile per head is generated on the GPU only)"
    elif kind == "ffn":
        M, N, P = w["M"], w["N"], w["P"]
        gated = w["act"] == "swiglu"
        rows = min(M, 256)
        h = orc.bench_ffn_inputs(rows, N, P, seed=0, gated=gated)
        fn = lambda: orc.ffn_block(h["X"], h["W_gate"], h.get("W_up"), h["W_down"], act=w["act"])
        units = 2.0 * rows * N * P * (3 if gated else 2) / 1e12
        sample = f"{rows} of {M} tokens per step, fp32 oracle port of baseline/ffn_ref.py"
    elif kind == "decode":
        M, D, N, P, H = (w[k] for k in "MDNPH")
        c = orc.ref_attention_inputs(M, N, D, P, seed=42)
        fn = lambda: orc.attention_block(c["X"], c["WQ"], c["WK"], c["WV"], c["K_cache"], c["V_cache"], past=P, head_dim=D)
        units = (2.0 * M * N * 3 * H * D + 4.0 * H * M * (P + M) * D) / 1e12
        sample = "the whole workload (one sequence of 16 tokens on 1024 cached keys) per step, fp32 oracle port of baseline/ref_rms.py"
    elif kind == "evict":
        B, H, Lc, D, topk, recent = (w[k] for k in ("B", "Hkv", "L", "D", "topk", "recent"))
        group = w.get("group", 1)
        g = torch.Generator().manual_seed(0)
        kc, vc = (torch.randn(H, Lc, D, generator=g).to(torch.bfloat16) for _ in range(2))
        ic = orc.stable_topk(torch.randn(H * group, Lc, generator=g), topk).view(H, group * topk)
        kept = int(orc.kv_compact(kc, vc, ic, Lc, recent)[3].sum())
        fn = lambda: orc.kv_compact(kc, vc, ic, Lc, recent)
        metric, unit, units = "kv_evict_gbs", "GB/s", kept * D * 8 / 1e9
        sample = f"1 of {B} sequences ({H} cache rows) per step, oracle port (the reference has no eviction step)"
    elif kind == "rmsnorm":
        rows, cols = 4096, w["cols"]
        g = torch.Generator().manual_seed(0)
        xc, wc = torch.randn(rows, cols, generator=g), 1 + 0.02 * torch.randn(cols, generator=g)
        fn = lambda: orc.rmsnorm(xc, wc, 1e-5)
        metric, unit, units = "rmsnorm_gbs", "GB/s", 2 * rows * cols * 2 / 1e9
        sample = f"4096 of {w['rows']} rows per step, fp32 oracle port of baseline/ref_rms.py:101-102; bytes counted as the 16-bit ones the GPU kernel moves"
    else:
        raise SystemExit(f"no reference arm for workload kind {kind!r}")
    dt = time_cpu(fn, args.steps, args.warmup)
    value = units / dt
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(name, w),
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# =============================================================================================== library kernels, for context
def run_competitor(args, w, name):
    """Library attention kernels on the attention stage of a workload (same q, k, v shapes, causal, bf16), timed like the
    native stage: the reference compares its kernels with FlashInfer and torch in the same way
    (baseline/ref_rms.py:1791-1827 FlashInfer_Vanilla, baseline/inductor.py:29-103 benchmark_rms).  Library kernels get
    this GPU's own tensors only.  One JSON line with "impl" naming the library; the value is the ATTENTION STAGE, not the block."""
    if w.get("kind") is not None:
        raise SystemExit("library arms exist for the attention workloads")
    if int(os.environ.get("RANK", "0")) != 0:
        return
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    B, S, Hq, Hkv, D = (w[k] for k in ("B", "S", "Hq", "Hkv", "D"))
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(B, Hq, S, D, generator=g, device=dev).to(torch.bfloat16)
    k = torch.randn(B, Hkv, S, D, generator=g, device=dev).to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, D, generator=g, device=dev).to(torch.bfloat16)
    scale = D ** -0.5
    try:
        if args.impl in ("torch_sdpa", "cudnn"):
            from torch.nn.attention import SDPBackend, sdpa_kernel
            backend = SDPBackend.CUDNN_ATTENTION if args.impl == "cudnn" else SDPBackend.FLASH_ATTENTION

            def step():
                with sdpa_kernel(backend):
                    return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale, enable_gqa=Hq != Hkv)
        elif args.impl == "flash_attn":
            from flash_attn import flash_attn_func
            qt, kt, vt = (t.transpose(1, 2).contiguous() for t in (q, k, v))

            def step():
                return flash_attn_func(qt, kt, vt, softmax_scale=scale, causal=True)
        else:   # flashinfer: one sequence per call, as the reference's FlashInfer_Vanilla does
            import flashinfer
            qs, ks, vs = ([t[b].transpose(0, 1).contiguous() for b in range(B)] for t in (q, k, v))

            def step():
                return [flashinfer.single_prefill_with_kv_cache(qs[b], ks[b], vs[b], causal=True, sm_scale=scale) for b in range(B)]
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
    except Exception as e:
        print(json.dumps({"impl": args.impl, "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}), flush=True)
        return
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    time.sleep(0.25)
    e0.record()
    for _ in range(BURST_PASSES):
        step()
    e1.record()
    torch.cuda.synchronize()
    burst = e0.elapsed_time(e1) / BURST_PASSES
    n = max(args.steps, int(0.5e3 / burst))
    e0.record()
    for _ in range(n):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    _, attn = block_flops(w)
    peaks = load_peaks()
    print(json.dumps({
        "impl": args.impl, "metric": "attention_stage_tflops", "value": attn / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": n, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(name, w), "burst": {"ms_per_pass": burst, "value": attn / (burst * 1e-3) / 1e12},
        "frac_of_peak": attn / (ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"],
        "note": "attention stage only (softmax(QK^T)V on ready q, k, v); compare with stages.attention_ms of the native line"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "torch_sdpa", "cudnn", "flash_attn", "flashinfer"])
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shard", default="batch", choices=["batch", "heads"],
                    help="attention at N > 1 GPUs: 'batch' = every rank its own batch (weak scaling), 'heads' = one batch, "
                         "KV-head groups dealt out over the ranks (strong scaling)")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        return run_reference(args, w, args.workload)
    if args.impl != "native":
        return run_competitor(args, w, args.workload)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: trinity_b200 has no CPU path (use --impl reference for the CPU oracle)")
    kind = w.get("kind", "attention")
    runner = {"attention": run_attention, "decode": run_decode, "evict": run_evict, "ffn": run_ffn, "rmsnorm": run_rmsnorm}[kind]
    return runner(args, w, args.workload)


if __name__ == "__main__":
    main()
