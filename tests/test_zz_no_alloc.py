"""tb200_gemm_static_scratch -- the GEMM for callers that must not allocate device memory.

Who needs it: a serving process that has handed all of HBM to its own memory pool, or a plugin that runs
under somebody else's allocator, cannot tolerate a library that calls cudaMalloc behind its back (the
pool has left nothing to give, and a foreign allocation breaks the host's accounting).  This entry point
keeps the split-K partial sums in a 16 MiB array that is part of the library image instead.

The test drives it through the C ABI exactly as such a caller would, twice in a row on different inputs
(the array is shared between calls and keeps the previous call's contents), and compares each result
with the regular entry point, tb200_gemm, on the same inputs.  It runs last in the suite (file name) and
also passes alone in a fresh process.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL = ATOL = 2e-2   # the tolerance of the other GPU tests (16-bit kernels)


def _call(fn_name, a, b, out, *, b2=None, row_scale=None, residual=None, act=0, split_k=0, workspace=None):
    from trinity_b200 import _lib as L
    lib = L.load()
    p = lambda t: None if t is None else t.data_ptr()
    args = L.GemmArgs(dtype=L.BF16 if a.dtype == torch.bfloat16 else L.F16, act=act, m=a.shape[0], n=b.shape[1], k=a.shape[1],
                      a=p(a), b=p(b), b2=p(b2), c=p(out), row_scale=p(row_scale), residual=p(residual), split_k=split_k,
                      workspace=p(workspace), workspace_bytes=0 if workspace is None else workspace.numel())
    return getattr(lib, fn_name)(C.byref(args), torch.cuda.current_stream().cuda_stream)


def _inputs(seed, M, N, K, dt, gated):
    g = torch.Generator().manual_seed(seed)
    dev = torch.device("cuda:0")
    a = torch.randn(M, K, generator=g).to(dt).to(dev)
    b = (torch.randn(K, N, generator=g) * K ** -0.5).to(dt).to(dev)
    b2 = (torch.randn(K, N, generator=g) * K ** -0.5).to(dt).to(dev) if gated else None
    rs = (torch.rand(M, generator=g) + 0.5).to(dev)
    res = None if gated else torch.randn(M, N, generator=g).to(dt).to(dev)
    return a, b, b2, rs, res


@pytest.mark.parametrize("M,N,K,dt,gated,split", [
    (16, 4096, 4096, torch.float16, False, 0),      # decode-sized projection, the library picks the slices
    (64, 1024, 2048, torch.bfloat16, True, 4),      # gated (SwiGLU) epilogue, four slices
])
def test_static_scratch_matches_regular_entry_point_twice(M, N, K, dt, gated, split):
    from trinity_b200 import _lib as L
    dev = torch.device("cuda:0")
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)          # workspace for the regular entry point
    for call, seed in enumerate((11, 12)):                              # two calls in a row, different data
        a, b, b2, rs, res = _inputs(seed, M, N, K, dt, gated)
        want = torch.full((M, N), float("nan"), dtype=dt, device=dev)
        got = torch.full((M, N), float("nan"), dtype=dt, device=dev)
        # The no-allocation entry point goes FIRST: run alone in a fresh process, its first call here is the first call
        # the library sees on this device (the one that looks up the array's address), before tb200_gemm has set anything up.
        free_before = torch.cuda.mem_get_info()[0] if call == 1 else None
        L.check(_call("tb200_gemm_static_scratch", a, b, got, b2=b2, row_scale=rs, residual=res, split_k=split),
                "tb200_gemm_static_scratch")
        torch.cuda.synchronize()
        if free_before is not None:    # the second call took no device memory (the first one also loads the kernels' code,
            assert torch.cuda.mem_get_info()[0] >= free_before   # which the driver places in device memory on first use)
        L.check(_call("tb200_gemm", a, b, want, b2=b2, row_scale=rs, residual=res, split_k=split, workspace=ws), "tb200_gemm")
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        torch.testing.assert_close(got.float(), want.float(), rtol=RTOL, atol=ATOL)
        # and both agree with plain fp32 arithmetic
        ref = (a.float() @ b.float()) * rs[:, None]
        if gated:
            ref = torch.nn.functional.silu(ref) * ((a.float() @ b2.float()) * rs[:, None])
        else:
            ref = ref + res.float()
        torch.testing.assert_close(got.float(), ref, rtol=RTOL, atol=ATOL)


def test_static_scratch_auto_split_and_limit():
    from trinity_b200 import _lib as L
    dev = torch.device("cuda:0")
    a, b, _, _, _ = _inputs(3, 48, 512, 4096, torch.bfloat16, False)
    got = torch.zeros(48, 512, dtype=torch.bfloat16, device=dev)
    L.check(_call("tb200_gemm_static_scratch", a, b, got, split_k=0), "tb200_gemm_static_scratch")
    torch.cuda.synchronize()
    torch.testing.assert_close(got.float(), a.float() @ b.float(), rtol=RTOL, atol=ATOL)
    # 8 slices x 2048 x 4096 fp32 = 256 MiB of partial sums: far beyond the built-in 16 MiB -> a clear refusal
    big_a = torch.zeros(2048, 512, dtype=torch.bfloat16, device=dev)
    big_b = torch.zeros(512, 4096, dtype=torch.bfloat16, device=dev)
    big_c = torch.zeros(2048, 4096, dtype=torch.bfloat16, device=dev)
    status = _call("tb200_gemm_static_scratch", big_a, big_b, big_c, split_k=8)
    assert status == -6
    assert b"16 MiB" in L.load().tb200_strerror(status)
