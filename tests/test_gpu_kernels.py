"""Parity of the individual sm_100a kernels against fp32 references, through the C ABI."""
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import ATOL, RTOL, close, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from trinity_b200 import ops as o
    return o


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,cols", [(1, 64), (16, 4544), (300, 4096), (5, 8200), (3, 16384)])
def test_rmsnorm(ops, dt, rows, cols):
    g = torch.Generator().manual_seed(rows * 7 + cols)
    x = torch.randn(rows, cols, generator=g).to(dt)
    w = (1 + 0.02 * torch.randn(cols, generator=g)).to(dt)
    close(ops.rmsnorm(x.to(dev()), w.to(dev()), 1e-5), orc.rmsnorm(x, w, 1e-5), msg="weighted")
    inv = torch.zeros(rows, dtype=torch.float32, device=dev())
    y = ops.rmsnorm(x.to(dev()), None, 0.0, inv_rms=inv)
    close(y, orc.rmsnorm(x), msg="reference point (no weight, eps 0)")
    close(inv, torch.rsqrt(x.float().pow(2).mean(-1)), rtol=1e-4, atol=1e-6, msg="inv_rms")


def test_rmsnorm_rejects_bad_arguments(ops):
    from trinity_b200._lib import Tb200Error
    x = torch.zeros(4, 60, dtype=torch.bfloat16, device=dev())      # cols % 8 != 0
    with pytest.raises(Tb200Error):
        ops.rmsnorm(x)
    with pytest.raises(TypeError):
        ops.rmsnorm(torch.zeros(4, 64, dtype=torch.float64, device=dev()))


def _gemm_ref(a, b, b2=None, rs=None, res=None, act=0):
    r = a.float() @ b.float()
    if rs is not None:
        r = r * rs[:, None]
    if b2 is not None:
        u = a.float() @ b2.float()
        if rs is not None:
            u = u * rs[:, None]
        r = torch.nn.functional.silu(r) * u
    if act == 1:
        r = torch.nn.functional.gelu(r)
    if res is not None:
        r = r + res.float()
    return r


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K,opts", [
    (128, 256, 64, {}), (1, 8, 8, {}), (200, 328, 192, {}), (1000, 4544, 4544, {}), (257, 264, 4096, {}),
    (384, 512, 512, dict(rs=True, res=True)), (384, 1024, 520, dict(gelu=True)), (300, 640, 1024, dict(gated=True, rs=True)),
    (130, 136, 72, dict(gated=True)), (64, 4096, 2048, dict(split=4)), (64, 1024, 2048, dict(split=4, gated=True, rs=True)),
    (16, 512, 4096, dict(split=0, res=True)), (16, 512, 4096, dict(split=7, gelu=True, res=True)), (2100, 520, 136, {}),
])
def test_gemm(ops, dt, M, N, K, opts):
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(dt).to(dev())
    b = (torch.randn(K, N, generator=g) * K ** -0.5).to(dt).to(dev())
    b2 = (torch.randn(K, N, generator=g) * K ** -0.5).to(dt).to(dev()) if opts.get("gated") else None
    rs = (torch.rand(M, generator=g) + 0.5).to(dev()) if opts.get("rs") else None
    res = torch.randn(M, N, generator=g).to(dt).to(dev()) if opts.get("res") else None
    act = 1 if opts.get("gelu") else 0
    out = torch.full((M, N), float("nan"), dtype=dt, device=dev())
    ops.gemm(a, b, b2=b2, row_scale=rs, residual=res, act=act, split_k=opts.get("split", 1), out=out)
    ops.device_status()
    close(out, _gemm_ref(a, b, b2, rs, res, act), msg=f"gemm {M}x{N}x{K} {opts}")


def test_gemm_is_deterministic(ops):
    g = torch.Generator().manual_seed(5)
    a = torch.randn(48, 4096, generator=g).to(torch.bfloat16).to(dev())
    b = (torch.randn(4096, 1024, generator=g) * 0.02).to(torch.bfloat16).to(dev())
    outs = [ops.gemm(a, b, split_k=0).clone() for _ in range(3)]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])


@pytest.mark.parametrize("rows,n,k", [(1, 2, 1), (3, 17, 17), (8, 1040, 128), (4, 4096, 1024), (2, 16384, 1000), (5, 1000, 999)])
def test_topk_is_a_stable_descending_sort(ops, rows, n, k):
    g = torch.Generator().manual_seed(n)
    s = torch.randn(rows, n, generator=g)
    s = s.round(decimals=1)          # a grid of values: many exact ties
    got = ops.topk(s.to(dev()), k)
    assert torch.equal(got.cpu(), orc.stable_topk(s, k))


def test_topk_handles_zero_signs_and_rejects_oversize(ops):
    from trinity_b200._lib import Tb200Error
    s = torch.tensor([[0.0, -0.0, 0.0, 1.0, -0.0]])
    assert ops.topk(s.to(dev()), 5).cpu().tolist() == [[3, 0, 1, 2, 4]]
    with pytest.raises(Tb200Error):
        ops.topk(torch.zeros(1, 20000, device=dev()), 4)
