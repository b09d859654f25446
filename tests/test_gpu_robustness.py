"""What happens around the kernels: a bounded device wait that runs out, and workspaces under CUDA-graph replay."""
import pytest
import torch

from oracle import oracle as orc
from trinity_b200 import _lib as L
from trinity_b200 import ops

from .gpu_util import close, dev

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_is_reported():
    """One CTA waits on an mbarrier that nothing arms, through the same mbar_wait / abort-flag code as the compute
    kernels, with a limit of 2e5 cycles (about 0.1 ms): the wait gives up, the kernel returns, the status call reports
    the timeout once and the device is healthy afterwards."""
    lib = L.load()
    ops.device_status()                                   # start clean
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.tb200_selftest_wait_timeout(200_000, stream) == 0
    with pytest.raises(L.Tb200Error) as e:
        ops.device_status()
    assert e.value.status == -5 and "device code 900" in str(e.value)
    assert ops.device_status() == 0                       # reading the word cleared it
    # the context is intact: a real kernel runs and is right
    x = torch.randn(8, 256, device=dev()).to(torch.bfloat16)
    close(ops.rmsnorm(x), orc.rmsnorm(x.cpu()), msg="rmsnorm after a reported timeout")
    assert ops.device_status() == 0


def test_wait_limit_reaches_the_kernels():
    """The host-set limit travels in the kernel parameters: with a generous but finite limit the blocks run as before."""
    lib = L.load()
    assert lib.tb200_set_wait_limit_cycles(500_000_000) == 0
    try:
        a = torch.randn(300, 512, device=dev()).to(torch.bfloat16)
        b = (torch.randn(512, 264, device=dev()) * 512 ** -0.5).to(torch.bfloat16)
        close(ops.gemm(a, b), a.float() @ b.float(), msg="gemm under a 5e8-cycle limit")
        assert ops.device_status() == 0
    finally:
        lib.tb200_set_wait_limit_cycles(4_000_000_000)


def test_graph_replay_survives_a_larger_eager_call():
    """A captured graph holds the address of the workspace it was captured with.  A later, larger eager call outgrows
    that buffer; the old one must stay alive (and unshared), or the replay would write partial sums into memory the
    allocator has handed to somebody else."""
    g = torch.Generator().manual_seed(3)
    M, N, K = 16, 1024, 4096                                # decode size: K is split, partial sums go to the workspace
    a = torch.randn(M, K, generator=g).to(torch.float16).to(dev())
    b = (torch.randn(K, N, generator=g) * K ** -0.5).to(torch.float16).to(dev())
    out = torch.zeros(M, N, dtype=torch.float16, device=dev())
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        ops.gemm(a, b, out=out)                             # sizes this stream's workspace
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            ops.gemm(a, b, out=out)
        # a larger call on the same stream: the buffer is replaced ...
        a2 = torch.randn(64, K, generator=g).to(torch.float16).to(dev())
        b2 = (torch.randn(K, 4096, generator=g) * K ** -0.5).to(torch.float16).to(dev())
        big = ops.gemm(a2, b2)
        # ... and fresh allocations may now land where a freed buffer would have been
        junk = [torch.full((1 << 20,), float("nan"), device=dev()) for _ in range(8)]
        out.zero_()
        graph.replay()
        side.synchronize()
    close(out, a.float() @ b.float(), msg="replayed graph after the workspace grew")
    close(big, a2.float() @ b2.float(), msg="the larger call")
    assert all(bool(torch.isnan(j).all()) for j in junk), "the replay wrote into memory it no longer owns"
    assert ops.device_status() == 0
