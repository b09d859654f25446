"""tb200_gemm_peer_reduce: the row-parallel projection whose all-reduce the kernels do themselves over peer memory.
With one GPU the communicator has one rank (the exchange degenerates to this GPU's own buffers, which still runs both
kernels, their counters and the completion word); with two or more GPUs a world_size-2 job of child processes checks the
real exchange against the unsharded product."""
import os
import socket
import subprocess
import sys

import pytest
import torch

from .gpu_util import close, dev

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("m,n,k,dt,res", [(256, 512, 1024, torch.bfloat16, False), (1024, 264, 520, torch.float16, True), (128, 4544, 2272, torch.bfloat16, True)])
def test_single_rank_communicator(m, n, k, dt, res):
    from trinity_b200 import ops
    from trinity_b200.peer import PeerReduce
    g = torch.Generator().manual_seed(m + n)
    a = torch.randn(m, k, generator=g).to(dt).to(dev())
    b = (torch.randn(k, n, generator=g) * k ** -0.5).to(dt).to(dev())
    r = torch.randn(m, n, generator=g).to(dt).to(dev()) if res else None
    comm = PeerReduce(m, n, dt, dev())
    for call in range(3):                                   # counters and flags grow from call to call
        out = comm.gemm_reduce(a, b, residual=r)
        ops.device_status()
        ref = a.float() @ b.float() + (r.float() if res else 0)
        close(out, ref, msg=f"call {call}")
        a = a.roll(1, 0)
    with pytest.raises(ValueError):
        comm.gemm_reduce(torch.cat([a, a]), b)
    comm.close()


def test_refuses_shapes_it_cannot_split():
    from trinity_b200.peer import PeerReduce
    with pytest.raises(ValueError):
        PeerReduce(200, 512, torch.bfloat16, dev())          # rows are dealt out in blocks of 128


WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from trinity_b200 import ops, shard
from trinity_b200.peer import PeerReduce
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
M, N, P = 1024, 1032, 4096
g = torch.Generator().manual_seed(0)
x = torch.randn(M, N, generator=g).to(torch.bfloat16)
wg, wu = ((torch.randn(N, P, generator=g) * N ** -0.5).to(torch.bfloat16) for _ in range(2))
wd = (torch.randn(P, N, generator=g) * P ** -0.5).to(torch.bfloat16)
sh = shard.shard_ffn_weights(wg, wu, wd, None, rank, world)
sh = shard.FfnShard(sh.w_gate.to(dev), sh.w_up.to(dev), sh.w_down.to(dev), None)
comm = PeerReduce(M, N, torch.bfloat16, dev)
xd = x.to(dev)
ref = (torch.nn.functional.silu(x.float() @ wg.float()) * (x.float() @ wu.float())) @ wd.float()
for call in range(3):
    fused = shard.tensor_parallel_ffn(xd, sh, act="swiglu", peer=comm)["FF2"].clone()
    nccl = shard.tensor_parallel_ffn(xd, sh, act="swiglu")["FF2"]
    ops.device_status()
    torch.testing.assert_close(fused.float().cpu(), ref, rtol=3e-2, atol=3e-2 * float(ref.abs().max()))
    torch.testing.assert_close(fused.float(), nccl.float(), rtol=2e-2, atol=2e-2 * float(ref.abs().max()))
    # every rank holds the same bits
    parts = [torch.empty_like(fused) for _ in range(world)]
    dist.all_gather(parts, fused)
    assert all(torch.equal(parts[0], q) for q in parts)
comm.close()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_against_the_unsharded_product(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                          "--master-port", str(port), str(script), ROOT], capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    assert out.stdout.count("ok") == 2
