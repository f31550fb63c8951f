"""Device runs of the all-reduce stage (NCCL inside the library) through the C ABI.

On one GPU: a communicator of one rank created through NCCL itself (rendezvous id, ncclCommInitRank); the K-split graph
then runs MatMul -> all-reduce (a copy on one rank) -> bias + GeLU and must equal the fused single-kernel graph.  With
two or more GPUs visible: one child process per GPU, K split over the ranks, every rank's result compared with the
oracle's evaluation of the unsplit graph under the MatMul tolerance (summation order differs).  Formulas:
tests/ut/comm/test_allreduce.py:128-155, examples/04_matmul_post_fusion.py:19-56 of the reference.
"""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from dvm_b200 import workloads as W
from tests.util import TOL_HALF, assert_close

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _inputs(m, n, k):
    rng = np.random.default_rng(5)
    a = rng.normal(0, 0.05, (m, k)).astype(np.float32)
    b = rng.normal(0, 0.05, (k, n)).astype(np.float32)
    bias = rng.normal(0, 0.05, (n,)).astype(np.float32)
    return a, b, bias


def _oracle(a, b, bias):
    from oracle.dvm_oracle import OracleKernel
    o = OracleKernel()
    return o.store(W.matmul_bias_gelu(o, o.load(a, 2), o.load(b, 2), o.load(bias, 2)))


def _run_rank(rank, world, uid, m, n, k):
    import dvm_b200 as dvm
    from dvm_b200 import frontend, sharding
    from dvm_b200.tester import Tester
    frontend.init_comm_with_id(rank, world, uid)
    a, b, bias = _inputs(m, n, k)
    ar, br = sharding.ksplit_operands(a, b, rank, world)
    t = Tester("mix", run_mode="dev")
    la, lb, lbias = t.load(ar, "bfloat16"), t.load(br, "bfloat16"), t.load(bias, "bfloat16")
    s = t.allreduce("sum", t.cast(t.matmul(la, lb, False, False), "float32"))
    y = t.store(t.cast(W.gelu_tanh(t, t.add(s, t.cast(lbias, "float32"))), "bfloat16"))
    t.run()
    return t.output(y), t.das()


def _check_scatter_gather(rank, world):
    """ReduceScatter, AllGather and AllReduce(max) as graph ops, against NumPy on every rank's inputs."""
    from dvm_b200.tester import Tester
    rows = 4 * world
    xs = [np.random.default_rng(100 + r).normal(size=(rows, 96)).astype(np.float32) for r in range(world)]
    t = Tester("vector", run_mode="dev")
    x = t.load(xs[rank])
    s_rs = t.store(t.add(t.reducescatter(x), 1.0))
    s_ag = t.store(t.allgather(t.mul(x, 0.5)))
    s_mx = t.store(t.allreduce("max", x))
    t.run()
    total = np.sum(xs, axis=0)
    assert_close(t.output(s_rs), total[rank * 4:(rank + 1) * 4][None] + 1.0, 1e-5, "reduce-scatter")
    assert_close(t.output(s_ag), np.concatenate([a * np.float32(0.5) for a in xs], axis=0), 0.0, "all-gather")
    assert_close(t.output(s_mx), np.max(xs, axis=0), 0.0, "all-reduce max")


def test_one_rank_communicator_runs_the_all_reduce_stage():
    from dvm_b200 import frontend
    m, n, k = 256, 512, 128
    got, das = _run_rank(0, 1, frontend.comm_unique_id(), m, n, k)
    assert "cmain.nccl(all_reduce.sum" in das
    assert_close(got, _oracle(*_inputs(m, n, k)), TOL_HALF, "K-split graph on one rank")
    _check_scatter_gather(0, 1)


_CHILD = """
import os, sys
sys.path.insert(0, {root!r})
import numpy as np, torch, torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
os.environ["DEVICE_ID"] = str(rank)
torch.cuda.set_device(rank)
dist.init_process_group("gloo", rank=rank, world_size=world)
from dvm_b200 import frontend
from tests import test_collective_gpu as T
box = [frontend.comm_unique_id() if rank == 0 else None]
dist.broadcast_object_list(box, src=0)
m, n, k = {m}, {n}, {k}
got, das = T._run_rank(rank, world, box[0], m, n, k)
assert "reduce_scatter" in das and "all_gather" in das, das
assert das.count("mmain.") == int(os.environ["DVM_B200_TP_CHUNKS"]), das
want = T._oracle(*T._inputs(m, n, k))
T.assert_close(got, want, T.TOL_HALF, "rank %d of %d" % (rank, world))
T._check_scatter_gather(rank, world)
dist.barrier()
print("RANK_OK", rank)
"""


@pytest.mark.parametrize("m,chunks", [(1024, 1), (2048, 4)])
def test_k_split_over_all_visible_gpus_matches_the_unsplit_graph(m, chunks):
    # (with four row chunks the collectives run on the kernel's second stream beside the next chunk's MatMul)
    import torch
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs two or more GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    n, k = 768, 128 * world
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   NCCL_NVLS_ENABLE="0", DVM_B200_TP_CHUNKS=str(chunks))
        procs.append(subprocess.Popen([sys.executable, "-c", _CHILD.format(root=ROOT, m=m, n=n, k=k)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "RANK_OK %d" % r in o, o[-2000:]
