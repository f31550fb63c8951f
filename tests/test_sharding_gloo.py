"""The multi-GPU host logic on CPU: two gloo ranks cut a MatMul along K, all-reduce their fp32 partial products and
finish with the bias + GeLU epilogue (the K-split path of the benchmark, src/ops_c.cc:366-645 in the
reference), and shard the other workloads along their leading dimension.  The oracle evaluates each rank's graph."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dvm_b200 import sharding


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    from dvm_b200 import workloads as W
    from oracle.dvm_oracle import BF16, F32, OracleKernel
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(5)
    a = rng.normal(0, 0.1, (48, 64)).astype(np.float32)
    b = rng.normal(0, 0.1, (64, 40)).astype(np.float32)
    bias = rng.normal(0, 0.1, (40,)).astype(np.float32)
    ar, br = sharding.ksplit_operands(a, b, rank, world)
    o = OracleKernel()
    partial = o.store(o.cast(o.matmul(o.load(ar, BF16), o.load(br, BF16), False, False), F32))
    t = torch.from_numpy(partial.copy())
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    total = t.numpy()
    o2 = OracleKernel()
    y = o2.store(o2.cast(W.gelu_tanh(o2, o2.add(o2.load(total), o2.cast(o2.load(bias, BF16), F32))), BF16))
    # leading-dimension shards cover the workload exactly once
    rows = sharding.shard_leading(a, rank, world)
    cnt = torch.tensor([rows.shape[0]], dtype=torch.int64)
    dist.all_reduce(cnt)
    if rank == 0:
        full = OracleKernel()
        want = full.store(W.matmul_bias_gelu(full, full.load(a, BF16), full.load(b, BF16), full.load(bias, BF16)))
        err = float(np.abs(y.astype(np.float32) - want.astype(np.float32)).max())
        out.put((err, int(cnt.item())))
    dist.barrier()
    dist.destroy_process_group()


def test_ksplit_allreduce_matches_the_unsplit_graph():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    err, rows = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert err <= 1e-2 and rows == 48


def test_leading_ranges_partition_every_extent():
    for extent in (0, 1, 7, 8, 100, 16384):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.leading_range(extent, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == extent
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    assert sharding.units_processed(10, 4, "weak") == 40 and sharding.units_processed(10, 4, "strong") == 10
