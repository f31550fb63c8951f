"""Host side of the K-split MatMul's all-reduce (Kernel::AllReduce, include/dvm.h:531; the reference's fused
MatMul + all-reduce, src/ops_c.cc:366-645): planning with a communicator that carries rank and size only
(Comm::kDummy), so that it runs without a GPU and without NCCL.

Two plans are pinned.  The general one: MatMul -> all-reduce into a workspace temporary -> the ops behind it.  The
sharded one, taken when everything behind the all-reduce is elementwise and row-independent: reduce-scatter in place,
the tail on the rank's own row block, all-gather of the stored result in the result's type.  A world of two gloo ranks
then checks that the row blocks of the ranks tile the tensor and that the sharded data path, replayed with the
oracle and gloo collectives, equals the unsplit graph.
"""
import os
import re
import socket

import numpy as np
import pytest

import dvm_b200 as dvm
from dvm_b200 import workloads as W


def _tp_kernel(rank, world, m, n, k, row_dependent_tail=False):
    dvm.PyKernel.init_comm(rank, world, "dummy")
    kk = dvm.PyKernel("mix", "das", 0)
    a, b = kk.load([m, k], dvm.bfloat16), kk.load([k, n], dvm.bfloat16)
    bias = kk.load([n], dvm.bfloat16)
    s = kk.allreduce("sum", kk.cast(kk.matmul(a, b, False, False), dvm.float32))
    t = kk.add(s, kk.cast(bias, dvm.float32))
    if row_dependent_tail:
        t = kk.sub(t, kk.max(t, (0,), True))   # a column maximum needs every row: the tail cannot run on a row block
    kk.store(kk.cast(W.gelu_tanh(kk, t), dvm.bfloat16))
    kk.codegen()
    return kk


def _collectives(das):
    out = []
    for m in re.finditer(r"cmain\.nccl\((\w+)\.?(\w*), (\w+), count=(\d+), rank=(\d+) of (\d+), wire_bytes=(\d+)\) \{\n\s+\w+ 0x([0-9a-f]+), load\(0x([0-9a-f]+)\)", das):
        out.append({"kind": m.group(1), "op": m.group(2), "dtype": m.group(3), "count": int(m.group(4)), "rank": int(m.group(5)),
                    "size": int(m.group(6)), "wire": int(m.group(7)), "recv": int(m.group(8), 16), "send": int(m.group(9), 16)})
    return out


def test_row_independent_tail_becomes_reduce_scatter_tail_all_gather(monkeypatch):
    monkeypatch.setenv("DVM_B200_TP_CHUNKS", "1")   # (the plan of one chunk; the pipelined plan is checked below)
    m, n, k, world, rank = 16384, 8192, 1024, 8, 3
    kk = _tp_kernel(rank, world, m, n, k)
    das = kk.das()
    names = re.findall(r"^(\w+main)\.", das, re.M)
    assert names == ["mmain", "cmain", "vmain", "cmain"], names
    rs, ag = _collectives(das)
    blk = m // world * n
    assert rs["kind"] == "reduce_scatter" and rs["op"] == "sum" and rs["dtype"] == "fp32" and rs["count"] == blk
    assert rs["recv"] - rs["send"] == rank * blk * 4                       # in place: the rank's rows of the temporary
    assert ag["kind"] == "all_gather" and ag["dtype"] == "bf16" and ag["count"] == blk
    assert ag["send"] - ag["recv"] == rank * blk * 2                       # in place on the caller's result
    # bytes this rank sends: 7/8 of the fp32 temporary, then 7 copies of its bf16 block
    assert rs["wire"] == blk * 4 * (world - 1) and ag["wire"] == blk * 2 * (world - 1)
    assert "group_elems=%d" % blk in das                                    # the tail works on m / world rows
    assert "workspace_bytes=%d" % (m * n * 4) in kk.inspect()


def test_products_can_be_cut_into_row_chunks_on_two_lanes(monkeypatch):
    # DVM_B200_TP_CHUNKS=4: four row chunks; chunk c's reduce-scatter, tail and all-gather are enqueued so that the launch
    # stream (MatMuls and tails) and the second stream (collectives) overlap, every rank in the same order
    monkeypatch.setenv("DVM_B200_TP_CHUNKS", "4")
    m, n, k, world, rank = 16384, 8192, 1024, 8, 3
    kk = _tp_kernel(rank, world, m, n, k)
    das = kk.das()
    names = re.findall(r"^(\w+main)\.", das, re.M)
    assert names == ["mmain", "mmain", "cmain", "cmain", "vmain", "mmain", "cmain", "cmain", "vmain", "mmain", "cmain", "cmain",
                     "vmain", "cmain", "vmain", "cmain"], names
    colls = _collectives(das)
    kinds = [c["kind"] for c in colls]
    assert kinds == ["reduce_scatter", "reduce_scatter", "all_gather", "reduce_scatter", "all_gather", "reduce_scatter",
                     "all_gather", "all_gather"]
    chunks, mc = 4, m // 4
    blk = mc // world * n                                   # a rank's rows of one chunk
    rs = [c for c in colls if c["kind"] == "reduce_scatter"]
    ag = [c for c in colls if c["kind"] == "all_gather"]
    for c in range(chunks):
        assert rs[c]["count"] == blk and ag[c]["count"] == blk
        assert rs[c]["send"] - rs[0]["send"] == c * mc * n * 4          # chunk c of the fp32 temporary ...
        assert rs[c]["recv"] - rs[c]["send"] == rank * blk * 4          # ... reduced in place onto the rank's rows of it
        assert ag[c]["recv"] - ag[0]["recv"] == c * mc * n * 2          # chunk c of the caller's bf16 result
        assert ag[c]["send"] - ag[c]["recv"] == rank * blk * 2
    assert das.count("m=%d, n=%d, k=%d" % (mc, n, k)) == chunks         # four MatMuls of a quarter of the rows
    assert das.count("group_elems=%d" % blk) >= chunks or das.count("groups=%d" % (mc // world)) >= chunks
    assert "workspace_bytes=%d" % (m * n * 4) in kk.inspect()
    # chunks that would split a MatMul tile or a rank's rows are not made; without the switch the plan is one chunk
    small = _tp_kernel(rank, world, 256, 512, 256)
    assert re.findall(r"^(\w+main)\.", small.das(), re.M) == ["mmain", "cmain", "vmain", "cmain"]
    monkeypatch.delenv("DVM_B200_TP_CHUNKS")
    plain = _tp_kernel(rank, world, m, n, k)
    assert re.findall(r"^(\w+main)\.", plain.das(), re.M) == ["mmain", "cmain", "vmain", "cmain"]


def test_row_dependent_tail_keeps_the_plain_all_reduce():
    kk = _tp_kernel(1, 4, 512, 256, 128, row_dependent_tail=True)
    das = kk.das()
    (ar,) = _collectives(das)
    assert ar["kind"] == "all_reduce" and ar["count"] == 512 * 256 and ar["send"] != ar["recv"]
    assert das.index("mmain") < das.index("cmain") < das.index("vmain")


def test_all_reduce_needs_a_communicator_and_a_supported_type():
    dvm.PyKernel.init_comm(0, 2, "dummy")
    kk = dvm.PyKernel("vector", "das", 0)
    x = kk.load([64], dvm.float32)
    with pytest.raises(ValueError):
        kk.allreduce("prod", x)
    with pytest.raises(RuntimeError):
        kk.allreduce("sum", kk.greater(x, 0.0))   # bool


def test_reduce_scatter_and_all_gather_shapes_and_plans():
    # Kernel::ReduceScatter / AllGather (include/dvm.h:225-227; shapes: src/ops_c.cc:90-111, 951-962)
    dvm.PyKernel.init_comm(2, 4, "dummy")
    kk = dvm.PyKernel("vector", "das", 0)
    x = kk.load([64, 48], dvm.float32)
    rs = kk.reducescatter(kk.mul(x, 2.0))
    ag = kk.allgather(kk.add(x, 1.0))
    one = kk.reducescatter(kk.load([4, 48], dvm.float32))      # leading dim == ranks: one row per rank
    s1, s2, s3 = kk.store(kk.add(rs, 1.0)), kk.store(ag), kk.store(one)
    kk.codegen()
    assert rs.shape() == (1, 16, 48) and ag.shape() == (256, 48) and one.shape() == (1, 48)
    plan = _collectives(kk.das())
    kinds = sorted((c["kind"], c["count"]) for c in plan)
    assert kinds == [("all_gather", 64 * 48), ("reduce_scatter", 48), ("reduce_scatter", 16 * 48)], kinds
    with pytest.raises(RuntimeError):
        bad = dvm.PyKernel("vector", "das", 0)
        bad.store(bad.reducescatter(bad.load([10, 8], dvm.float32)))   # 10 rows over 4 ranks
        bad.codegen()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    import torch
    import torch.distributed as dist
    from oracle.dvm_oracle import BF16, F32, OracleKernel
    from dvm_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    m, n, k = 64, 48, 32
    plan = _collectives(_tp_kernel(rank, world, m, n, k // world).das())
    rs, ag = plan
    rows = m // world
    row0 = (rs["recv"] - rs["send"]) // (n * 4)
    assert row0 == (ag["send"] - ag["recv"]) // (n * 2)
    rng = np.random.default_rng(5)
    a = rng.normal(0, 0.1, (m, k)).astype(np.float32)
    b = rng.normal(0, 0.1, (k, n)).astype(np.float32)
    bias = rng.normal(0, 0.1, (n,)).astype(np.float32)
    ar, br = sharding.ksplit_operands(a, b, rank, world)
    o = OracleKernel()
    partial = o.store(o.cast(o.matmul(o.load(ar, BF16), o.load(br, BF16), False, False), F32))
    t = torch.from_numpy(partial.copy())
    dist.all_reduce(t)                                   # reduce-scatter = the rank's rows of the sum
    mine = t.numpy()[row0:row0 + rows]
    o2 = OracleKernel()
    y = o2.store(o2.cast(W.gelu_tanh(o2, o2.add(o2.load(mine), o2.cast(o2.load(bias, BF16), F32))), BF16))
    parts = [None] * world
    dist.all_gather_object(parts, (row0, y.astype(np.float32)))
    if rank == 0:
        parts.sort(key=lambda p: p[0])
        assert [p[0] for p in parts] == [r * rows for r in range(world)]   # the row blocks tile the result
        got = np.concatenate([p[1] for p in parts], axis=0)
        full = OracleKernel()
        want = full.store(W.matmul_bias_gelu(full, full.load(a, BF16), full.load(b, BF16), full.load(bias, BF16)))
        out.put(float(np.abs(got - want.astype(np.float32)).max()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_tile_the_result_and_match_the_unsplit_graph():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    err = out.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert err <= 1e-2
