"""Tensor-parallel sharding of the packed layout, checked among CPU ranks (gloo,
world size 2): every rank slices the packed tensors exactly as the TP classes
do, computes its part with the CPU oracle, and the collective (all-gather for
column shards, all-reduce for row shards) must reproduce the un-sharded result.
The CUDA forward has no CPU path, so here the per-shard arithmetic is the
oracle's; the GPU tests run the same classes over NCCL."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import nanoquantization_b200 as nq
from oracle import awq_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        K, N, M, g = 512, 256, 5, 128
        c = O.make_case(K, N, M, group_size=g, dtype=torch.float16, seed=31, bias=True)
        full = O.w4a16_ref(c["x"], c["qweight"], c["qscales"], c["qzeros"], c["bias"])

        # column-parallel: slices are whole packed words; all-gather rebuilds the columns
        qw, qs, qz = nq.shard_columns(c["qweight"], c["qscales"], c["qzeros"], world, rank)
        n0, n1 = nq.column_shard_bounds(N, world, rank)
        assert qw.shape == (K, (n1 - n0) // 8) and qs.shape == (K // g, n1 - n0)
        assert np.array_equal(O.unpack_int4(qw.numpy()), c["iw"][:, n0:n1])
        y = O.w4a16_ref(c["x"], qw, qs, qz, c["bias"][n0:n1])
        parts = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(parts, y)
        err_col = float((torch.cat(parts, dim=-1) - full).abs().max())

        # row-parallel: group-boundary slices; partial sums all-reduced, bias on rank 0 only
        qw, qs, qz = nq.shard_rows(c["qweight"], c["qscales"], c["qzeros"], g, world, rank)
        k0, k1 = nq.row_shard_bounds(K, g, world, rank)
        assert qs.shape[0] == (k1 - k0) // g and np.array_equal(O.unpack_int4(qz.numpy()), c["iz"][k0 // g:k1 // g])
        y = O.w4a16_ref(c["x"][:, k0:k1], qw, qs, qz, c["bias"] if rank == 0 else None)
        dist.all_reduce(y)
        err_row = float((y - full).abs().max())

        # the module classes hold shards of the right shapes and load them from full tensors
        col = nq.ColumnParallelWQLinear(4, g, K, N, world, rank, bias=True, output_dtype=torch.float16)
        col.load_full(c["qweight"], c["qscales"], c["qzeros"], c["bias"])
        row = nq.RowParallelWQLinear(4, g, K, N, world, rank, bias=True, output_dtype=torch.float16)
        row.load_full(c["qweight"], c["qscales"], c["qzeros"], c["bias"])
        assert (row.shard.bias is not None) == (rank == 0)
        merged = nq.MergedColumnParallelWQLinear(4, g, K, [N, N // 2], world, rank, output_dtype=torch.float16)
        half = nq.shard_columns(c["qweight"], c["qscales"], c["qzeros"], 2, 0)  # a second, narrower matrix
        merged.load_full([(c["qweight"], c["qscales"], c["qzeros"]), half])
        ym = O.w4a16_ref(c["x"], merged.shard.qweight, merged.shard.qscales, merged.shard.qzeros)
        y_a, y_b = merged.split(ym)
        ref_a = O.w4a16_ref(c["x"], *nq.shard_columns(c["qweight"], c["qscales"], c["qzeros"], world, rank))
        ref_b = O.w4a16_ref(c["x"], *nq.shard_columns(*half, world, rank))
        err_m = max(float((y_a - ref_a).abs().max()), float((y_b - ref_b).abs().max()))
        shapes_ok = (col.shard.qweight.shape == (K, N // world // 8) and row.shard.qweight.shape == (K // world, N // 8)
                     and merged.shard.qweight.shape == (K, (N + N // 2) // world // 8))
        out.put((rank, err_col, err_row, err_m, shapes_ok))
    finally:
        dist.destroy_process_group()


def test_tp_sharding_world2_gloo():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err_col, err_row, err_m, shapes_ok in res:
        assert err_col == 0.0, (rank, err_col)     # columns are independent: identical to the full result
        assert err_row < 1e-4, (rank, err_row)     # fp32 partial sums in another order
        assert err_m == 0.0 and shapes_ok


def test_shard_bounds_reject_bad_splits():
    with pytest.raises(ValueError):
        nq.column_shard_bounds(136, 2, 0)          # 68 columns is not a whole number of packed words
    with pytest.raises(ValueError):
        nq.row_shard_bounds(3200, 128, 2, 0)       # 1600 rows is not a whole number of groups
    assert nq.row_shard_bounds(25600, 128, 8, 7) == (22400, 25600)   # Qwen3-32B down_proj at TP=8: 25 groups
    assert nq.column_shard_bounds(1024, 8, 3) == (384, 512)          # one KV head per rank
