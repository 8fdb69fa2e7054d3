"""The tensor-parallel classes over NCCL on real GPUs (needs at least two)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import nanoquantization_b200 as nq
    from oracle import awq_oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        errs = []
        for (K, N, M) in ((1024, 512, 3), (1024, 512, 200)):
            g = 128
            c = O.make_case(K, N, M, group_size=g, dtype=torch.float16, seed=5, bias=True)
            full = O.w4a16_ref(c["x"], c["qweight"], c["qscales"], c["qzeros"], c["bias"])
            col = nq.ColumnParallelWQLinear(4, g, K, N, world, rank, dev, True, torch.float16, gather_output=True)
            col.load_full(c["qweight"].to(dev), c["qscales"].to(dev), c["qzeros"].to(dev), c["bias"].to(dev))
            errs.append(O.rel_err(col(c["x"].to(dev)), full))
            row = nq.RowParallelWQLinear(4, g, K, N, world, rank, dev, True, torch.float16)
            row.load_full(c["qweight"].to(dev), c["qscales"].to(dev), c["qzeros"].to(dev), c["bias"].to(dev))
            errs.append(O.rel_err(row(row.input_slice(c["x"].to(dev)).contiguous()), full))
        # the peer-memory all-reduce: same sums as NCCL's, identical on every rank, repeatable
        from nanoquantization_b200.layers.peer_comm import PeerAllReduce
        comm = PeerAllReduce(slot_bytes=1 << 18, num_slots=4)
        c = O.make_case(1024, 512, 5, group_size=128, dtype=torch.float16, seed=9)
        row = nq.RowParallelWQLinear(4, 128, 1024, 512, world, rank, dev, False, torch.float16)
        row.load_full(c["qweight"].to(dev), c["qscales"].to(dev), c["qzeros"].to(dev))
        xs = row.input_slice(c["x"].to(dev)).contiguous()
        ref_nccl = row(xs)
        full = O.w4a16_ref(c["x"], c["qweight"], c["qscales"], c["qzeros"])
        outs = [comm.linear_all_reduce(row.shard, xs) for _ in range(11)]   # wraps the 4 slots more than twice
        errs.append(O.rel_err(outs[-1], full))
        same = all(torch.equal(o, outs[0]) for o in outs)
        gathered = [torch.empty_like(outs[0]) for _ in range(world)]
        dist.all_gather(gathered, outs[0])
        same = same and all(torch.equal(g_, outs[0]) for g_ in gathered)
        errs.append(0.0 if same else 1.0)
        errs.append(float((outs[0].float() - ref_nccl.float()).abs().max() / full.abs().max()))
        errs.append(float(comm.status()))
        # the reduction inside the GEMM's finishing kernel (the default above) and the stand-alone
        # all-reduce kernel after a GEMM into the slot give the same bits
        plain = PeerAllReduce(slot_bytes=1 << 18, num_slots=4, fused=False)
        outs2 = [plain.linear_all_reduce(row.shard, xs) for _ in range(5)]
        errs.append(0.0 if all(torch.equal(o, outs[0]) for o in outs2) else 1.0)
        errs.append(float(plain.status()))
        plain.close()
        # ... and with the residual add of the block in the same launches
        res = torch.randn(5, 512, generator=torch.Generator().manual_seed(3)).to(torch.float16).to(dev)
        assert comm.fused_residual_supported(row.shard, 5)
        for _ in range(3):
            h, ssq = comm.linear_all_reduce_residual(row.shard, xs, res)
            errs.append(0.0 if torch.equal(h, outs[0] + res) else 1.0)
            want_ss = (h.float() ** 2).sum(1)
            errs.append(float((ssq.sum(1) - want_ss).abs().max() / want_ss.max()))
        errs.append(float(comm.status()))
        big = comm.linear_all_reduce(row.shard, torch.randn(600, 512, device=dev, dtype=torch.float16))  # too large: NCCL path
        assert big.shape == (600, 512)
        comm.close()
        # prefill-sized results: the two-shot kernel (reduce-scatter + all-gather over peer memory in one launch)
        # against NCCL's sum and the oracle; identical on every rank and from call to call (result slots alternate)
        large = PeerAllReduce(slot_bytes=1 << 18, num_slots=4, large_bytes=4 << 20)
        for Mb in (600, 2048):
            cb = O.make_case(1024, 512, Mb, group_size=128, dtype=torch.float16, seed=21 + Mb)
            xb = row.input_slice(cb["x"].to(dev)).contiguous()
            row.load_full(cb["qweight"].to(dev), cb["qscales"].to(dev), cb["qzeros"].to(dev))
            want = O.w4a16_ref(cb["x"], cb["qweight"], cb["qscales"], cb["qzeros"])
            assert not large.fits(Mb, 512) and large.fits_large(Mb, 512) == ((Mb * 512) % 8 == 0)
            if not large.fits_large(Mb, 512):
                continue
            ys = [large.linear_all_reduce(row.shard, xb) for _ in range(4)]
            errs.append(O.rel_err(ys[-1], want))
            ok = all(torch.equal(y_, ys[0]) for y_ in ys)
            gathered = [torch.empty_like(ys[0]) for _ in range(world)]
            dist.all_gather(gathered, ys[0])
            ok = ok and all(torch.equal(g_, ys[0]) for g_ in gathered)
            errs.append(0.0 if ok else 1.0)
            errs.append(float((ys[0].float() - row(xb).float()).abs().max() / want.abs().max()))
        errs.append(float(large.status()))
        large.close()
        torch.cuda.synchronize()
        out.put((rank, errs))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp_classes_world2_nccl():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in res:
        # same tolerance as the single-GPU parity tests; the row-parallel sum adds one fp16 rounding per rank
        assert max(errs) <= 2e-3, (rank, errs)
