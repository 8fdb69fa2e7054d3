"""Benchmark of the AWQ W4A16 linear path on B200.

Workload ("w4a16_gemm_sweep"): the 30-point GEMM shape sweep at group size 128,
M in {1, 4, 16, 128, 1024, 4096} x (K, N) in {(4096,4096), (4096,12288),
(12288,4096), (5120,25600), (25600,5120)}, fp16, seeded synthetic inputs with
the benchmark's distributions (int4 weights and zero-points uniform in [0,15],
scales uniform in [1e-3,1e-2], activations N(0,1)).  One step is one pass over
all 30 points; the metric is the time of that pass in microseconds (lower is
better).  Weights rotate over enough distinct copies per shape that a call
never finds its weights in L2.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

With --gpus N > 1 (launched by torch.distributed.run) the same sweep runs
tensor-parallel: column-parallel shards along N, row-parallel shards along K on
group boundaries followed by an NCCL all-reduce (strong scaling).

--impl reference times the CPU restatement of the reference arithmetic (unpack
by shifts, (q - z) * s, fp32 matmul) on the host cores: every step is one real
pass over all 30 points.

On one GPU the line also carries `reference_gpu`: the reference's own
WQLinear_GEMM.forward (its Triton kernels, JIT-compiled on this GPU, and
torch.matmul) from the untracked install under baseline/_ref, on the same
tensors, after the timed regions.  With N > 1 it carries `tp_parity`: the
tensor-parallel results checked against the CPU oracle after the timed regions.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

MS = (1, 4, 16, 128, 1024, 4096)
# (K, N, how the layer is sharded under tensor parallelism)
SHAPES = ((4096, 4096, "column"), (4096, 12288, "column"), (12288, 4096, "row"),
          (5120, 25600, "column"), (25600, 5120, "row"))
GROUP = 128
L2_BYTES = 126 * 1024 * 1024


def weight_bytes(K, N, g=GROUP):
    return K * N // 2 + 2 * (K // g) * N + 4 * (K // g) * (N // 8)


def algo_bytes(M, K, N, g=GROUP):
    return weight_bytes(K, N, g) + 2 * M * K + 2 * M * N


def algo_flops(M, K, N):
    return 2 * M * N * K


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tflops_burst": p["bf16_tflops"],
                "tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------
# clocks sampled during the timed region
# --------------------------------------------------------------------------
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx = float(f[1])
            except ValueError:
                continue
            for nm, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------
def shard_shape(K, N, kind, world):
    if world == 1:
        return K, N
    if kind == "column":
        return K, N // world
    return K // world, N


def make_layer(K, N, seed, dev, dtype):
    """A WQLinear_GEMM filled on the device with the benchmark's distributions."""
    import nanoquantization_b200 as nq
    lin = nq.WQLinear_GEMM(4, GROUP, K, N, dev, False, dtype)
    fill_layer(lin, seed, dev, dtype)
    return lin


def fill_layer(lin, seed, dev, dtype):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    K, N = lin.in_features, lin.out_features
    # uniform 32-bit words = uniform nibbles, i.e. int4 weights / zero-points uniform in [0, 15]
    lin.qweight.copy_(torch.randint(-2 ** 31, 2 ** 31, (K, N // 8), generator=g, device=dev, dtype=torch.int64).to(torch.int32))
    lin.qzeros.copy_(torch.randint(-2 ** 31, 2 ** 31, (K // GROUP, N // 8), generator=g, device=dev, dtype=torch.int64).to(torch.int32))
    lin.qscales.copy_((torch.rand(K // GROUP, N, generator=g, device=dev) * 9e-3 + 1e-3).to(dtype))


def make_tp_layer(K, N, kind, world, rank, seed, dev, dtype):
    """The rank's shard of a (K, N) layer as the tensor-parallel class that an engine would use;
    the shard is filled directly (random init) instead of being sliced from a full tensor."""
    import nanoquantization_b200 as nq
    if kind == "column":
        lin = nq.ColumnParallelWQLinear(4, GROUP, K, N, world, rank, dev, False, dtype)
    else:
        lin = nq.RowParallelWQLinear(4, GROUP, K, N, world, rank, dev, False, dtype)
    fill_layer(lin.shard, seed, dev, dtype)
    return lin


def run_ours(args):
    import torch.distributed as dist
    import nanoquantization_b200 as nq  # noqa: F401
    from nanoquantization_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    stage = ["set-up"]
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner out of stdout: one JSON line only
        # A rank may leave through a watchdog below while others are still inside a collective: keep NCCL off
        # NVLink multicast objects, which a vanished rank must not be bound to.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)

        def give_up():
            # a multi-rank run that has not finished by now is stuck (one rank failed, the others wait for it)
            if rank == 0:
                emit(json.dumps({"metric": "w4a16_gemm_sweep_us", "n_gpus": world, "impl": "ours",
                                 "unavailable": f"the run did not finish within {args.max_seconds} s (stage: {stage[0]})"}))
            os._exit(0)
        overall = threading.Timer(args.max_seconds, give_up)
        overall.daemon = True
        overall.start()
    dtype = torch.float16
    lib = _lib.load()
    assert lib.nqb200_device_supported(local) == 1, "not a B200"

    # layers: enough copies per shape that one pass over the copies exceeds L2
    layers, xs_dev, xs_host, ys_host = {}, {}, {}, {}
    for si, (K, N, kind) in enumerate(SHAPES):
        k, n = shard_shape(K, N, kind, world)
        ncopy = max(2, -(-int(1.5 * L2_BYTES) // weight_bytes(k, n)))
        if world == 1:
            layers[si] = [make_layer(k, n, 1000 * si + c, dev, dtype) for c in range(ncopy)]
        else:
            layers[si] = [make_tp_layer(K, N, kind, world, rank, 1000 * si + c + 17 * rank, dev, dtype) for c in range(ncopy)]
        for M in MS:
            g = torch.Generator(device="cpu"); g.manual_seed(M * 31 + si)
            xh = torch.randn(M, k, generator=g).to(dtype).pin_memory()
            xs_host[(si, M)] = xh
            xs_dev[(si, M)] = xh.to(dev)
            ys_host[(si, M)] = torch.empty(M, n, dtype=dtype).pin_memory()
    points = [(si, M) for M in MS for si in range(len(SHAPES))]  # M-major: a shape's reuses are far apart

    # tensor parallelism: the row-parallel layers all-reduce over peer memory (inside the GEMM's finishing
    # kernel for decode sizes, stand-alone peer kernels above that, NCCL beyond the communicator's slot size)
    comm = None
    if world > 1 and not args.nccl_only:
        from nanoquantization_b200.layers.peer_comm import PeerAllReduce
        comm = PeerAllReduce(slot_bytes=2 << 20, num_slots=8, large_bytes=48 << 20, wait_limit_s=10.0)
        for si in layers:
            for lin in layers[si]:
                if hasattr(lin, "attach_comm"):
                    lin.attach_comm(comm)

    def call(si, M, copy, x):
        return layers[si][copy % len(layers[si])](x)  # row-parallel layers all-reduce inside

    # point j of a shape uses weight copy j, so a copy is reused only after the rest of the sweep
    # (>1 GB of other weights) has gone through L2
    def sweep_device(step=0):
        for j, (si, M) in enumerate(points):
            call(si, M, j // len(SHAPES) + step, xs_dev[(si, M)])

    # End to end: every point's activations come from pinned host memory and its result goes back to
    # pinned host memory inside the timed region, through WQLinear_GEMM.forward.  Three streams (copy in,
    # compute, copy out) so that a point's transfers overlap its neighbours' GEMMs, as a serving host would
    # drive a PCIe-attached GPU.
    s_in, s_mm, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in points]
    ev_mm = [torch.cuda.Event() for _ in points]
    used = [False] * len(points)

    def sweep_e2e(step):
        for j, (si, M) in enumerate(points):
            with torch.cuda.stream(s_in):
                if used[j]:
                    s_in.wait_event(ev_mm[j])       # the previous step's GEMM still reads this buffer
                xs_dev[(si, M)].copy_(xs_host[(si, M)], non_blocking=True)
                ev_in[j].record(s_in)
            with torch.cuda.stream(s_mm):
                s_mm.wait_event(ev_in[j])
                y = call(si, M, j // len(SHAPES) + step, xs_dev[(si, M)])
                ev_mm[j].record(s_mm)
            used[j] = True
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_mm[j])
                y.record_stream(s_out)
                ys_host[(si, M)].copy_(y, non_blocking=True)

    def e2e_begin():
        cur = torch.cuda.current_stream()
        for st in (s_in, s_mm, s_out):
            st.wait_stream(cur)

    def e2e_end():
        cur = torch.cuda.current_stream()
        for st in (s_in, s_mm, s_out):
            cur.wait_stream(st)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def capture(fn):
        """The launches of fn() as one CUDA graph (decode-sized calls are launch-bound from Python)."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        return graph

    def timed(fn, steps, begin=None, end=None):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if begin:
            begin()
        for s in range(steps):
            fn(s)
        if end:
            end()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    use_graph = True
    try:
        sweep_graph = capture(sweep_device)  # with tensor parallelism the NCCL all-reduces are captured too
    except RuntimeError:
        if world == 1:
            raise
        use_graph, sweep_graph = False, None  # plain launches if this NCCL build refuses capture
        torch.cuda.synchronize()
    run_sweep = (lambda s: sweep_graph.replay()) if use_graph else sweep_device
    for w in range(max(args.warmup, 3)):
        run_sweep(w)
        e2e_begin(); sweep_e2e(w); e2e_end()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    stage[0] = "timed sweep"
    ms_dev = timed(run_sweep, args.steps)
    ms_e2e = timed(sweep_e2e, args.steps, e2e_begin, e2e_end)

    # per-point pass: each point launched back to back over rotating weight copies
    stage[0] = "per-point pass"
    per_point = []
    for (si, M) in points:
        K, N, kind = SHAPES[si]
        k, n = shard_shape(K, N, kind, world)
        reps = max(8, 2 * len(layers[si])) if M <= 128 else 4

        def burst(si=si, M=M, reps=reps):
            for r in range(reps):
                call(si, M, r, xs_dev[(si, M)])
        fn = capture(burst).replay if use_graph else burst
        for r in range(3):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        per_point.append({"M": M, "K": k, "N": n, "us": us,
                          "kernel": lib.nqb200_gemm_kernel_name(M, n, k, GROUP, 0).decode()})
    clocks = sampler.stop() if rank == 0 else None
    barrier()
    # checker legs, after every timed region
    ref_gpu = tp_parity = None
    if world == 1 and not args.no_reference_gpu:
        ref_gpu = reference_gpu_leg(layers, xs_dev, points, per_point, dev)
    if world > 1:
        if comm is not None:
            for si in layers:
                for lin in layers[si]:
                    if hasattr(lin, "attach_comm"):
                        lin.attach_comm(None)
        stage[0] = "tp_parity"
        tp_parity = tp_parity_leg(world, rank, dev, dtype, comm)
        barrier()
    sweep_graph = fn = None  # graphs hold captured collectives: dropped well before the process group is destroyed
    decode, small, serve = None, None, None
    if not args.no_decode:
        for k in list(layers):
            del layers[k]
        torch.cuda.empty_cache()
        stage[0] = "decode_qwen3_8b"
        decode = decode_bench(world, rank, dev, dtype)
        barrier()
        if world == 1:
            torch.cuda.empty_cache()
            small = engine_bench_0p6b(dev, dtype)

    if rank == 0:
        pk = peaks()
        for p in per_point:
            gbs = algo_bytes(p["M"], p["K"], p["N"]) / p["us"] / 1e3
            tfl = algo_flops(p["M"], p["K"], p["N"]) / p["us"] / 1e6
            p.update({"gbs": round(gbs, 1), "tflops": round(tfl, 2), "hbm_frac": round(gbs / pk["hbm_gbs"], 4),
                      "tensor_frac": round(tfl / pk["tflops_burst"], 4), "us": round(p["us"], 2)})

        def agg(sel, kind):
            pts = [p for p in per_point if sel(p)]
            t = sum(p["us"] for p in pts)
            if kind == "hbm":
                a = sum(algo_bytes(p["M"], p["K"], p["N"]) for p in pts) / t / 1e3
                return {"bound": "hbm", "achieved": round(a, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                        "frac": round(a / pk["hbm_gbs"], 4), "traffic": None, "peak_source": pk["source"],
                        "kernel": pts[0]["kernel"], "points": len(pts)}
            a = sum(algo_flops(p["M"], p["K"], p["N"]) for p in pts) / t / 1e6
            return {"bound": "tensor", "achieved": round(a, 1), "peak": pk["tflops_burst"], "unit": "TFLOP/s",
                    "frac": round(a / pk["tflops_burst"], 4), "traffic": None, "peak_source": pk["source"],
                    "kernel": pts[0]["kernel"], "points": len(pts)}

        # the kernel where the sweep's time goes (about 90 % of the launch-list time): the tcgen05 prefill
        # kernel on its tensor-bound points (M >= 1024)
        dom = per_point[-1]["kernel"]
        roof_prefill = agg(lambda p: p["kernel"] == dom and p["M"] >= 1024, "tensor")
        dom_pts = [p for p in per_point if p["kernel"] == dom and p["M"] >= 1024]
        # DRAM bytes per launch, from the ncu capture of this kernel at M = K = N = 4096 (profiles/): reads 1.19 x
        # the algorithmic read bytes (packed weights + activations), writes 0.32 x the output (the rest is still
        # in L2 when the kernel ends); scaled to the points of the sweep in proportion to those bytes
        roof_prefill["traffic"] = round(sum(1.19 * (weight_bytes(p["K"], p["N"]) + 2 * p["M"] * p["K"]) + 0.32 * 2 * p["M"] * p["N"]
                                            for p in dom_pts) / len(dom_pts))
        roof_prefill["traffic_unit"] = "bytes per launch (mean over the kernel's points)"
        roof_decode = agg(lambda p: p["M"] <= 16, "hbm")
        # ncu: both decode kernels read exactly their algorithmic bytes from DRAM (profiles/)
        roof_decode["traffic"] = round(sum(algo_bytes(p["M"], p["K"], p["N"]) for p in per_point if p["M"] <= 16) / 15)
        h2d = sum(2 * M * shard_shape(*SHAPES[si], world)[0] for (si, M) in points)
        d2h = sum(2 * M * shard_shape(*SHAPES[si], world)[1] for (si, M) in points)
        us_step = ms_dev * 1e3 / args.steps
        line = {
            "metric": "w4a16_gemm_sweep_us", "value": round(us_step, 2), "unit": "us", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(us_step / 1e3, 4),
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": sweep_config(f"tp{world}",
                                   ("device-timed sweep replayed as one CUDA graph" if use_graph else "plain launches") +
                                   "; e2e through WQLinear_GEMM.forward, host<->device copies on their own streams"),
            "e2e": {"value": round(ms_e2e * 1e3 / args.steps, 2), "unit": "us", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h},
            "gpu_launches": args.steps * sum(lib.nqb200_gemm_launch_count(M, *shard_shape(*SHAPES[si], world)[::-1], GROUP, 0)
                                             for (si, M) in points),
            "roofline": roof_prefill, "roofline_decode": roof_decode,
            "clocks": clocks, "points": per_point, "decode_qwen3_8b": decode, "engine_qwen3_0p6b": small,
        }
        if ref_gpu is not None:
            line["reference_gpu"] = ref_gpu
        if tp_parity is not None:
            line["tp_parity"] = tp_parity
        if world == 1:
            line["cpu_baseline"] = cpu_baseline()
    if world == 8 and not args.no_serve and not args.no_decode:
        # The largest configuration: Qwen3-32B architecture, 256 requests, continuous batching, on all 8 GPUs.  The
        # line above stands whatever happens here: past its time budget every rank leaves, rank 0 printing the line
        # without this part (ranks that wait in a collective for one that failed would wait for NCCL's own
        # time-out, ten minutes).
        stage[0] = "serve"
        lock, printed = threading.Lock(), [False]

        def serve_over_budget():
            with lock:
                if printed[0]:
                    return
                printed[0] = True
                if rank == 0:
                    line["serve_qwen3_32b"] = {"unavailable": f"did not finish within {args.serve_budget} s"}
                    emit(json.dumps(line))
            os._exit(0)
        timer = threading.Timer(args.serve_budget, serve_over_budget)
        timer.daemon = True
        timer.start()
        torch.cuda.empty_cache()
        try:
            serve = serve_bench(world, rank, dev, dtype)
        except Exception as exc:
            serve = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        barrier()
        with lock:
            printed[0] = True
        timer.cancel()
        if rank == 0:
            line["serve_qwen3_32b"] = serve
    if rank == 0:
        emit(json.dumps(line))
    stage[0] = "teardown"
    if comm is not None:
        comm.close()
    leave_distributed(world)
    if world > 1:
        overall.cancel()


def sweep_config(parallelism, launch):
    """The `config` object, the same keys in both arms."""
    return {"workload": "w4a16_gemm_sweep g128 M{1,4,16,128,1024,4096} x 5 (K,N) shapes (config 2)",
            "points_per_step": len(MS) * len(SHAPES), "parallelism": parallelism,
            "l2": "weights rotate over copies totalling >1.5x L2 per shape", "launch": launch}


def leave_distributed(world):
    """Tear the process group down.  Captured CUDA graphs hold NCCL kernels of the communicator, so every
    graph is dropped (and collected) and the device is idle before the communicator is destroyed; a
    watchdog ends the process if the teardown still does not return."""
    if world <= 1:
        return
    import gc
    import torch.distributed as dist
    torch.cuda.synchronize()
    dist.barrier()
    gc.collect()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    watchdog = threading.Timer(30.0, lambda: os._exit(0))
    watchdog.daemon = True
    watchdog.start()
    dist.destroy_process_group()
    watchdog.cancel()


# --------------------------------------------------------------------------
# second half of the metric: Qwen3-8B-architecture AWQ decode tokens/s through the engine
# --------------------------------------------------------------------------
def engine_bench_0p6b(dev, dtype, prompts=32, prompt_len=512, steps=256):
    """Random-init Qwen3-0.6B (w4 g128) on one GPU through LLMEngine.generate: 32 prompts of 512 random
    ids, 256 greedy tokens each (prefill, then decode steps as CUDA graphs)."""
    from nanoquantization_b200 import WQLinear_GEMM
    from nanoquantization_b200.engine import LLMEngine
    from nanoquantization_b200.models import QWEN3_SHAPES, Qwen3QuantizedForCausalLM
    shp = QWEN3_SHAPES["qwen3-0.6b"]
    model = Qwen3QuantizedForCausalLM(shp["num_hidden_layers"], 151936, shp["hidden_size"], shp["total_num_heads"],
                                      shp["total_num_kv_heads"], 8192, shp["intermediate_size"], 4, GROUP, 128, False, 1e6,
                                      1e-6, device=dev, dtype=dtype)
    n = 0
    for mod in model.modules():
        if isinstance(mod, WQLinear_GEMM):
            fill_layer(mod, 9000 + n, dev, dtype)
            n += 1
    torch.nn.init.normal_(model.model.embed_tokens.weight, std=0.02)
    torch.nn.init.normal_(model.lm_head.weight, std=0.02)
    model.fuse_projections()
    block = 256
    per_seq = -(-(prompt_len + steps + 8) // block)
    eng = LLMEngine(model, num_blocks=prompts * per_seq + 4, block_size=block, max_batch=prompts)
    g = torch.Generator().manual_seed(2)
    ids = [torch.randint(0, 151936, (prompt_len,), generator=g).tolist() for _ in range(prompts)]
    eng.generate(ids[:prompts], 4)  # warm-up: graphs captured, workspaces allocated
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = eng.generate(ids, steps)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    new = sum(len(o) for o in outs)
    return {"model": "qwen3-0.6b-arch w4 g128 random init", "prompts": prompts, "prompt_len": prompt_len,
            "new_tokens": new, "wall_s": round(dt, 3), "generated_tok_per_s": round(new / dt, 1),
            "total_tok_per_s": round((new + prompts * prompt_len) / dt, 1)}


def serve_bench(world, rank, dev, dtype, requests=256, arch="qwen3-32b", max_batch=64):
    """Continuous batching through LLMEngine.generate: random-init model of `arch` (w4 g128, tensor-parallel
    over `world` ranks), `requests` requests with prompt lengths uniform in [128, 4096] and output lengths
    uniform in [64, 512], random ids, greedy decoding: the benchmark's largest configuration, which names the
    32B architecture on 8 GPUs.  Part of the `--gpus 8` line; on its own as `bench.py --serve`."""
    import torch.distributed as dist
    from nanoquantization_b200 import WQLinear_GEMM
    from nanoquantization_b200.engine import LLMEngine
    from nanoquantization_b200.models import QWEN3_SHAPES, Qwen3QuantizedForCausalLM
    shp = QWEN3_SHAPES[arch]
    model = Qwen3QuantizedForCausalLM(shp["num_hidden_layers"], 151936, shp["hidden_size"], shp["total_num_heads"],
                                      shp["total_num_kv_heads"], 8192, shp["intermediate_size"], 4, GROUP, 128, False, 1e6,
                                      1e-6, tp_size=world, tp_rank=rank, device=dev, dtype=dtype)
    n = 0
    for mod in model.modules():
        if isinstance(mod, WQLinear_GEMM):
            fill_layer(mod, 7000 + n + 100 * rank, dev, dtype)
            n += 1
    torch.nn.init.normal_(model.model.embed_tokens.weight, std=0.02)
    torch.nn.init.normal_(model.lm_head.weight, std=0.02)
    model.fuse_projections()
    comm = None
    if world > 1:
        from nanoquantization_b200.layers.peer_comm import PeerAllReduce
        comm = PeerAllReduce(slot_bytes=2 << 20, num_slots=8, large_bytes=48 << 20, wait_limit_s=10.0)
        model.attach_peer_comm(comm)
    g = torch.Generator().manual_seed(11)   # the same requests on every rank
    plen = torch.randint(128, 4097, (requests,), generator=g).tolist()
    olen = torch.randint(64, 513, (requests,), generator=g).tolist()
    prompts = [torch.randint(0, 151936, (n_,), generator=g).tolist() for n_ in plen]
    block = 256
    eng = LLMEngine(model, num_blocks=max_batch * (-(-(4096 + 512 + 8) // block)) + 4, block_size=block, max_batch=max_batch,
                    max_prefill_tokens=8192)
    eng.generate([p[:300] for p in prompts[:max_batch]], 3)   # warm-up: workspaces, first graphs
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    outs = eng.generate(prompts, olen)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([dt], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    new = sum(len(o) for o in outs)
    assert [len(o) for o in outs] == olen
    out = {"workload": f"{arch}-arch w4 g128 random init, continuous batching", "tp": world, "requests": requests,
           "prompt_tokens": sum(plen), "new_tokens": new, "max_batch": max_batch, "wall_s": round(dt, 2),
           "generated_tok_per_s": round(new / dt, 1), "total_tok_per_s": round((new + sum(plen)) / dt, 1),
           "decode_graphs": len(eng._graphs)}
    if comm is not None:
        out["peer_allreduce_status"] = comm.status()
    return out


def decode_bench(world, rank, dev, dtype, batches=(1, 16, 64), context=2048, steps=16, prefill=True):
    """Random-init Qwen3-8B (w4 g128, tensor-parallel over `world` ranks), sequences with a
    2048-token context in the paged KV cache, greedy decode steps replayed as a CUDA graph."""
    import torch.distributed as dist
    from nanoquantization_b200 import WQLinear_GEMM
    from nanoquantization_b200.engine import LLMEngine, Sequence
    from nanoquantization_b200.models import QWEN3_SHAPES, Qwen3QuantizedForCausalLM
    shp = QWEN3_SHAPES["qwen3-8b"]
    model = Qwen3QuantizedForCausalLM(shp["num_hidden_layers"], 151936, shp["hidden_size"], shp["total_num_heads"],
                                      shp["total_num_kv_heads"], 8192, shp["intermediate_size"], 4, GROUP, 128, False, 1e6,
                                      1e-6, tp_size=world, tp_rank=rank, device=dev, dtype=dtype)
    n = 0
    for mod in model.modules():
        if isinstance(mod, WQLinear_GEMM):
            fill_layer(mod, 5000 + n + 100 * rank, dev, dtype)
            n += 1
    torch.nn.init.normal_(model.model.embed_tokens.weight, std=0.02)
    torch.nn.init.normal_(model.lm_head.weight, std=0.02)
    model.fuse_projections()
    block = 256
    per_seq = -(-(context + steps + 8) // block)
    eng = LLMEngine(model, num_blocks=max(batches) * per_seq + 4, block_size=block, max_batch=max(batches))
    out = {"model": "qwen3-8b-arch w4 g128 random init", "tp": world, "context": context,
           "allreduce_variants": "nccl = NCCL after each row-parallel linear; peer = nqb200_gemm_allreduce "
                                 "(reduced over peer memory by the kernel that finishes the GEMM)",
           "attention": "flash_attn paged" if eng.paged_attention is not None else "sdpa over gathered pages", "points": []}
    g = torch.Generator().manual_seed(1)
    comm = None
    if world > 1:
        from nanoquantization_b200.layers.peer_comm import PeerAllReduce
        comm = PeerAllReduce(slot_bytes=1 << 20, num_slots=8, large_bytes=48 << 20, wait_limit_s=10.0)   # 72 all-reduces per step: a multiple of the slot count
    variants = [("nccl", None)] + ([("peer", comm)] if comm is not None else [])
    for (ar_name, ar_comm), B in [(v, b) for v in variants for b in batches]:
        model.attach_peer_comm(ar_comm)
        eng._graphs.clear()
        seqs = []
        for i in range(B):
            s = Sequence(i, torch.randint(0, 151936, (context,), generator=g).tolist(), 10 ** 9)
            assert eng.blocks.ensure(s, context + steps + 8)
            s.output.append(1)
            seqs.append(s)
        for _ in range(3):
            eng._decode(seqs)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            eng._decode(seqs)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        pt = {"batch": B, "ms_per_step": round(ms, 3), "tok_per_s": round(B / ms * 1e3, 1)}
        if world > 1:
            pt["allreduce"] = ar_name
        if world > 1 and ar_name == "nccl":  # share of the step spent in the 2 all-reduces per layer
            buf = torch.zeros(B, shp["hidden_size"], dtype=dtype, device=dev)
            gr = torch.cuda.CUDAGraph()
            for _ in range(2 * shp["num_hidden_layers"]):
                dist.all_reduce(buf)
            torch.cuda.synchronize()
            with torch.cuda.graph(gr):
                for _ in range(2 * shp["num_hidden_layers"]):
                    dist.all_reduce(buf)
            gr.replay(); torch.cuda.synchronize()
            e0.record(); gr.replay(); e1.record(); torch.cuda.synchronize()
            pt["allreduce_ms_per_step"] = round(e0.elapsed_time(e1), 3)
            pt["allreduce_share"] = round(e0.elapsed_time(e1) / ms, 3)
        out["points"].append(pt)
        for s in seqs:
            eng.blocks.release(s)
    # the configuration's 4096-token prefill: one sequence through the engine's prefill path
    seq = Sequence(10 ** 6, torch.randint(0, 151936, (4096,), generator=g).tolist(), 1)
    if prefill and eng.blocks.ensure(seq, 4096 + 8):
        model.attach_peer_comm(None)
        for _ in range(2):
            eng._prefill([seq])
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            eng._prefill([seq])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 3
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        out["prefill_4096"] = {"ms": round(ms, 3), "tok_per_s": round(4096 / ms * 1e3, 1)}
        eng.blocks.release(seq)
    if comm is not None:
        out["peer_allreduce_status"] = comm.status()
    del eng, model
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------
# checker legs of our arm (after the timed regions)
# --------------------------------------------------------------------------
def reference_gpu_leg(layers, xs_dev, points, per_point, dev):
    """The reference's own WQLinear_GEMM.forward on this GPU, on the same packed tensors and activations:
    its fused Triton kernel below 256 tokens (gemm.py:563-564), its Triton dequantise kernel followed by
    torch.matmul from 256 tokens (gemm.py:558-561).  Unmodified code imported from baseline/_ref; only
    the benchmark's shapes (N % 256 == 0, K % 32 == 0), for which its kernels' edge masks are not reached.
    Per point: microseconds (same rotation over weight copies, replayed as a CUDA graph when the reference
    can be captured) and the output's distance from ours."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "nanoquantization")):
        return {"unavailable": "baseline/_ref holds no install of the reference"}
    try:
        sys.path.insert(0, ref_root)
        from nanoquantization.layers.gemm import WQLinear_GEMM as RefLinear
    except Exception as exc:
        return {"unavailable": f"import of the reference failed: {type(exc).__name__}: {exc}"[:300]}
    finally:
        if ref_root in sys.path:
            sys.path.remove(ref_root)
    out, ours_us = [], {(p["M"], p["K"], p["N"]): p["us"] for p in per_point}
    try:
        refs = {}
        for si, copies in layers.items():
            refs[si] = []
            for lin in copies:
                r = RefLinear(4, GROUP, lin.in_features, lin.out_features, dev, False, lin.qscales.dtype)
                r.qweight, r.qscales, r.qzeros = lin.qweight, lin.qscales, lin.qzeros   # the same memory
                refs[si].append(r)
        graphs = 0
        for (si, M) in points:
            K, N, _ = SHAPES[si]
            x = xs_dev[(si, M)]
            copies = refs[si]
            reps = max(8, 2 * len(copies)) if M <= 128 else 4
            y_ref = copies[0](x)              # compiles the Triton kernels on first use
            y_ours = layers[si][0](x)
            torch.cuda.synchronize()
            err = float((y_ref.float() - y_ours.float()).abs().max() / y_ref.float().abs().max())

            def burst(copies=copies, x=x, reps=reps):
                for r in range(reps):
                    copies[r % len(copies)](x)
            fn, graphed = burst, False
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    burst()
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    burst()
                fn, graphed = g.replay, True
                graphs += 1
            except Exception:
                torch.cuda.synchronize()
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / reps
            mine = ours_us[(M, K, N)]
            out.append({"M": M, "K": K, "N": N, "us": round(us, 2), "ours_us": mine, "speedup": round(us / mine, 2),
                        "rel_err_vs_ours": float(f"{err:.3e}"), "graph": graphed})
            del fn, g
            torch.cuda.empty_cache()
    except Exception as exc:
        torch.cuda.synchronize()
        return {"unavailable": f"the reference did not run on this GPU: {type(exc).__name__}: {exc}"[:400],
                "points_done": out}
    total_ref, total_ours = sum(p["us"] for p in out), sum(p["ours_us"] for p in out)
    small = [p for p in out if p["M"] <= 16]
    return {"what": "reference WQLinear_GEMM.forward (Triton kernels JIT-compiled here, torch.matmul from 256 tokens), "
                    "unmodified, from baseline/_ref; same tensors, per-point bursts over rotating weight copies",
            "sweep_us": round(total_ref, 1), "ours_sweep_us": round(total_ours, 1),
            "speedup_sweep": round(total_ref / total_ours, 2),
            "speedup_decode_points": round(sum(p["us"] for p in small) / sum(p["ours_us"] for p in small), 2),
            "max_rel_err_vs_ours": max(p["rel_err_vs_ours"] for p in out),
            "graphed_points": graphs, "points": out}


def tp_parity_leg(world, rank, dev, dtype, comm):
    """Correctness of the tensor-parallel path on the GPUs of this run: one column-parallel and one
    row-parallel shape of the sweep at 1, 16 and 128 tokens.  Every rank builds the same full tensors from
    a seed and loads its shard; the gathered column-parallel result and the all-reduced row-parallel result
    (through NCCL, and through the peer-memory path when there is one) are compared with the CPU oracle on
    the full tensors, the peer path must give the same bits on every rank and on every repetition, and
    the peer communicator must have recorded no give-up."""
    import torch.distributed as dist
    import nanoquantization_b200 as nq
    from oracle import awq_oracle as O
    res = {"points": 0, "max_rel_err": 0.0, "peer_bits_equal_across_ranks": True, "peer_repeatable": True,
           "nccl_equals_peer_bits": True, "bound": 2e-3}
    for (K, N, kind) in ((4096, 12288, "column"), (12288, 4096, "row")):
        g = torch.Generator().manual_seed(K + N)
        qw = torch.randint(-2 ** 31, 2 ** 31, (K, N // 8), generator=g, dtype=torch.int64).to(torch.int32)
        qz = torch.randint(-2 ** 31, 2 ** 31, (K // GROUP, N // 8), generator=g, dtype=torch.int64).to(torch.int32)
        qs = (torch.rand(K // GROUP, N, generator=g) * 9e-3 + 1e-3).to(dtype)
        x_all = torch.randn(128, K, generator=g).to(dtype)
        W = O.dequantize(qw, qs, qz).float() if rank == 0 else None
        if kind == "column":
            lin = nq.ColumnParallelWQLinear(4, GROUP, K, N, world, rank, dev, False, dtype, gather_output=True)
        else:
            lin = nq.RowParallelWQLinear(4, GROUP, K, N, world, rank, dev, False, dtype)
        lin.load_full(qw.to(dev), qs.to(dev), qz.to(dev))
        for M in (1, 16, 128):
            x = x_all[:M].to(dev)
            xin = lin.input_slice(x).contiguous() if kind == "row" else x
            ys = [("nccl", lin(xin))]
            if kind == "row" and comm is not None:
                lin.attach_comm(comm)
                y1 = lin(xin)
                y2 = lin(xin)
                lin.attach_comm(None)
                res["peer_repeatable"] &= bool(torch.equal(y1, y2))
                parts = [torch.empty_like(y1) for _ in range(world)]
                dist.all_gather(parts, y1)
                res["peer_bits_equal_across_ranks"] &= all(bool(torch.equal(p_, y1)) for p_ in parts)
                res["nccl_equals_peer_bits"] &= bool(torch.equal(y1, ys[0][1]))
                ys.append(("peer", y1))
            torch.cuda.synchronize()
            if rank == 0:
                ref = x_all[:M].float() @ W
                for _name, y in ys:
                    res["max_rel_err"] = max(res["max_rel_err"], O.rel_err(y, ref))
            res["points"] += len(ys)
        del lin
    flags = torch.tensor([int(res["peer_bits_equal_across_ranks"]), int(res["peer_repeatable"]),
                          int(res["nccl_equals_peer_bits"])], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    res["peer_bits_equal_across_ranks"], res["peer_repeatable"], res["nccl_equals_peer_bits"] = (bool(v) for v in flags.tolist())
    res["peer_allreduce_status"] = comm.status() if comm is not None else None
    res["max_rel_err"] = float(f"{res['max_rel_err']:.3e}")
    res["ok"] = bool(res["max_rel_err"] <= res["bound"] and res["peer_bits_equal_across_ranks"] and res["peer_repeatable"]
                     and not res["peer_allreduce_status"]) if rank == 0 else None
    res["note"] = ("nccl_equals_peer_bits is reported, not required: NCCL adds the ranks' 16-bit partial results in its "
                   "own order and precision, the peer path adds them in rank order in fp32 and rounds once")
    return res


# --------------------------------------------------------------------------
# CPU arm: the restatement of the reference arithmetic on the host cores
# --------------------------------------------------------------------------
class CpuSweep:
    """The 30 points on the host: per point, unpack by shifts and (q - z) * s into the 16-bit weight (what
    the reference's forward does on every call, gemm.py:558-564), then the matmul in fp32.  Weights are made
    once per shape (uniform random words = uniform int4 values)."""

    def __init__(self):
        self.shapes = {}
        for si, (K, N, _kind) in enumerate(SHAPES):
            g = torch.Generator().manual_seed(100 + si)
            self.shapes[si] = (
                torch.randint(-2 ** 31, 2 ** 31, (K, N // 8), generator=g, dtype=torch.int64).to(torch.int32),
                (torch.rand(K // GROUP, N, generator=g) * 9e-3 + 1e-3).to(torch.float16),
                torch.randint(-2 ** 31, 2 ** 31, (K // GROUP, N // 8), generator=g, dtype=torch.int64).to(torch.int32))
        self.xs = {}
        for si, (K, N, _kind) in enumerate(SHAPES):
            g = torch.Generator().manual_seed(200 + si)
            big = torch.randn(max(MS), K, generator=g).to(torch.float16)
            for M in MS:
                self.xs[(si, M)] = big[:M]

    def run_pass(self):
        """One pass over all points; returns (seconds, per-point seconds)."""
        from oracle import awq_oracle as O
        per = []
        t_all = time.perf_counter()
        for M in MS:
            for si, (K, N, _kind) in enumerate(SHAPES):
                qw, qs, qz = self.shapes[si]
                t0 = time.perf_counter()
                W = O.dequantize_threaded(qw, qs, qz).float()
                y = self.xs[(si, M)].float() @ W
                per.append({"M": M, "K": K, "N": N, "ms": round((time.perf_counter() - t0) * 1e3, 2)})
                del W, y
        return time.perf_counter() - t_all, per


def cpu_baseline():
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sweep = CpuSweep()
    secs, per = sweep.run_pass()
    return {"value": round(secs * 1e6, 1), "unit": "us", "cores": cores, "kind": "port",
            "sample": ("one real pass over all 30 points of the sweep by the CPU restatement (unpack by shifts, (q-z)*s, "
                       "fp32 matmul; torch and numpy on all host threads), nothing extrapolated"),
            "wall_s": round(secs, 1), "points": per}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    steps, warm = args.steps, args.warmup
    sweep = CpuSweep()
    t_start = time.perf_counter()
    budget_s = args.reference_budget
    warm_done = 0
    for _ in range(min(warm, 1)):       # one pass warms the allocator and the thread pools; more would only cost minutes
        sweep.run_pass()
        warm_done += 1
    passes, per = [], None
    for i in range(steps):
        if passes and (time.perf_counter() - t_start) + passes[-1] > budget_s:
            break                        # a pass takes about 12 s: stop where the next one would pass the wall budget
        secs, per = sweep.run_pass()
        passes.append(secs)
    us = sum(passes) / len(passes) * 1e6
    sample = (f"{len(passes)} real passes over all 30 points by the CPU restatement of the reference arithmetic (unpack by shifts, "
              f"(q-z)*s, fp32 matmul; torch and numpy on all {cores} host threads), nothing extrapolated; {warm_done} warm-up pass")
    line = {"impl": "reference", "metric": "w4a16_gemm_sweep_us", "value": round(us, 1), "unit": "us",
            "n_gpus": args.gpus, "steps": len(passes), "steps_requested": steps, "steps_measured": len(passes),
            "warmup": warm_done, "ms_per_step": round(us / 1e3, 3),
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": sweep_config("host cores", "CPU restatement, one call per point"),
            "cpu_baseline": {"value": round(us, 1), "unit": "us", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": round(us, 1), "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "wall_s": round(time.perf_counter() - t_start, 1), "points": per}
    emit(json.dumps(line))


def run_serve(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    out = serve_bench(world, rank, dev, dtype, requests=args.requests, arch=args.serve)
    if rank == 0:
        emit(json.dumps(out))
    leave_distributed(world)


def run_point(args):
    """One (M, K, N) point launched --reps times over rotating weight copies, timed with CUDA
    events; the small, single-kernel case profilers are pointed at."""
    import nanoquantization_b200 as nq  # noqa: F401
    from nanoquantization_b200 import _lib
    M, K, N = (int(v) for v in args.point.split(","))
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    ncopy = max(2, -(-int(1.5 * L2_BYTES) // weight_bytes(K, N)))
    layers = [make_layer(K, N, 7 + c, dev, dtype) for c in range(ncopy)]
    x = torch.randn(M, K, device=dev).to(dtype)
    def burst():
        for r in range(args.reps):
            layers[r % ncopy](x)
    burst()
    torch.cuda.synchronize()
    fn = burst
    if not args.no_graph:  # replayed as one CUDA graph so that the number is device time, not Python launch time
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            burst()
        fn = graph.replay
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    _lib.check_workspaces()
    us = e0.elapsed_time(e1) * 1e3 / args.reps
    emit(json.dumps({"point": [M, K, N], "reps": args.reps, "us_per_call_incl_launch": round(us, 2),
                      "kernel": _lib.load().nqb200_gemm_kernel_name(M, N, K, GROUP, 0).decode()}))


_REAL_STDOUT = None


def protect_stdout():
    """Libraries (NCCL's version banner, for one) print to stdout; the contract is ONE JSON line
    there.  Everything written to fd 1 from here on goes to stderr; emit() writes to the real stdout."""
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)


def emit(text: str) -> None:
    if _REAL_STDOUT is None:
        print(text, flush=True)
    else:
        os.write(_REAL_STDOUT, (text + "\n").encode())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-decode", action="store_true", help="skip the Qwen3-8B decode tokens/s section")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip the reference's own GPU path (1 GPU)")
    ap.add_argument("--no-serve", action="store_true", help="with --gpus 8: skip the Qwen3-32B continuous-batching workload")
    ap.add_argument("--serve-budget", type=int, default=240, help="seconds the --gpus 8 serving workload may take before the line is printed without it")
    ap.add_argument("--max-seconds", type=int, default=840, help="a multi-GPU run that has not finished by then prints an `unavailable` line and leaves")
    ap.add_argument("--nccl-only", action="store_true", help="tensor parallel: all-reduce through NCCL only")
    ap.add_argument("--reference-budget", type=float, default=330.0,
                    help="--impl reference: wall-clock seconds after which no further pass is started")
    ap.add_argument("--point", default=None, help="M,K,N: run only this point (for profilers)")
    ap.add_argument("--reps", type=int, default=6)
    ap.add_argument("--no-graph", action="store_true", help="with --point: plain launches (what a profiler should see)")
    ap.add_argument("--dtype", default="f16", choices=["f16", "bf16"])
    ap.add_argument("--serve", nargs="?", const="qwen3-32b", default=None,
                    help="instead of the sweep: the continuous-batching workload on this architecture (tensor-parallel under torchrun)")
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--decode-only", type=int, default=0, metavar="BATCH",
                    help="only the Qwen3-8B decode point of this batch size, 1 GPU (the case a launch list is taken of)")
    args = ap.parse_args()
    protect_stdout()
    if args.decode_only:
        torch.cuda.set_device(0)
        dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
        emit(json.dumps(decode_bench(1, 0, torch.device("cuda", 0), dtype, batches=(args.decode_only,), steps=4, prefill=False)))
    elif args.serve:
        run_serve(args)
    elif args.point:
        run_point(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
