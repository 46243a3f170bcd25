#!/usr/bin/env python
"""Benchmark of the HTR-W1 packed-linear decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Metric: packed-weight GB/s of the batch-1 packed GEMV (bytes = m*n*K/8 + 2m + n/8 + m/8 per linear,
docs/METHODOLOGY.md:89 of the reference).  Workload "mlp_bitrate_sweep_batch1": the MLP-shaped linears
12288x4096 and 4096x12288 at K2, K3, K4 and K5, batch 1, bf16 activations ~N(0,1), synthetic packed weights
(uniform random words are valid streams; throughput is data-independent).  Each (shape, K) exists in COPIES
distinct copies so that every K-group alone is larger than the 126 MB L2: one step is one pass over all of
them, so no launch finds its weights in cache.

One JSON line is printed by rank 0:
  value     device-resident throughput of the whole pass, CUDA-event timed, max over ranks; the linears of a pass are
            independent, so they are launched with HTR_LINEAR_INPUT_INDEPENDENT (consecutive launches overlap);
            `stream_ordered` repeats the pass in the default form, in which each launch waits for its predecessor
  e2e       the same pass through the public operator (htr_b200.ops.linear) with the activations in pinned
            host memory and the outputs copied back to pinned host memory inside the timed region (one host->device
            copy of a K-group's activations before its linears, one device->host copy of its outputs after them)
  roofline  of the GEMV kernel: achieved = algorithmic packed bytes per launch / average launch duration,
            peak = measured HBM copy bandwidth (MEASURED_PEAKS.json, else the fallback 6650 GB/s)
  cpu_baseline  the CPU restatement of the reference's decode + matmul path (oracle/, OpenMP) on a bounded
            sample of the same linears, timed on the host cores of this box
With N > 1 every rank holds its own row shard of N-times taller linears (weak scaling); the bf16 outputs are
all-gathered over NCCL.  `--impl reference` times only the CPU path (rank 0).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = ((12288, 4096), (4096, 12288))      # (m out, n in): up/gate-like and down-like MLP linears
WIDTHS = (2, 3, 4, 5)
COPIES = 8
FALLBACK_HBM_GBS = 6650.0
_CPU_CASES = []          # synthetic linears of the CPU sample, generated once per process


def payload_bytes(m, n, K):
    return m * n * K // 8 + 2 * m + n // 8 + m // 8


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle sampling during the timed region (read-only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.index)], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def lines(self):
        try:
            return sum(1 for _ in open(self.path))
        except Exception:
            return 0

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                c = [t.strip() for t in line.split(",")]
                if len(c) < 9:
                    continue
                try:
                    sm.append(float(c[1]))
                    mx.append(float(c[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def cpu_sample(threads=None, repeats=1):
    """Decode + matmul of one linear per (shape, K) on the host cores with the CPU oracle (the port of the
    reference's wire.dequant + matmul).  Returns (GB/s, seconds, threads, description)."""
    import numpy as np
    from oracle import oracle as O

    O.build()
    c = O.COracle()
    threads = threads or os.cpu_count()
    rng = np.random.default_rng(0)
    cases = _CPU_CASES
    for (m, n) in (SHAPES if not cases else ()):
        for K in WIDTHS:
            qw = rng.integers(-2 ** 31, 2 ** 31, size=(m // 16, n // 16, 8 * K), dtype=np.int64).astype(np.int32)
            sc = (np.abs(rng.standard_normal(m)) * 0.01 + 0.01).astype(np.float16)
            su = rng.integers(0, 256, n // 8).astype(np.uint8)
            sv = rng.integers(0, 256, m // 8).astype(np.uint8)
            x = rng.standard_normal((1, n)).astype(np.float32)
            cases.append((x, qw, sc, su, sv, payload_bytes(m, n, K)))
    t0 = time.perf_counter()
    nbytes = 0
    for _ in range(repeats):
        for x, qw, sc, su, sv, b in cases:
            c.linear(x, qw, sc, su, sv, threads=threads)
            nbytes += b
    dt = time.perf_counter() - t0
    return nbytes / dt / 1e9, dt, threads, f"{repeats} pass(es) over one linear per (shape,K): {len(cases)} linears, {nbytes / 1e6:.1f} MB packed"


def base_line(args, impl=None):
    d = {"metric": "packed_gemv_weight_GBps_batch1", "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
         "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
         "config": {"workload": "mlp_bitrate_sweep_batch1", "shapes_m_x_n": [list(s) for s in SHAPES], "K": list(WIDTHS), "batch": 1,
                    "copies_per_shape_and_K": COPIES, "activations": "bf16 N(0,1)", "weights": "encoder output" if args.real_streams else "uniform random words",
                    "launch_form": "independent linears: htr_linear_ex(HTR_LINEAR_INPUT_INDEPENDENT), consecutive launches overlap; "
                                   "stream_ordered gives the default form",
                    "l2_policy": "inputs larger than L2: every K-group of a pass holds >= 201 MB of distinct packed weights",
                    "sharding": "rows" if args.gpus > 1 else "none",
                    "gather": (os.environ.get("HTR_BENCH_GATHER", "peer") + " (epilogue stores into every rank's buffer over NVLink + one barrier per K-group)"
                               if os.environ.get("HTR_BENCH_GATHER", "peer") == "peer" else "nccl all-gather on a side stream") if args.gpus > 1 else "none"}}
    if impl:
        d["impl"] = impl
    return d


def run_reference(args):
    """CPU arm: every step is one bounded sample (one linear per shape and K) on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    for _ in range(min(args.warmup, 1)):          # the CPU path has nothing to warm beyond a first pass
        cpu_sample()
    vals, secs = [], []
    for _ in range(args.steps):
        gbs, dt, threads, sample = cpu_sample()
        vals.append(gbs)
        secs.append(dt)
    v = sum(1.0 for _ in vals) / sum(1.0 / g for g in vals)       # bytes per step are equal: harmonic mean = total bytes / total time
    line = base_line(args, "reference")
    line.update(value=v, ms_per_step=1e3 * statistics.mean(secs), gpu_launches=0,
                cpu_baseline={"value": v, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample + " per step"},
                e2e={"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from htr_b200 import ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # ---- synthetic packed linears, resident in HBM (each rank: its own row shard of an N-times taller linear)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    groups = []          # per K: list of dict(x, w=(qw, sc, su, sv), gathered, xh, yh, xd)
    total_bytes, launches = 0, 0
    for K in WIDTHS:
        items = []
        for c in range(COPIES):
            for (m, n) in SHAPES:
                qw = torch.randint(-2 ** 31, 2 ** 31, (m // 16, n // 16, 8 * K), dtype=torch.int32, device=dev, generator=g)
                sc = (torch.randn(m, device=dev, generator=g).abs() * 0.01 + 0.01).half()
                su = torch.randint(0, 256, (n // 8,), dtype=torch.uint8, device=dev, generator=g)
                sv = torch.randint(0, 256, (m // 8,), dtype=torch.uint8, device=dev, generator=g)
                x = torch.randn(1, n, device=dev, generator=g).bfloat16()
                items.append(dict(x=x, w=(qw, sc, su, sv), m=m, n=n,
                                  gathered=torch.empty(world, m, dtype=torch.bfloat16, device=dev) if world > 1 else None,
                                  xd=None))
                total_bytes += payload_bytes(m, n, K)
                launches += 1
        groups.append(items)
    if args.real_streams:
        # replace the uniform random words by real encoder output: one synthetic weight per (K, shape), Hessian from activations with
        # 1 % outlier channels, encoded on this GPU (htr_b200.encoder), copied into every buffer of that (K, shape)
        from htr_b200 import encoder
        t_enc = time.time()
        for K, items in zip(WIDTHS, groups):
            done = {}
            for it in items:
                key = (it["m"], it["n"])
                if key not in done:
                    ge = torch.Generator().manual_seed(77 + K + it["m"])
                    W = (torch.randn(it["m"], it["n"], generator=ge) * 0.02).to(dev)
                    X = torch.randn(512, it["n"], generator=ge)
                    X[:, torch.randperm(it["n"], generator=ge)[: it["n"] // 100]] *= 10.0
                    X = X.to(dev)
                    r = encoder.encode_group([{"W": W, "H": X.T @ X / 512}], K, seed=1234)[0]
                    done[key] = (r["qweight"], r["scales"], r["su"], r["sv"])
                    del W, X, r
                for dst, src in zip(it["w"], done[key]):
                    dst.copy_(src)
            torch.cuda.empty_cache()
        if rank == 0:
            print(f"# encoded {len(WIDTHS) * len(SHAPES)} matrices in {time.time() - t_enc:.1f} s", file=sys.stderr, flush=True)
    # end-to-end form: the activations of a K-group travel in one host->device copy (pinned pool), its outputs in one
    # device->host copy; the items hold views of the pools
    for items in groups:
        n_in = sum(it["n"] for it in items)
        n_out = sum(max(world, 1) * it["m"] for it in items)
        xh_pool, xd_pool = torch.empty(n_in, dtype=torch.bfloat16).pin_memory(), torch.empty(n_in, dtype=torch.bfloat16, device=dev)
        yh_pool, yd_pool = torch.empty(n_out, dtype=torch.bfloat16).pin_memory(), torch.empty(n_out, dtype=torch.bfloat16, device=dev)
        at = 0
        for it in items:
            xh_pool[at:at + it["n"]].copy_(it["x"].view(-1).cpu())
            it["xd"] = xd_pool[at:at + it["n"]].view(1, it["n"])
            at += it["n"]
        items[0]["pools"] = (xh_pool, xd_pool, yh_pool, yd_pool)
    # N > 1: every rank's epilogue stores its rows into all ranks' gather buffers (symmetric memory, plain NVLink stores);
    # one cross-rank barrier per K-group orders the ranks.  HTR_BENCH_GATHER=nccl uses NCCL all-gathers on a side stream instead.
    side = torch.cuda.Stream(device=dev)
    gather_mode = os.environ.get("HTR_BENCH_GATHER", "peer") if world > 1 else "none"
    hdl = None
    if gather_mode == "peer":
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        elems = sum(world * it["m"] for items in groups for it in items)
        pool = symm_mem.empty(elems, dtype=torch.bfloat16, device=dev)
        hdl = symm_mem.rendezvous(pool, dist.group.WORLD)
        bases = [int(p) for p in hdl.buffer_ptrs]
        off = 0
        for items in groups:
            for it in items:
                it["gathered"] = pool[off:off + world * it["m"]].view(world, it["m"])
                it["peers"] = [b + off * 2 for b in bases]
                off += world * it["m"]

    def run_group(items, from_host=False):
        main = torch.cuda.current_stream()
        xh_pool, xd_pool, yh_pool, yd_pool = items[0]["pools"]
        if from_host:
            xd_pool.copy_(xh_pool, non_blocking=True)
        outs = []
        for it in items:
            xin = it["xd"] if from_host else it["x"]
            if gather_mode == "peer":
                ops.linear_into_peers(xin, *it["w"], None, it["peers"], rank * it["m"])
                continue
            y = ops.linear(xin, *it["w"])
            if gather_mode == "nccl":
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    dist.all_gather_into_tensor(it["gathered"], y)
                y.record_stream(side)
                outs.append(it["gathered"].view(-1))
            else:
                outs.append(y.view(-1))
        if gather_mode == "nccl":
            main.wait_stream(side)
        if gather_mode == "peer":
            hdl.barrier(channel=0)
            outs = [it["gathered"].view(-1) for it in items]
        if from_host:
            torch.cat(outs, out=yd_pool)
            yh_pool.copy_(yd_pool, non_blocking=True)

    # warm every kernel, the workspace and NCCL, then capture CUDA graphs (one per K-group and launch form)
    for items in groups:
        run_group(items)
        run_group(items, from_host=True)
    torch.cuda.synchronize()
    use_graphs = not args.no_graphs

    graph_note = []

    def capture(independent=False, from_host=False):
        out = []
        try:
            for items in groups:
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    if independent:
                        with ops.independent_inputs():
                            run_group(items, from_host)
                    else:
                        run_group(items, from_host)
                out.append(gr)
        except Exception as e:                   # e.g. a collective that cannot be captured: time eager launches instead
            graph_note.append(f"capture failed ({type(e).__name__}); eager launches")
            torch.cuda.synchronize()
            return None
        return out

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(graphs, steps, from_host=False, independent=False):
        """K steps bracketed by a barrier; returns (total ms, [ms per K-group per step])."""
        def one_pass(marks=None):
            for i, items in enumerate(groups):
                if marks is not None:
                    marks[i][0].record()
                if graphs is not None:
                    graphs[i].replay()
                elif independent:
                    with ops.independent_inputs():
                        run_group(items, from_host)
                else:
                    run_group(items, from_host)
                if marks is not None:
                    marks[i][1].record()
        for _ in range(max(3, args.warmup)):
            one_pass()
        barrier()
        marks = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in groups] for _ in range(steps)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(steps):
            one_pass(marks[s])
        e1.record()
        barrier()
        return e0.elapsed_time(e1), [sum(marks[s][i][0].elapsed_time(marks[s][i][1]) for s in range(steps)) / steps for i in range(len(groups))]

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # The linears of a pass do not feed one another, so they are launched the way the library asks for such work:
    # declared independent of their predecessor (HTR_LINEAR_INPUT_INDEPENDENT), which lets consecutive launches overlap.
    ms, per_k_ms = timed(capture(independent=True) if use_graphs else None, args.steps, independent=True)
    # the same pass in the default, stream-ordered form (what a chain of dependent linears gets)
    ov_ms, ov_per_k_ms = timed(capture() if use_graphs else None, args.steps)
    # end to end through the public operator: activations from pinned host memory, outputs back to pinned host memory
    e2e_steps = max(1, min(args.steps, 10))
    e2e_ms, _ = timed(capture(independent=True, from_host=True) if use_graphs else None, e2e_steps, from_host=True, independent=True)
    if rank == 0 and world == 1:
        # the timed regions last a fraction of a second; keep the same load up (untimed) until the sampler has a few samples
        t_end = time.time() + 2.0
        while sampler.lines() < 5 and time.time() < t_end:
            timed(None, 1, independent=True)
    clocks = sampler.stop() if rank == 0 else None
    h2d = sum(items[0]["pools"][0].numel() * 2 for items in groups)
    d2h = sum(items[0]["pools"][2].numel() * 2 for items in groups)

    if world > 1:
        t = torch.tensor([ms, e2e_ms, ov_ms] + per_k_ms + ov_per_k_ms, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, ov_ms = float(t[0]), float(t[1]), float(t[2])
        per_k_ms = [float(v) for v in t[3:3 + len(groups)]]
        ov_per_k_ms = [float(v) for v in t[3 + len(groups):]]

    if rank == 0:
        peak, peak_kind = measured_peak()
        job_bytes = total_bytes * world
        value = job_bytes * args.steps / (ms * 1e-3) / 1e9
        e2e_value = job_bytes * e2e_steps / (e2e_ms * 1e-3) / 1e9
        per_k = {}
        for i, K in enumerate(WIDTHS):
            kb = sum(payload_bytes(m, n, K) for (m, n) in SHAPES) * COPIES
            gbs = kb / (per_k_ms[i] * 1e-3) / 1e9
            per_k[f"K{K}"] = {"GBps_per_gpu": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4),
                              "us_per_launch": round(1e3 * per_k_ms[i] / (len(SHAPES) * COPIES), 3)}
        ogbs = total_bytes * args.steps / (ov_ms * 1e-3) / 1e9
        overlapped = {"what": "same pass, default launch form: every launch waits for its predecessor before reading activations",
                      "value": ogbs * world, "unit": "GB/s", "frac_of_peak_per_gpu": ogbs / peak,
                      "per_K": {f"K{K}": round(sum(payload_bytes(m, n, K) for (m, n) in SHAPES) * COPIES / (ov_per_k_ms[i] * 1e-3) / 1e9, 1)
                                for i, K in enumerate(WIDTHS)}}
        achieved = total_bytes * args.steps / (ms * 1e-3) / 1e9     # per GPU: one kernel family, launches back to back
        line = base_line(args)
        line.update(value=value, ms_per_step=ms / args.steps, gpu_launches=launches * args.steps, clocks=clocks,
                    e2e={"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps},
                    roofline={"bound": "hbm", "kernel": "packed_gemv_kernel<K,1>", "achieved": achieved, "peak": peak, "unit": "GB/s",
                              "frac": achieved / peak, "peak_source": f"{peak_kind} copy bandwidth", "traffic": None,
                              "traffic_note": "ncu dram__bytes_read+write on one 4096x12288 K4 launch of this workload: 25.25 MB for "
                                              "25.19 MB algorithmic (profiles/packed_gemv_K4_mlp_4096x12288_M1.md); 1.002x, "
                                              "proportional to packed bytes for the other widths",
                              "bytes_per_launch_avg": total_bytes / launches, "us_per_launch_avg": 1e3 * ms / args.steps / launches,
                              "per_K": per_k},
                    stream_ordered=overlapped,
                    timing="cuda events on the launch stream; " + ("one CUDA graph per K-group" if use_graphs and not graph_note else "eager launches " + "; ".join(graph_note)))
        line["roofline"]["traffic"] = round(1.0024 * total_bytes / launches)     # scaled from the captured launch (see traffic_note)
        if world == 1 and not args.no_cpu:
            gbs, dt, threads, sample = cpu_sample()
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample, "seconds": dt}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_extra(args):
    """Further workloads of the benchmark configurations, one GPU (or N ranks for the sharded LM head):
    lmhead   151936x4096 K4 LM head, batch 1 and 8, rows sharded over the ranks (strong scaling), peer-store gather
    decoder  the 9B-class dense decoder, K4 trunk + K4 head, 16-token prompt + 256 greedy tokens, one sequence
    moe      64 experts, top-8, SwiGLU 4096->1536->4096, K3, 1..32 tokens per step
    viterbi  the encoder's trellis search: 1024 tiles per call (the reference encoder's batch), K2..K5, with a CPU sample
    Prints one JSON line per workload (rank 0)."""
    import torch
    import torch.distributed as dist
    from htr_b200 import ops, wire

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peak, peak_kind = measured_peak()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def time_graph(fn, reps):
        fn(); sync_all()
        g = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(g):
                fn()
            run = g.replay
        except Exception:
            torch.cuda.synchronize()
            run = fn
        for _ in range(3):
            run()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            run()
        e1.record()
        sync_all()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    if args.workload == "lmhead":
        from htr_b200.sharded import RowShardedLinear
        m, n, K = 151936, 4096, 4
        copies = 3                                              # distinct heads rotate so that no launch finds its shard in L2
        heads = []
        for c in range(copies):
            qw, sc, su, sv = wire.random_packed(m, n, K, seed=300 + c)
            heads.append(RowShardedLinear(qw, sc, su, sv, device=dev, gather="peer" if world > 1 else "nccl"))
        for M in (1, 8):
            x = torch.randn(M, n, device=dev).bfloat16()
            ms = time_graph(lambda: [h(x) for h in heads], args.steps) / copies
            if rank == 0:
                gbs = payload_bytes(m, n, K) / (ms * 1e-3) / 1e9
                print(json.dumps({"metric": "lm_head_packed_GBps", "unit": "GB/s", "value": gbs, "n_gpus": world, "scaling": "strong",
                                  "ms_per_step": ms, "frac_of_peak_per_gpu": gbs / world / peak, "tokens_per_s": M / (ms * 1e-3),
                                  "config": {"workload": "lm_head_151936x4096_K4_row_sharded", "batch": M, "gather": "peer stores + barrier" if world > 1 else "none"}}), flush=True)
    elif args.workload == "decoder":
        # the dense trunk does not shard (an all-gather per linear would cost more than the step): N GPUs = N replicas, each
        # decoding its own sequence; the aggregate counts all of them over the slowest rank's time
        from htr_b200.decoder import DecoderConfig, PackedDecoder
        model = PackedDecoder(DecoderConfig(), dev, seed=1 + rank)
        prompt = torch.randint(0, 151936, (16,), generator=torch.Generator().manual_seed(2 + rank))
        model.generate(prompt, 8)                               # warm-up
        sync_all()
        toks, t_prompt, t_decode = model.generate(prompt, 256)
        t = torch.tensor([t_prompt, t_decode], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_prompt, t_decode = float(t[0]), float(t[1])
        bpt = model.packed_bytes_per_token()
        if rank == 0:
            print(json.dumps({"metric": "decode_tokens_per_s", "unit": "tok/s", "value": world * 256 / t_decode, "n_gpus": world,
                              "scaling": "weak", "wall_tokens_per_s_incl_prompt": world * 256 / (t_prompt + t_decode), "prompt_s": t_prompt,
                              "decode_s": t_decode, "packed_GBps": world * bpt * 256 / t_decode / 1e9,
                              "frac_of_peak_per_gpu": bpt * 256 / t_decode / 1e9 / peak, "packed_bytes_per_token": bpt,
                              "config": {"workload": "dense_9b_class_K4_trunk_K4_head", "prompt": 16, "new_tokens": 256, "batch": 1,
                                         "weights": "random packed", "graph": "one CUDA graph per decode step",
                                         "parallelism": "replicas only" if world > 1 else "one GPU"}}), flush=True)
    elif args.workload == "moe":
        from htr_b200.sharded import ExpertParallelMoE
        E, h, inter, K = 64, 4096, 1536, 3
        experts = [dict(gate_up=wire.random_packed(2 * inter, h, K, seed=2 * e), down=wire.random_packed(h, inter, K, seed=2 * e + 1)) for e in range(E)]
        moe = ExpertParallelMoE(experts, device=dev)
        g = torch.Generator().manual_seed(0)
        for T in (1, 4, 8, 32):
            x = torch.randn(T, h, generator=g).bfloat16().to(dev)
            ids = torch.stack([torch.randperm(E, generator=g)[:8] for _ in range(T)])
            w = torch.rand(T, 8, generator=g); w = (w / w.sum(-1, keepdim=True)).to(dev)
            ids_d = ids.to(dev)
            ms = time_graph(lambda: moe(x, ids_d, w), args.steps)          # grouped launches, routing on the device, graph replay
            active = len(set(ids.flatten().tolist()))
            nbytes = active * (payload_bytes(2 * inter, h, K) + payload_bytes(h, inter, K)) / max(world, 1)
            if rank == 0:
                print(json.dumps({"metric": "moe_layer_ms", "unit": "ms", "value": ms, "higher_is_better": False, "n_gpus": world,
                                  "tokens_per_s": T / (ms * 1e-3), "active_experts": active, "packed_GBps_per_gpu": nbytes / (ms * 1e-3) / 1e9,
                                  "config": {"workload": "moe_64x_top8_swiglu_4096_1536_K3", "tokens": T, "routing": "on device; two grouped GEMV launches per layer (gate_up, down), CUDA graph"}}), flush=True)
    elif args.workload == "viterbi":
        from htr_b200 import encoder
        B = 1024                                                 # max_batch of the reference encoder (htr/encode.py:47)
        g = torch.Generator().manual_seed(5)
        x = (torch.randn(B, 256, generator=g) * (1.0 + 0.25 * torch.rand(B, 1, generator=g))).to(dev)
        rs = (torch.rand(B, 16, generator=g) + 0.5).repeat_interleave(16, dim=1) ** 2
        w = (rs / rs.mean(dim=1, keepdim=True)).to(dev)
        cpu = None
        if not args.no_cpu:
            sys.path.insert(0, ROOT)
            from oracle import oracle
            oracle.build()
            cpu = oracle.COracle()
        for K in (2, 3, 4, 5):
            encoder.viterbi(x, w, None, K)
            ms = time_graph(lambda: encoder.viterbi(x, w, None, K), max(3, args.steps // 4))
            line = {"metric": "viterbi_tiles_per_s", "unit": "tiles/s", "value": B / (ms * 1e-3), "n_gpus": 1, "ms_per_call": ms,
                    "us_per_tile": ms * 1e3 / B, "candidates_per_s": B * 2 * 256 * 65536 / (ms * 1e-3),
                    "config": {"workload": "trellis_search_1024_tiles_x256_tailbiting", "K": K, "data": "synthetic N(0,1) targets, row-scale weights"}}
            if cpu is not None:
                nt = cpu.num_threads()
                t0 = time.perf_counter()
                cpu.viterbi(x[:nt].cpu().numpy(), w[:nt].cpu().numpy(), K)
                dt = time.perf_counter() - t0
                line["cpu_baseline"] = {"value": nt / dt, "unit": "tiles/s", "cores": nt, "kind": "port", "sample": f"{nt} tiles, one per core"}
            print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_case(spec):
    """A small fixed case for a profiler: `copies` random packed linears of one shape (more than L2 in total when the shape
    allows), each called once per repetition through `ops.linear`, eagerly.  spec: K=4,m=4096,n=12288,M=64[,copies=6,reps=1,dtype=bf16]"""
    import torch
    from htr_b200 import ops, wire
    if spec.startswith("viterbi:"):                          # viterbi:K=4,B=592 -- one call of the trellis search on B seeded tiles
        from htr_b200 import encoder
        kv = dict(item.split("=") for item in spec[len("viterbi:"):].split(","))
        K, B = int(kv["K"]), int(kv["B"])
        g = torch.Generator().manual_seed(5)
        x = torch.randn(B, 256, generator=g).cuda()
        w = (torch.rand(B, 256, generator=g) + 0.5).cuda()
        st, cost = encoder.viterbi(x, w, None, K, return_cost=True)
        torch.cuda.synchronize()
        print(json.dumps({"case": spec, "mean_cost": float(cost.mean())}))
        return
    kv = dict(item.split("=") for item in spec.split(","))
    K, m, n, M = int(kv["K"]), int(kv["m"]), int(kv["n"]), int(kv["M"])
    copies, reps = int(kv.get("copies", 6)), int(kv.get("reps", 1))
    dtype = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[kv.get("dtype", "bf16")]
    dev = torch.device("cuda:0")
    ws = [wire.random_packed(m, n, K, seed=s, device=dev) for s in range(copies)]
    x = torch.randn(M, n, device=dev).to(dtype)
    for _ in range(reps):
        for w in ws:
            ops.linear(x, *w)
    torch.cuda.synchronize()
    print(json.dumps({"case": spec, "launches": copies * reps, "gemm_errors": ops.gemm_error_codes()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--no-graphs", action="store_true", help="launch eagerly instead of replaying CUDA graphs")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--workload", default="mlp", choices=("mlp", "lmhead", "decoder", "moe", "viterbi"),
                    help="mlp = the default benchmark line; the others print lines for the remaining configurations")
    ap.add_argument("--real-streams", action="store_true",
                    help="mlp workload: packed words from the device-side encoder (real tail-biting streams) instead of uniform random words")
    ap.add_argument("--case", default=None, help="run one small fixed case for a profiler and exit, e.g. K=4,m=4096,n=12288,M=64")
    args = ap.parse_args()
    if args.case:
        run_case(args.case)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload != "mlp":
        run_extra(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
