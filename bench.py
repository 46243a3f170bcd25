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
            copy of a K-group's activations before its linears, one device->host copy of its outputs after them; the
            copies of a pass run on their own streams beside the linears of the neighbouring K-groups)
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
# DRAM traffic of one launch relative to its packed bytes, from the ncu capture of a launch of this workload
TRAFFIC_RATIO = 1.0024
TRAFFIC_NOTE = ("ncu dram__bytes_read+write on one 4096x12288 K4 launch of this workload: 25.25 MB for 25.19 MB algorithmic "
                "(profiles/packed_gemv_K4_mlp_4096x12288_M1.md); 1.002x, proportional to packed bytes for the other widths")
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
    """nvidia-smi clock / throttle sampling (read-only); `stop(window)` keeps the samples taken inside a wall-clock window."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
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

    def stop(self, window=None):
        """window = (t0, t1) in time.time() seconds: only samples stamped inside it count (the timed region)."""
        import datetime

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
                    if window is not None:
                        ts = datetime.datetime.strptime(c[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                        if ts < window[0] or ts > window[1]:
                            continue
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


def _time_graph(torch, dist, world, dev, fn, reps, calls=1):
    """ms per call of fn(): captured into a CUDA graph when possible, CUDA events, barrier on both sides, max over ranks.
    calls=2 captures two calls in a row per graph: the sharded layers alternate between the two halves of their exchange buffers
    from call to call, and a replayed graph must hold both halves to keep that ordering."""
    once = fn
    if calls > 1:
        fn = lambda: [once() for _ in range(calls)]     # noqa: E731
    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

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
    t = torch.tensor([e0.elapsed_time(e1) / (reps * calls)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def _solo_group(dist, rank, world):
    """A process group that holds this rank alone (every rank creates all of them, as torch.distributed requires)."""
    mine = None
    for r in range(world):
        g = dist.new_group([r])
        if r == rank:
            mine = g
    return mine


def lm_head_record(torch, dist, rank, world, dev, reps):
    """Benchmark configuration 3: LM head 151936x4096 K4, rows sharded over the ranks (strong scaling), the epilogue storing
    into every rank's gather buffer; batch 1 and 8.  With several ranks the same head is also timed on one GPU in the same run
    (every rank for itself), which gives the speed-up.  Three distinct heads rotate so that no launch finds its shard in L2."""
    from htr_b200 import wire
    from htr_b200.sharded import RowShardedLinear

    m, n, K, copies = 151936, 4096, 4, 3
    packed = [wire.random_packed(m, n, K, seed=300 + c, device=dev) for c in range(copies)]
    solo = _solo_group(dist, rank, world) if world > 1 else None
    sharded = [RowShardedLinear(*w, device=dev, gather="peer" if world > 1 else "nccl") for w in packed]
    single = [RowShardedLinear(*w, device=dev, group=solo) for w in packed] if world > 1 else sharded
    out = {"workload": "lm_head_151936x4096_K4_row_sharded",
           "gather": ("batch 1: epilogue peer stores + one cross-rank barrier kernel of the library (htr_peer_barrier); "
                      "batch 8: the tensor-core GEMM with the same peer-store epilogue and barrier") if world > 1 else "none"}
    for M in (1, 8):
        x = torch.randn(M, n, device=dev, generator=torch.Generator(device=dev).manual_seed(M)).bfloat16()
        if world > 1:
            # one row runs on the integer-exact kernel in both forms: the gathered result must be the single-GPU result bit for bit.
            # Eight rows: the shards run the 8-row GEMV, one GPU the tensor-core GEMM (float32 sums in different orders): bf16 rounding
            for a, b in zip(sharded, single):
                ya, yb = a(x), b(x)
                if M == 1 and not torch.equal(ya, yb):
                    raise RuntimeError("row-sharded LM head differs from the single-GPU result")
                if M > 1 and not float((ya.float() - yb.float()).norm() / yb.float().norm()) <= 4e-3:
                    raise RuntimeError("row-sharded LM head (batch 8) is not within bf16 rounding of the single-GPU result")
        t_n = _time_graph(torch, dist, world, dev, lambda: [h(x) for h in sharded], reps, calls=2) / copies
        t_1 = _time_graph(torch, dist, world, dev, lambda: [h(x) for h in single], reps, calls=2) / copies if world > 1 else t_n
        out[f"batch{M}"] = {"us": round(1e3 * t_n, 2), "one_gpu_us": round(1e3 * t_1, 2), "speedup": round(t_1 / t_n, 3),
                            "efficiency": round(t_1 / t_n / world, 3), "packed_GBps": round(payload_bytes(m, n, K) / (t_n * 1e-3) / 1e9, 1)}
        if world > 1:
            # where the time goes: the shard's kernel alone (no hand-over), and the other way of ordering the ranks
            out[f"batch{M}"]["shard_kernel_only_us"] = round(1e3 * _time_graph(torch, dist, world, dev, lambda: [h.local(x) for h in sharded], reps, calls=2) / copies, 2)
            if M == 1:
                from htr_b200 import sharded as sharded_mod
                default_order = sharded_mod.PEER_ORDER
                for order, key in (("flags", "with_delivery_flags_us"), ("barrier", "with_torch_symm_barrier_us")):
                    sharded_mod.PEER_ORDER = order
                    out[f"batch{M}"][key] = round(1e3 * _time_graph(torch, dist, world, dev, lambda: [h(x) for h in sharded], reps, calls=2) / copies, 2)
                sharded_mod.PEER_ORDER = default_order
    if world > 1:
        out["gather_check"] = "batch 1: bit-identical to the single-GPU result; batch 8: within bf16 rounding (4e-3 norm-relative)"
    return out


def moe_record(torch, dist, rank, world, dev, reps, tokens=(1, 8, 32)):
    """Benchmark configuration 4: 64 experts, top-8, SwiGLU 4096 -> 1536 -> 4096, K3, experts dealt to the ranks; two routed
    launches per rank and step, routing on the device, one CUDA graph.  With several ranks the whole layer is also timed on one
    GPU in the same run."""
    from htr_b200 import wire
    from htr_b200.sharded import ExpertParallelMoE

    E, h, inter, K = 64, 4096, 1536, 3
    experts = [dict(gate_up=wire.random_packed(2 * inter, h, K, seed=2 * e, device=dev), down=wire.random_packed(h, inter, K, seed=2 * e + 1, device=dev))
               for e in range(E)]
    solo = _solo_group(dist, rank, world) if world > 1 else None
    moe = ExpertParallelMoE(experts, device=dev)
    moe1 = ExpertParallelMoE(experts, device=dev, group=solo) if world > 1 else moe
    del experts
    out = {"workload": "moe_64x_top8_swiglu_4096_1536_K3",
           "combine": ("the down launch stores each pair's row into every rank (peer stores), one cross-rank barrier, the single-GPU weighted sum; "
                       "every rank holds the same bits; bit-identical to the single-GPU layer when planned like it, else to float32 rounding "
                       "(the timed form plans the launches for the rank's share of the pairs)") if world > 1 else "none"}
    g = torch.Generator().manual_seed(0)
    for T in tokens:
        x = torch.randn(T, h, generator=g).bfloat16().to(dev)
        ids = torch.stack([torch.randperm(E, generator=g)[:8] for _ in range(T)]).to(dev)
        w = torch.rand(T, 8, generator=g)
        w = (w / w.sum(-1, keepdim=True)).to(dev)
        if world > 1:
            moe.plan_for_share = False                      # with the single-GPU launch plan the layer equals one GPU bit for bit
            if not torch.equal(moe(x, ids, w), moe1(x, ids, w)):
                raise RuntimeError("expert-parallel MoE differs from the single-GPU layer")
            moe.plan_for_share = True                       # the default (timed below): same rows to float32 rounding
            a, b = moe(x, ids, w).float(), moe1(x, ids, w).float()
            if not float((a - b).norm() / b.norm()) <= 4e-3:
                raise RuntimeError("expert-parallel MoE differs from the single-GPU layer")
        t_n = _time_graph(torch, dist, world, dev, lambda: moe(x, ids, w), reps, calls=2)
        t_1 = _time_graph(torch, dist, world, dev, lambda: moe1(x, ids, w), reps, calls=2) if world > 1 else t_n
        out[f"tokens{T}"] = {"ms": round(t_n, 4), "one_gpu_ms": round(t_1, 4), "speedup": round(t_1 / t_n, 3)}
    return out


def batch_sweep_record(torch, dev, weights_by_k, reps):
    """Benchmark configuration 1 beyond batch 1: the 4096x12288 linears at batch 1, 4, 8, 16, 64 for every width, over the
    resident copies of the main workload (more than L2 per width), stream-ordered launches through ops.linear, one CUDA graph."""
    from htr_b200 import ops

    out = {"shape_m_x_n": [4096, 12288], "launch_form": "stream-ordered", "kernels": {"1": "packed_gemv_kernel<K,1>", "4": "packed_gemv_mma_kernel<K,8>",
                                                                                      "8": "packed_gemm_tc_kernel<K>", "16": "packed_gemm_tc_kernel<K>", "64": "packed_gemm_tc_kernel<K>"}}
    for K, ws in weights_by_k.items():
        n = ws[0][0].shape[1] * 16
        nbytes = payload_bytes(ws[0][0].shape[0] * 16, n, K)
        row = {}
        for M in (1, 4, 8, 16, 64):
            x = torch.randn(M, n, device=dev, generator=torch.Generator(device=dev).manual_seed(M)).bfloat16()
            ms = _time_graph(torch, None, 1, dev, lambda: [ops.linear(x, *w) for w in ws], reps) / len(ws)
            row[f"M{M}"] = {"us": round(1e3 * ms, 2), "packed_GBps": round(nbytes / (ms * 1e-3) / 1e9, 1)}
        out[f"K{K}"] = row
    return out


def gemv_kernels_record(torch, dev, weights_by_k, reps):
    """The three GEMV kernels side by side at batch 1 on the 4096x12288 linears of the main workload (resident copies, more than
    L2 per width): CUDA cores (the default at one row), warp-level int8 MMA, tcgen05 with the hashes in tensor memory.
    Independent launches (consecutive launches overlap), one CUDA graph per kernel and width."""
    from htr_b200 import _lib, ops

    names = {0: "packed_gemv_kernel<K,1> (CUDA cores)", 1: "packed_gemv_mma_kernel<K,4> (mma.sync u8 x s8)",
             2: "packed_gemv_tm_kernel<K> (tcgen05.mma kind::i8, A operand in tensor memory)"}
    out = {"shape_m_x_n": [4096, 12288], "batch": 1, "launch_form": "independent inputs", "kernels": names}
    try:
        for K, ws in weights_by_k.items():
            n = ws[0][0].shape[1] * 16
            nbytes = payload_bytes(ws[0][0].shape[0] * 16, n, K)
            x = torch.randn(1, n, device=dev, generator=torch.Generator(device=dev).manual_seed(K)).bfloat16()
            row = {}
            for kind in (0, 1, 2):
                _lib.lib.htr_set_gemv_kernel(kind)

                def run():
                    with ops.independent_inputs():
                        for w in ws:
                            ops.linear(x, *w)
                ms = _time_graph(torch, None, 1, dev, run, reps) / len(ws)
                row[f"kind{kind}"] = {"us": round(1e3 * ms, 2), "packed_GBps": round(nbytes / (ms * 1e-3) / 1e9, 1)}
            out[f"K{K}"] = row
    finally:
        _lib.lib.htr_set_gemv_kernel(-1)
    return out


def decoder_record(torch, dist, rank, world, dev):
    """Benchmark configuration 2: the dense 9B-class decoder (36 layers, K4 trunk and head), 16-token prompt, 256 greedy tokens,
    batch 1, one CUDA graph per decode step.  Several ranks = that many replicas (the trunk does not shard)."""
    from htr_b200.decoder import DecoderConfig, PackedDecoder

    model = PackedDecoder(DecoderConfig(), dev, seed=1 + rank)
    prompt = torch.randint(0, 151936, (16,), generator=torch.Generator().manual_seed(2 + rank))
    model.generate(prompt, 8)                               # warm-up
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    toks, t_prompt, t_decode = model.generate(prompt, 256)
    t = torch.tensor([t_prompt, t_decode], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    t_prompt, t_decode = float(t[0]), float(t[1])
    bpt = model.packed_bytes_per_token()
    del model
    torch.cuda.empty_cache()
    return {"workload": "dense_9b_class_K4_trunk_K4_head", "prompt": 16, "new_tokens": 256, "batch": 1, "tokens_per_s": round(world * 256 / t_decode, 2),
            "prompt_s": round(t_prompt, 4), "decode_s": round(t_decode, 4), "packed_bytes_per_token": bpt,
            "packed_GBps_per_gpu": round(bpt * 256 / t_decode / 1e9, 1), "parallelism": "replicas only" if world > 1 else "one GPU"}


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
        n_out = sum(it["m"] for it in items)                     # a rank returns its own rows
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
    flags = flag_ptrs = epoch = wait_status = None
    # how the ranks order themselves after a K-group: "kernel" = the library's barrier kernel, "barrier" = torch symmetric memory's,
    # "flags" = delivery flags raised by the kernels + one bounded wait
    peer_order = os.environ.get("HTR_BENCH_PEER_ORDER", "kernel")
    rank_barrier = None
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
        # delivery flags instead of a barrier: word r of a rank's array counts the launches of rank r whose rows have arrived there
        flags = symm_mem.empty(64, dtype=torch.int32, device=dev)
        flags.zero_()
        fh = symm_mem.rendezvous(flags, dist.group.WORLD)
        flag_ptrs = [int(p) + 4 * rank for p in fh.buffer_ptrs]
        epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        wait_status = torch.zeros(1, dtype=torch.int32, device=dev)
        if peer_order == "kernel":
            from htr_b200.sharded import RankBarrier
            rank_barrier = RankBarrier(world, rank, dev)
            wait_status = rank_barrier.status
        torch.cuda.synchronize()
        dist.barrier()

    def run_group(items, from_host=False, copies=True):
        """copies=False (with from_host): the caller moves the pools between host and device itself (pipelined end-to-end pass)."""
        main = torch.cuda.current_stream()
        xh_pool, xd_pool, yh_pool, yd_pool = items[0]["pools"]
        if from_host and copies:
            xd_pool.copy_(xh_pool, non_blocking=True)
        outs = []
        for it in items:
            xin = it["xd"] if from_host else it["x"]
            if gather_mode == "peer":
                ops.linear_into_peers(xin, *it["w"], None, it["peers"], rank * it["m"], flag_ptrs if peer_order == "flags" else None)
                continue
            y = ops.linear(xin, *it["w"])
            if gather_mode == "nccl":
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    dist.all_gather_into_tensor(it["gathered"], y)
                y.record_stream(side)
                outs.append(it["gathered"][rank])
            else:
                outs.append(y.view(-1))
        if gather_mode == "nccl":
            main.wait_stream(side)
        if gather_mode == "peer":
            # one bounded wait for the group: every rank has delivered the rows of all its launches (nobody reads the peers' rows in
            # the timed passes, so a rank that runs ahead may already overwrite them for the next pass)
            if peer_order == "flags":
                ops.peer_wait(flags, epoch, world, wait_status, count=len(items))
            elif peer_order == "kernel":
                rank_barrier()
            else:
                hdl.barrier(channel=0)
            outs = [it["gathered"][rank] for it in items]
        if from_host:
            # the consumer of a gathered result sits on one host: every rank returns its own rows (together they are the result)
            torch.cat(outs, out=yd_pool)
            if copies:
                yh_pool.copy_(yd_pool, non_blocking=True)

    # warm every kernel, the workspace and NCCL, then capture CUDA graphs (one per K-group and launch form)
    for items in groups:
        run_group(items)
        run_group(items, from_host=True)
    torch.cuda.synchronize()

    # N > 1: what the timed passes gather must be what every rank computed.  Each rank fingerprints its own rows (the operator's
    # plain output), the fingerprints travel by NCCL, and every rank compares them with the rows it received from its peers.
    gather_check = None
    if world > 1:
        def fingerprint(t):
            v = t.contiguous().view(torch.int16).to(torch.int64)
            return torch.stack([v.sum(), (v * torch.arange(1, v.numel() + 1, device=v.device)).sum()])
        for items in groups:
            it = items[0]
            run_group(items)
            mine = fingerprint(ops.linear(it["x"], *it["w"]).view(-1))
            every = torch.empty(world, 2, dtype=torch.int64, device=dev)
            dist.all_gather_into_tensor(every, mine)
            for r in range(world):
                if not torch.equal(fingerprint(it["gathered"][r]), every[r]):
                    raise RuntimeError(f"rank {rank}: the rows gathered from rank {r} differ from what that rank computed")
        gather_check = "bit-identical: every rank's gathered rows carry the fingerprint of the rank that computed them (one linear per K)"
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

    def timed(graphs, steps, passes, from_host=False, independent=False):
        """`steps` steps of `passes` passes each, bracketed by a barrier; returns (total ms, [ms per K-group per step], wall window)."""
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
        # per-width times come from the first pass of every step; the total covers all passes
        marks = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in groups] for _ in range(steps)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        e0.record()
        for s in range(steps):
            one_pass(marks[s])
            for _ in range(passes - 1):
                one_pass()
        e1.record()
        barrier()
        w1 = time.time()
        return e0.elapsed_time(e1), [sum(marks[s][i][0].elapsed_time(marks[s][i][1]) for s in range(steps)) / steps for i in range(len(groups))], (w0, w1)

    # The linears of a pass do not feed one another, so they are launched the way the library asks for such work:
    # declared independent of their predecessor (HTR_LINEAR_INPUT_INDEPENDENT), which lets consecutive launches overlap.
    g_ind = capture(independent=True) if use_graphs else None
    # a step is `passes` passes over the workload, chosen so that the timed region lasts about a second (clock samples then
    # come from inside it); every rank uses rank 0's count
    probe_ms, _, _ = timed(g_ind, 2, 1, independent=True)
    passes = args.passes if args.passes > 0 else max(1, int(1050.0 / max(probe_ms / 2 * args.steps, 1e-3) + 0.999))
    if world > 1:
        pt = torch.tensor([passes], device=dev)
        dist.broadcast(pt, 0)
        passes = int(pt[0])
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms, per_k_ms, window = timed(g_ind, args.steps, passes, independent=True)
    clocks = sampler.stop(window) if rank == 0 else None
    # the same pass in the default, stream-ordered form (what a chain of dependent linears gets)
    side_passes = max(1, passes // 4)
    ov_ms, ov_per_k_ms, _ = timed(capture() if use_graphs else None, args.steps, side_passes)
    # end to end through the public operator: activations from pinned host memory, outputs back to pinned host memory
    e2e_steps = max(1, min(args.steps, 10))
    e2e_form = "one K-group after the other: copy in, 16 linears, copy out"
    e2e_ms = None
    if use_graphs:
        # One graph per pass: the host->device copies of all K-groups run on a copy stream from the start of the pass, a group's
        # linears wait for its own copy only, and its outputs leave on a second copy stream while the next group computes.  Every
        # copy stays inside the timed region; graph replays are serialised, so passes do not overlap one another.
        try:
            cin, cout = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
            whole = torch.cuda.CUDAGraph()
            with torch.cuda.graph(whole):
                main = torch.cuda.current_stream()
                cin.wait_stream(main)
                arrived = []
                with torch.cuda.stream(cin):
                    for items in groups:
                        xh_pool, xd_pool, _, _ = items[0]["pools"]
                        xd_pool.copy_(xh_pool, non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(cin)
                        arrived.append(ev)
                cout.wait_stream(main)
                for items, ev in zip(groups, arrived):
                    main.wait_event(ev)
                    with ops.independent_inputs():
                        run_group(items, from_host=True, copies=False)
                    done = torch.cuda.Event()
                    done.record(main)
                    cout.wait_event(done)
                    with torch.cuda.stream(cout):
                        _, _, yh_pool, yd_pool = items[0]["pools"]
                        yh_pool.copy_(yd_pool, non_blocking=True)
                main.wait_stream(cin)
                main.wait_stream(cout)
            for _ in range(max(3, args.warmup)):
                whole.replay()
            barrier()
            q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            q0.record()
            for _ in range(e2e_steps * side_passes):
                whole.replay()
            q1.record()
            barrier()
            e2e_ms = q0.elapsed_time(q1)
            e2e_form = "one graph per pass: copies on their own streams, overlapped with the linears of the neighbouring K-groups"
        except Exception as e:
            graph_note.append(f"pipelined end-to-end capture failed ({type(e).__name__}); sequential form")
            torch.cuda.synchronize()
            e2e_ms = None
    if e2e_ms is None:
        e2e_ms, _, _ = timed(capture(independent=True, from_host=True) if use_graphs else None, e2e_steps, side_passes, from_host=True, independent=True)
    h2d = sum(items[0]["pools"][0].numel() * 2 for items in groups)
    d2h = sum(items[0]["pools"][2].numel() * 2 for items in groups)

    if wait_status is not None and int(wait_status.item()):
        raise RuntimeError(f"rank {rank}: a bounded wait for peer deliveries ran out (status {int(wait_status.item())})")
    if world > 1:
        t = torch.tensor([ms, e2e_ms, ov_ms] + per_k_ms + ov_per_k_ms, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, ov_ms = float(t[0]), float(t[1]), float(t[2])
        per_k_ms = [float(v) for v in t[3:3 + len(groups)]]
        ov_per_k_ms = [float(v) for v in t[3 + len(groups):]]

    # ---- the other benchmark configurations, as extra keys of the same line (after the headline passes)
    extras = {}
    if not args.no_extras:
        if world == 1:
            by_k = {K: [it["w"] for it in items if it["m"] == 4096] for K, items in zip(WIDTHS, groups)}
            extras["batch_sweep"] = batch_sweep_record(torch, dev, by_k, max(3, args.steps // 2))
            extras["gemv_kernels"] = gemv_kernels_record(torch, dev, by_k, max(3, args.steps // 2))
            del by_k
        # free the headline workload before the larger models are built
        groups.clear()
        del g_ind
        torch.cuda.empty_cache()
        if world == 1:
            extras["decoder"] = decoder_record(torch, dist, rank, world, dev)
        extras["lm_head_strong"] = lm_head_record(torch, dist, rank, world, dev, max(5, args.steps))
        torch.cuda.empty_cache()
        extras["moe_ep"] = moe_record(torch, dist, rank, world, dev, max(5, args.steps))

    if rank == 0:
        peak, peak_kind = measured_peak()
        job_bytes = total_bytes * world
        value = job_bytes * args.steps * passes / (ms * 1e-3) / 1e9
        e2e_value = job_bytes * e2e_steps * side_passes / (e2e_ms * 1e-3) / 1e9
        per_k = {}
        for i, K in enumerate(WIDTHS):
            kb = sum(payload_bytes(m, n, K) for (m, n) in SHAPES) * COPIES
            gbs = kb / (per_k_ms[i] * 1e-3) / 1e9
            per_k[f"K{K}"] = {"GBps_per_gpu": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4),
                              "us_per_launch": round(1e3 * per_k_ms[i] / (len(SHAPES) * COPIES), 3)}
        ogbs = total_bytes * args.steps * side_passes / (ov_ms * 1e-3) / 1e9
        overlapped = {"what": "same pass, default launch form: every launch waits for its predecessor before reading activations",
                      "value": ogbs * world, "unit": "GB/s", "frac_of_peak_per_gpu": ogbs / peak, "passes_per_step": side_passes,
                      "per_K": {f"K{K}": round(sum(payload_bytes(m, n, K) for (m, n) in SHAPES) * COPIES / (ov_per_k_ms[i] * 1e-3) / 1e9, 1)
                                for i, K in enumerate(WIDTHS)}}
        achieved = total_bytes * args.steps * passes / (ms * 1e-3) / 1e9     # per GPU: one kernel family, launches back to back
        line = base_line(args)
        line["config"]["passes_per_step"] = passes
        line.update(value=value, ms_per_step=ms / args.steps, timed_region_s=ms * 1e-3, gpu_launches=launches * args.steps * passes, clocks=clocks,
                    e2e={"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d * side_passes, "d2h_bytes_per_step": d2h * side_passes,
                         "steps": e2e_steps, "passes_per_step": side_passes, "form": e2e_form,
                         "returns": "every rank copies its own rows back to its host" if world > 1 else "all outputs"},
                    roofline={"bound": "hbm", "kernel": "packed_gemv_kernel<K,1>", "achieved": achieved, "peak": peak, "unit": "GB/s",
                              "frac": achieved / peak, "peak_source": f"{peak_kind} copy bandwidth", "traffic": None,
                              "traffic_note": TRAFFIC_NOTE,
                              "bytes_per_launch_avg": total_bytes / launches, "us_per_launch_avg": 1e3 * ms / args.steps / passes / launches,
                              "per_K": per_k},
                    stream_ordered=overlapped,
                    timing="cuda events on the launch stream; " + ("one CUDA graph per K-group" if use_graphs and not graph_note else "eager launches " + "; ".join(graph_note)))
        line["roofline"]["traffic"] = round(TRAFFIC_RATIO * total_bytes / launches)     # scaled from the captured launch (see traffic_note)
        if gather_check:
            line["gather_check"] = gather_check
        line.update(extras)
        if world == 1 and not args.no_cpu:
            gbs, dt, threads, sample = cpu_sample()
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample, "seconds": dt}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_extra(args):
    """The other benchmark configurations on their own (the default run carries them as extra keys of its line):
    lmhead   151936x4096 K4 LM head, batch 1 and 8, rows sharded over the ranks (strong scaling), peer-store gather
    decoder  the 9B-class dense decoder, K4 trunk + K4 head, 16-token prompt + 256 greedy tokens, one sequence per rank
    moe      64 experts, top-8, SwiGLU 4096->1536->4096, K3, 1..32 tokens per step, experts dealt to the ranks
    viterbi  the encoder's trellis search: 1024 tiles per call (the reference encoder's batch), K2..K5, with a CPU sample
    Prints one JSON line per workload (rank 0)."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def time_graph(fn, reps):
        return _time_graph(torch, dist, world, dev, fn, reps)

    if args.workload == "lmhead":
        rec = lm_head_record(torch, dist, rank, world, dev, args.steps)
        if rank == 0:
            print(json.dumps({"metric": "lm_head_us", "unit": "us", "higher_is_better": False, "n_gpus": world, "scaling": "strong", **rec}), flush=True)
    elif args.workload == "decoder":
        rec = decoder_record(torch, dist, rank, world, dev)
        if rank == 0:
            print(json.dumps({"metric": "decode_tokens_per_s", "unit": "tok/s", "value": rec["tokens_per_s"], "n_gpus": world, "scaling": "weak", **rec}), flush=True)
    elif args.workload == "moe":
        rec = moe_record(torch, dist, rank, world, dev, args.steps, tokens=(1, 4, 8, 32))
        if rank == 0:
            print(json.dumps({"metric": "moe_layer_ms", "unit": "ms", "higher_is_better": False, "n_gpus": world, **rec}), flush=True)
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
    ap.add_argument("--passes", type=int, default=0, help="passes over the workload per step (0 = as many as make the timed region last about a second)")
    ap.add_argument("--no-extras", action="store_true", help="skip the extra keys (batch sweep, decoder, LM head, MoE)")
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
