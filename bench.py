#!/usr/bin/env python
"""Benchmark of the B200-native web-rwkv hot path: Int8 batch-1 decode of an RWKV-v6-shaped model.

Workload (the configuration the target is quoted on): RWKV-v6 7B-shaped random-init model (n_embd 4096,
32 layers, FFN 14336, vocab 65536), every layer Int8 through the quantizer, a 64-token seeded prompt, then
batch-1 decode.  One *step* = `--decode` decoded tokens (default 256).

  value  tokens/s with the step's inputs (embedding rows) already resident in HBM and the logits left
         on the device: one stream-ordered device copy + the decode job per token.
  e2e    tokens/s through the reference-facing call (`SimpleRuntime::infer` = wrk_runtime_infer) with
         host token ids in and host logits out every token (pinned H2D of the embedding row and
         cursors, D2H of the [vocab] fp32 logits, greedy arg-max on the host feeding the next token).
  checked       before anything is timed, the logits of one decoded token from the fused job are compared
                with the one-launch-per-reference-op job of the same model (max-abs difference reported).
  roofline      the Int8 GEMV kernel (dominant: it streams ~91 % of a decode step's bytes), timed with
                CUDA events over a loop that runs every quantized matmul of every layer at T = 1 in
                model order (weights of all layers = 7 GB, larger than L2).
  decode_1p6b   secondary: the same measurement of `value` on the 1.6B-shaped model (BASELINE config 2).
  prefill       secondary: one 256-token chunk of the headline model through wrk_runtime_infer.
  cpu_baseline  the CPU oracle (a port of the reference's shader arithmetic; the reference itself is
                Rust + WGSL and cannot be built here) decoding a bounded sample on the host cores.

`--impl reference` times that CPU port on the same workload (bounded sample per step).
`--sweep matmul|wkv` runs the op-level sweep (BASELINE config 5) instead and prints one line per point.
With N > 1 GPUs every rank decodes its own replica of the same model (data-parallel replicas, weak
scaling, no data-path collective).
"""
import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def host_threads():
    """Cores this process may run on.  Launchers such as torch.distributed.run export OMP_NUM_THREADS=1 to
    their children; the CPU arms state their own thread count instead, before the OpenMP runtime loads."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


os.environ["OMP_NUM_THREADS"] = str(host_threads())

import numpy as np  # noqa: E402

CONFIG = "v6-7b"
SECONDARY = "v6-1.6b"
PROMPT = 64
DECODE = 256
SEED_WEIGHTS, SEED_TOKENS = 1002, 2002

# dram read + write per launch over algorithmic bytes, from the ncu capture of the GEMV kernel summarised
# under profiles/ (every Int8 launch of the captured token measured 1.01)
NCU_TRAFFIC_RATIO = 1.01


def max_over_ranks(value, dist, device="cuda"):
    """MAX of a per-rank scalar over the process group (identity without one)."""
    if dist is None:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def whole_job_rate(world, steps, units_per_step, ms):
    """Units all ranks processed divided by the slowest rank's time."""
    return world * steps * units_per_step / (ms * 1e-3)


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons during the timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])), mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_model(wrk, rt, synth, ctx, config, num_layer=None, keep=False):
    version, C, L, F, V = synth.CONFIGS[config]
    L = num_layer or L
    builder = rt.ModelBuilder(ctx)
    kept = {}
    for name, arr in synth.iter_tensors(config, SEED_WEIGHTS, L):
        builder.add_tensor(name, arr)
        if keep:
            kept[name] = arr
    builder.quant({i: wrk.QUANT_INT8 for i in range(L)})
    model = builder.build()
    del builder
    return model, kept, (version, C, L, F, V)


def serialize_round_trip(rt, ctx, model):
    """Writes the quantized model to a file and restores it (what a server does on every start after the first);
    returns the times next to which `model_build_s` (quantizing from fp16) is read."""
    import shutil
    import tempfile
    folder = tempfile.mkdtemp(prefix="wrk_model_")
    try:
        if shutil.disk_usage(folder).free < 24 << 30:
            return {"skipped": "less than 24 GB free for the model file"}
        path = os.path.join(folder, "model.cbor")
        t0 = time.perf_counter()
        model.save(path)
        t1 = time.perf_counter()
        loaded = rt.Model.load(ctx, path)
        ctx.synchronize()
        t2 = time.perf_counter()
        same = all(np.array_equal(a, b) for name in ("att.w_k", "ffn.w_v")
                   for a, b in zip(model.matrix_parts(0, name)[1:3], loaded.matrix_parts(0, name)[1:3]))
        del loaded
        return {"save_s": t1 - t0, "load_s": t2 - t1, "file_gb": os.path.getsize(path) / 1e9, "layer0_bytes_identical": bool(same)}
    except Exception as e:  # a full disk must not cost the benchmark
        return {"failed": str(e)[:200]}
    finally:
        shutil.rmtree(folder, ignore_errors=True)


def step_bytes(C, L, F, V, S=64):
    """Algorithmic HBM bytes of one batch-1 v6 Int8 decode token and of its quantized GEMVs."""
    int8 = lambda k, m: k * m * (1 + 4 / 128) + 2 * k + 4 * m  # weights + scales + fp16 x + <=fp32 y
    gemv = L * (6 * int8(C, C) + int8(C, F) + int8(F, C))
    adapters = L * 2 * (C * 160 + 5 * 32 * C + C * 64 + 64 * C)
    state = L * 2 * C * (S + 2) * 4
    head = 2 * C * V
    return gemv + adapters + state + head, gemv, 8 * L


def gemv_roofline(wrk, rt, ctx, model, dims, reps):
    """Times every Int8 matmul of every layer at T = 1 in model order; returns (avg seconds per launch,
    algorithmic bytes per launch, launches per pass)."""
    version, C, L, F, V = dims
    lib = wrk.lib()
    import ctypes
    ops = []
    x_c = ctx.from_numpy(np.random.default_rng(1).standard_normal((1, C)).astype(np.float16))
    x_f = ctx.from_numpy(np.random.default_rng(2).standard_normal((1, F)).astype(np.float16))
    y_c, y_f = ctx.tensor(wrk.F32, [C, 1]), ctx.tensor(wrk.F16, [F, 1])
    for layer in range(L):
        for name in ("att.w_k", "att.w_v", "att.w_r", "att.w_g", "att.w_o", "ffn.w_k", "ffn.w_v", "ffn.w_r"):
            h = ctypes.c_void_p()
            wrk.check(lib.wrk_model_matrix(model.handle, layer, name.encode(), ctypes.byref(h)))
            m = wrk.Matrix(ctx, None)
            m.handle = h
            xin, yout = (x_f, y_c) if name == "ffn.w_v" else (x_c, y_f) if name == "ffn.w_k" else (x_c, y_c)
            ops.append(m.matmul_op(xin, yout, turbo=False))
            m.handle = None  # borrowed from the model
    cmd = ctx.encode(wrk.op_list(ops), use_graph=True)
    for _ in range(3):
        cmd.submit()
    ctx.synchronize()
    ctx.timer_start()
    for _ in range(reps):
        cmd.submit()
    ms = ctx.timer_stop()
    _, gemv_bytes, launches = step_bytes(C, L, F, V)
    return ms * 1e-3 / (reps * launches), gemv_bytes / launches, launches


def cpu_decode(tensors, dims, sample_tokens, fast=True):
    """The oracle port decoding `sample_tokens` tokens after a 1-token prompt; returns tokens/s."""
    from oracle import model as omodel
    from oracle import oracle
    version, C, L, F, V = dims
    ref = omodel.OracleModel(tensors, {i: 1 for i in range(L)}, fast=fast)
    state = ref.init_state(1)
    out = ref.run(state, [[0]], [(1, 0)])[0]
    t0 = time.perf_counter()
    for _ in range(sample_tokens):
        tok = int(np.argmax(out[-1]))
        out = ref.run(state, [[tok]], [(1, 0)])[0]
    dt = time.perf_counter() - t0
    return sample_tokens / dt, oracle.num_threads(fast)


def workload_name(config, dims, decode):
    version, C, L, F, V = dims
    return (f"RWKV-v6-shaped {config} random-init (n_embd {C}, {L} layers, FFN {F}, vocab {V}), all layers "
            f"Int8, {PROMPT}-token seeded prompt then batch-1 decode, {decode} tokens per step")


def reference_arm(args, synth, dims, workload):
    """The reference's own implementation of the path is Rust + WGSL on wgpu and cannot be built or run here;
    its arithmetic restated in C++ (the oracle port) is timed on the host cores instead."""
    from oracle import model as omodel
    from oracle import oracle
    L = dims[2]
    tensors = synth.make_model(args.config, SEED_WEIGHTS, L)
    ref = omodel.OracleModel(tensors, {i: 1 for i in range(L)}, fast=True)
    state = ref.init_state(1)
    out = ref.run(state, [[0]], [(1, 0)])[0]
    sample = args.cpu_sample

    def one_step():
        nonlocal out
        for _ in range(sample):
            out = ref.run(state, [[int(np.argmax(out[-1]))]], [(1, 0)])[0]

    for _ in range(min(args.warmup, 1)):
        one_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one_step()
    dt = time.perf_counter() - t0
    value = args.steps * sample / dt
    cores = oracle.num_threads(True)
    print(json.dumps({
        "impl": "reference", "metric": "int8 batch-1 decode throughput", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "sample": f"{sample} decoded tokens per step"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{sample} decoded tokens per step, {args.steps} steps"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def device_decode(wrk, rt, ctx, bundle, embeds, decode, steps, warmup, sync):
    """Times `steps` x `decode` tokens of the T = 1 job with device-resident embedding rows; returns
    (milliseconds, kernels launched in the timed region, kernels per token)."""
    job = bundle.dispatch([(1, wrk.RNN_LAST)])

    def one_step():
        for t in range(decode):
            rt.job_load_embed(job, embeds, t)
            job.submit()

    for _ in range(warmup):
        one_step()
    sync()
    launches0 = ctx.launch_count()
    ctx.timer_start()
    for _ in range(steps):
        one_step()
    ms = ctx.timer_stop()
    sync()
    return ms, ctx.launch_count() - launches0, job.num_kernels()


TP_CONFIG, TP_BATCH = "v7-7b", 64


def c3_only(args):
    """BASELINE config 3 on one GPU: v6 3B-shaped (n_embd 2560, 32 layers, FFN 8960), all layers NF4, prefill of
    4 sequences x 2048 uniform-random tokens with token_chunk_size 256 through `wrk_runtime_infer` (host tokens in,
    last-token logits out per job).  `python bench.py --c3-only [--layers n]`."""
    host_threads()
    wrk = importlib.import_module("web-rwkv_b200")
    rt = importlib.import_module("web-rwkv_b200.runtime")
    synth = importlib.import_module("web-rwkv_b200.synth")
    ctx = wrk.Context(0)
    config, batch, length, chunk = "v6-3b", 4, 2048, 256
    version, C, L, F, V = synth.CONFIGS[config]
    L = args.layers or L
    t0 = time.perf_counter()
    builder = rt.ModelBuilder(ctx)
    for name, arr in synth.iter_tensors(config, SEED_WEIGHTS, L):
        builder.add_tensor(name, arr)
    builder.quant({i: wrk.QUANT_NF4 for i in range(L)})
    model = builder.build()
    del builder
    ctx.synchronize()
    build_s = time.perf_counter() - t0
    bundle = rt.Bundle(model, batch)
    rng = np.random.default_rng(SEED_TOKENS)
    logits = np.empty((batch, bundle.vocab), dtype=np.float32)

    def one_pass():
        seqs = [(rng.integers(0, V - 1, length).tolist(), wrk.RNN_LAST) for _ in range(batch)]
        inp = rt.RnnInput(seqs, chunk)
        jobs = 0
        while inp.num_token():
            bundle.infer(inp, logits)
            jobs += 1
        return jobs

    one_pass()  # builds the jobs' graphs
    ctx.synchronize()
    launches0 = ctx.launch_count()
    t0 = time.perf_counter()
    jobs = 0
    for _ in range(args.steps):
        jobs += one_pass()
    ctx.synchronize()
    seconds = time.perf_counter() - t0
    tokens = args.steps * batch * length
    flops_per_token = 2.0 * L * (5 * C * C + 2 * C * F)  # the seven large matrices of a layer
    print(json.dumps({"c3": {"workload": f"RWKV-v6-shaped {config} random-init (n_embd {C}, {L} layers, FFN {F}, vocab {V}), all layers NF4, "
                                         f"prefill of {batch} sequences x {length} tokens, token_chunk_size {chunk}, host tokens in",
                             "value": tokens / seconds, "unit": "tokens/s", "passes": args.steps, "jobs": jobs,
                             "kernels_per_job": (ctx.launch_count() - launches0) / max(1, jobs),
                             "tensor_tflops": tokens / seconds * flops_per_token / 1e12, "model_build_s": build_s}, "n_gpus": 1}))


def tp_only(args):
    """The split-model leg alone, for profiling: `python bench.py --tp-only [--tp-layers 2] --steps K` (one GPU) or under
    torch.distributed.run."""
    rank, local_rank, world = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1")))
    host_threads()
    wrk = importlib.import_module("web-rwkv_b200")
    rt = importlib.import_module("web-rwkv_b200.runtime")
    synth = importlib.import_module("web-rwkv_b200.synth")
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = wrk.Context(local_rank)
    out = tp_leg(wrk, rt, synth, ctx, rank, world, dist, args.steps, args.tp_layers or None)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps({"tp": out, "n_gpus": world}))


def tp_leg(wrk, rt, synth, ctx, rank, world, dist, steps, layers=None):
    """BASELINE config 4 (v7 7B-shaped, all layers Int8, 64 sequences decoding in step) as ONE model split over
    the ranks: time-mix heads and FFN columns sharded, one all-reduce after `output` and one after ffn `value`
    per layer, vocabulary slices gathered.  Strong scaling: the work is fixed, the ranks divide it.  At one
    GPU the same jobs run unsharded."""
    import ctypes
    version, C, L, F, V = synth.CONFIGS[TP_CONFIG]
    L = layers or L
    comm = None
    builder = rt.ModelBuilder(ctx)
    if world > 1:
        tp = importlib.import_module("web-rwkv_b200.tp")
        uid = [tp.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        comm = tp.Comm(ctx, uid[0], rank, world)
        builder.shard(rank, world, 64, 128)
    t0 = time.perf_counter()
    for name, arr in synth.iter_tensors(TP_CONFIG, SEED_WEIGHTS + 4, L):
        builder.add_tensor(name, arr)
    builder.quant({i: wrk.QUANT_INT8 for i in range(L)})
    model = builder.build()
    del builder
    ctx.synchronize()
    build_s = time.perf_counter() - t0
    bundle = rt.Bundle(model, TP_BATCH, comm)
    rng = np.random.default_rng(SEED_TOKENS + 4)  # the same tokens on every rank
    first = rng.integers(0, V - 1, TP_BATCH).tolist()
    inp = rt.RnnInput([([t], wrk.RNN_LAST) for t in first], TP_BATCH)
    logits = np.empty((TP_BATCH, bundle.vocab), dtype=np.float32)
    out = bundle.infer(inp, logits)
    checksum = float(np.abs(np.concatenate([o for o in out if o.size])).sum())
    job = bundle.dispatch([(1, wrk.RNN_LAST)] * TP_BATCH)
    tokens = rng.integers(0, V - 1, (16, TP_BATCH)).astype(np.uint32)

    def sync():
        ctx.synchronize()
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()

    def run(n):
        for i in range(n):
            job.load(tokens[i % 16])
            job.submit()

    run(3)
    sync()
    ctx.timer_start()
    run(steps)
    ms = ctx.timer_stop()
    sync()
    ms = max_over_ranks(ms, dist)
    result = {"workload": f"RWKV-v7-shaped {TP_CONFIG} random-init (n_embd {C}, {L} layers, FFN {F}, vocab {V}), all layers Int8, "
                          f"{TP_BATCH} sequences, one token each per step, host tokens in; one model split over the ranks",
              "value": steps * TP_BATCH / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms / steps, "steps": steps,
              "scaling": "strong", "parallelism": f"tp{world}" if world > 1 else "single GPU", "model_build_s": build_s,
              "kernels_per_step": job.num_kernels(), "logit_abs_sum_first_job": checksum}
    if comm is not None:
        # the collectives of one step alone, on the same communicator and sizes: 2 per layer of [C, 64] f32
        def time_ops(make):
            cmd = ctx.encode(wrk.op_list([make(i) for i in range(2 * L)]), use_graph=True)
            for _ in range(3):
                cmd.submit()
            sync()
            ctx.timer_start()
            for _ in range(steps):
                cmd.submit()
            t = max_over_ranks(ctx.timer_stop(), dist)
            sync()
            return t / steps

        part = ctx.tensor(wrk.F32, [C, TP_BATCH], zeros=True)
        nccl_ms = time_ops(lambda i: comm.all_reduce(part))
        result["all_reduce"] = {"count_per_step": 2 * L, "bytes_each": C * TP_BATCH * 4, "nccl_per_step_ms": nccl_ms,
                                "nccl": "NCCL all-reduce on the job's stream, NVLS off"}
        if bundle.peer_reduce():
            dst = ctx.tensor(wrk.F16, [C, TP_BATCH], zeros=True)
            peer_ms = time_ops(lambda i: comm.peer_all_reduce(i & 1, C * TP_BATCH, dst))
            # the same jobs with NCCL in place of the peer-memory reduce
            bundle.set_peer_reduce(0)
            job_nccl = bundle.dispatch([(1, wrk.RNN_LAST)] * TP_BATCH)
            for i in range(3):
                job_nccl.load(tokens[i % 16])
                job_nccl.submit()
            sync()
            ctx.timer_start()
            for i in range(steps):
                job_nccl.load(tokens[i % 16])
                job_nccl.submit()
            ms_nccl = max_over_ranks(ctx.timer_stop(), dist)
            sync()
            del job_nccl
            result["all_reduce"].update({"used": "one-shot reduce over peer memory (plain loads over NVLink, sums in rank order)",
                                         "per_step_ms": peer_ms, "share_of_step": peer_ms * steps / ms,
                                         "value_with_nccl": steps * TP_BATCH / (ms_nccl * 1e-3)})
        else:
            result["all_reduce"].update({"used": "NCCL", "per_step_ms": nccl_ms, "share_of_step": nccl_ms * steps / ms})
    del job, bundle, model
    if comm is not None:
        import gc
        gc.collect()
        del comm
        gc.collect()
    return result


def check_fused_against_strict(wrk, rt, model, prompt, vocab, mode):
    """One decoded token after the prompt through the fused job and through the op-by-op job."""
    outs = []
    for fused in (mode, 0):
        bundle = rt.Bundle(model, 1)
        bundle.set_fused(fused)
        inp = rt.RnnInput([(prompt, wrk.RNN_LAST)], PROMPT)
        logits = np.empty((PROMPT, vocab), dtype=np.float32)
        first = bundle.infer(inp, logits)[0].copy()
        inp.append(0, [int(np.argmax(first[-1]))])
        outs.append(bundle.infer(inp, logits)[0][-1].copy())
        del bundle
    return float(np.max(np.abs(outs[0] - outs[1]))), float(np.max(np.abs(outs[1])))


# ---- op-level sweep (BASELINE config 5) ---------------------------------------------------------------
BYTES_PER_WEIGHT = {"int8": 1.0 + 4.0 / 128.0, "nf4": 0.5 + 2.0 / 64.0, "fp16": 2.0}


def sweep_matmul(wrk, ctx, rng, kind, K, M, N, reps, matrices, single, group=0):
    """CUDA-event time per launch of a graph holding `matrices` different weight matrices of the shape (so that
    consecutive launches do not re-read one matrix from L2); `single` submits one op per launch without a graph
    (the form used under a profiler); `group` = g > 0 times `matrices` grouped ops of g matrices each (each matrix with
    its own activations and output), per group."""
    if group:
        sets = []
        for _ in range(matrices):
            ws = [ctx.from_numpy((rng.standard_normal((M, K), dtype=np.float32) * 0.02).astype(np.float16)) for _ in range(group)]
            sets.append([wrk.Matrix.quant_u8(w) if kind == "int8" else wrk.Matrix.quant_nf4(w) if kind == "nf4" else wrk.Matrix.fp16(w)
                         for w in ws])
        xs = [ctx.from_numpy(rng.standard_normal((N, K), dtype=np.float32).astype(np.float16)) for _ in range(group)]
        ys = [ctx.tensor(wrk.F16, [M, N]) for _ in range(group)]
        cmd = ctx.encode(wrk.op_list([wrk.matmul_group_op(ms, xs, ys, turbo=(N % 32 == 0)) for ms in sets]), use_graph=True)
        for _ in range(3):
            cmd.submit()
        ctx.synchronize()
        ctx.timer_start()
        for _ in range(reps):
            cmd.submit()
        us = ctx.timer_stop() * 1e3 / (reps * matrices)
        print(f"{kind} K={K} M={M} N={N} group of {group}: {us:8.1f} us  {2.0 * K * M * N * group / us / 1e6:8.1f} TFLOP/s", flush=True)
        return
    def make():
        w = ctx.from_numpy((rng.standard_normal((M, K), dtype=np.float32) * 0.02).astype(np.float16))
        return wrk.Matrix.quant_u8(w) if kind == "int8" else wrk.Matrix.quant_nf4(w) if kind == "nf4" else wrk.Matrix.fp16(w)

    mats = [make() for _ in range(1 if single else matrices)]
    x = ctx.from_numpy(rng.standard_normal((N, K), dtype=np.float32).astype(np.float16))
    y = ctx.tensor(wrk.F16, [M, N])
    ops = [m.matmul_op(x, y, turbo=(N % 32 == 0)) for m in mats]
    if single:
        for _ in range(reps):
            ctx.run(ops[0])
        ctx.synchronize()
        print(f"{kind} K={K} M={M} N={N}: {reps} single launches", flush=True)
        return
    cmd = ctx.encode(wrk.op_list(ops), use_graph=True)
    for _ in range(3):
        cmd.submit()
    ctx.synchronize()
    ctx.timer_start()
    for _ in range(reps):
        cmd.submit()
    us = ctx.timer_stop() * 1e3 / (reps * len(mats))
    nbytes = K * M * BYTES_PER_WEIGHT[kind] + 2.0 * N * (K + M)
    print(f"{kind} K={K} M={M} N={N}: {us:8.1f} us  {nbytes / us / 1e3:8.1f} GB/s  {2.0 * K * M * N / us / 1e6:8.1f} TFLOP/s",
          flush=True)


def sweep_wkv(wrk, ctx, rng, version, H, T, reps, blocks=False):
    """`time_mix_v7` (fp16 r, w, n, x) or `time_mix_v6` (f32 k, v, r, x; `blocks`: in blocks of 16 tokens) on one
    sequence of T tokens: H heads of 64 x 64 f32 state.  The state grows stale over the repetitions, which does not
    change the work."""
    S = 64
    C = S * H
    cursors = ctx.from_numpy(np.array([[0, 0, T]] * T, dtype=np.uint32))  # wide cursors: (batch, token, len) per token
    state = ctx.from_numpy((rng.standard_normal((1, S + 2, C)) * 0.1).astype(np.float32))
    if version == 7:
        f = np.float16
        r = ctx.from_numpy(rng.standard_normal((T, H, S)).astype(f))
        w = ctx.from_numpy(rng.standard_normal((T, H, S)).astype(f))
        kk = rng.standard_normal((T, H, S)).astype(np.float32)
        kk /= np.linalg.norm(kk, axis=-1, keepdims=True)  # the model L2-normalises kk per head
        n = np.stack([rng.standard_normal((T, H, S)), rng.standard_normal((T, H, S)), rng.uniform(0, 1, (T, H, S)), kk])
        x = ctx.from_numpy(rng.standard_normal((T, H, S)).astype(f))
        op = wrk.time_mix_v7(cursors, state.view(y=(0, S + 1)), r, w, ctx.from_numpy(n.astype(f)), x)
        nbytes = 2.0 * C * S * 4 + T * C * 2.0 * 8
    else:
        f = np.float32
        k, v, r, x = (ctx.from_numpy(rng.standard_normal((T, H, S)).astype(f) * 0.5) for _ in range(4))
        decay = ctx.from_numpy(np.exp(-np.exp(rng.uniform(-6, 1, (T, H, S)))).astype(f))
        first = ctx.from_numpy(rng.uniform(-1, 1, (H, S)).astype(f))
        if blocks:
            op = wrk.time_mix_blocks(True, cursors, decay, first, state.view(y=(0, S + 1)), k, v, r, x)
        else:
            op = wrk.time_mix_v6(cursors, decay, first, state.view(y=(0, S + 1)), k, v, r, x)
        nbytes = 2.0 * C * S * 4 + T * C * 4.0 * 6
    cmd = ctx.encode(wrk.op_list([op]), use_graph=True)
    for _ in range(3):
        cmd.submit()
    ctx.synchronize()
    ctx.timer_start()
    for _ in range(reps):
        cmd.submit()
    us = ctx.timer_stop() * 1e3 / reps
    flops = (10.0 if version == 7 else 7.0) * C * S * T
    print(f"time_mix_{'blocks' if blocks else 'v%d' % version} H={H} T={T}: {us:8.1f} us  {us / T:6.2f} us/token  {nbytes / us / 1e3:8.1f} GB/s  "
          f"{flops / us / 1e6:6.2f} TFLOP/s", flush=True)


def sweep(args):
    wrk = importlib.import_module("web-rwkv_b200")
    ctx = wrk.Context(0)
    rng = np.random.default_rng(4000)
    if args.sweep == "wkv":
        for version in (7, 6):
            for T in (1, 2, 8, 32, 64, 128, 256, 512):
                sweep_wkv(wrk, ctx, rng, version, 64, T, args.reps)
        for T in (16, 32, 64, 128, 256, 512, 2048):
            sweep_wkv(wrk, ctx, rng, 6, 64, T, args.reps, blocks=True)
        return
    shapes = [tuple(int(v) for v in s.split(",")) for s in (args.shape or ["2048,2048", "2560,8960", "4096,4096"])]
    for kind in args.kind.split(","):
        for K, M in shapes:
            for N in (int(v) for v in args.tokens.split(",")):
                sweep_matmul(wrk, ctx, rng, kind, K, M, N, args.reps, args.matrices, args.single, args.group)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=CONFIG)
    ap.add_argument("--layers", type=int, default=None, help="debug: truncate the model")
    ap.add_argument("--decode", type=int, default=DECODE)
    ap.add_argument("--cpu-sample", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-secondary", action="store_true")
    ap.add_argument("--strict", action="store_true", help="one launch per reference op (no fused kernels)")
    ap.add_argument("--fused", type=int, default=2, choices=[1, 2, 3],
                    help="decode job: 2 = one launch per fused phase (default), 1 = one persistent kernel, 3 = persistent, mma.sync only")
    ap.add_argument("--tp-only", action="store_true", help="only the split-model leg (for profiles); --tp-layers cuts the model")
    ap.add_argument("--tp-layers", type=int, default=0)
    ap.add_argument("--c3-only", action="store_true", help="only BASELINE config 3: NF4 3B-shaped prefill, 4 x 2048 tokens, chunk 256")
    ap.add_argument("--no-tp", action="store_true", help="skip the split-model leg (v7 7B-shaped, 64 sequences)")
    ap.add_argument("--no-serialize", action="store_true", help="skip the save / load timing of the quantized model")
    ap.add_argument("--sweep", choices=["matmul", "wkv"], help="op-level sweep instead of the model benchmark")
    ap.add_argument("--kind", default="int8,nf4,fp16")
    ap.add_argument("--shape", action="append", help="sweep: K,M (repeatable)")
    ap.add_argument("--tokens", default="1,4,16,64,256,1024")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--matrices", type=int, default=8)
    ap.add_argument("--single", action="store_true")
    ap.add_argument("--group", type=int, default=0, help="sweep matmul: time grouped ops of this many matrices (1-4)")
    args = ap.parse_args()

    if args.sweep:
        return sweep(args)
    if args.tp_only:
        return tp_only(args)
    if args.c3_only:
        return c3_only(args)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    synth = importlib.import_module("web-rwkv_b200.synth")
    version, C, L, F, V = synth.CONFIGS[args.config]
    L = args.layers or L
    dims = (version, C, L, F, V)
    workload = workload_name(args.config, dims, args.decode)

    if args.impl == "reference":
        if rank == 0:
            reference_arm(args, synth, dims, workload)
        return

    wrk = importlib.import_module("web-rwkv_b200")
    rt = importlib.import_module("web-rwkv_b200.runtime")
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    ctx = wrk.Context(local_rank)
    keep = rank == 0 and world == 1 and not args.no_cpu_baseline  # the CPU baseline is an N = 1 figure
    t_build = time.perf_counter()
    model, tensors, _ = build_model(wrk, rt, synth, ctx, args.config, L, keep=keep)
    ctx.synchronize()
    t_build = time.perf_counter() - t_build
    serialized = serialize_round_trip(rt, ctx, model) if rank == 0 and world == 1 and not args.no_serialize else None
    rng = np.random.default_rng(SEED_TOKENS + rank)
    prompt = rng.integers(0, V - 1, PROMPT).tolist()
    tokens = rng.integers(0, V - 1, args.decode).astype(np.uint32)

    # ---- parity of what is timed: the fused job against the op-by-op job, one decoded token ----
    checked = None
    if not args.strict:
        diff, scale = check_fused_against_strict(wrk, rt, model, prompt, (V + 7) // 8 * 8, args.fused)
        checked = {"checked": bool(diff <= 2e-2 * max(1.0, scale)), "max_abs": diff, "logit_scale": scale,
                   "against": "one-launch-per-reference-op job, same model, prompt and token"}

    bundle = rt.Bundle(model, 1)
    bundle.set_fused(0 if args.strict else args.fused)

    # prompt (GEMM path), untimed
    inp = rt.RnnInput([(prompt, wrk.RNN_LAST)], PROMPT)
    logits = np.empty((PROMPT, bundle.vocab), dtype=np.float32)
    out = bundle.infer(inp, logits)[0]
    next_token = int(np.argmax(out[-1]))

    def barrier():
        ctx.synchronize()
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()
        ctx.synchronize()

    # ---- device-resident decode: embedding rows of the step's tokens live in HBM ----
    emb = synth.make_globals(version, C, V, SEED_WEIGHTS)["emb.weight"]
    embeds = ctx.from_numpy(emb[tokens])  # [C, decode] fp16, reused by every step
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms, gpu_launches, kernels_per_token = device_decode(wrk, rt, ctx, bundle, embeds, args.decode, args.steps,
                                                        args.warmup, barrier)
    clocks = sampler.stop()
    ms = max_over_ranks(ms, dist)
    value = whole_job_rate(world, args.steps, args.decode, ms)

    # ---- end to end through the reference-facing call: host tokens in, host logits out ----
    host_logits = np.empty((1, bundle.vocab), dtype=np.float32)
    inp = rt.RnnInput([([next_token], wrk.RNN_LAST)], 32)

    def e2e_step(n):
        tok = None
        for _ in range(n):
            out = bundle.infer(inp, host_logits)[0]
            tok = int(np.argmax(out[0]))
            inp.append(0, [tok])
        return tok

    e2e_step(min(64, args.decode))
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step(args.decode)
    ctx.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_s = max_over_ranks(e2e_s, dist)
    e2e_value = whole_job_rate(world, args.steps, args.decode, e2e_s * 1e3)

    # ---- secondary: prefill of one 256-token chunk of the same model (tensor-memory GEMM path), rank 0 only ----
    prefill = None
    if rank == 0 and not args.no_prefill:
        chunk = 256
        p_tokens = rng.integers(0, V - 1, chunk).tolist()
        p_logits = np.empty((1, bundle.vocab), dtype=np.float32)

        def prefill_once():
            p_inp = rt.RnnInput([(p_tokens, wrk.RNN_LAST)], chunk)
            bundle.infer(p_inp, p_logits)

        for _ in range(2):
            prefill_once()
        ctx.synchronize()
        t0 = time.perf_counter()
        reps = 5
        for _ in range(reps):
            prefill_once()
        ctx.synchronize()
        prefill = {"value": reps * chunk / (time.perf_counter() - t0), "unit": "tokens/s",
                   "workload": f"{chunk}-token chunk of the same model, host tokens in, last-token logits out"}

    # ---- one model split over the ranks (BASELINE config 4), at every N ----
    tp = None
    if not args.no_tp:
        try:
            tp = tp_leg(wrk, rt, synth, ctx, rank, world, dist, max(args.steps, 3) * 8)
        except Exception as e:  # the headline stands on its own
            tp = {"failed": str(e)[:300]}

    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return

    # ---- roofline of the dominant kernel ----
    peak, peak_kind = _peaks()
    sec_per_launch, bytes_per_launch, launches = gemv_roofline(wrk, rt, ctx, model, dims, reps=10)
    achieved = bytes_per_launch / sec_per_launch / 1e9
    total_bytes, gemv_bytes, _ = step_bytes(C, L, F, V)
    traffic = NCU_TRAFFIC_RATIO * bytes_per_launch
    del bundle, embeds

    # ---- secondary: the 1.6B-shaped model (BASELINE config 2), device-resident decode only ----
    secondary = None
    if not args.no_secondary and args.config != SECONDARY and not args.layers:
        model2, _, dims2 = build_model(wrk, rt, synth, ctx, SECONDARY)
        _, C2, L2, F2, V2 = dims2
        bundle2 = rt.Bundle(model2, 1)
        bundle2.set_fused(0 if args.strict else args.fused)
        bundle2.infer(rt.RnnInput([(prompt, wrk.RNN_LAST)], PROMPT), logits)
        emb2 = synth.make_globals(6, C2, V2, SEED_WEIGHTS)["emb.weight"]
        embeds2 = ctx.from_numpy(emb2[tokens])
        ms2, _, k2 = device_decode(wrk, rt, ctx, bundle2, embeds2, args.decode, 3, 3, ctx.synchronize)
        bytes2, _, _ = step_bytes(C2, L2, F2, V2)
        rate2 = 3 * args.decode / (ms2 * 1e-3)
        secondary = {"value": rate2, "unit": "tokens/s", "workload": workload_name(SECONDARY, dims2, args.decode),
                     "kernels_per_token": int(k2), "algorithmic_bytes_per_token": bytes2,
                     "frac_of_roofline": rate2 / (peak * 1e9 / bytes2)}
        del bundle2, embeds2, model2

    cpu = None
    if not args.no_cpu_baseline and world == 1:
        cpu_tps, cores = cpu_decode(tensors, dims, args.cpu_sample)
        cpu = {"value": cpu_tps, "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": f"{args.cpu_sample} greedy decode tokens of the same model after a 1-token prompt"}

    print(json.dumps({
        "metric": "int8 batch-1 decode throughput", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 activations, f32 accumulate, u8 weights",
        "data": "synthetic",
        "config": {"workload": workload, "parallelism": f"replicas x{world}" if world > 1 else "single GPU",
                   "l2": f"weights of one token ({total_bytes / 1e9:.1f} GB) exceed L2 (126 MB); no flush needed",
                   "mode": "strict" if args.strict else {1: "fused, one persistent kernel", 2: "fused, launch per phase", 3: "fused, persistent mma.sync kernel"}[args.fused], "model_build_s": t_build, "model_file": serialized},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s",
                "h2d_bytes_per_step": args.decode * (C * 2 + 12), "d2h_bytes_per_step": args.decode * ((V + 7) // 8 * 8) * 4},
        "parity": checked,
        "prefill": prefill,
        "tp": tp,
        "decode_1p6b": secondary,
        "gpu_launches": int(gpu_launches),
        "kernels_per_token": int(kernels_per_token),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "traffic": traffic,
                     "kernel": "Int8 weight-streaming GEMV (T = 1, standalone launches over the model's matrices)",
                     "algorithmic_bytes_per_launch": bytes_per_launch, "us_per_launch": sec_per_launch * 1e6,
                     "launches_timed": launches * 10},
        "decode_step": {"algorithmic_bytes_per_token": total_bytes, "gemv_share": gemv_bytes / total_bytes,
                        "hbm_roofline_tokens_per_s": peak * 1e9 / total_bytes,
                        "frac_of_roofline": value / world / (peak * 1e9 / total_bytes)},
        "cpu_baseline": cpu,
    }))


if __name__ == "__main__":
    main()
