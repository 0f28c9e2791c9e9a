#!/usr/bin/env python
"""Benchmark of the B200-native web-rwkv hot path: Int8 batch-1 decode of an RWKV-v6-shaped model.

Workload (the configuration the headline metric is quoted on): RWKV-v6 1.6B-shaped random-init
model (n_embd 2048, 24 layers, FFN 7168, vocab 65536), every layer Int8 through the quantizer,
a 64-token seeded prompt, then batch-1 decode.  One *step* = 512 decoded tokens.

  value  tokens/s with the step's inputs (embedding rows) already resident in HBM and the logits left
         on the device: one stream-ordered device copy + one CUDA-graph launch per token.
  e2e    tokens/s through the reference-facing call (`SimpleRuntime::infer` = wrk_runtime_infer) with
         host token ids in and host logits out every token (pinned H2D of the embedding row and
         cursors, D2H of the [vocab] fp32 logits, greedy arg-max on the host feeding the next token).
  roofline      the Int8 GEMV kernel (dominant: it streams ~84 % of a decode step's bytes), timed with
                CUDA events over a loop that runs every quantized matmul of every layer at T = 1 in
                model order (weights of all layers = 1.3 GB, larger than L2).
  cpu_baseline  the CPU oracle (a port of the reference's shader arithmetic; the reference itself is
                Rust + WGSL and cannot be built here) decoding a bounded sample on the host cores.

`--impl reference` times that CPU port on the same workload (bounded sample per step).
With N > 1 GPUs every rank decodes its own replica of the same model (the model is tiny compared with
180 GB; data-parallel replicas, weak scaling, no data-path collective).
"""
import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIG = "v6-1.6b"
PROMPT = 64
DECODE = 512
SEED_WEIGHTS, SEED_TOKENS = 1002, 2002


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
    ops, keep = [], []
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


def cpu_decode(config, tensors, dims, sample_tokens, fast=True):
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=CONFIG)
    ap.add_argument("--layers", type=int, default=None, help="debug: truncate the model")
    ap.add_argument("--decode", type=int, default=DECODE)
    ap.add_argument("--cpu-sample", type=int, default=8)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--strict", action="store_true", help="one launch per reference op (no fused kernels)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    synth = importlib.import_module("web-rwkv_b200.synth")
    version, C, L, F, V = synth.CONFIGS[args.config]
    L = args.layers or L
    dims = (version, C, L, F, V)
    workload = (f"RWKV-v6-shaped {args.config} random-init (n_embd {C}, {L} layers, FFN {F}, vocab {V}), all layers "
                f"Int8, {PROMPT}-token seeded prompt then batch-1 decode, {args.decode} tokens per step")

    if args.impl == "reference":
        # The reference's own CPU implementation of the path does not exist (it is Rust + WGSL on wgpu and
        # cannot be built or run here); its arithmetic restated in C++ (the oracle port) is timed instead.
        if rank != 0:
            return
        tensors = synth.make_model(args.config, SEED_WEIGHTS, L)
        from oracle import model as omodel
        from oracle import oracle
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
    keep = rank == 0 and not args.no_cpu_baseline
    model, tensors, _ = build_model(wrk, rt, synth, ctx, args.config, L, keep=keep)
    bundle = rt.Bundle(model, 1)
    bundle.set_fused(not args.strict)
    rng = np.random.default_rng(SEED_TOKENS + rank)
    prompt = rng.integers(0, V - 1, PROMPT).tolist()
    total_tokens = args.decode * (args.steps + args.warmup)
    tokens = rng.integers(0, V - 1, total_tokens).astype(np.uint32)

    # prompt (GEMM path), untimed
    inp = rt.RnnInput([(prompt, wrk.RNN_LAST)], PROMPT)
    logits = np.empty((PROMPT, bundle.vocab), dtype=np.float32)
    out = bundle.infer(inp, logits)[0]
    next_token = int(np.argmax(out[-1]))

    # ---- device-resident decode: embedding rows of the step's tokens live in HBM ----
    emb = synth.make_globals(version, C, V, SEED_WEIGHTS)["emb.weight"]
    embeds = ctx.from_numpy(emb[tokens[: args.decode]])  # [C, decode] fp16, reused by every step
    del emb
    job = bundle.dispatch([(1, wrk.RNN_LAST)])
    kernels_per_token = job.num_kernels()

    def device_step():
        for t in range(args.decode):
            rt.job_load_embed(job, embeds, t)
            job.submit()

    def barrier():
        ctx.synchronize()
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()
        ctx.synchronize()

    for _ in range(args.warmup):
        device_step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = ctx.launch_count()
    ctx.timer_start()
    for _ in range(args.steps):
        device_step()
    ms = ctx.timer_stop()
    barrier()
    gpu_launches = ctx.launch_count() - launches0
    clocks = sampler.stop()
    ms = max_over_ranks(ms, dist)
    value = whole_job_rate(world, args.steps, args.decode, ms)

    # ---- end to end through the reference-facing call: host tokens in, host logits out ----
    import ctypes
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

    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return

    # ---- roofline of the dominant kernel ----
    peak, peak_kind = _peaks()
    sec_per_launch, bytes_per_launch, launches = gemv_roofline(wrk, rt, ctx, model, dims, reps=20)
    achieved = bytes_per_launch / sec_per_launch / 1e9
    total_bytes, gemv_bytes, _ = step_bytes(C, L, F, V)
    # dram read + write per launch: the ncu capture of the same kernel on this model's matrices (summary under
    # profiles/, fused_gemv_kernel) measured 1.01 x the algorithmic bytes for every Int8 launch
    traffic = NCU_TRAFFIC_RATIO * bytes_per_launch

    cpu = None
    if not args.no_cpu_baseline:
        cpu_tps, cores = cpu_decode(args.config, tensors, dims, args.cpu_sample)
        cpu = {"value": cpu_tps, "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": f"{args.cpu_sample} greedy decode tokens of the same model after a 1-token prompt"}

    print(json.dumps({
        "metric": "int8 batch-1 decode throughput", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 activations, f32 accumulate, u8 weights",
        "data": "synthetic",
        "config": {"workload": workload, "parallelism": f"replicas x{world}" if world > 1 else "single GPU",
                   "l2": "weights of one token (1.4 GB) exceed L2 (126 MB); no flush needed",
                   "mode": "strict" if args.strict else "fused"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s",
                "h2d_bytes_per_step": args.decode * (C * 2 + 12), "d2h_bytes_per_step": args.decode * bundle.vocab * 4},
        "prefill": prefill,
        "gpu_launches": int(gpu_launches),
        "kernels_per_token": int(kernels_per_token),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "traffic": traffic, "kernel": "fused_gemv_kernel (Int8 weights, T = 1, standalone launches)",
                     "algorithmic_bytes_per_launch": bytes_per_launch, "us_per_launch": sec_per_launch * 1e6,
                     "launches_timed": launches * 20},
        "decode_step": {"algorithmic_bytes_per_token": total_bytes, "gemv_share": gemv_bytes / total_bytes,
                        "hbm_roofline_tokens_per_s": peak * 1e9 / total_bytes,
                        "frac_of_roofline": value / world / (peak * 1e9 / total_bytes)},
        "cpu_baseline": cpu,
    }))


if __name__ == "__main__":
    main()
