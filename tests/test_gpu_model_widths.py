"""run() jobs at the widths the benchmark times, on two-layer cuts of the BASELINE configurations.

The fused decode job owns one row range per CTA and streams through multi-cell rings only at real
model widths (n_embd 2048 / 4096, FFN 7168 / 14336, vocab 65536); the tiny models of
test_gpu_model.py leave most CTAs with a handful of rows.  Every case here compares the CUDA runtime
with the full-model CPU oracle (max-abs 2e-2 / cosine >= 0.9995 on logits and recurrent state) and, for
the decode cases, the fused job with the one-launch-per-reference-op job on the same tokens.
Cuts keep the width, head count, FFN width and quantization of the configuration and drop layers only
(the oracle then finishes in seconds); v7 keeps two layers because its loader reads blocks.1.
"""
import importlib

import numpy as np
import pytest

from oracle import model as omodel
from tests.util import assert_close, assert_state_close

pytestmark = pytest.mark.gpu

rt = importlib.import_module("web-rwkv_b200.runtime")
synth = importlib.import_module("web-rwkv_b200.synth")
LAST, FULL = 0, 1
INT8, NF4 = 1, 2


def _cut(config, vocab=None, layers=2):
    version, C, L, F, V = synth.CONFIGS[config]
    return (version, C, layers, F, vocab or V)


def _models(ctx, cfg, quant, seed):
    tensors = synth.make_model(cfg, seed=seed, num_layer=cfg[2])
    q = {i: quant for i in range(cfg[2])}
    model = rt.ModelBuilder(ctx).add_tensors(tensors).quant(q).build()
    return model, omodel.OracleModel(tensors, q)


def _state(bundle, ref_state, batch=0):
    return bundle.state_back(batch), np.stack([s[batch] for s in ref_state])


@pytest.mark.parametrize("config,seed", [("v6-1.6b", 1002), ("v6-7b", 1006)])
def test_fused_decode_matches_oracle_and_strict_job(ctx, config, seed):
    # BASELINE configs 2 and 2b: 64-token prompt, then batch-1 decode; jobs of 1, 2 and 8 tokens take the
    # fused path, the prompt takes the token-batched GEMM path
    cfg = _cut(config)
    V = cfg[4]
    model, ref = _models(ctx, cfg, INT8, seed)
    rng = np.random.default_rng(seed + 1000)
    prompt = rng.integers(0, V - 1, 64).tolist()
    fused, phased, strict = rt.Bundle(model, 1), rt.Bundle(model, 1), rt.Bundle(model, 1)
    fused.set_fused(1)   # one persistent kernel per job of at most 8 tokens
    phased.set_fused(2)  # the same fused kernels, one launch per phase (the default)
    strict.set_fused(0)
    bundles = (fused, phased, strict)
    state = ref.init_state(1)

    def job(tokens, option, what):
        rows = len(tokens) if option == FULL else 1
        want = ref.run(state, [tokens], [(len(tokens), option)])[0]
        got = []
        for bundle in bundles:
            inp = bundle.pending
            inp.append(0, tokens)
            got.append(bundle.infer(inp)[0].copy())
            assert inp.num_token() == 0
        assert got[0].shape == want.shape == (rows, V)
        assert_close(got[0], want, f"{config} fused {what}")
        assert_close(got[1], want, f"{config} fused, launch per phase, {what}")
        assert_close(got[2], want, f"{config} strict {what}")
        assert_close(got[0], got[2], f"{config} fused vs strict {what}")
        assert_close(got[0], got[1], f"{config} one kernel vs launch per phase {what}")
        return want

    for bundle in bundles:
        bundle.pending = rt.RnnInput([([], LAST)], 64)
    want = job(prompt, LAST, "prompt")
    for step in range(8):
        want = job([int(np.argmax(want[-1]))], LAST, f"decode {step}")
    for bundle in bundles:  # Full: one head row per token of the job
        bundle.pending = rt.RnnInput([([], FULL)], 32)
    want = job(rng.integers(0, V - 1, 2).tolist(), FULL, "job of 2 tokens")
    want = job(rng.integers(0, V - 1, 8).tolist(), FULL, "job of 8 tokens")
    got_f, want_s = _state(fused, state)
    assert_state_close(got_f, want_s, f"{config} fused state")
    assert_state_close(_state(strict, state)[0], want_s, f"{config} strict state")
    assert_state_close(got_f, _state(strict, state)[0], f"{config} fused vs strict state")
    assert_state_close(_state(phased, state)[0], want_s, f"{config} fused, launch per phase, state")
    assert ctx.device_status() == 0


@pytest.mark.parametrize("packed", [False, True])
def test_nf4_prefill_chunk_of_256(ctx, packed):
    # BASELINE config 3: n_embd 2560, FFN 8960, all layers NF4, token_chunk_size 256: one sequence gets the
    # whole chunk.  Wide cursors carry the shift rows; packed cursors reproduce the reference's 8-bit wrap.
    cfg = _cut("v6-3b", vocab=8192)
    model, ref = _models(ctx, cfg, NF4, 1003)
    rng = np.random.default_rng(2003)
    tokens = rng.integers(0, cfg[4] - 1, 256 + 40).tolist()
    bundle = rt.Bundle(model, 1)
    bundle.set_packed_cursors(packed)
    state = ref.init_state(1)
    inp = rt.RnnInput([(tokens, LAST)], 256)
    remaining = tokens
    jobs = 0
    while inp.num_token():
        info = inp.iter().next()
        got = bundle.infer(inp)[0].copy()
        want = ref.run(state, [remaining], info, wide=not packed)[0]
        remaining = remaining[info[0][0]:]
        assert got.shape == want.shape
        if got.size:
            assert_close(got, want, f"v6-3b NF4 job {jobs} packed={packed}")
        jobs += 1
    assert jobs >= 2  # the iterator's own chunking decides (tests/test_rnn_schedule.py holds its known answers)
    got_s, want_s = _state(bundle, state)
    assert_state_close(got_s, want_s, f"v6-3b NF4 state packed={packed}")
    assert ctx.device_status() == 0


def test_v7_batched_decode_of_64_sequences(ctx):
    # BASELINE config 4: v7, n_embd 4096, FFN 16384, Int8, num_batch 64, mixed prompt lengths from a seed
    # (short ones, so that the oracle finishes in seconds), then two decode steps of 64 tokens
    cfg = _cut("v7-7b", vocab=8192)
    B, V = 64, cfg[4]
    model, ref = _models(ctx, cfg, INT8, 1004)
    rng = np.random.default_rng(3004)
    lens = rng.integers(1, 12, B)
    prompts = [rng.integers(0, V - 1, int(n)).tolist() for n in lens]
    bundle = rt.Bundle(model, B)
    state = ref.init_state(B)
    inp = rt.RnnInput([(p, LAST) for p in prompts], 128)
    remaining = [list(p) for p in prompts]
    last = [None] * B

    def drain(what):
        nonlocal remaining
        jobs = 0
        while inp.num_token():
            info = inp.iter().next()
            got = [g.copy() for g in bundle.infer(inp)]
            want = ref.run(state, remaining, info)
            remaining = [r[l:] for r, (l, _) in zip(remaining, info)]
            for b in range(B):
                assert got[b].shape == want[b].shape
                if got[b].size:
                    assert_close(got[b], want[b], f"v7 {what} job {jobs} batch {b}")
                    last[b] = want[b][-1]
            jobs += 1
        return jobs

    assert drain("prefill") >= 2
    for step in range(2):
        for b in range(B):
            tok = int(np.argmax(last[b]))
            inp.append(b, [tok])
            remaining[b] = [tok]
        assert drain(f"decode {step}") == 1
    for b in (0, 17, 63):
        got_s, want_s = _state(bundle, state, b)
        assert_state_close(got_s, want_s, f"v7 state batch {b}")
    assert ctx.device_status() == 0
