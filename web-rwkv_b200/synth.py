"""Seeded synthetic RWKV v5 / v6 / v7 checkpoints in the reference's safetensors naming.

No real weights or datasets are available offline, and the reference's own benchmark feeds
uniform-random token ids (examples/bench.rs:184-186), so the tests and the benchmark use
random-init models of the shapes BASELINE.json names.  Everything is fp16 as in a converted
checkpoint; shapes are outermost-first ({rows, columns}) as stored in a .st file.

Value ranges: matrices, embeddings and head N(0, 0.02^2); LayerNorm / GroupNorm weight
1 + N(0, 0.02^2), bias N(0, 0.02^2); token-shift mixes U(0, 1); v5/v6 time_decay U(-6, 1)
(before exp(-exp(.))), time_first U(-1, 1); v7 w0 U(-6, 1), a0 / v0 N(0, 1), r_k / k_k / k_a
U(0, 1).  The reference has no initialiser of its own (it only loads files), so these ranges
are this project's choice.
"""
import numpy as np

CONFIGS = {
    # name: (version, n_embd, n_layer, ffn, vocab)
    "v6-0.1b": (6, 768, 12, 2688, 65536),
    "v6-1.6b": (6, 2048, 24, 7168, 65536),
    "v6-3b": (6, 2560, 32, 8960, 65536),
    "v6-7b": (6, 4096, 32, 14336, 65536),
    "v7-7b": (7, 4096, 32, 16384, 65536),
    "v6-tiny": (6, 256, 3, 896, 512),
    "v5-tiny": (5, 256, 3, 896, 512),
    "v7-tiny": (7, 256, 3, 1024, 512),
    "v4-tiny": (4, 256, 3, 1024, 512),
}
HEAD_SIZE = 64
V6_TIME_MIX, V6_TIME_DECAY = 32, 64
V7_W, V7_A, V7_G, V7_V = 64, 64, 128, 32


def _normal(rng, shape, std=0.02, mean=0.0):
    out = rng.standard_normal(shape, dtype=np.float32)
    out *= std
    if mean:
        out += mean
    return out.astype(np.float16)


def _uniform(rng, shape, lo, hi):
    return rng.uniform(lo, hi, shape).astype(np.float16)


def make_layer(version, layer, C, F, seed):
    """One block's tensors as {name: fp16 array}."""
    rng = np.random.default_rng([seed, layer])
    H = C // HEAD_SIZE
    blk, att, ffn = f"blocks.{layer}", f"blocks.{layer}.att", f"blocks.{layer}.ffn"
    t = {}
    for ln in ("ln1", "ln2"):
        t[f"{blk}.{ln}.weight"] = _normal(rng, (C,), mean=1.0)
        t[f"{blk}.{ln}.bias"] = _normal(rng, (C,))
    if layer == 0:
        t[f"{blk}.ln0.weight"] = _normal(rng, (C,), mean=1.0)
        t[f"{blk}.ln0.bias"] = _normal(rng, (C,))
    if version != 4:
        t[f"{att}.ln_x.weight"] = _normal(rng, (C,), mean=1.0)
        t[f"{att}.ln_x.bias"] = _normal(rng, (C,))
    t[f"{att}.key.weight"] = _normal(rng, (C, C))
    t[f"{att}.value.weight"] = _normal(rng, (C, C))
    t[f"{att}.receptance.weight"] = _normal(rng, (C, C))
    t[f"{att}.output.weight"] = _normal(rng, (C, C))
    t[f"{ffn}.key.weight"] = _normal(rng, (F, C))
    t[f"{ffn}.value.weight"] = _normal(rng, (C, F))
    if version == 4:
        # per-channel decay (before -exp(.)) and bonus, three static token-shift mixes, receptance-gated FFN
        t[f"{ffn}.receptance.weight"] = _normal(rng, (C, C))
        t[f"{att}.time_decay"] = _uniform(rng, (C,), -6.0, 1.0)
        t[f"{att}.time_first"] = _uniform(rng, (C,), -1.0, 1.0)
        for n in ("k", "v", "r"):
            t[f"{att}.time_mix_{n}"] = _uniform(rng, (1, 1, C), 0.0, 1.0)
        t[f"{ffn}.time_mix_k"] = _uniform(rng, (1, 1, C), 0.0, 1.0)
        t[f"{ffn}.time_mix_r"] = _uniform(rng, (1, 1, C), 0.0, 1.0)
    if version in (5, 6):
        t[f"{att}.gate.weight"] = _normal(rng, (C, C))
        t[f"{ffn}.receptance.weight"] = _normal(rng, (C, C))
        t[f"{att}.time_decay"] = _uniform(rng, (H, HEAD_SIZE), -6.0, 1.0)
        t[f"{att}.time_first"] = _uniform(rng, (H, HEAD_SIZE), -1.0, 1.0)
        for n in ("k", "v", "r", "g"):
            t[f"{att}.time_mix_{n}"] = _uniform(rng, (1, 1, C), 0.0, 1.0)
        t[f"{ffn}.time_mix_k"] = _uniform(rng, (1, 1, C), 0.0, 1.0)
        t[f"{ffn}.time_mix_r"] = _uniform(rng, (1, 1, C), 0.0, 1.0)
    if version == 6:
        t[f"{att}.time_mix_x"] = _uniform(rng, (1, 1, C), 0.0, 1.0)
        t[f"{att}.time_mix_w"] = _uniform(rng, (1, 1, C), 0.0, 1.0)
        t[f"{att}.time_mix_w1"] = _normal(rng, (5 * V6_TIME_MIX, C))
        t[f"{att}.time_mix_w2"] = _normal(rng, (5, C, V6_TIME_MIX))
        t[f"{att}.time_decay_w1"] = _normal(rng, (V6_TIME_DECAY, C))
        t[f"{att}.time_decay_w2"] = _normal(rng, (C, V6_TIME_DECAY))
    if version == 7:
        for n in ("r", "w", "k", "v", "a", "g"):
            t[f"{att}.x_{n}"] = _uniform(rng, (1, 1, C), 0.0, 1.0)
        t[f"{ffn}.x_k"] = _uniform(rng, (1, 1, C), 0.0, 1.0)
        t[f"{att}.w0"] = _uniform(rng, (1, 1, C), -6.0, 1.0)
        t[f"{att}.a0"] = _normal(rng, (1, 1, C), std=1.0)
        t[f"{att}.w1"] = _normal(rng, (V7_W, C))
        t[f"{att}.w2"] = _normal(rng, (C, V7_W))
        t[f"{att}.a1"] = _normal(rng, (V7_A, C))
        t[f"{att}.a2"] = _normal(rng, (C, V7_A))
        t[f"{att}.g1"] = _normal(rng, (V7_G, C))
        t[f"{att}.g2"] = _normal(rng, (C, V7_G))
        if layer > 0:
            t[f"{att}.v0"] = _normal(rng, (1, 1, C), std=1.0)
            t[f"{att}.v1"] = _normal(rng, (V7_V, C))
            t[f"{att}.v2"] = _normal(rng, (C, V7_V))
        t[f"{att}.r_k"] = _uniform(rng, (H, HEAD_SIZE), 0.0, 1.0)
        t[f"{att}.k_k"] = _uniform(rng, (1, 1, C), 0.0, 1.0)
        t[f"{att}.k_a"] = _uniform(rng, (1, 1, C), 0.0, 1.0)
    return t


def make_globals(version, C, V, seed):
    rng = np.random.default_rng([seed, 1 << 20])
    return {
        "emb.weight": _normal(rng, (V, C)),
        "head.weight": _normal(rng, (V, C)),
        "ln_out.weight": _normal(rng, (C,), mean=1.0),
        "ln_out.bias": _normal(rng, (C,)),
    }


def iter_tensors(config, seed=1000, num_layer=None, workers=None):
    """Yields (name, fp16 array) for a whole model, one block at a time (bounded host memory).  Blocks are
    generated by a few threads ahead of the consumer (each has its own seeded generator, so the result does not
    depend on the thread count)."""
    import os
    from concurrent.futures import ThreadPoolExecutor
    version, C, L, F, V = CONFIGS[config] if isinstance(config, str) else config
    L = num_layer or L
    if workers is None:
        workers = max(1, min(16, len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else 4))
    with ThreadPoolExecutor(workers) as pool:
        head = pool.submit(make_globals, version, C, V, seed)
        pending = [pool.submit(make_layer, version, layer, C, F, seed) for layer in range(min(L, workers))]
        for name, arr in head.result().items():
            yield name, arr
        for layer in range(L):
            block = pending.pop(0).result()
            nxt = layer + workers
            if nxt < L:
                pending.append(pool.submit(make_layer, version, nxt, C, F, seed))
            for name, arr in block.items():
                yield name, arr


def make_model(config, seed=1000, num_layer=None):
    return dict(iter_tensors(config, seed, num_layer))
