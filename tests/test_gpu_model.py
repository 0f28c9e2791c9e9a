"""End-to-end run() jobs (v5 / v6 / v7) against the full-model CPU oracle: packed weights bit for
bit, logits and recurrent state within max-abs 2e-2 / cosine >= 0.9995, across chunked prefill,
mixed batches and decode.  The reference has no model-level test; the oracle restates its op lists.
"""
import importlib

import numpy as np
import pytest

from oracle import model as omodel
from oracle import oracle
from tests.util import assert_close, assert_state_close

pytestmark = pytest.mark.gpu

rt = importlib.import_module("web-rwkv_b200.runtime")
synth = importlib.import_module("web-rwkv_b200.synth")
LAST, FULL, NONE = 0, 1, 2


def _build(ctx, config, quant, seed=1000, num_layer=None):
    tensors = synth.make_model(config, seed=seed, num_layer=num_layer)
    model = rt.ModelBuilder(ctx).add_tensors(tensors).quant(quant).build()
    ref = omodel.OracleModel(tensors, quant)
    return tensors, model, ref


def _drive(bundle, ref, batches, chunk, wide=True):
    """Runs the same RnnInput through the CUDA runtime and the oracle; yields per-job logits pairs."""
    nb = len(batches)
    inp = rt.RnnInput(batches, chunk)
    remaining = [list(t) for t, _ in batches]
    state = ref.init_state(nb)
    pairs = []
    while inp.num_token():
        info = inp.iter().next()
        got = [g.copy() for g in bundle.infer(inp)]
        want = ref.run(state, remaining, info, wide=wide)
        remaining = [r[l:] for r, (l, _) in zip(remaining, info)]
        pairs.append((info, got, want))
    return pairs, state


def _check(pairs, bundle, state):
    for info, got, want in pairs:
        for b, (g, w) in enumerate(zip(got, want)):
            assert g.shape == w.shape, (info, b, g.shape, w.shape)
            if g.size:
                assert_close(g, w, f"logits batch {b} job {info}")
    for b in range(bundle.num_batch):
        got_state = bundle.state_back(b)
        want_state = np.stack([s[b] for s in state])
        assert_state_close(got_state, want_state, f"state batch {b}")  # relative to each layer's scale


@pytest.mark.parametrize("config,quant", [
    ("v6-tiny", {0: 1, 1: 2}),      # layer 0 Int8, layer 1 NF4, layer 2 fp16
    ("v5-tiny", {0: 1, 1: 2}),
    ("v7-tiny", {0: 1, 1: 2}),
    ("v4-tiny", {0: 1, 1: 2}),      # src/runtime/v4.rs: per-channel WKV with a running maximum, state [C, 5, B]
    ("v6-tiny", {0: 3, 1: 3, 2: 2}),  # Quant::SF4 (Student-t code book, nu = 5) on layers 0-1
])
def test_mixed_batches_chunked_prefill_then_decode(ctx, config, quant):
    rng = np.random.default_rng(2001)
    tensors, model, ref = _build(ctx, config, quant)
    bundle = rt.Bundle(model, 4)
    V = model.info.num_vocab
    batches = [(rng.integers(0, V - 1, 70).tolist(), LAST), (rng.integers(0, V - 1, 1).tolist(), LAST), ([], FULL),
               (rng.integers(0, V - 1, 37).tolist(), FULL)]
    pairs, state = _drive(bundle, ref, batches, 64)
    assert len(pairs) >= 2
    _check(pairs, bundle, state)


@pytest.mark.parametrize("config", ["v6-tiny", "v5-tiny", "v7-tiny", "v4-tiny"])
@pytest.mark.parametrize("fused", [0, 1, 2, 3])  # op by op / one persistent kernel per job (tensor-core, where the matrices allow) / one launch per phase / persistent mma.sync kernel
def test_decode_loop(ctx, config, fused):
    rng = np.random.default_rng(2002)
    tensors, model, ref = _build(ctx, config, {0: 1, 1: 1, 2: 1})
    bundle = rt.Bundle(model, 1)
    bundle.set_fused(fused)
    V = model.info.num_vocab
    prompt = rng.integers(0, V - 1, 9).tolist()
    state = ref.init_state(1)
    inp = rt.RnnInput([(prompt, LAST)], 32)
    got = bundle.infer(inp)[0].copy()
    want = ref.run(state, [prompt], [(len(prompt), LAST)])[0]
    assert_close(got, want, "prompt logits")
    for step in range(6):  # greedy decode on the oracle's token so both sides see the same input
        tok = int(np.argmax(want[-1]))
        inp.append(0, [tok])
        got = bundle.infer(inp)[0].copy()
        want = ref.run(state, [[tok]], [(1, LAST)])[0]
        assert_close(got, want, f"decode step {step}")
    assert_close(bundle.state_back(0), np.stack([s[0] for s in state]), "state")


@pytest.mark.parametrize("config,quant,saved", [("v7-tiny", {0: 1, 1: 2}, 16), ("v7-tiny", {}, 16), ("v5-tiny", {0: 1}, 10),
                                                ("v6-tiny", {0: 2}, 9)])
def test_merged_elementwise_launches_are_bit_identical_to_the_op_list(ctx, config, quant, saved):
    """layer_norm_copy, token_shift_multi / _lora, pack_v7, group_norm_gate and channel_mix_add stand for runs of the
    reference's elementwise ops (src/runtime/v7.rs:762-928, v6.rs:759-949, v5.rs:686-870); the strict mode runs those
    ops one by one."""
    rng = np.random.default_rng(2003)
    tensors, model, ref = _build(ctx, config, quant)
    V = model.info.num_vocab
    batches = [(rng.integers(0, V - 1, 45).tolist(), FULL), (rng.integers(0, V - 1, 3).tolist(), LAST)]
    results = []
    for fused in (2, 0):
        bundle = rt.Bundle(model, 2)
        bundle.set_fused(fused)
        inp = rt.RnnInput(batches, 32)
        outs = []
        while inp.num_token():
            outs += [g.copy() for g in bundle.infer(inp)]
        for _ in range(0 if config == "v6-tiny" else 3):  # single-token jobs (v6 has fused kernels of its own for those)
            inp.append(0, [5])
            inp.append(1, [7])
            outs += [g.copy() for g in bundle.infer(inp)]
        before = ctx.launch_count()
        inp.append(0, list(range(9, 20)))
        inp.append(1, [11])
        outs += [g.copy() for g in bundle.infer(inp)]
        results.append((outs, [bundle.state_back(b) for b in range(2)], ctx.launch_count() - before))
    (a, sa, la), (b, sb, lb) = results
    assert len(a) == len(b)
    # v7: bit for bit.  v5 / v6 jobs of more than 8 tokens also take the WKV recurrence in blocks of 16 tokens, which
    # sums in another order (the merged elementwise ops are compared bit for bit one by one in test_gpu_support.py)
    exact = config == "v7-tiny"
    for i, (x, y) in enumerate(zip(a, b)):
        if exact:
            assert np.array_equal(x, y), (i, float(np.abs(x - y).max()) if x.size else None)
        elif x.size:
            assert_close(x, y, f"logits {i}")
    for x, y in zip(sa, sb):
        if exact:
            assert np.array_equal(x, y), float(np.abs(x - y).max())
        else:
            assert_state_close(x, y, "state")
    assert lb - la == saved * model.info.num_layer, (la, lb)


def test_packed_bytes_and_scales_match_the_oracle(ctx):
    tensors, model, ref = _build(ctx, "v6-tiny", {0: 1, 1: 2})
    names = {"att.w_k": "w_k", "att.w_v": "w_v", "att.w_r": "w_r", "att.w_g": "w_g", "att.w_o": "w_o",
             "ffn.w_k": "ffn_k", "ffn.w_v": "ffn_v", "ffn.w_r": "ffn_r"}
    for layer in (0, 1):
        for cname, oname in names.items():
            kind, w, m, q = model.matrix_parts(layer, cname)
            want = ref.layers[layer][oname]
            assert kind == want.kind
            assert np.array_equal(w.reshape(want.w.shape), want.w), (layer, cname)
            assert np.array_equal(m.reshape(-1).view(np.uint16), want.scale.view(np.uint16)), (layer, cname)
    kind, w, m, q = model.matrix_parts(None, "head.w")
    assert kind == 0 and np.array_equal(w.reshape(tensors["head.weight"].shape), tensors["head.weight"])


def test_rescale_discount_is_applied_before_quantization(ctx):
    # rescale = 2: layers 2.. have output / ffn value weights halved in fp16 *before* packing
    tensors = synth.make_model("v6-tiny", seed=5)
    model = rt.ModelBuilder(ctx).add_tensors(tensors).quant({0: 1, 1: 1, 2: 1}).rescale(2).build()
    ref = omodel.OracleModel(tensors, {0: 1, 1: 1, 2: 1}, rescale=2)
    for cname, oname in (("att.w_o", "w_o"), ("ffn.w_v", "ffn_v"), ("att.w_k", "w_k")):
        kind, w, m, q = model.matrix_parts(2, cname)
        assert np.array_equal(w.reshape(ref.layers[2][oname].w.shape), ref.layers[2][oname].w)
        assert np.array_equal(m.reshape(-1).view(np.uint16), ref.layers[2][oname].scale.view(np.uint16))
    bundle = rt.Bundle(model, 1)
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, 511, 33).tolist()
    pairs, state = _drive(bundle, ref, [(prompt, FULL)], 32)
    _check(pairs, bundle, state)


def test_packed_cursors_reproduce_the_reference_wrap(ctx):
    # a single sequence receiving 256 tokens in one job: packed len wraps to 0 and neither carry row is
    # written (the reference's behaviour); the wide cursor form carries them
    tensors, model, ref = _build(ctx, "v6-tiny", {})
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, 511, 256).tolist()
    for packed in (True, False):
        bundle = rt.Bundle(model, 1)
        bundle.set_packed_cursors(packed)
        pairs, state = _drive(bundle, ref, [(prompt, LAST)], 256, wide=not packed)
        _check(pairs, bundle, state)
        carry = bundle.state_back(0)[:, 0, :]
        assert (carry == 0).all() == packed


def test_state_load_back_and_errors(ctx):
    tensors, model, ref = _build(ctx, "v6-tiny", {})
    bundle = rt.Bundle(model, 2)
    shape = bundle.state_shape()
    assert shape == [256, 66, 3, 1]
    rng = np.random.default_rng(4)
    st = rng.standard_normal((3, 66, 256)).astype(np.float32)
    bundle.state_load(st, 1)
    assert np.array_equal(bundle.state_back(1), st)
    assert (bundle.state_back(0) == 0).all()
    wrk = importlib.import_module("web-rwkv_b200")
    with pytest.raises(wrk.WrkError) as e:
        bundle.state_load(st, 2)
    assert e.value.status == -7
    with pytest.raises(wrk.WrkError) as e:
        bundle.infer(rt.RnnInput([([], LAST), ([], LAST)], 32))
    assert e.value.status == -30
    with pytest.raises(wrk.WrkError) as e:
        rt.ModelBuilder(ctx).add_tensors({"emb.weight": np.zeros((8, 64), np.float16)}).build()
    assert e.value.status in (-20, -21)


def test_state_write_read_embed(ctx):
    # State::write / read / embed (src/runtime/model.rs:98-102, src/runtime/v6.rs:223-262): device-to-device hand-off
    tensors, model, ref = _build(ctx, "v6-tiny", {})
    bundle = rt.Bundle(model, 3)
    V = model.info.num_vocab
    rng = np.random.default_rng(11)
    bundle.infer(rt.RnnInput([(rng.integers(0, V - 1, 9).tolist(), LAST), ([], LAST), ([], LAST)], 32))
    want = bundle.state_back(0)
    assert np.abs(want).max() > 0
    moved = bundle.state_read(0)                       # slot 0 as a device tensor [C, S + 2, L]
    assert moved.shape[:3] == [256, 66, 3]
    assert np.array_equal(moved.numpy().reshape(3, 66, 256), want)
    bundle.state_write(moved, 2)                       # ... into slot 2, no host copy
    assert np.array_equal(bundle.state_back(2), want)
    assert (bundle.state_back(1) == 0).all()
    for layer in range(3):
        assert np.array_equal(bundle.state_embed(layer, want), want[layer, 0])
    # the copied slot continues exactly like the original
    tok = int(rng.integers(0, V - 1))
    out = bundle.infer(rt.RnnInput([([tok], LAST), ([], LAST), ([tok], LAST)], 32))
    assert np.array_equal(out[0], out[2])
    wrk = importlib.import_module("web-rwkv_b200")
    with pytest.raises(wrk.WrkError) as e:
        bundle.state_write(moved, 3)
    assert e.value.status == -7
    with pytest.raises(wrk.WrkError) as e:
        bundle.state_write(ctx.tensor(wrk.F32, [256, 66, 2], zeros=True), 0)
    assert e.value.status == -5
    with pytest.raises(wrk.WrkError) as e:
        bundle.state_embed(3, want)
    assert e.value.status == -8
    assert ctx.device_status() == 0


def test_hooks_insert_ops_at_their_points(ctx):
    # HookMap (src/runtime/v6.rs:366-406, 572-581): a callback per (hook, layer) returns an op for the job's op list
    wrk = importlib.import_module("web-rwkv_b200")
    tensors, model, ref = _build(ctx, "v6-tiny", {0: 1})
    info = model.info
    V, C, L = info.num_vocab, info.num_emb, info.num_layer
    tokens = [5, 9, 2]
    plain = rt.Bundle(model, 1)
    want_plain = plain.infer(rt.RnnInput([(tokens, FULL)], 32))[0].copy()

    # (1) capture: the embedding after its layer norm
    bundle = rt.Bundle(model, 1)
    saved = ctx.tensor(wrk.F16, [C, len(tokens)])
    seen = []

    def capture(frame):
        seen.append(frame.num_token())
        return wrk.blit(frame.buffer("x"), saved)

    bundle.set_hook(rt.HOOK["POST_EMBED_LAYER_NORM"], 0, capture)
    got = bundle.infer(rt.RnnInput([(tokens, FULL)], 32))[0].copy()
    assert seen == [(3, 3)]
    assert np.array_equal(got, want_plain)  # a copy changes nothing ...
    emb = np.ascontiguousarray(tensors["emb.weight"][tokens])
    oracle.layer_norm(tensors["blocks.0.ln0.weight"].reshape(-1), tensors["blocks.0.ln0.bias"].reshape(-1), emb, 1e-5)
    assert_close(saved.numpy().reshape(len(tokens), C), emb, "captured embedding")

    # (2) an op that changes the result: the residual stream zeroed after the last layer -> logits = head . ln_out.bias
    bundle.set_hook(rt.HOOK["POST_EMBED_LAYER_NORM"], 0, None)
    bundle.set_hook(rt.HOOK["POST_FFN"], L - 1, lambda frame: wrk.affine(frame.buffer("x"), 0.0, 0.0))
    got = bundle.infer(rt.RnnInput([(tokens, LAST)], 32))[0].copy()
    bias = np.ascontiguousarray(tensors["ln_out.bias"].reshape(1, C))
    want = np.zeros((1, V), dtype=np.float32)
    oracle.matmul(oracle.MAT_FP16, np.ascontiguousarray(tensors["head.weight"]), None, bias, want)
    assert_close(got, want, "zeroed residual")

    # (3) hooks switch the fused kernels off (they have no such points); clearing brings them back
    hooked = bundle.dispatch([(1, LAST)]).num_kernels()
    bundle.set_hook(rt.HOOK["POST_FFN"], L - 1, None)
    fused = bundle.dispatch([(1, LAST)]).num_kernels()
    strict = rt.Bundle(model, 1)
    strict.set_fused(0)
    assert fused < hooked and hooked == strict.dispatch([(1, LAST)]).num_kernels() + 1
    with pytest.raises(wrk.WrkError):
        bundle.set_hook(rt.HOOK["PRE_ATT"], L, lambda frame: None)
    assert ctx.device_status() == 0


def test_two_jobs_of_one_shape_dispatched_before_back(ctx):
    # the reference dispatches the next job while the current one runs (src/runtime/mod.rs:215-260): two live jobs of
    # the same (tokens, header rows) but different per-batch lengths keep their own output ranges
    tensors, model, ref = _build(ctx, "v6-tiny", {0: 1})
    bundle = rt.Bundle(model, 2)
    V = model.info.num_vocab
    first = bundle.dispatch([(2, FULL), (0, FULL)])
    second = bundle.dispatch([(1, FULL), (1, FULL)])
    first.load([5, 6])
    first.submit()
    got_first = [g.copy() for g in first.back()]
    second.load([7, 8])
    second.submit()
    got_second = [g.copy() for g in second.back()]
    assert [g.shape[0] for g in got_first] == [2, 0]
    assert [g.shape[0] for g in got_second] == [1, 1]
    state = ref.init_state(2)
    want_first = ref.run(state, [[5, 6], []], [(2, FULL), (0, FULL)])
    want_second = ref.run(state, [[7], [8]], [(1, FULL), (1, FULL)])
    assert_close(got_first[0], want_first[0], "first job")
    assert_close(got_second[0], want_second[0], "second job, batch 0")
    assert_close(got_second[1], want_second[1], "second job, batch 1")


def test_second_context_on_another_device(ctx):
    # shared-memory opt-ins are per device: the first launches of every kernel family on a second GPU
    import subprocess
    if subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True).stdout.count("GPU ") < 2:
        pytest.skip("needs two GPUs")
    wrk = importlib.import_module("web-rwkv_b200")
    other = wrk.Context(1)
    tensors = synth.make_model("v6-tiny", seed=1000)
    outs = []
    for c in (ctx, other):
        model = rt.ModelBuilder(c).add_tensors(tensors).quant({0: 1, 1: 2}).build()
        bundle = rt.Bundle(model, 1)
        prompt = rt.RnnInput([(list(range(1, 41)), LAST)], 64)   # GEMM path
        while prompt.num_token():
            out = bundle.infer(prompt)[0].copy()
        prompt.append(0, [3])
        outs.append((out, bundle.infer(prompt)[0].copy()))      # fused decode path
        assert c.device_status() == 0
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    other.synchronize()


def test_config1_v6_0p1b_int8_256_tokens_chunk_32(ctx):
    # BASELINE config 1: n_embd 768, 12 layers, FFN 2688, vocab 65536, all layers Int8, one sequence of
    # 256 uniform-random tokens, token_chunk_size 32, num_batch 1
    rng = np.random.default_rng(2001)
    quant = {i: 1 for i in range(12)}
    tensors, model, ref = _build(ctx, "v6-0.1b", quant, seed=1001)
    bundle = rt.Bundle(model, 1)
    prompt = rng.integers(0, 65535, 256).tolist()
    pairs, state = _drive(bundle, ref, [(prompt, LAST)], 32)
    assert len(pairs) == 8 and pairs[-1][1][0].shape == (1, 65536)
    _check(pairs, bundle, state)


def test_lora_is_merged_before_quantization(ctx):
    # ModelBuilder::lora with LoraBlend::full(0.5): vectors of the LoRA replace the model's, matrices get
    # alpha / rank * lora.0 x lora.1 (TensorOp::blend_lora) before they are quantized (src/runtime/loader.rs:393-686)
    rng = np.random.default_rng(77)
    tensors = synth.make_model("v6-tiny", seed=1000)
    R, alpha = 8, 0.5
    lora, merged = {}, dict(tensors)
    for name in ("blocks.0.ln1.weight", "blocks.1.att.time_first", "blocks.2.ffn.time_mix_k"):
        lora[name] = (tensors[name].astype(np.float32) + 0.1 * rng.standard_normal(tensors[name].shape)).astype(np.float16)
        merged[name] = lora[name]
    for name in ("blocks.0.att.key.weight", "blocks.1.ffn.value.weight", "blocks.2.att.output.weight"):
        M, K = tensors[name].shape
        base = name.replace(".weight", "")
        lora[base + ".lora.0"] = (0.05 * rng.standard_normal((K, R))).astype(np.float16)
        lora[base + ".lora.1"] = (0.05 * rng.standard_normal((M, R))).astype(np.float16)
        w = tensors[name].copy()
        oracle.blend_lora([alpha / R, 1.0, 0, 0], lora[base + ".lora.0"], lora[base + ".lora.1"], w)
        assert np.abs(w.astype(np.float32) - tensors[name].astype(np.float32)).max() > 1e-3  # the LoRA does something
        merged[name] = w
    # a tensor of a matrix's own name is added with factor (alpha, 1); one that no pattern matches is ignored
    quant = {0: 1, 1: 2}
    model = rt.ModelBuilder(ctx).add_tensors(tensors).lora(lora, alpha=alpha).quant(quant).build()
    ref = omodel.OracleModel(merged, quant)
    kind, w, m, q = model.matrix_parts(2, "att.w_o")  # layer 2 stays fp16: the merged weights themselves
    want = merged["blocks.2.att.output.weight"]
    assert np.abs(w.reshape(want.shape).astype(np.float32) - want.astype(np.float32)).max() <= 2.5e-4
    bundle = rt.Bundle(model, 2)
    V = model.info.num_vocab
    batches = [(rng.integers(0, V - 1, 40).tolist(), LAST), (rng.integers(0, V - 1, 5).tolist(), FULL)]
    pairs, state = _drive(bundle, ref, batches, 32)
    _check(pairs, bundle, state)
    # and the LoRA changed the logits: the plain model's differ
    plain = rt.Bundle(rt.ModelBuilder(ctx).add_tensors(tensors).quant(quant).build(), 1)
    inp = rt.RnnInput([(batches[1][0], LAST)], 32)
    a = plain.infer(inp)[0].copy()
    with_lora = rt.Bundle(model, 1)
    inp = rt.RnnInput([(batches[1][0], LAST)], 32)
    bb = with_lora.infer(inp)[0].copy()
    assert np.abs(a - bb).max() > 1e-2
    with pytest.raises(rt.WrkError) as e:  # a pattern that is not a regular expression
        rt.ModelBuilder(ctx).add_tensors(tensors).lora({}, blend=[("(", 1.0)])
    assert e.value.status == -103


def test_read_state_from_the_model_file(ctx):
    # read_state (src/runtime/v6.rs:1175-1208): blocks.N.att.time_state (H, S, S) -> rows 1..S of the f32 [C, S + 2, L]
    # state, column h * S + j of row 1 + i holding time_state[h][i][j]; State::load takes it for a batch slot
    rng = np.random.default_rng(88)
    tensors = dict(synth.make_model("v6-tiny", seed=1000))
    info = rt.ModelBuilder(ctx).add_tensors(tensors).info()
    L, C, H = info.num_layer, info.num_emb, info.num_head
    S = C // H
    for layer in range(L):
        tensors[f"blocks.{layer}.att.time_state"] = rng.standard_normal((H, S, S)).astype(np.float16)
    builder = rt.ModelBuilder(ctx).add_tensors(tensors)
    got = builder.read_state()
    want = np.zeros((L, S + 2, C), dtype=np.float32)
    for layer in range(L):
        ts = tensors[f"blocks.{layer}.att.time_state"].astype(np.float32)  # [h][i][j]
        want[layer, 1:S + 1, :] = ts.transpose(1, 0, 2).reshape(S, C)
    assert np.array_equal(got, want)
    bundle = rt.Bundle(builder.build(), 2)
    bundle.state_load(got, 1)
    assert np.array_equal(bundle.state_back(1).reshape(got.shape), got)
    assert not bundle.state_back(0).any()
    with pytest.raises(rt.WrkError) as e:  # a file without the tensors
        rt.ModelBuilder(ctx).add_tensors(synth.make_model("v6-tiny", seed=1000)).read_state()
    assert e.value.status == -21
