"""Quantized-model serialization: build -> save -> load gives the same bytes and the same logits.

The reference round-trips its `Model` through CBOR (examples/serde.rs:218-268; every tensor a
`TensorBlob {shape, data}`, src/tensor/serialization.rs:11-75).  The file is decoded here by a small CBOR
reader of the test's own and its tree compared with the reference's struct declarations
(src/runtime/v6.rs:28-130, v5.rs:60-125, v7.rs:55-150, src/tensor/matrix.rs:82-94).
"""
import importlib
import struct

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

wrk = importlib.import_module("web-rwkv_b200")
rt = importlib.import_module("web-rwkv_b200.runtime")
synth = importlib.import_module("web-rwkv_b200.synth")
LAST = 0
QUANT = {0: 1, 1: 2}  # layer 0 Int8, layer 1 NF4, layer 2 fp16
MATRICES = ["att.w_k", "att.w_v", "att.w_r", "att.w_o", "ffn.w_k", "ffn.w_v"]


def _cbor(buf, pos=0):
    """(value, next position); maps become lists of (key, value) so that the order of fields is kept."""
    b = buf[pos]
    major, info = b >> 5, b & 31
    pos += 1
    if info < 24:
        v = info
    else:
        n = 1 << (info - 24)
        v = int.from_bytes(buf[pos:pos + n], "big")
        pos += n
    if major == 0:
        return v, pos
    if major in (2, 3):
        data = bytes(buf[pos:pos + v])
        return (data if major == 2 else data.decode()), pos + v
    if major == 4:
        out = []
        for _ in range(v):
            item, pos = _cbor(buf, pos)
            out.append(item)
        return out, pos
    if major == 5:
        out = []
        for _ in range(v):
            k, pos = _cbor(buf, pos)
            item, pos = _cbor(buf, pos)
            out.append((k, item))
        return out, pos
    assert major == 7 and info == 22
    return None, pos


def _keys(node):
    return [k for k, _ in node]


def _logits(model, tokens):
    bundle = rt.Bundle(model, 1)
    inp = rt.RnnInput([(tokens, LAST)], 64)
    while inp.num_token():  # the prompt may take several jobs; the last one carries the logits
        out = bundle.infer(inp)[0].copy()
    inp.append(0, [int(np.argmax(out[-1]))])
    return out, bundle.infer(inp)[0].copy(), bundle.state_back(0)


@pytest.mark.parametrize("config", ["v6-tiny", "v5-tiny", "v7-tiny", "v4-tiny"])
def test_save_load_round_trip(ctx, tmp_path, config):
    tensors = synth.make_model(config, seed=1234)
    model = rt.ModelBuilder(ctx).add_tensors(tensors).quant(QUANT).build()
    first, second = tmp_path / "model.cbor", tmp_path / "again.cbor"
    model.save(first)
    loaded = rt.Model.load(ctx, first)
    a, b = model.info, loaded.info
    for field in ("version", "num_layer", "num_emb", "num_hidden", "num_vocab", "num_head"):
        assert getattr(a, field) == getattr(b, field)
    assert list(a.custom) == list(b.custom)
    # every packed byte, scale and table entry
    names = MATRICES + (["att.w_g", "ffn.w_r"] if a.version in (5, 6) else ["ffn.w_r"] if a.version == 4 else [])
    for layer in range(a.num_layer):
        for name in names:
            ka, wa, ma, qa = model.matrix_parts(layer, name)
            kb, wb, mb, qb = loaded.matrix_parts(layer, name)
            assert ka == kb == QUANT.get(layer, 0)
            assert wa.dtype == wb.dtype and np.array_equal(wa, wb), (layer, name)
            for x, y in ((ma, mb), (qa, qb)):
                assert (x is None) == (y is None)
                if x is not None:
                    assert x.tobytes() == y.tobytes(), (layer, name)
    # ... and everything else: the loaded model serializes to the same file
    loaded.save(second)
    assert first.read_bytes() == second.read_bytes()
    tokens = np.random.default_rng(7).integers(0, a.num_vocab - 1, 40).tolist()
    for got, want in zip(_logits(loaded, tokens), _logits(model, tokens)):
        assert np.array_equal(got, want)
    assert ctx.device_status() == 0


def test_file_is_the_reference_tree(ctx, tmp_path):
    tensors = synth.make_model("v6-tiny", seed=1234)
    model = rt.ModelBuilder(ctx).add_tensors(tensors).quant(QUANT).build()
    path = tmp_path / "model.cbor"
    model.save(path)
    buf = path.read_bytes()
    tree, end = _cbor(memoryview(buf))
    assert end == len(buf)
    assert _keys(tree) == ["context", "info", "rescale", "sep", "tensor"]  # src/runtime/v6.rs:36-43
    top = dict(tree)
    assert top["context"] is None and top["rescale"] == 6 and top["sep"] == 1024
    info = dict(top["info"])
    assert _keys(top["info"]) == ["version", "num_layer", "num_emb", "num_hidden", "num_vocab", "num_head", "custom"]
    assert info["version"] == "V6" and info["num_emb"] == 256 and info["num_layer"] == 3
    assert info["custom"] == [("V6", [("time_mix", synth.V6_TIME_MIX), ("time_decay", synth.V6_TIME_DECAY)])]
    tensor = dict(top["tensor"])
    assert _keys(top["tensor"]) == ["embed", "head", "layers"]
    assert _keys(tensor["embed"]) == ["layer_norm", "w"] and _keys(tensor["head"]) == ["layer_norm", "w"]
    emb = dict(dict(tensor["embed"])["w"])
    assert emb["shape"] == [256, 512, 1, 1]
    assert emb["data"] == np.ascontiguousarray(tensors["emb.weight"]).tobytes()
    layer0, layer1, layer2 = (dict(l) for l in tensor["layers"])
    assert _keys(tensor["layers"][0]) == ["att_layer_norm", "ffn_layer_norm", "att", "ffn"]
    assert _keys(layer0["att"]) == ["time_decay", "time_first", "time_mix_x", "time_mix", "time_decay_w1", "time_decay_w2",
                                    "time_mix_w1", "time_mix_w2", "w_k", "w_v", "w_r", "w_g", "w_o", "group_norm"]
    assert _keys(layer0["ffn"]) == ["time_mix_k", "time_mix_r", "w_k", "w_v", "w_r"]
    # Matrix variants (src/tensor/matrix.rs:82-94): Int8 {w, m}, Fp4 {q, w, m}, Fp16(tensor)
    (tag, body), = dict(layer0["att"])["w_k"]
    assert tag == "Int8" and _keys(body) == ["w", "m"]
    w, m = dict(dict(body)["w"]), dict(dict(body)["m"])
    assert w["shape"] == [256, 256, 1, 1] and len(w["data"]) == 256 * 256
    # min and max per 128 values (src/tensor/matrix.rs:162-178)
    assert m["shape"] == [2 * 256 * 256 // 128, 1, 1, 1] and len(m["data"]) == 2 * 2 * 512
    kind, wq, mm, _ = model.matrix_parts(0, "att.w_k")
    assert kind == 1 and w["data"] == wq.tobytes() and m["data"] == mm.tobytes()
    (tag, body), = dict(layer1["ffn"])["w_v"]
    assert tag == "Fp4" and _keys(body) == ["q", "w", "m"]
    q = dict(dict(body)["q"])
    assert q["shape"] == [16, 1, 1, 1] and struct.unpack("<16f", q["data"])[0] == -1.0
    assert dict(dict(body)["w"])["shape"] == [896 // 2, 256, 1, 1]
    (tag, body), = dict(layer2["att"])["w_o"]
    assert tag == "Fp16" and _keys(body) == ["shape", "data"]
    # time_first is f32 in the reference's struct (src/runtime/v6.rs:79), time_decay f16
    assert len(dict(dict(layer0["att"])["time_first"])["data"]) == 256 * 4
    assert len(dict(dict(layer0["att"])["time_decay"])["data"]) == 256 * 2


def test_damaged_files_are_refused(ctx, tmp_path):
    tensors = synth.make_model("v6-tiny", seed=1234)
    model = rt.ModelBuilder(ctx).add_tensors(tensors).quant(QUANT).build()
    path = tmp_path / "model.cbor"
    model.save(path)
    buf = path.read_bytes()
    cut = tmp_path / "cut.cbor"
    cut.write_bytes(buf[:len(buf) // 2])
    with pytest.raises(wrk.WrkError):
        rt.Model.load(ctx, cut)
    cut.write_bytes(b"\xa0")  # an empty map
    with pytest.raises(wrk.WrkError):
        rt.Model.load(ctx, cut)
    cut.write_bytes(buf.replace(b"time_mix_x", b"time_mix_y", 1))
    with pytest.raises(wrk.WrkError):
        rt.Model.load(ctx, cut)
    with pytest.raises(wrk.WrkError):
        rt.Model.load(ctx, tmp_path / "absent.cbor")
    assert ctx.device_status() == 0
