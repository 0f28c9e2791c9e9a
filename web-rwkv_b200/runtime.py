"""ctypes harness over the run() job API of include/wrk_runtime.h: ModelBuilder, Bundle/State,
RnnInput chunking and the dispatch → load → submit → back protocol (src/runtime/*.rs)."""
import ctypes

import numpy as np

from . import (QUANT_INT8, QUANT_NF4, QUANT_NONE, RNN_FULL, RNN_LAST, RNN_NONE, Context, Matrix, Tensor, WrkError,
               check, lib)


class ModelInfo(ctypes.Structure):
    _fields_ = [("version", ctypes.c_uint32), ("num_layer", ctypes.c_uint32), ("num_emb", ctypes.c_uint32),
                ("num_hidden", ctypes.c_uint32), ("num_vocab", ctypes.c_uint32), ("num_head", ctypes.c_uint32),
                ("custom", ctypes.c_uint32 * 4)]


class ModelBuilder:
    """`ModelBuilder` (src/runtime/model.rs:137-185) fed tensor by tensor instead of through a Reader."""

    def __init__(self, ctx):
        self.ctx = ctx
        self.handle = ctypes.c_void_p()
        check(lib().wrk_model_builder_create(ctx.handle, ctypes.byref(self.handle)))

    def __del__(self):
        if getattr(self, "handle", None):
            lib().wrk_model_builder_destroy(self.handle)
            self.handle = None

    def add_tensor(self, name, arr):
        arr = np.ascontiguousarray(arr, dtype=np.float16)
        shape = (ctypes.c_uint64 * arr.ndim)(*arr.shape)
        check(lib().wrk_model_builder_add_tensor(self.handle, name.encode(), shape, arr.ndim,
                                                 arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(arr.nbytes)))
        return self

    def add_tensors(self, items):
        for name, arr in (items.items() if isinstance(items, dict) else items):
            self.add_tensor(name, arr)
        return self

    LORA_MATRICES = r"blocks\.([0-9]+)\.(att|ffn)\.(key|value|receptance|gate|output)\.weight"

    def lora(self, tensors, blend=None, alpha=1.0):
        """`ModelBuilder::lora`: tensors {name: fp16 array} of one LoRA file; blend: [(regex, alpha), ...] in order,
        default `LoraBlend::full(alpha)` (src/runtime/loader.rs:119-124)."""
        index = ctypes.c_uint32()
        check(lib().wrk_model_builder_lora(self.handle, ctypes.byref(index)))
        for name, arr in tensors.items():
            arr = np.ascontiguousarray(arr, dtype=np.float16)
            shape = (ctypes.c_uint64 * arr.ndim)(*arr.shape)
            check(lib().wrk_model_builder_lora_tensor(self.handle, index, name.encode(), shape, arr.ndim,
                                                      arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(arr.nbytes)))
        for pattern, a in (blend if blend is not None else [(r".+", 1.0), (self.LORA_MATRICES, alpha)]):
            check(lib().wrk_model_builder_lora_blend(self.handle, index, pattern.encode(), ctypes.c_float(a)))
        return self

    def shard(self, rank, world, head_size=64, block=1):
        """Keep rank `rank`'s part of a model split `world` ways (`wrk_model_builder_shard`): before any tensor.
        block: 128 when any layer is Int8, 64 for NF4 / SF4, 1 for fp16."""
        check(lib().wrk_model_builder_shard(self.handle, rank, world, head_size, block))
        return self

    def quant(self, mapping):
        for layer, q in mapping.items():
            check(lib().wrk_model_builder_quant(self.handle, layer, q))
        return self

    def rescale(self, value):
        check(lib().wrk_model_builder_rescale(self.handle, value))
        return self

    def read_state(self):
        """`read_state` (src/runtime/v6.rs:1175-1208): (L, S + 2, C) f32 from the blocks.N.att.time_state tensors."""
        info = self.info()
        S = info.num_emb // info.num_head
        out = np.empty((info.num_layer, S + 2, info.num_emb), dtype=np.float32)
        check(lib().wrk_model_builder_read_state(self.handle, out.ctypes.data_as(ctypes.c_void_p),
                                                 ctypes.c_size_t(out.nbytes)))
        return out

    def info(self):
        info = ModelInfo()
        check(lib().wrk_model_builder_info(self.handle, ctypes.byref(info)))
        return info

    def build(self):
        h = ctypes.c_void_p()
        check(lib().wrk_model_builder_build(self.handle, ctypes.byref(h)))
        return Model(self.ctx, h)


class Model:
    def __init__(self, ctx, handle):
        self.ctx, self.handle = ctx, handle

    def __del__(self):
        if getattr(self, "handle", None):
            lib().wrk_model_release(self.handle)
            self.handle = None

    def save(self, path):
        """Serialize for Model (src/tensor/serialization.rs:11-75; examples/serde.rs:218-268): one CBOR file."""
        check(lib().wrk_model_save(self.handle, str(path).encode()))

    @classmethod
    def load(cls, ctx, path):
        """Seed::<Context, Model>::deserialize (src/tensor/serialization.rs:96-159)."""
        h = ctypes.c_void_p()
        check(lib().wrk_model_load(ctx.handle, str(path).encode(), ctypes.byref(h)))
        return cls(ctx, h)

    @property
    def info(self):
        info = ModelInfo()
        check(lib().wrk_model_info_get(self.handle, ctypes.byref(info)))
        return info

    def matrix_parts(self, layer, name):
        """(kind, w, m, q) numpy arrays of a layer's matrix, for packing-parity checks."""
        h = ctypes.c_void_p()
        check(lib().wrk_model_matrix(self.handle, 0xFFFFFFFF if layer is None else layer, name.encode(),
                                     ctypes.byref(h)))
        lib().wrk_matrix_parts  # borrowed handle: wrap without taking ownership of the matrix
        m = Matrix(self.ctx, None)
        m.handle = h
        try:
            kind, w, mm, q = m.parts()
            return kind, w.numpy(), (mm.numpy() if mm is not None else None), (q.numpy() if q is not None else None)
        finally:
            m.handle = None


class RnnInput:
    """`RnnInput` (src/runtime/infer/rnn.rs:194-253)."""

    def __init__(self, batches, token_chunk_size):
        """batches: list of (tokens, option) with option RNN_LAST or RNN_FULL."""
        self.handle = ctypes.c_void_p()
        self.num_batch = len(batches)
        check(lib().wrk_rnn_input_create(len(batches), token_chunk_size, ctypes.byref(self.handle)))
        for b, (tokens, option) in enumerate(batches):
            check(lib().wrk_rnn_input_set_option(self.handle, b, option))
            self.append(b, tokens)

    def __del__(self):
        if getattr(self, "handle", None):
            lib().wrk_rnn_input_destroy(self.handle)
            self.handle = None

    def append(self, batch, tokens):
        arr = np.ascontiguousarray(tokens, dtype=np.uint32)
        check(lib().wrk_rnn_input_append(self.handle, batch, arr.ctypes.data_as(ctypes.c_void_p),
                                         ctypes.c_size_t(arr.size)))

    @property
    def token_chunk_size(self):
        v = ctypes.c_uint32()
        check(lib().wrk_rnn_input_token_chunk_size(self.handle, ctypes.byref(v)))
        return v.value

    def num_token(self):
        v = ctypes.c_uint64()
        check(lib().wrk_rnn_input_num_token(self.handle, ctypes.byref(v)))
        return v.value

    def remaining(self, batch):
        v = ctypes.c_uint64()
        check(lib().wrk_rnn_input_remaining(self.handle, batch, ctypes.byref(v)))
        return v.value

    def step(self):
        check(lib().wrk_rnn_input_step(self.handle))

    def iter(self):
        return RnnIter(self)


class RnnIter:
    def __init__(self, inp):
        self.num_batch = inp.num_batch
        self.handle = ctypes.c_void_p()
        check(lib().wrk_rnn_iter_create(inp.handle, ctypes.byref(self.handle)))

    def __del__(self):
        if getattr(self, "handle", None):
            lib().wrk_rnn_iter_destroy(self.handle)
            self.handle = None

    def next(self):
        """[(len, option)] per batch; option RNN_NONE stands for None."""
        lens = (ctypes.c_uint32 * self.num_batch)()
        opts = (ctypes.c_int32 * self.num_batch)()
        check(lib().wrk_rnn_iter_next(self.handle, lens, opts))
        return [(lens[i], opts[i]) for i in range(self.num_batch)]


def redirect(info):
    """RnnInfo::redirect → (headers, inputs, outputs)."""
    n = len(info)
    lens = (ctypes.c_uint32 * n)(*[l for l, _ in info])
    opts = (ctypes.c_int32 * n)(*[o for _, o in info])
    total = sum(l for l, _ in info)
    headers = (ctypes.c_uint32 * max(total, 1))()
    nh = ctypes.c_uint32()
    inputs = (ctypes.c_uint32 * (2 * n))()
    outputs = (ctypes.c_uint32 * (2 * n))()
    check(lib().wrk_rnn_redirect(lens, opts, n, headers, ctypes.byref(nh), inputs, outputs))
    return (list(headers[: nh.value]), [(inputs[2 * i], inputs[2 * i + 1]) for i in range(n)],
            [(outputs[2 * i], outputs[2 * i + 1]) for i in range(n)])


HOOK_FN = ctypes.CFUNCTYPE(ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p))
HOOKS = ["POST_EMBED_LOADED", "POST_EMBED_LAYER_NORM", "PRE_ATT", "POST_ATT_LAYER_NORM", "PRE_ATT_TOKEN_SHIFT",
         "POST_ATT_TOKEN_SHIFT", "PRE_ATT_TOKEN_SHIFT_ADAPT", "POST_ATT_TOKEN_SHIFT_ADAPT_ACTIVATE", "POST_ATT_TOKEN_SHIFT_ADAPT",
         "PRE_ATT_GATED_TOKEN_SHIFT", "POST_ATT_GATED_TOKEN_SHIFT", "PRE_ATT_LINEAR", "POST_ATT_LINEAR",
         "PRE_ATT_TIME_DECAY_ADAPT", "POST_ATT_TIME_DECAY_ADAPT_ACTIVATE", "POST_ATT_TIME_DECAY_ADAPT",
         "PRE_ATT_TIME_DECAY_ACTIVATE", "POST_ATT_TIME_DECAY_ACTIVATE", "PRE_ATT_ADAPT", "POST_ATT_ADAPT", "PRE_ATT_CONTROL",
         "POST_ATT_CONTROL", "PRE_ATT_VALUE_RESIDUAL", "POST_ATT_VALUE_RESIDUAL", "PRE_ATT_TIME_MIX", "POST_ATT_TIME_MIX",
         "PRE_ATT_GATE", "POST_ATT_GATE", "PRE_ATT_OUT", "POST_ATT_OUT", "POST_ATT", "PRE_FFN", "POST_FFN_LAYER_NORM",
         "PRE_FFN_TOKEN_SHIFT", "POST_FFN_TOKEN_SHIFT", "PRE_FFN_LINEAR", "POST_FFN_ACTIVATE", "POST_FFN_LINEAR",
         "PRE_FFN_CHANNEL_MIX", "POST_FFN_CHANNEL_MIX", "POST_FFN", "PRE_HEAD", "POST_HEAD_LAYER_NORM", "POST_HEAD"]
HOOK = {name: i for i, name in enumerate(HOOKS)}  # wrk_hook, include/wrk_runtime.h


class Frame:
    """`Frame` (src/runtime/v6.rs:479-487) as a hook sees it: valid only during the callback."""

    def __init__(self, bundle, handle):
        self.bundle, self.handle = bundle, ctypes.c_void_p(handle)  # the callback receives the pointer as an int

    def buffer(self, name):
        h = ctypes.c_void_p()
        check(lib().wrk_frame_buffer(self.handle, name.encode(), ctypes.byref(h)))
        check(lib().wrk_tensor_retain(h))
        return Tensor(self.bundle.model.ctx, h)

    def num_token(self):
        t, n = ctypes.c_uint32(), ctypes.c_uint32()
        check(lib().wrk_frame_num_token(self.handle, ctypes.byref(t), ctypes.byref(n)))
        return t.value, n.value


class Bundle:
    """`Bundle<f16>` + `State` (src/runtime/v6.rs:489-521, src/runtime/model.rs:78-120)."""

    def __init__(self, model, num_batch, comm=None):
        """comm: the communicator of a split model's rank (`wrk_bundle_create_sharded`)."""
        self.model, self.num_batch, self.comm = model, num_batch, comm
        self.handle = ctypes.c_void_p()
        if comm is None:
            check(lib().wrk_bundle_create(model.handle, num_batch, ctypes.byref(self.handle)))
        else:
            check(lib().wrk_bundle_create_sharded(model.handle, num_batch, comm.handle, ctypes.byref(self.handle)))
        info = model.info
        self.vocab = (info.num_vocab + 7) // 8 * 8 if info.version >= 6 else info.num_vocab  # v4 / v5 heads are not padded

    def __del__(self):
        if getattr(self, "handle", None):
            lib().wrk_bundle_release(self.handle)
            self.handle = None

    def set_packed_cursors(self, packed):
        check(lib().wrk_bundle_set_packed_cursors(self.handle, int(packed)))

    def set_use_graph(self, use):
        check(lib().wrk_bundle_set_use_graph(self.handle, int(use)))

    def set_fused(self, fused):
        """0: one launch per reference op; 2 (the default of a new bundle): fused kernels, one launch per phase;
        1: fused kernels, v6 jobs of at most 8 tokens as one persistent kernel; 3: as 1, mma.sync engine only."""
        check(lib().wrk_bundle_set_fused(self.handle, int(fused)))

    def set_peer_reduce(self, on):
        """A sharded bundle's partial sums through peer memory (1, the default where available) or NCCL (0)."""
        check(lib().wrk_bundle_set_peer_reduce(self.handle, int(on)))

    def peer_reduce(self):
        on = ctypes.c_int32()
        check(lib().wrk_bundle_peer_reduce(self.handle, ctypes.byref(on)))
        return bool(on.value)

    def set_hook(self, hook, layer, fn):
        """`HookMap` entry (src/runtime/v6.rs:366-406, 572-581): fn(frame) -> Op or None is called while a job is built,
        at `hook` (a HOOK_* index) of layer `layer`; None clears it."""
        if not hasattr(self, "_hooks"):
            self._hooks = {}
        key = (int(hook), int(layer))
        if fn is None:
            check(lib().wrk_bundle_set_hook(self.handle, key[0], key[1], None, None))
            self._hooks.pop(key, None)
            return
        bundle = self

        def trampoline(_user, frame, out):
            try:
                op = fn(Frame(bundle, frame))
                if op is not None:
                    out[0] = op.handle.value if hasattr(op.handle, "value") else op.handle
                    op.handle = None  # the job's op list owns the reference now (the op keeps its buffers alive)
                return 0
            except Exception:  # reported as an invalid argument: exceptions cannot cross the C frames
                import traceback
                traceback.print_exc()
                return -103

        cb = HOOK_FN(trampoline)
        self._hooks[key] = cb
        check(lib().wrk_bundle_set_hook(self.handle, key[0], key[1], cb, None))

    def set_phase_timeline(self, max_phases):
        check(lib().wrk_bundle_set_phase_timeline(self.handle, int(max_phases)))

    def state_shape(self):
        s = (ctypes.c_uint32 * 4)()
        check(lib().wrk_state_init_shape(self.handle, s))
        return list(s)

    def state_back(self, batch):
        s = self.state_shape()
        arr = np.empty((s[2], s[1], s[0]), dtype=np.float32)
        check(lib().wrk_state_back(self.handle, batch, arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(arr.nbytes)))
        return arr

    def state_read(self, batch):
        """State::read: the slot as a device tensor [C, S + 2, L]."""
        h = ctypes.c_void_p()
        check(lib().wrk_state_read(self.handle, batch, ctypes.byref(h)))
        return Tensor(self.model.ctx, h)

    def state_write(self, tensor, batch):
        """State::write: a device tensor [C, S + 2, L] into the slot."""
        check(lib().wrk_state_write(self.handle, tensor.handle, batch))

    def state_embed(self, layer, backed):
        """State::embed: the shift row of one layer of a backed state."""
        backed = np.ascontiguousarray(backed, dtype=np.float32)
        out = np.empty(backed.shape[-1], dtype=np.float32)
        check(lib().wrk_state_embed(self.handle, layer, backed.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(backed.nbytes),
                                    out.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(out.nbytes)))
        return out

    def state_load(self, arr, batch):
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        check(lib().wrk_state_load(self.handle, arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(arr.nbytes), batch))

    def dispatch(self, info):
        lens = (ctypes.c_uint32 * self.num_batch)(*[l for l, _ in info])
        opts = (ctypes.c_int32 * self.num_batch)(*[o for _, o in info])
        h = ctypes.c_void_p()
        check(lib().wrk_bundle_dispatch(self.handle, lens, opts, ctypes.byref(h)))
        return Job(self, h, sum(l for l, _ in info))

    def infer(self, inp, logits=None):
        """SimpleRuntime::infer: returns per batch an array (rows, vocab) of fp32 logits (0 rows if none)."""
        if logits is None:
            logits = np.empty((max(inp.token_chunk_size, 1), self.vocab), dtype=np.float32)
        outs = (ctypes.c_uint32 * (2 * self.num_batch))()
        nh = ctypes.c_uint32()
        check(lib().wrk_runtime_infer(self.handle, inp.handle, logits.ctypes.data_as(ctypes.c_void_p),
                                      ctypes.c_size_t(logits.size), outs, ctypes.byref(nh)))
        return [logits[outs[2 * i]: outs[2 * i + 1]] for i in range(self.num_batch)]


class Job:
    def __init__(self, bundle, handle, num_token):
        self.bundle, self.handle, self.num_token = bundle, handle, num_token

    def __del__(self):
        if getattr(self, "handle", None):
            lib().wrk_job_release(self.handle)
            self.handle = None

    def load(self, tokens):
        arr = np.ascontiguousarray(tokens, dtype=np.uint32)
        check(lib().wrk_job_load(self.handle, arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(arr.size)))

    def submit(self):
        check(lib().wrk_job_submit(self.handle))

    def back(self, logits=None):
        nb = self.bundle.num_batch
        if logits is None:
            logits = np.empty((max(self.num_token, 1), self.bundle.vocab), dtype=np.float32)
        outs = (ctypes.c_uint32 * (2 * nb))()
        nh = ctypes.c_uint32()
        check(lib().wrk_job_back(self.handle, logits.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(logits.size),
                                 outs, ctypes.byref(nh)))
        return [logits[outs[2 * i]: outs[2 * i + 1]] for i in range(nb)]

    def phase_timeline(self):
        """(num_phases, 2, num_ctas) uint64 device-timer stamps (ns) of the job's last run: [:, 0] phase starts,
        [:, 1] phase ends."""
        nph, ncta = ctypes.c_uint32(), ctypes.c_uint32()
        buf = np.zeros(2 * 4096 * 256, dtype=np.uint64)
        check(lib().wrk_job_phase_timeline(self.handle, buf.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(buf.size),
                                           ctypes.byref(nph), ctypes.byref(ncta)))
        return buf[: 2 * nph.value * ncta.value].reshape(nph.value, 2, ncta.value)

    def num_kernels(self):
        n = ctypes.c_uint64()
        check(lib().wrk_job_num_kernels(self.handle, ctypes.byref(n)))
        return n.value


def job_load_embed(job, embeds, row0):
    """Job::load for device-resident `Token::Embed` rows."""
    check(lib().wrk_job_load_embed(job.handle, embeds.handle, row0))


def job_output(job):
    h = ctypes.c_void_p()
    check(lib().wrk_job_output(job.handle, ctypes.byref(h)))
    check(lib().wrk_tensor_retain(h))
    return Tensor(job.bundle.model.ctx, h)
