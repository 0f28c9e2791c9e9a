"""Host side of a model split across GPUs: one process per GPU, every rank holds a slice of the weights
(`ModelBuilder.shard`) and a bundle built on a communicator (`Bundle(model, num_batch, comm)`); the op lists, the
collectives and the slicing rules live in the C library (csrc/runtime/model.cpp, bundle.cpp, comm.cpp).

The reference is single-GPU.  Per rank the op order is that of `dispatch_layer` (src/runtime/v6.rs:701-958,
src/runtime/v7.rs:716-1007) with these changes:
  * key / value / receptance / gate and the per-channel adapters' second matrices keep only the rows of the rank's
    heads; WKV, group norm and the gate run on those heads; `output` keeps the matching columns (a K shard) and
    produces a partial [C, T] sum in f32 that is all-reduced, then rounded to fp16 once;
  * ffn `key` keeps a block-aligned slice of rows, `value` the matching columns (K shard) -> f32 partial ->
    all-reduce; ffn `receptance`, layer norms, token shifts and the adapters' first matrices are replicated;
  * the head keeps a slice of the vocabulary; logits are all-gathered.
K shards are cut on quantization-block boundaries (128 for Int8, 64 for NF4), so quantizing a shard gives
exactly the bytes and scales of the corresponding slice of the unsharded quantized matrix.
"""
import ctypes

import numpy as np

from . import F32, QUANT_INT8, QUANT_NF4, QUANT_NONE, Op, WrkError, check, lib

HEAD_SIZE = 64


# ---------------------------------------------------------------------------------------------------
# shard plan (pure host logic)
def shard_ranges(total, world, align=1):
    """`world` contiguous half-open ranges covering [0, total), each a whole number of `align`-sized units,
    sizes differing by at most one unit (larger ranges first): the library's rule (wrk_shard_range)."""
    out = []
    for r in range(world):
        b, e = ctypes.c_uint32(), ctypes.c_uint32()
        try:
            check(lib().wrk_shard_range(total, align, world, r, ctypes.byref(b), ctypes.byref(e)))
        except WrkError as err:
            raise ValueError(str(err)) from None
        out.append((b.value, e.value))
    return out


def quant_block(quant):
    return 128 if quant == QUANT_INT8 else 64 if quant == QUANT_NF4 else 1


class ShardPlan:
    """Which heads, FFN columns and vocabulary rows a rank owns."""

    def __init__(self, C, F, V, world, quant=QUANT_NONE):
        H = C // HEAD_SIZE
        blk = quant_block(quant)
        # a rank's channels are a K shard of `output`: whole quantization blocks, i.e. whole groups of heads
        heads_per_unit = max(1, blk // HEAD_SIZE)
        self.world, self.C, self.F, self.V, self.H = world, C, F, V, H
        self.block = blk
        self.heads = shard_ranges(H, world, heads_per_unit)
        self.channels = [(a * HEAD_SIZE, b * HEAD_SIZE) for a, b in self.heads]
        self.ffn = shard_ranges(F, world, max(blk, 8))
        if V % world:
            raise ValueError("the vocabulary must divide by the number of ranks (logits are all-gathered)")
        self.vocab = shard_ranges(V, world, V // world)


# ---------------------------------------------------------------------------------------------------
class Comm:
    """NCCL communicator bound to a context's stream (`wrk_comm_*`)."""

    def __init__(self, ctx, unique_id, rank, world):
        self.ctx, self.rank, self.world = ctx, rank, world
        self.handle = ctypes.c_void_p()
        buf = (ctypes.c_uint8 * 128).from_buffer_copy(bytes(unique_id))
        check(lib().wrk_comm_create(ctx.handle, buf, rank, world, ctypes.byref(self.handle)))
        # NCCL sets up its transports at the first collective of each kind (allocations, handle exchange): do
        # that here, eagerly, so that no later collective has to do it inside a stream capture
        a = ctx.tensor(F32, [1024], zeros=True)
        g = ctx.tensor(F32, [1024, world], zeros=True)
        ctx.run(self.all_reduce(a))
        ctx.run(self.all_gather(a, g))
        ctx.synchronize()

    @staticmethod
    def unique_id():
        buf = (ctypes.c_uint8 * 128)()
        check(lib().wrk_comm_unique_id(buf))
        return bytes(buf)

    def __del__(self):
        if getattr(self, "handle", None):
            lib().wrk_comm_release(self.handle)
            self.handle = None

    def wait(self, timeout_ms=10000):
        """Host wait for everything submitted so far, with the async-error poll and the time limit (`wrk_comm_wait`)."""
        check(lib().wrk_comm_wait(self.handle, int(timeout_ms)))

    def enable_peer_reduce(self, slot_bytes):
        """Collective: sets up the exchange region of the one-shot all-reduce over peer memory."""
        check(lib().wrk_comm_enable_peer_reduce(self.handle, ctypes.c_size_t(slot_bytes)))

    def peer_slot(self, slot, dtype, shape):
        from . import Tensor, _shape4
        h = ctypes.c_void_p()
        check(lib().wrk_comm_peer_slot(self.handle, slot, dtype, _shape4(list(shape)), ctypes.byref(h)))
        return Tensor(self.ctx, h)

    def peer_all_reduce(self, slot, count, dst):
        h = ctypes.c_void_p()
        check(lib().wrk_op_peer_all_reduce(self.handle, slot, ctypes.c_size_t(count), dst.handle, ctypes.byref(h)))
        return Op(h, keep=(self, dst))

    def all_reduce(self, x):
        h = ctypes.c_void_p()
        check(lib().wrk_op_all_reduce(self.handle, x.handle, ctypes.byref(h)))
        return Op(h, keep=(self, x))

    def all_gather(self, src, dst):
        h = ctypes.c_void_p()
        check(lib().wrk_op_all_gather(self.handle, src.handle, dst.handle, ctypes.byref(h)))
        return Op(h, keep=(self, src, dst))
