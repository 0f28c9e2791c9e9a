"""Tensor-parallel v6 job over the C ABI: one process per GPU, time-mix heads and FFN columns sharded, one
all-reduce (NCCL, a deferred op on the context's stream) per sub-block.

The reference is single-GPU; the op order per rank is that of `dispatch_layer` (src/runtime/v6.rs:701-992)
with these changes:
  * key / value / receptance / gate and the decay adapter's second matrix keep only the rows of the rank's
    heads; WKV, group norm and the gate run on those heads; `output` keeps the matching columns (a K shard)
    and produces a partial [C, T] sum in f32 that is all-reduced, then rounded to fp16 once;
  * ffn `key` keeps a block-aligned slice of rows, `value` the matching columns (K shard) -> f32 partial ->
    all-reduce; `receptance`, layer norms, token shifts and the small adapters are replicated;
  * the token-shift carry rows need all C channels, so they live in their own replicated tensors; the rank's
    WKV state holds only its heads;
  * the head keeps a slice of the vocabulary; logits are all-gathered.
K shards are cut on quantization-block boundaries (128 for Int8, 64 for NF4), so quantizing a shard gives
exactly the bytes and scales of the corresponding slice of the unsharded quantized matrix.
"""
import ctypes

import numpy as np

from . import (ACT_NONE, ACT_SILU, ACT_SQUARED_RELU, ACT_STABLE_EXP, ACT_TANH, F16, F32, QUANT_INT8, QUANT_NF4, QUANT_NONE, U32,
               Matrix, Op, activate, add, affine, blit, channel_mix, check, group_norm, layer_norm, lib, mul_activate, op_list,
               time_mix_v6, token_shift, transpose)

LN_EPS, GN_EPS = 1.0e-5, 64.0e-5
HEAD_SIZE = 64


# ---------------------------------------------------------------------------------------------------
# shard plan (pure host logic)
def shard_ranges(total, world, align=1):
    """`world` contiguous half-open ranges covering [0, total), each a whole number of `align`-sized units,
    sizes differing by at most one unit (larger ranges first)."""
    if total % align:
        raise ValueError(f"{total} is not a multiple of the shard unit {align}")
    units = total // align
    if units < world:
        raise ValueError(f"{units} units of {align} cannot be split {world} ways")
    base, extra = divmod(units, world)
    out, start = [], 0
    for r in range(world):
        n = (base + (1 if r < extra else 0)) * align
        out.append((start, start + n))
        start += n
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
        self.heads = shard_ranges(H, world, heads_per_unit)
        self.channels = [(a * HEAD_SIZE, b * HEAD_SIZE) for a, b in self.heads]
        self.ffn = shard_ranges(F, world, blk)
        if V % world:
            raise ValueError("the vocabulary must divide by the number of ranks (logits are all-gathered)")
        self.vocab = shard_ranges(V, world, V // world)


def discount_f16(w, discount):
    """f16(discount * f32(w)): the load-time rescale of `output` and ffn `value` (src/runtime/loader.rs:660-661)."""
    return (w.astype(np.float32) * np.float32(discount)).astype(np.float16)


def shard_tensors_v6(tensors, plan, rank, rescale=6):
    """The rank's slice of a v6 checkpoint ({name: fp16 array}); replicated tensors are passed through."""
    t, out = tensors, {}
    (c0, c1), (f0, f1), (v0, v1), (h0, h1) = plan.channels[rank], plan.ffn[rank], plan.vocab[rank], plan.heads[rank]
    num_layer = 1 + max(int(n.split(".")[1]) for n in t if n.startswith("blocks."))
    for name, w in t.items():
        if not name.startswith("blocks."):
            out[name] = w[v0:v1] if name == "head.weight" else w
            continue
        layer = int(name.split(".")[1])
        leaf = name.split(".", 2)[2]
        discount = 2.0 ** -(layer // rescale)
        if leaf in ("att.key.weight", "att.value.weight", "att.receptance.weight", "att.gate.weight", "att.time_decay_w2"):
            out[name] = w[c0:c1]
        elif leaf == "att.output.weight":
            out[name] = discount_f16(w, discount)[:, c0:c1] if discount != 1.0 else w[:, c0:c1]
        elif leaf in ("att.time_decay", "att.time_first"):
            out[name] = w.reshape(plan.H, HEAD_SIZE)[h0:h1]
        elif leaf in ("att.ln_x.weight", "att.ln_x.bias"):
            out[name] = w.reshape(-1)[c0:c1]
        elif leaf == "ffn.key.weight":
            out[name] = w[f0:f1]
        elif leaf == "ffn.value.weight":
            out[name] = discount_f16(w, discount)[:, f0:f1] if discount != 1.0 else w[:, f0:f1]
        else:
            out[name] = w
    out["__num_layer__"] = num_layer
    return out


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

    def all_reduce(self, x):
        h = ctypes.c_void_p()
        check(lib().wrk_op_all_reduce(self.handle, x.handle, ctypes.byref(h)))
        return Op(h, keep=(self, x))

    def all_gather(self, src, dst):
        h = ctypes.c_void_p()
        check(lib().wrk_op_all_gather(self.handle, src.handle, dst.handle, ctypes.byref(h)))
        return Op(h, keep=(self, src, dst))


class TpModelV6:
    """One rank of a tensor-parallel v6 model: sharded weights, state, and the op list of a job."""

    def __init__(self, ctx, comm, tensors, quant=QUANT_NONE, num_batch=1, rescale=6, use_graph=False):
        self.ctx, self.comm, self.quant, self.num_batch, self.rescale = ctx, comm, quant, num_batch, rescale
        self.use_graph = use_graph  # capture a job's launches (collectives included) into a CUDA graph
        V, C = tensors["emb.weight"].shape
        F = tensors["blocks.0.ffn.key.weight"].shape[0]
        self.plan = plan = ShardPlan(C, F, V, comm.world, quant)
        self.C, self.F, self.V, self.S = C, F, V, HEAD_SIZE
        rank = comm.rank
        self.C_loc = plan.channels[rank][1] - plan.channels[rank][0]
        self.H_loc = plan.heads[rank][1] - plan.heads[rank][0]
        self.F_loc = plan.ffn[rank][1] - plan.ffn[rank][0]
        self.V_loc = V // comm.world
        local = shard_tensors_v6(tensors, plan, rank, rescale)
        self.L = local.pop("__num_layer__")
        self.emb = np.ascontiguousarray(tensors["emb.weight"], dtype=np.float16)  # host gather, as the reference
        dev = lambda a: ctx.from_numpy(np.ascontiguousarray(a, dtype=np.float16))
        vec = lambda n: dev(local[n].reshape(-1))

        def mat(name, q=None):
            w = dev(local[name])
            q = self.quant if q is None else q
            return Matrix.quant_u8(w) if q == QUANT_INT8 else Matrix.quant_nf4(w) if q == QUANT_NF4 else Matrix.fp16(w)

        self.ln0 = (vec("blocks.0.ln0.weight"), vec("blocks.0.ln0.bias"))
        self.ln_out = (vec("ln_out.weight"), vec("ln_out.bias"))
        self.head = mat("head.weight", QUANT_NONE)
        self.layers, self.state = [], []
        for i in range(self.L):
            a, f, b = f"blocks.{i}.att", f"blocks.{i}.ffn", f"blocks.{i}"
            td = ctx.from_numpy(local[f"{a}.time_decay"].astype(np.float16).reshape(-1))
            tf = ctx.from_numpy(local[f"{a}.time_first"].astype(np.float32).reshape(-1))
            mix5 = np.stack([local[f"{a}.time_mix_{n}"].reshape(-1) for n in "wkvrg"])  # [5, C]
            self.layers.append({
                "ln1": (vec(f"{b}.ln1.weight"), vec(f"{b}.ln1.bias")), "ln2": (vec(f"{b}.ln2.weight"), vec(f"{b}.ln2.bias")),
                "gn": (vec(f"{a}.ln_x.weight"), vec(f"{a}.ln_x.bias")),
                "w_k": mat(f"{a}.key.weight"), "w_v": mat(f"{a}.value.weight"), "w_r": mat(f"{a}.receptance.weight"),
                "w_g": mat(f"{a}.gate.weight"), "w_o": mat(f"{a}.output.weight"),
                "ffn_k": mat(f"{f}.key.weight"), "ffn_v": mat(f"{f}.value.weight"), "ffn_r": mat(f"{f}.receptance.weight"),
                "time_decay": td, "time_first": tf,
                "mix_x": vec(f"{a}.time_mix_x"), "mix5": ctx.from_numpy(mix5.astype(np.float16), shape=[C, 1, 5, 1]),
                "ffn_mix_k": vec(f"{f}.time_mix_k"), "ffn_mix_r": vec(f"{f}.time_mix_r"),
                "tm_w1": mat(f"{a}.time_mix_w1", QUANT_NONE),
                # [5, C, D] -> five [D -> C] matrices, batched along z
                "tm_w2": Matrix.fp16(ctx.from_numpy(np.ascontiguousarray(local[f"{a}.time_mix_w2"], dtype=np.float16))),
                "td_w1": mat(f"{a}.time_decay_w1", QUANT_NONE), "td_w2": mat(f"{a}.time_decay_w2", QUANT_NONE),
            })
            self.state.append({
                "wkv": ctx.tensor(F32, [self.C_loc, self.S + 1, num_batch], zeros=True),  # row 0 unused carry copy
                "att": ctx.tensor(F32, [C, 1, num_batch], zeros=True),
                "ffn": ctx.tensor(F32, [C, 1, num_batch], zeros=True),
            })
        self.tm_dim = local["blocks.0.att.time_mix_w1"].shape[0] // 5
        self.td_dim = local["blocks.0.att.time_decay_w1"].shape[0]
        self.jobs = {}

    # ---------------------------------------------------------------------------------------------
    def _build(self, lens):
        """Op list (captured into a graph) and buffers for a job with `lens[b]` tokens of batch b, logits for
        the last token of every batch that has tokens."""
        ctx, C, S, T = self.ctx, self.C, self.S, sum(lens)
        Cl, Hl, Fl = self.C_loc, self.H_loc, self.F_loc
        c0 = self.plan.channels[self.comm.rank][0]
        turbo = T % 32 == 0
        cur, p, last = [], 0, []
        for b, n in enumerate(lens):
            for _ in range(n):
                cur += [b, p, n]
            if n:
                last.append((b, p + n - 1))
            p += n
        B = {"cursors": ctx.from_numpy(np.asarray(cur, dtype=np.uint32), shape=[3 * T, 1, 1, 1])}
        f16 = lambda *s: ctx.tensor(F16, list(s))
        f32 = lambda *s: ctx.tensor(F32, list(s))
        B.update(x=f16(C, T), att_x=f16(C, T), att_xx=f16(C, T, 1), tmx=f16(5 * self.tm_dim, T), tmt=f16(self.tm_dim, T, 5),
                 tm=f16(C, T, 5), att_sx=f16(C, T, 5), att_k=f32(Cl, T), att_v=f32(Cl, T), att_r=f32(Cl, T), att_g=f16(Cl, T),
                 att_w=f16(self.td_dim, T), td=f32(Cl, T), aux=f32(Cl, T), att_xl=f16(Cl, T), o32=f32(C, T), att_o=f16(C, T),
                 ffn_x=f16(C, T), ffn_kx=f16(C, T, 1), ffn_rx=f16(C, T, 1), ffn_k=f16(Fl, T), ffn_v=f16(C, T), ffn_r=f16(C, T),
                 head_x=f16(C, len(last)), logits=f32(self.V_loc, len(last)), all_logits=f32(self.V_loc, len(last), self.comm.world))
        cursors, x = B["cursors"], B["x"]
        ops = [layer_norm(*self.ln0, x, LN_EPS)]
        for i, (L, st) in enumerate(zip(self.layers, self.state)):
            ops += [blit(x, B["att_x"]), layer_norm(*L["ln1"], B["att_x"], LN_EPS),
                    token_shift(cursors, L["mix_x"], st["att"], B["att_x"], B["att_xx"], True),
                    L["tm_w1"].matmul_op(B["att_xx"].view(z=0), B["tmx"], ACT_TANH, turbo),
                    transpose(B["tmx"].reshape(self.tm_dim, 5, T), B["tmt"]),
                    L["tm_w2"].matmul_op(B["tmt"], B["tm"], ACT_NONE, turbo),
                    add(L["mix5"], B["tm"]),
                    token_shift(cursors, B["tm"], st["att"], B["att_x"], B["att_sx"], True),
                    L["w_k"].matmul_op(B["att_sx"].view(z=1), B["att_k"], ACT_NONE, turbo),
                    L["w_v"].matmul_op(B["att_sx"].view(z=2), B["att_v"], ACT_NONE, turbo),
                    L["w_r"].matmul_op(B["att_sx"].view(z=3), B["att_r"], ACT_NONE, turbo),
                    L["w_g"].matmul_op(B["att_sx"].view(z=4), B["att_g"], ACT_NONE, turbo),
                    L["td_w1"].matmul_op(B["att_sx"].view(z=0), B["att_w"], ACT_TANH, turbo),
                    L["td_w2"].matmul_op(B["att_w"], B["td"], ACT_NONE, turbo),
                    add(L["time_decay"], B["td"]), activate(B["td"], ACT_STABLE_EXP),
                    # this rank's channels of the normalised input: the carry source of the WKV op (its copy is unused)
                    blit(B["att_x"].view(x=(c0, c0 + Cl)), B["aux"]),
                    time_mix_v6(cursors, B["td"].reshape(S, Hl, T), L["time_first"].reshape(S, Hl), st["wkv"],
                                B["att_k"].reshape(S, Hl, T), B["att_v"].reshape(S, Hl, T), B["att_r"].reshape(S, Hl, T),
                                B["aux"].reshape(S, Hl, T)),
                    group_norm(L["gn"][0].reshape(S, Hl), L["gn"][1].reshape(S, Hl), B["aux"].reshape(S, Hl, T), GN_EPS),
                    blit(B["aux"], B["att_xl"]),
                    mul_activate(B["att_g"], B["att_xl"], ACT_SILU, ACT_NONE, ACT_NONE),
                    L["w_o"].matmul_op(B["att_xl"], B["o32"], ACT_NONE, turbo),
                    self.comm.all_reduce(B["o32"]), blit(B["o32"], B["att_o"]), add(B["att_o"], x)]
            # replicated token-shift carry: the normalised input of each sequence's last token
            ops += [blit(B["att_x"].view(y=t), st["att"].view(z=b)) for b, t in last]
            ops += [blit(x, B["ffn_x"]), layer_norm(*L["ln2"], B["ffn_x"], LN_EPS),
                    token_shift(cursors, L["ffn_mix_k"], st["ffn"], B["ffn_x"], B["ffn_kx"], True),
                    token_shift(cursors, L["ffn_mix_r"], st["ffn"], B["ffn_x"], B["ffn_rx"], True),
                    L["ffn_k"].matmul_op(B["ffn_kx"].view(z=0), B["ffn_k"], ACT_SQUARED_RELU, turbo),
                    L["ffn_v"].matmul_op(B["ffn_k"], B["o32"], ACT_NONE, turbo),
                    self.comm.all_reduce(B["o32"]), blit(B["o32"], B["ffn_v"]),
                    L["ffn_r"].matmul_op(B["ffn_rx"].view(z=0), B["ffn_r"], ACT_NONE, turbo),
                    channel_mix(cursors, st["ffn"], B["ffn_r"], B["ffn_v"], B["ffn_x"]), add(B["ffn_x"], x)]
            if (i + 1) % self.rescale == 0:
                ops.append(affine(x, 0.5, 0.0))
        ops += [blit(x.view(y=t), B["head_x"].view(y=j)) for j, (_, t) in enumerate(last)]
        ops += [layer_norm(*self.ln_out, B["head_x"], LN_EPS),
                self.head.matmul_op(B["head_x"], B["logits"], ACT_NONE, len(last) % 32 == 0),
                self.comm.all_gather(B["logits"], B["all_logits"])]
        cmd = ctx.encode(op_list(ops), use_graph=self.use_graph)
        return cmd, B, last, ops

    def run(self, tokens):
        """tokens: per batch a list of token ids (may be empty).  Returns {batch: logits (V,) of its last token}."""
        lens = tuple(len(t) for t in tokens)
        if sum(lens) == 0:
            return {}
        if lens not in self.jobs:
            self.jobs[lens] = self._build(lens)
        cmd, B, last, _ = self.jobs[lens]
        flat = [tok for t in tokens for tok in t]
        B["x"].load(self.emb[np.asarray(flat)])
        cmd.submit()
        self.ctx.synchronize()
        al = B["all_logits"].numpy().reshape(self.comm.world, len(last), self.V_loc)
        full = np.concatenate([al[r] for r in range(self.comm.world)], axis=1)  # [NH, V]
        return {b: full[j] for j, (b, _) in enumerate(last)}
