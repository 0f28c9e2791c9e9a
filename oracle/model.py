"""Full-model CPU oracle: the v4 / v5 / v6 / v7 `run()` job of the reference, op by op.

TEST INFRASTRUCTURE ONLY (see oracle/wrk_oracle.cpp).  The op order, buffer dtypes (Bundle<f16>)
and load-time transforms follow src/runtime/v4.rs:630-829, v5.rs:656-920, v6.rs:701-992, v7.rs:716-1036 and
src/runtime/loader.rs; every tensor the reference stores as fp16 is an fp16 numpy array here, so
every rounding point of the reference is a rounding point of this oracle.  The reference has no
model-level test: end-to-end logits parity is unpinned beyond this restatement.
"""
import numpy as np

from . import oracle as o

LN_EPS, GN_EPS, L2_EPS = 1.0e-5, 64.0e-5, 1.0e-12
QUANT_NONE, QUANT_INT8, QUANT_NF4, QUANT_SF4 = 0, 1, 2, 3


class Mat:
    """`Matrix` of src/tensor/matrix.rs: (kind, packed weights, scales), rows of K contiguous elements."""

    def __init__(self, w_f16, quant, fast=False):
        w = np.ascontiguousarray(w_f16, dtype=np.float16)
        self.shape = w.shape  # (..., M, K)
        self.table = o.NF4_TABLE
        if quant == QUANT_INT8:
            self.kind = o.MAT_INT8
            self.w, self.scale = o.quantize_mat_int8(w, fast=fast)
        elif quant in (QUANT_NF4, QUANT_SF4):
            # Quant::SF4 is the Fp4 matrix with the Student-t code book, nu = 5 (src/runtime/model.rs:133-134)
            self.kind = o.MAT_NF4
            self.table = o.NF4_TABLE if quant == QUANT_NF4 else o.sf4_table(5.0)
            self.w, self.scale = o.quantize_mat_nf4(w, table=self.table, fast=fast)
        else:
            self.kind, self.w, self.scale = o.MAT_FP16, w, None

    def matmul(self, x, out, act=o.ACT_NONE, turbo=False, fast=False):
        o.matmul(self.kind, self.w, self.scale, x, out, act=act, mode=1 if turbo else 0, table=self.table, fast=fast)


class OracleModel:
    def __init__(self, tensors, quant=None, rescale=None, fast=False):
        """tensors: {name: fp16 array}; quant: {layer: QUANT_*}."""
        t = tensors
        self.fast = fast
        quant = quant or {}
        names = set(t)
        self.version = (7 if "blocks.0.att.x_r" in names else 6 if "blocks.0.att.time_mix_x" in names else
                        5 if "blocks.0.att.gate.weight" in names else 4)
        self.L = 1 + max(int(n.split(".")[1]) for n in names if n.startswith("blocks."))
        self.V, self.C = t["emb.weight"].shape
        self.F = t["blocks.0.ffn.key.weight"].shape[0]
        # Loader::info: v4 counts one head (src/runtime/loader.rs:290-294)
        self.H = 1 if self.version == 4 else (t["blocks.0.att.r_k"] if self.version == 7 else t["blocks.0.att.time_first"]).shape[0]
        self.S = self.C // self.H
        self.rescale = rescale if rescale is not None else (1024 if self.version == 7 else 6)
        f16 = lambda n: np.ascontiguousarray(t[n], dtype=np.float16).reshape(-1)
        self.emb = np.ascontiguousarray(t["emb.weight"], dtype=np.float16)
        self.ln0 = (f16("blocks.0.ln0.weight"), f16("blocks.0.ln0.bias"))
        self.ln_out = (f16("ln_out.weight"), f16("ln_out.bias"))
        self.head = Mat(t["head.weight"], QUANT_NONE)
        self.layers = []
        for i in range(self.L):
            q = quant.get(i, QUANT_NONE)
            discount = np.float32(2.0) ** np.float32(-(i // self.rescale))
            att, ffn, blk = f"blocks.{i}.att", f"blocks.{i}.ffn", f"blocks.{i}"
            mat = lambda n, d=None: Mat(t[n] if d is None else o.discount_f16(t[n], d), q, fast)
            L = {
                "ln1": (f16(f"{blk}.ln1.weight"), f16(f"{blk}.ln1.bias")),
                "ln2": (f16(f"{blk}.ln2.weight"), f16(f"{blk}.ln2.bias")),
                "gn": None if self.version == 4 else
                      (f16(f"{att}.ln_x.weight").reshape(self.H, self.S), f16(f"{att}.ln_x.bias").reshape(self.H, self.S)),
                "w_k": mat(f"{att}.key.weight"), "w_v": mat(f"{att}.value.weight"),
                "w_r": mat(f"{att}.receptance.weight"),
                "w_o": mat(f"{att}.output.weight", discount if discount != 1 else None),
                "ffn_k": mat(f"{ffn}.key.weight"),
                "ffn_v": mat(f"{ffn}.value.weight", discount if discount != 1 else None),
            }
            if self.version in (5, 6):
                L["w_g"] = mat(f"{att}.gate.weight")
                L["ffn_r"] = mat(f"{ffn}.receptance.weight")
                L["time_first"] = f16(f"{att}.time_first").astype(np.float32)
                L["ffn_mix_k"], L["ffn_mix_r"] = f16(f"{ffn}.time_mix_k"), f16(f"{ffn}.time_mix_r")
            if self.version == 4:
                L["ffn_r"] = mat(f"{ffn}.receptance.weight")
                L["time_first"] = f16(f"{att}.time_first").astype(np.float32)
                td = f16(f"{att}.time_decay").astype(np.float32)
                o.activate(td, o.ACT_OPPOSITE_EXP)  # load_vector_exp_f32: -exp(x), src/runtime/loader.rs:431-470
                L["time_decay"] = td
                for n in "kvr":
                    L[f"mix_{n}"] = f16(f"{att}.time_mix_{n}")
                L["ffn_mix_k"], L["ffn_mix_r"] = f16(f"{ffn}.time_mix_k"), f16(f"{ffn}.time_mix_r")
            if self.version == 5:
                td = f16(f"{att}.time_decay").astype(np.float32)
                o.activate(td, o.ACT_STABLE_EXP)  # load_vector_exp_exp_f32
                L["time_decay"] = td
                for n in "kvrg":
                    L[f"mix_{n}"] = f16(f"{att}.time_mix_{n}")
            if self.version == 6:
                L["time_decay"] = f16(f"{att}.time_decay")
                L["mix_x"] = f16(f"{att}.time_mix_x")
                L["mix"] = np.stack([f16(f"{att}.time_mix_{n}") for n in "wkvrg"]).reshape(5, 1, self.C)
                for n in ("time_decay_w1", "time_decay_w2", "time_mix_w1", "time_mix_w2"):
                    L[n] = Mat(t[f"{att}.{n}"], QUANT_NONE)
            if self.version == 7:
                for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g", "w0", "a0", "k_k", "k_a"):
                    L[n] = f16(f"{att}.{n}")
                L["r_k"] = f16(f"{att}.r_k").reshape(self.H, self.S)
                L["ffn_x_k"] = f16(f"{ffn}.x_k")
                for n in ("w1", "w2", "a1", "a2", "g1", "g2"):
                    L[n] = Mat(t[f"{att}.{n}"], QUANT_NONE)
                if i > 0:
                    L["v0"] = f16(f"{att}.v0")
                    L["v1"], L["v2"] = Mat(t[f"{att}.v1"], QUANT_NONE), Mat(t[f"{att}.v2"], QUANT_NONE)
            self.layers.append(L)

    def init_state(self, num_batch):
        """per layer f32 (B, S + 2, C), zeros (State::init); v4: (B, 5, C) with the running-maximum row at f32::MIN
        (src/runtime/v4.rs:163-180)."""
        if self.version == 4:
            st = [np.zeros((num_batch, 5, self.C), dtype=np.float32) for _ in range(self.L)]
            for s in st:
                s[:, 3, :] = np.finfo(np.float32).min
            return st
        return [np.zeros((num_batch, self.S + 2, self.C), dtype=np.float32) for _ in range(self.L)]

    # -------------------------------------------------------------------------------------
    def run(self, state, chunk, info, wide=True):
        """One job.  chunk: per batch a token list; info: [(len, option)] (0 Last, 1 Full, 2 None).
        Returns per batch an array (rows, vocab) of logits, and updates `state` in place."""
        fast = self.fast
        C, S, H = self.C, self.S, self.H
        lens = [l for l, _ in info]
        T = sum(lens)
        if T == 0:
            return [np.zeros((0, self.V), dtype=np.float32) for _ in info]
        tokens = [tok for b, l in zip(chunk, lens) for tok in b[:l]]
        cur, p = [], 0
        for b, l in enumerate(lens):
            cur.append((b, p, l))
            p += l
        cursors = o.pack_cursors(cur, wide=wide)
        turbo = T % 32 == 0
        f16z = lambda *s: np.zeros(s, dtype=np.float16)
        f32z = lambda *s: np.zeros(s, dtype=np.float32)

        inp = self.emb[np.asarray(tokens)].copy()  # (T, C) f16, CPU gather as in RnnJob::load
        o.layer_norm(*self.ln0, inp, LN_EPS, fast=fast)
        x = inp.copy()
        for i, L in enumerate(self.layers):
            st = state[i]
            st_att, st_ffn = o.View(st, y=(0, S + 1)), o.View(st, y=(S + 1, S + 2))
            if self.version == 4:
                st_att, st_ffn = o.View(st, y=(0, 4)), o.View(st, y=(4, 5))
            att_x = x.copy()
            o.layer_norm(*L["ln1"], att_x, LN_EPS, fast=fast)
            if self.version == 4:
                self._att_v4(L, st_att, cursors, att_x, T, turbo)
            elif self.version == 7:
                self._att_v7(i, L, st_att, cursors, att_x, T, turbo)
            else:
                self._att_v56(L, st_att, cursors, att_x, T, turbo)
            att_o = f16z(T, C)
            L["w_o"].matmul(att_x, att_o, turbo=turbo, fast=fast)
            o.binary(False, att_o, x)

            ffn_x = x.copy()
            o.layer_norm(*L["ln2"], ffn_x, LN_EPS, fast=fast)
            ffn_k, ffn_v = f16z(T, self.F), f16z(T, C)
            if self.version == 7:
                ffn_kx = f16z(1, T, C)
                o.token_shift(cursors, L["ffn_x_k"], st_ffn, ffn_x, ffn_kx, True)
                L["ffn_k"].matmul(ffn_kx[0], ffn_k, act=o.ACT_SQUARED_RELU, turbo=turbo, fast=fast)
                L["ffn_v"].matmul(ffn_k, ffn_v, turbo=turbo, fast=fast)
                o.channel_mix(cursors, st_ffn, None, ffn_v, ffn_x, v7=True)
            else:
                rev = self.version == 6  # v4 and v5 mix in the other direction
                ffn_kx, ffn_rx, ffn_r = f16z(1, T, C), f16z(1, T, C), f16z(T, C)
                o.token_shift(cursors, L["ffn_mix_k"], st_ffn, ffn_x, ffn_kx, rev)
                o.token_shift(cursors, L["ffn_mix_r"], st_ffn, ffn_x, ffn_rx, rev)
                L["ffn_k"].matmul(ffn_kx[0], ffn_k, act=o.ACT_SQUARED_RELU, turbo=turbo, fast=fast)
                L["ffn_v"].matmul(ffn_k, ffn_v, turbo=turbo, fast=fast)
                L["ffn_r"].matmul(ffn_rx[0], ffn_r, turbo=turbo, fast=fast)
                o.channel_mix(cursors, st_ffn, ffn_r, ffn_v, ffn_x)
            o.binary(False, ffn_x, x)
            if (i + 1) % self.rescale == 0:
                o.affine(x, 0.5, 0.0)

        # header: rows that need logits (RnnInfo::redirect), layer norm, fp16 head
        headers, outs, p_in, p_out = [], [], 0, 0
        for l, opt in info:
            if opt == 1:
                headers += list(range(p_in, p_in + l))
                outs.append((p_out, p_out + l))
                p_out += l
            elif opt == 0 and l > 0:
                headers.append(p_in + l - 1)
                outs.append((p_out, p_out + 1))
                p_out += 1
            else:
                outs.append((p_out, p_out))
            p_in += l
        nh = len(headers)
        if nh == 0:
            return [np.zeros((0, self.V), dtype=np.float32) for _ in info]
        head_x = np.ascontiguousarray(x[headers])
        o.layer_norm(*self.ln_out, head_x, LN_EPS, fast=fast)
        logits = f32z(nh, self.V)
        self.head.matmul(head_x, logits, turbo=nh % 32 == 0, fast=fast)
        return [logits[a:b] for a, b in outs]

    # -------------------------------------------------------------------------------------
    def _att_v4(self, L, st_att, cursors, att_x, T, turbo):
        """src/runtime/v4.rs:652-730.  att_x: LN'd input (T, C) f16; on return holds the WKV output (receptance applied)."""
        fast, C = self.fast, self.C
        f16z = lambda *s: np.zeros(s, dtype=np.float16)
        kx, vx, rx = f16z(1, T, C), f16z(1, T, C), f16z(1, T, C)
        o.token_shift(cursors, L["mix_k"], st_att, att_x, kx, False)
        o.token_shift(cursors, L["mix_v"], st_att, att_x, vx, False)
        o.token_shift(cursors, L["mix_r"], st_att, att_x, rx, False)
        f32z = lambda *s: np.zeros(s, dtype=np.float32)
        att_k, att_v, att_r = f32z(T, C), f32z(T, C), f32z(T, C)  # f32 buffers (src/runtime/v4.rs:234-256)
        L["w_k"].matmul(kx[0], att_k, turbo=turbo, fast=fast)
        L["w_v"].matmul(vx[0], att_v, turbo=turbo, fast=fast)
        L["w_r"].matmul(rx[0], att_r, turbo=turbo, fast=fast)
        aux = att_x.astype(np.float32)  # blit att_x -> aux_x (f32)
        o.time_mix_v4(cursors, L["time_decay"], L["time_first"], st_att, att_k, att_v, att_r, aux, fast=fast)
        att_x[...] = aux.astype(np.float16)  # blit aux_x -> att_x

    def _att_v56(self, L, st_att, cursors, att_x, T, turbo):
        """att_x: LN'd input (T, C) f16; on return holds the gated group-normed WKV output."""
        fast, C, S, H = self.fast, self.C, self.S, self.H
        f16z = lambda *s: np.zeros(s, dtype=np.float16)
        f32z = lambda *s: np.zeros(s, dtype=np.float32)
        att_k, att_v, att_r, att_g = f32z(T, C), f32z(T, C), f32z(T, C), f16z(T, C)
        if self.version == 6:
            att_xx = f16z(1, T, C)
            o.token_shift(cursors, L["mix_x"], st_att, att_x, att_xx, True)
            tmx = f16z(T, L["time_mix_w1"].shape[0])
            L["time_mix_w1"].matmul(att_xx[0], tmx, act=o.ACT_TANH, turbo=turbo, fast=fast)
            d = tmx.shape[1] // 5
            tmt = np.ascontiguousarray(tmx.reshape(T, 5, d).transpose(1, 0, 2))  # transpose [d,5,T] → [d,T,5]
            tm = f16z(5, T, C)
            L["time_mix_w2"].matmul(tmt, tm, turbo=turbo, fast=fast)
            o.binary(False, L["mix"], tm)
            att_sx = f16z(5, T, C)
            o.token_shift(cursors, tm, st_att, att_x, att_sx, True)
            L["w_k"].matmul(att_sx[1], att_k, turbo=turbo, fast=fast)
            L["w_v"].matmul(att_sx[2], att_v, turbo=turbo, fast=fast)
            L["w_r"].matmul(att_sx[3], att_r, turbo=turbo, fast=fast)
            L["w_g"].matmul(att_sx[4], att_g, turbo=turbo, fast=fast)
            att_w = f16z(T, L["time_decay_w1"].shape[0])
            L["time_decay_w1"].matmul(att_sx[0], att_w, act=o.ACT_TANH, turbo=turbo, fast=fast)
            td = f32z(T, C)
            L["time_decay_w2"].matmul(att_w, td, turbo=turbo, fast=fast)
            o.binary(False, L["time_decay"], td)
            o.activate(td, o.ACT_STABLE_EXP)
        else:
            sx = {}
            for n in "kvrg":
                sx[n] = f16z(1, T, C)
                o.token_shift(cursors, L[f"mix_{n}"], st_att, att_x, sx[n], False)
            L["w_k"].matmul(sx["k"][0], att_k, turbo=turbo, fast=fast)
            L["w_v"].matmul(sx["v"][0], att_v, turbo=turbo, fast=fast)
            L["w_r"].matmul(sx["r"][0], att_r, turbo=turbo, fast=fast)
            L["w_g"].matmul(sx["g"][0], att_g, turbo=turbo, fast=fast)
            td = L["time_decay"]
        aux_x = att_x.astype(np.float32)  # blit f16 → f32
        o.time_mix_v56(self.version == 6, cursors, td, L["time_first"], st_att, att_k, att_v, att_r, aux_x, S, H,
                       fast=fast)
        aux_x = aux_x.reshape(T, H, S)
        o.group_norm(*L["gn"], aux_x, GN_EPS, H, fast=fast)
        att_x[...] = aux_x.reshape(T, C).astype(np.float16)  # blit f32 → f16
        o.binary(True, att_g, att_x, act_x=o.ACT_SILU)

    def _att_v7(self, index, L, st_att, cursors, att_x, T, turbo):
        fast, C, S, H = self.fast, self.C, self.S, self.H
        f16z = lambda *s: np.zeros(s, dtype=np.float16)
        sx = {}
        for n in "rwkvag":
            sx[n] = f16z(1, T, C)
            o.token_shift(cursors, L[f"x_{n}"], st_att, att_x, sx[n], True)
        att_r, att_k, att_v = f16z(T, C), f16z(T, C), f16z(T, C)
        L["w_r"].matmul(sx["r"][0], att_r, turbo=turbo, fast=fast)
        L["w_k"].matmul(sx["k"][0], att_k, turbo=turbo, fast=fast)
        L["w_v"].matmul(sx["v"][0], att_v, turbo=turbo, fast=fast)
        aux_w, att_w = f16z(T, L["w1"].shape[0]), f16z(T, C)
        L["w1"].matmul(sx["w"][0], aux_w, act=o.ACT_TANH, turbo=turbo, fast=fast)
        L["w2"].matmul(aux_w, att_w, turbo=turbo, fast=fast)
        o.binary(False, L["w0"], att_w)
        aux_a, att_a = f16z(T, L["a1"].shape[0]), f16z(T, C)
        L["a1"].matmul(sx["a"][0], aux_a, turbo=turbo, fast=fast)
        L["a2"].matmul(aux_a, att_a, turbo=turbo, fast=fast)
        o.binary(False, L["a0"], att_a, act_out=o.ACT_SIGMOID)
        aux_g, att_g = f16z(T, L["g1"].shape[0]), f16z(T, C)
        L["g1"].matmul(sx["g"][0], aux_g, act=o.ACT_SIGMOID, turbo=turbo, fast=fast)
        L["g2"].matmul(aux_g, att_g, turbo=turbo, fast=fast)
        att_kk = att_k.copy()
        o.binary(True, L["k_k"], att_kk)
        att_kk = att_kk.reshape(T, H, S)
        o.l2_norm(att_kk, L2_EPS, fast=fast)
        att_kk = att_kk.reshape(T, C)
        o.control_k_v7(L["k_a"], att_a, att_k)
        if index == 0:
            self._v0 = att_v.copy()
        else:
            aux_v, att_vv = f16z(T, L["v1"].shape[0]), f16z(T, C)
            L["v1"].matmul(sx["v"][0], aux_v, turbo=turbo, fast=fast)
            L["v2"].matmul(aux_v, att_vv, turbo=turbo, fast=fast)
            o.binary(False, L["v0"], att_vv, act_out=o.ACT_SIGMOID)
            o.lerp(self._v0, att_v, att_vv, True)
        att_n = np.stack([att_k, att_v, att_a, att_kk])  # (4, T, C)
        o.time_mix_v7(cursors, st_att, att_r, att_w, att_n, att_x, S, H, fast=fast)
        ax = att_x.reshape(T, H, S)
        o.group_norm(*L["gn"], ax, GN_EPS, H, fast=fast)
        o.time_first_v7(L["r_k"], att_r, att_n, att_x, S, H, fast=fast)
        o.binary(True, att_g, att_x)
