"""Worker of the tensor-parallel tests: one process per rank (not collected by pytest).

mode "gpu": rank r builds its slice of the model on GPU r (wrk_model_builder_shard) and runs the sharded bundle
(wrk_bundle_create_sharded); rank 0 also runs the whole model on its GPU with the same tokens and compares logits,
packed bytes and state.
mode "watchdog": host-side failure detection: one gloo rank skips a collective, the other's wait times out.
mode "cpu": the sharding rules checked with the CPU oracle: every rank quantizes and multiplies only its
shard, partial sums meet in a gloo all-reduce, and the result must equal the unsharded oracle.
"""
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    mode = sys.argv[1]
    import torch
    import torch.distributed as dist

    import datetime
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    rank, world = dist.get_rank(), dist.get_world_size()
    say = lambda *a: print(f"[rank {rank}]", *a, flush=True)
    say("process group up")
    wrk = importlib.import_module("web-rwkv_b200")
    tp = importlib.import_module("web-rwkv_b200.tp")
    synth = importlib.import_module("web-rwkv_b200.synth")

    if mode == "cpu":
        from oracle import oracle as o
        rng = np.random.default_rng(7)  # same data on every rank
        for quant, kind, blk in ((wrk.QUANT_INT8, "int8", 128), (wrk.QUANT_NF4, "nf4", 64)):
            C, F, T = 512, 1280 if blk == 64 else 1792, 5  # F / blk = 20 resp. 14 units: uneven for 8 ranks, even for 2
            plan = tp.ShardPlan(C, F, 1024, world, quant)
            (c0, c1), (f0, f1) = plan.channels[rank], plan.ffn[rank]
            assert c0 % blk == 0 and f0 % blk == 0 and (c1 - c0) % blk == 0
            w_o = (rng.standard_normal((C, C)) * 0.05).astype(np.float16)   # K-sharded (columns)
            w_k = (rng.standard_normal((F, C)) * 0.05).astype(np.float16)   # row-sharded
            w_v = (rng.standard_normal((C, F)) * 0.05).astype(np.float16)   # K-sharded
            x = rng.standard_normal((T, C)).astype(np.float16)
            quantize = o.quantize_mat_int8 if kind == "int8" else o.quantize_mat_nf4
            mk = o.MAT_INT8 if kind == "int8" else o.MAT_NF4
            # packed bytes and scales of a shard are the slice of the unsharded quantization
            qf, sf = quantize(w_o)
            ql, sl = quantize(np.ascontiguousarray(w_o[:, c0:c1]))
            per = 1 if kind == "int8" else 2
            assert np.array_equal(ql, qf[:, c0 // per:c1 // per])
            assert np.array_equal(sl.reshape(C, -1), sf.reshape(C, -1)[:, (c0 // blk) * (2 if kind == "int8" else 1):(c1 // blk) * (2 if kind == "int8" else 1)])
            # attention output: partial sums over the rank's channels, all-reduced
            full = np.zeros((T, C), dtype=np.float32)
            o.matmul(mk, qf, sf, x, full)
            part = np.zeros((T, C), dtype=np.float32)
            o.matmul(mk, ql, sl, np.ascontiguousarray(x[:, c0:c1]), part)
            tpart = torch.from_numpy(part)
            dist.all_reduce(tpart)
            assert np.allclose(tpart.numpy(), full, rtol=1e-4, atol=1e-4), kind
            # ffn: row shard of key (squared relu is elementwise), K shard of value
            qk, sk = quantize(w_k)
            kfull = np.zeros((T, F), dtype=np.float16)
            o.matmul(mk, qk, sk, x, kfull, act=o.ACT_SQUARED_RELU)
            qkl, skl = quantize(np.ascontiguousarray(w_k[f0:f1]))
            kloc = np.zeros((T, f1 - f0), dtype=np.float16)
            o.matmul(mk, qkl, skl, x, kloc, act=o.ACT_SQUARED_RELU)
            assert np.array_equal(kloc, kfull[:, f0:f1])
            qv, sv = quantize(w_v)
            vfull = np.zeros((T, C), dtype=np.float32)
            o.matmul(mk, qv, sv, kfull, vfull)
            qvl, svl = quantize(np.ascontiguousarray(w_v[:, f0:f1]))
            vpart = np.zeros((T, C), dtype=np.float32)
            o.matmul(mk, qvl, svl, kloc, vpart)
            tv = torch.from_numpy(vpart)
            dist.all_reduce(tv)
            assert np.allclose(tv.numpy(), vfull, rtol=1e-4, atol=1e-3), kind
        dist.barrier()
        print("ok", rank, flush=True)
        return

    if mode == "watchdog":
        # Failure detection without a GPU fault: rank 1 never enters the second collective.  Rank 0 waits for it
        # through the library's watchdog loop (the loop under wrk_comm_wait), with the collective's completion as
        # `done`: the wait must end with WRK_ERR_TIMEOUT, not hang, and the rank must still be able to talk.
        import ctypes
        lib = wrk.lib()
        CB = ctypes.CFUNCTYPE(ctypes.c_int32, ctypes.c_void_p)
        t = torch.ones(4)
        work = dist.all_reduce(t, async_op=True)  # both ranks enter this one
        done = CB(lambda _: 1 if work.is_completed() else 0)
        assert lib.wrk_watchdog_wait(done, None, None, 20000, 200) == 0
        assert float(t[0]) == world
        if rank == 0:
            t2 = torch.ones(4)
            work2 = dist.all_reduce(t2, async_op=True)
            done2 = CB(lambda _: 1 if work2.is_completed() else 0)
            import time
            t0 = time.perf_counter()
            status = lib.wrk_watchdog_wait(done2, None, None, 1500, 200)
            waited = time.perf_counter() - t0
            assert status == wrk.ERR_TIMEOUT, status
            assert 1.4 <= waited < 10.0, waited
            assert b"did not finish within 1500 ms" in lib.wrk_last_error_message()
            # an asynchronous failure reported by the second question ends the wait at once
            failing = CB(lambda _: 7)
            assert lib.wrk_watchdog_wait(done2, failing, None, 20000, 200) == wrk.ERR_NCCL
            say("peer skipped a collective: the wait gave up after", round(waited, 2), "s")
        else:
            import time
            time.sleep(5.0)  # alive and connected, but never in the collective, while rank 0 waits
        # the skipped collective stays pending on rank 0: both ranks leave without another rendezvous
        print("ok", rank, flush=True)
        os._exit(0)

    # ---- gpu: every rank builds its slice in the C library and runs the same jobs; rank 0 also runs the whole
    # model on its GPU and compares ----
    rt = importlib.import_module("web-rwkv_b200.runtime")
    ctx = wrk.Context(rank)
    uid = [tp.Comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    say("unique id exchanged")
    comm = tp.Comm(ctx, uid[0], rank, world)
    say("communicator up")
    LAST, FULL = wrk.RNN_LAST, wrk.RNN_FULL
    for config, quant, block in (("v6-tiny", wrk.QUANT_INT8, 128), ("v7-tiny", wrk.QUANT_INT8, 128), ("v5-tiny", wrk.QUANT_NF4, 64),
                                 ("v7-tiny", wrk.QUANT_NONE, 1)):
        tensors = synth.make_model(config, 1000)
        L = synth.CONFIGS[config][2]
        qmap = {i: quant for i in range(L)}
        model = rt.ModelBuilder(ctx).shard(rank, world, 64, block).add_tensors(tensors).quant(qmap).build()
        bundle = rt.Bundle(model, 3, comm)
        rng = np.random.default_rng(5)
        V = tensors["emb.weight"].shape[0]
        prompts = [rng.integers(0, V - 1, 37).tolist(), rng.integers(0, V - 1, 3).tolist(), []]
        options = [LAST, FULL, LAST]
        steps = [[[int(rng.integers(0, V - 1))] for _ in range(3)] for _ in range(3)]

        def drive(b):
            """Chunked prefill of three sequences (one empty), then three decode steps of three tokens."""
            inp = rt.RnnInput(list(zip(prompts, options)), 32)
            outs = []
            while inp.num_token():
                outs.append([o.copy() for o in b.infer(inp)])
            for s in steps:
                for bi in range(3):
                    inp.append(bi, s[bi])
                while inp.num_token():
                    outs.append([o.copy() for o in b.infer(inp)])
            return outs

        got = drive(bundle)
        comm.wait(20000)
        assert ctx.device_status() == 0
        # the same jobs with the partial sums through NCCL instead of peer memory
        say(config, "peer reduce", bundle.peer_reduce())
        if bundle.peer_reduce():
            nccl_bundle = rt.Bundle(model, 3, comm)
            nccl_bundle.set_peer_reduce(0)
            got_nccl = drive(nccl_bundle)
            comm.wait(20000)
            for g, w in zip(got, got_nccl):
                for bi in range(3):
                    assert g[bi].shape == w[bi].shape
                    if w[bi].size:
                        err = float(np.max(np.abs(g[bi] - w[bi]) / np.maximum(1.0, np.abs(w[bi]))))
                        assert err <= 2e-2, (config, "peer vs nccl", err)
            del nccl_bundle
            if rank == 0:
                print("peer reduce matches nccl", config, flush=True)
        # packed bytes of a rank's slice are the slice of the whole model's packing
        if rank == 0:
            whole = rt.ModelBuilder(ctx).add_tensors(tensors).quant(qmap).build()
            ref = rt.Bundle(whole, 3)
            ref.set_fused(0)
            want = drive(ref)
            assert len(got) == len(want)
            worst = 0.0
            for j, (g, w) in enumerate(zip(got, want)):
                for bi in range(3):
                    assert g[bi].shape == w[bi].shape, (config, j, bi, g[bi].shape, w[bi].shape)
                    if not w[bi].size:
                        continue
                    err = float(np.max(np.abs(g[bi] - w[bi]) / np.maximum(1.0, np.abs(w[bi]))))
                    cos = float(np.dot(g[bi].ravel(), w[bi].ravel()) / (np.linalg.norm(g[bi]) * np.linalg.norm(w[bi])))
                    worst = max(worst, err)
                    assert err <= 2e-2 and cos >= 0.9995, (config, j, bi, err, cos)
            plan = tp.ShardPlan(synth.CONFIGS[config][1], synth.CONFIGS[config][3], V, world, quant)
            (c0, c1), (f0, f1) = plan.channels[0], plan.ffn[0]
            kind, w_l, m_l, _ = model.matrix_parts(1, "att.w_k")
            _, w_f, m_f, _ = whole.matrix_parts(1, "att.w_k")
            assert np.array_equal(w_l[0, 0], w_f[0, 0, c0:c1]), config  # arrays are (w, z, rows, columns)
            kind, w_l, _, _ = model.matrix_parts(1, "ffn.w_v")
            _, w_f, _, _ = whole.matrix_parts(1, "ffn.w_v")
            per = 2 if kind == 2 else 1
            assert np.array_equal(w_l[0, 0], w_f[0, 0, :, f0 // per:f1 // per]), config
            # the state a rank holds: its own heads' rows, and the shift rows of every channel
            sl, sw = bundle.state_back(0), ref.state_back(0)
            assert np.allclose(sl[:, 0], sw[:, 0], atol=2e-2) and np.allclose(sl[:, -1], sw[:, -1], atol=2e-2), config
            scale = max(1.0, float(np.abs(sw).max()))
            assert np.max(np.abs(sl[:, 1:-1, c0:c1] - sw[:, 1:-1, c0:c1])) <= 2e-2 * scale, config
            say(config, "sharded logits match the whole model, worst max-abs", worst)
            del ref, whole
        del bundle, model
    if rank == 0:
        print("tp logits match the single-GPU runtime", flush=True)
    dist.barrier()
    print("ok", rank, flush=True)
    # orderly teardown: bundles and models before the communicator, the communicator before the context
    import gc
    gc.collect()
    del comm
    gc.collect()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
