"""Worker of the tensor-parallel tests: one process per rank (not collected by pytest).

mode "gpu": rank r drives GPU r through web-rwkv_b200/tp.py; rank 0 also runs the single-GPU runtime on the
same checkpoint and tokens and compares the logits.
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

    # ---- gpu ----
    rt = importlib.import_module("web-rwkv_b200.runtime")
    config, quant = "v6-tiny", wrk.QUANT_INT8
    tensors = synth.make_model(config, 1000)
    ctx = wrk.Context(rank)
    uid = [tp.Comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    say("unique id exchanged")
    comm = tp.Comm(ctx, uid[0], rank, world)
    say("communicator up")
    model = tp.TpModelV6(ctx, comm, tensors, quant=quant, num_batch=2)
    say("model sharded")
    rng = np.random.default_rng(5)
    V = tensors["emb.weight"].shape[0]
    steps = [[rng.integers(0, V - 1, 5).tolist(), rng.integers(0, V - 1, 3).tolist()]]      # prompt, two sequences
    steps += [[[int(rng.integers(0, V - 1))], [int(rng.integers(0, V - 1))]] for _ in range(3)]  # three decode steps
    outs = []
    for s in steps:
        outs.append(model.run(s))
        say("job done", [len(t) for t in s])
    assert ctx.device_status() == 0
    # the same jobs captured into CUDA graphs (collectives included) must give the same logits
    graphed = tp.TpModelV6(ctx, comm, tensors, quant=quant, num_batch=2, use_graph=True)
    for s, want in zip(steps, outs):
        got = graphed.run(s)
        for bi in want:
            assert np.allclose(got[bi], want[bi], rtol=1e-5, atol=1e-5), "graph-captured job differs"
    say("graph-captured jobs match")
    if rank == 0:
        b = rt.ModelBuilder(ctx)
        b.add_tensors(tensors)
        b.quant({i: quant for i in range(model.L)})
        ref_model = b.build()
        bundle = rt.Bundle(ref_model, 2)
        inp = rt.RnnInput([(steps[0][0], wrk.RNN_LAST), (steps[0][1], wrk.RNN_LAST)], 32)
        worst = 0.0
        for si, s in enumerate(steps):
            if si:
                inp.append(0, s[0])
                inp.append(1, s[1])
            ref = bundle.infer(inp)
            for bi in range(2):
                got, want = outs[si][bi], ref[bi][-1]
                err = float(np.max(np.abs(got - want) / np.maximum(1.0, np.abs(want))))
                cos = float(np.dot(got, want) / (np.linalg.norm(got) * np.linalg.norm(want)))
                worst = max(worst, err)
                assert err <= 2e-2 and cos >= 0.9995, (si, bi, err, cos)
        print("tp logits match the single-GPU runtime, worst max-abs", worst, flush=True)
    dist.barrier()
    print("ok", rank, flush=True)
    # orderly teardown: graphs and models before the communicator, the communicator before the context
    del graphed, model, outs
    import gc
    gc.collect()
    del comm
    gc.collect()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
