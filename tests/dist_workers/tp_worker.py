"""Tensor-parallel worker (one process per rank).  ``--device cpu`` runs on gloo ranks, ``--device cuda`` on NCCL.

Checks, on every rank:
  1. (cuda) the peer-memory all-reduce against ``dist.all_reduce``;
  2. (cuda) the row-parallel GEMV fused with its all-reduce against the unsharded matmul;
  3. ``auto_tp`` + conversion of a tiny Llama: logits equal to the single-process low-bit model of the same
     checkpoint, identical on all ranks; (cuda) greedy decode through the graph engine agrees across ranks;
  4. (cuda) the whole-step decode kernel with the all-reduce inside against the per-kernel path.
Exit code 0 = all passed.
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--model-dir", required=True)
    args = ap.parse_args()
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    cuda = args.device == "cuda"
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        dev = torch.device("cuda", torch.cuda.current_device())
    else:
        dist.init_process_group("gloo")
        dev = torch.device("cpu")

    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.parallel.tp import TPGroup

    tp = TPGroup()
    assert tp.world_size == world and tp.rank == rank

    if cuda:
        from ipex_llm_b200.ops import cuda_ops
        from ipex_llm_b200.ops.cuda_quant import quantize_to_device_layout
        from ipex_llm_b200.quant import qtypes as qt
        comm = tp.symm()
        # 1. stand-alone all-reduce
        for dtype in (torch.float16, torch.bfloat16, torch.float32):
            for n in (8, 8192, 100003, 1 << 20):
                torch.manual_seed(100 + rank)
                t = torch.randn(n, device=dev).to(dtype)
                ref = t.clone().float()
                dist.all_reduce(ref)
                out = comm.all_reduce(t.clone())
                tol = 1e-5 if dtype == torch.float32 else 3e-2
                assert (out.float() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item()), (dtype, n)
        # 1b. staged all-reduce with the row-parallel epilogue (+ residual + per-column bias) in the same kernel
        for dtype in (torch.float16, torch.bfloat16):
            for rows, cols in ((1, 4096), (3, 1000)):
                torch.manual_seed(200 + rank)
                part = torch.randn(rows, cols, device=dev).to(dtype)
                torch.manual_seed(300)
                res = torch.randn(rows, cols, device=dev).to(dtype)
                bias = torch.randn(cols, device=dev).to(dtype)
                ref = part.clone().float()
                dist.all_reduce(ref)
                ref = ref + res.float() + bias.float()
                for _ in range(2):
                    stage, token = comm.ar_stage(rows * cols, dtype)
                    stage.view(rows, cols).copy_(part)
                    out = res.clone()
                    comm.all_reduce_staged(token, out, residual=out, bias=bias)
                torch.cuda.synchronize()
                assert (out.float() - ref).abs().max().item() <= 3e-2 * max(1.0, ref.abs().max().item()), (dtype, rows)
        # 2. fused row-parallel GEMV + all-reduce, every tiled family
        torch.manual_seed(7)
        N, K, M = 1024, 512 * world, 3
        w = torch.randn(N, K, device=dev) * 0.05
        x = torch.randn(M, K, device=dev).half()
        res = torch.randn(M, N, device=dev).half()
        ks = K // world
        for name in ("sym_int4", "asym_int4", "nf4", "fp8_e4m3", "sym_int8"):
            q = qt.qtype_from_name(name)
            w_r = w[:, rank * ks:(rank + 1) * ks].contiguous()
            packed = quantize_to_device_layout(w_r.half(), q)
            deq = cuda_ops.dequantize_device(packed, (N, ks), q, torch.float32)
            part = x[:, rank * ks:(rank + 1) * ks].float() @ deq.t()
            dist.all_reduce(part)
            ref = part + res.float()
            out = torch.empty(M, N, device=dev, dtype=torch.float16)
            for _ in range(3):   # repeated calls exercise the parity alternation and the self-cleaning counters
                cuda_ops.gemv_lowbit_ar(x[:, rank * ks:(rank + 1) * ks].contiguous(), packed, q, N, ks, out, comm,
                                        residual=res)
            torch.cuda.synchronize()
            err = (out.float() - ref).abs().max().item() / ref.abs().max().item()
            assert err < 5e-3, (name, err)
        cuda_ops.check_error_flag(dev)
        # 2b. row-parallel GEMM (prompt sized) with the all-reduce fused into the tcgen05 epilogue
        from ipex_llm_b200.ops import tcgen05_gemm
        for Mtok, Nout in ((70, 384), (300, 1024)):
            xg = torch.randn(Mtok, K, device=dev).half()
            rg = torch.randn(Mtok, Nout, device=dev).half()
            bg = torch.randn(Nout, device=dev).half()
            wg = torch.randn(Nout, K, device=dev) * 0.05
            for name in ("sym_int4", "fp8_e4m3"):
                q = qt.qtype_from_name(name)
                w_r = wg[:, rank * ks:(rank + 1) * ks].contiguous()
                packed = quantize_to_device_layout(w_r.half(), q)
                deq = cuda_ops.dequantize_device(packed, (Nout, ks), q, torch.float32)
                part = xg[:, rank * ks:(rank + 1) * ks].float() @ deq.t()
                dist.all_reduce(part)
                ref = part + rg.float() + bg.float()
                for _ in range(3):     # both staging parities and the self-cleaning counters
                    out = tcgen05_gemm.gemm_lowbit_ar(xg[:, rank * ks:(rank + 1) * ks].contiguous(), packed, q, Nout,
                                                      ks, comm, bias=bg, residual=rg)
                torch.cuda.synchronize()
                err = (out.float() - ref).abs().max().item() / ref.abs().max().item()
                assert err < 1e-2, ("gemm_ar", name, Mtok, err)
        cuda_ops.check_error_flag(dev)
        # 2c. column-parallel GEMM with the all-gather of its activation fused in front (each rank owns a slice of
        #     the token rows and its own output columns)
        if hasattr(cuda_ops.cuda_lib(), "ipex_gemm_lowbit_tcgen05_ag"):
            for Mtot, Nout, act in ((70, 384, 0), (301, 1024, 0), (520, 512, 1)):
                torch.manual_seed(11)                      # same activation on every rank, sliced by rows
                xfull = torch.randn(Mtot, K, device=dev).half()
                rows = (Mtot + world - 1) // world
                x_loc = xfull[rank * rows:(rank + 1) * rows].contiguous()
                torch.manual_seed(50 + rank)               # rank-specific weights: its own output columns
                wcol = torch.randn(Nout, K, device=dev) * 0.05
                bcol = torch.randn(Nout, device=dev).half()
                for name in ("sym_int4", "fp8_e4m3"):
                    q = qt.qtype_from_name(name)
                    packed = quantize_to_device_layout(wcol.half(), q)
                    deq = cuda_ops.dequantize_device(packed, (Nout, K), q, torch.float32)
                    full = xfull.float() @ deq.t()
                    if act:
                        # gate / up alternate in 16-row tiles of the weight
                        t16 = full.view(Mtot, Nout // 32, 2, 16)
                        ref = (torch.nn.functional.silu(t16[:, :, 0]) * t16[:, :, 1]).reshape(Mtot, Nout // 2)
                    else:
                        ref = full + bcol.float()
                    for _ in range(3):
                        out = tcgen05_gemm.gemm_lowbit_ag(x_loc, packed, q, Nout, K, Mtot, comm,
                                                          bias=None if act else bcol, act=act)
                    torch.cuda.synchronize()
                    err = (out.float() - ref).abs().max().item() / ref.abs().max().item()
                    assert err < 1e-2, ("gemm_ag", name, Mtot, act, err)
            cuda_ops.check_error_flag(dev)

    # 3. tiny llama, tensor parallel
    torch.manual_seed(0)
    ids = torch.randint(0, 32000, (2, 24))
    dtype = torch.float16 if cuda else torch.float32
    full = AutoModelForCausalLM.from_pretrained(args.model_dir, load_in_low_bit="sym_int8", torch_dtype=dtype)
    shard = AutoModelForCausalLM.from_pretrained(args.model_dir, load_in_low_bit="sym_int8", torch_dtype=dtype,
                                                 tp_group=tp)
    if cuda:
        full, shard = full.to(dtype).to(dev), shard.to(dtype).to(dev)
    with torch.no_grad():
        a = full(ids.to(dev)).logits[:, -1].float()
        b = shard(ids.to(dev)).logits[:, -1].float()
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    assert cos > 0.999, cos
    gathered = [torch.empty_like(b) for _ in range(world)]
    dist.all_gather(gathered, b)
    for g in gathered:
        assert torch.allclose(g, gathered[0], atol=1e-3), "ranks disagree"
    out = shard.generate(ids.to(dev), max_new_tokens=6, do_sample=False)
    toks = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(toks, out)
    for t in toks:
        assert torch.equal(t, toks[0]), "ranks generated different tokens"
    # 3b. random-init models: with consistent_tp_shards the sharded model IS the whole model of the same seed
    # (every sharded matrix drawn whole, this rank keeps its rows / columns), and replicated parameters
    # (embeddings, norms) are the same on every rank with or without the switch
    from transformers import LlamaConfig
    cfg = LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=512, max_position_embeddings=128, tie_word_embeddings=False)
    ids_small = torch.randint(0, 512, (2, 16))
    whole = AutoModelForCausalLM.from_config(cfg, load_in_low_bit="sym_int8", device=str(dev), torch_dtype=dtype,
                                             seed=3)
    parts = AutoModelForCausalLM.from_config(cfg, load_in_low_bit="sym_int8", device=str(dev), torch_dtype=dtype,
                                             seed=3, tp_group=tp, consistent_tp_shards=True)
    with torch.no_grad():
        lw = whole(ids_small.to(dev)).logits[:, -1].float()
        lp = parts(ids_small.to(dev)).logits[:, -1].float()
    cos = torch.nn.functional.cosine_similarity(lw, lp, dim=-1).min().item()
    assert cos > 0.999, f"consistent shards do not reproduce the whole model: {cos}"
    loose = AutoModelForCausalLM.from_config(cfg, load_in_low_bit="sym_int8", device=str(dev), torch_dtype=dtype,
                                             seed=3, tp_group=tp)
    emb = loose.model.embed_tokens.weight.data.float()
    embs = [torch.empty_like(emb) for _ in range(world)]
    dist.all_gather(embs, emb)
    for e in embs:
        assert torch.equal(e, embs[0]), "replicated parameters differ between ranks"
    if cuda:
        assert getattr(shard, "_ipex_engine", None) is not None
        from ipex_llm_b200.ops import cuda_ops
        cuda_ops.check_error_flag(dev)
        # 4. whole-step decode kernel with the all-reduce inside (fp8 weights, grouped-query heads): logits and tokens
        #    against the per-kernel path of the same sharded model, identical on every rank
        from transformers import LlamaConfig
        from ipex_llm_b200.engine import get_engine
        from ipex_llm_b200.engine.mega import MegaStep
        for low_bit, dt in (("fp8_e4m3", torch.bfloat16), ("sym_int4", torch.float16)):
            cfg = LlamaConfig(hidden_size=1024, intermediate_size=2816, num_hidden_layers=3, num_attention_heads=16,
                              num_key_value_heads=2, vocab_size=32000, max_position_embeddings=1024,
                              tie_word_embeddings=False)
            m = AutoModelForCausalLM.from_config(cfg, load_in_low_bit=low_bit, device=str(dev), torch_dtype=dt,
                                                 seed=0, tp_group=tp)
            eng = get_engine(m, 2, 512)
            assert MegaStep.supported(eng) is None, MegaStep.supported(eng)
            g = torch.Generator(device="cpu").manual_seed(5)
            pids = torch.randint(0, 32000, (2, 90), generator=g).to(dev)
            recs = {}
            for mega in (False, True):
                lg = eng.prefill(pids)
                eng.tokens[:2] = lg.argmax(-1)
                eng._mega = None if mega else False
                eng._graphs = {}
                rec = []
                for _ in range(4):
                    eng.decode_step(2, use_graph=False)
                    rec.append((eng.gather_logits(2).float().clone(), eng.tokens[:2].clone()))
                torch.cuda.synchronize()
                cuda_ops.check_error_flag(dev)
                recs[mega] = rec
            assert eng._mega not in (None, False)
            l0, l1 = recs[False][0][0], recs[True][0][0]
            cos = torch.nn.functional.cosine_similarity(l0.flatten(), l1.flatten(), dim=0).item()
            assert cos > 0.999, (low_bit, cos)
            toks = torch.stack([t for _, t in recs[True]])
            allt = [torch.empty_like(toks) for _ in range(world)]
            dist.all_gather(allt, toks)
            for t in allt:
                assert torch.equal(t, allt[0]), "ranks chose different tokens in the fused step"
            lgs = recs[True][-1][0].contiguous()
            alll = [torch.empty_like(lgs) for _ in range(world)]
            dist.all_gather(alll, lgs)
            for t in alll:
                # replicated projections are summed in a timing-dependent order on each rank: equal up to rounding
                assert torch.allclose(t, alll[0], atol=0.06 if dt == torch.bfloat16 else 0.01), \
                    "ranks disagree on the fused step's logits"
            # graph replay of the fused step
            lg = eng.prefill(pids)
            eng.tokens[:2] = lg.argmax(-1)
            for i in range(4):
                eng.decode_step(2, use_graph=True)
                assert torch.equal(eng.tokens[:2], recs[True][i][1]), (low_bit, i)
            torch.cuda.synchronize()
            cuda_ops.check_error_flag(dev)
            if rank == 0:
                print(f"fused step, tensor parallel {world} ranks, {low_bit}: cos {cos:.6f}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: ok")


if __name__ == "__main__":
    main()
