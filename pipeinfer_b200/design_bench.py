"""`bench.py --design rapisun | fabivik | lulenex | putazen`: prefill and decode throughput of a layer-list design at sizes that resemble a real
model's layers (random weights drawn in the loader from a seed), beside the closest existing model of the library at equal width / depth /
vocabulary -- for Rapisun the llama architecture in Q4_K (prompts on its tcgen05 GEMM, decoding on its tensor-core GEMVs), for Fabivik
the Rapisun design (the other layer-list model: same runtime, same dense matmuls), for Lulenex the Fabivik design (attention over cached
key / value heads and recurrences on the same kernels), for Putazen the Lulenex design (a state-space scan beside attention over cached
key / value heads, a dense feed-forward in every layer, a layer walked twice) -- plus the share and the roofline fraction of every kind of launch.  Everything goes through llama_decode on host batches; times are medians of CUDA-side
work as seen by the caller (llama_decode returns after the run's event), the per-kind numbers come from CUDA events around each
launch (llama_pib_profile_layer).  One JSON line on stdout."""
import ctypes as C
import json
import math
import os
import statistics
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def latent(heads, dim, rot, vdim, kv_rank, q_rank, window, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "mask": {"size": window},
         "rot": {"base": 500000.0, "dims": rot}, "scale": 1.0 / math.sqrt(dim + rot)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def design_config(width, vocab, blocks, heads, window, ff, experts, top, ff_e, ff_s, kv_rank, q_rank):
    """one block = [latent + dense, latent (cache of the first) + MoE, hgrn2 + MoE, hgrn2 + dense]"""
    dim = 128
    layers = []
    for b in range(blocks):
        base = 4 * b
        moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff_e}, "shared": {"ff": ff_s}}
        dense = {"kind": "dense", "ff": ff}
        h = {"heads": heads, "dim": dim, "vdim": dim}
        layers += [{"type": "latent_attention", "mixer": latent(heads, dim, 64, dim, kv_rank, q_rank, window), "mlp": dense},
                   {"type": "latent_attention", "mixer": latent(heads, dim, 64, dim, kv_rank, q_rank, window, kv_from=base), "mlp": moe},
                   {"type": "hgrn2", "mixer": h, "mlp": moe},
                   {"type": "hgrn2", "mixer": h, "mlp": dense}]
    return {"architecture": "Rapisun", "width": width, "vocab": vocab, "canon": {"taps": 4}, "norm": {"eps": 1e-5}, "layers": layers}


def fabivik_config(width, vocab, blocks, heads, window, experts, top, ff_e, ff_s, **_):
    """one block = [attention + MoE, delta rule + MoE, attention (values mixed with the first one's) + MoE, time mixing + MoE]"""
    dim = 128
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff_e, "limit": 7.0}, "shared": {"ff": ff_s, "limit": 7.0}}
    att = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": dim, "vdim": dim, "conv": 4, "mask": {"size": window}, "scale": 1.0 / math.sqrt(dim), "v_mix": True}
    dlt = {"heads": heads, "kv_heads": max(1, heads // 2), "dim": dim, "vdim": dim, "conv": 4}
    wkv = {"heads": width // 64, "dim": 64, "decay_rank": 64}
    layers = []
    for _ in range(blocks):
        layers += [{"type": "attention", "mixer": att, "mlp": moe}, {"type": "delta", "mixer": dlt, "mlp": moe},
                   {"type": "attention", "mixer": att, "mlp": moe}, {"type": "wkv", "mixer": wkv, "mlp": moe}]
    return {"architecture": "Fabivik", "width": width, "vocab": vocab, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0}, "logit_scale": 0.5, "layers": layers}


def lulenex_config(width, vocab, blocks, heads, window, ff, **_):
    """4 * blocks layer runs: [state-space scan, two-branch, two-branch, two-branch] per block without the last layer, the second layer walked twice;
    every layer with a dense feed-forward"""
    ssm = {"inner": 2 * width, "state": 16, "dt_rank": width // 16, "conv": 4}
    two = {"left": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "mask": {"size": window}, "rot": {"base": 500000.0, "dims": 64},
                    "scale": 1.0 / math.sqrt(128)},
           "right": {"heads": max(1, heads // 2), "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** (-5 - 3 * h / max(1, heads // 2)) for h in range(max(1, heads // 2))]},
           "left_scale": 0.7, "right_scale": 0.9}
    dense = {"kind": "dense", "ff": ff}
    layers = ([{"type": "mamba1", "mixer": ssm, "mlp": dense}] + [{"type": "parallel", "mixer": two, "mlp": dense}] * 3) * blocks
    return {"architecture": "Lulenex", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "layers": layers[:-1], "loop": {"start": 1, "stop": 2, "times": 2}}


def putazen_config(width, vocab, blocks, heads, ff, kv_rank, **_):
    """4 * blocks layer runs: [Mamba-2, differential attention, Mamba-2, latent attention] per block without the last layer, the second layer
    walked twice; four residual streams; every layer with a dense clamped gated feed-forward"""
    m2 = {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 1, "conv": 4, "norm_groups": 1}
    dif = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 64, "vdim": 128, "diff": 0.5, "scale": 1.0 / math.sqrt(64),
           "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}}
    lat = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": kv_rank, "rot": {"base": 500000.0, "dims": 64}, "scale": 1.0 / math.sqrt(192)}
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    layers = [{"type": t, "mixer": mx, "mlp": dense} for t, mx in (("mamba2", m2), ("attention", dif), ("mamba2", m2), ("latent_attention", lat))] * blocks
    return {"architecture": "Putazen", "width": width, "vocab": vocab, "streams": 4, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "layers": layers[:-1],
            "loop": {"start": 1, "stop": 2, "times": 2}}


# design -> (its name, its configuration, the comparator's key)
DESIGNS = {"rapisun": ("Rapisun", design_config, "llama_q4k"), "fabivik": ("Fabivik", fabivik_config, "rapisun"), "lulenex": ("Lulenex", lulenex_config, "fabivik"),
           "putazen": ("Putazen", putazen_config, "lulenex")}
COMPARATORS = {"llama_q4k": "llama architecture, Q4_K", "rapisun": "Rapisun (layer-list design of this library), same width / depth / vocabulary / experts",
               "fabivik": "Fabivik (layer-list design of this library), same width / layer runs / vocabulary",
               "lulenex": "Lulenex (layer-list design of this library), same width / layer runs / vocabulary / feed-forward width"}

SIZES = {
    # name: (design arguments, llama comparator (n_layer, n_embd, n_head, n_head_kv, n_ff, n_vocab))
    "w2048": (dict(width=2048, vocab=32000, blocks=2, heads=16, window=1024, ff=5632, experts=16, top=2, ff_e=1408, ff_s=2816, kv_rank=512, q_rank=768),
              (8, 2048, 16, 16, 5632, 32000)),
    "w4096": (dict(width=4096, vocab=32000, blocks=1, heads=32, window=2048, ff=11008, experts=8, top=2, ff_e=2816, ff_s=2816, kv_rank=512, q_rank=1536),
              (4, 4096, 32, 32, 11008, 32000)),
    "w1024": (dict(width=1024, vocab=16000, blocks=2, heads=8, window=512, ff=2816, experts=8, top=2, ff_e=704, ff_s=1408, kv_rank=256, q_rank=384),
              (8, 1024, 8, 8, 2816, 16000)),
}


def _median_ms(fn, reps, flush):
    out = []
    for _ in range(reps):
        flush()
        t0 = time.perf_counter()
        fn()
        out.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(out)


def _measure(ctx, lib, prompt_lens, n_decode, batch, vocab, flush, warmup, reps):
    """prefill of one sequence at each length, then single-token decoding of `batch` sequences behind a prompt"""
    res = {}
    toks = lambda n, s: [(7 + 31 * i + s) % vocab for i in range(n)]
    for T in prompt_lens:
        def go():
            lib.llama_kv_cache_clear(ctx.ctx)
            rc, _ = ctx_decode(ctx, toks(T, 0), list(range(T)), 0)
            assert rc == 0, lib.pib_last_error().decode()
        for _ in range(warmup):
            go()
        ms = _median_ms(go, reps, flush)
        res["prefill_%d" % T] = {"ms": ms, "tokens_per_s": T / ms * 1e3}
    for b in batch:
        lib.llama_kv_cache_clear(ctx.ctx)
        P = 256
        for s in range(b):
            rc, _ = ctx_decode(ctx, toks(P, s), list(range(P)), s)
            assert rc == 0, lib.pib_last_error().decode()
        times = []
        for i in range(warmup + n_decode):
            flush()
            t0 = time.perf_counter()
            rc = ctx_decode_multi(ctx, [(11 * i + s) % vocab for s in range(b)], [P + i] * b, list(range(b)))
            assert rc == 0, lib.pib_last_error().decode()
            if i >= warmup:
                times.append((time.perf_counter() - t0) * 1e3)
        ms = statistics.median(times)
        res["decode_b%d" % b] = {"ms_per_step": ms, "tokens_per_s": b / ms * 1e3}
    return res


def ctx_decode(ctx, tokens, pos, seq):
    from . import llama
    b, keep = llama.make_batch(tokens, pos, [[seq]] * len(tokens), ctx._bid, ctx.max_seq)
    ctx._bid += 1
    return ctx.L.llama_decode(ctx.ctx, b), None


def ctx_decode_multi(ctx, tokens, pos, seqs):
    from . import llama
    b, keep = llama.make_batch(tokens, pos, [[s] for s in seqs], ctx._bid, ctx.max_seq)
    ctx._bid += 1
    return ctx.L.llama_decode(ctx.ctx, b)


def _profile_design(ctx, lib, T, vocab, decode, peaks):
    """per-kind totals of one prefill of T tokens (decode=False) or of 16 decode steps behind it"""
    lib.llama_kv_cache_clear(ctx.ctx)
    toks = [(7 + 31 * i) % vocab for i in range(T)]
    if decode:
        ctx_decode(ctx, toks, list(range(T)), 0)
    lib.llama_pib_profile_layer(ctx.ctx, 0)
    n_runs = 1
    if decode:
        n_runs = 16
        for i in range(n_runs):
            ctx_decode(ctx, [(3 * i) % vocab], [T + i], 0)
    else:
        ctx_decode(ctx, toks, list(range(T)), 0)
    lib.llama_pib_profile_layer(ctx.ctx, -1)
    n = 1 << 16
    kind, ms, fl, by = (C.c_int32 * n)(), (C.c_float * n)(), (C.c_double * n)(), (C.c_double * n)()
    cnt = lib.llama_pib_hybrid_profile_read(ctx.ctx, kind, ms, fl, by, n)
    agg = {}
    for i in range(cnt):
        a = agg.setdefault(lib.llama_pib_hybrid_kind_name(kind[i]).decode(), [0, 0.0, 0.0, 0.0])
        a[0] += 1; a[1] += ms[i]; a[2] += fl[i]; a[3] += by[i]
    total = sum(a[1] for a in agg.values()) or 1.0
    out = {}
    for name, (launches, t, f, b) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        floor_ms = max(f / (peaks["tflops"] * 1e9), b / (peaks["gbs"] * 1e6))
        out[name] = {"launches": launches // n_runs, "ms": t / n_runs, "share": t / total, "tflops": f / t / 1e9 if t else 0.0, "gbs": b / t / 1e6 if t else 0.0,
                     "roofline_frac": floor_ms / t if t else 0.0, "bound": "tensor" if f / (peaks["tflops"] * 1e9) > b / (peaks["gbs"] * 1e6) else "hbm"}
    return {"total_ms": total / n_runs, "kinds": out}


def _profile_llama(ctx, lib, layer, T, vocab, peaks):
    """the comparator's per-launch events exist for single-chunk decodes: 64 decode steps behind a prompt"""
    KIND = {0: "qkv", 1: "attn_out", 2: "gate_up", 3: "down", 4: "lm_head", 5: "attn_norm_quant", 7: "rope_kv_attention", 8: "attn_out_quant", 9: "resid_ffn_norm_quant",
            10: "silu_mul_quant"}
    lib.llama_kv_cache_clear(ctx.ctx)
    ctx_decode(ctx, [(7 + 31 * i) % vocab for i in range(T)], list(range(T)), 0)
    lib.llama_pib_profile_layer(ctx.ctx, layer)
    for i in range(64):
        ctx_decode(ctx, [(3 * i) % vocab], [T + i], 0)
    lib.llama_pib_profile_layer(ctx.ctx, -1)
    n = 8192
    kind, bb, ms = (C.c_int32 * n)(), (C.c_int32 * n)(), (C.c_float * n)()
    cnt = lib.llama_pib_profile_read(ctx.ctx, kind, bb, ms, n)
    per = {}
    for i in range(cnt):
        per.setdefault(kind[i], []).append(ms[i])
    out = {}
    for k, lst in per.items():
        mean = sum(lst) / len(lst)
        e = {"launches_sampled": len(lst), "ms": mean}
        if k <= 4:
            N_, K_, byt = C.c_int64(), C.c_int64(), C.c_uint64()
            lib.llama_pib_matrix_shape(ctx.model, layer, k, C.byref(N_), C.byref(K_), C.byref(byt))
            alg = byt.value + 4.0 * (N_.value + K_.value)
            e.update(N=N_.value, K=K_.value, gbs=alg / mean / 1e6, roofline_frac=alg / mean / 1e6 / peaks["gbs"], bound="hbm")
        out[KIND.get(k, str(k))] = e
    return out


def run(args):
    from . import llama
    lib = llama.api()
    lib.llama_pib_profile_layer.argtypes = [C.c_void_p, C.c_int]
    lib.llama_pib_profile_read.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
    lib.llama_pib_matrix_shape.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_uint64)]
    lib.llama_pib_hybrid_profile_read.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
    lib.llama_pib_hybrid_kind_name.restype = C.c_char_p
    lib.llama_pib_hybrid_kind_name.argtypes = [C.c_int]
    peaks = {"gbs": 6650.0, "tflops": 1590.0, "source": "fallback"}
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        peaks = {"gbs": float(d["hbm_gbs"]), "tflops": float(d["bf16_tflops"]), "source": "measured (MEASURED_PEAKS.json)"}
    import torch                                            # only for the L2 flush between timed calls
    torch.cuda.set_device(0)
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def flush():
        scratch.zero_()
        torch.cuda.synchronize()

    key = args.design
    title, make_config, cmp_key = DESIGNS[key]
    out = {"design": title, "metric": "prefill / decode tokens per second, one GPU",
           "dtype": "bf16 operands, fp32 accumulation" + (" (comparator: Q4_K x Q8_K)" if cmp_key == "llama_q4k" else ""),
           "comparator": COMPARATORS[cmp_key],
           "data": "synthetic (random weights from a seed)", "peaks": peaks, "l2_policy": "256 MB written between timed calls", "sizes": {}}
    lens = [int(x) for x in args.design_prompt.split(",")]
    for name in args.design_size.split(","):
        dargs, cmp_shape = SIZES[name]
        cfg = make_config(**dargs)
        vocab = dargs["vocab"]
        n_ctx = max(lens) + 512
        t0 = time.time()
        ours = llama.Context(config=json.dumps(cfg), seed=1, n_ctx=4 * 320 + n_ctx, max_seq=8, state_slots=4)
        entry = {"config": dargs, "layers": len(cfg["layers"]), "load_s": round(time.time() - t0, 1)}
        entry[key] = _measure(ours, lib, lens, 32, [1, 4], vocab, flush, args.warmup, args.steps)
        entry[key + "_prefill_kinds"] = _profile_design(ours, lib, max(lens), vocab, False, peaks)
        entry[key + "_decode_kinds"] = _profile_design(ours, lib, 256, vocab, True, peaks)
        ours.close()
        if cmp_key != "llama_q4k":
            cmpc = llama.Context(config=json.dumps(DESIGNS[cmp_key][1](**dargs)), seed=1, n_ctx=4 * 320 + n_ctx, max_seq=8, state_slots=4)
            entry[cmp_key] = _measure(cmpc, lib, lens, 32, [1, 4], vocab, flush, args.warmup, args.steps)
            entry[cmp_key + "_prefill_kinds"] = _profile_design(cmpc, lib, max(lens), vocab, False, peaks)
            entry[cmp_key + "_decode_kinds"] = _profile_design(cmpc, lib, 256, vocab, True, peaks)
            cmpc.close()
        else:
            L, E, H, HKV, FF, V = cmp_shape
            cmpc = llama.Context(None, n_ctx=4 * 320 + n_ctx, max_seq=8, synthetic=(L, E, H, HKV, FF, V, 12, 1, 1, 1.0))
            entry["llama_q4k"] = _measure(cmpc, lib, lens, 32, [1, 4], vocab, flush, args.warmup, args.steps)
            entry["llama_q4k_decode_kinds"] = _profile_llama(cmpc, lib, L // 2, 256, vocab, peaks)
            cmpc.close()
        out["sizes"][name] = entry
    print(json.dumps(out))
    return 0
