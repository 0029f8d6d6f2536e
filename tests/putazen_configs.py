"""Small Putazen configurations for the tests (sizes chosen to differ from each other: streams, heads, key / value heads, groups, states,
taps, norm parts, rotated dimensions with and without scaled frequencies, latent ranks, walks)."""
import math


def mamba2(heads, vdim, state, groups=1, conv=4, norm_groups=1):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def yarn(factor, original, fast=32.0, slow=1.0):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def diff_attn(heads, kv_heads, dim, vdim, rot_dims, diff=0.5, base=10000.0, scaling=None, scale=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = scaling
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "rot": rot, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}


def latent(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "rot": {"base": base, "dims": rot_dim},
            "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}


def dense(ff, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def model(width, vocab, streams, layers, loop=None, eps=1e-5, embed_scale=2.0):
    cfg = {"architecture": "Putazen", "width": width, "vocab": vocab, "streams": streams, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
           "layers": [{"type": t, "mixer": mx, "mlp": ml} for t, mx, ml in layers]}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def mixed_small():
    """all three mixers, three streams, a walked run in the middle, a layer without feed-forward"""
    return model(80, 190, 3, [("attention", diff_attn(4, 2, 12, 10, 8, diff=0.3, scaling=yarn(3.0, 48, fast=8.0)), dense(100)),
                              ("mamba2", mamba2(4, 10, 6, groups=2, conv=3, norm_groups=2), None),
                              ("latent_attention", latent(3, 10, 6, 14, 20, base=500.0), dense(72, limit=0.8)),
                              ("mamba2", mamba2(3, 12, 17, groups=3, conv=2, norm_groups=3), dense(64)),
                              ("attention", diff_attn(2, 2, 20, 8, 20, diff=0.7, base=300.0, scale=0.3), None)], loop=(1, 4, 2))


def mamba_only():
    return model(48, 100, 2, [("mamba2", mamba2(6, 8, 8, groups=3, conv=4, norm_groups=2), None), ("mamba2", mamba2(2, 25, 33, groups=1, conv=3, norm_groups=5), dense(40))])


def diff_only():
    """what the logits show is the differential attention: biases, partial rotation in halves, scaled frequencies, lambda, the head norm"""
    return model(64, 120, 2, [("attention", diff_attn(4, 2, 16, 12, 10, diff=0.4, base=100.0, scaling=yarn(4.0, 32, fast=6.0, slow=1.0), scale=0.5), None),
                              ("attention", diff_attn(3, 1, 12, 20, 12, diff=0.8, base=77.0), None)])


def latent_only():
    return model(56, 90, 5, [("latent_attention", latent(3, 12, 8, 10, 24, base=1000.0), None),
                             ("latent_attention", latent(2, 6, 2, 30, 7, scale=0.6), dense(30))])


def walks():
    """the whole model is one walked run, four walks"""
    return model(40, 70, 2, [("mamba2", mamba2(2, 12, 4, conv=2), dense(32)), ("attention", diff_attn(2, 1, 8, 8, 4), dense(48)),
                             ("latent_attention", latent(2, 8, 4, 8, 12), None)], loop=(0, 3, 4))


def one_layer_walk():
    """a run of one layer walked three times, between other layers"""
    return model(40, 70, 4, [("attention", diff_attn(2, 1, 8, 8, 8), dense(48)), ("mamba2", mamba2(3, 8, 5, conv=4), None),
                             ("latent_attention", latent(2, 8, 4, 8, 12), dense(16))], loop=(1, 2, 3))


def ones():
    """values that happen to be 1 or equal: one stream, one head, one group, one state, one tap, one norm part, one walk, scales and factors 1,
    no rotated dimensions, diff 0"""
    return model(32, 40, 1, [("mamba2", mamba2(1, 32, 1, groups=1, conv=1, norm_groups=1), dense(32, limit=1.0)),
                             ("attention", diff_attn(1, 1, 16, 16, 0, diff=0.0, scale=1.0), dense(32)),
                             ("latent_attention", latent(1, 16, 0, 16, 16, scale=1.0), None),
                             ("attention", diff_attn(1, 1, 16, 16, 16, diff=0.5, scaling=yarn(1.0, 16)), None)], loop=(0, 4, 1), embed_scale=1.0)


def far_keys():
    """peaky softmaxes over long prompts: single keys hundreds of tokens back carry the output"""
    return model(64, 300, 2, [("attention", diff_attn(2, 1, 24, 16, 12, diff=0.2, scale=1.2), None),
                              ("latent_attention", latent(4, 8, 8, 8, 16, scale=1.5), None)])


def wide_heads():
    """head sizes that are multiples of 8: long portions take the tensor-core (matmul) form of both attentions in served mode"""
    return model(64, 160, 4, [("attention", diff_attn(4, 2, 32, 16, 16, scaling=yarn(2.0, 128)), dense(96)),
                              ("mamba2", mamba2(4, 16, 16, groups=2, norm_groups=2), None),
                              ("latent_attention", latent(2, 16, 8, 24, 32), None)], loop=(0, 2, 2))


def medium():
    """wider layers in another order: more query heads per key head, 64 states, a walked pair in the middle"""
    return model(128, 500, 4, [("latent_attention", latent(4, 24, 8, 32, 48, base=50000.0), dense(200)),
                               ("mamba2", mamba2(8, 32, 64, groups=2, conv=4, norm_groups=4), dense(160)),
                               ("attention", diff_attn(8, 2, 32, 16, 32, diff=0.6, base=1000.0, scaling=yarn(8.0, 256)), None),
                               ("mamba2", mamba2(4, 48, 24, groups=4, conv=3, norm_groups=1), dense(96))], loop=(1, 3, 2))


def drawn(seed):
    """a configuration drawn from a seed: layer order, every size, the constants and the walked run all vary"""
    import numpy as np
    r = np.random.default_rng(seed)
    pick = lambda xs: xs[int(r.integers(0, len(xs)))]
    n = int(r.integers(2, 6))
    layers = []
    for _ in range(n):
        u = r.random()
        if u < 0.4:
            g, rep, vd = pick([1, 2, 3]), pick([1, 2, 4]), pick([4, 8, 12, 16, 40])
            parts = pick([d for d in (1, 2, 3, 4, 6) if (g * rep * vd) % d == 0 and g * rep * vd // d >= 8 or d == 1])   # parts of 8 channels and more: a norm over a handful of values magnifies rounding
            kind, mx = "mamba2", mamba2(g * rep, vd, pick([1, 3, 8, 16, 24, 40, 72]), groups=g, conv=int(r.integers(1, 6)), norm_groups=parts)
        elif u < 0.75:
            kv, rep, dim = pick([1, 2, 3]), pick([1, 2, 4]), pick([6, 8, 16, 20, 24, 40])
            rd = pick([0, 2, dim // 2 // 2 * 2, dim])
            sc = yarn(float(pick([1.5, 4.0, 16.0])), pick([16, 64, 512, 4096]), fast=float(pick([4.0, 32.0])), slow=float(pick([0.5, 1.0, 2.0]))) if rd and r.random() < 0.6 else None
            kind, mx = "attention", diff_attn(kv * rep, kv, dim, pick([8, 12, 16, 40]), rd, diff=float(r.uniform(0.1, 0.6)), base=pick([100.0, 10000.0, 1e6]), scaling=sc,
                                              scale=float(r.uniform(0.5, 2.0)) / math.sqrt(dim))
        else:
            dim, rd = pick([4, 8, 16, 24, 40]), pick([0, 2, 8, 12, 32])
            kind, mx = "latent_attention", latent(int(r.integers(1, 6)), dim, rd, pick([4, 8, 12, 16, 40]), pick([5, 16, 24, 64]), base=pick([100.0, 10000.0, 1e6]),
                                                  scale=float(r.uniform(0.5, 2.0)) / math.sqrt(dim + rd))
        layers.append((kind, mx, dense(pick([16, 50, 128]), limit=float(pick([0.5, 1.0, 7.0]))) if r.random() < 0.7 else None))
    loop = None
    if r.random() < 0.7:
        start = int(r.integers(0, n))
        loop = (start, int(r.integers(start + 1, n + 1)), int(r.integers(1, 4)))
    return model(pick([24, 40, 72, 96, 136]), int(r.integers(30, 400)), int(r.integers(1, 7)), layers, loop=loop, eps=pick([1e-6, 1e-5]), embed_scale=float(pick([1.0, 0.5, 3.5])))


CONFIGS = {f.__name__: f for f in (medium, mixed_small, mamba_only, diff_only, latent_only, walks, one_layer_walk, ones, far_keys, wide_heads)}
