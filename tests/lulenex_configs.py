"""Small Lulenex configurations for the tests (sizes chosen to differ from each other: heads, key / value heads, dims, chunks, rotated
dimensions, states, taps, walks)."""
import math


def ssm(inner, state, dt_rank, conv):
    return {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}


def softmax_branch(heads, kv_heads, dim, chunk, rot_dims, base=10000.0, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": chunk}, "rot": {"base": base, "dims": rot_dims},
            "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}


def linear_branch(heads, dim, vdim, decay):
    assert len(decay) == heads
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def two(left, right, a=0.7, b=1.2):
    return {"left": left, "right": right, "left_scale": a, "right_scale": b}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def model(width, vocab, layers, loop=None, eps=1e-6):
    cfg = {"architecture": "Lulenex", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": [{"type": t, "mixer": mx, "mlp": ml} for t, mx, ml in layers]}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def mixed_small():
    """both mixers, a walked run in the middle that ends with the state-space layer, a layer without feed-forward"""
    return model(80, 190, [("parallel", two(softmax_branch(4, 2, 12, 7, 8), linear_branch(3, 10, 14, [0.5, 0.9, 0.97])), dense(100)),
                           ("parallel", two(softmax_branch(2, 2, 20, 11, 20, base=500.0, scale=0.4), linear_branch(1, 24, 8, [0.8]), a=1.3, b=0.5), None),
                           ("mamba1", ssm(96, 6, 5, 3), dense(72)),
                           ("mamba1", ssm(40, 17, 9, 2), None),
                           ("parallel", two(softmax_branch(6, 3, 8, 5, 4), linear_branch(2, 12, 12, [0.3, 0.99])), dense(64))], loop=(1, 3, 2))


def ssm_only():
    return model(48, 100, [("mamba1", ssm(72, 8, 4, 4), None), ("mamba1", ssm(50, 33, 7, 3), dense(40))])


def softmax_mostly():
    """the linear branch nearly silent: what the logits show is the chunked attention (rotation, unit norms, sink, values = keys, gates)"""
    return model(64, 120, [("parallel", two(softmax_branch(4, 2, 16, 9, 10, scale=0.6), linear_branch(1, 4, 4, [0.5]), a=1.0, b=0.01), None),
                           ("parallel", two(softmax_branch(3, 1, 12, 9, 12, base=77.0), linear_branch(1, 4, 4, [0.5]), a=1.0, b=0.01), None)])


def linear_mostly():
    return model(56, 90, [("parallel", two(softmax_branch(1, 1, 8, 4, 2), linear_branch(3, 20, 12, [0.6, 0.95, 0.999]), a=0.01, b=1.0), None),
                          ("parallel", two(softmax_branch(1, 1, 8, 4, 2), linear_branch(2, 6, 30, [0.2, 1.0]), a=0.01, b=1.0), dense(30))])


def walks():
    """the whole model is one walked run, four walks"""
    return model(40, 70, [("mamba1", ssm(48, 4, 3, 2), dense(32)), ("parallel", two(softmax_branch(2, 1, 8, 6, 8), linear_branch(2, 8, 8, [0.7, 0.9])), dense(48))], loop=(0, 2, 4))


def one_layer_walk():
    """a run of one layer walked twice, between other layers"""
    return model(40, 70, [("parallel", two(softmax_branch(2, 1, 8, 6, 8), linear_branch(2, 8, 8, [0.7, 0.9])), dense(48)),
                          ("mamba1", ssm(48, 4, 3, 2), None), ("mamba1", ssm(24, 5, 2, 4), dense(16))], loop=(1, 2, 2))


def ones():
    """values that happen to be 1 or equal: one head, one key head, one state, rank 1, one tap, chunks of 1, one walk, scales 1"""
    return model(32, 40, [("parallel", two(softmax_branch(1, 1, 16, 1, 16, scale=1.0), linear_branch(1, 16, 16, [1.0]), a=1.0, b=1.0), dense(32)),
                          ("mamba1", ssm(32, 1, 1, 1), dense(32)),
                          ("parallel", two(softmax_branch(1, 1, 16, 4096, 0), linear_branch(1, 16, 16, [0.5]), a=1.0, b=1.0), None)], loop=(0, 3, 1))


def far_keys():
    """long chunks and a peaky softmax: single keys hundreds of tokens back carry the output"""
    return model(64, 300, [("parallel", two(softmax_branch(2, 1, 24, 260, 12, scale=2.0), linear_branch(1, 8, 8, [0.9]), a=1.0, b=0.05), None),
                           ("parallel", two(softmax_branch(4, 4, 8, 193, 8, scale=3.0), linear_branch(1, 8, 8, [0.9]), a=1.0, b=0.05), None)])


def wide_heads():
    """head sizes that are multiples of 8: long portions take the tensor-core (matmul) form of the attention in served mode"""
    return model(64, 160, [("parallel", two(softmax_branch(4, 2, 32, 150, 16), linear_branch(2, 16, 16, [0.8, 0.95])), dense(96)),
                           ("mamba1", ssm(128, 16, 4, 4), None),
                           ("parallel", two(softmax_branch(2, 2, 16, 37, 16), linear_branch(2, 16, 24, [0.9, 0.99])), None)], loop=(0, 2, 2))


def medium():
    """wider layers in another order: full rotation, more query heads per key head, 16 states, a walked pair in the middle"""
    return model(128, 500, [("parallel", two(softmax_branch(8, 2, 32, 100, 32, base=1000.0), linear_branch(4, 16, 32, [0.5, 0.9, 0.99, 0.999])), dense(200)),
                            ("mamba1", ssm(256, 16, 8, 4), dense(160)),
                            ("parallel", two(softmax_branch(4, 4, 48, 64, 24), linear_branch(2, 32, 16, [0.95, 0.8]), a=0.5, b=1.5), None),
                            ("mamba1", ssm(192, 8, 6, 3), dense(96))], loop=(1, 3, 2))


def drawn(seed):
    """a configuration drawn from a seed: layer order, every size, the constants and the walked run all vary"""
    import numpy as np
    r = np.random.default_rng(seed)
    pick = lambda xs: xs[int(r.integers(0, len(xs)))]
    n = int(r.integers(2, 6))
    layers = []
    for _ in range(n):
        if r.random() < 0.45:
            kind, mx = "mamba1", ssm(pick([16, 40, 56, 96, 160]), pick([1, 3, 8, 16, 24, 40]), int(r.integers(1, 12)), int(r.integers(1, 5)))
        else:
            kv, rep, dim = pick([1, 2, 3]), pick([1, 2, 4]), pick([6, 8, 16, 20, 24, 40])
            left = softmax_branch(kv * rep, kv, dim, pick([1, 3, 16, 50, 129, 1000]), pick([0, 2, dim // 2 // 2 * 2, dim]), base=pick([100.0, 10000.0, 1e6]),
                                  scale=float(r.uniform(0.5, 2.0)) / math.sqrt(dim))
            h2 = int(r.integers(1, 4))
            right = linear_branch(h2, pick([4, 10, 16, 32]), pick([4, 12, 16, 40]), [float(x) for x in r.uniform(0.3, 1.0, h2)])
            kind, mx = "parallel", two(left, right, a=float(r.uniform(0.3, 1.5)), b=float(r.uniform(0.3, 1.5)))
        layers.append((kind, mx, dense(pick([16, 50, 128])) if r.random() < 0.7 else None))
    loop = None
    if r.random() < 0.7:
        start = int(r.integers(0, n))
        loop = (start, int(r.integers(start + 1, n + 1)), int(r.integers(1, 4)))
    return model(pick([24, 40, 72, 96, 136]), int(r.integers(30, 400)), layers, loop=loop, eps=pick([1e-6, 1e-5]))


CONFIGS = {f.__name__: f for f in (medium, mixed_small, ssm_only, softmax_mostly, linear_mostly, walks, one_layer_walk, ones, far_keys, wide_heads)}
