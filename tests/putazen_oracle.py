"""Plain, slow restatement of the Putazen design in numpy float64 (test infrastructure only; shares no code with the library).

A model is (cfg, W): cfg the parsed config.json, W a dict name -> float64 array.  One function per mechanism; `Sequence` carries what a
sequence keeps between calls (convolution tails, recurrent matrices, cached keys / values / latents of every layer run), so the same
functions serve whole prompts, portions and token-by-token decoding.

Notation: X the residual streams [T, streams, width].  A sublayer f with read weights a [streams], write weights b [streams] and mixing
matrix M [streams, streams] does  u = sum_s a_s X_s,  y = f(LN(u)),  X'_t = sum_s M[s, t] X_s + b_t y.  A run of layers [start, stop) is
walked `times` times with the same weights; every walk keeps a state of its own.
"""
import math

import numpy as np

from tests.rapisun_oracle import bf16_round, write_model  # noqa: F401  (helpers for writing test models)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


# ---- the layer's frame ----------------------------------------------------------------------------------------------------------------
def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b, var the mean of the squared deviations"""
    d = x - x.mean(-1, keepdims=True)
    return d / np.sqrt((d * d).mean(-1, keepdims=True) + eps) * w + b


def hyper_read(X, a):
    """u = sum_s a_s X_s"""
    return np.einsum("s,tsw->tw", a, X)


def hyper_write(X, M, b, y):
    """X'_t = sum_s M[s, t] X_s + b_t y, every new stream formed from the streams as they were before the sublayer"""
    return np.einsum("su,Tsw->Tuw", M, X) + b[None, :, None] * y[:, None, :]


def clamped_glu_ff(h, W, pre, limit):
    """g = min(W_g h, L), u = clamp(W_u h, -L, L); W_d (g sigmoid(1.702 g) (u + 1))"""
    g = np.minimum(h @ W[pre + "gate"].T, limit)
    u = np.clip(h @ W[pre + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[pre + "down"].T


# ---- state-space duality mixer ----------------------------------------------------------------------------------------------------------
def conv_bias_silu(u, w, b, st):
    """causal per-channel convolution, w [C, taps] with the last column on the current token, zeros before the sequence's start"""
    taps = w.shape[1]
    tail = st.get("tail")
    if tail is None:
        tail = np.zeros((taps - 1, u.shape[1]))
    ext = np.concatenate([tail, u], 0)
    out = np.tile(b, (u.shape[0], 1)).astype(np.float64)
    for t in range(u.shape[0]):
        for j in range(taps):
            out[t] += w[:, j] * ext[t + j]
    st["tail"] = ext[ext.shape[0] - (taps - 1):].copy()
    return silu(out)


def scalar_decay_scan(x, dt, A, B, C, D, S):
    """per head h (group g of B, C): S_h [N, P] <- exp(-A_h dt) S_h + dt B x^T, y = S_h^T C + D_h x.
    x [T, H, P], dt [T, H], B, C [T, G, N]; S [H, N, P] updated in place."""
    T, H, _ = x.shape
    G = B.shape[1]
    y = np.zeros_like(x)
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            S[h] = math.exp(-A[h] * dt[t, h]) * S[h] + dt[t, h] * np.outer(B[t, g], x[t, h])
            y[t, h] = S[h].T @ C[t, g] + D[h] * x[t, h]
    return y


def grouped_rms(y, parts, w, eps):
    """RMS norm in `parts` equal parts of the last axis, each by its own root mean square, then times w"""
    T, C = y.shape
    return rms_unit(y.reshape(T, parts, C // parts), eps).reshape(T, C) * w


def mamba2(h, W, pre, mx, eps, st):
    H, P, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
    I, T = H * P, h.shape[0]
    p = h @ W[pre + "in"].T
    z, xbc, dt = p[:, :I], p[:, I:2 * I + 2 * G * N], p[:, 2 * I + 2 * G * N:]
    xbc = conv_bias_silu(xbc, W[pre + "conv"], W[pre + "conv.b"], st)
    x, B, C = xbc[:, :I].reshape(T, H, P), xbc[:, I:I + G * N].reshape(T, G, N), xbc[:, I + G * N:].reshape(T, G, N)
    dt = softplus(dt + W[pre + "dt_bias"])
    if "S" not in st:
        st["S"] = np.zeros((H, N, P))
    y = scalar_decay_scan(x, dt, np.exp(W[pre + "A_log"]), B, C, W[pre + "D"], st["S"]).reshape(T, I)
    y = grouped_rms(y * silu(z), mx["norm_groups"], W[pre + "norm"], eps)           # gated first, normed after
    return y @ W[pre + "o"].T


# ---- rotations ---------------------------------------------------------------------------------------------------------------------------
def rot_frequencies(rot):
    """(frequencies [dims / 2], factor on cos and sin).  With rot["scaling"] (factor, original, fast, slow): frequencies whose wavelength is
    long against the original context are divided by the factor, short ones stay, a linear ramp between; cos and sin times 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], rot["base"]
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def dim_of(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(sc["fast"])), 0)
    hi = min(math.ceil(dim_of(sc["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(v, pos, rot, interleaved):
    """v [T, heads, dim]: within the first rot.dims coordinates the pairs (i, i + dims/2) -- or (2i, 2i+1) when interleaved -- turn by pos * f_i"""
    dims = rot["dims"]
    if dims == 0:
        return v.copy()
    f, mag = rot_frequencies(rot)
    ang = np.asarray(pos, np.float64)[:, None] * f
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    out = v.copy()
    if interleaved:
        a, b = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        half = dims // 2
        a, b = v[..., :half], v[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    return out


def causal_softmax_attention(q, keys, vals, pos, scale):
    """q [T, H, D] at positions pos; keys [n, H, D], vals [n, H, V] of positions 0 .. n-1; token at p reads j <= p"""
    T, H, _ = q.shape
    out = np.zeros((T, H, vals.shape[2]))
    for t in range(T):
        p = pos[t]
        for h in range(H):
            s = keys[:p + 1, h] @ q[t, h] * scale
            e = np.exp(s - s.max())
            out[t, h] = (e[:, None] * vals[:p + 1, h]).sum(0) / e.sum()
    return out


# ---- differential attention ----------------------------------------------------------------------------------------------------------------
def differential_attention(h, W, pre, mx, eps, st, pos):
    """two softmax maps per head over the same values: o = a1 - lambda a2, lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff; o / rms(o) * (1 - diff)"""
    H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    T, diff = h.shape[0], mx["diff"]
    q = (h @ W[pre + "q"].T + W[pre + "q.b"]).reshape(T, 2 * H, D)            # head by head: [map 1 | map 2]
    k = (h @ W[pre + "k"].T + W[pre + "k.b"]).reshape(T, 2 * G, D)
    v = (h @ W[pre + "v"].T + W[pre + "v.b"]).reshape(T, G, V)
    q = rotate(q, pos, mx["rot"], False)
    k = rotate(k, pos, mx["rot"], False)
    st["K"] = np.concatenate([st["K"], k], 0) if "K" in st else k
    st["V"] = np.concatenate([st["V"], v], 0) if "V" in st else v
    rep = H // G
    # one attention per (head, map): its keys are map m of the head's key / value head, its values that head's values
    kk = np.stack([st["K"][:, (a // 2 // rep) * 2 + a % 2] for a in range(2 * H)], 1)
    vv = np.stack([st["V"][:, a // 2 // rep] for a in range(2 * H)], 1)
    a = causal_softmax_attention(q, kk, vv, pos, mx["scale"]).reshape(T, H, 2, V)
    lam = math.exp(float(W[pre + "lq1"] @ W[pre + "lk1"])) - math.exp(float(W[pre + "lq2"] @ W[pre + "lk2"])) + diff
    o = rms_unit(a[:, :, 0] - lam * a[:, :, 1], eps) * (1.0 - diff)
    return o.reshape(T, H * V) @ W[pre + "o"].T


# ---- latent attention ------------------------------------------------------------------------------------------------------------------------
def latent_attention(h, W, pre, mx, eps, st, pos):
    """keys and values are expanded from a cached latent c [kv_rank]; one rotated key part [rot_dim] is shared by all heads"""
    H, D, rd, V, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    T = h.shape[0]
    q = (h @ W[pre + "q"].T).reshape(T, H, D + rd)
    ckr = h @ W[pre + "dkv"].T
    c = rms_unit(ckr[:, :R], eps) * W[pre + "dkv.norm"]
    rot = dict(mx["rot"], dims=rd)
    kr = rotate(ckr[:, None, R:], pos, rot, True)[:, 0]
    qr = rotate(q[:, :, D:], pos, rot, True)
    st["C"] = np.concatenate([st["C"], c], 0) if "C" in st else c
    st["KR"] = np.concatenate([st["KR"], kr], 0) if "KR" in st else kr
    n = st["C"].shape[0]
    ku = (st["C"] @ W[pre + "uk"].T).reshape(n, H, D)
    vv = (st["C"] @ W[pre + "uv"].T).reshape(n, H, V)
    kk = np.concatenate([ku, np.repeat(st["KR"][:, None, :], H, 1)], 2)
    qq = np.concatenate([q[:, :, :D], qr], 2)
    o = causal_softmax_attention(qq, kk, vv, pos, mx["scale"])
    return o.reshape(T, H * V) @ W[pre + "o"].T


# ---- the model --------------------------------------------------------------------------------------------------------------------------
def layer_runs(cfg):
    """the layers in the order they run"""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    a, b, times = lp["start"], lp["stop"], lp["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


class Sequence:
    def __init__(self, cfg):
        self.n = 0
        self.runs = [dict() for _ in layer_runs(cfg)]


def run_mixer(h, cfg, W, il, st, pos):
    jl, eps, pre = cfg["layers"][il], cfg["norm"]["eps"], "l%d.mix." % il
    if jl["type"] == "mamba2":
        return mamba2(h, W, pre, jl["mixer"], eps, st)
    if jl["type"] == "attention":
        return differential_attention(h, W, pre, jl["mixer"], eps, st, pos)
    if jl["type"] == "latent_attention":
        return latent_attention(h, W, pre, jl["mixer"], eps, st, pos)
    raise ValueError(jl["type"])


def layer(X, cfg, W, il, st, pos):
    jl, eps, p = cfg["layers"][il], cfg["norm"]["eps"], "l%d." % il
    h = layer_norm(hyper_read(X, W[p + "hc1.in"]), W[p + "norm1"], W[p + "norm1.b"], eps)
    X = hyper_write(X, W[p + "hc1.mix"], W[p + "hc1.out"], run_mixer(h, cfg, W, il, st, pos))
    if jl.get("mlp"):
        h = layer_norm(hyper_read(X, W[p + "hc2.in"]), W[p + "norm2"], W[p + "norm2.b"], eps)
        X = hyper_write(X, W[p + "hc2.mix"], W[p + "hc2.out"], clamped_glu_ff(h, W, p + "mlp.", jl["mlp"]["limit"]))
    return X


def forward(cfg, W, seq, tokens, trace=None):
    """logits [T, vocab] of the next `tokens` of the sequence; trace (a list) receives the sum of the streams after every layer run"""
    T = len(tokens)
    pos = list(range(seq.n, seq.n + T))
    e = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    X = np.repeat(e[:, None, :], cfg["streams"], 1)
    for il, st in zip(layer_runs(cfg), seq.runs):
        X = layer(X, cfg, W, il, st, pos)
        if trace is not None:
            trace.append(X.sum(1))
    seq.n += T
    return layer_norm(X.sum(1), W["final.norm"], W["final.norm.b"], cfg["norm"]["eps"]) @ W["head"].T


# ---- test models --------------------------------------------------------------------------------------------------------------------------
def tensor_shapes(cfg):
    """name -> shape of every tensor a model of this configuration holds"""
    Wd, S, s = cfg["width"], cfg["streams"], {}
    s["embed"] = (cfg["vocab"], Wd)
    s["head"] = (cfg["vocab"], Wd)
    s["final.norm"] = s["final.norm.b"] = (Wd,)
    for i, jl in enumerate(cfg["layers"]):
        p, mx = "l%d." % i, jl["mixer"]
        s[p + "norm1"] = s[p + "norm1.b"] = (Wd,)
        s.update({p + "hc1.in": (S,), p + "hc1.out": (S,), p + "hc1.mix": (S, S)})
        if jl["type"] == "mamba2":
            H, P, N, G, K = mx["heads"], mx["vdim"], mx["state"], mx["groups"], mx["conv"]
            I, C = H * P, H * P + 2 * G * N
            s.update({p + "mix.in": (I + C + H, Wd), p + "mix.conv": (C, K), p + "mix.conv.b": (C,), p + "mix.dt_bias": (H,), p + "mix.A_log": (H,),
                      p + "mix.D": (H,), p + "mix.norm": (I,), p + "mix.o": (Wd, I)})
        elif jl["type"] == "attention":
            H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            s.update({p + "mix.q": (2 * H * D, Wd), p + "mix.q.b": (2 * H * D,), p + "mix.k": (2 * G * D, Wd), p + "mix.k.b": (2 * G * D,),
                      p + "mix.v": (G * V, Wd), p + "mix.v.b": (G * V,), p + "mix.lq1": (D,), p + "mix.lk1": (D,), p + "mix.lq2": (D,), p + "mix.lk2": (D,),
                      p + "mix.o": (Wd, H * V)})
        else:
            H, D, rd, V, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
            s.update({p + "mix.q": (H * (D + rd), Wd), p + "mix.dkv": (R + rd, Wd), p + "mix.dkv.norm": (R,), p + "mix.uk": (H * D, R), p + "mix.uv": (H * V, R),
                      p + "mix.o": (Wd, H * V)})
        if jl.get("mlp"):
            F = jl["mlp"]["ff"]
            s[p + "norm2"] = s[p + "norm2.b"] = (Wd,)
            s.update({p + "hc2.in": (S,), p + "hc2.out": (S,), p + "hc2.mix": (S, S)})
            s.update({p + "mlp.gate": (F, Wd), p + "mlp.up": (F, Wd), p + "mlp.down": (Wd, F)})
    return s


def random_weights(cfg, seed):
    """bfloat16-representable random weights, float64"""
    rng = np.random.default_rng(seed)
    S = cfg["streams"]
    W = {}
    for name, s in tensor_shapes(cfg).items():
        if name.endswith(".in") and ".hc" in name:
            w = rng.uniform(0.1, 0.6, s) * rng.choice([-1.0, 1.0], s, p=[0.2, 0.8])
        elif name.endswith(".out") and ".hc" in name:
            w = rng.uniform(0.3, 1.0, s) * rng.choice([-1.0, 1.0], s, p=[0.2, 0.8])
        elif name.endswith(".mix") and ".hc" in name:
            w = 0.8 * np.eye(S) + 0.25 * rng.standard_normal(s) / math.sqrt(S)
        elif name.endswith("norm1") or name.endswith("norm2") or name.endswith("norm"):
            w = 1.0 + 0.2 * rng.standard_normal(s)
        elif name.endswith(".conv"):
            w = 0.4 * rng.standard_normal(s)
            w[:, -1] += 0.6
        elif name.endswith("A_log"):
            w = rng.uniform(-3.0, 0.5, s)
        elif name.endswith("dt_bias"):
            w = rng.uniform(-3.0, 0.5, s)
        elif name.endswith("mix.D"):
            w = 0.5 * rng.standard_normal(s)
        elif name[-4:-1] == ".lq" or name[-4:-1] == ".lk":
            w = 0.3 * rng.standard_normal(s)
        elif name.endswith(".b"):
            w = 0.3 * rng.standard_normal(s)
        elif name == "embed":
            w = rng.standard_normal(s)
        else:
            w = rng.standard_normal(s) * (1.2 / math.sqrt(s[-1]))
        W[name] = bf16_round(w)
    return W
