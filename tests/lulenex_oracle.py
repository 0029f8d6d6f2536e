"""Plain, slow restatement of the Lulenex design in numpy float64 (test infrastructure only; shares no code with the library).

A model is (cfg, W): cfg the parsed config.json, W a dict name -> float64 array.  One function per mechanism; `Sequence` carries
what a sequence keeps between calls (the previous token's mixer input of every layer run, convolution tails, recurrent matrices, cached
keys and values), so the same functions serve whole prompts, portions and token-by-token decoding.

Notation: x residual stream [T, width]; e the embedding rows of the same tokens; a layer is u = x + mixer(shift(N1 x)),
x' = u + ff(N2 u) with N(x) = x / rms(x) * g, g ONE number.  A run of layers [start, stop) is walked `times` times with the same
weights; every walk r opens with x <- W_loop [x ; e] + step_r and keeps a state of its own.
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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ---- the layer's frame ----------------------------------------------------------------------------------------------------------------
def scalar_norm(x, g, eps):
    """RMS norm whose weight is a single number"""
    return rms_unit(x, eps) * float(g)


def token_shift(h, mu, st):
    """h_t <- h_t + (h_{t-1} - h_t) * mu, h_{t-1} the UNshifted row of the token before (zeros for a sequence's first token)"""
    prev = st.get("prev")
    if prev is None:
        prev = np.zeros(h.shape[1])
    before = np.concatenate([prev[None], h[:-1]], 0)
    st["prev"] = h[-1].copy()
    return h + (before - h) * mu


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2"""
    ap, aq = softplus(np.float64(p)), 0.5 + softplus(np.float64(q))
    zn = np.minimum(z, 0.0)
    return np.where(z > 0, ap * z * z + 0.5 * z, aq * (np.expm1(zn) - zn) + 0.5 * z)


def dense_ff(h, W, pre):
    return xielu(h @ W[pre + "up"].T, W[pre + "act"][0], W[pre + "act"][1]) @ W[pre + "down"].T


# ---- selective state space mixer --------------------------------------------------------------------------------------------------------
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


def selective_scan(u, dt, A, B, C, D, S):
    """S [inner, state] <- exp(dt A) S + dt u B^T per token; y = S C + D u.  Returns y; S is updated in place."""
    y = np.zeros_like(u)
    for t in range(u.shape[0]):
        S *= np.exp(dt[t][:, None] * A)
        S += (dt[t] * u[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * u[t]
    return y


def mamba1(h, W, pre, mx, st):
    inner, N, R = mx["inner"], mx["state"], mx["dt_rank"]
    xz = h @ W[pre + "in"].T
    u = conv_bias_silu(xz[:, :inner], W[pre + "conv"], W[pre + "conv.b"], st)
    z = xz[:, inner:]
    p = u @ W[pre + "x"].T
    dt = softplus(p[:, :R] @ W[pre + "dt"].T + W[pre + "dt.b"])
    if "S" not in st:
        st["S"] = np.zeros((inner, N))
    y = selective_scan(u, dt, -np.exp(W[pre + "A_log"]), p[:, R:R + N], p[:, R + N:R + 2 * N], W[pre + "D"], st["S"])
    return (y * silu(z)) @ W[pre + "o"].T


# ---- the two-branch mixer ---------------------------------------------------------------------------------------------------------------
def rotate_half(v, pos, dims, base):
    """v [T, heads, dim]: within the first `dims` coordinates of every head, (a_i, a_{i + dims/2}) turns by pos * base^(-2i/dims)"""
    half = dims // 2
    ang = np.asarray(pos, np.float64)[:, None] * base ** (-2.0 * np.arange(half) / dims)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = v.copy()
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def chunk_softmax_attention(q, keys, vals, pos, size, scale, sink):
    """q [T, H, D] at positions pos; keys [n, G, D], vals [n, G, V] of positions 0 .. n-1.  Token at p reads j <= p with j // size == p // size;
    the denominator holds one more term exp(sink_h)."""
    T, H, _ = q.shape
    G = keys.shape[1]
    out = np.zeros((T, H, vals.shape[2]))
    for t in range(T):
        p = pos[t]
        lo = (p // size) * size
        for hh in range(H):
            g = hh // (H // G)
            s = keys[lo:p + 1, g] @ q[t, hh] * scale
            m = max(s.max(), sink[hh])
            e = np.exp(s - m)
            out[t, hh] = (e[:, None] * vals[lo:p + 1, g]).sum(0) / (e.sum() + math.exp(sink[hh] - m))
    return out


def softmax_branch(h, W, pre, mx, eps, st, pos):
    H, G, D = mx["heads"], mx["kv_heads"], mx["dim"]
    T = h.shape[0]
    q = (h @ W[pre + "q"].T + W[pre + "q.b"]).reshape(T, H, D)
    k = (h @ W[pre + "k"].T + W[pre + "k.b"]).reshape(T, G, D)
    v = k.copy()                                                  # the values are the keys as projected
    rot = mx["rot"]
    q = rms_unit(rotate_half(q, pos, rot["dims"], rot["base"]), eps)
    k = rms_unit(rotate_half(k, pos, rot["dims"], rot["base"]), eps)
    st["K"] = np.concatenate([st["K"], k], 0) if "K" in st else k
    st["V"] = np.concatenate([st["V"], v], 0) if "V" in st else v
    o = chunk_softmax_attention(q, st["K"], st["V"], pos, mx["mask"]["size"], mx["scale"], W[pre + "sink"])
    o = o * sigmoid(h @ W[pre + "g"].T)[:, :, None]
    return o.reshape(T, -1) @ W[pre + "o"].T + W[pre + "o.b"]


def decayed_outer_scan(q, k, v, decay, S):
    """per head: S <- decay_h S + k v^T, o = S^T q.  q, k [T, H, D], v [T, H, V], S [H, D, V] updated in place."""
    T, H, _ = q.shape
    o = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        for hh in range(H):
            S[hh] = decay[hh] * S[hh] + np.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ q[t, hh]
    return o


def linear_branch(h, W, pre, mx, eps, st):
    H, D, V = mx["heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = silu(h @ W[pre + "q"].T).reshape(T, H, D)
    k = silu(h @ W[pre + "k"].T).reshape(T, H, D)
    v = silu(h @ W[pre + "v"].T).reshape(T, H, V)
    if "S" not in st:
        st["S"] = np.zeros((H, D, V))
    o = decayed_outer_scan(q, k, v, np.asarray(mx["decay"], np.float64), st["S"]).reshape(T, H * V)
    o = rms_unit(o, eps) * W[pre + "norm"] * sigmoid(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T


def two_branch(h, W, pre, mx, eps, st, pos):
    a = softmax_branch(h, W, pre + "left.", mx["left"], eps, st.setdefault("left", {}), pos)
    b = linear_branch(h, W, pre + "right.", mx["right"], eps, st.setdefault("right", {}))
    return mx["left_scale"] * a + mx["right_scale"] * b


# ---- the model --------------------------------------------------------------------------------------------------------------------------
def layer_runs(cfg):
    """[(layer, walk r or None, opens a walk)] in the order they run"""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, None, False) for i in range(n)]
    a, b, times = lp["start"], lp["stop"], lp["times"]
    runs = [(i, None, False) for i in range(a)]
    for r in range(times):
        runs += [(i, r, i == a) for i in range(a, b)]
    return runs + [(i, None, False) for i in range(b, n)]


class Sequence:
    def __init__(self, cfg):
        self.n = 0
        self.runs = [dict() for _ in layer_runs(cfg)]


def layer(x, cfg, W, il, st, pos):
    jl = cfg["layers"][il]
    eps = cfg["norm"]["eps"]
    p = "l%d." % il
    h = token_shift(scalar_norm(x, W[p + "norm1"], eps), W[p + "shift"], st)
    if jl["type"] == "mamba1":
        y = mamba1(h, W, p + "mix.", jl["mixer"], st.setdefault("mix", {}))
    elif jl["type"] == "parallel":
        y = two_branch(h, W, p + "mix.", jl["mixer"], eps, st.setdefault("mix", {}), pos)
    else:
        raise ValueError(jl["type"])
    x = x + y
    if jl.get("mlp"):
        x = x + dense_ff(scalar_norm(x, W[p + "norm2"], eps), W, p + "mlp.")
    return x


def forward(cfg, W, seq, tokens, trace=None):
    """logits [T, vocab] of the next `tokens` of the sequence; trace (a list) receives the residual stream after every layer run"""
    T = len(tokens)
    pos = list(range(seq.n, seq.n + T))
    e = W["embed"][np.asarray(tokens)]
    x = e.copy()
    for (il, r, opens), st in zip(layer_runs(cfg), seq.runs):
        if opens:
            x = np.concatenate([x, e], 1) @ W["loop.in"].T + W["loop.step"][r]
        x = layer(x, cfg, W, il, st, pos)
        if trace is not None:
            trace.append(x.copy())
    seq.n += T
    return scalar_norm(x, W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T


# ---- test models --------------------------------------------------------------------------------------------------------------------------
def tensor_shapes(cfg):
    """name -> shape of every tensor a model of this configuration holds"""
    Wd, s = cfg["width"], {}
    s["embed"] = (cfg["vocab"], Wd)
    s["head"] = (cfg["vocab"], Wd)
    s["final.norm"] = ()
    if cfg.get("loop"):
        s["loop.in"] = (Wd, 2 * Wd)
        s["loop.step"] = (cfg["loop"]["times"], Wd)
    for i, jl in enumerate(cfg["layers"]):
        p, mx = "l%d." % i, jl["mixer"]
        s[p + "norm1"] = ()
        s[p + "shift"] = (Wd,)
        if jl["type"] == "mamba1":
            I, N, R, K = mx["inner"], mx["state"], mx["dt_rank"], mx["conv"]
            s.update({p + "mix.in": (2 * I, Wd), p + "mix.conv": (I, K), p + "mix.conv.b": (I,), p + "mix.x": (R + 2 * N, I), p + "mix.dt": (I, R),
                      p + "mix.dt.b": (I,), p + "mix.A_log": (I, N), p + "mix.D": (I,), p + "mix.o": (Wd, I)})
        else:
            a, b = mx["left"], mx["right"]
            H, G, D = a["heads"], a["kv_heads"], a["dim"]
            s.update({p + "mix.left.q": (H * D, Wd), p + "mix.left.q.b": (H * D,), p + "mix.left.k": (G * D, Wd), p + "mix.left.k.b": (G * D,),
                      p + "mix.left.sink": (H,), p + "mix.left.g": (H, Wd), p + "mix.left.o": (Wd, H * D), p + "mix.left.o.b": (Wd,)})
            H, D, V = b["heads"], b["dim"], b["vdim"]
            s.update({p + "mix.right.q": (H * D, Wd), p + "mix.right.k": (H * D, Wd), p + "mix.right.v": (H * V, Wd), p + "mix.right.g": (H * V, Wd),
                      p + "mix.right.o": (Wd, H * V), p + "mix.right.norm": (H * V,)})
        if jl.get("mlp"):
            s[p + "norm2"] = ()
            s.update({p + "mlp.up": (jl["mlp"]["ff"], Wd), p + "mlp.down": (Wd, jl["mlp"]["ff"]), p + "mlp.act": (2,)})
    return s


def random_weights(cfg, seed):
    """bfloat16-representable random weights, float64"""
    rng = np.random.default_rng(seed)
    W = {}
    for name, s in tensor_shapes(cfg).items():
        if name.endswith("norm1") or name.endswith("norm2") or name == "final.norm":
            w = np.asarray(rng.uniform(0.7, 1.4))
        elif name.endswith("norm"):
            w = 1.0 + 0.2 * rng.standard_normal(s)
        elif name.endswith("shift"):
            w = rng.uniform(0.0, 1.0, s)
        elif name.endswith(".conv"):
            w = 0.4 * rng.standard_normal(s)
            w[:, -1] += 0.6
        elif name.endswith("A_log"):
            w = rng.uniform(-2.0, 1.0, s)
        elif name.endswith("dt.b"):
            w = rng.uniform(-3.0, 0.0, s)
        elif name.endswith(".b") or name.endswith("sink") or name.endswith("mix.D") or name == "loop.step":
            w = 0.5 * rng.standard_normal(s)
        elif name.endswith(".act"):
            w = rng.uniform(-1.0, 1.0, s)
        elif name == "embed":
            w = rng.standard_normal(s)
        elif name == "loop.in":
            w = rng.standard_normal(s) * (1.0 / math.sqrt(s[-1] / 2))
        else:
            w = rng.standard_normal(s) * (1.2 / math.sqrt(s[-1]))
        W[name] = bf16_round(w)
    return W
