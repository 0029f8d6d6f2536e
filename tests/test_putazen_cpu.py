"""CPU: the float64 restatement of the Putazen design agrees with itself over cuts (whole prompt, portions, token by token) for every test
configuration, and its parts do what their definitions say on inputs whose answer is known."""
import math

import numpy as np
import pytest

from tests import putazen_oracle as O
from tests.putazen_configs import CONFIGS, drawn


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_oracle_cuts_agree(name):
    cfg = CONFIGS[name]()
    W = O.random_weights(cfg, 3)
    toks = np.random.default_rng(1).integers(0, cfg["vocab"], 23).tolist()
    whole = O.forward(cfg, W, O.Sequence(cfg), toks)
    assert whole.shape == (23, cfg["vocab"]) and np.isfinite(whole).all()
    for cuts in ([1], range(1, 23), [2, 4, 5, 12, 14, 21]):
        seq, out, a = O.Sequence(cfg), [], 0
        for b in list(cuts) + [23]:
            out.append(O.forward(cfg, W, seq, toks[a:b]))
            a = b
        assert np.abs(np.concatenate(out) - whole).max() < 1e-9


def test_drawn_configurations_are_well_formed():
    for seed in range(40):
        cfg = drawn(seed)
        W = O.random_weights(cfg, seed)
        lg = O.forward(cfg, W, O.Sequence(cfg), [1, 2, 3])
        assert lg.shape == (3, cfg["vocab"]) and np.isfinite(lg).all()


def test_layer_runs_order():
    assert O.layer_runs(CONFIGS["mixed_small"]()) == [0, 1, 2, 3, 1, 2, 3, 4]
    assert O.layer_runs(CONFIGS["one_layer_walk"]()) == [0, 1, 1, 1, 2]
    assert O.layer_runs(CONFIGS["mamba_only"]()) == [0, 1]


def test_hyper_connections_one_stream_is_a_weighted_residual():
    X = np.arange(6.0).reshape(2, 1, 3)
    y = np.ones((2, 3))
    assert np.allclose(O.hyper_read(X, np.array([2.0])), 2 * X[:, 0])
    assert np.allclose(O.hyper_write(X, np.array([[0.5]]), np.array([3.0]), y)[:, 0], 0.5 * X[:, 0] + 3.0)


def test_hyper_write_reads_the_old_streams_and_indexes_from_to():
    X = np.zeros((1, 2, 1))
    X[0, 0, 0], X[0, 1, 0] = 1.0, 10.0
    M = np.array([[0.0, 1.0], [0.0, 0.0]])                   # stream 0 goes to stream 1, nothing else moves
    out = O.hyper_write(X, M, np.zeros(2), np.zeros((1, 1)))
    assert np.allclose(out[0, :, 0], [0.0, 1.0])


def test_layer_norm_centres_and_adds_the_bias():
    x = np.array([[1.0, 2.0, 3.0, 6.0]])
    out = O.layer_norm(x, np.full(4, 2.0), np.full(4, 0.5), 0.0)
    assert np.allclose(out.mean(), 0.5) and np.allclose(((out - 0.5) ** 2).mean(), 4.0)


def test_clamped_glu_branches():
    W = {"gate": np.eye(3), "up": np.eye(3), "down": np.eye(3)}
    h = np.array([[-4.0, 0.5, 4.0]])
    g = np.array([-4.0, 0.5, 2.0])                            # the gate is capped from above only
    u = np.array([-2.0, 0.5, 2.0])                            # the linear part on both sides
    assert np.allclose(O.clamped_glu_ff(h, W, "", 2.0), g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0))


def test_scalar_decay_scan_two_steps_by_hand():
    x = np.array([[[2.0]], [[3.0]]])
    dt = np.array([[0.5], [0.25]])
    B = np.array([[[1.0, 0.0]], [[0.0, 1.0]]])
    C = np.array([[[1.0, 1.0]], [[1.0, 1.0]]])
    S = np.zeros((1, 2, 1))
    y = O.scalar_decay_scan(x, dt, np.array([2.0]), B, C, np.array([0.1]), S)
    # step 1: S = [[1], [0]], y = 1 + 0.2; step 2: S = e^{-0.5} [[1], [0]] + [[0], [0.75]], y = e^{-0.5} + 0.75 + 0.3
    assert np.allclose(y[:, 0, 0], [1.2, math.exp(-0.5) + 1.05])
    assert np.allclose(S[0, :, 0], [math.exp(-0.5), 0.75])


def test_heads_share_the_group_of_their_block():
    # 4 heads in 2 groups: heads 0, 1 read group 0; heads 2, 3 group 1
    x = np.ones((1, 4, 1))
    dt = np.ones((1, 4))
    B = np.array([[[1.0], [5.0]]])
    C = np.ones((1, 2, 1))
    y = O.scalar_decay_scan(x, dt, np.zeros(4), B, C, np.zeros(4), np.zeros((4, 1, 1)))
    assert np.allclose(y[0, :, 0], [1.0, 1.0, 5.0, 5.0])


def test_convolution_last_column_is_the_current_token():
    u = np.array([[1.0], [10.0], [100.0]])
    st = {}
    big = 50.0                                                # silu(z) ~ z for large z
    out = O.conv_bias_silu(u * big, np.array([[0.0, 1.0]]), np.zeros(1), st)
    assert np.allclose(out[:, 0], u[:, 0] * big)
    out = O.conv_bias_silu(u * big, np.array([[1.0, 0.0]]), np.zeros(1), {})
    assert np.allclose(out[1:, 0], u[:-1, 0] * big) and out[0, 0] == 0.0
    assert np.allclose(st["tail"], [[100.0 * big]])


def test_grouped_rms_parts_are_normed_apart():
    y = np.array([[1.0, 1.0, 100.0, 100.0]])
    assert np.allclose(O.grouped_rms(y, 2, np.ones(4), 0.0), 1.0)
    assert not np.allclose(O.grouped_rms(y, 1, np.ones(4), 0.0), 1.0)


def test_rotation_half_pairs_first_dims_only():
    v = np.arange(1.0, 9.0).reshape(1, 1, 8)
    r = O.rotate(v, [1], {"base": 100.0, "dims": 4}, False)
    a0, a1 = 1.0, 100.0 ** -0.5
    assert np.allclose(r[0, 0, 4:], v[0, 0, 4:])
    assert np.allclose(r[0, 0, :4], [1 * np.cos(a0) - 3 * np.sin(a0), 2 * np.cos(a1) - 4 * np.sin(a1), 3 * np.cos(a0) + 1 * np.sin(a0), 4 * np.cos(a1) + 2 * np.sin(a1)])


def test_rotation_adjacent_pairs():
    v = np.arange(1.0, 5.0).reshape(1, 1, 4)
    r = O.rotate(v, [2], {"base": 100.0, "dims": 4}, True)
    a0, a1 = 2.0, 2.0 * 100.0 ** -0.5
    assert np.allclose(r[0, 0], [1 * np.cos(a0) - 2 * np.sin(a0), 2 * np.cos(a0) + 1 * np.sin(a0), 3 * np.cos(a1) - 4 * np.sin(a1), 4 * np.cos(a1) + 3 * np.sin(a1)])


def test_scaled_frequencies_ramp():
    rot = {"base": 100.0, "dims": 16, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    f, mag = O.rot_frequencies(rot)
    plain = 100.0 ** (-2.0 * np.arange(8) / 16)
    # dim(8 turns) = 0.42 -> lo 0; dim(1 turn) = 4.03 -> hi 5: pair 0 keeps its frequency, pairs 5.. are divided by the factor, a line between
    assert np.allclose(f[0], plain[0]) and np.allclose(f[5:], plain[5:] / 4.0)
    assert np.allclose(f[2], plain[2] / 4.0 * 0.4 + plain[2] * 0.6)
    assert np.isclose(mag, 0.1 * math.log(4.0) + 1.0)


def test_differential_attention_equal_maps_cancel_by_lambda():
    """both maps given the same queries and keys: a1 = a2, so o = (1 - lambda) a before the unit norm; with lambda < 1 the normed output is a / rms(a) (1 - diff)"""
    mx = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 3, "diff": 0.25, "rot": {"base": 10.0, "dims": 0}, "scale": 1.0}
    rng = np.random.default_rng(0)
    Wq, Wk = rng.standard_normal((2, 4)), rng.standard_normal((2, 4))
    W = {"q": np.concatenate([Wq, Wq]), "k": np.concatenate([Wk, Wk]), "v": rng.standard_normal((3, 4)), "q.b": np.zeros(4), "k.b": np.zeros(4), "v.b": np.zeros(3),
         "lq1": np.zeros(2), "lk1": np.zeros(2), "lq2": np.zeros(2), "lk2": np.zeros(2), "o": np.eye(3)}
    h = rng.standard_normal((5, 4))
    out = O.differential_attention(h, W, "", mx, 0.0, {}, list(range(5)))           # lambda = 1 - 1 + 0.25
    q, k, v = (h @ Wq.T)[:, None], (h @ Wk.T)[:, None], (h @ W["v"].T)[:, None]
    a = O.causal_softmax_attention(q, k, v, list(range(5)), 1.0)[:, 0]
    assert np.allclose(out, O.rms_unit(a, 0.0) * 0.75)


def test_latent_attention_equals_explicit_keys_and_values():
    mx = {"heads": 2, "dim": 3, "rot_dim": 2, "vdim": 4, "kv_rank": 5, "rot": {"base": 10.0, "dims": 2}, "scale": 0.7}
    rng = np.random.default_rng(1)
    W = {"q": rng.standard_normal((10, 6)), "dkv": rng.standard_normal((7, 6)), "dkv.norm": rng.standard_normal(5), "uk": rng.standard_normal((6, 5)),
         "uv": rng.standard_normal((8, 5)), "o": np.eye(8)}
    h = rng.standard_normal((4, 6))
    pos = list(range(4))
    whole = O.latent_attention(h, W, "", mx, 1e-5, {}, pos)
    st, parts = {}, []
    for t in range(4):
        parts.append(O.latent_attention(h[t:t + 1], W, "", mx, 1e-5, st, [t]))
    assert np.allclose(np.concatenate(parts), whole)
    assert st["C"].shape == (4, 5) and st["KR"].shape == (4, 2)                     # what a sequence keeps: the latent and one rotated key part
