"""CPU: the float64 restatement of the Lulenex design agrees with itself over cuts (whole prompt, portions, token by token) for every test
configuration, and its parts do what their definitions say on inputs whose answer is known."""
import numpy as np
import pytest

from tests import lulenex_oracle as O
from tests.lulenex_configs import CONFIGS


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


def test_layer_runs_order():
    cfg = CONFIGS["mixed_small"]()
    assert [(i, r) for i, r, _ in O.layer_runs(cfg)] == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (3, None), (4, None)]
    assert [o for _, _, o in O.layer_runs(cfg)] == [False, True, False, True, False, False, False]


def test_xielu_branches():
    z = np.array([-2.0, 0.0, 3.0])
    p, q = 0.3, -0.4
    ap, aq = np.log1p(np.exp(p)), 0.5 + np.log1p(np.exp(q))
    assert np.allclose(O.xielu(z, p, q), [aq * (np.exp(-2.0) - 1 + 2.0) - 1.0, 0.0, ap * 9.0 + 1.5])


def test_chunk_mask_and_sink():
    # one head, keys = values = unit vectors: a token reads only its own chunk, and the sink takes its share without adding a value
    k = np.eye(6)[:, None, :]
    q = np.zeros((6, 1, 6))
    out = O.chunk_softmax_attention(q, k, k, list(range(6)), 4, 1.0, np.array([0.0]))
    assert np.allclose(out[3, 0], [0.2, 0.2, 0.2, 0.2, 0, 0]) and np.allclose(out[4, 0], [0, 0, 0, 0, 0.5, 0]) and np.allclose(out[5, 0], [0, 0, 0, 0, 1 / 3, 1 / 3])


def test_rotation_pairs_first_dims_only():
    v = np.arange(1.0, 9.0).reshape(1, 1, 8)
    r = O.rotate_half(v, [1], 4, 100.0)
    a0, a1 = 1.0, 100.0 ** -0.5
    assert np.allclose(r[0, 0, 4:], v[0, 0, 4:])
    assert np.allclose(r[0, 0, :4], [1 * np.cos(a0) - 3 * np.sin(a0), 2 * np.cos(a1) - 4 * np.sin(a1), 3 * np.cos(a0) + 1 * np.sin(a0), 4 * np.cos(a1) + 2 * np.sin(a1)])
