"""GPU: the Putazen design through the library's own entry points (llama_decode on a llama_batch, llama_kv_cache_seq_rm, the
plain-generation scheduler, bin/trace_run) against the float64 oracle of tests/putazen_oracle.py, on small random models written to a
folder (config.json + model.safetensors) and loaded like any other model.

float32 contexts are compared at 2e-4 of the logits' spread, which is what makes a lost state or convolution tail, a walk that read
another walk's cache, a stream written from already-updated streams, a rotation pairing or a map read from the wrong key head show;
bfloat16 contexts at 6e-2.  Every schedule (whole prompt, portions, token by token, mixed batches, reused cells and slots) is compared
with the oracle AND, in float32, with the whole-prompt run."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests import putazen_oracle as O
from tests.putazen_configs import CONFIGS, drawn
from tests.test_gpu_rapisun import Served, row_err, spread, TOL32, TOL16

pytestmark = pytest.mark.gpu


def oracle_logits(cfg, W, toks):
    return O.forward(cfg, W, O.Sequence(cfg), list(toks))


def tokens(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def spotlight(cfg, W, special_token, fi=3, fj=5):
    """Random weights would hide a far key that is lost among hundreds.  This makes ONE key stand out in layer 0's first head (its first
    map, if it has two): the layer reads the streams with positive weights through a LayerNorm with weight 1 and bias 0; the head's query
    is a single unrotated coordinate that reads an input feature which is positive for all tokens, its key the same coordinate reading a
    feature that is negative for all tokens but `special_token`.  The special key's score is far above every other."""
    W = dict(W)
    E = W["embed"].copy()
    E[:, fi], E[:, fj] = 0.5, -0.5
    E[special_token, fj] = 0.5
    W["embed"] = E
    W["l0.hc1.in"] = np.abs(W["l0.hc1.in"])
    W["l0.norm1"], W["l0.norm1.b"] = np.ones_like(W["l0.norm1"]), np.zeros_like(W["l0.norm1.b"])
    mx = cfg["layers"][0]["mixer"]
    D = mx["dim"]
    if cfg["layers"][0]["type"] == "attention":
        assert mx["rot"]["dims"] < D
        for name, f in (("q", fi), ("k", fj)):
            M, b = W["l0.mix." + name].copy(), W["l0.mix.%s.b" % name].copy()
            M[:D, :], b[:D] = 0.0, 0.0
            M[D - 1, f] = 8.0
            W["l0.mix." + name], W["l0.mix.%s.b" % name] = M, b
    else:
        q, dkv, g, uk = W["l0.mix.q"].copy(), W["l0.mix.dkv"].copy(), W["l0.mix.dkv.norm"].copy(), W["l0.mix.uk"].copy()
        q[:D + mx["rot_dim"], :] = 0.0                     # head 0: unrotated coordinate 0 only, nothing in the rotated part
        q[0, fi] = 8.0
        dkv[0, :] = 0.0
        dkv[0, fj] = 4.0                                   # latent coordinate 0 carries the feature's sign through the unit RMS
        g[0] = 1.0
        uk[:D, :] = 0.0
        uk[0, 0] = 8.0
        W["l0.mix.q"], W["l0.mix.dkv"], W["l0.mix.dkv.norm"], W["l0.mix.uk"] = q, dkv, g, uk
    return W


# ---- each mechanism alone, float32 and bfloat16 -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["mamba_only", "diff_only", "latent_only", "walks", "one_layer_walk", "ones", "mixed_small"])
@pytest.mark.parametrize("float32", [True, False])
def test_whole_prompt_matches_oracle(tmp_path, name, float32):
    cfg = CONFIGS[name]()
    W = O.random_weights(cfg, 11)
    toks = tokens(cfg, 37, 1)
    ref = oracle_logits(cfg, W, toks)
    s = Served(tmp_path, cfg, W, float32=float32)
    got = s.feed(0, toks, [])
    s.close()
    assert row_err(got, ref).max() < (TOL32 if float32 else TOL16 * (1.5 if name in ("mixed_small", "walks") else 1.0))


@pytest.mark.parametrize("seed", range(10))
def test_drawn_configurations(tmp_path, seed):
    """configurations drawn from a seed (layer order, 1 to 6 streams, sizes that are odd, 1 or large, rotated dimensions from none to all with
    and without scaled frequencies, walks anywhere): a prompt long enough for the long-portion paths, whole and cut, in float32; whole in bfloat16"""
    cfg = drawn(100 + seed)
    W = O.random_weights(cfg, 200 + seed)
    toks = tokens(cfg, 280, 300 + seed)
    ref = oracle_logits(cfg, W, toks)
    # a drawn model may magnify rounding (a unit norm over a few nearly cancelling values, a difference of two nearly equal maps): how much
    # is measured on the oracle itself, as the answer to weights moved by 1e-7 of their size; the tolerances grow with it beyond a usual 15
    rng = np.random.default_rng(0)
    moved = {k: v * (1.0 + 1e-7 * rng.standard_normal(v.shape)) for k, v in W.items()}
    gain = max(1.0, float(np.median(row_err(oracle_logits(cfg, moved, toks[:80]), ref[:80])) / 1e-7) / 15.0)

    def close32(e):
        return np.quantile(e, 0.98) < TOL32 * gain and e.max() < 10 * TOL32 * gain
    s = Served(tmp_path / "a", cfg, W, n_ctx=900)
    whole = s.feed(0, toks, [])
    assert close32(row_err(whole, ref)), json.dumps(cfg)
    cut = s.feed(1, toks, [2, 131, 132, 260] + list(range(270, 280)))
    assert close32(row_err(cut, ref)) and close32(row_err(cut, whole)), json.dumps(cfg)
    s.close()
    s = Served(tmp_path / "b", cfg, W, float32=False, n_ctx=300)
    e = row_err(s.feed(0, toks, []), ref)
    assert np.median(e) < TOL16 * gain and np.quantile(e, 0.95) < 3 * TOL16 * gain, json.dumps(cfg)
    s.close()


def test_residual_stream_after_every_layer_run(tmp_path, monkeypatch):
    """the library's debugging dump (the sum of the streams) against the oracle's trace: one row block per layer RUN, walks included"""
    cfg = CONFIGS["mixed_small"]()
    W = O.random_weights(cfg, 31)
    toks = tokens(cfg, 19, 5)
    trace = []
    O.forward(cfg, W, O.Sequence(cfg), toks, trace)
    dump = tmp_path / "dump"
    dump.mkdir()
    monkeypatch.setenv("PIB_HYBRID_DUMP", str(dump))
    s = Served(tmp_path / "m", cfg, W)
    s.feed(0, toks, [])
    s.close()
    assert len(trace) == 8
    for i, ref in enumerate(trace):
        got = np.fromfile(dump / ("d0_l%d.f32" % i), "<f4").reshape(ref.shape)
        assert np.abs(got - ref).max() < 1e-4 * max(1.0, np.abs(ref).max()), "layer run %d" % i


# ---- prefill against token-by-token decoding, and portions down to two tokens ------------------------------------------------------------
@pytest.mark.parametrize("name", ["mixed_small", "mamba_only", "diff_only", "latent_only", "walks", "ones"])
def test_cuts_do_not_matter(tmp_path, name):
    cfg = CONFIGS[name]()
    W = O.random_weights(cfg, 12)
    toks = tokens(cfg, 41, 2)
    ref = oracle_logits(cfg, W, toks)
    s = Served(tmp_path, cfg, W)
    whole = s.feed(0, toks, [])
    schedules = {"token by token": range(1, 41), "twos": range(2, 41, 2), "mixed sizes": [2, 4, 5, 12, 14, 15, 17, 30, 32],
                 "prompt then decode": [20] + list(range(21, 41)), "one, then the rest": [1], "threes after two": range(2, 41, 3)}
    for i, (label, cuts) in enumerate(schedules.items()):
        got = s.feed(1 + i, toks, cuts)
        s.end(1 + i)
        assert row_err(got, ref).max() < TOL32, label
        assert row_err(got, whole).max() < TOL32, label
    s.close()


def test_cuts_do_not_matter_bfloat16(tmp_path):
    cfg = CONFIGS["wide_heads"]()
    W = O.random_weights(cfg, 13)
    toks = tokens(cfg, 33, 3)
    ref = oracle_logits(cfg, W, toks)
    s = Served(tmp_path, cfg, W, float32=False)
    for i, cuts in enumerate([[], range(1, 33), [2, 4, 11, 13, 29]]):
        got = s.feed(i, toks, cuts)
        assert row_err(got, ref).max() < TOL16
    s.close()


# ---- the first tokens of a sequence: shorter than the convolution's reach, empty states and caches ------------------------------------------
def test_first_tokens(tmp_path):
    cfg = CONFIGS["mixed_small"]()
    W = O.random_weights(cfg, 25)
    s = Served(tmp_path, cfg, W)
    for r, n in enumerate([1, 2, 3, 4]):
        toks = tokens(cfg, n, 40 + r)
        ref = oracle_logits(cfg, W, toks)
        assert row_err(s.feed(r, toks, []), ref).max() < TOL32
    for r in range(4):
        s.end(r)
    # the same slots again, one token at a time: nothing of the earlier owners may be left in the tails or matrices
    for r, n in enumerate([3, 1, 4, 2]):
        toks = tokens(cfg, n, 50 + r)
        ref = oracle_logits(cfg, W, toks)
        assert row_err(s.feed(r, toks, range(1, n)), ref).max() < TOL32
    s.close()


# ---- keys far away: one that stands out, and many among hundreds; in prompts and in decoding ---------------------------------------------------
@pytest.mark.parametrize("kind", ["attention", "latent_attention"])
def test_one_far_key_stands_out(tmp_path, kind):
    """one early key carries the first head's output for every later token: 400 tokens on it must still be read, whole, in portions whose
    edges sit at 63 / 64 / 65 and in decoded tokens, and another token in its place must change the answer"""
    cfg = CONFIGS["far_keys"]()
    cfg["layers"] = [l for l in cfg["layers"] if l["type"] == kind]
    W = spotlight(cfg, O.random_weights(cfg, 26), cfg["vocab"] - 1)
    toks = np.random.default_rng(7).integers(0, cfg["vocab"] - 1, 420).tolist()
    special = 9
    toks[special] = cfg["vocab"] - 1
    ref = oracle_logits(cfg, W, toks)
    other = list(toks)
    other[special] = 0
    assert np.median(row_err(oracle_logits(cfg, W, other), ref)[special + 1:]) > 0.02
    s = Served(tmp_path, cfg, W, n_ctx=1400)
    assert row_err(s.feed(0, toks, []), ref).max() < TOL32
    assert row_err(s.feed(1, toks, [special, special + 1, 63, 64, 65, 128, 191, 193] + list(range(380, 420))), ref).max() < TOL32
    s.close()
    s = Served(tmp_path, cfg, W, float32=False, n_ctx=900)               # served mode: the long portion runs as tensor-core matmuls
    TOL = 0.1                                                            # one key carries whole outputs here: rounding shows more than with random weights
    assert row_err(s.feed(0, toks, []), ref).max() < TOL
    assert row_err(s.feed(1, toks, [200] + list(range(400, 420))), ref).max() < TOL
    s.close()


def test_far_keys_among_hundreds(tmp_path):
    cfg = CONFIGS["far_keys"]()
    W = O.random_weights(cfg, 16)
    toks = tokens(cfg, 300, 6)
    ref = oracle_logits(cfg, W, toks)
    s = Served(tmp_path, cfg, W, n_ctx=640)
    whole = s.feed(0, toks, [])
    assert row_err(whole, ref).max() < TOL32
    got = s.feed(1, toks, [64, 128, 191, 192, 193, 194, 258, 259, 260, 261, 262] + list(range(263, 300)))
    assert row_err(got, ref).max() < TOL32
    s.close()


def test_long_prompt_carries_the_recurrent_state(tmp_path):
    """700 tokens through state-space layers with slow and fast decays: whole, as two long portions of which the second starts from the
    matrices and convolution tails the first one left, and as portions of 100"""
    cfg = CONFIGS["mamba_only"]()
    W = O.random_weights(cfg, 27)
    W["l0.mix.A_log"] = O.bf16_round(np.linspace(-6.0, 1.0, W["l0.mix.A_log"].size))
    toks = tokens(cfg, 700, 14)
    ref = oracle_logits(cfg, W, toks)
    s = Served(tmp_path, cfg, W, n_ctx=2200)
    whole = s.feed(0, toks, [])
    assert row_err(whole, ref).max() < TOL32
    assert row_err(s.feed(1, toks, [300, 650] + list(range(651, 700))), ref).max() < TOL32
    plain = s.feed(2, toks, range(100, 700, 100))
    assert row_err(plain, ref).max() < TOL32 and row_err(plain, whole).max() < TOL32
    s.close()


def test_lambda_and_stream_weights_show(tmp_path):
    """the oracle with lambda's learned part, the streams' mixing or the gate's place changed differs by far more than the tolerance, so
    the comparison with the library can see each of them"""
    cfg = CONFIGS["mixed_small"]()
    W = O.random_weights(cfg, 28)
    toks = tokens(cfg, 30, 9)
    ref = oracle_logits(cfg, W, toks)
    for name in ("l0.mix.lq1", "l1.hc1.mix", "l2.hc2.out", "l3.mix.D", "l1.mix.conv.b"):
        W2 = dict(W)
        W2[name] = W[name].T.copy() if name.endswith(".mix") else W[name] * 1.5
        assert np.median(row_err(oracle_logits(cfg, W2, toks), ref)) > 20 * TOL32, name
    s = Served(tmp_path, cfg, W)
    assert row_err(s.feed(0, toks, []), ref).max() < TOL32
    assert row_err(s.feed(1, toks, range(1, 30)), ref).max() < TOL32
    s.close()


# ---- batches of unequal requests against each alone; cells and slots freed and used again -------------------------------------------------
def test_mixed_batches_and_reuse(tmp_path):
    cfg = CONFIGS["mixed_small"]()
    W = O.random_weights(cfg, 17)
    lens = [45, 9, 30, 2, 17, 26, 1, 38]
    reqs = [tokens(cfg, n, 20 + i) for i, n in enumerate(lens)]
    refs = [oracle_logits(cfg, W, t) for t in reqs]
    # 3 slots and 120 cells for 168 tokens: both have to come back and be used again, cells out of order
    s = Served(tmp_path, cfg, W, n_ctx=120, slots=3)
    rng = np.random.default_rng(7)
    got = [[] for _ in reqs]
    at = [0] * len(reqs)
    live, nxt = [], 0
    while nxt < len(reqs) or live:
        while nxt < len(reqs) and len(live) < 3:
            live.append(nxt)
            nxt += 1
        entries = []
        for r in live:
            left = len(reqs[r]) - at[r]
            n = min(left, int(rng.choice([1, 1, 2, 3, 7, 16])))
            if sum(len(t) for _, t in entries) + n > 120 - sum(at[q] for q in live):
                continue
            entries.append((r, reqs[r][at[r]:at[r] + n]))
        assert entries
        out = s.step(entries)
        for r, t in entries:
            got[r].append(out[r])
            at[r] += len(t)
        for r in list(live):
            if at[r] == len(reqs[r]):
                s.end(r)
                live.remove(r)
    for r in range(len(reqs)):
        assert row_err(np.concatenate(got[r]), refs[r]).max() < TOL32, "request %d" % r
    used, _ = s.ctx.kv_view()
    assert used == 0 and s.ctx.L.llama_pib_state_slots_free(s.ctx.ctx) == 3
    s.close()


# ---- long decoding, and greedy generation through the scheduler's entry point ----------------------------------------------------------------
def test_long_decoding(tmp_path):
    cfg = CONFIGS["mixed_small"]()
    W = O.random_weights(cfg, 19)
    toks = tokens(cfg, 150, 8)
    ref = oracle_logits(cfg, W, toks)
    s = Served(tmp_path, cfg, W)
    got = s.feed(0, toks, [6] + list(range(7, 150)))
    s.close()
    e = row_err(got, ref)
    assert e.max() < TOL32 and e[-20:].max() < TOL32


def test_long_portions_take_the_matmul_attention(tmp_path):
    """served mode: portions of 128 tokens and more of an attention whose head sizes are multiples of 8 run as tensor-core matmuls (one
    problem per key / value head and map; the latent attention over the cached latents); shorter portions and decoded tokens stay with the
    per-token kernels.  Both against the oracle, against each other, and mixed in one batch"""
    cfg = CONFIGS["wide_heads"]()
    W = O.random_weights(cfg, 23)
    toks, other = tokens(cfg, 450, 10), tokens(cfg, 60, 11)
    ref, ref_o = oracle_logits(cfg, W, toks), oracle_logits(cfg, W, other)
    s = Served(tmp_path, cfg, W, float32=False, n_ctx=1600)
    whole = s.feed(0, toks, [])                                            # one portion of 450
    small = s.feed(1, toks, range(100, 450, 100))                          # portions of 100: the per-token kernels
    cut = s.feed(2, toks, [130, 131, 300, 449])                            # 130 (matmul) + 1 + 169 (matmul) + 149 (matmul) + 1
    assert row_err(whole, ref).max() < TOL16 and row_err(small, ref).max() < TOL16 and row_err(cut, ref).max() < TOL16
    assert row_err(whole, small).max() < TOL16 and row_err(cut, small).max() < TOL16
    for r in range(3):
        s.end(r)
    a = s.step([(3, toks[:200]), (4, other[:59])])                         # a long portion beside a short one and a decoded token in ONE batch
    b = s.step([(4, other[59:]), (3, toks[200:])])
    assert row_err(np.concatenate([a[3], b[3]]), ref).max() < TOL16
    assert row_err(np.concatenate([a[4], b[4]]), ref_o).max() < TOL16
    s.close()
    s = Served(tmp_path, cfg, W, float32=True, n_ctx=600)                  # float32 contexts never take it
    assert row_err(s.feed(0, toks, []), ref).max() < TOL32
    s.close()


@pytest.mark.parametrize("float32", [True, False])
def test_medium_model_long_prompt_cuts_and_batches(tmp_path, float32):
    """a wider model with its layers in another order: a long prompt whole, cut (long portions, short ones, decoded tokens), and two
    requests sharing batches -- both compute types"""
    cfg = CONFIGS["medium"]()
    W = O.random_weights(cfg, 33)
    toks, other = tokens(cfg, 330, 12), tokens(cfg, 140, 13)
    ref, ref_o = oracle_logits(cfg, W, toks), oracle_logits(cfg, W, other)
    tol = TOL32 if float32 else TOL16
    s = Served(tmp_path, cfg, W, float32=float32, n_ctx=1400)
    assert row_err(s.feed(0, toks, []), ref).max() < tol
    assert row_err(s.feed(1, toks, [150, 151, 153, 290] + list(range(300, 330))), ref).max() < tol
    s.end(0)
    s.end(1)
    a = s.step([(2, toks[:129]), (3, other[:7])])
    b = s.step([(3, other[7:139]), (2, toks[129:131])])
    c = s.step([(2, toks[131:]), (3, other[139:])])
    assert row_err(np.concatenate([a[2], b[2], c[2]]), ref).max() < tol
    assert row_err(np.concatenate([a[3], b[3], c[3]]), ref_o).max() < tol
    s.close()


def test_decode_steps_around_growing_prompts(tmp_path):
    """single-token steps are replayed from captured graphs; a later, longer prompt makes the context grow its buffers, and the steps
    after it must not run on the old ones"""
    cfg = CONFIGS["mixed_small"]()
    W = O.random_weights(cfg, 22)
    s = Served(tmp_path, cfg, W, n_ctx=512)
    for r, n_prompt in enumerate([5, 40, 18, 130, 70]):
        toks = tokens(cfg, n_prompt + 9, 30 + r)
        ref = oracle_logits(cfg, W, toks)
        got = s.feed(r, toks, [n_prompt] + list(range(n_prompt + 1, n_prompt + 9)))
        s.end(r)
        assert row_err(got, ref).max() < TOL32, "request %d" % r
    s.close()


@pytest.mark.parametrize("float32", [True, False])
def test_greedy_generation_through_the_scheduler(tmp_path, float32):
    from pipeinfer_b200 import llama
    cfg = CONFIGS["mixed_small"]()
    W = O.random_weights(cfg, 21)
    O.write_model(str(tmp_path), cfg, W)
    prompt = tokens(cfg, 9, 9)
    ctx = llama.Context(model_dir=str(tmp_path), n_ctx=128, max_seq=4, float32=float32)
    out, res, _ = llama.plain_generate(ctx, prompt, 24)
    ctx.close()
    assert len(out) == 24
    # the oracle follows the library's tokens; wherever its own choice differs the two best logits must be a near tie
    seq = O.Sequence(cfg)
    lg = O.forward(cfg, W, seq, prompt)[-1]
    for t in out:
        best = int(np.argmax(lg))
        if best != t:
            assert lg[best] - lg[t] < (1e-3 if float32 else 0.15) * spread(lg), "token %d instead of %d" % (t, best)
        lg = O.forward(cfg, W, seq, [t])[-1]


def test_trace_runner_replays_steps(tmp_path):
    """bin/trace_run as a user starts it: JSON steps on standard input (portions beside single tokens, requests ending, more requests
    than state slots over time, cells for the live ones only), logits files out, one 'done' line per step"""
    cfg = CONFIGS["mixed_small"]()
    W = O.random_weights(cfg, 24)
    model = tmp_path / "model"
    O.write_model(str(model), cfg, W)
    reqs = {"a": tokens(cfg, 50, 1), "b": tokens(cfg, 21, 2), "c": tokens(cfg, 33, 3), "d": tokens(cfg, 2, 4), "e": tokens(cfg, 40, 5)}
    refs = {k: oracle_logits(cfg, W, v) for k, v in reqs.items()}
    plan = [[("a", 30), ("b", 2)], [("a", 1), ("b", 19), ("c", 7)], [("a", 19), ("c", 1)], [("c", 25), ("d", 2)], [("e", 38)], [("e", 1)], [("e", 1)]]
    at, steps, wanted = {k: 0 for k in reqs}, [], []
    for n, step in enumerate(plan):
        entries, end, rows = [], [], []
        for rid, cnt in step:
            lo, hi = at[rid], at[rid] + cnt
            want = sorted({0, cnt - 1}) if cnt > 1 else [0]
            entries.append({"id": rid, "tokens": reqs[rid][lo:hi], "want": want})
            rows += [(rid, lo + w) for w in want]
            at[rid] = hi
            if hi == len(reqs[rid]):
                end.append(rid)
        steps.append(json.dumps({"step": n, "entries": entries, "end": end}))
        wanted.append(rows)
    root = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
    for dtype, tol in (("float32", TOL32), ("bfloat16", 1.5 * TOL16)):
        out = tmp_path / ("out_" + dtype)
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "128", "--slots", "3"], input="\n".join(steps) + "\n", capture_output=True, text=True, timeout=300)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.split("\n") if l.startswith("done")] == ["done %d" % json.loads(s)["step"] for s in steps]
        for n, rows in enumerate(wanted):
            got = np.fromfile(out / ("%d.f32" % n), "<f4").reshape(len(rows), -1)
            ref = np.stack([refs[rid][i] for rid, i in rows])
            assert got.shape == ref.shape and np.isfinite(got).all()
            assert row_err(got, ref).max() < tol, (dtype, n)
