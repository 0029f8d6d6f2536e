"""GPU: the Lulenex design through the library's own entry points (llama_decode on a llama_batch, llama_kv_cache_seq_rm, the
plain-generation scheduler, bin/trace_run) against the float64 oracle of tests/lulenex_oracle.py, on small random models written to a
folder (config.json + model.safetensors) and loaded like any other model.

float32 contexts are compared at 2e-4 of the logits' spread, which is what makes a chunk one token off, a lost state, a shift row or a
convolution tail that was not carried, a walk that read another walk's cache or a missing sink show; bfloat16 contexts at 6e-2.  Every
schedule (whole prompt, portions, token by token, mixed batches, reused cells and slots) is compared with the oracle AND, in float32, with
the whole-prompt run."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests import lulenex_oracle as O
from tests.lulenex_configs import CONFIGS, drawn
from tests.test_gpu_rapisun import Served, row_err, spread, TOL32, TOL16

pytestmark = pytest.mark.gpu


def oracle_logits(cfg, W, toks):
    return O.forward(cfg, W, O.Sequence(cfg), list(toks))


def tokens(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def spotlight(cfg, W, special_token, fi=3, fj=5):
    """Random weights would hide a key that is wrongly cut off (or let in) among hundreds.  This makes ONE key stand out in layer 0's first
    softmax head: the head's query is a single unrotated coordinate that reads an input feature which is positive for all tokens, the
    key the same coordinate reading a feature that is negative for all tokens but `special_token`; no token shift, no biases.  After the
    unit norms the score is +scale * dim for the special key and -scale * dim for every other, and the special key's VALUE (the key as
    projected) has the opposite sign on that coordinate."""
    W = dict(W)
    E = W["embed"].copy()
    E[:, fi], E[:, fj] = 0.5, -0.5
    E[special_token, fj] = 0.5
    W["embed"] = E
    W["l0.shift"] = np.zeros_like(W["l0.shift"])
    D = cfg["layers"][0]["mixer"]["left"]["dim"]
    for name, f in (("q", fi), ("k", fj)):
        M, b = W["l0.mix.left." + name].copy(), W["l0.mix.left.%s.b" % name].copy()
        M[:D, :], b[:D] = 0.0, 0.0
        M[D - 1, f] = 4.0
        W["l0.mix.left." + name], W["l0.mix.left.%s.b" % name] = M, b
    Wo = W["l0.mix.left.o"].copy()
    Wo[:, D - 1] *= 8.0                                # the coordinate that flips reaches the stream with some weight
    W["l0.mix.left.o"] = Wo
    return W


# ---- each mechanism alone, float32 and bfloat16 -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["ssm_only", "softmax_mostly", "linear_mostly", "walks", "one_layer_walk", "ones", "mixed_small"])
@pytest.mark.parametrize("float32", [True, False])
def test_whole_prompt_matches_oracle(tmp_path, name, float32):
    cfg = CONFIGS[name]()
    W = O.random_weights(cfg, 11)
    toks = tokens(cfg, 37, 1)
    ref = oracle_logits(cfg, W, toks)
    s = Served(tmp_path, cfg, W, float32=float32)
    got = s.feed(0, toks, [])
    s.close()
    # seven layer runs on a width of 80: the bfloat16 operands' rounding adds up to a little more than in the other configurations
    assert row_err(got, ref).max() < (TOL32 if float32 else TOL16 * (1.5 if name == "mixed_small" else 1.0))


def test_sizes_the_configuration_omits_come_from_tensor_shapes(tmp_path):
    cfg = CONFIGS["mixed_small"]()
    W = O.random_weights(cfg, 29)
    toks = tokens(cfg, 21, 15)
    ref = oracle_logits(cfg, W, toks)
    bare = copy.deepcopy(cfg)
    for l in bare["layers"]:
        if l["type"] == "mamba1":
            l["mixer"] = {}
        else:
            for k in ("heads", "kv_heads", "dim", "vdim"):
                l["mixer"]["left"].pop(k)
            for k in ("heads", "dim", "vdim"):
                l["mixer"]["right"].pop(k)
        if l["mlp"]:
            l["mlp"] = {"kind": "dense"}
    s = Served(tmp_path, bare, W)
    got = s.feed(0, toks, [5])
    s.close()
    assert row_err(got, ref).max() < TOL32


@pytest.mark.parametrize("seed", range(8))
def test_drawn_configurations(tmp_path, seed):
    """configurations drawn from a seed (layer order, sizes that are odd, 1 or large, rotated dimensions from none to all, chunks from 1 to longer
    than the prompt, walks anywhere): a prompt long enough for the long-segment paths, whole and cut, in float32; whole in bfloat16"""
    cfg = drawn(100 + seed)
    W = O.random_weights(cfg, 200 + seed)
    toks = tokens(cfg, 280, 300 + seed)
    ref = oracle_logits(cfg, W, toks)
    s = Served(tmp_path / "a", cfg, W, n_ctx=900)
    assert row_err(s.feed(0, toks, []), ref).max() < TOL32, json.dumps(cfg)
    assert row_err(s.feed(1, toks, [2, 131, 132, 260] + list(range(270, 280))), ref).max() < TOL32, json.dumps(cfg)
    s.close()
    s = Served(tmp_path / "b", cfg, W, float32=False, n_ctx=300)
    assert row_err(s.feed(0, toks, []), ref).max() < 2 * TOL16, json.dumps(cfg)
    s.close()


def test_residual_stream_after_every_layer_run(tmp_path, monkeypatch):
    """the library's debugging dump against the oracle's trace: one row block per layer RUN, walks included"""
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
    assert len(trace) == 7
    for i, ref in enumerate(trace):
        got = np.fromfile(dump / ("d0_l%d.f32" % i), "<f4").reshape(ref.shape)
        assert np.abs(got - ref).max() < 1e-4 * max(1.0, np.abs(ref).max()), "layer run %d" % i


# ---- prefill against token-by-token decoding, and portions down to two tokens ------------------------------------------------------------
@pytest.mark.parametrize("name", ["mixed_small", "ssm_only", "softmax_mostly", "linear_mostly", "walks", "ones"])
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


# ---- the first tokens of a sequence: no previous token, shorter than the convolution's reach, empty states ------------------------------------
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
    # the same slots again, one token at a time: nothing of the earlier owners may be left in the shift rows, tails or matrices
    for r, n in enumerate([3, 1, 4, 2]):
        toks = tokens(cfg, n, 50 + r)
        ref = oracle_logits(cfg, W, toks)
        assert row_err(s.feed(r, toks, range(1, n)), ref).max() < TOL32
    s.close()


# ---- chunks: keys just inside and just outside, in prompts and in decoding -------------------------------------------------------------------
def test_chunk_edges_prompt_and_decode(tmp_path):
    cfg = CONFIGS["softmax_mostly"]()
    size = cfg["layers"][0]["mixer"]["left"]["mask"]["size"]
    W = O.random_weights(cfg, 14)
    toks = tokens(cfg, 3 * size + 2, 4)
    ref = oracle_logits(cfg, W, toks)
    for d in (-1, 1):                              # the oracle with the chunks one off differs: the comparison below can see it
        c2 = copy.deepcopy(cfg)
        for l in c2["layers"]:
            l["mixer"]["left"]["mask"]["size"] += d
        assert np.median(row_err(oracle_logits(c2, W, toks), ref)[size + 1:]) > 50 * TOL32
    s = Served(tmp_path, cfg, W)
    assert row_err(s.feed(0, toks, []), ref).max() < TOL32
    assert row_err(s.feed(1, toks, range(1, len(toks))), ref).max() < TOL32
    # portions that end and start at, one before and one after a chunk's edge
    assert row_err(s.feed(2, toks, [size - 1, size, size + 1, 2 * size - 1, 2 * size + 1]), ref).max() < TOL32
    s.close()


def test_one_key_at_the_chunks_edge(tmp_path):
    """one key made to stand out early in a chunk of 260: the chunk's last position must still see it, the next chunk's first must not.
    In a prompt, and decoded token by token."""
    cfg = CONFIGS["far_keys"]()
    cfg["layers"] = cfg["layers"][:1]
    size = cfg["layers"][0]["mixer"]["left"]["mask"]["size"]
    W = spotlight(cfg, O.random_weights(cfg, 26), cfg["vocab"] - 1)
    toks = np.random.default_rng(7).integers(0, cfg["vocab"] - 1, 2 * size + 30).tolist()
    special = size + 17
    toks[special] = cfg["vocab"] - 1
    ref = oracle_logits(cfg, W, toks)
    edge = 2 * size - 1                                # the last position of the special key's chunk
    for d, at in ((1, edge + 1), (-1, edge - 1)):      # chunks one longer: position 2 size would still see it; one shorter: position 2 size - 2 opens a chunk
        c2 = copy.deepcopy(cfg)
        c2["layers"][0]["mixer"]["left"]["mask"]["size"] = size + d
        assert row_err(oracle_logits(c2, W, toks), ref)[at:at + 3].max() > 0.3
    s = Served(tmp_path, cfg, W, n_ctx=2048)
    assert row_err(s.feed(0, toks, []), ref).max() < TOL32
    assert row_err(s.feed(1, toks, [edge - 1] + list(range(edge, len(toks)))), ref).max() < TOL32
    assert row_err(s.feed(2, toks, [special, special + 1, edge, edge + 2]), ref).max() < TOL32   # portions that start at the key, at the edge, and end just behind it
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


def test_heavy_sink_takes_its_share(tmp_path):
    """sinks large enough to take most of the weight: leaving them out (or scaling them) would change every output"""
    cfg = CONFIGS["softmax_mostly"]()
    W = O.random_weights(cfg, 18)
    for i in range(2):
        W["l%d.mix.left.sink" % i] = O.bf16_round(np.full_like(W["l%d.mix.left.sink" % i], 3.0) + 0.5 * np.arange(W["l%d.mix.left.sink" % i].size))
    toks = tokens(cfg, 30, 9)
    ref = oracle_logits(cfg, W, toks)
    W0 = dict(W)
    for i in range(2):
        W0["l%d.mix.left.sink" % i] = np.full_like(W["l%d.mix.left.sink" % i], -30.0)
    assert np.median(row_err(oracle_logits(cfg, W0, toks), ref)) > 100 * TOL32
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
    """served mode: portions of 128 tokens and more of a softmax branch whose head size is a multiple of 8 run as tensor-core matmuls
    (scores per key / value head, chunk-masked softmax with the sink, weighted sums); shorter portions and decoded tokens stay with the
    per-token kernel.  Both against the oracle, against each other, and mixed in one batch"""
    cfg = CONFIGS["wide_heads"]()
    size = cfg["layers"][0]["mixer"]["left"]["mask"]["size"]
    W = spotlight(cfg, O.random_weights(cfg, 23), cfg["vocab"] - 1)
    toks, other = np.random.default_rng(10).integers(0, cfg["vocab"] - 1, 450).tolist(), tokens(cfg, 60, 11)
    toks[size + 20] = cfg["vocab"] - 1                                     # a key that stands out: its chunk ends inside the long portions
    ref, ref_o = oracle_logits(cfg, W, toks), oracle_logits(cfg, W, other)
    c2 = copy.deepcopy(cfg)
    c2["layers"][0]["mixer"]["left"]["mask"]["size"] = size + 1
    assert row_err(oracle_logits(c2, W, toks), ref)[2 * size:2 * size + 3].max() > 0.3
    TOL = 0.1                                                              # one key carries whole outputs here: rounding shows more than with random weights
    s = Served(tmp_path, cfg, W, float32=False, n_ctx=1600)
    whole = s.feed(0, toks, [])                                            # one portion of 450, chunks of 150 and 37 inside
    small = s.feed(1, toks, range(100, 450, 100))                          # portions of 100: the per-token kernel
    cut = s.feed(2, toks, [130, 131, 300, 449])                            # 130 (matmul) + 1 + 169 (matmul) + 149 (matmul) + 1
    assert row_err(whole, ref).max() < TOL and row_err(small, ref).max() < TOL and row_err(cut, ref).max() < TOL
    assert row_err(whole, small).max() < TOL and row_err(cut, small).max() < TOL
    for r in range(3):
        s.end(r)
    a = s.step([(3, toks[:200]), (4, other[:59])])                         # a long portion beside a short one and a decoded token in ONE batch
    b = s.step([(4, other[59:]), (3, toks[200:])])
    assert row_err(np.concatenate([a[3], b[3]]), ref).max() < TOL
    assert row_err(np.concatenate([a[4], b[4]]), ref_o).max() < TOL
    s.close()
    s = Served(tmp_path, cfg, W, float32=True, n_ctx=600)                  # float32 contexts never take it
    assert row_err(s.feed(0, toks, []), ref).max() < TOL32
    s.close()


@pytest.mark.parametrize("float32", [True, False])
def test_medium_model_long_prompt_cuts_and_batches(tmp_path, float32):
    """a wider model with its layers in another order: a prompt over several chunks whole, cut (long portions, short ones, decoded tokens),
    and two requests sharing batches -- both compute types"""
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


def test_long_segment_walks_the_linear_branch_in_parts(tmp_path):
    """a batch that is one segment of 256 tokens or more walks the constant-decay recurrence in several parts at once (each part from zeros,
    then the matrix in front of it is added to its outputs); shorter portions and batches of several requests take the plain walk.  Decays from
    0.2 to exactly 1; a second long portion starts from the matrix the first one left, and decoding goes on from the combined matrix."""
    cfg = CONFIGS["linear_mostly"]()
    W = O.random_weights(cfg, 27)
    toks = tokens(cfg, 700, 14)
    ref = oracle_logits(cfg, W, toks)
    s = Served(tmp_path, cfg, W, n_ctx=2200)
    whole = s.feed(0, toks, [])                                                    # 8 parts
    assert row_err(whole, ref).max() < TOL32
    assert row_err(s.feed(1, toks, [300, 650] + list(range(651, 700))), ref).max() < TOL32      # 5 parts, 6 parts behind them, decoded tokens
    plain = s.feed(2, toks, range(100, 700, 100))                                  # portions of 100: the plain walk
    assert row_err(plain, ref).max() < TOL32 and row_err(plain, whole).max() < TOL32
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
    for dtype, tol in (("float32", TOL32), ("bfloat16", TOL16)):
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
