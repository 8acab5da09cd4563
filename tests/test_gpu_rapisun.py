"""GPU: the Rapisun design through the library's own entry points (llama_decode on a llama_batch, llama_kv_cache_seq_rm, the
plain-generation scheduler) against the float64 oracle of tests/rapisun_oracle.py, on small random models written to a folder
(config.json + model.safetensors) and loaded like any other model.

float32 contexts are compared at 2e-4 of the logits' spread (measured: a few 1e-6), which is what makes a window one token off, a
lost state, a missing sink or a wrong cell show; bfloat16 contexts at 6e-2.  Every schedule (whole prompt, portions, token by
token, mixed batches, reused cells and slots) is compared with the oracle AND, in float32, with the whole-prompt run."""
import copy

import numpy as np
import pytest

from tests import rapisun_oracle as O
from tests.rapisun_configs import CONFIGS

pytestmark = pytest.mark.gpu

TOL32, TOL16 = 2e-4, 6e-2


def spread(ref):
    return float(np.sqrt(((ref - ref.mean(-1, keepdims=True)) ** 2).mean()))


def row_err(got, ref):
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / spread(ref)


class Served:
    """one model folder + one context"""

    def __init__(self, tmp_path, cfg, W, float32=True, n_ctx=256, slots=4):
        from pipeinfer_b200 import llama
        O.write_model(str(tmp_path), cfg, W)
        self.ctx = llama.Context(model_dir=str(tmp_path), n_ctx=n_ctx, max_seq=32, float32=float32, state_slots=slots)
        self.fed = {}

    def step(self, entries):
        """entries: [(seq, tokens)]; returns {seq: logits of its tokens}"""
        toks, pos, seqs, spans = [], [], [], {}
        for s, t in entries:
            spans[s] = (len(toks), len(toks) + len(t))
            p0 = self.fed.get(s, 0)
            toks += list(t)
            pos += list(range(p0, p0 + len(t)))
            seqs += [[s]] * len(t)
            self.fed[s] = p0 + len(t)
        rc, lg = self.ctx.decode(toks, pos, seqs)
        assert rc == 0, self.ctx.L.pib_last_error().decode()
        return {s: lg[a:b] for s, (a, b) in spans.items()}

    def end(self, s):
        self.ctx.seq_rm(s, -1, -1)
        self.fed.pop(s, None)

    def feed(self, s, toks, cuts):
        """one sequence alone, cut at `cuts`"""
        out, a = [], 0
        for b in list(cuts) + [len(toks)]:
            if b > a:
                out.append(self.step([(s, toks[a:b])])[s])
            a = b
        return np.concatenate(out)

    def close(self):
        self.ctx.close()


def oracle_logits(cfg, W, toks):
    return O.forward(cfg, W, O.Sequence(cfg), list(toks))


def tokens(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


# ---- each mechanism alone, float32 and bfloat16 -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["attention_only", "recurrent_only", "experts_only", "partial_rotation", "ones", "mixed_small"])
@pytest.mark.parametrize("float32", [True, False])
def test_whole_prompt_matches_oracle(tmp_path, name, float32):
    cfg = CONFIGS[name]()
    W = O.random_weights(cfg, 11)
    toks = tokens(cfg, 37, 1)
    ref = oracle_logits(cfg, W, toks)
    s = Served(tmp_path, cfg, W, float32=float32)
    got = s.feed(0, toks, [])
    s.close()
    assert row_err(got, ref).max() < (TOL32 if float32 else TOL16)


# ---- prefill against token-by-token decoding, and portions down to two tokens ------------------------------------------------------------
@pytest.mark.parametrize("name", ["mixed_small", "recurrent_only", "ones"])
def test_cuts_do_not_matter(tmp_path, name):
    cfg = CONFIGS[name]()
    W = O.random_weights(cfg, 12)
    toks = tokens(cfg, 41, 2)
    ref = oracle_logits(cfg, W, toks)
    s = Served(tmp_path, cfg, W)
    whole = s.feed(0, toks, [])
    schedules = {"token by token": range(1, 41), "twos": range(2, 41, 2), "mixed sizes": [2, 4, 5, 12, 14, 15, 17, 30, 32],
                 "prompt then decode": [20] + list(range(21, 41)), "one, then the rest": [1]}
    for i, (label, cuts) in enumerate(schedules.items()):
        got = s.feed(1 + i, toks, cuts)
        s.end(1 + i)
        assert row_err(got, ref).max() < TOL32, label
        assert row_err(got, whole).max() < TOL32, label
    s.close()


def test_cuts_do_not_matter_bfloat16(tmp_path):
    cfg = CONFIGS["mixed_small"]()
    W = O.random_weights(cfg, 13)
    toks = tokens(cfg, 33, 3)
    ref = oracle_logits(cfg, W, toks)
    s = Served(tmp_path, cfg, W, float32=False)
    for i, cuts in enumerate([[], range(1, 33), [2, 4, 11, 13, 29]]):
        got = s.feed(i, toks, cuts)
        assert row_err(got, ref).max() < TOL16
    s.close()


# ---- windows: keys just inside and just outside, in prompts and in decoding ----------------------------------------------------------------
def test_window_edges_prompt_and_decode(tmp_path):
    cfg = CONFIGS["attention_only"]()
    win = cfg["layers"][0]["mixer"]["mask"]["size"]
    W = O.random_weights(cfg, 14)
    for k in W:
        if k.endswith("sink"):
            W[k] = O.bf16_round(W[k] - 6.0)                      # the real keys carry the weight, so a key cut off (or let in) moves the logits
    toks = tokens(cfg, 3 * win + 2, 4)
    ref = oracle_logits(cfg, W, toks)
    for d in (-1, 1):                              # the oracle with the window one off differs: the comparison below can see it
        c2 = copy.deepcopy(cfg)
        for l in c2["layers"]:
            l["mixer"]["mask"]["size"] += d
        assert np.median(row_err(oracle_logits(c2, W, toks), ref)[win + 1:]) > 50 * TOL32
    s = Served(tmp_path, cfg, W)
    assert row_err(s.feed(0, toks, []), ref).max() < TOL32
    assert row_err(s.feed(1, toks, range(1, len(toks))), ref).max() < TOL32
    # portions that end and start at, one before and one after a window's edge
    assert row_err(s.feed(2, toks, [win - 1, win, win + 1, 2 * win - 1, 2 * win + 1]), ref).max() < TOL32
    s.close()


def test_sink_is_counted_once(tmp_path):
    cfg = CONFIGS["attention_only"]()
    W = O.random_weights(cfg, 15)
    for k in W:
        if k.endswith("sink"):
            W[k] = O.bf16_round(W[k] + 3.0)                      # a heavy sink: leaving it out, scaling it or counting it per key share shows at once
    toks = tokens(cfg, 40, 5)
    ref = oracle_logits(cfg, W, toks)
    W0 = {k: (v - 60.0 if k.endswith("sink") else v) for k, v in W.items()}
    assert np.median(row_err(oracle_logits(cfg, W0, toks), ref)) > 50 * TOL32
    s = Served(tmp_path, cfg, W)
    assert row_err(s.feed(0, toks, [7, 8]), ref).max() < TOL32
    s.close()


def test_far_keys_among_hundreds(tmp_path):
    cfg = CONFIGS["far_keys"]()
    W = O.random_weights(cfg, 16)
    for k in W:
        if k.endswith("sink"):
            W[k] = O.bf16_round(W[k] - 8.0)
    toks = tokens(cfg, 300, 6)
    ref = oracle_logits(cfg, W, toks)
    s = Served(tmp_path, cfg, W, n_ctx=640)
    whole = s.feed(0, toks, [])
    assert row_err(whole, ref).max() < TOL32
    got = s.feed(1, toks, [64, 128, 191, 192, 193, 194, 258, 259, 260, 261, 262] + list(range(263, 300)))
    assert row_err(got, ref).max() < TOL32
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


def test_refusals_leave_the_context_usable(tmp_path):
    cfg = CONFIGS["ones"]()
    W = O.random_weights(cfg, 18)
    s = Served(tmp_path, cfg, W, n_ctx=32, slots=2)
    a, b = tokens(cfg, 12, 1), tokens(cfg, 12, 2)
    s.step([(0, a)])
    s.step([(1, b)])
    rc, _ = s.ctx.decode([1], [0], [[2]])
    assert rc != 0, "a third sequence with two slots"
    rc, _ = s.ctx.decode(tokens(cfg, 9, 3), list(range(12, 21)), [[0]] * 9)
    assert rc != 0, "9 more tokens with 8 cells left"
    rc, _ = s.ctx.decode([1, 2], [13, 14], [[0]] * 2)
    assert rc != 0, "a gap in the positions"
    nxt = tokens(cfg, 3, 4)
    got = s.step([(0, nxt)])[0]
    ref = oracle_logits(cfg, W, a + nxt)[12:]
    assert row_err(got, ref).max() < TOL32
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
    """served mode: portions of 128 tokens and more of a layer with wide latent rows run their attention as tensor-core matmuls (scores,
    masked softmax with the sink, weighted sums); shorter portions and decoded tokens stay with the per-token kernel.  Both against the
    oracle, against each other, and mixed in one batch"""
    cfg = CONFIGS["wide_latent"]()
    W = O.random_weights(cfg, 23)
    for k in W:
        if k.endswith("sink"):
            W[k] = O.bf16_round(W[k] - 4.0)
    toks, other = tokens(cfg, 450, 10), tokens(cfg, 60, 11)
    ref, ref_o = oracle_logits(cfg, W, toks), oracle_logits(cfg, W, other)
    s = Served(tmp_path, cfg, W, float32=False, n_ctx=1600)
    whole = s.feed(0, toks, [])                                            # one portion of 450: blocks of 256 + 194, windows of 150 and 37 inside
    small = s.feed(1, toks, range(100, 450, 100))                          # portions of 100: the per-token kernel
    cut = s.feed(2, toks, [130, 131, 300, 449])                            # 130 (matmul) + 1 + 169 (matmul) + 149 (matmul) + 1
    assert row_err(whole, ref).max() < TOL16 and row_err(small, ref).max() < TOL16 and row_err(cut, ref).max() < TOL16
    assert row_err(whole, small).max() < TOL16 / 2 and row_err(cut, small).max() < TOL16 / 2
    # a long portion beside a short one and a decoded token in ONE batch
    for r in range(3):
        s.end(r)
    a = s.step([(3, toks[:200]), (4, other[:59])])
    b = s.step([(4, other[59:]), (3, toks[200:])])
    assert row_err(np.concatenate([a[3], b[3]]), ref).max() < TOL16
    assert row_err(np.concatenate([a[4], b[4]]), ref_o).max() < TOL16
    s.close()
    s = Served(tmp_path, cfg, W, float32=True, n_ctx=600)                  # float32 contexts never take it
    assert row_err(s.feed(0, toks, []), ref).max() < TOL32
    s.close()


def test_decode_steps_around_growing_prompts(tmp_path):
    """single-token steps are replayed from captured graphs; a later, longer prompt makes the context grow its buffers (logits rows of a
    run slot, work buffers), and the steps after it must not run on the old ones"""
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
    import json
    import os
    import subprocess
    import sys
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
    steps.insert(3, json.dumps({"step": 99, "entries": [], "end": []}))          # a step that brings nothing still answers
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
            assert row_err(got, ref).max() < tol, (dtype, n)
