"""CPU-only: the consistency of the Fabivik test oracle itself (tests/fabivik_oracle.py).  Feeding a prompt whole, in portions and
token by token must give the same logits, and the mechanisms the GPU tests are meant to catch must move the oracle's logits, or those
tests would compare against a moving or an indifferent target."""
import copy

import numpy as np
import pytest

from tests import fabivik_oracle as O
from tests.fabivik_configs import CONFIGS


def tokens(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def run(cfg, W, toks, cuts=()):
    seq, out, a = O.Sequence(cfg), [], 0
    for b in list(cuts) + [len(toks)]:
        if b > a:
            out.append(O.forward(cfg, W, seq, toks[a:b]))
        a = b
    return np.concatenate(out)


def rel(a, b):
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-30))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_oracle_does_not_depend_on_the_cuts(name):
    cfg = CONFIGS[name]()
    W = O.random_weights(cfg, 3)
    toks = tokens(cfg, 23, 1)
    whole = run(cfg, W, toks)
    assert np.isfinite(whole).all() and whole.std() > 1e-3
    assert rel(run(cfg, W, toks, range(1, 23)), whole) < 1e-9
    assert rel(run(cfg, W, toks, [2, 4, 5, 12, 14, 21]), whole) < 1e-9


def test_short_conv_reads_the_tail():
    rng = np.random.default_rng(0)
    u, w = rng.standard_normal((9, 5)), rng.standard_normal((5, 4))
    whole, tail = O.short_conv(u, w, np.zeros((3, 5)))
    assert np.allclose(whole[0], w[:, 3] * u[0]) and np.allclose(whole[3], (w * u[0:4].T).sum(1))
    a, t1 = O.short_conv(u[:2], w, np.zeros((3, 5)))
    b, t2 = O.short_conv(u[2:], w, t1)
    assert np.allclose(np.concatenate([a, b]), whole) and np.allclose(t2, tail) and np.allclose(t2, u[6:])


def test_mechanisms_move_the_logits():
    cfg = CONFIGS["mixed_small"]()
    W = O.random_weights(cfg, 5)
    toks = tokens(cfg, 30, 2)
    ref = run(cfg, W, toks)

    def changed(c2=None, W2=None):
        return rel(run(c2 or cfg, W2 or W, toks), ref)
    for i, l in enumerate(cfg["layers"]):
        if l["type"] == "attention" and l["mixer"].get("mask"):
            for d in (-1, 1):
                c2 = copy.deepcopy(cfg)
                c2["layers"][i]["mixer"]["mask"]["size"] += d
                assert changed(c2) > 1e-4, "window of layer %d" % i
    for key in ("l4.mix.vmix", "l0.mix.u", "l0.mix.mu.w", "l3.mix.dt_bias", "l3.mix.A_log", "l0.mlp.shared.sg", "l2.mix.k.conv", "l3.mix.q.conv"):
        W2 = dict(W)
        W2[key] = W[key] * 0.5 + 0.25
        assert changed(W2=W2) > 1e-4, key
    c2 = copy.deepcopy(cfg)
    c2["layers"][0]["mlp"]["expert"]["limit"] = 5.0
    assert changed(c2) > 1e-4, "the experts' clamp"
    c2 = copy.deepcopy(cfg)
    c2["layers"][2]["mixer"]["v_mix"] = False
    assert changed(c2) > 1e-4, "which layer's values are mixed in"


def test_expert_weight_is_on_the_input():
    """with an active clamp, expert(w h) differs from w expert(h)"""
    cfg = CONFIGS["experts_only"]()
    W = O.random_weights(cfg, 6)
    h = np.random.default_rng(1).standard_normal((4, cfg["width"])) * 2.0
    ml = cfg["layers"][0]["mlp"]
    got = O.expert_mixture(h, dict(ml, shared=None), W, "l0.mlp.")
    score = O.sigmoid(h @ W["l0.mlp.router"].T)
    alt = np.zeros_like(h)
    for t in range(4):
        for e in np.argsort(-score[t], kind="stable")[:ml["router"]["top"]]:
            alt[t] += score[t, e] * O.gated_expert(h[t:t + 1], W, "l0.mlp.e%d." % e, ml["expert"]["limit"])[0]
    assert rel(got, alt) > 1e-2
