"""Plain, slow restatement of the Fabivik design in numpy float64 (test infrastructure only; shares no code with the library).

A model is (cfg, W): cfg the parsed config.json, W a dict name -> float64 array.  One function per mechanism; `Sequence` carries
what a sequence keeps between calls (convolution tails, the previous token's mixer input, recurrent matrices, cached keys and
values), so the same functions serve whole prompts, portions and token-by-token decoding.

Notation: x residual stream [T, width]; a layer is x <- x + mixer(N1(x)) + ff(N2(x)) with N(x) = x / rms(x) * (1 + w).
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


def norm_one_plus(x, w, eps):
    """RMS norm whose weight is stored around zero"""
    return rms_unit(x, eps) * (1.0 + w)


def short_conv(u, w, tail):
    """u [T, C], w [C, taps] (last column = the current token), tail [taps-1, C] = the inputs before u (zeros at a sequence's start).
    Returns (out, new tail)."""
    taps = w.shape[1]
    ext = np.concatenate([tail, u], 0)
    out = np.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(taps):
            out[t] += w[:, j] * ext[t + j]
    return out, ext[ext.shape[0] - (taps - 1):].copy()


def conv_qkv(parts, W, pre, st, act=None):
    """the short convolution on each of the projections named in `parts` ({'q': array, ...}); tails live in st"""
    out = {}
    for name, u in parts.items():
        key = pre + name + ".conv"
        if key in W:
            w = W[key]
            tail = st.get("tail_" + name)
            if tail is None:
                tail = np.zeros((w.shape[1] - 1, u.shape[1]))
            u, st["tail_" + name] = short_conv(u, w, tail)
        out[name] = act(u) if act else u
    return out


def window_attention(h, pos0, mx, W, pre, eps, st, step):
    """softmax attention of H query heads over G cached key / value heads inside a sliding window.  `step` is shared by the layers
    of one forward call: the first value-mixing layer leaves its values there."""
    H, G, D, V = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx.get("vdim", mx["dim"])
    T = h.shape[0]
    c = conv_qkv({"q": h @ W[pre + "q"].T, "k": h @ W[pre + "k"].T, "v": h @ W[pre + "v"].T}, W, pre, st)
    q = rms_unit(c["q"].reshape(T, H, D), eps) * W[pre + "q.norm"]
    k = rms_unit(c["k"].reshape(T, G, D), eps) * W[pre + "k.norm"]
    v = c["v"].reshape(T, G, V)
    if mx.get("v_mix"):
        if "v_first" in step:
            lam = float(W[pre + "vmix"])
            v = (1.0 - lam) * v + lam * step["v_first"]
        else:
            step["v_first"] = v.copy()
    st["K"] = np.concatenate([st.get("K", np.zeros((0, G, D))), k], 0)
    st["V"] = np.concatenate([st.get("V", np.zeros((0, G, V))), v], 0)
    size = (mx.get("mask") or {}).get("size")
    out = np.zeros((T, H, V))
    for t in range(T):
        i = pos0 + t
        lo = max(0, i - size + 1) if size else 0
        for a in range(H):
            g = a // (H // G)
            s = st["K"][lo:i + 1, g] @ q[t, a] * mx["scale"]
            e = np.exp(s - s.max())
            out[t, a] = (e / e.sum()) @ st["V"][lo:i + 1, g]
    return out.reshape(T, H * V) @ W[pre + "o"].T


def time_mix(h, mx, W, pre, eps, st):
    """RWKV-style: every projection reads its own blend of this token's and the previous token's input; per head
    o_t = (S + diag(u) k_t v_t^T)^T r_t and then S <- diag(w_t) S + k_t v_t^T, w_t = exp(-exp(.))"""
    H, D = mx["heads"], mx["dim"]
    T, width = h.shape
    before = st.get("prev")
    if before is None:
        before = np.zeros((1, width))
    prev = np.concatenate([before, h[:-1]], 0)
    st["prev"] = h[-1:].copy()

    def blend(s):
        return h + (prev - h) * W[pre + "mu." + s]
    r = (blend("r") @ W[pre + "r"].T).reshape(T, H, D)
    k = (blend("k") @ W[pre + "k"].T).reshape(T, H, D)
    v = (blend("v") @ W[pre + "v"].T).reshape(T, H, D)
    gate = silu(blend("g") @ W[pre + "g"].T)
    w = np.exp(-np.exp(np.tanh(blend("w") @ W[pre + "w1"].T) @ W[pre + "w2"].T + W[pre + "w0"])).reshape(T, H, D)
    S = st.get("S")
    if S is None:
        S = np.zeros((H, D, D))
    o = np.zeros((T, H, D))
    for t in range(T):
        for a in range(H):
            kv = np.outer(k[t, a], v[t, a])
            o[t, a] = (S[a] + W[pre + "u"][a][:, None] * kv).T @ r[t, a]
            S[a] = w[t, a][:, None] * S[a] + kv
    st["S"] = S
    return (rms_unit(o, eps).reshape(T, H * D) * W[pre + "norm"] * gate) @ W[pre + "o"].T


def delta_rule(h, mx, W, pre, eps, st):
    """gated delta rule per head: S <- g S; e = beta (v - S^T k); S <- S + k e^T; o = S^T q"""
    H, G, D, V = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"]
    T = h.shape[0]
    c = conv_qkv({"q": h @ W[pre + "q"].T, "k": h @ W[pre + "k"].T, "v": h @ W[pre + "v"].T}, W, pre, st, act=silu)
    q, k, v = c["q"].reshape(T, G, D), c["k"].reshape(T, G, D), c["v"].reshape(T, H, V)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) / math.sqrt(D)
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W[pre + "b"].T)
    g = np.exp(-np.exp(W[pre + "A_log"]) * softplus(h @ W[pre + "a"].T + W[pre + "dt_bias"]))
    S = st.get("S")
    if S is None:
        S = np.zeros((H, D, V))
    o = np.zeros((T, H, V))
    for t in range(T):
        for a in range(H):
            j = a // (H // G)
            S[a] = g[t, a] * S[a]
            e = beta[t, a] * (v[t, a] - S[a].T @ k[t, j])
            S[a] = S[a] + np.outer(k[t, j], e)
            o[t, a] = S[a].T @ q[t, j]
    st["S"] = S
    o = rms_unit(o, eps) * W[pre + "norm"]
    return (o.reshape(T, H * V) * silu(h @ W[pre + "g"].T)) @ W[pre + "o"].T


def gated_expert(h, W, pre, limit):
    a = np.minimum(h @ W[pre + "gate"].T, limit)
    b = np.clip(h @ W[pre + "up"].T, -limit, limit)
    return (a * sigmoid(1.702 * a) * (b + 1.0)) @ W[pre + "down"].T


def expert_mixture(h, ml, W, pre):
    """sigmoid router; the chosen experts' scores, as they are, multiply the experts' INPUTS; a shared expert behind a sigmoid gate"""
    top = ml["router"]["top"]
    score = sigmoid(h @ W[pre + "router"].T)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in np.argsort(-score[t], kind="stable")[:top]:
            out[t] += gated_expert(score[t, e] * h[t:t + 1], W, "%se%d." % (pre, e), ml["expert"]["limit"])[0]
    if ml.get("shared"):
        y = gated_expert(h, W, pre + "shared.", ml["shared"]["limit"])
        out += y * sigmoid(h @ W[pre + "shared.sg"].T)
    return out


class Sequence:
    """what one sequence keeps between calls"""

    def __init__(self, cfg):
        self.n = 0
        self.st = [dict() for _ in cfg["layers"]]


def forward(cfg, W, seq, tokens, layers_out=None):
    """feeds `tokens` after what `seq` already holds; returns logits [T, vocab]"""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    step = {}
    for i, l in enumerate(cfg["layers"]):
        pre = "l%d." % i
        h = norm_one_plus(x, W[pre + "norm1"], eps)
        if l["type"] == "attention":
            y = window_attention(h, seq.n, l["mixer"], W, pre + "mix.", eps, seq.st[i], step)
        elif l["type"] == "wkv":
            y = time_mix(h, l["mixer"], W, pre + "mix.", eps, seq.st[i])
        elif l["type"] == "delta":
            y = delta_rule(h, l["mixer"], W, pre + "mix.", eps, seq.st[i])
        else:
            raise ValueError(l["type"])
        if l.get("mlp"):
            y = y + expert_mixture(norm_one_plus(x, W[pre + "norm2"], eps), l["mlp"], W, pre + "mlp.")
        x = x + y
        if layers_out is not None:
            layers_out.append(x.copy())
    seq.n += len(tokens)
    return norm_one_plus(x, W["final.norm"], eps) @ W["head"].T * cfg["logit_scale"]


# ---- random models for the tests -----------------------------------------------------------------------------------------------
def tensor_shapes(cfg, decay_rank=6):
    """name -> shape of every tensor a model of this configuration holds"""
    Wd, sh = cfg["width"], {}
    sh["embed"], sh["final.norm"], sh["head"] = (cfg["vocab"], Wd), (Wd,), (cfg["vocab"], Wd)
    for i, l in enumerate(cfg["layers"]):
        p, mx = "l%d." % i, l["mixer"]
        sh[p + "norm1"] = (Wd,)
        H, D = mx["heads"], mx["dim"]
        G, V = mx.get("kv_heads", H), mx.get("vdim", D)
        if l["type"] == "attention":
            sh.update({p + "mix.q": (H * D, Wd), p + "mix.k": (G * D, Wd), p + "mix.v": (G * V, Wd), p + "mix.q.norm": (D,), p + "mix.k.norm": (D,),
                       p + "mix.o": (Wd, H * V)})
            if mx.get("conv"):
                sh.update({p + "mix.q.conv": (H * D, mx["conv"]), p + "mix.k.conv": (G * D, mx["conv"]), p + "mix.v.conv": (G * V, mx["conv"])})
            if mx.get("v_mix"):
                sh[p + "mix.vmix"] = ()
        elif l["type"] == "wkv":
            for s in "rkvgw":
                sh[p + "mix.mu." + s] = (Wd,)
            for s in "rkvg":
                sh[p + "mix." + s] = (H * D, Wd)
            sh.update({p + "mix.w1": (decay_rank + i, Wd), p + "mix.w2": (H * D, decay_rank + i), p + "mix.w0": (H * D,), p + "mix.u": (H, D),
                       p + "mix.norm": (H * D,), p + "mix.o": (Wd, H * D)})
        else:
            sh.update({p + "mix.q": (G * D, Wd), p + "mix.k": (G * D, Wd), p + "mix.v": (H * V, Wd), p + "mix.g": (H * V, Wd), p + "mix.b": (H, Wd), p + "mix.a": (H, Wd),
                       p + "mix.q.conv": (G * D, mx["conv"]), p + "mix.k.conv": (G * D, mx["conv"]), p + "mix.v.conv": (H * V, mx["conv"]),
                       p + "mix.A_log": (H,), p + "mix.dt_bias": (H,), p + "mix.norm": (V,), p + "mix.o": (Wd, H * V)})
        ml = l.get("mlp")
        if ml:
            sh[p + "norm2"] = (Wd,)
            F = ml["expert"]["ff"]
            for e in range(ml["router"]["experts"]):
                sh.update({"%smlp.e%d.gate" % (p, e): (F, Wd), "%smlp.e%d.up" % (p, e): (F, Wd), "%smlp.e%d.down" % (p, e): (Wd, F)})
            sh[p + "mlp.router"] = (ml["router"]["experts"], Wd)
            if ml.get("shared"):
                Fs = ml["shared"]["ff"]
                sh.update({p + "mlp.shared.gate": (Fs, Wd), p + "mlp.shared.up": (Fs, Wd), p + "mlp.shared.down": (Wd, Fs), p + "mlp.shared.sg": (1, Wd)})
    return sh


def random_weights(cfg, seed):
    """bfloat16-representable random weights, float64"""
    rng = np.random.default_rng(seed)
    W = {}
    for name, s in tensor_shapes(cfg).items():
        if name.endswith("norm1") or name.endswith("norm2") or name == "final.norm":
            w = 0.2 * rng.standard_normal(s)                                  # stored around zero
        elif name.endswith("norm"):
            w = 1.0 + 0.2 * rng.standard_normal(s)
        elif ".mu." in name:
            w = rng.uniform(0.0, 1.0, s)
        elif name.endswith("vmix"):
            w = np.asarray(rng.uniform(0.2, 0.6))
        elif name.endswith(".conv"):
            w = 0.4 * rng.standard_normal(s)
            w[:, -1] += 0.6
        elif name.endswith("w0"):
            w = rng.uniform(-2.5, 0.5, s)                                     # decays between about 0.92 and 0.19 per token
        elif name.endswith("w1") or name.endswith("w2"):
            w = rng.standard_normal(s) * (1.0 / math.sqrt(s[-1]))
        elif name.endswith("mix.u"):
            w = 0.5 * rng.standard_normal(s)
        elif name.endswith("A_log"):
            w = rng.uniform(-1.5, 0.5, s)
        elif name.endswith("dt_bias"):
            w = rng.uniform(-2.0, 1.0, s)
        elif name == "embed":
            w = rng.standard_normal(s) / cfg["embedding"]["scale"]
        else:
            w = rng.standard_normal(s) * (1.5 / math.sqrt(s[-1]))
        W[name] = bf16_round(w)
    return W
