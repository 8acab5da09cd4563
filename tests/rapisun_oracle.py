"""Plain, slow restatement of the Rapisun design in numpy float64 (test infrastructure only; shares no code with the library).

A model is (cfg, W): cfg the parsed config.json, W a dict name -> float64 array.  One function per mechanism; `Sequence`
carries what a sequence keeps between calls (conv tails, recurrent matrices, latent rows), so the same functions serve whole
prompts and token-by-token decoding.
"""
import math

import numpy as np


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def causal_conv(h, w, tail):
    """h [T, C], w [C, taps], tail [taps-1, C] = the inputs before h (zeros at a sequence's start).
    out_t = sum_j w[:, j] * h_(t - taps + 1 + j); returns (out, new tail)."""
    taps = w.shape[1]
    ext = np.concatenate([tail, h], 0)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(taps):
            out[t] += w[:, j] * ext[t + j]
    return out, ext[ext.shape[0] - (taps - 1):].copy() if taps > 1 else tail


def rotate_half(x, pos, base, dims):
    """x [..., >= dims]: the first `dims` entries rotate, pair (i, i + dims/2), angle pos * base^(-2i/dims)."""
    out = x.copy()
    half = dims // 2
    for i in range(half):
        a = pos * base ** (-2.0 * i / dims)
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * math.cos(a) - v * math.sin(a)
        out[..., i + half] = v * math.cos(a) + u * math.sin(a)
    return out


def latent_rows(h, pos0, mx, W, pre, eps):
    """what a latent-attention layer with its own down-projection appends to its cache: [T, kv_rank + rot_dim]"""
    R, rd = mx["kv_rank"], mx["rot_dim"]
    d = h @ W[pre + "dkv"].T
    c = rms_norm(d[:, :R], W[pre + "dkv.norm"], eps)
    kr = np.stack([rotate_half(d[t, R:], pos0 + t, mx["rot"]["base"], mx["rot"]["dims"]) for t in range(h.shape[0])])
    return np.concatenate([c, kr], 1)


def latent_attention(h, pos0, mx, W, pre, eps, rows):
    """h [T, width] at positions pos0 ..; rows [pos0 + T, kv_rank + rot_dim] = the cache (this layer's or the one it borrows)."""
    H, D, rd, V, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    T = h.shape[0]
    cq = rms_norm(h @ W[pre + "dq"].T, W[pre + "dq.norm"], eps)
    q = (cq @ W[pre + "uq"].T).reshape(T, H, D + rd)
    kn = (rows[:, :R] @ W[pre + "uk"].T).reshape(-1, H, D)
    vv = (rows[:, :R] @ W[pre + "uv"].T).reshape(-1, H, V)
    kr = rows[:, R:]
    out = np.zeros((T, H, V))
    win = mx["mask"]["size"]
    for t in range(T):
        p = pos0 + t
        lo = max(0, p - win + 1)
        for hh in range(H):
            qr = rotate_half(q[t, hh, D:], p, mx["rot"]["base"], mx["rot"]["dims"])
            s = (kn[lo:p + 1, hh] @ q[t, hh, :D] + kr[lo:p + 1] @ qr) * mx["scale"]
            sink = W[pre + "sink"][hh]
            m = max(s.max(), sink)
            e = np.exp(s - m)
            out[t, hh] = (e[:, None] * vv[lo:p + 1, hh]).sum(0) / (e.sum() + math.exp(sink - m))
    return out.reshape(T, H * V) @ W[pre + "o"].T


def hgrn2(h, mx, W, pre, eps, S):
    """S [heads, dim, vdim] is updated in place."""
    H, D, V = mx["heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = silu(h @ W[pre + "q"].T).reshape(T, H, D)
    v = (h @ W[pre + "v"].T).reshape(T, H, V)
    lo = W[pre + "lower"]
    f = (lo + (1.0 - lo) * sigmoid(h @ W[pre + "f"].T + W[pre + "f.b"])).reshape(T, H, D)
    o = np.zeros((T, H, V))
    for t in range(T):
        for hh in range(H):
            S[hh] = f[t, hh][:, None] * S[hh] + (1.0 - f[t, hh])[:, None] * v[t, hh][None, :]
            o[t, hh] = S[hh].T @ q[t, hh]
    o = rms_norm(o, W[pre + "norm"], eps)
    return o.reshape(T, H * V) @ W[pre + "o"].T


def polynorm(z, act, eps):
    a, b, c, e = act
    return a * rms_unit(z, eps) + b * rms_unit(z ** 2, eps) + c * rms_unit(z ** 3, eps) + e


def dense_mlp(h, W, pre, eps):
    return polynorm(h @ W[pre + "up"].T, W[pre + "act"], eps) @ W[pre + "down"].T


def relu2_expert(h, W, pre):
    return (np.maximum(h @ W[pre + "up"].T, 0.0) ** 2) @ W[pre + "down"].T


def moe_mlp(h, ml, W, pre):
    E, top = ml["router"]["experts"], ml["router"]["top"]
    z = h @ W[pre + "router"].T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(-1, keepdims=True)
    out = np.zeros((h.shape[0], W[pre + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        pick = np.argsort(-s[t], kind="stable")[:top]
        den = s[t, pick].sum() + 1e-20
        for e in pick:
            out[t] += s[t, e] / den * relu2_expert(h[t:t + 1], W, "%se%d." % (pre, e))[0]
    if ml.get("shared"):
        out += relu2_expert(h, W, pre + "shared.")
    return out


class Sequence:
    """what one sequence keeps between calls"""

    def __init__(self, cfg):
        self.n = 0
        L = cfg["layers"]
        taps = cfg["canon"]["taps"]
        self.tail = [np.zeros((taps - 1, cfg["width"])) for _ in L]
        self.S = [np.zeros((l["mixer"]["heads"], l["mixer"]["dim"], l["mixer"]["vdim"])) if l["type"] == "hgrn2" else None for l in L]
        self.rows = [np.zeros((0, l["mixer"]["kv_rank"] + l["mixer"]["rot_dim"]))
                     if l["type"] == "latent_attention" and "kv_from" not in l["mixer"] else None for l in L]


def forward(cfg, W, seq, tokens, layers_out=None):
    """feeds `tokens` after what `seq` already holds; returns logits [T, vocab]"""
    eps = cfg["norm"]["eps"]
    x = layer_norm(W["embed"][np.asarray(tokens)], W["embed.norm"], eps)
    for i, l in enumerate(cfg["layers"]):
        pre, mx = "l%d." % i, l["mixer"]
        c, seq.tail[i] = causal_conv(x, W[pre + "canon1"], seq.tail[i])
        h = x + c
        if l["type"] == "hgrn2":
            y = hgrn2(h, mx, W, pre + "mix.", eps, seq.S[i])
        elif l["type"] == "latent_attention":
            src = mx.get("kv_from", i)
            if src == i:
                seq.rows[i] = np.concatenate([seq.rows[i], latent_rows(h, seq.n, mx, W, pre + "mix.", eps)], 0)
            y = latent_attention(h, seq.n, mx, W, pre + "mix.", eps, seq.rows[src])
        else:
            raise ValueError(l["type"])
        x = x + layer_norm(y, W[pre + "norm1"], eps)
        ml = l.get("mlp")
        if ml:
            y = dense_mlp(x, W, pre + "mlp.", eps) if ml["kind"] == "dense" else moe_mlp(x, ml, W, pre + "mlp.")
            x = x + layer_norm(y, W[pre + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    seq.n += len(tokens)
    return layer_norm(x, W["final.norm"], eps) @ W["head"].T


# ---- random models for the tests -----------------------------------------------------------------------------------------------
def bf16_round(a):
    """round float arrays to the nearest bfloat16 (ties to even), returned as float64"""
    u = np.asarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


def tensor_shapes(cfg):
    """name -> shape of every tensor a model of this configuration holds"""
    Wd, sh = cfg["width"], {}
    sh["embed"], sh["embed.norm"], sh["final.norm"], sh["head"] = (cfg["vocab"], Wd), (Wd,), (Wd,), (cfg["vocab"], Wd)
    for i, l in enumerate(cfg["layers"]):
        p, mx = "l%d." % i, l["mixer"]
        sh[p + "norm1"], sh[p + "canon1"] = (Wd,), (Wd, cfg["canon"]["taps"])
        if l["type"] == "hgrn2":
            H, D, V = mx["heads"], mx["dim"], mx["vdim"]
            sh.update({p + "mix.q": (H * D, Wd), p + "mix.f": (H * D, Wd), p + "mix.f.b": (H * D,), p + "mix.lower": (H * D,),
                       p + "mix.v": (H * V, Wd), p + "mix.norm": (V,), p + "mix.o": (Wd, H * V)})
        else:
            H, D, rd, V, R, Q = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"], mx["q_rank"]
            sh.update({p + "mix.dq": (Q, Wd), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (D + rd), Q), p + "mix.uk": (H * D, R),
                       p + "mix.uv": (H * V, R), p + "mix.sink": (H,), p + "mix.o": (Wd, H * V)})
            if "kv_from" not in mx:
                sh.update({p + "mix.dkv": (R + rd, Wd), p + "mix.dkv.norm": (R,)})
        ml = l.get("mlp")
        if ml:
            sh[p + "norm2"] = (Wd,)
            if ml["kind"] == "dense":
                sh.update({p + "mlp.up": (ml["ff"], Wd), p + "mlp.down": (Wd, ml["ff"]), p + "mlp.act": (4,)})
            else:
                for e in range(ml["router"]["experts"]):
                    sh.update({"%smlp.e%d.up" % (p, e): (ml["expert"]["ff"], Wd), "%smlp.e%d.down" % (p, e): (Wd, ml["expert"]["ff"])})
                sh[p + "mlp.router"] = (ml["router"]["experts"], Wd)
                if ml.get("shared"):
                    sh.update({p + "mlp.shared.up": (ml["shared"]["ff"], Wd), p + "mlp.shared.down": (Wd, ml["shared"]["ff"])})
    return sh


def random_weights(cfg, seed):
    """bfloat16-representable random weights, float64"""
    rng = np.random.default_rng(seed)
    W = {}
    for name, s in tensor_shapes(cfg).items():
        if name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2"):
            w = 1.0 + 0.2 * rng.standard_normal(s)
        elif name.endswith("lower"):
            w = rng.uniform(0.0, 0.9, s)
        elif name.endswith("sink"):
            w = rng.standard_normal(s)
        elif name.endswith("act"):
            w = np.array([0.6, 0.3, 0.2, 0.05]) + 0.05 * rng.standard_normal(4)
        elif name.endswith("f.b"):
            w = rng.standard_normal(s)
        elif name.endswith("canon1"):
            w = 0.3 * rng.standard_normal(s)
        elif name == "embed":
            w = rng.standard_normal(s)
        else:
            w = rng.standard_normal(s) * (1.5 / math.sqrt(s[-1]))
        W[name] = bf16_round(w)
    return W


def write_model(folder, cfg, W):
    """config.json + model.safetensors (bfloat16) as the library's loader reads them"""
    import json
    import os
    import struct
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    head, blobs, off = {}, [], 0
    for name, w in W.items():
        assert np.array_equal(bf16_round(w), np.asarray(w, np.float64)), "%s is not bfloat16-representable: round it first" % name
        b = (np.asarray(w, np.float32).view(np.uint32) >> 16).astype(np.uint16).tobytes()
        head[name] = {"dtype": "BF16", "shape": list(np.shape(w)), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(head).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
