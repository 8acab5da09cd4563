"""Small Fabivik configurations for the tests (sizes chosen to differ from each other: heads, key / value heads, dims, windows, taps, experts)."""
import math


def attention(heads, kv_heads, dim, vdim, window=None, conv=None, v_mix=False, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if window:
        m["mask"] = {"size": window}
    if conv:
        m["conv"] = conv
    if v_mix:
        m["v_mix"] = True
    return m


def wkv(heads, dim):
    return {"heads": heads, "dim": dim}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def moe(experts, top, ff, limit, shared=None, shared_limit=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        m["shared"] = {"ff": shared, "limit": shared_limit if shared_limit is not None else limit}
    return m


def model(width, vocab, layers, eps=1e-5, embed_scale=6.0, logit_scale=0.7):
    return {"architecture": "Fabivik", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "logit_scale": logit_scale,
            "layers": [{"type": t, "mixer": mx, "mlp": ml} for t, mx, ml in layers]}


def mixed_small():
    """every mixer, a recurrent layer first, the first value-mixing layer not the first attention layer, a layer without feed-forward"""
    return model(96, 210, [("wkv", wkv(3, 20), moe(6, 3, 40, 0.9, shared=48, shared_limit=1.4)),
                           ("attention", attention(2, 2, 12, 20, window=7), moe(5, 2, 24, 1.1)),
                           ("attention", attention(6, 2, 24, 16, window=11, conv=3, v_mix=True), None),
                           ("delta", delta(4, 2, 20, 24, 2), moe(6, 3, 40, 0.9, shared=48, shared_limit=1.4)),
                           ("attention", attention(4, 2, 8, 16, window=5, conv=4, v_mix=True, scale=0.5), moe(4, 1, 16, 2.0, shared=8)),
                           ("attention", attention(2, 2, 16, 16, conv=2, v_mix=True), None)])


def attention_only():
    return model(64, 120, [("attention", attention(4, 2, 16, 24, window=9, conv=4, v_mix=True, scale=0.45), None),
                           ("attention", attention(2, 2, 16, 24, window=9, conv=4, v_mix=True, scale=0.45), None)])


def wkv_only():
    return model(72, 90, [("wkv", wkv(3, 36), None), ("wkv", wkv(1, 70), None)])


def delta_only():
    return model(80, 100, [("delta", delta(6, 2, 12, 20, 4), None), ("delta", delta(2, 2, 40, 16, 3), None)])


def experts_only():
    """small limits: the clamps act, so a weight on an expert's output instead of its input would show"""
    return model(48, 64, [("wkv", wkv(1, 8), moe(9, 4, 20, 0.5, shared=12, shared_limit=0.7)), ("wkv", wkv(1, 8), moe(3, 3, 56, 0.8))])


def ones():
    """values that happen to be 1 or equal: one head, one key head, top 1 of 1 expert, one tap, window 1, dim == vdim, no scaling"""
    return model(32, 40, [("attention", attention(1, 1, 16, 16, window=1, conv=1), moe(1, 1, 16, 1.0)),
                          ("delta", delta(1, 1, 16, 16, 1), moe(2, 1, 8, 1.5, shared=16)),
                          ("wkv", wkv(1, 16), None),
                          ("attention", attention(1, 1, 16, 16, window=4096), None)], embed_scale=1.0, logit_scale=1.0)


def far_keys():
    """long windows and a peaky softmax: single keys hundreds of tokens back carry the output"""
    return model(64, 300, [("attention", attention(2, 1, 24, 16, window=260, conv=2, scale=2.0), None),
                           ("attention", attention(4, 4, 8, 8, window=193, scale=3.0), None)])


def wide_heads():
    """head sizes that are multiples of 8: long portions take the tensor-core (matmul) form of the attention in served mode.
    No routed experts: the test compares bfloat16 runs with each other, and a router's near tie would turn rounding into a discrete change"""
    return model(64, 160, [("attention", attention(4, 2, 32, 24, window=150, conv=3, v_mix=True), None), ("delta", delta(2, 1, 16, 16, 4), None),
                           ("attention", attention(2, 2, 16, 24, window=37, conv=2, v_mix=True), None), ("wkv", wkv(2, 16), None)])


CONFIGS = {f.__name__: f for f in (mixed_small, attention_only, wkv_only, delta_only, experts_only, ones, far_keys, wide_heads)}
