"""Small Rapisun configurations for the tests (sizes chosen to differ from each other: heads, dims, ranks, windows, taps, experts)."""
import math


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, base=10000.0, kv_from=None, scale=None, rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "mask": {"size": window},
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def hgrn2(heads, dim, vdim):
    return {"heads": heads, "dim": dim, "vdim": vdim}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def model(width, vocab, layers, taps=3, eps=1e-5):
    return {"architecture": "Rapisun", "width": width, "vocab": vocab, "canon": {"taps": taps}, "norm": {"eps": eps},
            "layers": [{"type": t, "mixer": mx, "mlp": ml} for t, mx, ml in layers]}


def mixed_small():
    a = latent(3, 24, 8, 40, 56, 72, 11, base=5000.0)
    b = dict(a, kv_from=1)
    return model(96, 210, [("hgrn2", hgrn2(2, 20, 24), moe(6, 3, 40, shared=48)),
                           ("latent_attention", a, dense(136)),
                           ("latent_attention", b, moe(6, 3, 40, shared=48)),
                           ("hgrn2", hgrn2(2, 20, 24), None),
                           ("latent_attention", latent(2, 16, 16, 16, 40, 24, 5, base=300.0), moe(5, 2, 24))], taps=3)


def attention_only():
    return model(64, 120, [("latent_attention", latent(2, 16, 8, 24, 32, 40, 9, scale=0.6), dense(96)),
                           ("latent_attention", latent(2, 16, 8, 24, 32, 40, 9, scale=0.6, kv_from=0), None)], taps=2)


def recurrent_only():
    return model(72, 90, [("hgrn2", hgrn2(3, 36, 16), None), ("hgrn2", hgrn2(1, 70, 32), dense(80))], taps=4)


def experts_only():
    return model(48, 64, [("hgrn2", hgrn2(1, 8, 8), moe(9, 4, 20, shared=12)), ("hgrn2", hgrn2(1, 8, 8), moe(3, 3, 56))], taps=2)


def ones():
    """values that happen to be 1 or equal: one head, top 1, one tap, dim == vdim == rot_dim, window 1 and a window longer than any prompt"""
    return model(32, 40, [("latent_attention", latent(1, 16, 16, 16, 16, 16, 1), moe(2, 1, 16)),
                          ("hgrn2", hgrn2(1, 16, 16), dense(32)),
                          ("latent_attention", latent(1, 16, 16, 16, 16, 16, 4096), None)], taps=1)


def far_keys():
    """a long window and a peaky softmax (large scale, sinks pushed down by the test): single keys hundreds of tokens back carry the output"""
    return model(64, 300, [("latent_attention", latent(2, 24, 8, 16, 48, 32, 260, scale=1.2), dense(64)),
                           ("latent_attention", latent(4, 8, 8, 8, 48, 32, 193, scale=1.5, kv_from=0), None)], taps=2)


def partial_rotation():
    """rot.dims smaller than rot_dim: the tail of the rotated part passes unchanged"""
    return model(40, 50, [("latent_attention", latent(2, 8, 12, 8, 24, 16, 6, rot_dims=8), dense(40))], taps=5)


def wide_latent():
    """latent rows of 192 floats: long portions of such a layer take the tensor-core (matmul) form of the attention in served mode.
    No routed experts: the test compares bfloat16 runs with each other, and a router's near tie would turn rounding into a discrete change"""
    a = latent(2, 32, 16, 24, 176, 48, 150, base=20000.0)
    return model(64, 160, [("latent_attention", a, dense(72)), ("hgrn2", hgrn2(2, 16, 16), None),
                           ("latent_attention", dict(a, kv_from=0, mask={"size": 37}), dense(48))], taps=3)


CONFIGS = {f.__name__: f for f in (wide_latent, mixed_small, attention_only, recurrent_only, experts_only, ones, far_keys, partial_rotation)}
