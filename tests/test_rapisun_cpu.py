"""CPU-only: the host side of what the Rapisun design adds -- the scattered cell allocator and the state slots (hooks of
libpipeinfer_b200.so that make no CUDA call) -- and the consistency of the test oracle itself (tests/rapisun_oracle.py): feeding a
prompt whole, in portions and token by token must give the same logits, or the GPU tests would compare against a moving target."""
import ctypes as C
import os

import numpy as np
import pytest

from tests import rapisun_oracle as O
from tests.rapisun_configs import CONFIGS

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
SO = os.path.join(ROOT, "pipeinfer_b200", "libpipeinfer_b200.so")
KVOP_CLEAR, KVOP_RM, KVOP_CP, KVOP_KEEP = 1, 2, 3, 4


class SlotTest:
    def __init__(self, n_ctx, max_seq, n_slots):
        if not os.path.exists(SO):
            import __graft_entry__
            __graft_entry__.build()
        self.L = C.CDLL(SO)
        self.L.pib_slottest_new.restype = C.c_void_p
        self.L.pib_slottest_new.argtypes = [C.c_uint32, C.c_int32, C.c_int]
        self.L.pib_slottest_free.argtypes = [C.c_void_p]
        self.L.pib_slottest_op.argtypes = [C.c_void_p] + [C.c_int] * 5
        self.L.pib_slottest_feed.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
        self.L.pib_slottest_state.argtypes = [C.c_void_p] + [C.c_void_p] * 4
        self.h = self.L.pib_slottest_new(n_ctx, max_seq, n_slots)
        self.n_ctx, self.n_slots = n_ctx, n_slots

    def feed(self, seq, pos0, n):
        pos = np.arange(pos0, pos0 + n, dtype=np.int32)
        cells = np.full(n, -1, np.int32)
        rc = self.L.pib_slottest_feed(self.h, n, pos.ctypes.data, seq, cells.ctypes.data)
        return rc, cells

    def op(self, op, a=0, b=0, p0=-1, p1=-1):
        return self.L.pib_slottest_op(self.h, op, a, b, p0, p1)

    def state(self):
        used = C.c_int32()
        pos = np.zeros(self.n_ctx, np.int32)
        ss = np.zeros(self.n_slots, np.int32)
        sl = np.zeros(self.n_slots, np.int32)
        self.L.pib_slottest_state(self.h, C.byref(used), pos.ctypes.data, ss.ctypes.data, sl.ctypes.data)
        return used.value, pos, ss, sl


def test_cells_are_scattered_and_reused():
    t = SlotTest(16, 8, 3)
    rc, a = t.feed(0, 0, 5)
    assert rc == 0 and list(a) == [0, 1, 2, 3, 4]
    rc, b = t.feed(1, 0, 4)
    assert rc == 1 and list(b) == [5, 6, 7, 8]
    rc, a2 = t.feed(0, 5, 3)
    assert rc == 0 and list(a2) == [9, 10, 11]
    assert t.op(KVOP_RM, 1) == 0                       # sequence 1 ends: cells 5..8 and slot 1 come back
    used, pos, ss, sl = t.state()
    assert used == 8 and list(ss) == [0, -1, -1] and all(pos[5:9] == -1)
    rc, c = t.feed(2, 0, 7)                            # 4 free at the end, 4 in the hole: no run of 7 neighbours exists
    assert rc == 1, "the freed slot is taken again"
    assert sorted(c) == [5, 6, 7, 8, 12, 13, 14], c
    used, pos, ss, sl = t.state()
    assert used == 15 and list(sl[:2]) == [8, 7]
    rc, _ = t.feed(0, 8, 2)
    assert rc == -2, "one cell left: a two-token portion must be refused, and nothing may change"
    assert t.state()[0] == 15
    rc, d = t.feed(0, 8, 1)
    assert rc == 0 and t.state()[0] == 16


def test_slots_run_out_and_come_back():
    t = SlotTest(64, 16, 2)
    assert t.feed(3, 0, 2)[0] == 0 and t.feed(9, 0, 2)[0] == 1
    assert t.feed(4, 0, 1)[0] == -1, "two slots, a third sequence"
    assert t.state()[0] == 4, "a refused sequence takes no cells"
    assert t.op(KVOP_KEEP, 9) == 0
    used, pos, ss, sl = t.state()
    assert list(ss) == [-1, 9] and used == 2
    assert t.feed(4, 0, 1)[0] == 0
    assert t.op(KVOP_CLEAR) == 0
    assert list(t.state()[2]) == [-1, -1] and t.state()[0] == 0


def test_ops_a_state_cannot_follow_are_reported():
    t = SlotTest(64, 16, 2)
    t.feed(0, 0, 10)
    assert t.op(KVOP_RM, 0, 0, 4, -1) == -1, "removing the tail of a fed sequence would need the state rolled back"
    assert t.op(KVOP_RM, 0, 0, 10, -1) == 0, "a range behind what was fed touches nothing"
    assert t.op(KVOP_CP, 0, 1) == -1
    assert t.op(KVOP_RM, 0, 0, 0, -1) == 0
    assert list(t.state()[2]) == [-1, -1]


@pytest.mark.parametrize("name", ["mixed_small", "ones"])
def test_oracle_is_cut_invariant(name):
    cfg = CONFIGS[name]()
    W = O.random_weights(cfg, 5)
    rng = np.random.default_rng(1)
    toks = rng.integers(0, cfg["vocab"], 19).tolist()
    whole = O.forward(cfg, W, O.Sequence(cfg), toks)
    s = O.Sequence(cfg)
    parts = np.concatenate([O.forward(cfg, W, s, toks[a:b]) for a, b in [(0, 7), (7, 9), (9, 10), (10, 19)]])
    np.testing.assert_allclose(parts, whole, rtol=0, atol=1e-9)
    s = O.Sequence(cfg)
    single = np.concatenate([O.forward(cfg, W, s, [t]) for t in toks])
    np.testing.assert_allclose(single, whole, rtol=0, atol=1e-9)


def test_oracle_window_and_sink_matter():
    """the oracle itself must react to a window that is one token off and to a sink that is left out: then a library that agrees
    with it has both right"""
    cfg = CONFIGS["attention_only"]()
    W = O.random_weights(cfg, 2)
    toks = np.random.default_rng(3).integers(0, cfg["vocab"], 30).tolist()
    base = O.forward(cfg, W, O.Sequence(cfg), toks)
    import copy
    for d in (-1, 1):
        c2 = copy.deepcopy(cfg)
        for l in c2["layers"]:
            l["mixer"]["mask"]["size"] += d
        other = O.forward(c2, W, O.Sequence(c2), toks)
        win = cfg["layers"][0]["mixer"]["mask"]["size"]
        assert np.abs(other[:win - 1] - base[:win - 1]).max() < 1e-9, "inside the first window nothing is cut off"
        assert np.abs(other[win + 1:] - base[win + 1:]).max() > 1e-2
    W2 = dict(W)
    for k in W:
        if k.endswith("sink"):
            W2[k] = W[k] - 40.0
    assert np.abs(O.forward(cfg, W2, O.Sequence(cfg), toks) - base).max() > 1e-2


def test_safetensors_round_trip(tmp_path):
    import json
    import struct
    cfg = CONFIGS["ones"]()
    W = O.random_weights(cfg, 9)
    O.write_model(str(tmp_path), cfg, W)
    raw = open(tmp_path / "model.safetensors", "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    head = json.loads(raw[8:8 + n])
    assert set(head) == set(O.tensor_shapes(cfg))
    a, b = head["head"]["data_offsets"]
    u = np.frombuffer(raw[8 + n + a:8 + n + b], np.uint16).astype(np.uint32) << 16
    np.testing.assert_array_equal(u.view(np.float32).astype(np.float64).reshape(W["head"].shape), W["head"])
