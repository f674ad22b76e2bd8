"""CPU: the speculative decoding loop against a toy engine (same surface as `_moe_infer_rs.Engine`), and the layout
conversions of the cache file.  The property under test is the one that matters: the tokens are exactly those of the
ordinary greedy loop, whatever the drafter guesses."""
import numpy as np
import pytest

from moe_infer_b200 import _moe_infer_rs as rs
from moe_infer_b200.speculative import greedy_decode, speculative_decode

V = 50


class ToyCache:
    def __init__(self):
        self.pos = 0


class ToyEngine:
    """A deterministic 'model': the logits after a history are a hash of it.  The drafter is right when `hit(history)`."""

    def __init__(self, hit):
        self.hist, self.hit, self.forwards, self.mtp_calls = [], hit, 0, 0

    def _logits(self, hist):
        rng = np.random.default_rng(abs(hash(tuple(hist))) % (2 ** 32))
        return rng.standard_normal(V).astype(np.float32)

    def forward(self, ids, cache, mtp=False):
        assert cache.pos == len(self.hist)
        rows = []
        for t in ids:
            self.hist.append(int(t))
            rows.append(self._logits(self.hist))
        cache.pos = len(self.hist)
        self.forwards += 1
        return np.stack(rows)

    def mtp_forward(self, token_id):
        self.mtp_calls += 1
        nxt = int(np.argmax(self._logits(self.hist + [int(token_id)])))
        guess = nxt if self.hit(self.hist) else (nxt + 1) % V
        out = np.zeros(V, np.float32)
        out[guess] = 1.0
        return out

    def snapshot_state(self):
        return list(self.hist)

    def restore_snapshot(self, snap):
        self.hist = list(snap)


def _run(hit, n, eos=()):
    first = np.random.default_rng(1).standard_normal(V).astype(np.float32)
    a, ca = ToyEngine(hit), ToyCache()
    want, _ = greedy_decode(first, a, ca, max_tokens=n, eos_ids=eos)
    b, cb = ToyEngine(hit), ToyCache()
    got, st = speculative_decode(first, b, cb, max_tokens=n, eos_ids=eos)
    return want, got, st, a, b, ca, cb


@pytest.mark.parametrize("hit", [lambda h: True, lambda h: False, lambda h: len(h) % 3 != 0])
@pytest.mark.parametrize("n", [1, 2, 7, 16])
def test_speculative_tokens_equal_greedy_tokens(hit, n):
    want, got, st, a, b, ca, cb = _run(hit, n)
    assert got == want and len(got) == n
    assert st["tokens"] == n and st["drafted"] == st["mtp_steps"] and 0 <= st["accepted"] <= st["drafted"]
    # the engine's history is the emitted tokens (all but possibly the last one's successor): nothing speculative is left behind
    assert b.hist == got[:len(b.hist)] and cb.pos == len(b.hist) and len(b.hist) >= n - 1


def test_accept_and_reject_counts():
    _, got, st, _, b, _, _ = _run(lambda h: True, 16)
    assert st["accepted"] == st["drafted"] == 8 and st["forwards"] == 8 and st["forward_tokens"] == 16
    _, got, st, _, b, _, _ = _run(lambda h: False, 16)
    assert st["accepted"] == 0 and st["forwards"] == 2 * st["drafted"] + 1


def test_eos_stops_both_loops_at_the_same_token():
    want, _, _, _, _, _, _ = _run(lambda h: True, 12)
    eos = (want[5],)
    w2, g2, st, *_ = _run(lambda h: True, 12, eos)
    assert g2 == w2 == want[:want.index(eos[0])]


def test_engine_without_mtp_is_refused():
    class NoMtp(ToyEngine):
        def mtp_forward(self, token_id):
            return np.zeros(0, np.float32)
    with pytest.raises(RuntimeError, match="no MTP block"):
        speculative_decode(np.ones(V, np.float32), NoMtp(lambda h: True), ToyCache(), max_tokens=4)


@pytest.mark.parametrize("pos", [0, 1, 2, 3, 4, 9])
def test_conv_state_ring_and_shifted_layouts_convert_both_ways(pos):
    """The reference keeps the last kernel - 1 conv inputs oldest first (src/math_util.rs:149-168); the device keeps a ring
    indexed by step.  Feeding the same inputs into both layouts and converting must agree."""
    ks, C = 4, 6
    rng = np.random.default_rng(pos)
    ring = np.zeros((ks, C), np.float32)
    shifted = np.zeros((ks - 1, C), np.float32)
    for step in range(pos):
        x = rng.standard_normal(C).astype(np.float32)
        ring[step % ks] = x
        shifted = np.concatenate([shifted[1:], x[None]])
    assert np.array_equal(rs._shifted_from_ring(ring, pos), shifted)
    back = rs._ring_from_shifted(shifted, pos)
    for k in range(ks - 1):  # the rows the next step reads; the remaining row is the one it overwrites
        assert np.array_equal(back[(pos - (ks - 1) + k) % ks], shifted[k])


def test_cache_file_round_trip_in_the_reference_format(tmp_path):
    """src/cache.rs:133-233: tensor names, dtypes, MAX_SEQ rows for K / V, `len` per full layer and `cache.pos` last."""
    import json

    class M:
        cfg = {"num_hidden_layers": 4, "num_key_value_heads": 2, "head_dim": 8, "linear_num_value_heads": 2, "linear_num_key_heads": 1,
               "linear_key_head_dim": 4, "linear_value_head_dim": 4, "linear_conv_kernel_dim": 4, "full_attention_interval": 4}

        def get(self, k, default=None):
            return self.cfg.get(k, default)

    model = type("Model", (), {"inner": M()})()
    c = rs.Cache(model)
    assert c.cpu_dirty and not c.gpu_dirty and c.states is None and [c.is_full(l) for l in range(4)] == [False, False, False, True]
    rng = np.random.default_rng(3)
    c.states = c._zero_states()
    c.pos = 3
    for st in c.states:
        for k in st:
            shape = (3, 16) if k in ("k_cache", "v_cache") else st[k].shape
            st[k] = rng.standard_normal(shape).astype(np.float32)
    b, j = str(tmp_path / "c.bin"), str(tmp_path / "c.json")
    c.save(b, j)
    man = json.load(open(j))["tensors"]
    assert list(man)[-1] == "cache.pos" and man["cache.pos"] == {"offset": man["cache.pos"]["offset"], "size": 4, "shape": [], "dtype": "uint32"}
    assert man["cache.layer_3.k_cache"]["shape"] == [rs.MAX_SEQ, 16] and man["cache.layer_3.k_cache"]["dtype"] == "float32"
    assert man["cache.layer_0.conv_state"]["shape"] == [3, 16] and man["cache.layer_0.ssm_state"]["shape"] == [2 * 4 * 4]
    assert "cache.layer_3.len" in man and "cache.layer_0.len" not in man
    d = rs.Cache.load(b, j)
    assert d.pos == 3 and d.cpu_dirty and not d.gpu_dirty and len(d.states) == 4
    for a, e in zip(d.states, c.states):
        assert a.keys() == e.keys() and all(np.array_equal(a[k], e[k]) for k in a)
    with pytest.raises(IOError):
        rs.Cache.load(str(tmp_path / "missing.bin"), j)
