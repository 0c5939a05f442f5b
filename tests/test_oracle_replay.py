"""The RFC 6479 window of the CPU checker: properties the standard states, for 32- and 128-block rings."""
import numpy as np
import pytest


@pytest.mark.parametrize("blocks", [32, 128])
def test_window_semantics(oracle, blocks):
    window = (blocks - 1) * 64
    r = oracle.Replay(blocks)
    assert r.validate(0) and not r.validate(0)          # counter 0 once
    assert r.validate(1) and r.validate(5) and not r.validate(5)
    assert r.validate(3) and not r.validate(3)          # late but inside the window, once
    big = 10 * window
    assert r.validate(big)
    assert r.validate(big - window) and not r.validate(big - window)  # oldest counter still inside
    assert not r.validate(big - window - 1)             # one further back: outside
    assert not r.validate(4)                            # long gone
    assert r.validate(big + window * 3)                 # a jump past the whole ring clears it
    assert r.validate(big + window * 3 - 1)
    assert not r.validate(oracle.REJECT_AFTER_MESSAGES) and not r.validate(2**64 - 1)
    assert r.validate(oracle.REJECT_AFTER_MESSAGES - 1)
    assert r.last == oracle.REJECT_AFTER_MESSAGES - 1


@pytest.mark.parametrize("blocks", [2, 32, 128])
def test_against_set_model(oracle, blocks):
    """Random walks checked against the definition: accept iff new, below the limit and not more than
    `window` behind the highest accepted counter."""
    rng = np.random.default_rng(blocks)
    window = (blocks - 1) * 64
    r = oracle.Replay(blocks)
    seen, top = set(), 0
    c = 1000
    for _ in range(20000):
        step = int(rng.integers(-3 * window // 2 - 5, 200)) if rng.random() < 0.3 else int(rng.integers(-70, 70))
        if rng.random() < 0.01:
            step = int(rng.integers(0, 5 * blocks * 64))
        c = max(0, c + step)
        want = c not in seen and (c > top or top - c <= window)
        got = r.validate(c)
        assert got == want, (c, top)
        if want:
            seen.add(c)
            top = max(top, c)
    assert r.last == top


def test_both_ring_sizes_agree_on_config2_order(oracle):
    """Reordering within 64 and duplicates: a 2048-bit and an 8192-bit ring give the same verdicts."""
    from bnk_b200 import gen

    w = gen.config2()
    a = {p: oracle.Replay(32) for p in range(w.n_peers)}
    b = {p: oracle.Replay(128) for p in range(w.n_peers)}
    verdicts = []
    for i in w.arrival:
        p, c = int(w.base.peer[i]), int(w.base.counter[i])
        va, vb = a[p].validate(c), b[p].validate(c)
        assert va == vb
        verdicts.append(va)
    n_dup = len(w.arrival) - len(w.base.payloads)
    assert verdicts.count(False) == n_dup  # exactly the duplicates are rejected


def test_state_round_trip(oracle):
    r = oracle.Replay(32)
    for c in (5, 9, 700, 650):
        r.validate(c)
    s = oracle.Replay(32)
    s.load(r.last, r.ring())
    assert not s.validate(650) and s.validate(651) and np.array_equal(s.ring()[:0], r.ring()[:0])
