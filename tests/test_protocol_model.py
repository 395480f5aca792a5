"""Hand-shake protocols of the persistent kernels, checked on a CPU model (no GPU, no oracle)."""
import random

import pytest

import protocol_model as pm

# B, H, T, W: ragged ends with one valid row and several rounds of items, one item per CTA, the
# benchmark shapes, a window of one key, more items than three rounds, a window under 15 keys over
# several tiles (every edge tile keeps a dS residual in the second buffer)
SHAPES = [(12, 3, 2049, 1000), (19, 5, 2049, 100), (10, 4, 1100, 300), (7, 6, 1100, 0), (16, 4, 2048, 1024),
          (16, 4, 2048, 0), (3, 5, 333, 77), (40, 4, 129, 0), (30, 2, 65, 1), (9, 7, 2305, 500), (20, 4, 700, 8)]


@pytest.mark.parametrize("B,H,T,W", SHAPES)
def test_no_deadlock_or_phase_aliasing(B, H, T, W):
    for c in list(range(0, 148, 9)) + [147]:
        for seed in range(2):
            random.seed(1000 * seed + c)
            assert pm.run_fwd(B, H, T, W, c), f"forward, CTA {c}"
            assert pm.run_dkv(B, H, T, W, c), f"dK/dV, CTA {c}"
            for fuse in (False, True):
                assert pm.run_dq(B, H, T, W, c, fuse), f"dQ (D fused: {fuse}), CTA {c}"


def test_any_item_order():
    """The hand-shakes do not depend on the order of a CTA's items: random orders, including a ragged
    item between complete ones."""
    B, H, T, W = 12, 3, 2049, 1000
    rng = random.Random(7)
    try:
        for trial in range(6):
            n_fwd = ((T + 255) // 256) * B * H
            n_bwd = ((T + 127) // 128) * B * H
            for n_items, runs in ((n_fwd, [lambda c: pm.run_fwd(B, H, T, W, c)]),
                                  (n_bwd, [lambda c: pm.run_dkv(B, H, T, W, c), lambda c: pm.run_dq(B, H, T, W, c, True)])):
                items = list(range(n_items))
                rng.shuffle(items)
                pm.TABLE = {c: items[c::37] for c in range(37)}
                for c in (0, 5, 36):
                    random.seed(trial * 100 + c)
                    for run in runs:
                        assert run(c)
    finally:
        pm.TABLE = None
