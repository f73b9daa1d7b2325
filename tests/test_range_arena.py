"""CPU: the device memory arena's sub-allocation logic (tnn_plugin/b200_range_arena.h) against a fake backing store.

The self-test inside the plug-in drives seeded random requests and releases (sizes from 0 bytes to three slabs) and,
after every step, checks that live blocks and free ranges tile every slab exactly, that adjacent free ranges were
merged, that no two live blocks overlap or leave their slab, and that the byte counts agree; at the end everything is
released and every slab must go back to the backing store.  No CUDA call is made.
"""
import pytest

from tnn_b200 import tnn_runtime as rt

pytestmark = pytest.mark.skipif(not rt.available(), reason="the host framework and the plug-in are not built")


@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_pooled_arena_keeps_its_invariants(seed):
    step, why = rt.selftest_range_arena(seed, 6000, pooled=True)
    assert step == 0, "invariant broken at step %d: %s" % (step, why)


def test_one_allocation_per_block_mode():
    step, why = rt.selftest_range_arena(7, 3000, pooled=False)
    assert step == 0, "invariant broken at step %d: %s" % (step, why)
