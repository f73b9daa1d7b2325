"""CPU: the tensor-map (TMA descriptor) cache under concurrent lookups and evictions.

The launchers copy a cached 128-byte map out under the cache's lock; a second instance or replica thread in the same
process can make the cache drop all of its entries at any moment.  The library's self-test hammers a tiny cache from
several threads with a stand-in for the driver's encoder (no GPU needed) and counts maps that came back wrong."""
from tnn_b200 import capi


def test_concurrent_lookups_survive_evictions():
    lib = capi.lib()
    assert lib.b200_selftest_tensor_map_cache(8, 2000, 64) == 0      # capacity far below the key count: constant eviction
    assert lib.b200_selftest_tensor_map_cache(4, 500, 100000) == 0   # no eviction: plain hits


def test_bad_arguments():
    lib = capi.lib()
    assert lib.b200_selftest_tensor_map_cache(0, 10, 10) == capi.ERR_PARAM
    assert lib.b200_selftest_tensor_map_cache(2, 10, 0) == capi.ERR_PARAM
