"""The allocation-free dispatch entry point, checked against the ordinary one.

Kept in a file that pytest collects last: should it fail, a run that stops at the first failure
has already executed every other test.

Some callers of the library cannot allocate while they work: a decode loop that has committed
all spare device memory, where an allocation may fail and cudaMalloc stalls the device.  For them
qw4cu_group_pairs_device_noalloc computes the per-expert pair lists with its working memory in
an array built into the library.  The array is shared by all calls and keeps the previous
call's contents, so the test calls it twice in a row with different ids and expects both
results to equal qw4_moe_group_pairs exactly (integer lists: no tolerance)."""
import ctypes as C

import numpy as np
import pytest

from picoforge_b200 import abi
from picoforge_b200.layer import group_pairs

pytestmark = pytest.mark.gpu


def device_lists(lib, ids, experts):
    tokens, k = ids.shape
    pairs = tokens * k
    d_ids = lib.qw4cu_malloc(max(ids.nbytes, 4))          # the caller's own buffers: inputs and outputs
    d_off = lib.qw4cu_malloc((experts + 1) * 4)
    d_p2r = lib.qw4cu_malloc(max(pairs * 4, 4))
    d_r2p = lib.qw4cu_malloc(max(pairs * 4, 4))
    try:
        assert lib.qw4cu_upload(d_ids, ids.ctypes.data, ids.nbytes) == 0
        err = abi.Qwen4Error()
        status = lib.qw4cu_group_pairs_device_noalloc(experts, k, tokens, d_ids, d_off, d_p2r, d_r2p, C.byref(err))
        offsets = np.empty(experts + 1, np.uint32)
        p2r, r2p = np.empty(pairs, np.uint32), np.empty(pairs, np.uint32)
        assert lib.qw4cu_download(offsets.ctypes.data, d_off, offsets.nbytes) == 0
        if pairs:
            assert lib.qw4cu_download(p2r.ctypes.data, d_p2r, p2r.nbytes) == 0
            assert lib.qw4cu_download(r2p.ctypes.data, d_r2p, r2p.nbytes) == 0
        return status, err, offsets, p2r, r2p
    finally:
        for p in (d_ids, d_off, d_p2r, d_r2p):
            lib.qw4cu_free(p)


def test_no_alloc_dispatch_matches_the_ordinary_entry_point_twice_in_a_row(gpu):
    lib = gpu.lib
    rng = np.random.default_rng(20261125)
    cases = [(64, 512, 10), (5, 7, 3)]                       # second call: fewer experts, stale counters behind it
    for tokens, experts, k in cases:
        ids = np.stack([rng.permutation(experts)[:k] for _ in range(tokens)]).astype(np.uint32)
        want_offsets, want_p2r, want_r2p = group_pairs(gpu, ids, experts)
        status, err, offsets, p2r, r2p = device_lists(lib, ids, experts)
        assert status == abi.OK, err.detail
        np.testing.assert_array_equal(offsets, want_offsets)
        np.testing.assert_array_equal(p2r, want_p2r)
        np.testing.assert_array_equal(r2p, want_r2p)


def test_no_alloc_dispatch_rejects_what_it_cannot_hold(gpu):
    lib = gpu.lib
    ids = np.zeros((1, 1), np.uint32)
    status, err, *_ = device_lists(lib, ids, 4097)
    assert status == abi.CAPACITY and b"4096" in err.detail
    err = abi.Qwen4Error()
    too_many = (1 << 18) // 10 + 1
    assert lib.qw4cu_group_pairs_device_noalloc(512, 10, too_many, None, None, None, None, C.byref(err)) == abi.CAPACITY
    bad = np.array([[1, 9]], np.uint32)                      # id 9 of 4 experts
    status, err, *_ = device_lists(lib, bad, 4)
    assert status == abi.RANGE
    good = np.array([[2, 0], [1, 2], [2, 0]], np.uint32)     # and the next call is clean again
    status, err, offsets, p2r, r2p = device_lists(lib, good, 4)
    assert status == abi.OK and offsets.tolist() == [0, 2, 3, 6, 6] and r2p.tolist() == [1, 5, 2, 0, 3, 4]


def test_no_alloc_dispatch_takes_ids_straight_from_the_route_call_and_allocates_nothing(gpu):
    """ids written by qw4cu_moe_route_device on the library's stream are consumed with no
    synchronisation in between (the dispatch is enqueued on the same stream), and the free device
    memory is the same before and after the call."""
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent))
    from cases import small_layer
    from picoforge_b200 import synth
    from picoforge_b200.layer import MoeLayer
    lib = gpu.lib
    spec = small_layer(91, experts=32, top_k=4)
    tokens, k, experts = 48, spec.top_k, spec.experts
    x = synth.activations(91, tokens, spec.hidden)
    with MoeLayer(gpu, spec, tokens) as layer:
        _, want_ids, _ = layer.forward(x)
        want_offsets, want_p2r, want_r2p = group_pairs(gpu, want_ids, experts)
        pairs = tokens * k
        d_x = lib.qw4cu_malloc(x.nbytes)
        d_ids, d_off = lib.qw4cu_malloc(pairs * 4), lib.qw4cu_malloc((experts + 1) * 4)
        d_p2r, d_r2p = lib.qw4cu_malloc(pairs * 4), lib.qw4cu_malloc(pairs * 4)
        try:
            assert lib.qw4cu_upload(d_x, x.ctypes.data, x.nbytes) == 0
            err = abi.Qwen4Error()
            # first call on this device (address look-up) before the bytes are counted
            assert lib.qw4cu_moe_route_device(layer.moe, d_x, tokens, d_ids, None, layer.work, C.byref(err)) == abi.OK, err.detail
            assert lib.qw4cu_group_pairs_device_noalloc(experts, k, tokens, d_ids, d_off, d_p2r, d_r2p, C.byref(err)) == abi.OK
            free_before, free_after, total = C.c_size_t(), C.c_size_t(), C.c_size_t()
            assert lib.qw4cu_mem_info(C.byref(free_before), C.byref(total)) == 0
            assert lib.qw4cu_upload(d_ids, np.zeros(pairs, np.uint32).ctypes.data, pairs * 4) == 0     # stale ids would be caught
            assert lib.qw4cu_moe_route_device(layer.moe, d_x, tokens, d_ids, None, layer.work, C.byref(err)) == abi.OK, err.detail
            status = lib.qw4cu_group_pairs_device_noalloc(experts, k, tokens, d_ids, d_off, d_p2r, d_r2p, C.byref(err))   # no sync before it
            assert status == abi.OK, err.detail
            assert lib.qw4cu_mem_info(C.byref(free_after), C.byref(total)) == 0
            assert free_after.value == free_before.value
            offsets, p2r, r2p = np.empty(experts + 1, np.uint32), np.empty(pairs, np.uint32), np.empty(pairs, np.uint32)
            assert lib.qw4cu_download(offsets.ctypes.data, d_off, offsets.nbytes) == 0
            assert lib.qw4cu_download(p2r.ctypes.data, d_p2r, p2r.nbytes) == 0
            assert lib.qw4cu_download(r2p.ctypes.data, d_r2p, r2p.nbytes) == 0
        finally:
            for p in (d_x, d_ids, d_off, d_p2r, d_r2p):
                lib.qw4cu_free(p)
    np.testing.assert_array_equal(offsets, want_offsets)
    np.testing.assert_array_equal(p2r, want_p2r)
    np.testing.assert_array_equal(r2p, want_r2p)
