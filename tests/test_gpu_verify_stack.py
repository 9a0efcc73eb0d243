"""Speculative verify over a stack of layers: 1 + 3 rows appended as one batch through every layer, keep,
and the route log in the reference's record format."""
import ctypes as C
import struct
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).parent))

pytestmark = pytest.mark.gpu


def _check(status, err):
    assert status == 0, (status, err.subject, err.detail)


def test_one_plus_three_rows_through_three_layers_with_route_log(gpu, tmp_path):
    import oracle
    from picoforge_b200 import abi, synth
    from picoforge_b200.layer import MoeLayer
    lib = gpu.lib
    specs = [synth.make_layer(900, layer=l, routed_type=abi.IQ2_XXS, shared_type=abi.Q4_K, experts=32, top_k=4) for l in range(3)]
    layers = [MoeLayer(gpu, spec, 4) for spec in specs]
    handles = (C.c_void_p * 3)(*[layer.moe for layer in layers])
    cfg = specs[0].config()
    verify, err = C.c_void_p(), abi.Qwen4Error()
    _check(lib.qw4cu_verify_create(handles, 3, C.byref(cfg), C.byref(verify), C.byref(err)), err)
    try:
        log = tmp_path / "routes.bin"
        _check(lib.qw4cu_verify_route_log(verify, str(log).encode(), C.byref(err)), err)
        x = synth.activations(901, 4) * 8.0                     # outputs grow with the square of the input: the chain stays away from zero
        y = np.empty_like(x)
        ids = np.empty((3, 4, 4), np.uint32)
        lib.qw4cu_launch_log_begin()
        _check(lib.qw4cu_verify_append(verify, x.ctypes.data, 4, y.ctypes.data, ids.ctypes.data, C.byref(err)), err)
        names = gpu.launch_names()
        assert names.count("fused_decode_kernel") == 3, names                 # one kernel per layer
        # the same chain layer by layer through the host entry point; ids against the oracle on each layer's own input
        cur = x
        for l, (layer, spec) in enumerate(zip(layers, specs)):
            want = oracle.forward(spec, cur, threads=synth.threads())
            np.testing.assert_array_equal(ids[l], want["ids"])
            nxt, ids_l, _ = layer.forward(cur)
            np.testing.assert_array_equal(ids_l, ids[l])
            assert np.abs(nxt - want["y"]).max() <= 1e-3 * max(1.0, float(np.abs(want["y"]).max()))   # relative at these magnitudes
            cur = nxt
        np.testing.assert_array_equal(y.view(np.uint32), cur.view(np.uint32))
        assert lib.qw4cu_verify_position(verify) == 0 and lib.qw4cu_verify_pending(verify) == 4
        assert lib.qw4cu_verify_keep(verify, 5, C.byref(err)) == abi.RANGE
        _check(lib.qw4cu_verify_keep(verify, 2, C.byref(err)), err)     # two of the three drafts were wrong
        assert lib.qw4cu_verify_position(verify) == 2
        assert lib.qw4cu_verify_keep(verify, 1, C.byref(err)) == abi.BAD_STATE
        # an ordinary one-row append, left pending, then another: the pending row counts as kept
        y1, ids1 = np.empty((1, x.shape[1]), np.float32), np.empty((3, 1, 4), np.uint32)
        _check(lib.qw4cu_verify_append(verify, x[1:2].ctypes.data, 1, y1.ctypes.data, ids1.ctypes.data, C.byref(err)), err)
        _check(lib.qw4cu_verify_append(verify, x[2:3].ctypes.data, 1, y1.ctypes.data, None, C.byref(err)), err)
        assert lib.qw4cu_verify_position(verify) == 3
        assert lib.qw4cu_verify_append(verify, x.ctypes.data, 5, y.ctypes.data, None, C.byref(err)) == abi.CAPACITY
        _check(lib.qw4cu_verify_route_log(verify, None, C.byref(err)), err)
        # the log: {position, rows, layers, top_k} then [layer][row][top_k]
        blob = log.read_bytes()
        records, at = [], 0
        while at < len(blob):
            position, rows, n_layers, k = struct.unpack_from("<4I", blob, at)
            body = np.frombuffer(blob, np.uint32, n_layers * rows * k, at + 16).reshape(n_layers, rows, k)
            records.append((position, rows, n_layers, k, body))
            at += 16 + body.nbytes
        assert [(r[0], r[1], r[2], r[3]) for r in records] == [(0, 4, 3, 4), (2, 1, 3, 4), (3, 1, 3, 4)]
        np.testing.assert_array_equal(records[0][4], ids)
        np.testing.assert_array_equal(records[1][4], ids1)
        np.testing.assert_array_equal(records[1][4][0, 0], ids[0, 1])       # row 1 alone routes as it did inside the batch
    finally:
        lib.qw4cu_verify_destroy(verify)
        for layer in layers:
            layer.close()
