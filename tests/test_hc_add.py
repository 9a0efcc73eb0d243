"""The hyper-connection add fused behind the layer: the NumPy restatement pinned to the reference's own
qwen4_hc_add, and (GPU) every launch path's residual equal, bit for bit, to that restatement applied to the
same path's y."""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).parent))
sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import oracle  # noqa: E402

from picoforge_b200 import abi, synth  # noqa: E402


def _inputs(seed, tokens, streams, hidden):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((tokens, streams, hidden)).astype(np.float32),
            (rng.standard_normal((tokens, streams)) * 0.7).astype(np.float32))


@pytest.mark.skipif(not oracle.reference_available(), reason="the reference's objects are not built")
def test_restatement_equals_the_reference():
    residual, inject = _inputs(1, 5, 4, 96)
    block = np.random.default_rng(2).standard_normal((5, 96)).astype(np.float32) * 3.0
    want = oracle.reference_hc_add(residual, block, inject)
    got = oracle.hc_add(residual, block, inject)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    assert not np.array_equal(got, residual)


def _run(gpu, spec, x, streams, seed):
    from picoforge_b200.layer import MoeLayer
    lib = gpu.lib
    tokens, hidden = x.shape
    residual, inject = _inputs(seed, tokens, streams, hidden)
    with MoeLayer(gpu, spec, tokens) as layer:
        d = [lib.qw4cu_malloc(n) for n in (x.nbytes, x.nbytes, x.nbytes, residual.nbytes, inject.nbytes)]
        d_x, d_y, d_plain, d_r, d_g = d
        try:
            for pointer, array in ((d_x, x), (d_r, residual), (d_g, inject)):
                assert lib.qw4cu_upload(pointer, array.ctypes.data, array.nbytes) == 0
            err = abi.Qwen4Error()
            st = lib.qw4cu_moe_forward_device(layer.moe, d_x, d_plain, tokens, None, None, layer.work, C.byref(err))
            assert st == 0, err.detail
            st = lib.qw4cu_moe_forward_hc_add_device(layer.moe, d_x, d_y, tokens, d_r, d_g, streams, layer.work, C.byref(err))
            assert st == 0, err.detail
            st = lib.qw4cu_moe_work_sync(layer.work, C.byref(err))
            assert st == 0, err.detail
            y, plain, got = np.empty_like(x), np.empty_like(x), np.empty_like(residual)
            for array, pointer in ((y, d_y), (plain, d_plain), (got, d_r)):
                assert lib.qw4cu_download(array.ctypes.data, pointer, array.nbytes) == 0
        finally:
            for pointer in d:
                lib.qw4cu_free(pointer)
    np.testing.assert_array_equal(y.view(np.uint32), plain.view(np.uint32))           # y itself is what the plain call writes
    np.testing.assert_array_equal(got.view(np.uint32), oracle.hc_add(residual, y, inject).view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("name,routed,tokens,streams", [("one-kernel decode", abi.IQ2_XXS, 4, 4), ("four-row grouped", abi.Q4_K, 24, 4),
                                                        ("tile", abi.Q2_K, 96, 2), ("tcgen05 prefill", abi.Q4_K, 320, 4)])
def test_residual_after_every_tensor_core_path(gpu, name, routed, tokens, streams):
    spec = synth.make_layer(500 + tokens, routed_type=routed, shared_type=abi.Q4_K, experts=32, top_k=4)
    _run(gpu, spec, synth.activations(500 + tokens, tokens), streams, tokens)


@pytest.mark.gpu
def test_residual_after_the_cuda_core_fallback(gpu):
    import cases
    spec = cases.float_layer(77, hidden=64, experts=8, top_k=2, inter=48, shared_inter=32)
    x = np.random.default_rng(78).standard_normal((6, 64)).astype(np.float32)
    _run(gpu, spec, x, 4, 79)


@pytest.mark.gpu
def test_nonfinite_residual_is_reported(gpu):
    from picoforge_b200.layer import MoeLayer
    lib = gpu.lib
    spec = synth.make_layer(504, routed_type=abi.IQ2_XXS, shared_type=abi.Q4_K, experts=32, top_k=4)
    x = synth.activations(504, 4)
    residual, inject = _inputs(5, 4, 4, spec.hidden)
    inject[2, 1] = 1.0e38
    residual[2, 1] = 3.4e38                                                          # 3.4e38 + 1e38 * y overflows wherever y > 3e-4
    with MoeLayer(gpu, spec, 4) as layer:
        d = [lib.qw4cu_malloc(n) for n in (x.nbytes, x.nbytes, residual.nbytes, inject.nbytes)]
        try:
            for pointer, array in ((d[0], x), (d[2], residual), (d[3], inject)):
                assert lib.qw4cu_upload(pointer, array.ctypes.data, array.nbytes) == 0
            err = abi.Qwen4Error()
            assert lib.qw4cu_moe_forward_hc_add_device(layer.moe, d[0], d[1], 4, d[2], d[3], 4, layer.work, C.byref(err)) == 0
            assert lib.qw4cu_moe_work_sync(layer.work, C.byref(err)) == abi.NONFINITE
            layer.reset()
        finally:
            for pointer in d:
                lib.qw4cu_free(pointer)
