"""The one-kernel decode path (up to four tokens) against the CPU oracle and against the
multi-kernel sequence: route ids bit-exact, y within 1e-3 (max abs) of the oracle's FP32 result."""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).parent))

pytestmark = pytest.mark.gpu

Y_TOLERANCE = 1e-3


def _forward(gpu, spec, x, fused):
    from picoforge_b200.layer import MoeLayer
    gpu.lib.qw4cu_set_fused_decode(fused)
    try:
        with MoeLayer(gpu, spec, x.shape[0]) as layer:
            before = gpu.lib.qw4cu_launch_count()
            y, ids, weights = layer.forward(x)
            launches = gpu.lib.qw4cu_launch_count() - before
            y2, ids2, _ = layer.forward(x)            # the barrier counters are ready for a second launch
    finally:
        gpu.lib.qw4cu_set_fused_decode(-1)
    np.testing.assert_array_equal(ids, ids2)
    np.testing.assert_array_equal(y, y2)              # deterministic
    return y, ids, weights, launches


@pytest.mark.parametrize("routed,shared,tokens,top_k", [
    (12, 12, 1, 10), (12, 12, 4, 10), (12, 12, 3, 10), (16, 12, 4, 10), (16, 16, 2, 6), (12, 16, 4, 6), (16, 12, 1, 10)])
def test_one_kernel_decode_matches_the_oracle(gpu, routed, shared, tokens, top_k):
    import oracle
    from picoforge_b200 import synth
    spec = synth.make_layer(500 + routed + tokens, routed_type=routed, shared_type=shared, experts=64, top_k=top_k)
    x = synth.activations(500 + tokens, tokens)
    want = oracle.forward(spec, x, threads=synth.threads())
    y, ids, weights, launches = _forward(gpu, spec, x, -1)
    assert launches == 1, launches                    # the whole layer was one kernel
    np.testing.assert_array_equal(ids, want["ids"])
    np.testing.assert_array_equal(weights, want["weights"])     # exact router mode: the reference's bits
    assert np.abs(y - want["y"]).max() <= Y_TOLERANCE
    y_multi, ids_multi, _, launches_multi = _forward(gpu, spec, x, 0)
    assert launches_multi > 1
    np.testing.assert_array_equal(ids_multi, ids)
    assert np.abs(y - y_multi).max() <= Y_TOLERANCE


def test_one_kernel_decode_at_config_shapes_both_router_modes(gpu):
    """512 experts, top-10, IQ2_XXS routed + Q4_K shared, four tokens; fast router mode too."""
    import oracle
    from picoforge_b200 import abi, synth
    spec = synth.make_layer(1, routed_type=abi.IQ2_XXS, shared_type=abi.Q4_K)
    x = synth.activations(1, 4)
    want = oracle.forward(spec, x, threads=synth.threads())
    for mode in (0, 1):
        gpu.lib.qw4cu_set_router_mode(mode)
        try:
            y, ids, weights, launches = _forward(gpu, spec, x, -1)
        finally:
            gpu.lib.qw4cu_set_router_mode(0)
        assert launches == 1
        np.testing.assert_array_equal(ids, want["ids"])
        assert np.abs(y - want["y"]).max() <= Y_TOLERANCE
        assert np.abs(weights - want["weights"]).max() <= 1e-6


@pytest.mark.parametrize("routed,tokens,experts", [(16, 4, 64), (12, 1, 512), (16, 3, 512)])
def test_wrong_speculation_is_repaired(gpu, routed, tokens, experts):
    """The kernel starts the experts from tree-summed logits and checks that guess against the exact
    routes.  With a wrong expert forced into the guess of token 0 the launch must notice, run the
    experts again with the exact ids, and still return the reference's ids, weights and y."""
    import oracle
    from picoforge_b200 import synth
    from picoforge_b200.layer import MoeLayer
    spec = synth.make_layer(640 + routed + tokens, routed_type=routed, shared_type=12, experts=experts, top_k=10)
    x = synth.activations(640 + tokens, tokens)
    want = oracle.forward(spec, x, threads=synth.threads())
    repairs = C.c_uint32()
    with MoeLayer(gpu, spec, tokens) as layer:
        y0, ids0, weights0 = layer.forward(x)
        assert gpu.lib.qw4cu_decode_repairs(layer.work, C.byref(repairs)) == 0 and repairs.value == 0
        gpu.lib.qw4cu_set_decode_wrong_speculation(1)
        try:
            gpu.lib.qw4cu_launch_log_begin()
            y, ids, weights = layer.forward(x)
            assert gpu.launch_names() == ["fused_decode_kernel"]
        finally:
            gpu.lib.qw4cu_set_decode_wrong_speculation(0)
        assert gpu.lib.qw4cu_decode_repairs(layer.work, C.byref(repairs)) == 0 and repairs.value == 1
        y2, ids2, _ = layer.forward(x)                  # and the workspace is fit for the next launch
    np.testing.assert_array_equal(ids, want["ids"])
    np.testing.assert_array_equal(weights, want["weights"])
    assert np.abs(y - want["y"]).max() <= Y_TOLERANCE
    np.testing.assert_array_equal(ids0, ids)
    np.testing.assert_array_equal(y2, y0)
    assert np.abs(y - y0).max() <= 1e-4                 # same experts, possibly in another source order


def test_nonfinite_logit_leaves_outputs_untouched(gpu):
    """A NaN router weight makes every logit NaN: status NONFINITE, y keeps its fill value."""
    from picoforge_b200 import abi, synth
    from picoforge_b200.layer import MoeLayer
    spec = synth.make_layer(77, routed_type=abi.Q4_K, shared_type=abi.Q4_K, experts=64, top_k=4)
    router = spec.tensors[0].view(np.float32).copy()
    router[5] = np.nan
    spec.tensors[0] = router.view(np.uint8)
    x = synth.activations(77, 2)
    with MoeLayer(gpu, spec, 2) as layer:
        with pytest.raises(abi.MoeError) as info:
            layer.forward(x)
        assert info.value.status == abi.NONFINITE
        layer.reset()
