"""The tensor-core prefill path (tcgen05 grouped GEMM on exact integer codes) against the CPU
oracle: route ids and per-expert lists bit-exact, y within 1e-3 (max abs) of the FP32 result."""
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).parent))

pytestmark = pytest.mark.gpu

Y_TOLERANCE = 1e-3


def _forward(gpu, spec, x, prefill):
    from picoforge_b200.layer import MoeLayer
    gpu.lib.qw4cu_set_prefill_path(prefill)
    try:
        with MoeLayer(gpu, spec, x.shape[0]) as layer:
            y, ids, weights = layer.forward(x)
            y2, ids2, _ = layer.forward(x)
    finally:
        gpu.lib.qw4cu_set_prefill_path(-1)
    np.testing.assert_array_equal(ids, ids2)
    np.testing.assert_array_equal(y, y2)              # deterministic: no atomics on the data path
    return y, ids, weights


@pytest.mark.parametrize("tokens,experts,top_k", [(65, 16, 4), (100, 8, 2), (300, 16, 4), (129, 32, 6)])
def test_tensor_core_prefill_matches_the_oracle(gpu, tokens, experts, top_k):
    """65..300 tokens over few experts: groups of exactly 32, ragged last groups, several groups
    per expert; shared expert through the same kernels."""
    import oracle
    from picoforge_b200 import abi, synth
    spec = synth.make_layer(700 + tokens, routed_type=abi.Q4_K, shared_type=abi.Q4_K, experts=experts, top_k=top_k)
    x = synth.activations(700 + tokens, tokens)
    want = oracle.forward(spec, x, threads=synth.threads())
    y, ids, weights = _forward(gpu, spec, x, -1)
    np.testing.assert_array_equal(ids, want["ids"])
    np.testing.assert_array_equal(weights, want["weights"])
    error = np.abs(y - want["y"]).max()
    assert error <= Y_TOLERANCE, error
    # the CUDA-core kernels on the same input: both inside the bound, and close to each other
    y_cc, ids_cc, _ = _forward(gpu, spec, x, 0)
    np.testing.assert_array_equal(ids_cc, ids)
    assert np.abs(y - y_cc).max() <= Y_TOLERANCE


def test_tensor_core_prefill_accuracy_is_near_fp32(gpu):
    """Exact integer codes x (fp16 hi + lo) activations: the error against the FP32 oracle stays
    orders of magnitude under the bound (about 1e-6 at these magnitudes)."""
    import oracle
    from picoforge_b200 import abi, synth
    spec = synth.make_layer(801, routed_type=abi.Q4_K, shared_type=abi.Q4_K, experts=16, top_k=4)
    x = synth.activations(801, 96)
    want = oracle.forward(spec, x, threads=synth.threads())
    y, _, _ = _forward(gpu, spec, x, -1)
    assert np.abs(y - want["y"]).max() <= 2e-5
