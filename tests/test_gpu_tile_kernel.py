"""The tile kernels (groups of up to 16 rows per expert on the int8 tensor cores) against the CPU
oracle and against the four-row grouped kernels: route ids bit-exact, y within 1e-3 (max abs)."""
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).parent))

pytestmark = pytest.mark.gpu

Y_TOLERANCE = 1e-3


def _forward(gpu, spec, x, tile):
    from picoforge_b200.layer import MoeLayer
    gpu.lib.qw4cu_set_tile_path(tile)
    try:
        with MoeLayer(gpu, spec, x.shape[0]) as layer:
            gpu.lib.qw4cu_launch_log_begin()
            y, ids, weights = layer.forward(x)
            names = gpu.launch_names()
            y2, _, _ = layer.forward(x)
    finally:
        gpu.lib.qw4cu_set_tile_path(-1)
    np.testing.assert_array_equal(y, y2)              # deterministic
    return y, ids, weights, names


@pytest.mark.parametrize("routed,shared,tokens,experts,top_k", [
    (12, 12, 5, 64, 10),      # one ragged column tile
    (16, 12, 16, 64, 10),     # IQ2_XXS routed + Q4_K shared
    (12, 16, 33, 64, 6),      # dense shared groups of 16 + 16 + 1
    (16, 16, 64, 16, 4),      # every expert sees several column tiles; groups split at 16 rows
    (16, 12, 100, 64, 10),    # beyond the small-batch dispatch: bitmap dispatch + tile kernels
    (10, 12, 7, 64, 10),      # Q2_K routed: scales folded into the codes, minima through a second MMA
    (10, 10, 40, 32, 6),      # Q2_K everywhere
    (10, 12, 130, 64, 10),
])
def test_tile_kernels_match_the_oracle(gpu, routed, shared, tokens, experts, top_k):
    import oracle
    from picoforge_b200 import synth
    spec = synth.make_layer(900 + routed + tokens, routed_type=routed, shared_type=shared, experts=experts, top_k=top_k)
    x = synth.activations(900 + tokens, tokens)
    want = oracle.forward(spec, x, threads=synth.threads())
    y, ids, weights, names = _forward(gpu, spec, x, 1)
    assert names.count("expert_tile_kernel") == 4, names
    assert "grouped_mma_kernel" not in names
    np.testing.assert_array_equal(ids, want["ids"])
    np.testing.assert_array_equal(weights, want["weights"])
    assert np.abs(y - want["y"]).max() <= Y_TOLERANCE
    if tokens > 64 or routed == 10:
        assert _forward(gpu, spec, x, -1)[3].count("expert_tile_kernel") == 4       # the automatic choice for IQ2_XXS beyond 64 rows and for Q2_K
    else:
        y4, ids4, _, names4 = _forward(gpu, spec, x, 0)
        assert "expert_tile_kernel" not in names4
        np.testing.assert_array_equal(ids4, ids)
        assert np.abs(y - y4).max() <= Y_TOLERANCE


def test_tile_kernels_at_config_shapes(gpu):
    """512 experts, top-10, 64 single-token streams (the batched-decode configuration), Q4_K."""
    import oracle
    from picoforge_b200 import abi, synth
    spec = synth.make_layer(3, routed_type=abi.Q4_K, shared_type=abi.Q4_K)
    x = synth.activations(3, 64)
    want = oracle.forward(spec, x, threads=synth.threads())
    y, ids, weights, names = _forward(gpu, spec, x, 1)
    assert names.count("expert_tile_kernel") == 4, names
    np.testing.assert_array_equal(ids, want["ids"])
    assert np.abs(y - want["y"]).max() <= Y_TOLERANCE


def test_skewed_routing_fills_whole_groups(gpu):
    """A router that sends every token to the same experts: each list splits into full 16-row groups."""
    import oracle
    from picoforge_b200 import abi, synth
    spec = synth.make_layer(11, routed_type=abi.IQ2_XXS, shared_type=abi.Q4_K, experts=64, top_k=4)
    router = spec.tensors[0].view(np.float32).reshape(64, -1).copy()
    router[:] = 0.0
    spec.tensors[0] = router.reshape(-1).view(np.uint8)           # all logits equal: the lowest four ids win for every token
    x = synth.activations(11, 48)
    want = oracle.forward(spec, x, threads=synth.threads())
    y, ids, _, names = _forward(gpu, spec, x, 1)
    assert names.count("expert_tile_kernel") == 4
    np.testing.assert_array_equal(ids, want["ids"])
    assert (ids == np.arange(4, dtype=np.uint32)).all()
    assert np.abs(y - want["y"]).max() <= Y_TOLERANCE


def test_q2k_decode_takes_the_tile_kernels(gpu):
    """Q2_K has no one-kernel decode path: one or two tokens still run on the tensor cores."""
    import oracle
    from picoforge_b200 import abi, synth
    spec = synth.make_layer(21, routed_type=abi.Q2_K, shared_type=abi.Q2_K, experts=64, top_k=10)
    x = synth.activations(21, 2)
    want = oracle.forward(spec, x, threads=synth.threads())
    y, ids, _, names = _forward(gpu, spec, x, -1)
    assert names.count("expert_tile_kernel") == 4, names
    np.testing.assert_array_equal(ids, want["ids"])
    assert np.abs(y - want["y"]).max() <= Y_TOLERANCE
