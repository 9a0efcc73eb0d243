"""Parity at the shapes and routing laws of the sharded benchmark configurations, on the
kernels the library picks by itself:

* the 1024-token prefill chunk with Q2_K routed + Q4_K shared experts and uniform routing;
* the 64-stream batched decode with Q4_K experts and Zipf(1.1) expert popularity;
* a three-layer stack fed layer to layer.

Route ids and the whole-chunk per-expert lists are bit-exact against the CPU oracle; y holds
1e-3 (max abs).  The reference's own kernel metric |y - y_oracle| / sum|w . a| (picoforge
tests/qwen4_kernel_tolerances.json:3, bound 2^-22 for its FP32 down+reduce kernels, 2^-11 for
its half-operand tensor mode) is computed for a few tokens per path and printed.
"""
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).parent))
import oracle  # noqa: E402
from picoforge_b200 import abi, synth  # noqa: E402
from picoforge_b200.layer import MoeLayer, group_pairs  # noqa: E402

pytestmark = pytest.mark.gpu
Y_TOLERANCE = 1e-3


def full_ids(spec, x):
    """Route ids of every token from the oracle's router product and routing alone (cheap)."""
    router = spec.tensors[0]
    logits = oracle.matmul(abi.F32, router, spec.hidden, spec.hidden, spec.experts, x)
    return oracle.route(logits, spec.top_k, spec.norm)[1]


def relative_metric(spec, x_row, ids_row, weights_row, y_got, y_want):
    """max_c |y_got - y_want| / S[c], S = sum over the selected experts (and the shared one) of
    route weight x sum_j |down[c, j] * act[j]|: the reference's kernel metric (b) applied to the
    down + combine stage, in float64 from the oracle's decoded weights."""
    def expert(gate, up, down, inter):
        g = oracle.decode_rows(gate[0], gate[1], inter, spec.hidden).astype(np.float64) @ x_row
        u = oracle.decode_rows(up[0], up[1], inter, spec.hidden).astype(np.float64) @ x_row
        a = g / (1.0 + np.exp(-g)) * u
        d = oracle.decode_rows(down[0], down[1], spec.hidden, spec.down_physical if down[2] else inter).astype(np.float64)[:, :inter]
        return np.abs(d * a[None, :]).sum(axis=1)
    layouts = spec.layouts()
    s = np.zeros(spec.hidden)
    for e, w in zip(ids_row, weights_row):
        part = lambda i: (spec.types[i], spec.tensors[i][int(e) * layouts[i].expert_bytes:(int(e) + 1) * layouts[i].expert_bytes], i == 3)  # noqa: E731
        s += float(w) * expert(part(1), part(2), part(3), spec.inter)
    shared_logit = float(spec.tensors[7].view(np.float32).astype(np.float64) @ x_row)
    s += 1.0 / (1.0 + np.exp(-shared_logit)) * expert((spec.types[4], spec.tensors[4], False), (spec.types[5], spec.tensors[5], False),
                                                      (spec.types[6], spec.tensors[6], False), spec.shared_inter)
    return float((np.abs(y_got.astype(np.float64) - y_want) / np.maximum(s, 2.0 ** -126)).max())


def report_metric(name, spec, x, rows, ids, weights, y, want_y):
    worst = max(relative_metric(spec, x[r].astype(np.float64), ids[r], weights[r], y[r], want_y[i]) for i, r in enumerate(rows))
    print(f"\n[{name}] |y - y_oracle| / sum|w.a| over {len(rows)} tokens: {worst:.3g} = 2^{np.log2(max(worst, 1e-300)):.1f}")
    assert worst <= 2.0 ** -11
    return worst


def test_prefill_chunk_q2k_uniform_routing_default_path(gpu):
    spec = synth.make_layer(3, layer=0, routed_type=abi.Q2_K, shared_type=abi.Q4_K)
    x = synth.activations(3, 1024)
    want_ids = full_ids(spec, x)
    sample = np.arange(0, 1024, 8)                           # 128 tokens through the whole oracle layer
    want = oracle.forward(spec, x[sample], threads=synth.threads())
    np.testing.assert_array_equal(want["ids"], want_ids[sample])
    with MoeLayer(gpu, spec, 1024) as layer:
        gpu.lib.qw4cu_launch_log_begin()
        y, ids, weights = layer.forward(x)
        names = gpu.launch_names()
    assert "expert_tile_kernel" in names or "prefill_tc_kernel" in names, names     # a tensor-core path, chosen automatically
    assert "gate_up_kernel" not in names
    np.testing.assert_array_equal(ids, want_ids)
    assert np.isfinite(y).all()
    assert np.abs(y[sample].astype(np.float64) - want["y"]).max() <= Y_TOLERANCE
    got = group_pairs(gpu, ids, spec.experts)
    for a, b in zip(got, oracle.group(want_ids, spec.experts)):
        np.testing.assert_array_equal(a, b)
    report_metric("c3 chunk, " + "+".join(sorted(set(names) & {"expert_tile_kernel", "prefill_tc_kernel"})), spec, x, sample[:3], ids, weights,
                  y, want["y"])


def c4_layer(layer_index):
    spec = synth.make_layer(4, layer=layer_index, routed_type=abi.Q4_K, shared_type=abi.Q4_K)
    synth.zipf_router_bias(spec, 4 + layer_index)
    return spec


def test_batched_decode_zipf_default_path(gpu):
    spec = c4_layer(0)
    x = synth.activations(4, 64)
    x[:, 0] = 1.0
    want = oracle.forward(spec, x, threads=synth.threads())
    counts = np.bincount(want["ids"].reshape(-1), minlength=spec.experts)
    assert counts.max() >= 4 * max(1, int(np.median(counts[counts > 0])))       # skewed popularity
    with MoeLayer(gpu, spec, 64) as layer:
        gpu.lib.qw4cu_launch_log_begin()
        y, ids, weights = layer.forward(x)
        names = gpu.launch_names()
    assert "grouped_mma_kernel" in names or "expert_tile_kernel" in names, names
    assert "gate_up_kernel" not in names and "fused_decode_kernel" not in names
    np.testing.assert_array_equal(ids, want["ids"])
    assert np.abs(y.astype(np.float64) - want["y"]).max() <= Y_TOLERANCE
    report_metric("c4 layer, " + "+".join(sorted(set(names) & {"grouped_mma_kernel", "expert_tile_kernel"})), spec, x, [0, 31, 63], ids,
                  weights, y, want["y"][[0, 31, 63]])


def test_decode_one_kernel_path_metric(gpu):
    """The reference's relative metric on the one-kernel decode path (4 tokens, IQ2_XXS routed)."""
    spec = synth.make_layer(1, routed_type=abi.IQ2_XXS, shared_type=abi.Q4_K)
    x = synth.activations(1, 4)
    want = oracle.forward(spec, x, threads=synth.threads())
    with MoeLayer(gpu, spec, 4) as layer:
        gpu.lib.qw4cu_launch_log_begin()
        y, ids, weights = layer.forward(x)
        names = gpu.launch_names()
    assert names == ["fused_decode_kernel"], names
    np.testing.assert_array_equal(ids, want["ids"])
    report_metric("c1 decode, fused_decode_kernel", spec, x, [0, 3], ids, weights, y, want["y"][[0, 3]])


def test_tensor_core_prefill_path_metric(gpu):
    """The same metric on the tcgen05 prefill path (Q4_K, more than 64 tokens): exact integer codes and a 22-bit
    hi + lo split of the activations, so it lands orders of magnitude under the int8-digit paths."""
    spec = synth.make_layer(2, routed_type=abi.Q4_K, shared_type=abi.Q4_K, experts=64, top_k=6)
    x = synth.activations(2, 96)
    want = oracle.forward(spec, x, threads=synth.threads())
    with MoeLayer(gpu, spec, 96) as layer:
        gpu.lib.qw4cu_launch_log_begin()
        y, ids, weights = layer.forward(x)
        names = gpu.launch_names()
    assert "prefill_tc_kernel" in names and "expert_tile_kernel" not in names, names
    np.testing.assert_array_equal(ids, want["ids"])
    worst = report_metric("96-token prefill, prefill_tc_kernel", spec, x, [0, 47, 95], ids, weights, y, want["y"][[0, 47, 95]])
    assert worst <= 2.0 ** -20


def test_three_layer_stack_fed_layer_to_layer(gpu):
    """Layer l + 1 reads the GPU's output of layer l, brought back to unit RMS on the host (the
    engine has norms and other blocks in between).  Every layer is checked against the oracle run
    on the very input the GPU layer saw: ids bit-exact, y within the tolerance."""
    x = synth.activations(4, 64)
    x[:, 0] = 1.0
    for index in range(3):
        spec = c4_layer(index)
        want = oracle.forward(spec, x, threads=synth.threads())
        with MoeLayer(gpu, spec, 64) as layer:
            y, ids, _ = layer.forward(x)
        np.testing.assert_array_equal(ids, want["ids"], err_msg=f"layer {index}")
        assert np.abs(y.astype(np.float64) - want["y"]).max() <= Y_TOLERANCE, index
        x = (y / np.sqrt(np.mean(y.astype(np.float64) ** 2, axis=1, keepdims=True))).astype(np.float32)
        x[:, 0] = 1.0                                         # the constant column that carries the popularity bias
