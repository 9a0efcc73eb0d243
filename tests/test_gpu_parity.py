"""GPU parity tests: every call goes through the C ABI of the CUDA library and is compared
with the CPU oracle (and with the golden vectors generated from the reference's objects).

Bars: decoded weights, route ids, per-expert lists: bit-exact.  Probabilities and route
weights: bit-exact in the exact router mode.  Layer output y: max |y - y_oracle| <= 1e-3
(the reference's stated end-to-end tolerance), checked together with a relative bound.
"""
import ctypes as C
import hashlib
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).parent))
import cases  # noqa: E402
import oracle  # noqa: E402
from golden.make_golden import FORWARD_CASES, forward_case  # noqa: E402
from picoforge_b200 import abi, synth  # noqa: E402
from picoforge_b200.layer import LayerSpec, MoeLayer, group_pairs, route  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = np.load(Path(__file__).parent / "golden" / "golden.npz")
Y_TOLERANCE = 1e-3


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def check_layer(out, y, ids, weights, exact_weights=True):
    np.testing.assert_array_equal(ids, out["ids"])
    if exact_weights:
        np.testing.assert_array_equal(bits(weights), bits(out["weights"]))
    else:
        np.testing.assert_allclose(weights, out["weights"], atol=2e-6, rtol=2e-5)
    assert np.isfinite(y).all()
    error = np.abs(y.astype(np.float64) - out["y"]).max()
    assert error <= Y_TOLERANCE, error
    rms = np.sqrt(np.mean(out["y"].astype(np.float64) ** 2))
    assert np.sqrt(np.mean((y.astype(np.float64) - out["y"]) ** 2)) <= 1e-4 * max(rms, 1e-6)
    return error


# ---- dequantised weights: bit-exact -------------------------------------------------------
@pytest.mark.parametrize("gguf_type", [abi.Q4_K, abi.Q2_K, abi.IQ2_XXS, abi.Q8_0, abi.MXFP4, abi.F16, abi.BF16])
def test_resident_image_decodes_to_the_reference_bits(gpu, gguf_type):
    """The exhaustive block patterns, uploaded as the routed gate tensor (so they go through the
    regrouping of the resident layout), decode to the oracle's bits and the golden hash."""
    _, block, size = abi.FORMATS[gguf_type]
    blocks = cases.pattern_blocks(gguf_type)
    hidden = 256 if block != 1 else 64
    per_row = hidden // block
    experts, inter = 8, len(blocks) // per_row // 8
    spec = LayerSpec(hidden, experts, 2, inter, 32 if block == 1 else 256, inter, True,
                     (abi.F32, gguf_type, abi.F32, abi.F32, abi.F32, abi.F32, abi.F32, abi.F32))
    rng = np.random.default_rng(1)
    spec.tensors = [np.zeros(l.tensor_bytes, np.uint8) for l in spec.layouts()]
    spec.tensors[1] = blocks.reshape(-1)[:spec.layouts()[1].tensor_bytes].copy()
    want = oracle.decode_rows(gguf_type, spec.tensors[1], experts * inter, hidden)
    with MoeLayer(gpu, spec, 1) as layer:
        got = np.concatenate([layer.decode_rows(1, e, 0, inter) for e in range(experts)])
    np.testing.assert_array_equal(bits(got), bits(want))
    if block == hidden or block == 1:
        flat = got.reshape(-1, block) if block != 1 else got.reshape(-1, 1)
        assert hashlib.sha256(flat.tobytes()).digest() == GOLDEN[f"decode_{gguf_type}_sha256"].tobytes()


@pytest.mark.parametrize("routed", [abi.Q4_K, abi.Q2_K, abi.IQ2_XXS])
def test_decode_at_layer_shapes(gpu, routed):
    """Rows of 8 blocks (K = 2048) and of 2 blocks (K = 512), several experts, all three tensors."""
    spec = synth.make_layer(21, routed_type=routed, shared_type=abi.Q4_K, experts=4, top_k=2)
    with MoeLayer(gpu, spec, 1) as layer:
        for tensor in (1, 2, 3, 4, 6):
            k, _, n_out, n_experts = spec.shapes()[tensor]
            rb = abi.row_bytes(spec.types[tensor], k)
            for expert in {0, n_experts - 1}:
                got = layer.decode_rows(tensor, expert, n_out - 16, 16)
                raw = spec.tensors[tensor][(expert * n_out + n_out - 16) * rb:(expert + 1) * n_out * rb]
                np.testing.assert_array_equal(bits(got), bits(oracle.decode_rows(spec.types[tensor], raw, 16, k)))


def test_expanded_image_decodes_to_the_oracle_bits(gpu):
    """The second resident image of IQ2_XXS expert tensors (4-bit codes, read by the one-kernel decode path): whole
    rows of every expert tensor, routed and shared, against the oracle's decode of the GGUF bytes, bit for bit."""
    import ctypes as C
    spec = synth.make_layer(22, routed_type=abi.IQ2_XXS, shared_type=abi.IQ2_XXS, experts=4, top_k=2)
    with MoeLayer(gpu, spec, 1) as layer:
        for tensor in (1, 2, 3, 4, 5, 6):
            k, _, n_out, n_experts = spec.shapes()[tensor]
            rb = abi.row_bytes(spec.types[tensor], k)
            for expert, row0, rows in ((0, 0, 24), (n_experts - 1, n_out - 40, 40)):
                got = np.empty((rows, k), np.float32)
                err = abi.Qwen4Error()
                st = gpu.lib.qw4cu_moe_decode_rows_expanded(layer.moe, tensor, expert, row0, rows, got.ctypes.data, got.size, C.byref(err))
                assert st == 0, err.detail
                raw = spec.tensors[tensor][(expert * n_out + row0) * rb:(expert * n_out + row0 + rows) * rb]
                np.testing.assert_array_equal(bits(got), bits(oracle.decode_rows(spec.types[tensor], raw, rows, k)))
    other = synth.make_layer(23, routed_type=abi.Q4_K, shared_type=abi.Q4_K, experts=4, top_k=2)
    with MoeLayer(gpu, other, 1) as layer:                                      # no IQ2_XXS tensor: no expanded image
        got = np.empty((1, other.hidden), np.float32)
        err = abi.Qwen4Error()
        assert gpu.lib.qw4cu_moe_decode_rows_expanded(layer.moe, 1, 0, 0, 1, got.ctypes.data, got.size, C.byref(err)) == abi.UNSUPPORTED


# ---- routing -------------------------------------------------------------------------------
def test_route_known_answers(gpu):
    z = np.array([[0.0, 1e-9, 0.0, -1e-9], [0.0, 2.0, 2.0, -1000.0]], np.float32)
    probs, ids, weights = route(gpu, z, 2, True)
    np.testing.assert_array_equal(ids, [[0, 1], [1, 2]])
    np.testing.assert_array_equal(weights, [[0.5, 0.5], [0.5, 0.5]])
    assert probs[0, 0] == 0.25 and probs[1, 3] == 0.0
    assert route(gpu, z, 2, False)[2][0, 0] == 0.25
    z[0, 0], z[0, 1] = -3e38, 3e38
    _, ids, weights = route(gpu, z, 2, True)
    assert list(ids[0]) == [1, 0] and list(weights[0]) == [1.0, 0.0]
    for bad in (np.nan, np.inf):
        z[1, 2] = bad
        with pytest.raises(abi.MoeError) as info:
            route(gpu, z, 2, True)
        assert info.value.status == abi.NONFINITE and info.value.row == 1


def test_route_matches_golden_and_oracle(gpu):
    for seed in range(4):
        for norm in (0, 1):
            tag = f"route_{seed}_{norm}"
            k = GOLDEN[tag + "_ids"].shape[1]
            probs, ids, weights = route(gpu, GOLDEN[tag + "_logits"], k, bool(norm))
            np.testing.assert_array_equal(ids, GOLDEN[tag + "_ids"])
            np.testing.assert_array_equal(bits(probs), bits(GOLDEN[tag + "_probs"]))
            np.testing.assert_array_equal(bits(weights), bits(GOLDEN[tag + "_weights"]))
    rng = np.random.default_rng(3811)
    for (t, e, k) in [(1024, 17, 5), (33, 512, 10), (1000, 512, 10), (3, 2048, 32), (9, 33, 33)]:
        logits = (rng.standard_normal((t, e + 3)) * 4).astype(np.float32)[:, :e]      # padded rows
        logits[::7, : min(e, 3)] = logits[::7, :1]                                   # ties
        probs, ids, weights = route(gpu, logits, k, True)
        want = oracle.route(logits, k, True)
        np.testing.assert_array_equal(ids, want[1])
        np.testing.assert_array_equal(bits(probs), bits(want[0]))
        np.testing.assert_array_equal(bits(weights), bits(want[2]))


# ---- dispatch lists ----------------------------------------------------------------------------
def test_group_matches_golden_oracle_and_stable_argsort(gpu):
    for seed in range(3):
        tag = f"group_{seed}"
        ids = GOLDEN[tag + "_ids"]
        offsets, p2r, r2p = group_pairs(gpu, ids, len(GOLDEN[tag + "_offsets"]) - 1)
        np.testing.assert_array_equal(offsets, GOLDEN[tag + "_offsets"])
        np.testing.assert_array_equal(p2r, GOLDEN[tag + "_p2r"])
        np.testing.assert_array_equal(r2p, GOLDEN[tag + "_r2p"])
    rng = np.random.default_rng(3812)
    for (t, e, k) in [(1024, 512, 10), (1, 512, 10), (64, 512, 10), (300, 7, 7), (2048, 2048, 1)]:
        popularity = rng.random(e) ** 4 + 1e-6
        ids = np.stack([rng.choice(e, k, replace=False, p=popularity / popularity.sum()) for _ in range(t)]).astype(np.uint32)
        offsets, p2r, r2p = group_pairs(gpu, ids, e)
        want = oracle.group(ids, e)
        np.testing.assert_array_equal(offsets, want[0])
        np.testing.assert_array_equal(p2r, want[1])
        np.testing.assert_array_equal(r2p, want[2])
        np.testing.assert_array_equal(r2p, np.argsort(ids.reshape(-1), kind="stable"))
    offsets, p2r, r2p = group_pairs(gpu, np.zeros((0, 2), np.uint32), 4)
    assert offsets.tolist() == [0] * 5 and len(p2r) == 0


# ---- whole layer ---------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(FORWARD_CASES))
def test_forward_matches_golden(gpu, name):
    spec, x = forward_case(name)
    with MoeLayer(gpu, spec, len(x)) as layer:
        y, ids, weights = layer.forward(x)
    np.testing.assert_array_equal(ids, GOLDEN[f"fwd_{name}_ids"])
    np.testing.assert_array_equal(bits(weights), bits(GOLDEN[f"fwd_{name}_weights"]))
    assert np.abs(y - GOLDEN[f"fwd_{name}_y"]).max() <= Y_TOLERANCE


def test_analytic_block(gpu):
    spec = LayerSpec(1, 2, 1, 1, 1, 1, True, (abi.F32,) * 8)
    f = lambda *v: np.array(v, np.float32).view(np.uint8)
    spec.tensors = [f(2, 1), f(1, 2), f(3, 4), f(5, 6), f(1), f(2), f(3), f(0)]
    with MoeLayer(gpu, spec, 1) as layer:
        y, ids, weights = layer.forward(np.ones((1, 1), np.float32))
    sigmoid1 = 1 / (1 + np.exp(-1.0))
    assert ids.tolist() == [[0]] and weights.tolist() == [[1.0]]
    np.testing.assert_allclose(y, 18 * sigmoid1, rtol=2e-6)


def config_layer(index):
    """The benchmark configurations at full layer shapes (hidden 2048, 512 experts, top-10)."""
    if index == 0:
        return synth.make_layer(0, routed_type=abi.Q4_K, shared_type=abi.Q4_K), synth.activations(0, 1)
    if index == 1:
        spec = synth.make_layer(1, routed_type=abi.IQ2_XXS, shared_type=abi.Q4_K)
        x = synth.activations(1, 4)
        synth.correlated_tokens(x, 1, 0, 1, 0.95)
        return spec, x
    spec = synth.make_layer(0, routed_type=abi.Q4_K, shared_type=abi.Q4_K)
    synth.zipf_router_bias(spec, 2)
    x = synth.activations(2, 1024)
    x[:, 0] = 1.0
    return spec, x


@pytest.mark.parametrize("mode", [0, 1])
def test_config0_single_token_q4k(gpu, mode):
    spec, x = config_layer(0)
    out = oracle.forward(spec, x, threads=synth.threads())
    gpu.lib.qw4cu_set_router_mode(mode)
    try:
        with MoeLayer(gpu, spec, 1) as layer:
            y, ids, weights = layer.forward(x)
    finally:
        gpu.lib.qw4cu_set_router_mode(0)
    check_layer(out, y, ids, weights, exact_weights=mode == 0)


@pytest.mark.parametrize("mode", [0, 1])
def test_config1_four_tokens_iq2xxs(gpu, mode):
    spec, x = config_layer(1)
    out = oracle.forward(spec, x, threads=synth.threads())
    shared = len(set(out["ids"][0]) & set(out["ids"][1]))
    assert shared >= 5, shared                      # the configuration asks for >= 5 shared experts
    gpu.lib.qw4cu_set_router_mode(mode)
    try:
        with MoeLayer(gpu, spec, 4) as layer:
            y, ids, weights = layer.forward(x)
            y2, ids2, _ = layer.forward(x)           # same workspace twice: no state carried over
    finally:
        gpu.lib.qw4cu_set_router_mode(0)
    check_layer(out, y, ids, weights, exact_weights=mode == 0)
    np.testing.assert_array_equal(bits(y), bits(y2))
    np.testing.assert_array_equal(ids, ids2)


def test_config2_prefill_chunk_zipf(gpu):
    spec, x = config_layer(2)
    out = oracle.forward(spec, x, threads=synth.threads())
    counts = np.bincount(out["ids"].reshape(-1), minlength=spec.experts)
    assert counts.max() > 8 * np.median(counts[counts > 0])       # skewed popularity
    with MoeLayer(gpu, spec, 1024) as layer:
        y, ids, weights = layer.forward(x)
        check_layer(out, y, ids, weights)
        # a token's result does not depend on the rest of the batch (ragged tail, 37 tokens)
        y_tail, ids_tail, _ = layer.forward(x[-37:])
    np.testing.assert_array_equal(ids_tail, out["ids"][-37:])
    assert np.abs(y_tail - out["y"][-37:]).max() <= Y_TOLERANCE
    want = oracle.group(out["ids"], spec.experts)
    got = group_pairs(gpu, ids, spec.experts)
    for a, b in zip(got, want):
        np.testing.assert_array_equal(a, b)


@pytest.mark.parametrize("path", [0, 1])
@pytest.mark.parametrize("routed,shared,tokens", [(abi.Q4_K, abi.Q4_K, 1), (abi.IQ2_XXS, abi.Q4_K, 4), (abi.Q4_K, abi.IQ2_XXS, 23),
                                                  (abi.IQ2_XXS, abi.IQ2_XXS, 70)])
def test_both_expert_paths(gpu, path, routed, shared, tokens):
    """The CUDA-core kernels (path 0) and the tensor-core grouped kernels (path 1) both hold the
    tolerance; 23 and 70 tokens over 16 experts give groups of more than four rows."""
    spec = synth.make_layer(60 + routed + tokens, routed_type=routed, shared_type=shared, experts=16, top_k=4)
    x = synth.activations(60 + tokens, tokens)
    out = oracle.forward(spec, x, threads=synth.threads())
    gpu.lib.qw4cu_set_expert_path(path)
    try:
        with MoeLayer(gpu, spec, tokens) as layer:
            y, ids, weights = layer.forward(x)
    finally:
        gpu.lib.qw4cu_set_expert_path(-1)
    check_layer(out, y, ids, weights)


@pytest.mark.parametrize("routed,shared", [(abi.Q2_K, abi.Q4_K), (abi.Q4_K, abi.Q2_K), (abi.IQ2_XXS, abi.IQ2_XXS)])
def test_mixed_formats_small(gpu, routed, shared):
    spec = cases.small_layer(90 + routed, routed, shared, experts=32, top_k=6)
    x = synth.activations(9, 70, spec.hidden)
    out = oracle.forward(spec, x, threads=synth.threads())
    with MoeLayer(gpu, spec, 70) as layer:
        y, ids, weights = layer.forward(x)
    check_layer(out, y, ids, weights)


def test_k_padding_and_generic_formats(gpu):
    """Routed down stored with 512 columns of which 256 are logical; Q8_0 shared expert; F16 gate."""
    spec = synth.make_layer(5, routed_type=abi.Q2_K, shared_type=abi.Q4_K, experts=4, top_k=2, hidden=256,
                            inter=256, shared_inter=256)
    spec.down_physical = 512
    spec.tensors[3] = synth.tensor(abi.Q2_K, 5, 3, spec.hidden * spec.experts, 512)
    rng = np.random.default_rng(5)
    types = list(spec.types)
    for index in (4, 5, 6):
        k, _, n, ex = spec.shapes()[index]
        blocks = rng.integers(0, 256, (n * ex * k // 32, 34), dtype=np.uint8)
        blocks[:, :2] = np.float16(rng.uniform(1e-4, 4e-4, len(blocks))).view(np.uint8).reshape(-1, 2)
        spec.tensors[index], types[index] = blocks.reshape(-1), abi.Q8_0
    spec.types = tuple(types)
    x = synth.activations(5, 3, spec.hidden)
    out = oracle.forward(spec, x)
    with MoeLayer(gpu, spec, 3) as layer:
        y, ids, weights = layer.forward(x)
    check_layer(out, y, ids, weights)


# ---- lifecycle and errors (picoforge tests/test_qwen4_moe.c:234-287) ---------------------------
def test_lifecycle_and_error_latch(gpu):
    lib = gpu.lib
    spec = cases.float_layer(3)
    for t in spec.tensors:
        t[:] = 0
    layer = MoeLayer(gpu, spec, 1024)
    err = abi.Qwen4Error()
    x = np.zeros((2, 8), np.float32)
    y = np.full((2, 8), -99, np.float32)

    def forward(xv, yv, work=None):
        return lib.qwen4_moe_forward(layer.moe, xv, yv, None, work or layer.work, C.byref(err))

    alias = abi.f32_view(y); alias.data = x.ctypes.data
    assert forward(abi.f32_view(x), alias) == abi.INVALID_ARGUMENT
    short = abi.f32_view(y); short.capacity_bytes = 63
    assert forward(abi.f32_view(x), short) == abi.CAPACITY
    pitch = abi.f32_view(y); pitch.stride_bytes[0] = 28
    assert forward(abi.f32_view(x), pitch) == abi.STRIDE
    onto_weights = abi.f32_view(y); onto_weights.data = spec.tensors[1].ctypes.data
    assert forward(abi.f32_view(x), onto_weights) == abi.INVALID_ARGUMENT
    assert (y == -99).all()
    assert forward(abi.f32_view(x), abi.f32_view(y)) == abi.OK and (y == 0).all()      # zero weights -> zero y
    y[:] = -99
    x[1, 3] = np.inf
    assert forward(abi.f32_view(x), abi.f32_view(y)) == abi.NONFINITE and (y == -99).all()
    x[1, 3] = 0
    assert forward(abi.f32_view(x), abi.f32_view(y)) == abi.OK                          # bad input does not latch
    big = np.zeros((2000, 8), np.float32)
    assert forward(abi.f32_view(big), abi.f32_view(np.zeros_like(big))) == abi.CAPACITY
    empty = abi.f32_view(None, 0, 8)
    assert forward(empty, empty) == abi.OK
    other = MoeLayer(gpu, spec, 4)
    assert forward(abi.f32_view(x), abi.f32_view(y), other.work) == abi.OWNER
    other.close()
    lib.qwen4_moe_destroy(layer.moe)                   # workspace keeps the image alive
    assert lib.qwen4_moe_work_reset(layer.work, C.byref(err)) == abi.BAD_STATE
    assert forward(abi.f32_view(x), abi.f32_view(y)) == abi.BAD_STATE
    lib.qwen4_moe_work_destroy(layer.work)
    layer.moe = layer.work = C.c_void_p()

    # a nonfinite WEIGHT fails inside the layer: NONFINITE, then BAD_STATE until reset
    spec = cases.float_layer(4)
    spec.tensors[1].view(np.float32)[0] = np.nan
    x = np.ones((2, 8), np.float32)
    y[:] = -99
    with MoeLayer(gpu, spec, 2) as poisoned:
        st = lib.qwen4_moe_forward(poisoned.moe, abi.f32_view(x), abi.f32_view(y), None, poisoned.work, C.byref(err))
        if st == abi.OK:      # expert 0 not routed for these tokens: poison the router instead
            pytest.skip("poisoned expert not selected")
        assert st == abi.NONFINITE and (y == -99).all()
        assert lib.qwen4_moe_forward(poisoned.moe, abi.f32_view(x), abi.f32_view(y), None, poisoned.work, C.byref(err)) == abi.BAD_STATE
        assert lib.qwen4_moe_work_reset(poisoned.work, C.byref(err)) == abi.OK
        assert lib.qwen4_moe_forward(poisoned.moe, abi.f32_view(x), abi.f32_view(y), None, poisoned.work, C.byref(err)) == abi.NONFINITE


def test_work_size_budget(gpu):
    spec = cases.float_layer(6)
    lib, err = gpu.lib, abi.Qwen4Error()
    with MoeLayer(gpu, spec, 8) as layer:
        size = C.c_size_t()
        assert lib.qwen4_moe_work_size(layer.moe, 1024, C.byref(size), C.byref(err)) == abi.OK and size.value > 0
        assert size.value <= 32 << 20                  # the engine's per-layer host budget
        work = C.c_void_p()
        assert lib.qwen4_moe_work_create(layer.moe, 1024, size.value - 1, C.byref(work), C.byref(err)) == abi.CAPACITY
        assert not work
        assert lib.qwen4_moe_work_create(layer.moe, 0, size.value, C.byref(work), C.byref(err)) == abi.OK
        x = np.zeros((1, 8), np.float32)
        assert lib.qwen4_moe_forward(layer.moe, abi.f32_view(x), abi.f32_view(x.copy()), None, work, C.byref(err)) == abi.CAPACITY
        lib.qwen4_moe_work_destroy(work)
        assert lib.qw4cu_moe_work_device_bytes(layer.work) > 0 and lib.qw4cu_moe_device_bytes(layer.moe) > 0


def test_device_pointer_forward_matches_host_forward(gpu):
    lib, err = gpu.lib, abi.Qwen4Error()
    spec = cases.small_layer(31, abi.Q4_K, abi.Q4_K)
    x = synth.activations(31, 6, spec.hidden)
    with MoeLayer(gpu, spec, 6) as layer:
        y, ids, _ = layer.forward(x)
        dx, dy = lib.qw4cu_malloc(x.nbytes), lib.qw4cu_malloc(x.nbytes)
        dids = lib.qw4cu_malloc(ids.nbytes)
        assert lib.qw4cu_upload(dx, x.ctypes.data, x.nbytes) == 0
        launches = lib.qw4cu_launch_count()
        assert lib.qw4cu_moe_forward_device(layer.moe, dx, dy, 6, dids, None, layer.work, C.byref(err)) == abi.OK
        assert lib.qw4cu_moe_work_sync(layer.work, C.byref(err)) == abi.OK
        assert lib.qw4cu_launch_count() > launches
        y2, ids2 = np.empty_like(y), np.empty_like(ids)
        assert lib.qw4cu_download(y2.ctypes.data, dy, y.nbytes) == 0 and lib.qw4cu_download(ids2.ctypes.data, dids, ids.nbytes) == 0
        for p in (dx, dy, dids):
            lib.qw4cu_free(p)
    np.testing.assert_array_equal(bits(y), bits(y2))
    np.testing.assert_array_equal(ids, ids2)
