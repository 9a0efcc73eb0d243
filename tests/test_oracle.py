"""CPU tests of the oracle: pins against the reference's known-answer tests, against the
golden vectors generated from the reference's own objects, and (where those objects are
present) against the reference live."""
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
from picoforge_b200.layer import MoeLayer, group_pairs, route  # noqa: E402

GOLDEN = np.load(Path(__file__).parent / "golden" / "golden.npz")
needs_reference = pytest.mark.skipif(not oracle.reference_available(), reason="reference objects not built here")


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def test_iq2xxs_codebook_is_the_published_table():
    text = (Path(__file__).parents[1] / "picoforge_b200/csrc/iq2xxs_codebook.h").read_text()
    body = text[text.index("#define QW4_IQ2XXS_LEVEL_LIST"):]
    words = [int(w, 16) for w in __import__("re").findall(r"0x([0-9a-f]{4})", body)]
    assert len(words) == 256
    raw = bytearray()
    for w in words:
        for j in range(8):
            level = (w >> (2 * j)) & 3
            raw.append(8 + 17 * level + (level >> 1))
    assert hashlib.sha256(raw).hexdigest() == "05826b5d3e472a3a78f196be62ac78acf81df0f909626e12ab9fa2a5d490dd54"


def test_q2k_known_block():
    # picoforge tests/test_qwen4_packed.c:16-33: scale byte 0x23, codes 0xE4, d = 1, dmin = 0.5
    block = np.zeros(84, np.uint8)
    block[:16], block[16:80], block[81], block[83] = 0x23, 0xE4, 0x3C, 0x38
    row = np.tile(block, 3)
    out = oracle.decode_rows(abi.Q2_K, row, 1, 768)[0]
    np.testing.assert_array_equal(out, np.array([-1, 2, 5, 8], np.float32)[np.arange(768) % 128 // 32])


def test_matmul_reads_only_logical_columns():
    # picoforge tests/test_qwen4_packed.c:71-91: all-ones Q2_K row . ones(640) = 640, padding poisoned
    block = np.zeros(84, np.uint8)
    block[:16], block[16:80], block[81] = 1, 0x55, 0x3C
    rows = np.tile(block, 6).reshape(2, 252).copy()
    rows[:, 2 * 84 + 16 + 32:2 * 84 + 16 + 64] = 0xFF
    y = oracle.matmul(abi.Q2_K, rows.reshape(-1), 768, 640, 2, np.ones((1, 640), np.float32))
    np.testing.assert_array_equal(y, [[640, 640]])


def test_route_known_answers():
    # picoforge tests/test_qwen4_moe.c:50-63
    z = np.array([[0.0, 1e-9, 0.0, -1e-9], [0.0, 2.0, 2.0, -1000.0]], np.float32)
    probs, ids, weights = oracle.route(z, 2, True)
    np.testing.assert_array_equal(ids, [[0, 1], [1, 2]])
    np.testing.assert_array_equal(weights, [[0.5, 0.5], [0.5, 0.5]])
    assert probs[0, 0] == 0.25 and probs[1, 3] == 0.0
    _, _, raw = oracle.route(z, 2, False)
    assert raw[0, 0] == 0.25
    z[0, 0], z[0, 1] = -3e38, 3e38
    _, ids, weights = oracle.route(z, 2, True)
    assert list(ids[0]) == [1, 0] and list(weights[0]) == [1.0, 0.0]
    z[1, 2] = np.nan
    with pytest.raises(oracle.OracleError) as info:
        oracle.route(z, 2, True)
    assert info.value.status == abi.NONFINITE and info.value.row == 1


def test_group_known_answers():
    # picoforge tests/test_qwen4_moe.c:139-187
    offsets, p2r, r2p = oracle.group(np.array([[2, 0], [1, 2], [2, 0]], np.uint32), 4)
    np.testing.assert_array_equal(offsets, [0, 2, 3, 6, 6])
    np.testing.assert_array_equal(r2p, [1, 5, 2, 0, 3, 4])
    np.testing.assert_array_equal(p2r[r2p], np.arange(6))
    with pytest.raises(oracle.OracleError):
        oracle.group(np.array([[2, 4]], np.uint32), 4)
    with pytest.raises(oracle.OracleError):
        oracle.group(np.array([[2, 2]], np.uint32), 4)


def test_analytic_block():
    # picoforge tests/test_qwen4_moe.py:49-70: x = 1, two experts, top-1
    from picoforge_b200.layer import LayerSpec
    spec = LayerSpec(1, 2, 1, 1, 1, 1, True, (abi.F32,) * 8)
    f = lambda *v: np.array(v, np.float32).view(np.uint8)
    spec.tensors = [f(2, 1), f(1, 2), f(3, 4), f(5, 6), f(1), f(2), f(3), f(0)]
    out = oracle.forward(spec, np.ones((1, 1), np.float32))
    sigmoid1 = 1 / (1 + np.exp(-1.0))
    assert out["ids"].tolist() == [[0]] and out["weights"].tolist() == [[1.0]]
    np.testing.assert_allclose(out["routed"], 15 * sigmoid1, rtol=2e-6)
    np.testing.assert_allclose(out["y"], 18 * sigmoid1, rtol=2e-6)
    spec.norm = False
    out = oracle.forward(spec, np.ones((1, 1), np.float32))
    np.testing.assert_allclose(out["weights"], sigmoid1, rtol=2e-6)
    np.testing.assert_allclose(out["y"], 15 * sigmoid1 ** 2 + 3 * sigmoid1, rtol=2e-6)


@pytest.mark.parametrize("gguf_type", [abi.Q4_K, abi.Q2_K, abi.IQ2_XXS, abi.Q8_0, abi.MXFP4, abi.F16, abi.BF16, abi.F32])
def test_decode_matches_golden(gguf_type):
    blocks = cases.pattern_blocks(gguf_type)
    decoded = oracle.decode_rows(gguf_type, blocks.reshape(-1), len(blocks), abi.FORMATS[gguf_type][1])
    digest = hashlib.sha256(decoded.tobytes()).digest()
    assert digest == GOLDEN[f"decode_{gguf_type}_sha256"].tobytes()


def test_route_matches_golden():
    for seed in range(4):
        for norm in (0, 1):
            tag = f"route_{seed}_{norm}"
            k = GOLDEN[tag + "_ids"].shape[1]
            probs, ids, weights = oracle.route(GOLDEN[tag + "_logits"], k, bool(norm))
            np.testing.assert_array_equal(ids, GOLDEN[tag + "_ids"])
            np.testing.assert_array_equal(bits(probs), bits(GOLDEN[tag + "_probs"]))
            np.testing.assert_array_equal(bits(weights), bits(GOLDEN[tag + "_weights"]))


def test_group_matches_golden_and_stable_argsort():
    for seed in range(3):
        tag = f"group_{seed}"
        ids = GOLDEN[tag + "_ids"]
        experts = len(GOLDEN[tag + "_offsets"]) - 1
        offsets, p2r, r2p = oracle.group(ids, experts)
        np.testing.assert_array_equal(offsets, GOLDEN[tag + "_offsets"])
        np.testing.assert_array_equal(p2r, GOLDEN[tag + "_p2r"])
        np.testing.assert_array_equal(r2p, GOLDEN[tag + "_r2p"])
        np.testing.assert_array_equal(r2p, np.argsort(ids.reshape(-1), kind="stable"))


@pytest.mark.parametrize("name", list(FORWARD_CASES))
def test_forward_matches_golden(name):
    spec, x = forward_case(name)
    out = oracle.forward(spec, x, threads=2)
    np.testing.assert_array_equal(out["ids"], GOLDEN[f"fwd_{name}_ids"])
    np.testing.assert_array_equal(bits(out["weights"]), bits(GOLDEN[f"fwd_{name}_weights"]))
    np.testing.assert_array_equal(bits(out["y"]), bits(GOLDEN[f"fwd_{name}_y"]))


def test_expf_restatement_matches_libm():
    lib = oracle.port()
    lib.qw4o_expf_mismatches.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32]
    lib.qw4o_expf_mismatches.restype = C.c_uint64
    # every 997th negative binary32 from -0 down to -104, plus a dense run around -1
    assert lib.qw4o_expf_mismatches(0x80000000, 0xC2D00001, 997) == 0
    assert lib.qw4o_expf_mismatches(0xBF800000, 0xBF800000 + 2_000_000, 1) == 0


@needs_reference
def test_port_matches_reference_live():
    ref = oracle.reference_api()
    rng = np.random.default_rng(48)
    for (t, e, k) in [(7, 512, 10), (33, 17, 5), (3, 2048, 32)]:
        logits = (rng.standard_normal((t, e)) * 2).astype(np.float32)
        for norm in (False, True):
            a, b = route(ref, logits, k, norm), oracle.route(logits, k, norm)
            np.testing.assert_array_equal(a[1], b[1])
            np.testing.assert_array_equal(bits(a[0]), bits(b[0]))
            np.testing.assert_array_equal(bits(a[2]), bits(b[2]))
        ids = np.stack([rng.permutation(e)[:k] for _ in range(t)]).astype(np.uint32)
        for a, b in zip(group_pairs(ref, ids, e), oracle.group(ids, e)):
            np.testing.assert_array_equal(a, b)
    for routed in (abi.Q4_K, abi.Q2_K, abi.IQ2_XXS):
        spec = cases.small_layer(700 + routed, routed, abi.Q4_K, experts=8, top_k=3)
        x = synth.activations(routed, 40, spec.hidden)          # > 32 tokens: two reference microbatches
        with MoeLayer(ref, spec, len(x)) as layer:
            y, ids, weights = layer.forward(x)
        out = oracle.forward(spec, x, threads=4)
        np.testing.assert_array_equal(ids, out["ids"])
        np.testing.assert_array_equal(bits(y), bits(out["y"]))
        np.testing.assert_array_equal(bits(weights), bits(out["weights"]))
    spec = cases.small_layer(5, abi.Q2_K, abi.Q4_K, experts=4, top_k=2, hidden=256, inter=256 + 0, shared_inter=256)
    # K padding on the routed down projection: stored 512 columns, 256 logical
    spec = synth.make_layer(5, routed_type=abi.Q2_K, shared_type=abi.Q4_K, experts=4, top_k=2, hidden=256,
                            inter=256, shared_inter=256)
    spec.down_physical = 512
    spec.tensors[3] = synth.tensor(abi.Q2_K, 5, 3, spec.hidden * spec.experts, 512)
    x = synth.activations(5, 3, spec.hidden)
    with MoeLayer(ref, spec, 3) as layer:
        y, ids, _ = layer.forward(x)
    out = oracle.forward(spec, x)
    np.testing.assert_array_equal(bits(y), bits(out["y"]))
