"""CPU tests of the C-ABI library: it loads without a GPU, exports every declared symbol, and
rejects bad arguments with the reference's status codes before touching the device."""
import ctypes as C
import re
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).parent))
import cases  # noqa: E402
from picoforge_b200 import abi  # noqa: E402
from picoforge_b200.layer import group_pairs, route  # noqa: E402

ROOT = Path(__file__).parents[1]


def declared_functions():
    names = []
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names += re.findall(r"\b((?:qwen4_moe|qw4_moe|qw4cu)_\w+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol(product):
    names = declared_functions()
    assert len(names) >= 30
    for name in abi.MoeApi.REFERENCE_SYMBOLS:
        assert name in names
    for name in names:
        assert hasattr(product.lib, name), name


def test_source_has_no_cpu_fallback():
    for path in (ROOT / "picoforge_b200").rglob("*"):
        if path.suffix in (".py", ".c", ".cu", ".cuh", ".h"):
            text = path.read_text()
            assert "oracle" not in text.lower() or path.name == "build.py", path


def test_create_rejects_bad_arguments_before_the_device(product):
    spec = cases.float_layer(1)
    cfg, weights = spec.config(), spec.weights()
    handle, err = C.c_void_p(), abi.Qwen4Error()
    lib = product.lib
    assert lib.qwen4_moe_create(None, C.byref(weights), C.byref(handle), C.byref(err)) == abi.INVALID_ARGUMENT
    assert lib.qwen4_moe_create(C.byref(cfg), None, C.byref(handle), C.byref(err)) == abi.INVALID_ARGUMENT
    assert err.code == abi.INVALID_ARGUMENT and err.subject == b"qwen4_moe"
    bad = spec.config(); bad.top_k = 5
    assert lib.qwen4_moe_create(C.byref(bad), C.byref(weights), C.byref(handle), C.byref(err)) == abi.RANGE
    # picoforge tests/test_qwen4_moe.c:271-277: wrong logical K, short span, inconsistent row bytes
    w = spec.weights(); w.down.layout.k_logical = 4
    assert lib.qwen4_moe_create(C.byref(cfg), C.byref(w), C.byref(handle), C.byref(err)) == abi.SHAPE and not handle
    w = spec.weights(); w.up.span.bytes -= 1
    assert lib.qwen4_moe_create(C.byref(cfg), C.byref(w), C.byref(handle), C.byref(err)) == abi.CAPACITY and not handle
    w = spec.weights(); w.gate.layout.row_bytes += 1
    assert lib.qwen4_moe_create(C.byref(cfg), C.byref(w), C.byref(handle), C.byref(err)) == abi.FORMAT and not handle
    w = spec.weights(); w.router.layout.gguf_type = abi.F16
    assert lib.qwen4_moe_create(C.byref(cfg), C.byref(w), C.byref(handle), C.byref(err)) == abi.FORMAT


def test_route_rejects_bad_views_before_the_device(product):
    # the fourteen error cases of picoforge tests/test_qwen4_moe.c:64-86 that do not need data
    z = np.zeros((2, 7), np.float32)[:, :4]
    z[0] = [0, 1e-9, 0, -1e-9]
    z[1] = [0, 2, 2, -1000]
    p = np.full((2, 8), -99, np.float32)[:, :4]
    w = np.full((2, 4), -99, np.float32)[:, :2]
    ids = np.full((2, 5), 0xFFFFFFFF, np.uint32)[:, :2]

    def run(mutate):
        cfg = abi.Qwen4MoeConfig(8, 4, 2, 5, 3, 5, True, (C.c_uint32 * 3)(0, 0, 0))
        logits, probs = abi.f32_view(z), abi.f32_view(p)
        routes = abi.Qwen4MoeRoutes(abi.u32_view(ids), abi.f32_view(w))
        args = {"cfg": cfg, "logits": logits, "probs": probs, "routes": routes}
        mutate(args)
        err = abi.Qwen4Error()
        st = product.lib.qwen4_moe_route(C.byref(args["cfg"]) if args["cfg"] is not None else None, args["logits"],
                                         args["routes"], args["probs"], C.byref(err))
        assert err.code == st
        assert (p == -99).all() and (w == -99).all() and (ids == 0xFFFFFFFF).all()
        return st

    def set_(path, value):
        def mutate(a):
            obj = a[path[0]]
            for name in path[1:-1]:
                obj = getattr(obj, name)
            if isinstance(path[-1], tuple):
                getattr(obj, path[-1][0])[path[-1][1]] = value
            else:
                setattr(obj, path[-1], value)
        return mutate

    assert run(set_(("logits", "data"), None)) == abi.INVALID_ARGUMENT
    assert run(set_(("logits", "rank"), 1)) == abi.SHAPE
    assert run(set_(("probs", ("stride_bytes", 1)), 8)) == abi.STRIDE
    assert run(set_(("routes", "weights", "capacity_bytes"), 23)) == abi.CAPACITY
    assert run(set_(("routes", "ids", "row_stride_bytes"), 7)) == abi.STRIDE
    assert run(set_(("cfg", "top_k"), 5)) == abi.RANGE
    assert run(set_(("routes", "ids", "cols"), 3)) == abi.SHAPE
    assert run(set_(("probs", "capacity_bytes"), 47)) == abi.CAPACITY
    assert run(set_(("probs", "data"), z.ctypes.data + 4)) == abi.INVALID_ARGUMENT
    assert run(set_(("routes", "weights", "data"), p.ctypes.data)) == abi.INVALID_ARGUMENT
    assert run(set_(("logits", ("dim", 0)), 2**64 - 1)) == abi.OVERFLOW
    assert run(set_(("probs", "data"), z.ctypes.data)) == abi.INVALID_ARGUMENT

    def null_config(a):
        a["cfg"] = None
    assert run(null_config) == abi.INVALID_ARGUMENT


def test_group_rejects_bad_ids_before_the_device(product):
    # picoforge tests/test_qwen4_moe.c:148-171
    with pytest.raises(abi.MoeError) as info:
        group_pairs(product, np.array([[2, 0], [1, 2], [2, 4]], np.uint32), 4)
    assert info.value.status == abi.RANGE
    with pytest.raises(abi.MoeError) as info:
        group_pairs(product, np.array([[2, 0], [1, 2], [2, 2]], np.uint32), 4)
    assert info.value.status == abi.INVALID_ARGUMENT
    with pytest.raises(abi.MoeError) as info:
        group_pairs(product, np.array([[2], [1]], np.uint32), 4 * 0 + 1)   # id 2 >= 1 expert
    assert info.value.status == abi.RANGE


def test_empty_route_needs_no_device(product):
    probs, ids, weights = route(product, np.zeros((0, 4), np.float32), 2)
    assert probs.shape == (0, 4) and ids.shape == (0, 2) and weights.shape == (0, 2)


def test_empty_group_views_are_checked_without_dividing_by_their_pitch(product):
    """No tokens: the pair arrays are empty (zero bytes per row).  The view checks must pass them
    (picoforge tests/test_qwen4_moe.c:90-93 runs the empty batch) and only the device step may fail here."""
    try:
        offsets, p2r, r2p = group_pairs(product, np.zeros((0, 2), np.uint32), 4)
        assert (offsets == 0).all() and p2r.size == 0 and r2p.size == 0
    except abi.MoeError as error:                       # no GPU on this machine
        assert error.status == abi.GPU_ERROR
