"""The GGUF slice reader: one layer's eight MoE tensors found in a file, described exactly as the
reference's own container parser and layout code describe them, malformed files answered with a
status, and (GPU) a layer created from the file equal to one created from memory."""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).parent))
import gguf_fixture  # noqa: E402

from picoforge_b200 import abi, synth  # noqa: E402

REF = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libqw4ref.so"


def _spec(routed=abi.IQ2_XXS, shared=abi.Q4_K, **kw):
    return synth.make_layer(41, routed_type=routed, shared_type=shared, experts=8, top_k=2, hidden=512, inter=256, shared_inter=256, **kw)


def _describe(api, path, layer=0):
    slice_, err = abi.QW4CuGgufSlice(), abi.Qwen4Error()
    status = api.lib.qw4cu_gguf_slice_describe(str(path).encode(), layer, C.byref(slice_), C.byref(err))
    return status, slice_, err


def test_describe_finds_the_layer(tmp_path):
    api = abi.product()
    spec = _spec()
    where = gguf_fixture.write_layer(tmp_path / "m.gguf", spec, layer=3, alignment=64)
    status, got, err = _describe(api, tmp_path / "m.gguf", 3)
    assert status == 0, (err.subject, err.detail)
    c = got.config
    assert (c.hidden_size, c.experts, c.top_k, c.intermediate, c.shared_intermediate, c.down_physical, c.norm_topk_prob) == \
        (512, 8, 2, 256, 256, 256, True)
    assert list(c.trunk_type) == [abi.IQ2_XXS] * 3
    for role, (suffix, layout) in enumerate(zip(gguf_fixture.ROLE_SUFFIX, spec.layouts())):
        t, l = got.tensor[role], got.layout[role]
        assert t.name.decode() == f"blk.3.{suffix}"
        assert (t.file_offset, t.bytes) == where[t.name.decode()]
        assert t.file_offset % 64 == 0 and t.type == spec.types[role]
        for field, _ in abi.QW4PackedLayout._fields_:
            assert getattr(l, field) == getattr(layout, field), (role, field)
    # the payload at those offsets is the tensor
    blob = (tmp_path / "m.gguf").read_bytes()
    for role in range(8):
        t = got.tensor[role]
        assert blob[t.file_offset:t.file_offset + t.bytes] == spec.tensors[role].tobytes()
    status, _, err = _describe(api, tmp_path / "m.gguf", 2)                    # another layer is not in the file
    assert status == abi.MISSING and b"blk.2." in err.subject


class _RefTensor(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("type", C.c_uint32), ("rank", C.c_uint32), ("shape", C.c_size_t * 4),
                ("file_offset", C.c_size_t), ("bytes", C.c_size_t)]


class _RefGguf(C.Structure):
    _fields_ = [("fd", C.c_int), ("header", C.c_void_p), ("header_size", C.c_size_t), ("file_size", C.c_size_t),
                ("data_offset", C.c_size_t), ("tensor_count", C.c_size_t), ("metadata_count", C.c_size_t),
                ("tensors", C.POINTER(_RefTensor)), ("metadata", C.c_void_p)]


@pytest.mark.skipif(not REF.exists(), reason="the reference's objects are not built")
@pytest.mark.parametrize("routed,down_physical", [(abi.Q4_K, None), (abi.Q2_K, None), (abi.IQ2_XXS, None)])
def test_description_equals_the_reference_parser(tmp_path, routed, down_physical):
    """The reference's own container parser (gguf_open) and layout code (qw4_packed_layout_init) on the same file."""
    api = abi.product()
    ref = C.CDLL(str(REF))
    spec = _spec(routed=routed)
    gguf_fixture.write_layer(tmp_path / "m.gguf", spec, layer=1)
    status, got, err = _describe(api, tmp_path / "m.gguf", 1)
    assert status == 0, (err.subject, err.detail)
    g = _RefGguf()
    ref.gguf_open(str(tmp_path / "m.gguf").encode(), C.byref(g))
    try:
        assert g.data_offset == got.data_offset and g.file_size == got.file_bytes
        by_name = {g.tensors[i].name.decode(): g.tensors[i] for i in range(g.tensor_count)}
        logical = [512, 512, 512, 256, 512, 512, 256, 512]
        for role in range(8):
            mine = got.tensor[role]
            theirs = by_name[mine.name.decode()]
            assert (mine.type, mine.rank, mine.file_offset, mine.bytes) == (theirs.type, theirs.rank, theirs.file_offset, theirs.bytes)
            assert list(mine.shape)[:mine.rank] == list(theirs.shape)[:theirs.rank]
            layout = abi.QW4PackedLayout()
            assert ref.qw4_packed_layout_init(C.byref(theirs), C.c_size_t(logical[role]), C.byref(layout), None) == 0
            for field, _ in abi.QW4PackedLayout._fields_:
                assert getattr(got.layout[role], field) == getattr(layout, field), (role, field)
    finally:
        ref.gguf_close(C.byref(g))


def test_padded_down_projection(tmp_path):
    """Q2_K stores K rounded up to 256: 640 logical columns in 768 (the real model's routed down projection)."""
    api = abi.product()
    spec = synth.make_layer(43, routed_type=abi.Q2_K, shared_type=abi.Q4_K, experts=4, top_k=2, hidden=256, inter=640,
                            shared_inter=256, down_physical=768)
    gguf_fixture.write_layer(tmp_path / "m.gguf", spec)
    status, got, err = _describe(api, tmp_path / "m.gguf")
    assert status == 0, (err.subject, err.detail)
    assert got.config.down_physical == 768 and got.layout[3].k_storage == 768 and got.layout[3].k_logical == 640
    import struct
    bad = gguf_fixture._kv("ds4.qwen4.down.physical_input", 4, struct.pack("<I", 1024))
    gguf_fixture.write_layer(tmp_path / "n.gguf", spec, extra_metadata=[bad])
    assert _describe(api, tmp_path / "n.gguf")[0] == abi.SHAPE


def test_malformed_files_are_statuses(tmp_path):
    api = abi.product()
    spec = _spec()
    path = tmp_path / "m.gguf"
    assert _describe(api, tmp_path / "absent.gguf")[0] == abi.IO
    gguf_fixture.write_layer(path, spec, truncate=16)
    assert _describe(api, path)[0] == abi.FORMAT
    gguf_fixture.write_layer(path, spec, truncate=300)                             # inside the metadata
    assert _describe(api, path)[0] == abi.FORMAT
    where = gguf_fixture.write_layer(path, spec)
    last = max(at + size for name, (at, size) in where.items() if name.startswith("blk."))
    gguf_fixture.write_layer(path, spec, truncate=last - 100)                    # header whole, payload cut
    assert _describe(api, path)[0] == abi.FORMAT
    gguf_fixture.write_layer(path, spec, architecture="llama")
    assert _describe(api, path)[0] == abi.FORMAT
    gguf_fixture.write_layer(path, spec, drop=5)
    status, _, err = _describe(api, path)
    assert status == abi.MISSING and b"ffn_up_shexp" in err.subject
    gguf_fixture.write_layer(path, spec, overrides={"qwen4exp.expert_count": 16})
    assert _describe(api, path)[0] == abi.SHAPE
    path.write_bytes(b"GGML" + bytes(100))
    assert _describe(api, path)[0] == abi.FORMAT
    status, got, _ = _describe(api, path)
    assert got.config.hidden_size == 0 and got.tensor[0].bytes == 0               # nothing left behind on error


@pytest.mark.gpu
def test_layer_created_from_a_file_equals_one_created_from_memory(gpu, tmp_path):
    import oracle
    from picoforge_b200.layer import MoeLayer
    spec = synth.make_layer(44, routed_type=abi.IQ2_XXS, shared_type=abi.Q4_K, experts=32, top_k=4)
    gguf_fixture.write_layer(tmp_path / "m.gguf", spec, layer=5)
    x = synth.activations(44, 4)
    want = oracle.forward(spec, x, threads=synth.threads())
    with MoeLayer(gpu, spec, 4) as memory:
        y_memory, ids_memory, _ = memory.forward(x)
    handle, err = C.c_void_p(), abi.Qwen4Error()
    status = gpu.lib.qw4cu_moe_create_from_gguf(str(tmp_path / "m.gguf").encode(), 5, C.byref(handle), None, C.byref(err))
    assert status == 0, (err.subject, err.detail)
    (tmp_path / "m.gguf").unlink()                                                 # the resident image is the only copy now
    with MoeLayer(gpu, spec, 4, moe=handle) as filed:
        y_file, ids_file, _ = filed.forward(x)
    np.testing.assert_array_equal(ids_file, want["ids"])
    np.testing.assert_array_equal(y_file.view(np.uint32), y_memory.view(np.uint32))
    assert np.abs(y_file - want["y"]).max() <= 1e-3
