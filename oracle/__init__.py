"""CPU oracle for the Qwen4 MoE layer -- TEST INFRASTRUCTURE.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg import this package.
Two checkers live here:

* `port`: oracle/qw4_oracle.c, this project's restatement of the reference arithmetic;
* `reference_api()`: the reference's own CPU objects (oracle/_ref/libqw4ref.so), built by
  oracle/Makefile from the reference sources where those are mounted.  They bind through the
  same ctypes `MoeApi` as the product, because the entry points are the same.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
PORT_LIBRARY = HERE / "libqw4oracle.so"
REFERENCE_LIBRARY = HERE / "_ref" / "libqw4ref.so"


class _Tensor(C.Structure):
    _fields_ = [("type", C.c_uint32), ("data", C.c_void_p)]


class _Layer(C.Structure):
    _fields_ = [("hidden", C.c_uint32), ("experts", C.c_uint32), ("k", C.c_uint32), ("inter", C.c_uint32),
                ("shared_inter", C.c_uint32), ("down_physical", C.c_uint32), ("norm", C.c_int),
                ("w", _Tensor * 8)]


_port = None


def port():
    global _port
    if _port is None:
        if not PORT_LIBRARY.exists():
            raise FileNotFoundError(f"{PORT_LIBRARY} is missing: run `make -C oracle`")
        lib = C.CDLL(str(PORT_LIBRARY))
        lib.qw4o_row_bytes.argtypes = [C.c_uint32, C.c_size_t]
        lib.qw4o_row_bytes.restype = C.c_size_t
        lib.qw4o_decode_row.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_void_p]
        lib.qw4o_matmul.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p,
                                    C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t]
        lib.qw4o_route.argtypes = [C.c_uint32, C.c_uint32, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t,
                                   C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_uint64)]
        lib.qw4o_group.argtypes = [C.c_uint32, C.c_uint32, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.qw4o_forward.argtypes = [C.POINTER(_Layer), C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_void_p, C.c_int]
        lib.qw4o_sigmoid.argtypes = [C.c_float]
        lib.qw4o_sigmoid.restype = C.c_float
        lib.qw4o_silu.argtypes = [C.c_float]
        lib.qw4o_silu.restype = C.c_float
        _port = lib
    return _port


class OracleError(RuntimeError):
    def __init__(self, status, row=0):
        self.status, self.row = status, row
        super().__init__(f"oracle status {status}")


def decode_rows(gguf_type: int, packed: np.ndarray, rows: int, k_storage: int) -> np.ndarray:
    """packed: uint8 [rows * row_bytes] in the natural GGUF layout -> float32 [rows, k_storage]."""
    lib = port()
    rb = lib.qw4o_row_bytes(gguf_type, k_storage)
    assert rb and packed.size >= rows * rb
    out = np.empty((rows, k_storage), np.float32)
    status = 0
    for r in range(rows):
        status |= lib.qw4o_decode_row(gguf_type, packed.ctypes.data + r * rb, k_storage, out[r].ctypes.data)
    if status:
        raise OracleError(status)
    return out


def matmul(gguf_type: int, packed: np.ndarray, k_storage: int, k_logical: int, n_out: int, x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty((x.shape[0], n_out), np.float32)
    st = port().qw4o_matmul(gguf_type, packed.ctypes.data, k_storage, k_logical, n_out, x.ctypes.data, x.shape[1],
                            x.shape[0], y.ctypes.data, n_out)
    if st:
        raise OracleError(st)
    return y


def route(logits: np.ndarray, top_k: int, norm: bool = True):
    logits = np.ascontiguousarray(logits, np.float32)
    t, e = logits.shape
    probs = np.empty((t, e), np.float32)
    ids = np.empty((t, top_k), np.uint32)
    weights = np.empty((t, top_k), np.float32)
    bad = C.c_uint64(0)
    st = port().qw4o_route(e, top_k, int(norm), logits.ctypes.data, e, t, probs.ctypes.data, ids.ctypes.data,
                           weights.ctypes.data, C.byref(bad))
    if st:
        raise OracleError(st, bad.value)
    return probs, ids, weights


def group(ids: np.ndarray, experts: int):
    ids = np.ascontiguousarray(ids, np.uint32)
    t, k = ids.shape
    offsets = np.empty(experts + 1, np.uint64)
    p2r = np.empty(t * k, np.uint64)
    r2p = np.empty(t * k, np.uint64)
    st = port().qw4o_group(experts, k, t, ids.ctypes.data, offsets.ctypes.data, p2r.ctypes.data, r2p.ctypes.data)
    if st:
        raise OracleError(st)
    return offsets, p2r, r2p


def forward(spec, x: np.ndarray, threads: int = 1):
    """spec: picoforge_b200.layer.LayerSpec.  Returns dict(y, ids, weights, logits, routed)."""
    x = np.ascontiguousarray(x, np.float32)
    t = x.shape[0]
    layer = _Layer(spec.hidden, spec.experts, spec.top_k, spec.inter, spec.shared_inter, spec.down_physical,
                   int(spec.norm))
    for i, (gguf_type, array) in enumerate(zip(spec.types, spec.tensors)):
        layer.w[i] = _Tensor(gguf_type, array.ctypes.data)
    y = np.empty((t, spec.hidden), np.float32)
    ids = np.empty((t, spec.top_k), np.uint32)
    weights = np.empty((t, spec.top_k), np.float32)
    logits = np.empty((t, spec.experts), np.float32)
    routed = np.empty((t, spec.hidden), np.float32)
    st = port().qw4o_forward(C.byref(layer), x.ctypes.data, t, y.ctypes.data, ids.ctypes.data, weights.ctypes.data,
                             logits.ctypes.data, routed.ctypes.data, threads)
    if st:
        raise OracleError(st)
    return {"y": y, "ids": ids, "weights": weights, "logits": logits, "routed": routed}


def hc_add(residual: np.ndarray, block: np.ndarray, inject: np.ndarray) -> np.ndarray:
    """The hyper-connection add that follows the layer (picoforge src/qwen4_base.c:160-176):
    residual[t, h, :] + inject[t, h] * block[t, :], product and sum each rounded to FP32 (NumPy's
    float32 multiply and add round once each and never fuse).  Returns the new residual."""
    r, y, g = (np.asarray(a, np.float32) for a in (residual, block, inject))
    assert r.ndim == 3 and y.shape == (r.shape[0], r.shape[2]) and g.shape == r.shape[:2]
    out = r + g[:, :, None] * y[:, None, :]
    assert out.dtype == np.float32
    return out


def reference_hc_add(residual: np.ndarray, block: np.ndarray, inject: np.ndarray) -> np.ndarray:
    """qwen4_hc_add of the reference's own objects on copies of the arguments."""
    from picoforge_b200 import abi

    class Shape(C.Structure):
        _fields_ = [("streams", C.c_size_t), ("hidden_size", C.c_size_t), ("low_rank", C.c_size_t), ("rms_eps", C.c_float)]

    class View(C.Structure):
        _fields_ = [("data", C.c_void_p), ("capacity_bytes", C.c_size_t), ("rank", C.c_size_t), ("dim", C.c_size_t * 4),
                    ("stride_bytes", C.c_size_t * 4)]

    def view(a):
        strides = list(a.strides) + [0] * (4 - a.ndim)
        dims = list(a.shape) + [0] * (4 - a.ndim)
        return View(a.ctypes.data, a.nbytes, a.ndim, (C.c_size_t * 4)(*dims), (C.c_size_t * 4)(*strides))

    lib = C.CDLL(str(REFERENCE_LIBRARY))
    r = np.ascontiguousarray(residual, np.float32).copy()
    y, g = np.ascontiguousarray(block, np.float32), np.ascontiguousarray(inject, np.float32)
    shape = Shape(r.shape[1], r.shape[2], 1, 1e-6)
    err = abi.Qwen4Error()
    lib.qwen4_hc_add.argtypes = [C.POINTER(Shape), View, View, View, C.POINTER(abi.Qwen4Error)]
    status = lib.qwen4_hc_add(C.byref(shape), view(r), view(y), view(g), C.byref(err))
    if status:
        raise OracleError(status)
    return r


def reference_available() -> bool:
    return REFERENCE_LIBRARY.exists()


_reference = None


def reference_api():
    """The reference's own CPU MoE objects behind the shared ctypes binding."""
    global _reference
    if _reference is None:
        from picoforge_b200 import abi
        _reference = abi.MoeApi(REFERENCE_LIBRARY)
        lib = _reference.lib
        lib.qw4_packed_decode_row.argtypes = [C.POINTER(abi.QW4PackedCpuView), C.c_size_t, C.c_size_t, C.c_void_p,
                                              C.c_size_t, C.POINTER(abi.Qwen4Error)]
        lib.qw4_packed_decode_row.restype = C.c_int
        lib.qw4_packed_matmul.argtypes = [C.POINTER(abi.QW4PackedCpuView), C.c_size_t, abi.Qwen4F32, abi.Qwen4F32Mut,
                                          C.POINTER(abi.Qwen4Error)]
        lib.qw4_packed_matmul.restype = C.c_int
    return _reference


def reference_decode_rows(gguf_type: int, packed: np.ndarray, rows: int, k_storage: int) -> np.ndarray:
    from picoforge_b200 import abi
    api = reference_api()
    view = abi.QW4PackedCpuView(abi.Qwen4CpuSpan(packed.ctypes.data, packed.size),
                                abi.make_layout(gguf_type, k_storage, k_storage, rows, 1))
    out = np.empty((rows, k_storage), np.float32)
    err = abi.Qwen4Error()
    for r in range(rows):
        st = api.lib.qw4_packed_decode_row(C.byref(view), 0, r, out[r].ctypes.data, k_storage, C.byref(err))
        if st:
            raise abi.MoeError(st, err)
    return out
