"""ctypes mirror of the MoE operator's C ABI (include/qwen4_moe_b200.h).

The same struct layouts and entry points are exported by two shared objects:

* ``picoforge_b200/libqwen4_moe_b200.so`` -- the CUDA product library, and
* the reference's own CPU objects when they have been built for the tests
  (picoforge src/qwen4_moe.h:13-27, src/qwen4_moe_internal.h:15,94).

`MoeApi` binds either, so a test reads the same against both.  Nothing here computes:
a missing product library is an ImportError-like failure, never a fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

PACKAGE_DIR = Path(__file__).resolve().parent
PRODUCT_LIBRARY = PACKAGE_DIR / "libqwen4_moe_b200.so"

# GGUF tensor types the operator accepts: id -> (name, weights per block, bytes per block)
# (picoforge src/gguf.c:13-17).
FORMATS = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 8: ("Q8_0", 32, 34), 10: ("Q2_K", 256, 84),
    12: ("Q4_K", 256, 144), 16: ("IQ2_XXS", 256, 66), 30: ("BF16", 1, 2), 39: ("MXFP4", 32, 17),
}
F32, F16, Q8_0, Q2_K, Q4_K, IQ2_XXS, BF16, MXFP4 = 0, 1, 8, 10, 12, 16, 30, 39

STATUS = ["OK", "INVALID_ARGUMENT", "MISSING", "TYPE", "RANGE", "SHAPE", "STRIDE", "FORMAT",
          "UNSUPPORTED", "OVERFLOW", "CAPACITY", "OOM", "OWNER", "BUSY", "STALE", "BAD_STATE",
          "NONFINITE", "IO", "EOF", "CANCELLED", "GPU_ERROR"]
(OK, INVALID_ARGUMENT, MISSING, TYPE, RANGE, SHAPE, STRIDE, FORMAT, UNSUPPORTED, OVERFLOW,
 CAPACITY, OOM, OWNER, BUSY, STALE, BAD_STATE, NONFINITE, IO, EOF, CANCELLED, GPU_ERROR) = range(21)


class Qwen4Error(C.Structure):
    _fields_ = [("code", C.c_int), ("os_errno", C.c_int), ("file_offset", C.c_uint64),
                ("row", C.c_uint64), ("requested_bytes", C.c_size_t),
                ("completed_bytes", C.c_size_t), ("subject", C.c_char * 128),
                ("detail", C.c_char * 256)]


class Qwen4CpuSpan(C.Structure):
    _fields_ = [("data", C.c_void_p), ("bytes", C.c_size_t)]


class Qwen4F32(C.Structure):
    _fields_ = [("data", C.c_void_p), ("capacity_bytes", C.c_size_t), ("rank", C.c_size_t),
                ("dim", C.c_size_t * 4), ("stride_bytes", C.c_size_t * 4)]


Qwen4F32Mut = Qwen4F32  # identical layout; constness is not visible to ctypes


class Qwen4U32Mut(C.Structure):
    _fields_ = [("data", C.c_void_p), ("capacity_bytes", C.c_size_t), ("rows", C.c_size_t),
                ("cols", C.c_size_t), ("row_stride_bytes", C.c_size_t)]


class Qwen4MoeConfig(C.Structure):
    _fields_ = [("hidden_size", C.c_uint32), ("experts", C.c_uint32), ("top_k", C.c_uint32),
                ("intermediate", C.c_uint32), ("shared_intermediate", C.c_uint32),
                ("down_physical", C.c_uint32), ("norm_topk_prob", C.c_bool),
                ("trunk_type", C.c_uint32 * 3)]


class QW4PackedLayout(C.Structure):
    _fields_ = [("gguf_type", C.c_uint32), ("k_storage", C.c_size_t), ("k_logical", C.c_size_t),
                ("n_out", C.c_size_t), ("n_experts", C.c_size_t), ("row_bytes", C.c_size_t),
                ("expert_bytes", C.c_size_t), ("tensor_bytes", C.c_size_t)]


class QW4PackedCpuView(C.Structure):
    _fields_ = [("span", Qwen4CpuSpan), ("layout", QW4PackedLayout)]


class QW4CuGgufTensor(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("type", C.c_uint32), ("rank", C.c_uint32), ("shape", C.c_uint64 * 4),
                ("file_offset", C.c_uint64), ("bytes", C.c_uint64)]


class QW4CuGgufSlice(C.Structure):
    _fields_ = [("config", Qwen4MoeConfig), ("tensor", QW4CuGgufTensor * 8), ("layout", QW4PackedLayout * 8),
                ("data_offset", C.c_uint64), ("file_bytes", C.c_uint64)]


class Qwen4MoeWeights(C.Structure):
    _fields_ = [(name, QW4PackedCpuView) for name in
                ("router", "gate", "up", "down", "shared_gate", "shared_up", "shared_down",
                 "shared_router")]


class Qwen4MoeRoutes(C.Structure):
    _fields_ = [("ids", Qwen4U32Mut), ("weights", Qwen4F32Mut)]


class QW4MoeGrouping(C.Structure):
    _fields_ = [("offsets", C.c_void_p), ("offsets_capacity_bytes", C.c_size_t),
                ("cursors", C.c_void_p), ("cursors_capacity_bytes", C.c_size_t),
                ("pair_to_row", C.c_void_p), ("row_to_pair", C.c_void_p),
                ("pair_to_row_capacity_bytes", C.c_size_t),
                ("row_to_pair_capacity_bytes", C.c_size_t)]


assert C.sizeof(Qwen4F32) == 88 and C.sizeof(Qwen4Error) == 424
assert C.sizeof(Qwen4MoeConfig) == 40 and C.sizeof(QW4PackedLayout) == 64

TENSOR_NAMES = ("router", "gate", "up", "down", "shared_gate", "shared_up", "shared_down",
                "shared_router")


def row_bytes(gguf_type: int, k_storage: int) -> int:
    _, block, size = FORMATS[gguf_type]
    if k_storage % block:
        raise ValueError(f"k_storage {k_storage} is not a whole number of {block}-weight blocks")
    return k_storage // block * size


def make_layout(gguf_type, k_storage, k_logical, n_out, n_experts) -> QW4PackedLayout:
    rb = row_bytes(gguf_type, k_storage)
    return QW4PackedLayout(gguf_type, k_storage, k_logical, n_out, n_experts, rb, rb * n_out,
                           rb * n_out * n_experts)


def f32_view(array: np.ndarray | None, rows: int | None = None, cols: int | None = None) -> Qwen4F32:
    """Rank-2 view of a float32 array whose last axis is contiguous (row pitch may be padded)."""
    if array is None:
        return Qwen4F32(None, 0, 2, (C.c_size_t * 4)(rows or 0, cols or 0, 1, 1),
                        (C.c_size_t * 4)((cols or 0) * 4, 4, 0, 0))
    assert array.dtype == np.float32 and array.ndim == 2 and array.strides[1] == 4
    r, c = array.shape
    extent = (r - 1) * array.strides[0] + c * 4 if r else 0
    return Qwen4F32(array.ctypes.data, extent, 2, (C.c_size_t * 4)(r, c, 1, 1),
                    (C.c_size_t * 4)(array.strides[0], 4, 0, 0))


def u32_view(array: np.ndarray | None, rows: int = 0, cols: int = 0) -> Qwen4U32Mut:
    if array is None:
        return Qwen4U32Mut(None, 0, rows, cols, cols * 4)
    assert array.dtype == np.uint32 and array.ndim == 2 and array.strides[1] == 4
    r, c = array.shape
    extent = (r - 1) * array.strides[0] + c * 4 if r else 0
    return Qwen4U32Mut(array.ctypes.data, extent, r, c, array.strides[0])


class MoeError(RuntimeError):
    def __init__(self, status: int, error: Qwen4Error | None = None):
        self.status = status
        self.detail = error.detail.decode(errors="replace") if error is not None else ""
        self.row = error.row if error is not None else 0
        super().__init__(f"QW4_{STATUS[status] if 0 <= status < len(STATUS) else status}: {self.detail}")


class MoeApi:
    """Typed bindings of the operator entry points shared by the product and the reference."""

    def __init__(self, path: str | Path):
        path = Path(path)
        if not path.exists():
            raise FileNotFoundError(
                f"{path} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()')")
        self.path = path
        self.lib = lib = C.CDLL(str(path), mode=C.RTLD_LOCAL)
        E = C.POINTER(Qwen4Error)
        P = C.c_void_p
        sig = {
            "qwen4_moe_create": ([C.POINTER(Qwen4MoeConfig), C.POINTER(Qwen4MoeWeights), C.POINTER(P), E], C.c_int),
            "qwen4_moe_destroy": ([P], None),
            "qwen4_moe_work_size": ([P, C.c_size_t, C.POINTER(C.c_size_t), E], C.c_int),
            "qwen4_moe_work_create": ([P, C.c_size_t, C.c_size_t, C.POINTER(P), E], C.c_int),
            "qwen4_moe_work_reset": ([P, E], C.c_int),
            "qwen4_moe_work_destroy": ([P], None),
            "qwen4_moe_route": ([C.POINTER(Qwen4MoeConfig), Qwen4F32, Qwen4MoeRoutes, Qwen4F32Mut, E], C.c_int),
            "qwen4_moe_forward": ([P, Qwen4F32, Qwen4F32Mut, C.POINTER(Qwen4MoeRoutes), P, E], C.c_int),
            "qw4_moe_group_pairs": ([C.POINTER(Qwen4MoeConfig), Qwen4U32Mut, QW4MoeGrouping, E], C.c_int),
        }
        for name, (argtypes, restype) in sig.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = argtypes, restype
        self.has_extensions = hasattr(lib, "qw4cu_device_count")
        if self.has_extensions:
            self._bind_extensions()

    # names of every symbol include/qwen4_moe_b200.h declares, for the export test
    REFERENCE_SYMBOLS = ("qwen4_moe_create", "qwen4_moe_destroy", "qwen4_moe_work_size",
                         "qwen4_moe_work_create", "qwen4_moe_work_reset", "qwen4_moe_work_destroy",
                         "qwen4_moe_route", "qwen4_moe_forward", "qw4_moe_group_pairs",
                         "qw4_moe_observe")

    def launch_names(self) -> list[str]:
        """Kernel names launched since `lib.qw4cu_launch_log_begin()` (product library only)."""
        buf = C.create_string_buffer(1 << 16)
        self.lib.qw4cu_launch_log(buf, len(buf))
        return [n for n in buf.value.decode().split(",") if n]

    def _bind_extensions(self):
        lib, P, E = self.lib, C.c_void_p, C.POINTER(Qwen4Error)
        sig = {
            "qw4cu_device_count": ([], C.c_int),
            "qw4cu_set_device": ([C.c_int], C.c_int),
            "qw4cu_last_error": ([], C.c_char_p),
            "qw4cu_set_router_mode": ([C.c_int], None),
            "qw4cu_get_router_mode": ([], C.c_int),
            "qw4cu_moe_device_bytes": ([P], C.c_size_t),
            "qw4cu_moe_work_device_bytes": ([P], C.c_size_t),
            "qw4cu_moe_forward_device": ([P, P, P, C.c_size_t, P, P, P, E], C.c_int),
            "qw4cu_moe_work_sync": ([P, E], C.c_int),
            "qw4cu_moe_create_sharded": ([C.POINTER(Qwen4MoeConfig), C.POINTER(Qwen4MoeWeights), C.c_uint32, C.c_uint32, C.POINTER(P), E], C.c_int),
            "qw4cu_moe_route_device": ([P, P, C.c_size_t, P, P, P, E], C.c_int),
            "qw4cu_ep_unique_id": ([C.c_char_p], C.c_int),
            "qw4cu_ep_create": ([C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_void_p), E], C.c_int),
            "qw4cu_ep_destroy": ([P], None),
            "qw4cu_ep_row_floats": ([P], C.c_size_t),
            "qw4cu_ep_trace": ([C.c_int], None),
            "qw4cu_ep_trace_read": ([C.POINTER(C.c_double), C.c_int], C.c_uint64),
            "qw4cu_moe_ep_forward_device": ([P, P, P, P, C.c_size_t, P, P, P, E], C.c_int),
            "qw4cu_moe_ep_begin_device": ([P, P, C.c_size_t, P, P, P, P, E], C.c_int),
            "qw4cu_moe_ep_experts_device": ([P, P, C.c_size_t, C.c_size_t, P, P, E], C.c_int),
            "qw4cu_set_stream": ([P], C.c_int),
            "qw4cu_moe_work_timer_begin": ([P], C.c_int),
            "qw4cu_moe_work_timer_end": ([P], C.c_int),
            "qw4cu_moe_work_timer_elapsed_ms": ([P], C.c_float),
            "qw4cu_launch_count": ([], C.c_uint64),
            "qw4cu_launch_log_begin": ([], None),
            "qw4cu_launch_log": ([C.c_char_p, C.c_size_t], C.c_size_t),
            "qw4cu_set_graph_mode": ([C.c_int], None),
            "qw4cu_get_graph_mode": ([], C.c_int),
            "qw4cu_set_stage_timing": ([C.c_int], None),
            "qw4cu_set_expert_path": ([C.c_int], None),
            "qw4cu_set_only_step": ([C.c_int], None),
            "qw4cu_set_fused_decode": ([C.c_int], None),
            "qw4cu_set_prefill_path": ([C.c_int], None),
            "qw4cu_set_tile_path": ([C.c_int], None),
            "qw4cu_prefill_debug": ([P], None),
            "qw4cu_decode_phase_clocks": ([P, C.POINTER(C.c_uint64)], C.c_int),
            "qw4cu_decode_repairs": ([P, C.POINTER(C.c_uint32)], C.c_int),
            "qw4cu_decode_debug_words": ([P, C.POINTER(C.c_uint32), C.c_size_t], C.c_int),
            "qw4cu_set_decode_wrong_speculation": ([C.c_int], None),
            "qw4cu_stage_times": ([C.POINTER(C.c_double), C.POINTER(C.c_uint64)], C.c_int),
            "qw4cu_moe_decode_rows": ([P, C.c_uint32, C.c_size_t, C.c_size_t, C.c_size_t, P, C.c_size_t, E], C.c_int),
            "qw4cu_moe_decode_rows_expanded": ([P, C.c_uint32, C.c_size_t, C.c_size_t, C.c_size_t, P, C.c_size_t, E], C.c_int),
            "qw4cu_group_pairs_device_noalloc": ([C.c_uint32, C.c_uint32, C.c_size_t, P, P, P, P, E], C.c_int),
            "qw4cu_malloc": ([C.c_size_t], P),
            "qw4cu_free": ([P], None),
            "qw4cu_host_alloc": ([C.c_size_t], P),
            "qw4cu_host_free": ([P], None),
            "qw4cu_upload": ([P, P, C.c_size_t], C.c_int),
            "qw4cu_download": ([P, P, C.c_size_t], C.c_int),
            "qw4cu_flush_l2": ([], C.c_int),
            "qw4cu_moe_forward_hc_add_device": ([P, P, P, C.c_size_t, P, P, C.c_size_t, P, C.POINTER(Qwen4Error)], C.c_int),
            "qw4cu_verify_create": ([C.POINTER(P), C.c_size_t, C.POINTER(Qwen4MoeConfig), C.POINTER(P), C.POINTER(Qwen4Error)], C.c_int),
            "qw4cu_verify_destroy": ([P], None),
            "qw4cu_verify_route_log": ([P, C.c_char_p, C.POINTER(Qwen4Error)], C.c_int),
            "qw4cu_verify_append": ([P, P, C.c_size_t, P, P, C.POINTER(Qwen4Error)], C.c_int),
            "qw4cu_verify_keep": ([P, C.c_size_t, C.POINTER(Qwen4Error)], C.c_int),
            "qw4cu_verify_position": ([P], C.c_uint64),
            "qw4cu_verify_pending": ([P], C.c_size_t),
            "qw4cu_moe_work_sync_many": ([C.POINTER(P), C.c_size_t, C.POINTER(Qwen4Error)], C.c_int),
            "qw4cu_ep_transport": ([P], C.c_int),
            "qw4cu_ep_wait_probe": ([C.c_uint32, C.c_int], C.c_int),
            "qw4cu_mem_info": ([C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)], C.c_int),
            "qw4cu_gguf_slice_describe": ([C.c_char_p, C.c_uint32, C.POINTER(QW4CuGgufSlice), C.POINTER(Qwen4Error)], C.c_int),
            "qw4cu_moe_create_from_gguf": ([C.c_char_p, C.c_uint32, C.POINTER(P), C.POINTER(QW4CuGgufSlice), C.POINTER(Qwen4Error)], C.c_int),
            "qw4cu_device_synchronize": ([], C.c_int),
        }
        for name, (argtypes, restype) in sig.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = argtypes, restype


_product: MoeApi | None = None


def product() -> MoeApi:
    """The CUDA product library.  Raises if it has not been built: there is no CPU path."""
    global _product
    if _product is None:
        _product = MoeApi(PRODUCT_LIBRARY)
    return _product
