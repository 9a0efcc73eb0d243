"""Python handle over the MoE operator's C entry points.

`MoeLayer` owns one `Qwen4Moe` and one workspace created through a `MoeApi`
(picoforge_b200.abi): the CUDA product library in normal use, or the reference's CPU objects
in the parity tests -- the call sequence is the reference's own (picoforge
src/qwen4_forward.c:174-187 create + workspace, :365 forward).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import abi


@dataclass
class LayerSpec:
    """Shapes and GGUF types of one MoE layer plus its packed weight bytes (host, natural layout)."""
    hidden: int = 2048
    experts: int = 512
    top_k: int = 10
    inter: int = 512
    shared_inter: int = 512
    down_physical: int | None = None
    norm: bool = True
    types: tuple = (abi.F32, abi.Q4_K, abi.Q4_K, abi.Q4_K, abi.Q4_K, abi.Q4_K, abi.Q4_K, abi.F32)
    tensors: list = field(default_factory=list)   # eight uint8 arrays in Qwen4MoeWeights order
    first_expert: int = 0                         # expert shard held by the routed tensors
    local_experts: int | None = None              # None: all of them

    def __post_init__(self):
        if self.down_physical is None:
            self.down_physical = self.inter

    @property
    def sharded(self) -> bool:
        return self.local_experts is not None and self.local_experts != self.experts

    def shard(self, first: int, count: int) -> "LayerSpec":
        """A spec whose routed tensors are experts [first, first + count) of this (complete) one."""
        assert not self.sharded
        out = LayerSpec(self.hidden, self.experts, self.top_k, self.inter, self.shared_inter, self.down_physical, self.norm,
                        self.types, list(self.tensors), first, count)
        for index, layout in zip((1, 2, 3), self.layouts()[1:4]):
            eb = layout.expert_bytes
            out.tensors[index] = self.tensors[index][first * eb:(first + count) * eb]
        return out

    def shapes(self):
        """(k_storage, k_logical, n_out, n_experts) of the eight tensors."""
        h, i, s, dp = self.hidden, self.inter, self.shared_inter, self.down_physical
        e = self.experts if self.local_experts is None else self.local_experts
        return [(h, h, self.experts, 1), (h, h, i, e), (h, h, i, e), (dp, i, h, e),
                (h, h, s, 1), (h, h, s, 1), (s, s, h, 1), (h, h, 1, 1)]

    def layouts(self):
        return [abi.make_layout(t, *shape) for t, shape in zip(self.types, self.shapes())]

    def config(self) -> abi.Qwen4MoeConfig:
        return abi.Qwen4MoeConfig(self.hidden, self.experts, self.top_k, self.inter, self.shared_inter,
                                  self.down_physical, self.norm, (C.c_uint32 * 3)(*self.types[1:4]))

    def weights(self) -> abi.Qwen4MoeWeights:
        views = []
        for array, layout in zip(self.tensors, self.layouts()):
            assert array.dtype == np.uint8 and array.flags.c_contiguous and array.size == layout.tensor_bytes, \
                (array.size, layout.tensor_bytes)
            views.append(abi.QW4PackedCpuView(abi.Qwen4CpuSpan(array.ctypes.data, array.size), layout))
        return abi.Qwen4MoeWeights(*views)

    def weight_bytes(self) -> int:
        return sum(l.tensor_bytes for l in self.layouts())


class MoeLayer:
    def __init__(self, api: abi.MoeApi, spec: LayerSpec, token_cap: int, moe=None):
        """`moe`: an existing handle (e.g. from qw4cu_moe_create_from_gguf) that this object takes over."""
        self.api, self.spec, self.token_cap = api, spec, token_cap
        self.moe = C.c_void_p()
        self.work = C.c_void_p()
        err = abi.Qwen4Error()
        if moe is not None:
            self.moe, st = moe, 0
        elif spec.sharded:
            cfg, weights = spec.config(), spec.weights()
            st = api.lib.qw4cu_moe_create_sharded(C.byref(cfg), C.byref(weights), spec.first_expert, spec.local_experts,
                                                  C.byref(self.moe), C.byref(err))
        else:
            cfg, weights = spec.config(), spec.weights()
            st = api.lib.qwen4_moe_create(C.byref(cfg), C.byref(weights), C.byref(self.moe), C.byref(err))
        if st:
            raise abi.MoeError(st, err)
        size = C.c_size_t()
        st = api.lib.qwen4_moe_work_size(self.moe, token_cap, C.byref(size), C.byref(err))
        if not st:
            st = api.lib.qwen4_moe_work_create(self.moe, token_cap, size.value, C.byref(self.work), C.byref(err))
        if st:
            api.lib.qwen4_moe_destroy(self.moe)
            self.moe = C.c_void_p()
            raise abi.MoeError(st, err)

    def close(self):
        if self.work:
            self.api.lib.qwen4_moe_work_destroy(self.work)
            self.work = C.c_void_p()
        if self.moe:
            self.api.lib.qwen4_moe_destroy(self.moe)
            self.moe = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reset(self):
        err = abi.Qwen4Error()
        st = self.api.lib.qwen4_moe_work_reset(self.work, C.byref(err))
        if st:
            raise abi.MoeError(st, err)

    def forward(self, x: np.ndarray, want_routes: bool = True):
        """x [T, hidden] float32 (host).  Returns (y, ids, weights); raises MoeError on failure."""
        t, k = x.shape[0], self.spec.top_k
        y = np.full((t, self.spec.hidden), np.nan, np.float32)
        ids = np.full((t, k), 0xFFFFFFFF, np.uint32)
        weights = np.full((t, k), np.nan, np.float32)
        routes = abi.Qwen4MoeRoutes(abi.u32_view(ids if t else None, t, k), abi.f32_view(weights if t else None, t, k))
        err = abi.Qwen4Error()
        st = self.api.lib.qwen4_moe_forward(self.moe, abi.f32_view(x if t else None, t, self.spec.hidden),
                                            abi.f32_view(y if t else None, t, self.spec.hidden),
                                            C.byref(routes) if want_routes else None, self.work, C.byref(err))
        if st:
            raise abi.MoeError(st, err)
        return y, ids, weights

    def decode_rows(self, tensor: int, expert: int, row0: int, rows: int) -> np.ndarray:
        """Exact decode of rows of the RESIDENT image (product library only)."""
        k = self.spec.shapes()[tensor][0]
        out = np.empty((rows, k), np.float32)
        err = abi.Qwen4Error()
        st = self.api.lib.qw4cu_moe_decode_rows(self.moe, tensor, expert, row0, rows, out.ctypes.data, out.size, C.byref(err))
        if st:
            raise abi.MoeError(st, err)
        return out


def route(api: abi.MoeApi, logits: np.ndarray, top_k: int, norm: bool = True):
    """qwen4_moe_route on host arrays.  Returns (probs, ids, weights)."""
    t, e = logits.shape
    cfg = abi.Qwen4MoeConfig(8, e, top_k, 5, 3, 5, norm, (C.c_uint32 * 3)(0, 0, 0))
    probs = np.full((t, e), -99, np.float32)
    ids = np.full((t, top_k), 0xFFFFFFFF, np.uint32)
    weights = np.full((t, top_k), -99, np.float32)
    routes = abi.Qwen4MoeRoutes(abi.u32_view(ids if t else None, t, top_k), abi.f32_view(weights if t else None, t, top_k))
    err = abi.Qwen4Error()
    st = api.lib.qwen4_moe_route(C.byref(cfg), abi.f32_view(logits if t else None, t, e), routes,
                                 abi.f32_view(probs if t else None, t, e), C.byref(err))
    if st:
        raise abi.MoeError(st, err)
    return probs, ids, weights


def group_pairs(api: abi.MoeApi, ids: np.ndarray, experts: int):
    """qw4_moe_group_pairs on host arrays.  Returns (offsets, pair_to_row, row_to_pair) as uint64."""
    t, k = ids.shape
    cfg = abi.Qwen4MoeConfig(8, experts, k, 5, 3, 5, True, (C.c_uint32 * 3)(0, 0, 0))
    offsets = np.full(experts + 1, 2**64 - 1, np.uint64)
    cursors = np.full(experts, 2**64 - 1, np.uint64)
    p2r = np.full(max(t * k, 1), 2**64 - 1, np.uint64)
    r2p = np.full(max(t * k, 1), 2**64 - 1, np.uint64)
    g = abi.QW4MoeGrouping(offsets.ctypes.data, offsets.nbytes, cursors.ctypes.data, cursors.nbytes,
                           p2r.ctypes.data if t else None, r2p.ctypes.data if t else None,
                           t * k * 8, t * k * 8)
    err = abi.Qwen4Error()
    st = api.lib.qw4_moe_group_pairs(C.byref(cfg), abi.u32_view(ids if t else None, t, k), g, C.byref(err))
    if st:
        raise abi.MoeError(st, err)
    return offsets, p2r[:t * k], r2p[:t * k]
