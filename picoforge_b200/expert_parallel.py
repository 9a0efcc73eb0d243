"""Expert-parallel execution of the MoE layer over the ranks of one node (ctypes plumbing).

The reference is a single-device engine; expert parallelism is new design and lives in the C
library (csrc/ep_nccl.cu, `qw4cu_moe_ep_forward_device`): experts in equal contiguous blocks, one
per rank; router and shared expert replicated; tokens data-parallel.  One layer step:

    route own tokens, pack one row per token (x | ids | weights)     [this rank]
    all-gather of the rows                                            [NCCL, in the library]
    own experts on the tokens routed to them, per-token partial sums  [this rank]
    reduce-scatter (sum) of the partial rows                          [NCCL, in the library]

This module holds what a Python caller needs around that: the NCCL unique id handed from rank 0
to the others over any `torch.distributed` group, a per-rank layer object that owns its device
buffers through the library's allocator, a loop that plays several ranks inside ONE process with
the two compute pieces (for boxes with one GPU), and the same scheme in NumPy for CPU ranks.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import abi
from .layer import LayerSpec, MoeLayer


def owner_of(ids: np.ndarray, experts: int, world: int) -> np.ndarray:
    """Rank that owns each expert id (equal contiguous blocks)."""
    return np.asarray(ids) // (experts // world)


class Communicator:
    """The library's NCCL communicator of this rank.  `group_broadcast(bytes_or_None) -> bytes` moves the
    unique id from rank 0 to everybody (e.g. over a gloo or nccl torch.distributed group)."""

    def __init__(self, api: abi.MoeApi, rank: int, world: int, group_broadcast=None):
        self.api, self.rank, self.world = api, rank, world
        self.handle = C.c_void_p()
        ident = None
        if world > 1:
            buffer = C.create_string_buffer(128)
            if rank == 0 and api.lib.qw4cu_ep_unique_id(buffer) != 0:
                raise RuntimeError(api.lib.qw4cu_last_error().decode())
            ident = group_broadcast(buffer.raw if rank == 0 else None)
            assert len(ident) == 128
        err = abi.Qwen4Error()
        st = api.lib.qw4cu_ep_create(ident, rank, world, C.byref(self.handle), C.byref(err))
        if st:
            raise abi.MoeError(st, err)

    def close(self):
        if self.handle:
            self.api.lib.qw4cu_ep_destroy(self.handle)
            self.handle = C.c_void_p()


def torch_broadcast(group=None):
    """A `group_broadcast` over torch.distributed (object broadcast from rank 0)."""
    import torch.distributed as dist

    def broadcast(payload):
        box = [payload]
        dist.broadcast_object_list(box, src=0, group=group)
        return box[0]
    return broadcast


class EpLayer:
    """One rank's shard of one layer: the sharded MoE handle, a workspace for (world + 1) * tokens tokens,
    and the ids / weights of the last step in device memory."""

    def __init__(self, api: abi.MoeApi, spec: LayerSpec, tokens_local: int, world: int, rank: int):
        assert spec.sharded or world == 1
        self.api, self.spec, self.tokens, self.world, self.rank = api, spec, tokens_local, world, rank
        self.layer = MoeLayer(api, spec, (world + 1) * tokens_local)
        self.ids_dev = api.lib.qw4cu_malloc(max(4, tokens_local * spec.top_k * 4))
        self.weights_dev = api.lib.qw4cu_malloc(max(4, tokens_local * spec.top_k * 4))

    def _check(self, status, err):
        if status:
            raise abi.MoeError(status, err)

    def forward(self, comm: Communicator, x_dev, y_dev):
        """x_dev, y_dev: device pointers [tokens_local, hidden].  Enqueues the whole step (collectives included)."""
        err = abi.Qwen4Error()
        self._check(self.api.lib.qw4cu_moe_ep_forward_device(self.layer.moe, comm.handle, x_dev, y_dev, self.tokens, self.ids_dev,
                                                             self.weights_dev, self.layer.work, C.byref(err)), err)

    def begin(self, x_dev, rows_local_dev):
        err = abi.Qwen4Error()
        self._check(self.api.lib.qw4cu_moe_ep_begin_device(self.layer.moe, x_dev, self.tokens, rows_local_dev, self.ids_dev, self.weights_dev,
                                                           self.layer.work, C.byref(err)), err)

    def experts(self, rows_all_dev, tokens_total, own_first, partial_dev):
        err = abi.Qwen4Error()
        self._check(self.api.lib.qw4cu_moe_ep_experts_device(self.layer.moe, rows_all_dev, tokens_total, own_first, partial_dev,
                                                             self.layer.work, C.byref(err)), err)

    def sync(self):
        err = abi.Qwen4Error()
        self._check(self.api.lib.qw4cu_moe_work_sync(self.layer.work, C.byref(err)), err)

    def routes(self):
        ids = np.empty((self.tokens, self.spec.top_k), np.uint32)
        weights = np.empty((self.tokens, self.spec.top_k), np.float32)
        assert self.api.lib.qw4cu_download(ids.ctypes.data, self.ids_dev, ids.nbytes) == 0
        assert self.api.lib.qw4cu_download(weights.ctypes.data, self.weights_dev, weights.nbytes) == 0
        return ids, weights

    def close(self):
        self.layer.close()
        for pointer in (self.ids_dev, self.weights_dev):
            if pointer:
                self.api.lib.qw4cu_free(pointer)
        self.ids_dev = self.weights_dev = None


def forward_emulated(api: abi.MoeApi, layers: list[EpLayer], xs: list[np.ndarray]) -> list[np.ndarray]:
    """Plays len(layers) ranks on ONE device with the library's two compute pieces; the all-gather is a
    concatenation and the reduce-scatter a sum, both done here on the host.  Returns y per rank."""
    lib = api.lib
    world, per = len(layers), xs[0].shape[0]
    hidden = layers[0].spec.hidden
    pitch = lib.qw4cu_ep_row_floats(layers[0].layer.moe)
    rows_all = np.empty((world * per, pitch), np.float32)
    d_x, d_rows = lib.qw4cu_malloc(per * hidden * 4), lib.qw4cu_malloc(per * pitch * 4)
    d_all, d_partial = lib.qw4cu_malloc(world * per * pitch * 4), lib.qw4cu_malloc(world * per * hidden * 4)
    try:
        # every rank's begin (and with it the start of its shared expert) comes before any rank's experts
        for r, layer in enumerate(layers):
            x = np.ascontiguousarray(xs[r], np.float32)
            assert lib.qw4cu_upload(d_x, x.ctypes.data, x.nbytes) == 0
            layer.begin(d_x, d_rows)
            layer.sync()
            block = rows_all[r * per:(r + 1) * per]
            assert lib.qw4cu_download(block.ctypes.data, d_rows, block.nbytes) == 0
        assert lib.qw4cu_upload(d_all, rows_all.ctypes.data, rows_all.nbytes) == 0
        total = np.zeros((world * per, hidden), np.float64)
        partial = np.empty((world * per, hidden), np.float32)
        for r, layer in enumerate(layers):
            layer.experts(d_all, world * per, r * per, d_partial)
            layer.sync()
            assert lib.qw4cu_download(partial.ctypes.data, d_partial, partial.nbytes) == 0
            total += partial
        return [total[r * per:(r + 1) * per].astype(np.float32) for r in range(world)]
    finally:
        for pointer in (d_x, d_rows, d_all, d_partial):
            lib.qw4cu_free(pointer)


def partial_sums_reference(expert_outputs, ids: np.ndarray, weights: np.ndarray, first: int, count: int) -> np.ndarray:
    """The per-token partial sums of one rank, in NumPy: expert_outputs(token, expert) -> row [hidden] for the
    experts [first, first + count) this rank owns.  Used with CPU ranks to check the scheme itself."""
    tokens = ids.shape[0]
    out = None
    for t in range(tokens):
        for s in range(ids.shape[1]):
            e = int(ids[t, s])
            if first <= e < first + count:
                row = np.asarray(expert_outputs(t, e), np.float64) * float(weights[t, s])
                if out is None:
                    out = np.zeros((tokens, row.shape[0]), np.float64)
                out[t] += row
    return out
