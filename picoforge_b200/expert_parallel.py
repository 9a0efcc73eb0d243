"""Expert-parallel execution of the MoE layer over the ranks of one node.

The reference is a single-device engine; this module is new design.  The 512 experts are cut
into contiguous blocks, one per rank; the router and the shared expert are replicated; tokens
are data-parallel.  One layer step on a rank:

    route (own tokens)  ->  dispatch all-to-all (x rows + local expert ids to the owners)
    ->  experts (rows received from every rank)  ->  combine all-to-all (outputs back)
    ->  slot-order weighted sum + shared expert (own tokens)

The three compute pieces are the library's; this file owns the buffers (torch tensors) and calls
`torch.distributed` all-to-all over NCCL/NVLink between them.  Exchange buffers have a fixed capacity per
destination (every pair could go to one rank), so no step needs a host round trip for sizes; unused
slots carry the id 0xffffffff.

Two forms of the same step:
  packed (default)  `qw4cu_moe_ep_{route_pack,experts,combine}_device`: the library plans and packs the message
                    itself (rows and ids in one message: two all-to-alls per layer) and runs the shared expert
                    on a second stream under the exchange
  plain             `qw4cu_moe_{route,experts,combine}_device` with the plan in torch ops and separate row / id
                    messages (three all-to-alls); kept as the cross-check of the packed form
"""
from __future__ import annotations

import ctypes as C

import torch

from . import abi
from .layer import LayerSpec, MoeLayer

NO_EXPERT = -1      # 0xffffffff as int32


def dispatch_plan(ids: torch.Tensor, experts_per_rank: int, world: int):
    """ids [T, k] (global expert ids, any integer dtype).  Returns, per pair in pair order
    (token * k + slot): destination rank, position inside that rank's buffer (stable: pairs keep
    their order), and the expert index inside the destination's shard."""
    flat = ids.reshape(-1).to(torch.int64)
    dest = torch.div(flat, experts_per_rank, rounding_mode="floor")
    order = torch.argsort(dest, stable=True)
    counts = torch.bincount(dest, minlength=world)
    starts = torch.cumsum(counts, 0) - counts
    pos = torch.empty_like(flat)
    pos[order] = torch.arange(flat.numel(), device=flat.device) - starts[dest[order]]
    return dest, pos, flat - dest * experts_per_rank, counts


class TorchExchange:
    """all-to-all of equally sized per-destination blocks through torch.distributed."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)

    def all_to_all(self, send: torch.Tensor) -> torch.Tensor:
        recv = torch.empty_like(send)
        self.dist.all_to_all_single(recv, send, group=self.group)
        return recv


class EpLayer:
    """One rank's share of one layer."""

    def __init__(self, api: abi.MoeApi, spec: LayerSpec, tokens_local: int, world: int, rank: int, exchange, packed: bool = True):
        assert spec.experts % world == 0
        self.api, self.world, self.rank, self.exchange, self.packed = api, world, rank, exchange, packed
        self.epr = spec.experts // world
        assert spec.local_experts == self.epr and spec.first_expert == rank * self.epr
        self.spec, self.tokens, self.k, self.hidden = spec, tokens_local, spec.top_k, spec.hidden
        self.cap = tokens_local * spec.top_k                 # rows one source may send to one destination
        # tokens_local rows beyond the exchange capacity: room for the shared expert's x digits beside the routed rows
        self.layer = MoeLayer(api, spec, world * self.cap + tokens_local)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.slot_floats = api.lib.qw4cu_ep_slot_floats(self.layer.moe)
        self.msg = torch.zeros((world, self.cap, self.slot_floats), dtype=torch.float32, device=dev)
        self.slots = torch.empty((tokens_local * self.k,), dtype=torch.int32, device=dev)
        self.ids = torch.empty((tokens_local, self.k), dtype=torch.int32, device=dev)
        self.send_rows = torch.zeros((world, self.cap, self.hidden), dtype=torch.float32, device=dev)
        self.send_ids = torch.empty((world, self.cap), dtype=torch.int32, device=dev)
        self.out_rows = torch.zeros((world * self.cap, self.hidden), dtype=torch.float32, device=dev)
        self.y = torch.empty((tokens_local, self.hidden), dtype=torch.float32, device=dev)
        self.err = abi.Qwen4Error()

    def close(self):
        self.layer.close()

    def _check(self, status):
        if status:
            raise abi.MoeError(status, self.err)

    def _use_torch_stream(self):
        # torch's default stream has handle 0, which the library reads as "back to my own stream":
        # name it by CUDA's legacy-default-stream handle (1) instead.
        self.api.lib.qw4cu_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream or 1))

    def phase_route(self, x: torch.Tensor):
        """Routes this rank's tokens and fills the per-destination send buffers."""
        lib, layer = self.api.lib, self.layer
        assert x.is_contiguous() and x.shape == (self.tokens, self.hidden)
        self._use_torch_stream()
        self._check(lib.qw4cu_moe_route_device(layer.moe, x.data_ptr(), self.tokens, self.ids.data_ptr(), None, layer.work,
                                               C.byref(self.err)))
        self.dest, self.pos, local, _ = dispatch_plan(self.ids, self.epr, self.world)
        token = torch.arange(self.tokens * self.k, device=x.device) // self.k
        self.send_ids.fill_(NO_EXPERT)
        self.send_ids[self.dest, self.pos] = local.to(torch.int32)
        self.send_rows[self.dest, self.pos] = x[token]
        return self.send_rows, self.send_ids

    def phase_experts(self, recv_rows: torch.Tensor, recv_ids: torch.Tensor) -> torch.Tensor:
        """Runs this rank's experts on the rows received from every rank."""
        self._use_torch_stream()
        self._check(self.api.lib.qw4cu_moe_experts_device(self.layer.moe, recv_rows.data_ptr(), self.world * self.cap,
                                                          recv_ids.data_ptr(), self.out_rows.data_ptr(), self.layer.work,
                                                          C.byref(self.err)))
        return self.out_rows.view(self.world, self.cap, self.hidden)

    def phase_combine(self, x: torch.Tensor, back: torch.Tensor) -> torch.Tensor:
        """back [world, cap, hidden]: block d holds the outputs of the rows sent to rank d."""
        self._use_torch_stream()
        pair_out = back[self.dest, self.pos].contiguous()
        self._check(self.api.lib.qw4cu_moe_combine_device(self.layer.moe, x.data_ptr(), self.tokens, pair_out.data_ptr(),
                                                          self.y.data_ptr(), self.layer.work, C.byref(self.err)))
        return self.y

    # ---- packed form ----
    def packed_route(self, x: torch.Tensor) -> torch.Tensor:
        assert x.is_contiguous() and x.shape == (self.tokens, self.hidden)
        self._use_torch_stream()
        self._check(self.api.lib.qw4cu_moe_ep_route_pack_device(self.layer.moe, x.data_ptr(), self.tokens, self.cap, self.msg.data_ptr(),
                                                                self.slots.data_ptr(), self.ids.data_ptr(), self.layer.work,
                                                                C.byref(self.err)))
        return self.msg

    def packed_experts(self, recv: torch.Tensor) -> torch.Tensor:
        self._use_torch_stream()
        self._check(self.api.lib.qw4cu_moe_ep_experts_device(self.layer.moe, recv.data_ptr(), self.world * self.cap, self.out_rows.data_ptr(),
                                                             self.layer.work, C.byref(self.err)))
        return self.out_rows.view(self.world, self.cap, self.hidden)

    def packed_combine(self, x: torch.Tensor, back: torch.Tensor) -> torch.Tensor:
        self._use_torch_stream()
        self._check(self.api.lib.qw4cu_moe_ep_combine_device(self.layer.moe, x.data_ptr(), self.tokens, back.data_ptr(), self.slots.data_ptr(),
                                                             self.y.data_ptr(), self.layer.work, C.byref(self.err)))
        return self.y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [tokens_local, hidden] float32 on this rank's GPU.  Work is enqueued on torch's current
        stream (the library is pointed at it), so it orders with the NCCL all-to-alls."""
        if self.packed:
            recv = self.exchange.all_to_all(self.packed_route(x))
            back = self.exchange.all_to_all(self.packed_experts(recv))
            return self.packed_combine(x, back)
        send_rows, send_ids = self.phase_route(x)
        recv_rows = self.exchange.all_to_all(send_rows)
        recv_ids = self.exchange.all_to_all(send_ids)
        out = self.phase_experts(recv_rows, recv_ids)
        back = self.exchange.all_to_all(out)
        return self.phase_combine(x, back)

    def sync(self):
        self._check(self.api.lib.qw4cu_moe_work_sync(self.layer.work, C.byref(self.err)))


def transpose_blocks(sends):
    """What an all-to-all does, for `world` ranks emulated in one process (tests on one GPU or on
    the CPU): sends[r] = [world, cap, ...] of rank r -> result[r][s] = sends[s][r]."""
    stacked = torch.stack(list(sends))                        # [src, dst, cap, ...]
    return [stacked[:, r].contiguous() for r in range(stacked.shape[1])]


def forward_emulated(layers, xs):
    """Runs the ranks of `layers` (EpLayer objects sharing one GPU) in lockstep."""
    if layers[0].packed:
        recvs = transpose_blocks([layer.packed_route(x) for layer, x in zip(layers, xs)])
        backs = transpose_blocks([layer.packed_experts(r) for layer, r in zip(layers, recvs)])
        return [layer.packed_combine(x, b.contiguous()).clone() for layer, x, b in zip(layers, xs, backs)]
    sends = [layer.phase_route(x) for layer, x in zip(layers, xs)]
    recv_rows = transpose_blocks([s[0] for s in sends])
    recv_ids = transpose_blocks([s[1] for s in sends])
    outs = [layer.phase_experts(r, i) for layer, r, i in zip(layers, recv_rows, recv_ids)]
    backs = transpose_blocks(outs)
    return [layer.phase_combine(x, b).clone() for layer, x, b in zip(layers, xs, backs)]
