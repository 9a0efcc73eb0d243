"""Expert parallelism: the exchange scheme (one row per token out by all-gather, per-token partial
sums back by a summed reduce-scatter) among CPU ranks over gloo, a rank that leaves between steps,
and the library's sharded layer against the oracle: ranks played inside one process on one GPU, and
one process per GPU with the collectives issued by the library through NCCL."""
import os
import sys
from datetime import timedelta
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).parent))


def _routes(seed, tokens, experts, k):
    rng = np.random.default_rng(seed)
    ids = np.stack([rng.permutation(experts)[:k] for _ in range(tokens)]).astype(np.uint32)
    weights = rng.random((tokens, k)).astype(np.float32)
    return ids, weights / weights.sum(axis=1, keepdims=True)


def _scheme_worker(rank, world, port, results):
    import torch
    import torch.distributed as dist
    from picoforge_b200.expert_parallel import owner_of, partial_sums_reference
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        experts, k, per, hidden = 8, 3, 5, 4
        epr = experts // world
        x = np.arange(per * hidden, dtype=np.float32).reshape(per, hidden) + 1000 * rank
        ids, weights = _routes(100 + rank, per, experts, k)
        # one row per token: x | ids | weights
        row = torch.tensor(np.concatenate([x, ids.view(np.float32), weights], axis=1))
        gathered = [torch.empty_like(row) for _ in range(world)]
        dist.all_gather(gathered, row)
        rows_all = torch.cat(gathered).numpy()
        x_all = rows_all[:, :hidden]
        ids_all = np.ascontiguousarray(rows_all[:, hidden:hidden + k]).view(np.uint32)
        w_all = rows_all[:, hidden + k:]
        assert (owner_of(ids_all, experts, world) < world).all()
        expert = lambda t, e: x_all[t] * (1.0 + e)                              # noqa: E731  a stand-in for the expert's SwiGLU
        partial = partial_sums_reference(expert, ids_all, w_all, rank * epr, epr)
        total = torch.tensor(partial if partial is not None else np.zeros((world * per, hidden)))
        dist.all_reduce(total)                                                   # gloo has no reduce-scatter: sum, then keep the own rows
        mine = total.numpy()[rank * per:(rank + 1) * per]
        want = sum(weights[:, s:s + 1] * x * (1.0 + ids[:, s:s + 1]) for s in range(k))
        np.testing.assert_allclose(mine, want, rtol=1e-6)
        results[rank] = int((owner_of(ids_all, experts, world) == rank).sum())
    finally:
        dist.destroy_process_group()


def test_exchange_scheme_on_two_cpu_ranks():
    import torch.multiprocessing as mp
    world = 2
    results = mp.Manager().dict()
    mp.spawn(_scheme_worker, args=(world, 29500 + os.getpid() % 1000, results), nprocs=world, join=True)
    assert sum(results[r] for r in range(world)) == world * 5 * 3              # every pair has exactly one owner


def _leaving_worker(rank, world, port, results):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=5))
    value = torch.ones(4)
    dist.all_reduce(value)                                                       # step 1: everybody is there
    if rank == 1:
        results[rank] = "left between steps"
        os._exit(0)                                                              # a rank that dies between two steps, nothing in flight
    try:
        dist.all_reduce(value)                                                   # step 2: the peer is gone
        results[rank] = "no error"
    except Exception as error:                                                   # noqa: BLE001
        results[rank] = "error: " + type(error).__name__


def test_a_rank_that_leaves_between_steps_ends_the_next_collective_with_an_error():
    """Failure detection on the host: the survivor's next collective fails (connection closed or timeout)
    instead of hanging, so its caller can stop issuing layer steps."""
    import torch.multiprocessing as mp
    results = mp.Manager().dict()
    context = mp.spawn(_leaving_worker, args=(2, 30500 + os.getpid() % 1000, results), nprocs=2, join=False)
    for process in context.processes:
        process.join(60)
        assert not process.is_alive()
    assert results[1] == "left between steps"
    assert results[0].startswith("error"), results[0]


def test_owners_match_the_oracle_grouping():
    import oracle
    from picoforge_b200.expert_parallel import owner_of
    rng = np.random.default_rng(7)
    ids = np.stack([rng.permutation(64)[:6] for _ in range(40)]).astype(np.uint32)
    owners = owner_of(ids, 64, 4)
    offsets, _, _ = oracle.group(ids, 64)
    for rank in range(4):                                                        # a rank's rows are the oracle's rows of its experts
        assert int((owners == rank).sum()) == int(offsets[16 * (rank + 1)] - offsets[16 * rank])


def test_shard_bytes_equal_the_slice_of_the_whole_tensor():
    from picoforge_b200 import abi, synth
    whole = synth.make_layer(9, routed_type=abi.IQ2_XXS, shared_type=abi.Q4_K, experts=8, top_k=2, hidden=512, inter=256,
                             shared_inter=256)
    part = synth.make_layer(9, routed_type=abi.IQ2_XXS, shared_type=abi.Q4_K, experts=8, top_k=2, hidden=512, inter=256,
                            shared_inter=256, shard=(2, 4))
    sliced = whole.shard(2, 4)
    for a, b in zip(part.tensors, sliced.tensors):
        np.testing.assert_array_equal(a, b)


@pytest.mark.gpu
@pytest.mark.parametrize("routed,world,tokens", [(12, 4, 16), (16, 2, 6), (10, 4, 32), (10, 2, 160), (12, 1, 24)])
def test_sharded_layer_matches_the_oracle_with_the_ranks_played_in_one_process(gpu, routed, world, tokens):
    """`world` ranks share one GPU; the all-gather is a concatenation and the reduce-scatter a sum on the host.
    Q4_K and IQ2_XXS shards take the four-row grouped kernels, Q2_K (and more than 64 tokens) the tile kernels;
    80 own tokens per rank put the shared expert on the tile kernels too."""
    import oracle
    from picoforge_b200 import abi, synth
    from picoforge_b200.expert_parallel import EpLayer, forward_emulated
    spec = synth.make_layer(300 + routed, routed_type=routed, shared_type=abi.Q4_K, experts=32, top_k=4)
    x = synth.activations(300 + world, tokens)
    want = oracle.forward(spec, x, threads=synth.threads())
    per, epr = tokens // world, spec.experts // world
    layers = [EpLayer(gpu, spec.shard(r * epr, epr) if world > 1 else spec, per, world, r) for r in range(world)]
    try:
        ys = forward_emulated(gpu, layers, [x[r * per:(r + 1) * per] for r in range(world)])
        routes = [layer.routes() for layer in layers]
    finally:
        for layer in layers:
            layer.close()
    y = np.concatenate(ys)
    np.testing.assert_array_equal(np.concatenate([r[0] for r in routes]), want["ids"])
    np.testing.assert_array_equal(np.concatenate([r[1] for r in routes]).view(np.uint32), want["weights"].view(np.uint32))
    assert np.abs(y - want["y"]).max() <= 1e-3


@pytest.mark.gpu
def test_a_wait_that_nothing_satisfies_runs_out_and_reports(gpu):
    """The epoch wait of the peer transport is bounded: on a flag that no peer raises it gives up after its poll
    limit and records the state error; the context stays usable (the next forward works)."""
    from picoforge_b200 import abi, synth
    from picoforge_b200.layer import MoeLayer
    assert gpu.lib.qw4cu_ep_wait_probe(2000, 1) == 0                            # the peer is already there: satisfied at once
    assert gpu.lib.qw4cu_ep_wait_probe(2000, 0) == 1                            # nobody raises the flag: the wait runs out
    spec = synth.make_layer(5, routed_type=abi.Q4_K, shared_type=abi.Q4_K, experts=8, top_k=2, hidden=512, inter=256, shared_inter=256)
    with MoeLayer(gpu, spec, 2) as layer:
        y, _, _ = layer.forward(synth.activations(5, 2, 512))
    assert np.isfinite(y).all()


def _nccl_worker(rank, world, port, routed, tokens, results):
    import ctypes as C
    import torch.distributed as dist
    from picoforge_b200 import abi, synth
    from picoforge_b200.expert_parallel import Communicator, EpLayer, torch_broadcast
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("gloo", rank=rank, world_size=world)                 # only to hand the NCCL id round
    try:
        api = abi.product()
        lib = api.lib
        assert lib.qw4cu_set_device(rank) == 0
        per, epr = tokens // world, 32 // world
        spec = synth.make_layer(300 + routed, routed_type=routed, shared_type=abi.Q4_K, experts=32, top_k=4, shard=(rank * epr, epr))
        x = np.ascontiguousarray(synth.activations(300 + world, tokens)[rank * per:(rank + 1) * per])
        comm = Communicator(api, rank, world, torch_broadcast())
        layer = EpLayer(api, spec, per, world, rank)
        d_x, d_y = lib.qw4cu_malloc(x.nbytes), lib.qw4cu_malloc(x.nbytes)
        assert lib.qw4cu_upload(d_x, x.ctypes.data, x.nbytes) == 0
        for _ in range(2):                                                       # twice: the buffers and counters are reusable
            layer.forward(comm, d_x, d_y)
        layer.sync()
        y = np.empty_like(x)
        assert lib.qw4cu_download(y.ctypes.data, d_y, y.nbytes) == 0
        results[rank] = (y, layer.routes()[0])
        dist.barrier()
        layer.close()
        comm.close()
        lib.qw4cu_free(d_x); lib.qw4cu_free(d_y)
        del C
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("routed", [12, 10])
def test_sharded_layer_over_nccl_on_two_gpus(gpu, routed):
    """One process per GPU, the library's own all-gather and reduce-scatter over NCCL; skipped on a one-GPU box."""
    import torch.multiprocessing as mp
    import oracle
    from picoforge_b200 import abi, synth
    if gpu.lib.qw4cu_device_count() < 2:
        pytest.skip("needs two GPUs")
    world, tokens = 2, 12
    spec = synth.make_layer(300 + routed, routed_type=routed, shared_type=abi.Q4_K, experts=32, top_k=4)
    x = synth.activations(300 + world, tokens)
    want = oracle.forward(spec, x, threads=synth.threads())
    results = mp.Manager().dict()
    mp.spawn(_nccl_worker, args=(world, 29600 + os.getpid() % 300, routed, tokens, results), nprocs=world, join=True)
    y = np.concatenate([results[r][0] for r in range(world)])
    ids = np.concatenate([results[r][1] for r in range(world)])
    np.testing.assert_array_equal(ids, want["ids"])
    assert np.abs(y - want["y"]).max() <= 1e-3
