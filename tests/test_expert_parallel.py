"""Expert parallelism: the dispatch plan and exchange on CPU ranks (gloo, world size 2), and the
whole sharded layer against the oracle with the ranks emulated on one GPU."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).parent))


def _plan_worker(rank, world, port, results):
    import torch
    import torch.distributed as dist
    from picoforge_b200.expert_parallel import NO_EXPERT, dispatch_plan
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        experts, k, tokens, hidden = 8, 3, 5, 4
        epr, cap = experts // world, tokens * k
        rng = np.random.default_rng(100 + rank)
        ids = torch.tensor(np.stack([rng.permutation(experts)[:k] for _ in range(tokens)]), dtype=torch.int32)
        x = torch.arange(tokens * hidden, dtype=torch.float32).reshape(tokens, hidden) + 1000 * rank
        dest, pos, local, counts = dispatch_plan(ids, epr, world)
        send_rows = torch.zeros(world, cap, hidden)
        send_ids = torch.full((world, cap), NO_EXPERT, dtype=torch.int32)
        token = torch.arange(tokens * k) // k
        send_rows[dest, pos] = x[token]
        send_ids[dest, pos] = local.to(torch.int32)
        recv_rows, recv_ids = torch.empty_like(send_rows), torch.empty_like(send_ids)
        dist.all_to_all_single(recv_rows, send_rows)
        dist.all_to_all_single(recv_ids, send_ids)
        # every received id belongs to this rank's shard; pretend expert output = row * (1 + local id)
        valid = recv_ids != NO_EXPERT
        assert bool(((recv_ids[valid] >= 0) & (recv_ids[valid] < epr)).all())
        out = recv_rows * (1 + recv_ids.clamp(min=0)).unsqueeze(-1).float()
        back = torch.empty_like(out)
        dist.all_to_all_single(back, out)
        pair_out = back[dest, pos]
        want = x[token] * (1 + (ids.reshape(-1).to(torch.int64) % epr)).unsqueeze(-1).float()
        assert torch.equal(pair_out, want)
        # stable order inside a destination, counts add up
        for d in range(world):
            assert torch.equal(pos[dest == d], torch.arange(int(counts[d])))
        gathered = [None] * world
        dist.all_gather_object(gathered, int(valid.sum()))
        results[rank] = (int(counts.sum()), gathered)
    finally:
        dist.destroy_process_group()


def test_dispatch_plan_and_exchange_on_two_cpu_ranks():
    import torch.multiprocessing as mp
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_plan_worker, args=(world, 29500 + os.getpid() % 1000, results), nprocs=world, join=True)
    assert len(results) == world
    sent = sum(results[r][0] for r in range(world))
    received = sum(results[0][1])
    assert sent == received == world * 5 * 3


def test_dispatch_plan_matches_the_oracle_grouping():
    import torch
    import oracle
    from picoforge_b200.expert_parallel import dispatch_plan
    rng = np.random.default_rng(7)
    ids = np.stack([rng.permutation(64)[:6] for _ in range(40)]).astype(np.uint32)
    dest, pos, local, counts = dispatch_plan(torch.tensor(ids.astype(np.int64)), 16, 4)
    offsets, p2r, r2p = oracle.group(ids, 64)
    # rows of one destination rank are the oracle's rows of its experts, as a set
    for d in range(4):
        assert int(counts[d]) == int(offsets[16 * (d + 1)] - offsets[16 * d])
    assert torch.equal(local, torch.tensor(ids.reshape(-1).astype(np.int64) % 16))


@pytest.mark.gpu
@pytest.mark.parametrize("packed", [True, False])
@pytest.mark.parametrize("routed,world,tokens", [(12, 4, 16), (16, 2, 6), (10, 4, 32)])
def test_sharded_layer_matches_the_oracle_with_emulated_ranks(gpu, routed, world, tokens, packed):
    """`world` ranks share one GPU; the all-to-all is a block transpose.  Q4_K and IQ2_XXS shards
    take the tensor-core grouped kernels, Q2_K the CUDA-core kernels.  Both forms of the step: packed
    messages planned by the library (shared expert on a second stream), and the plan in torch ops."""
    import torch
    import oracle
    from picoforge_b200 import abi, synth
    from picoforge_b200.expert_parallel import EpLayer, forward_emulated
    spec = synth.make_layer(300 + routed, routed_type=routed, shared_type=abi.Q4_K, experts=32, top_k=4)
    x = synth.activations(300 + world, tokens)
    want = oracle.forward(spec, x, threads=synth.threads())
    per = tokens // world
    epr = spec.experts // world
    torch.cuda.set_device(0)
    layers = [EpLayer(gpu, spec.shard(r * epr, epr), per, world, r, None, packed) for r in range(world)]
    try:
        xs = [torch.tensor(x[r * per:(r + 1) * per]).cuda().contiguous() for r in range(world)]
        ys = forward_emulated(layers, xs)
        for layer in layers:
            layer.sync()
        y = torch.cat(ys).cpu().numpy()
        ids = torch.cat([layer.ids for layer in layers]).cpu().numpy().astype(np.uint32)
    finally:
        for layer in layers:
            layer.close()
        gpu.lib.qw4cu_set_stream(None)
    np.testing.assert_array_equal(ids, want["ids"])
    assert np.abs(y - want["y"]).max() <= 1e-3


def test_shard_bytes_equal_the_slice_of_the_whole_tensor():
    from picoforge_b200 import abi, synth
    whole = synth.make_layer(9, routed_type=abi.IQ2_XXS, shared_type=abi.Q4_K, experts=8, top_k=2, hidden=512, inter=256,
                             shared_inter=256)
    part = synth.make_layer(9, routed_type=abi.IQ2_XXS, shared_type=abi.Q4_K, experts=8, top_k=2, hidden=512, inter=256,
                            shared_inter=256, shard=(2, 4))
    sliced = whole.shard(2, 4)
    for a, b in zip(part.tensors, sliced.tensors):
        np.testing.assert_array_equal(a, b)


def _nccl_worker(rank, world, port, routed, tokens, results):
    import torch
    import torch.distributed as dist
    from picoforge_b200 import abi, synth
    from picoforge_b200.expert_parallel import EpLayer, TorchExchange
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        api = abi.product()
        assert api.lib.qw4cu_set_device(rank) == 0
        per, epr = tokens // world, 32 // world
        spec = synth.make_layer(300 + routed, routed_type=routed, shared_type=abi.Q4_K, experts=32, top_k=4, shard=(rank * epr, epr))
        x = synth.activations(300 + world, tokens)[rank * per:(rank + 1) * per]
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            layer = EpLayer(api, spec, per, world, rank, TorchExchange())
            y = layer.forward(torch.tensor(x).cuda().contiguous())
            layer.sync()
            results[rank] = (y.cpu().numpy(), layer.ids.cpu().numpy().astype(np.uint32))
            layer.close()
        api.lib.qw4cu_set_stream(None)
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("routed", [12, 16])
def test_sharded_layer_over_nccl_on_two_gpus(gpu, routed):
    """One process per GPU, rows exchanged by NCCL all-to-all; skipped on a one-GPU box."""
    import torch
    import torch.multiprocessing as mp
    import oracle
    from picoforge_b200 import abi, synth
    if torch.cuda.device_count() < 2:
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
