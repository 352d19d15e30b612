"""CPU-only (gloo, world size 2): the external-mode partitioning used by bench.py --gpus N.

Each rank contracts its slice with the oracle standing in for the GPU; gathering the slices must
reproduce the unsharded result bit for bit, because no sum crosses a rank boundary."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, result_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle_lib import F64, Contraction, Oracle
    from tcont_b200 import TCEquation, ScalarType, sharding
    oracle = Oracle()
    eq = TCEquation("abcd", "aebf", "cfde", dict(a=8, b=6, c=4, d=6, e=5, f=3), "-", ScalarType.Float64)
    cfull = Contraction(eq.modeC, eq.modeA, eq.modeB, dict(eq.extent), F64)
    A, B = oracle.inputs(cfull, 5)
    local, sl = sharding.shard_equation(eq, mode, world, rank)
    a_loc = sharding.take_slice(A, eq.modeA, eq.extent, mode, sl)
    b_loc = sharding.take_slice(B, eq.modeB, eq.extent, mode, sl)
    part = oracle.contract(Contraction(local.modeC, local.modeA, local.modeB, dict(local.extent), F64), a_loc, b_loc)
    parts = [torch.empty(part.size, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(part))
    if rank == 0:
        out = np.zeros(cfull.size(cfull.modeC))
        for r, t in enumerate(parts):
            _, s = sharding.shard_equation(eq, mode, world, r)
            sharding.put_slice(out, t.numpy(), eq.modeC, eq.extent, mode, s)
        np.save(result_path, np.stack([out, oracle.contract(cfull, A, B)]))
    dist.barrier()
    dist.destroy_process_group()


def _worker_ksplit(rank, world, port, result_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle_lib import F64, Contraction, Oracle
    from tcont_b200 import TCEquation, ScalarType, sharding
    oracle = Oracle()
    eq = TCEquation("abcd", "aebf", "cfde", dict(a=8, b=6, c=4, d=6, e=4, f=3), "-", ScalarType.Float64)
    cfull = Contraction(eq.modeC, eq.modeA, eq.modeB, dict(eq.extent), F64)
    A, B = oracle.inputs(cfull, 6)
    local, sl = sharding.shard_contracted(eq, "e", world, rank)
    a_loc = sharding.take_slice(A, eq.modeA, eq.extent, "e", sl)
    b_loc = sharding.take_slice(B, eq.modeB, eq.extent, "e", sl)
    partial = torch.from_numpy(oracle.contract(Contraction(local.modeC, local.modeA, local.modeB, dict(local.extent), F64), a_loc, b_loc))
    # reduce-scatter expressed with what gloo offers on CPU: all-reduce, then keep this rank's chunk of C
    dist.all_reduce(partial)
    n = partial.numel() // world
    mine = partial[rank * n:(rank + 1) * n].clone()
    chunks = [torch.empty(n, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(chunks, mine)
    if rank == 0:
        np.save(result_path, np.stack([torch.cat(chunks).numpy(), oracle.contract(cfull, A, B)]))
    dist.barrier()
    dist.destroy_process_group()


def _worker_owner_slots(rank, world, port, result_path):
    """The protocol of the fused contracted split: rank r sends range o of its partial C to owner o (the GPU
    kernel stores it there tile by tile), every owner adds its `world` slots in rank order, and the owners'
    ranges laid end to end are C."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle_lib import F64, Contraction, Oracle
    from tcont_b200 import TCEquation, ScalarType, sharding
    oracle = Oracle()
    eq = TCEquation("abcd", "aebf", "cfde", dict(a=8, b=6, c=4, d=6, e=4, f=3), "-", ScalarType.Float64)
    cfull = Contraction(eq.modeC, eq.modeA, eq.modeB, dict(eq.extent), F64)
    A, B = oracle.inputs(cfull, 6)
    local, sl = sharding.shard_contracted(eq, "e", world, rank)
    a_loc = sharding.take_slice(A, eq.modeA, eq.extent, "e", sl)
    b_loc = sharding.take_slice(B, eq.modeB, eq.extent, "e", sl)
    partial = oracle.contract(Contraction(local.modeC, local.modeA, local.modeB, dict(local.extent), F64), a_loc, b_loc)
    n = partial.size
    slots = [None] * world
    slots[rank] = partial[sharding.owner_range(n, world, rank)].copy()
    sends = []
    for o in range(world):
        if o != rank:
            sends.append(dist.isend(torch.from_numpy(partial[sharding.owner_range(n, world, o)].copy()), dst=o))
    for src in range(world):
        if src != rank:
            buf = torch.empty(n // world, dtype=torch.float64)
            dist.recv(buf, src=src)
            slots[src] = buf.numpy()
    for w in sends:
        w.wait()
    mine = torch.from_numpy(sharding.sum_owner_slots(slots))
    chunks = [torch.empty(n // world, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(chunks, mine)
    if rank == 0:
        np.save(result_path, np.stack([torch.cat(chunks).numpy(), oracle.contract(cfull, A, B)]))
    dist.barrier()
    dist.destroy_process_group()


def test_owner_slot_protocol_sums_to_unsharded(tmp_path, engine):
    path = str(tmp_path / "out.npy")
    mp.spawn(_worker_owner_slots, args=(2, _free_port(), path), nprocs=2, join=True)
    got, want = np.load(path)
    np.testing.assert_allclose(got, want, rtol=1e-13, atol=1e-13)   # the order of the partial sums differs


def test_contracted_split_sums_to_unsharded(tmp_path, engine):
    path = str(tmp_path / "out.npy")
    mp.spawn(_worker_ksplit, args=(2, _free_port(), path), nprocs=2, join=True)
    got, want = np.load(path)
    np.testing.assert_allclose(got, want, rtol=1e-13, atol=1e-13)   # the order of the partial sums differs


@pytest.mark.parametrize("mode", ["a", "b", "d"])   # stride-1 mode of A and C, a middle mode, the slowest mode (in B)
def test_external_split_equals_unsharded(tmp_path, engine, mode):
    path = str(tmp_path / "out.npy")
    mp.spawn(_worker, args=(2, _free_port(), mode, path), nprocs=2, join=True)
    got, want = np.load(path)
    np.testing.assert_array_equal(got, want)


def test_split_rejects_contracted_and_ragged_modes(engine):
    from tcont_b200 import TCEquation, sharding
    eq = TCEquation("abc", "adc", "db", dict(a=8, b=6, c=4, d=6))
    with pytest.raises(ValueError):
        sharding.shard_equation(eq, "d", 2, 0)          # contracted mode: needs shard_contracted + a reduction
    with pytest.raises(ValueError):
        sharding.shard_contracted(eq, "a", 2, 0)        # an external mode is not summed over
    loc, sl = sharding.shard_contracted(eq, "d", 2, 1)
    assert loc.extent["d"] == 3 and (sl.start, sl.stop) == (3, 6)
    with pytest.raises(ValueError):
        sharding.shard_equation(eq, "b", 4, 0)          # 6 does not divide over 4 ranks
    grown = sharding.grow_equation(eq, "c", 8)
    assert grown.extent["c"] == 32 and eq.extent["c"] == 4
