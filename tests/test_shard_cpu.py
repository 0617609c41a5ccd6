"""World sharding over ranks, checked with two gloo processes on the CPU: each rank
solves its contiguous world range (with the oracle standing in for the GPU kernel),
results are gathered, and the union must equal the unsharded solve bit for bit.  No
data-path collective is involved; the gather exists only for the check."""

import copy
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from instantmimic_b200 import mjw_model, synthetic


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, nworld, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle

    m, d, _ = synthetic.make_workload("humanoid", nworld, seed=5, rowless_fraction=0.1)
    lo, hi = mjw_model.shard_bounds(nworld, world)[rank]
    shard = mjw_model.slice_worlds(d, lo, hi)
    assert shard.nworld == hi - lo and shard.efc.J.shape[0] == hi - lo
    oracle.solve(m, shard, threads=1)  # writes through the views into d
    mine = torch.from_numpy(np.ascontiguousarray(d.qacc[lo:hi]))
    sizes = [b - a for a, b in mjw_model.shard_bounds(nworld, world)]
    parts = [torch.zeros((n, m.nv)) for n in sizes]
    # ragged shards: all_gather needs equal shapes, so pad to the largest
    pad = max(sizes)
    padded = torch.zeros((pad, m.nv))
    padded[: hi - lo] = mine
    gathered = [torch.zeros((pad, m.nv)) for _ in range(world)]
    dist.all_gather(gathered, padded)
    for g, n, p in zip(gathered, sizes, parts):
        p.copy_(g[:n])
    niter = torch.tensor([int(d.solver_niter[lo:hi].sum())])
    dist.all_reduce(niter)
    if rank == 0:
        np.save(os.path.join(out_dir, "qacc.npy"), torch.cat(parts).numpy())
        np.save(os.path.join(out_dir, "niter.npy"), niter.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharded_solve_equals_unsharded(oracle, tmp_path):
    nworld = 37  # ragged: 19 + 18
    mp.spawn(_worker, args=(2, _free_port(), nworld, str(tmp_path)), nprocs=2, join=True)
    m, d, _ = synthetic.make_workload("humanoid", nworld, seed=5, rowless_fraction=0.1)
    whole = copy.deepcopy(d)
    oracle.solve(m, whole, threads=2)
    np.testing.assert_array_equal(np.load(tmp_path / "qacc.npy"), whole.qacc)
    assert int(np.load(tmp_path / "niter.npy")[0]) == int(whole.solver_niter.sum())


def test_slice_worlds_is_a_view_of_every_world_major_array():
    m, d, _ = synthetic.make_workload("humanoid", 8, seed=1)
    s = mjw_model.slice_worlds(d, 2, 5)
    s.qacc[:] = 7.0
    s.efc.force[:] = 3.0
    assert (d.qacc[2:5] == 7.0).all() and (d.qacc[:2] == 0).all()
    assert (d.efc.force[2:5] == 3.0).all() and (d.efc.force[5:] == 0).all()
    assert s.nworld == 3 and s.M.shape[0] == 3 and s.nefc.shape[0] == 3
