"""The N > 1 host logic on CPU: two gloo ranks partition the block-rows by block count, each produces
its shard of C (with the oracle standing in for the device kernel), and the shards tile the full
result with no overlap and no collective on the data path except the final check."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
import smat_b200 as S
from smat_b200 import generators as gen


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    p = gen.make_config("powerlaw", scale=0.006)  # every rank builds the same seeded matrix
    perm = torch.zeros(p.M, dtype=torch.int64)
    if rank == 0:  # one rank computes the permutation, the others receive it (as bench.py does)
        perm = torch.from_numpy(S.reorder_rows(p.rowptr, p.colidx)[1])
    dist.broadcast(perm, 0)
    rp, ci, v = S.apply_row_permutation(p.rowptr, p.colidx, p.vals, perm.numpy())
    brp, bci, bv = oracle.csr_to_bcsr(p.M, p.K, rp, ci, v)
    bounds = S.partition_block_rows(brp, world)
    b0, b1 = int(bounds[rank]), int(bounds[rank + 1])
    shard = oracle.bcsr_spmm(bv, brp, bci, p.B_nk, p.M, p.N, p.K, b0, b1)
    # ranges of all ranks
    mine = torch.tensor([b0, b1, int(brp[b1] - brp[b0])])
    allr = [torch.zeros(3, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(allr, mine)
    if rank == 0:
        full = oracle.bcsr_spmm(bv, brp, bci, p.B_nk, p.M, p.N, p.K)
        np.save(os.path.join(out_dir, "full.npy"), full)
        np.save(os.path.join(out_dir, "ranges.npy"), torch.stack(allr).numpy())
        np.save(os.path.join(out_dir, "total.npy"), np.array([len(bci), p.M // 16]))
    np.save(os.path.join(out_dir, f"shard{rank}.npy"), shard)
    # the host-buffer product of a shard: every rank contributes its slice of B, one all_gather rebuilds the whole
    for n_cols in (p.N, 40):  # slices that tile B exactly / a last slice that is shorter
        B_host = torch.from_numpy(p.B_nk[:n_cols].view(np.int16).copy())
        _, _, pad = S.b_slice_of_rank(n_cols, world, rank)
        staging = torch.full((world * pad, p.K), -1, dtype=torch.int16)
        B_full = S.gather_b_slices(B_host if rank == 0 else B_host.clone(), staging)
        assert torch.equal(B_full, B_host)
    # the optional exchange step: every rank assembles the whole C from the shards of unequal height
    gathered = S.all_gather_rows(torch.from_numpy(shard), bounds)
    np.save(os.path.join(out_dir, f"gathered{rank}.npy"), gathered.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_partition_and_tile_the_result(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    ranges = np.load(tmp_path / "ranges.npy")
    nnzb, Mb = np.load(tmp_path / "total.npy")
    assert ranges[0, 0] == 0 and ranges[-1, 1] == Mb and ranges[0, 1] == ranges[1, 0]
    assert ranges[:, 2].sum() == nnzb
    assert abs(int(ranges[0, 2]) - int(ranges[1, 2])) <= 0.2 * nnzb  # balanced by block count
    full = np.load(tmp_path / "full.npy")
    tiled = np.concatenate([np.load(tmp_path / f"shard{r}.npy") for r in range(world)])
    assert np.array_equal(tiled.view(np.uint32), full.view(np.uint32))
    for r in range(world):
        assert np.array_equal(np.load(tmp_path / f"gathered{r}.npy").view(np.uint32), full.view(np.uint32))


def test_b_slices_tile_the_columns():
    for N in (8, 40, 256, 4096, 4104):
        for world in (1, 2, 3, 4, 8):
            at = 0
            for r in range(world):
                lo, hi, pad = S.b_slice_of_rank(N, world, r)
                assert lo == at and lo <= hi <= N and (hi - lo) % 8 == 0 and hi - lo <= pad and pad % 8 == 0
                at = hi
            assert at == N
