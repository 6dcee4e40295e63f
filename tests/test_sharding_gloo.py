"""The N>1 path on CPU: two gloo ranks each project their row shard (the oracle stands in for the
kernel here), all-gather the slices, and must reproduce the unsharded result exactly."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from qw38_b200 import synth
from qw38_b200.sharding import gathered_to_token_major, row_shard


def test_row_shard_covers_rows_once():
    for n in (8, 137, 5120, 7168, 34816, 17):
        for world in (1, 2, 3, 4, 8):
            rows = []
            for r in range(world):
                r0, cnt, per = row_shard(n, world, r)
                assert (cnt == 0 or r0 % 8 == 0) and per % 8 == 0 and cnt <= per
                rows += list(range(r0, r0 + cnt))
            assert rows == list(range(n))
    with pytest.raises(ValueError):
        row_shard(8, 2, 2)


def _worker(rank, world, port, n, k, m, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as orc
    codes, meta = synth.logical_q4k(n, k, seed=3)
    hc, hs = synth.split_tiles(codes, meta)
    x = synth.activations(m, k, seed=4)
    z, a, s, _ = orc.q8_quantize(x)                      # replicated quantisation
    r0, cnt, per = row_shard(n, world, rank)
    tiles_k = k // 256
    mine = np.zeros((m, per), dtype=np.float32)
    if cnt:
        sl_c = hc[r0 // 8 * tiles_k * 1024:]               # a row-group run is a view of the matrix
        sl_m = hs[r0 // 8 * tiles_k * 128:]
        mine[:, :cnt] = orc.project(sl_c, sl_m, cnt, k, z, a, s)
    flat = torch.empty((world * m, per), dtype=torch.float32)   # rank g's slice lands in rows [g*m, (g+1)*m)
    dist.all_gather_into_tensor(flat, torch.from_numpy(mine))
    full = gathered_to_token_major(flat.view(world, m, per), n).numpy()
    if rank == 0:
        ref = orc.project(hc, hs, n, k, z, a, s)
        np.save(out_path, np.array([float((full == ref).all())]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("n", [264, 200])
def test_two_gloo_ranks_reproduce_the_unsharded_projection(tmp_path, n):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = str(tmp_path / "ok.npy")
    mp.spawn(_worker, args=(2, port, n, 512, 3, out), nprocs=2, join=True)
    assert np.load(out)[0] == 1.0
