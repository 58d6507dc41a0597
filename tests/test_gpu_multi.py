"""Feature-sharded training on 2 GPUs reproduces the single-GPU trees bit for bit."""

import datetime
import os
import socket

import numpy as np
import pytest
import torch

import cases
from gpu_util import flatten_trees

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, name, shard, out, comm="torch"):
    import torch.distributed as dist
    os.environ["PACKBOOST_SHARD_CODES"] = "1" if shard else "0"
    os.environ["PACKBOOST_COMM"] = comm
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))  # a stuck collective fails instead of hanging
    from packboost_b200 import PackBoost, PackBoostConfig
    X, y, era, cfg, rounds, Xh = cases.CASES[name]()
    b = PackBoost(PackBoostConfig(device="cuda", **cfg))
    b.fit(X, y, era, num_rounds=rounds)
    off, cols = flatten_trees(b.trees)
    out[rank] = (off, cols, b.train_predictions(), b.predict(Xh))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("name,shard,comm", [("prebinned5", True, "torch"), ("prebinned5", False, "torch"),
                                             ("ragged_eras", True, "torch"), ("dro_direction", False, "torch"),
                                             ("prebinned5", True, "native"), ("config1", False, "native")])
def test_two_gpu_fit_equals_one_gpu_fit(name, shard, comm):
    """`shard`: every rank holds only its own feature rows and the go-left bitmask is exchanged;
    otherwise the packed matrix is replicated and only the candidate table is exchanged.
    `comm`: the exchanges go through torch.distributed, or through the library's own NCCL entry
    points (pb_comm_*)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from packboost_b200 import PackBoost, PackBoostConfig
    X, y, era, cfg, rounds, Xh = cases.CASES[name]()
    single = PackBoost(PackBoostConfig(device="cuda", **cfg))
    single.fit(X, y, era, num_rounds=rounds)
    off1, cols1 = flatten_trees(single.trees)
    p1, h1 = single.train_predictions(), single.predict(Xh)
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), name, shard, out, comm), nprocs=2, join=True)
    for rank in range(2):
        off, cols, p, h = out[rank]
        np.testing.assert_array_equal(off, off1)
        for k in cols:
            a, b = cols[k], cols1[k]
            if k == "value":
                a, b = a.view(np.int64), b.view(np.int64)
            np.testing.assert_array_equal(a, b, err_msg=f"rank {rank} {k}")
        np.testing.assert_array_equal(p.view(np.int32), p1.view(np.int32))
        np.testing.assert_array_equal(h.view(np.int32), h1.view(np.int32))
