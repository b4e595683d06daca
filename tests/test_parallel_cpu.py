"""World-size-2 test of the tensor-parallel shardings on CPU (gloo).

No GPU kernel runs here: each rank computes its shard with the CPU oracle, so what is checked
is the sharding of codes / scales / zeros (group alignment included) and the collective wiring:
column shards concatenate to the unsharded result, row shards all-reduce to it."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import qf_oracle as O
from qfactory import parallel


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, bits, sym, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K, GS = 3, 256, 512, 128
        x, q, s, z = O.make_case(M, N, K, bits, GS, sym, seed=17)
        ze = O.symmetric_zero(bits) if z is None else O.effective_zero(z.numpy(), bits)
        full = torch.from_numpy(O.qlinear_exact(x, O.dequant_effective(q, s, ze))).float()

        # column parallel: local slice, gathered for the check only
        qc, sc, zc = parallel.shard_columns(q, s, z, rank, world)
        zec = O.symmetric_zero(bits) if zc is None else O.effective_zero(zc.numpy(), bits)
        yc = torch.from_numpy(O.qlinear_exact(x, O.dequant_effective(qc, sc, zec))).float()
        parts = [torch.empty_like(yc) for _ in range(world)]
        dist.all_gather(parts, yc)
        col_err = (torch.cat(parts, dim=1) - full).abs().max().item()

        # row parallel: K shard of x and W, one all-reduce
        qr, sr, zr = parallel.shard_rows(q, s, z, rank, world, GS)
        zer = O.symmetric_zero(bits) if zr is None else O.effective_zero(zr.numpy(), bits)
        ks = K // world
        yr = torch.from_numpy(O.qlinear_exact(x[:, rank * ks : (rank + 1) * ks], O.dequant_effective(qr, sr, zer))).float()
        parallel.all_reduce_sum(yr)
        row_err = (yr - full).abs().max().item()
        scale = full.abs().max().item()
        ret[rank] = (col_err / scale, row_err / scale, tuple(qr.shape), tuple(sr.shape))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("bits,sym", [(4, False), (8, True)])
def test_column_and_row_sharding_world2(bits, sym):
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, bits, sym, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    for r in range(world):
        col, row, qshape, sshape = ret[r]
        assert col < 1e-6 and row < 1e-5
        assert qshape == (256, 256) and sshape == (2, 256)


def test_row_shards_must_hold_whole_groups():
    q = torch.zeros(384, 8, dtype=torch.int32)
    s = torch.ones(3, 8, dtype=torch.float16)
    with pytest.raises(AssertionError):
        parallel.shard_rows(q, s, None, 0, 2, 128)  # 192 rows per rank: not a whole number of groups
    with pytest.raises(AssertionError):
        parallel.shard_columns(q, s, None, 0, 3)


def test_all_reduce_is_a_no_op_without_a_group():
    t = torch.ones(4)
    assert parallel.all_reduce_sum(t) is t and torch.equal(t, torch.ones(4))
