"""Sharding helpers (CPU): partition arithmetic, and the N>1 flow on two gloo ranks: every rank computes its own shard
(the numpy oracle stands in for the GPU kernel here), shards are gathered, and the result equals the unsharded one."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _shard_mod(pkg):
    return pkg.shard


@pytest.mark.parametrize("total,world,multiple", [(28672, 8, 8), (28672, 3, 128), (100, 4, 8), (7, 4, 8), (0, 2, 8),
                                                   (18432, 8, 128), (32, 8, 1), (5, 8, 1), (1000, 1, 128)])
def test_split_range_covers_everything_once(pkg, total, world, multiple):
    sh = _shard_mod(pkg)
    parts = [sh.split_range(total, world, r, multiple) for r in range(world)]
    pos = 0
    for b, e in parts:
        assert b <= e
        if e > b:
            assert b == pos
            assert b % multiple == 0
            pos = e
    assert pos == total
    sizes = [e - b for b, e in parts]
    assert max(sizes) - min(s for s in sizes) <= multiple + (total % multiple)


def test_split_range_rejects_bad_rank(pkg):
    sh = _shard_mod(pkg)
    with pytest.raises(ValueError):
        sh.split_range(10, 2, 2)


def test_shard_w4a16_slices_are_views_and_reassemble(pkg):
    from oracle import wqbmm_oracle

    sh = _shard_mod(pkg)
    rng = np.random.default_rng(5)
    k, n, g = 64, 80, 32
    w = rng.integers(-8, 8, (k, n), dtype=np.int8)
    words = wqbmm_oracle.pack_int4_words(w)
    scale = rng.uniform(0.01, 0.02, (k // g, n)).astype(np.float32)
    cols = []
    for r in range(3):
        ww, sc, of, bi, (b, e) = sh.shard_w4a16(words, scale, None, None, 3, r)
        assert of is None and bi is None
        assert ww.base is not None  # a view
        assert np.array_equal(wqbmm_oracle.unpack_int4_words(ww), w[:, b:e])
        assert np.array_equal(sc, scale[:, b:e])
        cols.append((b, e))
    assert cols[0][0] == 0 and cols[-1][1] == n and all(c[0] % 8 == 0 for c in cols)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import ml_dtypes
    import torch
    import torch.distributed as dist

    import __graft_entry__ as ge
    from oracle import qbmm_oracle, wqbmm_oracle

    sh = ge.load_package().shard
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    try:
        # --- n-sharded W4A16 (the decode workload's partition) ---
        rng = np.random.default_rng(21)  # same seed on every rank: x replicated, weights "resident" everywhere
        m, k, n, g = 4, 128, 200, 64
        x = rng.standard_normal((m, k)).astype(np.float32).astype(ml_dtypes.bfloat16)
        w = rng.integers(-8, 8, (k, n), dtype=np.int8)
        words = wqbmm_oracle.pack_int4_words(w)
        scale = rng.uniform(0.005, 0.02, (k // g, n)).astype(np.float32).astype(ml_dtypes.bfloat16)
        offset = rng.uniform(-1, 1, (k // g, n)).astype(np.float32).astype(ml_dtypes.bfloat16)
        full = wqbmm_oracle.weight_quant_batch_matmul(x, w, scale, offset, None, g)
        ww, sc, of, _, (b, e) = sh.shard_w4a16(words, scale, offset, None, world, rank)
        mine = wqbmm_oracle.weight_quant_batch_matmul(x, wqbmm_oracle.unpack_int4_words(ww), sc, of, None, g)
        y_local = torch.from_numpy(mine.view(np.int16).copy()).view(torch.bfloat16)
        y = sh.gather_columns(y_local, n, world, rank)
        ok1 = np.array_equal(y.view(torch.int16).numpy(), full.view(np.int16))
        # --- batch-sharded int8 matmul (the batched workloads' partition) ---
        bsz = 3
        x1 = rng.integers(-127, 128, (bsz, 8, 32), dtype=np.int8)
        x2 = rng.integers(-127, 128, (bsz, 32, 16), dtype=np.int8)
        acc_full = np.stack([qbmm_oracle.int_matmul(x1[i], x2[i]) for i in range(bsz)])
        (lx1, lx2), (bb, be) = sh.shard_batch([x1, x2], world, rank)
        acc = np.stack([qbmm_oracle.int_matmul(lx1[i], lx2[i]) for i in range(be - bb)]) if be > bb else np.zeros((0, 8, 16), np.int32)
        out = sh.gather_batch(torch.from_numpy(acc.astype(np.int32)), bsz, world, rank)
        ok2 = np.array_equal(out.numpy(), acc_full)
        ret[rank] = (bool(ok1), bool(ok2))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_shard_compute_gather():
    import torch.multiprocessing as mp

    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_rank_main, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
        for p in procs:
            assert p.exitcode == 0
        assert dict(ret) == {0: (True, True), 1: (True, True)}


def test_c_abi_shard_range_equals_the_python_mirror(aclnn, pkg):
    """opsnn_shard_range (the C-ABI planner a non-Python host binds) and shard.split_range are the same function."""
    sh = pkg.shard
    for total in (0, 1, 7, 8, 100, 127, 128, 1000, 3584, 18432, 28672):
        for world in (1, 2, 3, 4, 8):
            for multiple in (1, 8, 128, 512):
                got = [aclnn.shard_range(total, world, r, multiple) for r in range(world)]
                want = [sh.split_range(total, world, r, multiple) for r in range(world)]
                assert got == want, (total, world, multiple, got, want)
                assert got[0][0] == 0 and got[-1][1] <= total and sum(e - b for b, e in got) == total
