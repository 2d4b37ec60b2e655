"""GPU: the library's own NCCL communicator and the gather of output shards (include/opsnn_b200_shard.h).

A single-rank communicator exercises the whole path on one GPU (NCCL resolved at run time, strided copy, all-gather, interleave
kernel). With two or more GPUs the same calls run as two child processes, one per GPU, over NVLink; the ranks only meet in the
collective, and each leaves between steps with nothing in flight."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_single_rank_gather_columns_and_batch(aclnn):
    import torch

    dev = torch.device("cuda", 0)
    comm = aclnn.Comm(1, 0, dev)
    try:
        y = torch.arange(16 * 520, dtype=torch.float32, device=dev).reshape(16, 520).to(torch.bfloat16)
        view = y[:, :512]  # a row-strided shard: 512 of 520 columns
        full = comm.gather_columns(view, 512, 8)
        torch.cuda.synchronize()
        assert torch.equal(full, view.contiguous())
        dense = view.contiguous()  # a dense shard is sent from where it lies
        assert torch.equal(comm.gather_columns(dense, 512, 8), dense)
        odd = y[:, :500].contiguous()  # 1000-byte rows: the element-wise interleave instead of 16-byte pieces
        assert torch.equal(comm.gather_columns(odd, 500, 4), odd)
        b = torch.randn((4, 8, 32), device=dev)
        out = comm.gather_batch(b, 4)
        torch.cuda.synchronize()
        assert torch.equal(out, b)
        assert _fused_gather_check(aclnn, comm, dev, 1, 0)
    finally:
        comm.close()


def _fused_gather_check(aclnn, comm, dev, world, rank):
    """Column shards of a W4A16 decode call stored by the kernel itself into every rank's full output (symmetric memory, peer
    stores), then arrive_and_wait: must equal the NCCL gather of the same shards bit for bit; a bound call that cannot run on
    a streaming decode kernel is refused."""
    import torch

    m, k, n, g = 16, 2048, 4096, 128
    gen = torch.Generator(device=dev).manual_seed(99)  # the same tensors on every rank
    x = torch.randn((m, k), generator=gen, device=dev).to(torch.bfloat16)
    w = torch.randint(-2 ** 31, 2 ** 31 - 1, (k, n // 8), generator=gen, device=dev, dtype=torch.int32)
    sc = (torch.rand((k // g, n), generator=gen, device=dev) * 0.01 + 0.005).to(torch.bfloat16)
    of = (torch.rand((k // g, n), generator=gen, device=dev) * 2 - 1).to(torch.bfloat16)
    b, e = aclnn.shard_range(n, world, rank, 512)
    ws, ss, os_ = w[:, b // 8:e // 8].contiguous(), sc[:, b:e].contiguous(), of[:, b:e].contiguous()
    y_local = torch.empty((m, e - b), dtype=torch.bfloat16, device=dev)
    y_full = comm.symmetric_empty((m, n), torch.bfloat16)
    y_push = comm.symmetric_empty((m, n), torch.bfloat16)
    comm.bind_columns(y_local, y_full, 512)
    ok = True
    try:
        for rep in range(3):  # repeated steps: the arrival epochs advance
            xr = (x.float() * (rep + 1)).to(torch.bfloat16)
            aclnn.weight_quant_batch_matmul(aclnn.from_torch(xr), aclnn.from_torch(ws), aclnn.from_torch(ss), aclnn.from_torch(y_local),
                                            aclnn.from_torch(os_), None, g)
            assert aclnn.last_kernel_name() == "wqbmm_decode"
            comm.arrive_and_wait()
            torch.cuda.synchronize()
            fused = y_full.clone()
            comm.arrive_and_wait()  # nobody overwrites a full output another rank is still reading
            torch.cuda.synchronize()
            ref = comm.gather_columns(y_local, n, 512)
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(fused, ref)) and not bool((fused == 0).all())
            # the one-kernel peer all-gather of the same shard (no binding involved) into a second full output
            comm.allgather_columns_peer(y_local, y_push, 512)
            torch.cuda.synchronize()
            pushed = y_push.clone()
            comm.arrive_and_wait()
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(pushed, ref))
        # the other streaming decode kernels store into the peers the same way: INT4 weight stored (n,k) with (n, groups) scales, and
        # an INT8 weight with a per-channel scale
        w_nk = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), generator=gen, device=dev, dtype=torch.int32)
        sc_nk = (torch.rand((n, k // g), generator=gen, device=dev) * 0.01 + 0.005).to(torch.bfloat16)
        of_nk = (torch.rand((n, k // g), generator=gen, device=dev) * 2 - 1).to(torch.bfloat16)
        w8 = torch.randint(-128, 128, (k, n), generator=gen, device=dev, dtype=torch.int8)
        sc8 = (torch.rand((n,), generator=gen, device=dev) * 0.01 + 0.002).to(torch.bfloat16)
        calls = [
            ("wqbmm_decode", lambda: aclnn.weight_quant_batch_matmul(
                aclnn.from_torch(x), aclnn.from_torch(w_nk[b:e].contiguous().t()), aclnn.from_torch(sc_nk[b:e].contiguous().t()),
                aclnn.from_torch(y_local), aclnn.from_torch(of_nk[b:e].contiguous().t()), None, g)),
            ("wqbmm_decode8", lambda: aclnn.weight_quant_batch_matmul(
                aclnn.from_torch(x), aclnn.from_torch(w8[:, b:e].contiguous()), aclnn.from_torch(sc8[b:e].contiguous()),
                aclnn.from_torch(y_local), None, None, 0)),
        ]
        for name, call in calls:
            call()
            assert aclnn.last_kernel_name() == name, aclnn.last_kernel_name()
            comm.arrive_and_wait()
            torch.cuda.synchronize()
            fused = y_full.clone()
            comm.arrive_and_wait()
            torch.cuda.synchronize()
            ref = comm.gather_columns(y_local, n, 512)
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(fused, ref)) and not bool((fused == 0).all())
        refused = False
        try:  # m = 32 runs as two decode launches on row chunks: not a path that stores into the peers
            x32 = torch.randn((32, k), generator=gen, device=dev).to(torch.bfloat16)
            y32 = torch.empty((32, e - b), dtype=torch.bfloat16, device=dev)
            comm.bind_columns(y32, y_full, 512)
            aclnn.weight_quant_batch_matmul(aclnn.from_torch(x32), aclnn.from_torch(ws), aclnn.from_torch(ss), aclnn.from_torch(y32),
                                            aclnn.from_torch(os_), None, g)
        except aclnn.AclnnError:
            refused = True
        finally:
            comm.unbind(y32)
        ok = ok and refused and comm.status() == 0
        if world > 1:
            # A rank that does not show up: rank 0 announces its arrival and waits; nobody else does. Its wait is bounded (shortened
            # here), the kernel returns by itself and the status word says so. The ranks talk on the host (gloo) in between, and
            # when the others then make the same call they find rank 0's flag already there: the arrival counters agree again.
            import torch.distributed as dist

            os.environ["OPSNN_COMM_POLL_LIMIT"] = "200000"
            if rank == 0:
                comm.arrive_and_wait()
                torch.cuda.synchronize()
                ok = ok and comm.status() == 1
            dist.barrier()
            if rank != 0:
                comm.arrive_and_wait()
                torch.cuda.synchronize()
                ok = ok and comm.status() == 0
            dist.barrier()
            os.environ.pop("OPSNN_COMM_POLL_LIMIT")
            comm.arrive_and_wait()  # and an ordinary one afterwards
            torch.cuda.synchronize()
            ok = ok and comm.status() == 0
    finally:
        comm.unbind(y_local)
    return ok


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, ret):
    import sys

    import torch
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from conftest import load_package

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)  # host-side rendezvous only: hands the NCCL id around
    try:
        pkg = load_package()
        aclnn = pkg.aclnn
        comm = aclnn.Comm(world, rank, dev)
        ok_cols = True
        # 193 units of 8 columns: uneven shares (97 / 96 units), runs of whole 16-byte pieces; 385 units of 4 columns: shares of
        # 1544 and 1536 bytes per row, moved element by element
        for m, n, mult in ((16, 1544, 8), (16, 1540, 4)):
            full = (torch.arange(m * n, dtype=torch.float32).reshape(m, n) % 251).to(torch.bfloat16)
            b, e = aclnn.shard_range(n, world, rank, mult)
            got = comm.gather_columns(full[:, b:e].to(dev), n, mult)
            torch.cuda.synchronize()
            ok_cols = ok_cols and bool(torch.equal(got.cpu(), full))
        bat = torch.arange(4 * 6 * 10, dtype=torch.float32).reshape(4, 6, 10)
        bb, be = aclnn.shard_range(4, world, rank, 1)
        gotb = comm.gather_batch(bat[bb:be].to(dev), 4)
        torch.cuda.synchronize()
        ok_fused = _fused_gather_check(aclnn, comm, dev, world, rank)
        ret[rank] = (ok_cols, bool(torch.equal(gotb.cpu(), bat)), ok_fused)
        comm.close()
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_over_nccl(aclnn):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs; the single-rank test above covers the same calls on one")
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_rank_main, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(240)
        for p in procs:
            assert p.exitcode == 0
        assert dict(ret) == {0: (True, True, True), 1: (True, True, True)}
