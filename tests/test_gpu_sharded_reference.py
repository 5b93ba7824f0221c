"""`sharded.reference_sharded` on two GPUs (one process each, NCCL): every rank uploads and quantizes only its rows,
codes and scales are all-gathered, and each rank's [M, N / 2] slice must equal `reference()` on the same columns bit for
bit - quantization is row-local, so sharding the rows changes nothing.  Skipped on a one-GPU box; the host-side
arrangement of the gathered scales is also tested on CPU under gloo (tests/test_sharded_gloo.py)."""

import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, m, k, n, result_queue):
    try:
        sys.path.insert(0, ROOT)
        import torch.distributed as dist
        import gaudi_kernels_b200 as gk
        from gaudi_kernels_b200 import sharded
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        g = torch.Generator().manual_seed(99 + m + n)                        # every rank builds the same problem
        x = torch.randn((m, k), generator=g).to(torch.bfloat16)
        w = torch.randn((n, k), generator=g) * 0.02
        w_ocp, s_ocp = gk.quantize_block128(w.cuda())
        w_ocp, s_ocp = w_ocp.cpu(), s_ocp.cpu()
        bias = torch.randn(n, generator=g) * 0.1
        lo, hi = sharded.shard_bounds(n, world, rank)
        rows = m // world
        for half in (True, False):
            want = gk.reference(x, w_ocp[lo:hi].contiguous(), s_ocp[lo // 128:hi // 128].contiguous(), native_half=half,
                                bias=bias[lo:hi])                            # the unsharded call on this rank's columns
            got = sharded.reference_sharded(x[rank * rows:(rank + 1) * rows].contiguous(), w_ocp[lo:hi].contiguous(),
                                            s_ocp[lo // 128:hi // 128].contiguous(), native_half=half,
                                            bias_local=bias[lo:hi])
            assert got.device.type == "cpu" and tuple(got.shape) == (m, hi - lo)
            assert torch.equal(got, want), half
            # device tensors in, device tensor out
            got_dev = sharded.reference_sharded(x[rank * rows:(rank + 1) * rows].cuda(), w_ocp[lo:hi].cuda(),
                                                s_ocp[lo // 128:hi // 128].cuda(), native_half=half, bias_local=bias[lo:hi].cuda())
            assert got_dev.device.type == "cuda" and torch.equal(got_dev.cpu(), want)
        bad = x[rank * rows:(rank + 1) * rows].clone()
        if rank == 0:
            bad[0, 0] = float("inf")                                         # only this rank sees it; every rank must raise
        try:
            sharded.reference_sharded(bad, w_ocp[lo:hi].contiguous(), s_ocp[lo // 128:hi // 128].contiguous(), native_half=True)
            raised = False
        except ValueError:
            raised = True
        assert raised
        dist.barrier()
        dist.destroy_process_group()
        result_queue.put((rank, "ok", ""))
    except Exception as e:                                                   # noqa: BLE001 - reported to the parent
        import traceback
        result_queue.put((rank, "fail", traceback.format_exc() + repr(e)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("m,k,n", [(256, 1024, 512), (4096, 2048, 1024), (6, 384, 256)])
def test_reference_sharded_two_gpus(m, k, n):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29800 + (m + n) % 150
    procs = [ctx.Process(target=_worker, args=(r, 2, port, m, k, n, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in procs:
            results.append(q.get(timeout=240))
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    assert sorted(r[0] for r in results) == [0, 1]
    for rank, state, info in results:
        assert state == "ok", "rank %d: %s" % (rank, info)
