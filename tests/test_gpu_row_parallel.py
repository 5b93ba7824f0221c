"""Two-GPU test of the row-parallel (K-sharded) GEMM with the rank-order sum over peer memory.

Needs two GPUs of one box; skipped otherwise.  Each rank is a child process on its own GPU (never two ranks on
one GPU: the barrier kernels of the ranks wait for one another).  Host-side rendezvous over gloo on 127.0.0.1.
"""

import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, m, k, n, partial_name, use_bias, result_queue):
    try:
        sys.path.insert(0, ROOT)
        import torch.distributed as dist
        from oracle import block_fp8_ref, rank_sum_ref
        import gaudi_kernels_b200 as gk
        from gaudi_kernels_b200 import row_parallel as rp
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        partial_dtype = getattr(torch, partial_name)
        g = torch.Generator().manual_seed(1234 + m + n)                     # every rank builds the same problem
        x = torch.randn((m, k), generator=g).to(torch.bfloat16)
        w = (torch.randn((n, k), generator=g) * 0.02)
        grid = ((n + 127) // 128, (k + 127) // 128)
        s = torch.rand(grid, generator=g) * 2e-4 + 1e-4
        kp, npad = grid[1] * 128, grid[0] * 128
        wp = torch.nn.functional.pad(w, (0, kp - k, 0, npad - n))
        q = (wp.view(grid[0], 128, grid[1], 128) / s.view(grid[0], 1, grid[1], 1)).clamp(-448, 448)
        codes = q.reshape(npad, kp)[:n, :k].contiguous().to(torch.float8_e4m3fn)
        bias = torch.randn(n, generator=g) * 0.1 if use_bias else None

        k0, k1 = rp.k_shard_bounds(k, world, rank)
        w_dev, s_dev = gk.prepare_weight(codes.cuda(), s.cuda(), native_half=True)
        w_loc, s_loc = rp.shard_weight_k(w_dev, s_dev, world, rank)
        a_codes, a_scales = gk.quantize_act_1x128(x[:, k0:k1].contiguous().cuda(), native_half=True)
        ex = rp.PeerExchange(m * n * 4)
        outs = []
        for _ in range(3):                                                   # the buffer is reused call after call
            outs.append(rp.gemm_k_sharded(a_codes, a_scales, w_loc, s_loc, ex, bias=bias, partial_dtype=partial_dtype))
        fused = rp.push_supported(m, n, world, partial_dtype)
        if fused:
            # the same product with the exchange done by the sum kernel instead of the GEMM's epilogue: same bits
            outs.append(rp.gemm_k_sharded(a_codes, a_scales, w_loc, s_loc, ex, bias=bias, partial_dtype=partial_dtype,
                                          fused=False))
        else:
            with pytest.raises(ValueError):
                rp.gemm_k_sharded(a_codes, a_scales, w_loc, s_loc, ex, bias=bias, partial_dtype=partial_dtype, fused=True)
        torch.cuda.synchronize()
        assert not ex.timed_out()
        assert all(torch.equal(outs[0], o) for o in outs[1:])
        r0, r1 = rp.row_bounds(m, world, rank)
        got = outs[0].cpu()
        assert tuple(got.shape) == (r1 - r0, n) and got.dtype == partial_dtype

        # expected: every rank's partial by the oracle (this rank's rows only), rounded as the kernel stores it,
        # then the restated rank-order sum
        parts64, parts = [], []
        for r in range(world):
            a0, a1 = rp.k_shard_bounds(k, world, r)
            y64, ybf = block_fp8_ref.reference_rows(x[r0:r1, a0:a1].contiguous(), codes[:, a0:a1].contiguous(),
                                                    s[:, a0 // 128:(a1 + 127) // 128].contiguous(), native_half=True)
            parts64.append(y64)
            parts.append(ybf if partial_dtype == torch.bfloat16 else y64.float())
        want = rank_sum_ref.rank_sum(torch.stack(parts).reshape(-1).contiguous(), world).view(r1 - r0, n)
        if bias is not None:
            want = (want.float() + bias).to(partial_dtype)
        total64 = sum(parts64) + (bias.double() if bias is not None else 0.0)
        rms = float(total64.pow(2).mean().sqrt())
        err = float((got.double() - total64).abs().max())
        step = 2.0 ** -7 * float(total64.abs().max()) if partial_dtype == torch.bfloat16 else 0.0
        assert err <= 1e-2 * rms * world + (world + 1) * step, (err, rms)
        close = float((got.double() - want.double()).abs().max())
        assert close <= 1e-2 * rms * world + (world + 1) * step, close
        ex.close()
        dist.destroy_process_group()
        result_queue.put((rank, "ok", (err / rms, fused)))
    except Exception as e:                                                   # noqa: BLE001 - reported to the parent
        import traceback
        result_queue.put((rank, "fail", traceback.format_exc() + repr(e)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("m,k,n,partial,bias", [(256, 1024, 512, "bfloat16", True), (300, 1152, 640, "float32", False),
                                                 (5, 2048, 1024, "bfloat16", False), (2048, 4096, 2048, "bfloat16", True),
                                                 (8, 2048, 1024, "bfloat16", True), (64, 14336, 4096, "bfloat16", False),
                                                 (128, 512, 8192, "bfloat16", False)])
def test_row_parallel_gemm_two_gpus(m, k, n, partial, bias):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (m + n) % 200
    procs = [ctx.Process(target=_worker, args=(r, 2, port, m, k, n, partial, bias, q)) for r in range(2)]
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
        # which form ran: the fused one for M a multiple of 128 * 2, and for the decode bucket with even M
        assert info[1] == (partial == "bfloat16" and n % 64 == 0 and (m % 256 == 0 or (m <= 128 and m % 2 == 0)))
