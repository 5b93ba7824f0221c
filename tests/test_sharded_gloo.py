"""Host logic of the N-sharded GEMM on CPU: two gloo ranks, each computing its column slice with the
CPU oracle (no GPU), gathered and compared with the unsharded oracle result bit for bit."""

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from gaudi_kernels_b200 import sharded
        from oracle import block_fp8_ref, fp8_codec_ref
        rng = np.random.default_rng(0)                       # same inputs on every rank
        m, k, n = 6, 384, 512
        x = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).to(torch.bfloat16)
        codes, scales = fp8_codec_ref.quantize_block128(rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
        w = torch.from_numpy(codes).view(torch.float8_e4m3fn)
        s = torch.from_numpy(scales)
        full = block_fp8_ref.reference(x, w, s, native_half=True)
        w_loc, s_loc = sharded.shard_weight(w, s, world, rank)
        start, stop = sharded.shard_bounds(n, world, rank)
        assert w_loc.shape[0] == stop - start == n // world and s_loc.shape[0] == (stop - start) // 128
        local = block_fp8_ref.reference(x, w_loc.contiguous(), s_loc.contiguous(), native_half=True)
        assert torch.equal(local, full[:, start:stop])       # a slice equals the same columns of the full product
        gathered = sharded.gather_columns(local)
        assert torch.equal(gathered, full)
        # row-sharded quantization + gather of codes and scales (the exchange of reference_sharded) equals
        # quantizing all rows in one place
        rows = m // world
        c_all, s_all = fp8_codec_ref.quantize_act_1x128(x.float().numpy(), native_half=True)          # [M, K], [M, G]
        c_loc, s_loc_a = fp8_codec_ref.quantize_act_1x128(x[rank * rows:(rank + 1) * rows].float().numpy(), native_half=True)
        codes_g, scales_g = sharded.gather_quantized_rows(torch.from_numpy(c_loc),
                                                          torch.from_numpy(np.ascontiguousarray(s_loc_a.T)))
        assert np.array_equal(codes_g.numpy(), c_all) and np.array_equal(scales_g.numpy(), s_all.T)
        open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_column_sharding(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / ("ok%d" % r)).exists() for r in range(world))


def test_shard_bounds():
    sys.path.insert(0, ROOT)
    from gaudi_kernels_b200 import sharded
    assert [sharded.shard_bounds(28672, 8, r) for r in (0, 7)] == [(0, 3584), (25088, 28672)]
    assert sharded.shard_bounds(14336, 1, 0) == (0, 14336)
    with pytest.raises(ValueError):
        sharded.shard_bounds(14336, 3, 0)                     # 112 block rows do not split over 3 ranks
    with pytest.raises(ValueError):
        sharded.shard_bounds(1024, 2, 2)


def test_row_parallel_bounds_cover_everything_once():
    """K slices are whole scale blocks, row slices are contiguous; both partition their range for every world size."""
    from gaudi_kernels_b200.row_parallel import k_shard_bounds, row_bounds
    import pytest
    for world in range(1, 9):
        for k in (1024, 1152, 4096, 14336, 1000, 28672):
            if (k + 127) // 128 < world:
                with pytest.raises(ValueError):
                    k_shard_bounds(k, world, 0)
                continue
            edges = [k_shard_bounds(k, world, r) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == k
            for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
                assert a1 == b0 and a0 % 128 == 0 and a1 % 128 == 0 and a1 > a0
            sizes = [(b - a + 127) // 128 for a, b in edges]
            assert max(sizes) - min(sizes) <= 1
        for m in (1, 5, 8, 300, 8192):
            rows = [row_bounds(m, world, r) for r in range(world)]
            assert rows[0][0] == 0 and rows[-1][1] == m
            assert all(a[1] == b[0] for a, b in zip(rows, rows[1:]))
    with pytest.raises(ValueError):
        k_shard_bounds(1024, 4, 4)


def _row_parallel_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from gaudi_kernels_b200 import row_parallel as rp
        from oracle import block_fp8_ref, fp8_codec_ref, rank_sum_ref
        rng = np.random.default_rng(1)                       # same inputs on every rank
        m, k, n = 8, 640, 256                                # 5 scale blocks of K over 2 ranks: 3 + 2
        x = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).to(torch.bfloat16)
        codes, scales = fp8_codec_ref.quantize_block128(rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
        w = torch.from_numpy(codes).view(torch.float8_e4m3fn)
        s = torch.from_numpy(scales)
        k0, k1 = rp.k_shard_bounds(k, world, rank)
        w_loc, s_loc = rp.shard_weight_k(w, s, world, rank)
        assert tuple(w_loc.shape) == (n, k1 - k0) and tuple(s_loc.shape) == (n // 128, (k1 - k0) // 128)
        assert torch.equal(w_loc.view(torch.uint8), w.view(torch.uint8)[:, k0:k1])
        # this rank's partial over its K slice, in both precisions the sum kernel takes
        y64, ybf = block_fp8_ref.reference_rows(x[:, k0:k1].contiguous(), w_loc, s_loc, native_half=True)
        full64, _ = block_fp8_ref.reference_rows(x, w, s, native_half=True)
        rms = float(full64.pow(2).mean().sqrt())
        for part in (ybf, y64.float()):
            # what the runtime's all-gather hands to rank_sum: world slices back to back, in rank order
            gathered = torch.empty((world,) + tuple(part.shape), dtype=part.dtype)
            dist.all_gather_into_tensor(gathered.view(world * m, n), part.contiguous())
            total = rank_sum_ref.rank_sum(gathered.reshape(-1), world).view(m, n)
            # the 1x128 groups never straddle ranks, so the K-sharded sum is the full product up to rounding
            tol = 1e-5 * rms if part.dtype == torch.float32 else 2.0 ** -7 * float(full64.abs().max()) * (world + 1)
            assert float((total.double() - full64).abs().max()) <= tol
            r0, r1 = rp.row_bounds(m, world, rank)
            mine = total[r0:r1]                              # the rows this rank keeps after the reduce-scatter
            rows = [torch.empty((rp.row_bounds(m, world, r)[1] - rp.row_bounds(m, world, r)[0], n), dtype=part.dtype)
                    for r in range(world)]
            dist.all_gather(rows, mine.contiguous())
            assert torch.equal(torch.cat(rows), total)
        open(os.path.join(out_dir, "rp%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_row_parallel_logic(tmp_path):
    """K sharding + rank-order sum on CPU: two gloo ranks, oracle partials, restated rank_sum, full-K oracle."""
    world = 2
    mp.spawn(_row_parallel_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / ("rp%d" % r)).exists() for r in range(world))
