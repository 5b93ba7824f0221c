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
