"""GPU parity of the rank-order sum (through the C ABI) against its CPU restatement: bit-exact."""

import ctypes

import pytest
import torch

from oracle import rank_sum_ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    from gaudi_kernels_b200 import _lib
    return _lib.load()


def _data(world, elems, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(world * elems, generator=g) * 3
    # magnitudes far apart make the order of the fp32 additions visible in the result
    x[::7] *= 1e6
    x[3::11] *= 1e-6
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("world,elems", [(2, 1), (2, 4096), (3, 1000), (4, 4096), (5, 777), (8, 65536), (8, 12345), (4, 1 << 20)])
def test_rank_sum_matches_restatement_bit_for_bit(lib, world, elems, dtype):
    from gaudi_kernels_b200 import _lib
    x = _data(world, elems, dtype, seed=world * 1000 + elems)
    want = rank_sum_ref.rank_sum(x, world)
    xd = x.cuda()
    out = torch.full((elems + 16,), 7.0, dtype=dtype, device="cuda")
    code = _lib.OUT_BF16 if dtype == torch.bfloat16 else _lib.OUT_F32
    rc = lib.bfp8_rank_sum(xd.data_ptr(), out.data_ptr(), elems, world, code, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert torch.equal(out[:elems].cpu(), want)
    assert bool((out[elems:] == 7.0).all())
    # the order matters for this data: summing in reverse rank order gives different bits somewhere
    if world > 2 and elems > 100 and dtype == torch.float32:
        rev = rank_sum_ref.rank_sum(x.view(world, elems).flip(0).reshape(-1).contiguous(), world)
        assert not torch.equal(rev, want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rank_sum_slices_unaligned_and_bias(lib, dtype):
    """Slices given by pointer: separate allocations, an odd element offset (scalar path), and the bias."""
    from gaudi_kernels_b200 import _lib
    world, rows, n = 3, 5, 264
    elems = rows * n
    code = _lib.OUT_BF16 if dtype == torch.bfloat16 else _lib.OUT_F32
    x = _data(world, elems, dtype, seed=5)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(1))
    want = rank_sum_ref.rank_sum(x, world)
    # the bias joins the fp32 sum before the single rounding
    want_b = (rank_sum_ref.rank_sum(x.float(), world).view(rows, n) + bias).to(dtype).view(-1)
    for offset in (0, 1):
        holders = [torch.zeros(elems + 8, dtype=dtype, device="cuda") for _ in range(world)]
        for r in range(world):
            holders[r][offset:offset + elems] = x[r * elems:(r + 1) * elems].cuda()
        ptrs = (ctypes.c_void_p * world)(*[h.data_ptr() + offset * h.element_size() for h in holders])
        out = torch.empty(elems, dtype=dtype, device="cuda")
        stream = torch.cuda.current_stream().cuda_stream
        assert lib.bfp8_rank_sum_slices(ptrs, out.data_ptr(), elems, world, code, None, 0, stream) == 0
        assert torch.equal(out.cpu(), want)
        assert lib.bfp8_rank_sum_slices(ptrs, out.data_ptr(), elems, world, code, bias.cuda().data_ptr(), n, stream) == 0
        assert torch.equal(out.cpu(), want_b)


def test_single_rank_exchange_and_barrier(lib):
    """The peer buffer, its torch view and the barrier kernel with one rank (a world of one needs no peer)."""
    import os
    import torch.distributed as dist
    from gaudi_kernels_b200.row_parallel import PeerExchange, reduce_scatter_rows
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29591")
    created = not dist.is_initialized()
    if created:
        dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        ex = PeerExchange(64 * 128 * 4)
        p = ex.partial(64, 128, torch.float32)
        assert p.data_ptr() == ex.ptrs[0] and not bool(p.any())            # zero-filled, at the buffer's start
        p.copy_(torch.arange(64 * 128, dtype=torch.float32, device="cuda").view(64, 128))
        out = reduce_scatter_rows(ex, p, bias=torch.ones(128))
        assert torch.equal(out, p + 1) and ex.epoch == 2 and not ex.timed_out()
        with pytest.raises(ValueError):
            ex.partial(65, 128, torch.float32)
        ex.close()
    finally:
        if created:
            dist.destroy_process_group()


def test_barrier_wait_expires_with_a_status_not_a_hang(lib):
    """Failure detection on the device: a rank that never arrives makes the bounded wait run out; the kernel
    raises BFP8_STATUS_WAIT_TIMEOUT and returns, and the context stays usable.  The absent rank is simply a flag
    array nothing writes to (no second process, no fault)."""
    import time
    from gaudi_kernels_b200 import _lib
    mine = torch.zeros(8, dtype=torch.int32, device="cuda")
    absent = torch.zeros(8, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    flags = (ctypes.c_void_p * 2)(mine.data_ptr(), absent.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    rc = lib.bfp8_peer_barrier(flags, 0, 2, 1, 2_000_000, status.data_ptr() + 8, stream)      # about a millisecond
    assert rc == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert int(status.cpu()[2]) & _lib.STATUS_WAIT_TIMEOUT
    assert int(absent.cpu()[0]) == 1 and int(mine.cpu()[0]) == 1        # this rank did publish its epoch to both
    # when the other rank has arrived (its flag is set), the same call completes without the status bit
    status.zero_()
    mine[1] = 2
    assert lib.bfp8_peer_barrier(flags, 0, 2, 2, 2_000_000, status.data_ptr() + 8, stream) == 0
    torch.cuda.synchronize()
    assert int(status.cpu()[2]) == 0
    # host-visible argument errors launch nothing
    assert lib.bfp8_peer_barrier(flags, 2, 2, 1, 0, status.data_ptr() + 8, stream) == -3
    assert lib.bfp8_peer_barrier(flags, 0, 9, 1, 0, status.data_ptr() + 8, stream) == -3
    x = torch.arange(8, device="cuda")
    assert int(x.sum()) == 28                                           # the context still works
