"""Row-parallel (K-sharded) block-FP8 GEMM with a deterministic rank-order reduction over peer memory.

A row-parallel projection (the FFN down projection behind a column-parallel gate/up) keeps on rank r
the K range [k0_r, k1_r) of the weight and receives the matching columns of the activations, so every rank
computes a partial [M, N] product and the partials have to be added.  The reference's only multi-device
kernel defines how: gk_rank_sum_{bf16,f32}_v1 (csrc/tpc/generic_dense/rank_sum.c:4-42) adds the per-rank
slices in canonical rank order with fp32 accumulation, which makes the result independent of timing and of
the collective's algorithm.  There the runtime all-gathers the partials first; here each rank's partial
stays where the GEMM wrote it, in memory the other GPUs of the box have mapped, and the sum kernel of rank r
reads rows [r M / W, (r+1) M / W) of every partial straight over NVLink (plain peer loads, no multicast, no
NCCL on the data path): a reduce-scatter whose order of additions is fixed.

One process per GPU.  The host-side exchange of the memory handles uses the process group (any backend);
the GPUs synchronise through bfp8_peer_barrier, a stream-ordered flag exchange with a bounded wait.
"""

import ctypes

import torch
import torch.distributed as dist

from . import _lib
from .fp8_codec import BLOCK, _status_buffer, _stream_ptr


def k_shard_bounds(k, world, rank):
    """[start, stop) of the K range owned by `rank`: whole 128-wide scale blocks, as even as possible."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    groups = (k + BLOCK - 1) // BLOCK
    if groups < world:
        raise ValueError("K=%d has %d scale blocks, fewer than the %d ranks" % (k, groups, world))
    per, rem = divmod(groups, world)
    g0 = rank * per + min(rank, rem)
    g1 = g0 + per + (1 if rank < rem else 0)
    return g0 * BLOCK, min(k, g1 * BLOCK)


def row_bounds(m, world, rank):
    """[start, stop) of the output rows rank `rank` reduces and keeps (may be empty for tiny M)."""
    per, rem = divmod(m, world)
    r0 = rank * per + min(rank, rem)
    return r0, r0 + per + (1 if rank < rem else 0)


def shard_weight_k(w_codes, w_scales, world, rank):
    """The rank's K slice of a prepared weight: contiguous codes [N, K_local] and scales [ceil(N/128), G_local]."""
    k0, k1 = k_shard_bounds(w_codes.shape[1], world, rank)
    return w_codes[:, k0:k1].contiguous(), w_scales[:, k0 // BLOCK:(k1 + BLOCK - 1) // BLOCK].contiguous()


class _DeviceBytes:
    """Lets torch wrap a raw device pointer (CUDA array interface, bytes)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerExchange:
    """This rank's partial-result buffer, mapped into every rank of the group, plus the barrier flags.

    nbytes  size of the partial-result area (M_max * N * bytes per partial element)
    group   process group whose ranks are the GPUs of one box, one process each (default: the world)
    All ranks must construct it collectively.  close() unmaps and frees; the object is not usable afterwards.
    """

    _FLAG_BYTES = 256

    def __init__(self, nbytes, group=None, device=None):
        if not torch.cuda.is_available():
            raise _lib.Bfp8Error("a CUDA device is required; this package has no CPU path")
        self.lib = _lib.load()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if not 1 <= self.world <= 8:
            raise ValueError("1 to 8 ranks supported (rank_sum's range, generic_dense_glue.cpp:576)")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.epoch = 0
        self._opened = []
        with torch.cuda.device(self.device):
            own = ctypes.c_void_p()
            _lib.check(self.lib.bfp8_peer_alloc(self.nbytes + self._FLAG_BYTES, ctypes.byref(own)), "bfp8_peer_alloc")
            self._own = own.value
            handle = (ctypes.c_uint8 * 64)()
            _lib.check(self.lib.bfp8_peer_export(self._own, handle), "bfp8_peer_export")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            self.ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.ptrs.append(self._own)
                    continue
                p = ctypes.c_void_p()
                buf = (ctypes.c_uint8 * 64).from_buffer_copy(h)
                _lib.check(self.lib.bfp8_peer_open(buf, ctypes.byref(p)), "bfp8_peer_open")
                self._opened.append(p.value)
                self.ptrs.append(p.value)
            self._flag_ptrs = (ctypes.c_void_p * self.world)(*[p + self.nbytes for p in self.ptrs])
            self._bytes = torch.as_tensor(_DeviceBytes(self._own, self.nbytes), device=self.device)
            self.status = _status_buffer(self.device)
        dist.barrier(group=group)              # every rank has mapped every buffer before anyone uses them

    def partial(self, m, n, dtype):
        """This rank's partial-result tensor [m, n] of `dtype` at the start of the shared buffer."""
        need = m * n * torch.empty((), dtype=dtype).element_size()
        if need > self.nbytes:
            raise ValueError("partial result of %d bytes exceeds the exchange buffer (%d)" % (need, self.nbytes))
        return self._bytes[:need].view(dtype).view(m, n)

    def barrier(self):
        """Enqueue the inter-GPU barrier on the current stream (every rank must call it equally often)."""
        self.epoch = (self.epoch + 1) & 0xFFFFFFFF
        with torch.cuda.device(self.device):
            rc = self.lib.bfp8_peer_barrier(self._flag_ptrs, self.rank, self.world, self.epoch, 0,
                                            self.status.data_ptr() + 8, _stream_ptr())
        _lib.check(rc, "bfp8_peer_barrier")

    def timed_out(self):
        """True if a bounded wait expired in a barrier or in a GEMM launched by gemm_k_sharded (reads the status
        word: one synchronisation).  The cached small-M workspaces are dropped then: their arrival counters may
        have been left non-zero."""
        from .block_fp8_gemm import wait_timed_out
        return wait_timed_out(self.status)

    def close(self):
        if self._own is None:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            dist.barrier(group=self.group)     # nobody unmaps while a peer may still read
            for p in self._opened:
                self.lib.bfp8_peer_close(p)
            dist.barrier(group=self.group)
            self.lib.bfp8_peer_free(self._own)
        self._own, self._opened, self._bytes = None, [], None


def reduce_scatter_rows(exchange, partial, bias=None, out=None, out_dtype=None):
    """Rank-order sum of all ranks' `partial` ([M, N], from exchange.partial) over this rank's rows.

    Enqueues barrier -> sum kernel -> barrier on the current stream: the first makes every rank's partial
    complete and visible, the second keeps a rank from overwriting its partial while a peer still reads it.
    Returns [rows of this rank, N] of the partial's dtype (bf16 or fp32), with fp32 `bias` [N] added after the sum.
    """
    m, n = partial.shape
    dtype = partial.dtype
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("partials must be bfloat16 or float32")
    out_dtype = dtype if out_dtype is None else out_dtype
    if out_dtype != dtype:
        raise ValueError("the sum keeps the partials' dtype (rank_sum.c:24-41)")
    esz = partial.element_size()
    r0, r1 = row_bounds(m, exchange.world, exchange.rank)
    if out is None:
        out = torch.empty((r1 - r0, n), dtype=dtype, device=exchange.device)
    elif tuple(out.shape) != (r1 - r0, n) or out.dtype != dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous [rows of this rank, N] tensor of the partials' dtype")
    if bias is not None:
        if bias.numel() != n:
            raise ValueError("bias with N elements required")
        bias = bias.to(device=exchange.device, dtype=torch.float32).contiguous().view(-1)
    exchange.barrier()
    if r1 > r0:
        if exchange.world == 1:
            out.copy_(partial[r0:r1] if bias is None else (partial[r0:r1].float() + bias).to(dtype))
        else:
            slices = (ctypes.c_void_p * exchange.world)(*[p + r0 * n * esz for p in exchange.ptrs])
            with torch.cuda.device(exchange.device):
                rc = exchange.lib.bfp8_rank_sum_slices(
                    slices, out.data_ptr(), (r1 - r0) * n, exchange.world,
                    _lib.OUT_BF16 if dtype == torch.bfloat16 else _lib.OUT_F32,
                    bias.data_ptr() if bias is not None else None, n, _stream_ptr())
            _lib.check(rc, "bfp8_rank_sum_slices")
    exchange.barrier()
    return out


def push_supported(m, n, world, partial_dtype=torch.bfloat16):
    """True where the GEMM can scatter its result itself (bfp8_gemm_block128_push): M a multiple of 128 * world
    (large-tile schedule) or the decode bucket M <= 128 with M a multiple of world (weight-streaming schedule)."""
    if world < 2 or partial_dtype != torch.bfloat16 or n % 64 != 0:
        return False
    return m % (BLOCK * world) == 0 or (m <= 128 and m % world == 0)


def gemm_k_sharded(a_codes_local, a_scales_local, w_codes_local, w_scales_local, exchange, bias=None,
                   partial_dtype=torch.bfloat16, out=None, fused=None):
    """Row-parallel GEMM: this rank's K slice in, this rank's rows of the full-K product out.

    a_codes_local [M, K_local] / a_scales_local [M, G_local] quantize this rank's activation columns
    (the 1x128 groups never straddle ranks because K slices are whole scale blocks); w_*_local from
    shard_weight_k.  Two forms, same rank-order result:

    fused    the GEMM's epilogue stores every bf16 tile into the receive area of the GPU that owns its rows
             (bfp8_gemm_block128_push), so the exchange overlaps the math; after the barrier each rank holds the
             `gathered` layout of rank_sum.c and sums it locally.  Needs N % 64 == 0 and M % (128 * world) == 0, or
             the decode bucket M <= 128 with M % world == 0 (each activation row is stored to its owner).
    unfused  the partial is written locally in `partial_dtype` (bf16 or fp32) and reduce_scatter_rows reads the
             peers' rows over NVLink.  fp32 partials take any shape; bf16 partials need N % 8 == 0 (their rows are
             stored in 16-byte units, BFP8_ERR_ALIGN otherwise).
    Either form reports an expired bounded wait (GEMM or barrier) through exchange.timed_out().
    fused=None picks the fused form where it applies.
    """
    from .block_fp8_gemm import _group_major, _workspace, gemm_block_fp8
    m, k = a_codes_local.shape
    n = w_codes_local.shape[0]
    world, rank = exchange.world, exchange.rank
    can_push = push_supported(m, n, world, partial_dtype) and k % 16 == 0
    if fused is None:
        fused = can_push
    if fused and not can_push:
        raise ValueError("the fused form needs bf16 partials, N % 64 == 0, K % 16 == 0 and M % (128 * world) == 0 "
                         "(or M <= 128 with M % world == 0)")
    if not fused:
        partial = exchange.partial(m, n, partial_dtype)
        gemm_block_fp8(a_codes_local, a_scales_local, w_codes_local, w_scales_local, out=partial,
                       out_dtype=partial_dtype, check=False, status=exchange.status)
        return reduce_scatter_rows(exchange, partial, bias=bias, out=out)

    rows = m // world
    if m * n * 2 > exchange.nbytes:
        raise ValueError("receive area of %d bytes exceeds the exchange buffer (%d)" % (m * n * 2, exchange.nbytes))
    g = (k + BLOCK - 1) // BLOCK
    dev = exchange.device
    if out is None:
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=dev)
    elif tuple(out.shape) != (rows, n) or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError("out must be a contiguous bf16 [M / world, N] tensor")
    if bias is not None:
        if bias.numel() != n:
            raise ValueError("bias with N elements required")
        bias = bias.to(device=dev, dtype=torch.float32).contiguous().view(-1)
    lib = exchange.lib
    with torch.cuda.device(dev):
        sa, ldsa = _group_major(a_scales_local, m, g)
        recv = (ctypes.c_void_p * world)(*exchange.ptrs)
        ws_bytes = lib.bfp8_gemm_block128_workspace_bytes(m, n, k) if m <= 128 else 0
        ws = _workspace(dev, ws_bytes) if ws_bytes else None
        rc = lib.bfp8_gemm_block128_push(
            a_codes_local.data_ptr(), a_codes_local.stride(0), sa.data_ptr(), ldsa, w_codes_local.data_ptr(),
            w_codes_local.stride(0), w_scales_local.data_ptr(), recv, rank, world, m, n, k,
            ws.data_ptr() if ws is not None else None, ws_bytes, exchange.status.data_ptr() + 8, _stream_ptr())
        _lib.check(rc, "bfp8_gemm_block128_push")
        exchange.barrier()                                   # every rank's tiles have landed here
        slices = (ctypes.c_void_p * world)(*[exchange.ptrs[rank] + r * rows * n * 2 for r in range(world)])
        rc = lib.bfp8_rank_sum_slices(slices, out.data_ptr(), rows * n, world, _lib.OUT_BF16,
                                      bias.data_ptr() if bias is not None else None, n, _stream_ptr())
        _lib.check(rc, "bfp8_rank_sum_slices")
        exchange.barrier()                                   # the receive area may be overwritten again
    return out
