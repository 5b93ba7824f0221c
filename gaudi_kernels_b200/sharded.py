"""Column (N) sharding of the block-FP8 GEMM across the GPUs of one box.

Output columns are independent, so rank r keeps the weight rows [r*N/world, (r+1)*N/world) with
their scale rows, activations are replicated, and every rank runs the single-GPU kernel on its slice.
There is no collective on the data path.  `gather_columns` is the one exchange a caller adds when it
needs the full [M, N] output on every rank (one all-gather of the bf16 slices over NCCL / NVLink);
a column-parallel projection that feeds a row-parallel one never calls it.

The reference has no distributed code; the only multi-device artefact there is the rank-order local
sum gk_rank_sum (csrc/tpc/generic_dense/rank_sum.c:4-42), which belongs to the row-parallel case.
"""

import torch
import torch.distributed as dist

from .fp8_codec import BLOCK


def shard_bounds(n, world, rank):
    """[start, stop) of the weight rows (output columns) owned by `rank`; slices are 128-aligned."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    blocks = (n + BLOCK - 1) // BLOCK
    if blocks % world != 0:
        raise ValueError("the %d scale-block rows of N=%d do not split evenly over %d ranks" % (blocks, n, world))
    per = blocks // world
    start = rank * per * BLOCK
    stop = min(n, (rank + 1) * per * BLOCK)
    return start, stop


def shard_weight(w_codes, w_scales, world, rank):
    """The rank's slice of a prepared weight: codes [N_local, K] and scales [N_local/128, G] (views)."""
    n = w_codes.shape[0]
    start, stop = shard_bounds(n, world, rank)
    return w_codes[start:stop], w_scales[start // BLOCK:(stop + BLOCK - 1) // BLOCK]


def gemm_sharded(a_codes, a_scales, w_codes_local, w_scales_local, bias_local=None, out=None, status=None):
    """This rank's [M, N_local] slice of the product (no communication).

    The launch is not followed by a synchronisation.  Pass `status` (block_fp8_gemm.new_status(device), shared by
    as many calls as you like) and test it with block_fp8_gemm.wait_timed_out(status) once the step is complete:
    a kernel whose bounded wait expired reports it there and its output is invalid.
    """
    from .block_fp8_gemm import gemm_block_fp8
    return gemm_block_fp8(a_codes, a_scales, w_codes_local, w_scales_local, bias=bias_local, out=out, check=False,
                          status=status)


def gather_columns(local_out, group=None):
    """All-gather equally sized column slices [M, N_local] into the full [M, world * N_local] on every rank."""
    world = dist.get_world_size(group)
    m, n_local = local_out.shape
    stacked = torch.empty((world * m, n_local), dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(stacked, local_out.contiguous(), group=group)     # rank r's slice at rows [r*m, (r+1)*m)
    return stacked.view(world, m, n_local).permute(1, 0, 2).reshape(m, world * n_local)


def gather_quantized_rows(codes_local, scales_local, group=None):
    """All-gather row-sharded quantized activations: rank r holds rows [r R, (r + 1) R) as codes [R, K] and
    group-major 1x128 scales [G, R].  Returns (codes [W R, K], scales [G, W R]) - the layout the GEMM reads
    (scale of row i, group g at scales[g, i]).  Two collectives; works on any backend."""
    world = dist.get_world_size(group)
    rows, k = codes_local.shape
    groups = scales_local.shape[0]
    if tuple(scales_local.shape) != (groups, rows):
        raise ValueError("scales must be group-major [G, rows]")
    codes = torch.empty((world * rows, k), dtype=codes_local.dtype, device=codes_local.device)
    gathered = torch.empty((world, groups, rows), dtype=scales_local.dtype, device=scales_local.device)
    dist.all_gather_into_tensor(codes.view(-1), codes_local.contiguous().view(-1), group=group)
    dist.all_gather_into_tensor(gathered.view(-1), scales_local.contiguous().view(-1), group=group)
    return codes, gathered.permute(1, 0, 2).reshape(groups, world * rows)


def reference_sharded(x_local, weight_local, scales_local, *, native_half=True, bias_local=None, out=None, group=None):
    """Column-sharded form of `reference()` for host (or device) tensors, one call per rank.

    The unsharded call uploads and quantizes all of `x` on every GPU.  Here rank r is given only its rows
    x_local = x[r M / W : (r + 1) M / W] (bf16 [M / W, K]) and its weight slice (weight_local float8_e4m3fn
    [N / W, K] OCP codes, scales_local fp32 [N / W / 128, G]): it uploads and quantizes those rows
    (block_fp8_oracle.py:25-28, :31-34), the ranks all-gather the E4M3 codes and the 1x128 scales over NCCL
    (1.03 bytes per activation element instead of 2 over PCIe on every GPU), and each rank multiplies the full
    activation matrix with its weight slice.  Returns this rank's [M, N / W] slice of the product, on the host
    when x_local is a host tensor (into `out` when given; a pinned tensor keeps the copy asynchronous until the
    final wait).  Results equal `reference()` on the same columns bit for bit: the quantization is row-local.
    Every rank must pass the same number of rows (M is a multiple of the group size), and every rank makes the call:
    it contains two all-gathers and one small all-reduce of the status bits.
    """
    from . import _lib
    from .block_fp8_gemm import _copy_stream, _workspaces, _WAIT_TIMEOUT_MSG, gemm_block_fp8
    from .fp8_codec import _device_for, _status_buffer, _stream_ptr
    if (x_local.dtype != torch.bfloat16 or weight_local.dtype != torch.float8_e4m3fn or scales_local.dtype != torch.float32
            or x_local.ndim != 2 or weight_local.ndim != 2 or x_local.shape[1] != weight_local.shape[1]):
        raise ValueError("BF16 activation rows, original OCP FP8 weight slice and FP32 scales required")
    world = dist.get_world_size(group)
    rows, k = x_local.shape
    n_local = weight_local.shape[0]
    groups = (k + BLOCK - 1) // BLOCK
    if tuple(scales_local.shape) != ((n_local + BLOCK - 1) // BLOCK, groups):
        raise ValueError("original block128 scale grid mismatch")
    m = rows * world
    lib = _lib.load()
    dev = _device_for(x_local, weight_local, scales_local)
    on_host = x_local.device.type == "cpu"
    with torch.cuda.device(dev):
        st = _status_buffer(dev)
        wd = weight_local.to(dev, non_blocking=True).contiguous()
        sd = scales_local.to(dev, non_blocking=True).contiguous()
        if native_half:
            enc, sw = torch.empty_like(wd), torch.empty_like(sd)
            rc = lib.bfp8_reencode_half(wd.data_ptr(), enc.data_ptr(), wd.numel(), sd.data_ptr(), sw.data_ptr(), sd.numel(),
                                        st.data_ptr(), st.data_ptr() + 8, _stream_ptr())
            _lib.check(rc, "bfp8_reencode_half")
        else:
            enc, sw = wd, sd
            rc = lib.bfp8_validate_e4m3(wd.data_ptr(), wd.numel(), sd.data_ptr(), sd.numel(), st.data_ptr() + 8, _stream_ptr())
            _lib.check(rc, "bfp8_validate_e4m3")
        xd = x_local.to(dev, non_blocking=True).contiguous()
        codes_local = torch.empty((rows, k), dtype=torch.uint8, device=dev)
        scales_l = torch.empty((groups, rows), dtype=torch.float32, device=dev)
        rc = lib.bfp8_quant_act_1x128_bf16(xd.data_ptr(), rows, k, xd.stride(0), codes_local.data_ptr(), k, scales_l.data_ptr(),
                                           1, rows, int(bool(native_half)), st.data_ptr() + 8, _stream_ptr())
        _lib.check(rc, "bfp8_quant_act_1x128_bf16")
        # the one exchange: codes [M, K] (rank r's rows at [r rows, (r + 1) rows)) and group-major scales [G, M]
        a_codes, a_scales = gather_quantized_rows(codes_local, scales_l, group)
        if not on_host:
            y = gemm_block_fp8(a_codes, a_scales.t(), enc, sw, bias=bias_local,
                               out=out if (out is not None and out.device.type == "cuda") else None, check=False, status=st)
        else:
            if out is None:
                out = torch.empty((m, n_local), dtype=torch.bfloat16)
            elif tuple(out.shape) != (m, n_local) or out.dtype != torch.bfloat16:
                raise ValueError("out must be bf16 [M, N / world]")
            # the copy of the result back to the host dominates: row blocks, each copied on a second stream while
            # the next block is multiplied
            blocks = max(1, min(8, m // 2048))
            per = ((m + blocks - 1) // blocks + BLOCK - 1) // BLOCK * BLOCK
            main, side = torch.cuda.current_stream(), _copy_stream(dev)
            keep = []
            for r0 in range(0, m, per):
                r1 = min(m, r0 + per)
                yr = gemm_block_fp8(a_codes[r0:r1], a_scales[:, r0:r1].t(), enc, sw, bias=bias_local, check=False, status=st)
                done = torch.cuda.Event()
                done.record(main)
                side.wait_event(done)
                with torch.cuda.stream(side):
                    out[r0:r1].copy_(yr, non_blocking=True)
                keep.append(yr)
            main.wait_stream(side)
            y = out
        # a condition seen by one rank (a non-finite activation in its rows, a bad code in its weight slice, an
        # expired wait) invalidates every rank's slice: the status bits are OR-ed over the group (as a MAX over
        # one flag per bit, NCCL has no bitwise reduction) before anybody reads them
        bits = (st[2:3] >> torch.arange(4, dtype=torch.int32, device=dev)) & 1
        dist.all_reduce(bits, op=dist.ReduceOp.MAX, group=group)
        status = sum(int(b) << i for i, b in enumerate(bits.cpu().tolist()))   # synchronises: also completes the copies
        if status & (_lib.STATUS_NONFINITE_CODE | _lib.STATUS_BAD_SCALE | _lib.STATUS_NONFINITE_INPUT):
            raise ValueError("finite original inputs required")
        if status & _lib.STATUS_WAIT_TIMEOUT:
            _workspaces.clear()
            raise _lib.Bfp8Error(_WAIT_TIMEOUT_MSG)
    return y
