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
