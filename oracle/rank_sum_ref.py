"""CPU restatement of the reference's rank-order sum. TEST INFRASTRUCTURE ONLY.

Only the test-suite imports this module.  gk_rank_sum_{bf16,f32}_v1 is a Gaudi2 TPC kernel
(csrc/tpc/generic_dense/rank_sum.c:4-42); the reference tests its contract only - world_size 2..8, gathered
size = world_size * elems (tests/generic_dense_glue_contract_test.cpp:533-586, glue
csrc/host/generic_dense_glue.cpp:569-600) - and holds no numeric vector for it, so the values are unpinned
and this file restates the kernel's arithmetic from its source: the accumulator starts as slice 0 widened to
fp32 (:24-25, :36), slices 1 .. W-1 are added one after the other with fp32 additions (:26-32, :37-39), and
bf16 data is rounded once at the end, round-to-nearest-even (:33-34).
"""

import numpy as np
import torch


def check_contract(gathered_elems, dst_elems, world_size):
    """The glue's acceptance rule (generic_dense_glue.cpp:576-589)."""
    if world_size < 2 or world_size > 8:
        raise ValueError("world_size must be 2..8")
    if dst_elems <= 0 or gathered_elems != dst_elems * world_size:
        raise ValueError("gathered must hold world_size * elems values")


def rank_sum(gathered, world_size):
    """gathered: torch bf16 or fp32 [world_size * elems] -> [elems] of the same dtype."""
    if gathered.dtype not in (torch.bfloat16, torch.float32) or gathered.ndim != 1:
        raise ValueError("1-D bf16 or fp32 expected")
    elems = gathered.numel() // world_size
    check_contract(gathered.numel(), elems, world_size)
    slices = gathered.float().numpy().reshape(world_size, elems)
    acc = slices[0].astype(np.float32).copy()
    for r in range(1, world_size):
        acc = (acc + slices[r]).astype(np.float32)             # one fp32 addition per rank, in rank order
    out = torch.from_numpy(acc)
    return out.to(torch.bfloat16) if gathered.dtype == torch.bfloat16 else out
