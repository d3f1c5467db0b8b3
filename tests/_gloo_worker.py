"""Worker of tests/test_shard_gloo.py: one rank of a world_size-N CPU (gloo) run
of the one-process-per-GPU sharding logic.  The per-rank attention is computed by
the oracle here (test-only stand-in for the device call); what is under test is
the partition, the slicing, the dropout origin and the reduction of timings."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from nnlib_jl_b200.shard import rank_rects  # noqa: E402
from oracle import attention_oracle as O  # noqa: E402
from oracle import philox_oracle as P  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    E, H, Lq, Lkv, B, p, seed = 12, 3, 5, 6, 3, 0.25, 11
    rng = np.random.default_rng(0)                       # every rank builds the same global problem
    q = rng.standard_normal((E, Lq, B)).astype(np.float32)
    k = rng.standard_normal((E, Lkv, B)).astype(np.float32)
    v = rng.standard_normal((E, Lkv, B)).astype(np.float32)
    d = E // H
    x = np.zeros((E, Lq, B), np.float32)
    for r in rank_rects(B, H, rank, world):
        bs = slice(r.b0, r.b0 + r.nb)
        fs = slice(r.h0 * d, (r.h0 + r.nh) * d)
        keep = P.keep_mask((Lkv, Lq, r.nh, r.nb), p, seed, 0, h0=r.h0, b0=r.b0, H_total=H)
        y, _ = O.dot_product_attention(q[fs, :, bs], k[fs, :, bs], v[fs, :, bs], nheads=r.nh,
                                       fdrop=lambda a: a * keep / np.float32(1 - p))
        x[fs, :, bs] = y
    t = torch.from_numpy(x)
    dist.all_reduce(t)                                   # shards are disjoint: the sum assembles x
    ms = torch.tensor([10.0 + rank], dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)            # bench.py's max-over-ranks timing
    if rank == 0:
        keep = P.keep_mask((Lkv, Lq, H, B), p, seed, 0)
        want, _ = O.dot_product_attention(q, k, v, nheads=H, fdrop=lambda a: a * keep / np.float32(1 - p))
        np.testing.assert_allclose(t.numpy(), want, rtol=1e-5, atol=1e-6)
        assert ms.item() == 10.0 + world - 1
        print("GLOO_SHARD_OK")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
