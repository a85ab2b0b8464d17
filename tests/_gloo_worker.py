"""One rank of the two-process sharding test (started by test_sharding_gloo.py).

Checks, over a gloo process group on 127.0.0.1 and without a GPU:
  * Stream.batch(B).partition(world, rank) - the sharding the multi-GPU runs
    use - hands every batch to exactly one rank, batch j to rank j % world;
  * bench.py's sample_list picks the same samples for a rank;
  * the max-over-ranks reduction bench.py applies to its step time.
Writes "ok" to the file given on the command line when every check passed.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests"))
sys.path.insert(0, ROOT)

from conftest import load_package  # noqa: E402


def main():
    out_path = sys.argv[1]
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dx = load_package()
    import bench

    n, batch = 37, 4   # ragged: the last batch holds one sample
    samples = [{"idx": np.array(i, dtype=np.int64)} for i in range(n)]
    stream = dx.buffer_from_vector(samples).to_stream().batch(batch).partition(world, rank)
    mine = [b["idx"].tolist() for b in stream]

    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    n_batches = (n + batch - 1) // batch
    expect = [list(range(j * batch, min((j + 1) * batch, n))) for j in range(n_batches)]
    for r in range(world):
        assert gathered[r] == [expect[j] for j in range(n_batches) if j % world == r], (r, gathered[r])
    flat = sorted(i for per_rank in gathered for b in per_rank for i in b)
    assert flat == list(range(n))

    # bench.py shards the same way: whole batches by index, batch j on rank j % world
    pool = list(range(1000))
    full = n // batch
    per_rank = full // world
    got = [d["image"] for d in bench.sample_list(pool, None, 0, per_rank, batch, world, rank)]
    want = [i for j in range(per_rank * world) if j % world == rank for i in expect[j]]
    assert got == want, (got, want)

    # the step time reported is the slowest rank's
    t = torch.tensor([10.0 + rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert float(t.item()) == 10.0 + world - 1

    dist.barrier()
    dist.destroy_process_group()
    with open(out_path, "w") as f:
        f.write("ok")


if __name__ == "__main__":
    main()
