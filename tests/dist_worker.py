"""One rank of the world_size-2 CPU test of bench.py's cross-rank logic (gloo backend).
Usage: python dist_worker.py <out_file>; RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT from the env."""
import json
import os
import sys

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # each rank pretends to have measured its own replica: rank r is r*10% slower
    dev_ms, wall_s = 500.0 * (1 + 0.1 * rank), 0.6 * (1 + 0.1 * rank)
    dist.barrier()
    dev_max, wall_max = bench.reduce_max_over_ranks([dev_ms, wall_s], dist, "cpu")
    value, e2e = bench.whole_job_rates(world, 3, 200, dev_max, wall_max)
    with open(sys.argv[1] + ".%d" % rank, "w") as f:
        json.dump({"rank": rank, "dev_max": dev_max, "wall_max": wall_max, "value": value, "e2e": e2e}, f)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
