"""gloo ranks run the bootstrap exchange of the peer runtime with stand-in handles (no GPU): every rank must
reach the same verdict on the gathered records.

    torchrun --nproc-per-node 2 tests/multiproc/peer_bootstrap_check.py [--bad-size-rank R | --bad-handle-rank R]
"""

import argparse
import json
import os
import sys
from datetime import timedelta
from pathlib import Path

import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from moeflow_b200.parallel.peer import check_exchange  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--bad-size-rank", type=int, default=-1)
    ap.add_argument("--bad-handle-rank", type=int, default=-1)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=60))
    nbytes = 4096
    mine = nbytes * 2 if rank == args.bad_size_rank else nbytes
    handle = b"\x01" * (10 if rank == args.bad_handle_rank else 64)
    gathered = [None] * world
    dist.all_gather_object(gathered, (rank, mine, handle))
    error = None
    try:
        check_exchange(gathered, world, mine)
    except RuntimeError as exc:
        error = str(exc)
    verdicts = [None] * world
    dist.all_gather_object(verdicts, error is not None)
    dist.barrier()
    if rank == 0:
        print(json.dumps({"world": world, "raised": verdicts, "error": error}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
