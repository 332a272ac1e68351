"""One rank of the 2-GPU decoder tests: launched by tests/test_gpu_tp.py through torch.distributed.run
(``--peer`` switches the all-reduce to the peer-memory reduction).  Prints ``REPORT <json>``."""

import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch
import torch.distributed as dist


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    import test_gpu_tp

    report = test_gpu_tp.two_rank_step(rank, world, "--peer" in sys.argv)
    dist.barrier()
    sys.stdout.write("\nREPORT " + json.dumps(report) + "\n")   # one write, so the ranks' lines do not interleave
    sys.stdout.flush()
    dist.destroy_process_group()   # the exchange buffers stay mapped until the process exits


if __name__ == "__main__":
    main()
