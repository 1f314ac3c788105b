"""Worker of the multi-GPU parity test: run under torch.distributed.run, one rank per GPU.
Runs tests/parity_cases.py on every rank and writes each rank's report as JSON."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "mixture-of-kittens_b200")):
    sys.path.insert(0, p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from tests.parity_cases import run_parity  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    report = run_parity(rank, world, dev)
    out_dir = os.environ.get("MOKB_TEST_OUT", "/tmp")
    with open(os.path.join(out_dir, f"multirank_rank{rank}.json"), "w") as f:
        json.dump(report, f)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if report["ok"] else 1)


if __name__ == "__main__":
    main()
