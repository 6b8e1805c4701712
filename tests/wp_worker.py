"""Worker of the multi-GPU window-parallel parity test (one process per GPU, started by torch.distributed.run).

Every rank builds the same small model, runs it (a) on the whole image alone and (b) window-parallel on its own block
with the peer-memory halo gather, and compares outputs and all-reduced gradients
(:func:`aeris_gb_b200.parallel.parity.wp_parity`). Exit code 0 = parity."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from aeris_gb_b200.parallel.parity import wp_parity  # noqa: E402


def main():
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    sp = int(sys.argv[1]) if len(sys.argv) > 1 else 1
    res = wp_parity(dev, sp, verbose=True)
    dist.destroy_process_group()
    sys.exit(0 if res["max_rel_err"] < 3e-2 else 1)


if __name__ == "__main__":
    main()
