"""Child of tests/test_utils_misc_on_cpu.py: one rank of a communicator found by name (no torchrun, no env rendezvous)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, name, reg = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    from verl_b200.utils.rendezvous import create_communicator_by_name

    pg = create_communicator_by_name(rank, world, name, registry_dir=reg, interval_s=0.05)
    t = torch.tensor([float(rank + 1)])
    pg.allreduce([t]).wait()
    assert float(t) == world * (world + 1) / 2, float(t)
    print(f"RENDEZVOUS_OK {rank}")


if __name__ == "__main__":
    main()
