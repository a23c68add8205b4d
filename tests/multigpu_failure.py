"""Failure detection on 2 GPUs without faulting one: rank 1 simply does not launch its half
of a flag barrier, so rank 0's bounded wait runs out, its kernel returns, and the host reads
the timeout from the status word.  Afterwards both ranks synchronise on the host, catch up on
the epoch and the same barrier works again.  NVLS stays off (a rank that left while bound
to a multicast object has upset its peers' GPUs on some fabrics); the barrier kernels use
plain peer stores.

    NCCL_NVLS_ENABLE=0 python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 \
        --master-addr 127.0.0.1 --master-port 29513 tests/multigpu_failure.py
"""
from __future__ import annotations

import os
import sys

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
os.environ["MB200_NVLS"] = "0"

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from monarch_b200.ops import kernels as K  # noqa: E402
from monarch_b200.parallel.symm import FlagArray  # noqa: E402


def main() -> int:
    rank = int(os.environ["RANK"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    flags = FlagArray(4, dev)
    flags.barrier(0)                       # both ranks: works
    torch.cuda.synchronize()
    K.check_status(dev)
    dist.barrier()
    # rank 1 stays out of the next barrier
    timed_out = False
    if rank == 0:
        flags.barrier(0)
        torch.cuda.synchronize()           # returns after the bounded wait (about 1.5 s)
        try:
            K.check_status(dev)
        except K.KernelError as e:
            timed_out = "flag timed out" in str(e)
        assert timed_out, "the withheld barrier did not report a timeout"
    else:
        flags._barrier_epoch += 1          # host-side catch-up: the epoch rank 0 has used
    dist.barrier()                         # the ranks learn of each other on the host
    flags.barrier(0)                       # and the device barrier works again
    torch.cuda.synchronize()
    K.check_status(dev)
    dist.barrier()
    if rank == 0:
        print("FAILURE PATH OK")
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
