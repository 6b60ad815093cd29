"""Worker of test_gpu_comm.py::test_one_process_per_gpu_over_torch_distributed (run under
torch.distributed.run, one process per GPU)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ampstein_b200.comm import P2PComm          # noqa: E402
from oracle import exl3_oracle                  # noqa: E402  (checker)


def partial(rank, n, call):
    i = np.arange(n, dtype=np.float64)
    return (np.sin(0.37 * i + 1.7 * rank + 0.11 * call) * (1.0 + 0.25 * rank)).astype(np.float16)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")
    comm = P2PComm.from_process_group(40960)
    for call, n in enumerate([5120, 40960, 8, 8 * 777, 5120, 40960]):
        x = torch.from_numpy(partial(rank, n, call)).cuda()
        y = comm.allreduce(x)
        torch.cuda.synchronize()
        want = exl3_oracle.allreduce_fp16([partial(r, n, call) for r in range(world)]).view(np.uint16)
        assert np.array_equal(y.cpu().numpy().view(np.uint16), want), (rank, call)
    assert comm.status() == 0
    dist.barrier()
    comm.close()
    print("comm_worker ok rank %d" % rank, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
