"""One rank of the two-process CPU check of the data-parallel rule: shard the
points in rank order, evaluate the shard with the local cotangent scaled by
1/world (a mean), all-reduce the flat [loss, gradients] buffer with SUM, and
compare with the full-batch oracle.  Also checks that the NCCL-id broadcast
helper hands every rank the bytes rank 0 made."""

import sys

import numpy as np
import torch
import torch.distributed as dist

from oracle import contracted
from quabla_b200 import distributed, workloads
from quabla_b200._transforms import CompiledLoss


def main() -> None:
    rank, world = int(sys.argv[1]), int(sys.argv[2])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    unique = distributed.broadcast_unique_id(rank, make_id=lambda: bytes(range(128)))
    assert unique == bytes(range(128))

    w = workloads.make("poisson2d", 64)
    full_args = (w.params, *w.data)
    full = CompiledLoss(w.loss, full_args, (0,), 0, build_plan=False)
    expected_loss, expected_grads = contracted.value_and_grad(full.spec, full.named_inputs(full_args))

    local_data = tuple(distributed.shard(a, rank, world) for a in w.data)
    local_args = (w.params, *local_data)
    local = CompiledLoss(w.loss, local_args, (0,), 0, build_plan=False)
    loss, grads = contracted.value_and_grad(local.spec, local.named_inputs(local_args), cotangent=1.0 / world)
    flat = np.concatenate([[loss / world]] + [g.reshape(-1) for g in grads])
    tensor = torch.from_numpy(flat)
    dist.all_reduce(tensor, op=dist.ReduceOp.SUM)
    reduced = tensor.numpy()
    want = np.concatenate([[expected_loss]] + [g.reshape(-1) for g in expected_grads])
    error = np.max(np.abs(reduced - want)) / np.max(np.abs(want))
    assert error < 1e-12, error
    dist.barrier()
    if rank == 0:
        print("PARITY OK", error)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
