"""Data-parallel replicas: how N GPUs of one node run the inference path.

Positions (batch items) are independent, so the path shards without any exchange step: every rank owns one GPU, holds a
full copy of the weights and runs its own batches -- the way minml's own multi-GPU host code keeps one context and one
graph copy per device.  The only communication is bookkeeping: a barrier around the timed region and a MAX over the ranks'
device times, so that the reported throughput is (positions all ranks processed) / (time of the slowest rank).

The process group is NCCL on GPUs and gloo on CPUs (the tests run this module with two gloo ranks).
"""
import os

import torch
import torch.distributed as dist


class Replicas:
    def __init__(self, backend=None, device_index=None):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        self.device = torch.device("cuda", self.local_rank if device_index is None else device_index) if self.backend == "nccl" else torch.device("cpu")
        self.owns_group = False
        if self.world > 1 and not dist.is_initialized():
            if self.backend == "nccl":
                dist.init_process_group("nccl", device_id=self.device)
            else:
                dist.init_process_group("gloo")
            self.owns_group = True

    # ------------------------------------------------------------------ work assignment (weak scaling)
    def input_seed(self, base_seed):
        """Every rank draws its own synthetic batch: same distribution, different positions."""
        return base_seed + 1 + self.rank

    def global_units(self, units_per_rank):
        return units_per_rank * self.world

    # ------------------------------------------------------------------ synchronisation and timing
    def barrier(self):
        if self.world > 1:
            dist.barrier()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def max_over_ranks(self, values):
        """Element-wise maximum of a list of floats over all ranks (identical result on every rank)."""
        t = torch.tensor(list(values), dtype=torch.float64, device=self.device)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def gather_floats(self, value):
        """This rank's number from every rank, in rank order (identical list on every rank): used to name the slowest rank."""
        t = torch.zeros(self.world, dtype=torch.float64, device=self.device)
        t[self.rank] = float(value)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return [float(v) for v in t]

    def throughput(self, units_per_rank, local_seconds):
        """Whole-job units per second: all ranks' units over the slowest rank's time."""
        slowest = self.max_over_ranks([local_seconds])[0]
        return self.global_units(units_per_rank) / slowest, slowest

    def close(self):
        if self.owns_group and dist.is_initialized():
            dist.destroy_process_group()
            self.owns_group = False
