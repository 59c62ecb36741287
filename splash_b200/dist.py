"""Rendezvous, barrier and max-over-ranks for multi-GPU runs (one process per GPU). Tensor-parallel ranks exchange
inside the kernels, through each other's memory (splash_b200.tp); here the ranks only pass each other the handles of
that memory, agree on when the timed region starts and on its longest duration. Independent replicas exchange
nothing. torch.distributed is plumbing (nccl on GPUs, gloo in CPU tests)."""
import os


class Group:
    def __init__(self, backend=None):
        self.rank = int(os.environ.get("RANK", 0))
        self.world = int(os.environ.get("WORLD_SIZE", 1))
        self.local = int(os.environ.get("LOCAL_RANK", 0))
        self.dist = None
        self.device = "cpu"
        if self.world > 1:
            import torch
            import torch.distributed as dist
            backend = backend or "nccl"
            if backend == "nccl":
                torch.cuda.set_device(self.local)
                self.device = "cuda"
                dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            else:
                dist.init_process_group(backend)
            self.dist = dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
            if self.device == "cuda":
                import torch
                torch.cuda.synchronize()

    def reduce_max(self, value):
        """The largest `value` over the ranks (a duration: the job takes as long as its slowest rank)."""
        if self.dist is None:
            return float(value)
        import torch
        v = torch.tensor([float(value)], device=self.device, dtype=torch.float64)
        self.dist.all_reduce(v, op=self.dist.ReduceOp.MAX)
        return float(v.item())

    def reduce_sum(self, value):
        if self.dist is None:
            return float(value)
        import torch
        v = torch.tensor([float(value)], device=self.device, dtype=torch.float64)
        self.dist.all_reduce(v, op=self.dist.ReduceOp.SUM)
        return float(v.item())

    def all_gather_bytes(self, mine):
        """Every rank's `mine` (bytes), in rank order: the host transport of splash_b200.tp.connect."""
        if self.dist is None:
            return [bytes(mine)]
        out = [None] * self.world
        self.dist.all_gather_object(out, bytes(mine))
        return out

    def aggregate_rate(self, units_per_rank, seconds):
        """Whole-job throughput: all ranks' units over the slowest rank's time."""
        return self.world * units_per_rank / self.reduce_max(seconds)

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()
            self.dist = None
