"""Replica plumbing for the multi-GPU runs: one process per GPU, no data-path collective.

The reference walks its GPUs one after another in one process
(src/cuda/cuda_peak.cpp:109-208); here every GPU runs the same benchmark at the
same time and the box figure is "work of all replicas / slowest replica's time".
torch.distributed only carries the start barrier and that max; the backend is
NCCL on GPUs and gloo in the CPU tests of this module.
"""
from __future__ import annotations

import os


class Replicas:
    """rank / world of this process and the two collectives the benchmark needs."""

    def __init__(self, backend: str | None = None, device=None):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.local_world = int(os.environ.get("LOCAL_WORLD_SIZE", str(self.world)))
        self.device = device
        self._dist = None
        self._host_group = None
        if self.world > 1:
            import torch.distributed as dist
            if not dist.is_initialized():
                kw = {}
                if backend in (None, "nccl") and device is not None:
                    kw["device_id"] = device
                dist.init_process_group(backend or "nccl", **kw)
            self._dist = dist
            # A second, CPU-only group for waits that must not occupy the GPUs: an NCCL barrier is a kernel
            # that spins on every waiting rank's GPU until the last rank arrives.
            self._host_group = dist.new_group(backend="gloo") if dist.get_backend() != "gloo" else None

    @property
    def active(self) -> bool:
        return self._dist is not None

    def barrier(self) -> None:
        if self._dist is not None:
            self._dist.barrier()

    def host_barrier(self) -> None:
        """Wait for all ranks on the host only (gloo): the GPUs of the waiting ranks stay idle, so that one rank
        can meanwhile run something on all of them."""
        if self._dist is not None:
            self._dist.barrier(group=self._host_group)

    def max_over_ranks(self, value: float) -> float:
        """The slowest replica's figure (a time): what every box-level rate divides by."""
        if self._dist is None:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64, device=self.device if self.device is not None else "cpu")
        self._dist.all_reduce(t, op=self._dist.ReduceOp.MAX)
        return float(t.item())

    def whole_job_rate(self, units_per_replica: float, local_ms: float) -> tuple[float, float]:
        """(units per second over all replicas, max-over-ranks milliseconds)."""
        ms = self.max_over_ranks(local_ms)
        return self.world * units_per_replica / (ms * 1e-3), ms

    def close(self) -> None:
        if self._dist is not None:
            self._dist.barrier()
            self._dist.destroy_process_group()
            self._dist = None
