"""Data-parallel plumbing of the token loop: sequences are independent (no cross-sequence operation
exists anywhere on the path), so ranks own disjoint slices of the batch and exchange nothing on the
data path.  torch.distributed only carries bookkeeping (max-over-ranks timings, gathered token ids)."""
from typing import List, Tuple

import torch
import torch.distributed as dist


def shard_range(global_batch: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [start, end) slice of the global batch owned by `rank` (sizes differ by at most one)."""
    base, extra = divmod(global_batch, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def max_over_ranks(values: List[float], device=None) -> List[float]:
    """Element-wise max of per-rank timings (the time of a data-parallel job is its slowest rank)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(values)
    t = torch.tensor(values, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def gather_token_ids(local_ids: torch.Tensor, global_batch: int) -> torch.Tensor:
    """Concatenate the per-rank [b_local, T] id tensors in rank order into the [global_batch, T] result."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local_ids
    world = dist.get_world_size()
    sizes = [shard_range(global_batch, world, r) for r in range(world)]
    width = max(e - s for s, e in sizes)
    padded = torch.zeros(width, local_ids.shape[1], dtype=local_ids.dtype, device=local_ids.device)
    padded[: local_ids.shape[0]] = local_ids
    out = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(out, padded)
    return torch.cat([o[: e - s] for o, (s, e) in zip(out, sizes)], dim=0)


class RankLost(RuntimeError):
    """A rank of the job did not reach a step fence in time (it raised, exited or never joined)."""


class StepFence:
    """Host-side membership check between token steps of a multi-rank job.

    Every rank calls `arrive(step)` between steps, with none of its kernels or collectives in flight; the call
    returns once all `world` ranks have arrived at that step and raises RankLost after `timeout_s` otherwise, so the
    survivors learn of a lost rank on the host BEFORE they launch a collective that would wait for it.  The state
    lives in a torch.distributed store (TCPStore / FileStore): one counter per step, nothing on the GPU."""

    def __init__(self, store, world: int, timeout_s: float = 5.0, poll_s: float = 0.01, prefix: str = "stu_fence"):
        self.store, self.world, self.timeout_s, self.poll_s, self.prefix = store, world, timeout_s, poll_s, prefix

    def arrive(self, step: int) -> None:
        import time
        key = f"{self.prefix}/{step}"
        self.store.add(key, 1)
        deadline = time.monotonic() + self.timeout_s
        while True:
            n = self.store.add(key, 0)
            if n >= self.world:
                return
            if time.monotonic() > deadline:
                raise RankLost(f"step {step}: {n} of {self.world} ranks arrived within {self.timeout_s} s")
            time.sleep(self.poll_s)
