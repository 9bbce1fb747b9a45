"""Row-sharded multi-GPU plumbing: one process per GPU, torch.distributed for rendezvous and collectives.

The path shards by rows (the reference's VectorSplit::ROWS contract, src/runtime/local/vectorized/Tasks.h:85-110):
rank g owns the contiguous row block [g*n/G, (g+1)*n/G).  ROWS/COLS outputs stay sharded; ADD/MIN/MAX partials
(VectorCombine, src/runtime/local/vectorized/Tasks.cpp:51-82) are combined with one all-reduce per pipeline."""
from __future__ import annotations

import os
from typing import Optional

import numpy as np

COMBINE_ROWS, COMBINE_COLS, COMBINE_ADD, COMBINE_MIN, COMBINE_MAX = 1, 2, 3, 4, 5


def row_block(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous row block of `rank`; the first n_rows % world ranks get one extra row."""
    base, extra = divmod(n_rows, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


class Comm:
    """Collectives over the row shards.  world == 1 needs no torch at all."""

    def __init__(self, rank: int = 0, world: int = 1, backend: Optional[str] = None):
        self.rank, self.world, self.backend = rank, world, backend
        self._dist = None
        if world > 1:
            import torch.distributed as dist
            if not dist.is_initialized():
                raise RuntimeError("torch.distributed must be initialised before creating a Comm with world > 1")
            self._dist = dist

    @staticmethod
    def from_env(device_backend: str = "nccl") -> "Comm":
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        if world > 1:
            import torch.distributed as dist
            if not dist.is_initialized():
                dist.init_process_group(backend=device_backend, rank=rank, world_size=world)
        return Comm(rank, world, device_backend if world > 1 else None)

    def _op(self, combine: int):
        d = self._dist
        return {COMBINE_ADD: d.ReduceOp.SUM, COMBINE_MIN: d.ReduceOp.MIN, COMBINE_MAX: d.ReduceOp.MAX}[combine]

    def allreduce_tensor(self, t, combine: int = COMBINE_ADD):
        """In-place all-reduce of a torch tensor (CUDA tensor under nccl, CPU tensor under gloo)."""
        if self.world > 1:
            self._dist.all_reduce(t, op=self._op(combine))
        return t

    def allreduce_numpy(self, a: np.ndarray, combine: int = COMBINE_ADD) -> np.ndarray:
        if self.world == 1:
            return a
        import torch
        t = torch.from_numpy(np.ascontiguousarray(a))
        if self.backend == "nccl":
            t = t.cuda()
        self._dist.all_reduce(t, op=self._op(combine))
        return t.cpu().numpy()

    def allgather_numpy(self, a: np.ndarray) -> np.ndarray:
        """Concatenates equally shaped row shards in rank order."""
        if self.world == 1:
            return a
        import torch
        t = torch.from_numpy(np.ascontiguousarray(a))
        if self.backend == "nccl":
            t = t.cuda()
        out = [torch.empty_like(t) for _ in range(self.world)]
        self._dist.all_gather(out, t)
        return torch.cat(out, dim=0).cpu().numpy()

    def allgather_ragged(self, a: np.ndarray) -> np.ndarray:
        """Concatenates row shards of possibly different heights in rank order (host side, for results)."""
        if self.world == 1:
            return a
        gathered = [None] * self.world
        self._dist.all_gather_object(gathered, np.ascontiguousarray(a))
        return np.concatenate(gathered, axis=0)

    # ---- device-resident collectives through the runtime's NCCL communicator ----
    def init_device(self, ctx) -> None:
        """Gives the runtime context an NCCL communicator; the 128-byte id travels over torch.distributed."""
        import ctypes as C

        import torch

        from .lib import check, lib
        if self.world == 1:
            return
        ident = torch.zeros(128, dtype=torch.uint8)
        if self.rank == 0:
            buf = (C.c_ubyte * 128)()
            check(lib.db2_comm_unique_id(buf))
            ident = torch.tensor(list(buf), dtype=torch.uint8)
        if self.backend == "nccl":
            ident = ident.cuda()
        self._dist.broadcast(ident, src=0)
        raw = bytes(ident.cpu().tolist())
        check(lib.db2_comm_init(ctx.handle, self.rank, self.world, raw))
        self._device_ctx = ctx

    def device_collectives(self, ctx) -> bool:
        return ctx is not None and getattr(self, "_device_ctx", None) is ctx

    def allreduce_device(self, ctx, m, combine: int = COMBINE_ADD) -> None:
        from .lib import check, lib
        check(lib.db2_allreduce(ctx.handle, m.handle, int(combine)))

    def allgather_rows(self, ctx, m, total_rows: int, k=None):
        """Concatenates the row shards of `row_block(total_rows, rank, world)` in rank order; the shards may differ in
        height by one row.  A shard of any other height is refused before anything is exchanged."""
        lo, hi = row_block(total_rows, self.rank, self.world)
        if m.rows != hi - lo:
            raise ValueError(f"rank {self.rank} of {self.world} holds {m.rows} rows, its block of {total_rows} rows "
                             f"has {hi - lo}")
        if self.device_collectives(ctx):
            import ctypes as C

            from . import kernels as K
            from .lib import check, lib
            h = C.c_void_p()
            check(lib.db2_allgatherv_rows(ctx.handle, m.handle, int(total_rows), C.byref(h)))
            return K.DenseMatrix(ctx, h)
        return k.DenseMatrix.from_numpy(ctx, self.allgather_ragged(m.to_numpy()))

    def barrier(self):
        if self.world > 1:
            self._dist.barrier()

    def max_float(self, x: float) -> float:
        if self.world == 1:
            return x
        return float(self.allreduce_numpy(np.array([x], dtype=np.float64), COMBINE_MAX)[0])
