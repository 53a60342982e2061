"""Control plane of the data-parallel run: one process per GPU, launched by torchrun.

Gradients travel over the library's own NCCL communicator (ctk_comm_*); this module only carries the
128-byte NCCL id, barriers and small host-side reductions, over torch.distributed with the gloo
backend, and decides which rows a rank owns.
"""
import os

import numpy as np


class ControlPlane:
    def __init__(self, rank=None, world=None, init=True):
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.world = int(os.environ.get("WORLD_SIZE", "1")) if world is None else world
        self.local_rank = int(os.environ.get("LOCAL_RANK", str(self.rank)))
        self.dist = None
        if self.world > 1 and init:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            if not dist.is_initialized():
                dist.init_process_group(backend="gloo", rank=self.rank, world_size=self.world)
            self.dist = dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()

    def broadcast_bytes(self, buf, src=0):
        """buf: a numpy uint8 array, filled on `src`; returns it filled on every rank."""
        if self.dist is None:
            return buf
        import torch
        t = torch.from_numpy(buf)
        self.dist.broadcast(t, src=src)
        return buf

    def max_over_ranks(self, value):
        if self.dist is None:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t[0])

    def sum_over_ranks(self, array):
        """Element-wise sum of a float32 numpy array over ranks (host side; used by tests)."""
        if self.dist is None:
            return array
        import torch
        t = torch.from_numpy(np.ascontiguousarray(array, dtype=np.float32).copy())
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return t.numpy()

    def close(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()
            self.dist = None


def shard_seed(base_seed, rank):
    """Each rank draws its own rows: weak scaling, a different data seed per rank."""
    return base_seed + 1000 * rank


def _init_comm(cb, cp, max_ctas, nvls_ctas):
    import ctypes
    idbuf = np.zeros(128, np.uint8)
    if cp.rank == 0:
        cb.check(cb.lib.ctk_comm_unique_id(idbuf.ctypes.data_as(ctypes.c_void_p)))
    cp.broadcast_bytes(idbuf, 0)
    comm = ctypes.c_void_p()
    cb.check(cb.lib.ctk_comm_init_rank_config(ctypes.byref(comm), idbuf.ctypes.data_as(ctypes.c_void_p), cp.world, cp.rank, int(max_ctas), int(nvls_ctas)))
    return comm


def make_comm(cb, cp, max_ctas=0, nvls_ctas=0, algo=""):
    """Creates the NCCL communicator of this rank (ctk_comm_init_rank_config) from an id made on rank 0.
    max_ctas / nvls_ctas bound the CTAs a collective may take from the MatMul kernels (0: NCCL's choice).
    algo: "" leaves the algorithm to NCCL's tuner; a name (e.g. "NVLS": reduction inside the NVSwitch,
    which the tuner of NCCL 2.27/2.28 does not pick by itself for these sizes on 4 GPUs although it is
    the fastest under a running backward pass) is set as NCCL_ALGO for this communicator and tried
    with one small all-reduce on every rank; if any rank cannot run it, all ranks fall back to NCCL's
    choice.  Returns (communicator, algo in effect)."""
    import ctypes
    if algo:
        saved = os.environ.get("NCCL_ALGO")
        os.environ["NCCL_ALGO"] = algo
        ok = 1.0
        comm = None
        try:
            comm = _init_comm(cb, cp, max_ctas, nvls_ctas)
            probe = cb.zeros((1 << 20,))
            cb.check(cb.lib.ctk_allreduce_sum_f32(comm, probe.p, ctypes.c_int64(probe.size), None))
            cb.synchronize()
        except Exception:
            ok = 0.0
        if -cp.max_over_ranks(-ok) > 0.5:   # the minimum over ranks
            return comm, algo
        if comm is not None:
            try:
                cb.lib.ctk_comm_abort(comm)
                cb.lib.ctk_comm_destroy(comm)
            except Exception:
                pass
        if saved is None:
            os.environ.pop("NCCL_ALGO", None)
        else:
            os.environ["NCCL_ALGO"] = saved
    return _init_comm(cb, cp, max_ctas, nvls_ctas), ""


class Watchdog:
    """The library's bounded wait (ctk_watchdog_wait) over Python callables: query() -> 1 done / 0 pending
    / < 0 error, health() -> 0 while fine, abort() once before an error is reported.  The GPU path uses
    the same loop with a CUDA event and ncclCommGetAsyncError behind it (ctk_comm_wait)."""

    def __init__(self, cb):
        import ctypes
        self.cb = cb
        self.FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)

    def wait(self, query, health=None, abort=None, timeout_ms=1000, poll_us=50):
        q = self.FN(lambda _u: int(query()))
        h = self.FN(lambda _u: int(health())) if health else None
        a = self.FN(lambda _u: int(abort() or 0)) if abort else None
        return self.cb.lib.ctk_watchdog_wait(q, h, a, None, int(timeout_ms), int(poll_us))
