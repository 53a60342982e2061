"""Worker of the data-parallel tests (one process per rank; started by the tests, not collected).

mode "cpu": gloo only -- each rank computes the oracle's gradient on its own shard, the ranks sum
            them, and rank 0 writes the sum (the host-side logic of the data-parallel step).
mode "watchdog": gloo only -- failure detection without a GPU.  Round 1: every rank contributes to an
            asynchronous all-reduce and the bounded wait returns 0.  Round 2: rank 1 never contributes
            (the failure is made on the host: it simply does not call); the wait on the other ranks has
            to give up at its deadline, call the abort callback once and return CTK_ERR_NCCL.
mode "gpu": each rank trains the MLP on its shard on its own GPU with the NCCL all-reduce switched
            on; rank 0 writes losses, gradients and final weights.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def case(dims, batch, n_batches, world, seed=77):
    import oracle
    from ctorch_b200.dp import shard_seed
    xs, labs = [], []
    for r in range(world):
        rng = np.random.default_rng(shard_seed(seed, r))
        xs.append(rng.integers(0, 256, (n_batches, batch, dims[0])).astype(np.float32) / np.float32(255.0))
        labs.append(rng.integers(0, dims[-1], (n_batches, batch)).astype(np.float32))
    rw = np.random.default_rng(seed + 1)
    Ws, bs = [], []
    for i, j in zip(dims[:-1], dims[1:]):
        lim = np.sqrt(6.0 / i)
        Ws.append(rw.uniform(-lim, lim, (i, j)).astype(np.float32))
        bs.append(np.zeros(j, np.float32))
    return np.stack(xs), np.stack(labs), oracle.pack_params(Ws, bs)


DIMS, BATCH, NB, STEPS, LR = [96, 64, 40, 10], 32, 3, 4, 0.001


def main():
    mode, out = sys.argv[1], sys.argv[2]
    from ctorch_b200 import dp
    cp = dp.ControlPlane()
    x, lab, p = case(DIMS, BATCH, NB, cp.world)
    if mode == "cpu":
        import oracle
        orc = oracle.Oracle()
        mine = orc.mlp_train(DIMS, x[cp.rank:cp.rank + 1], lab[cp.rank:cp.rank + 1], p, LR, 1, grad_steps=(0,))
        gsum = cp.sum_over_ranks(mine["grads"][0])
        slowest = cp.max_over_ranks(float(cp.rank + 1))
        token = np.zeros(128, np.uint8)
        if cp.rank == 0:
            token[:] = np.arange(128, dtype=np.uint8)
        cp.broadcast_bytes(token, 0)
        ok = np.array_equal(token, np.arange(128, dtype=np.uint8))
        if cp.rank == 0:
            np.savez(out, gsum=gsum, slowest=slowest, token_ok=ok, world=cp.world)
        cp.close()
        return
    if mode == "watchdog":
        import time
        import torch
        import ctorch_b200 as cb
        wd = dp.Watchdog(cb)
        t = torch.ones(4)
        work = cp.dist.all_reduce(t, async_op=True)
        rc_ok = wd.wait(lambda: 1 if work.is_completed() else 0, timeout_ms=20000)
        sum_ok = bool((t == cp.world).all())
        cp.dist.barrier()
        rc_bad, aborts, waited = 0, [0], 0.0
        if cp.rank != 1:
            t2 = torch.ones(4)
            work2 = cp.dist.all_reduce(t2, async_op=True)   # rank 1 never joins this one
            t0 = time.perf_counter()
            rc_bad = wd.wait(lambda: 1 if work2.is_completed() else 0, health=lambda: 0,
                             abort=lambda: aborts.__setitem__(0, aborts[0] + 1), timeout_ms=700)
            waited = time.perf_counter() - t0
            msg = cb.lib.ctk_last_error().decode()
            if cp.rank == 0:
                np.savez(out, rc_ok=rc_ok, sum_ok=sum_ok, rc_bad=rc_bad, aborts=aborts[0], waited=waited, msg=msg)
        else:
            time.sleep(2.5)   # alive but absent while the others wait
        sys.stdout.flush()
        os._exit(0)           # the unmatched collective can never be completed: no orderly shutdown of gloo
    import ctorch_b200 as cb
    from ctorch_b200 import frontend as F
    cb.check(cb.lib.ctk_set_device(cp.local_rank))
    F.set_quiet(True)
    comm, _ = dp.make_comm(cb, cp)
    tr = F.MlpTrainer(DIMS, p, LR)
    tr.set_dp_mode(os.environ.get("CTORCH_TEST_DP_MODE", "inplace"))
    tr.set_comm(comm)
    losses, grads = [], []
    for s in range(STEPS):
        bi = s % NB
        losses.append(tr.step_host(x[cp.rank, bi], lab[cp.rank, bi]))
        grads.append(tr.grads())
    params = tr.params()
    all_losses = cp.sum_over_ranks(np.eye(cp.world, dtype=np.float32)[cp.rank][:, None] * np.asarray(losses, np.float32)[None, :])
    # largest difference between any rank's weights and rank 0's
    mine = params.copy()
    ref0 = cp.broadcast_bytes(params.view(np.uint8).copy(), 0).view(np.float32)
    spread = cp.max_over_ranks(float(np.abs(mine - ref0).max()))
    if cp.rank == 0:
        np.savez(out, losses=all_losses.T, grads=np.stack(grads), params=params, status=cb.ops.matmul_status(), spread=spread)
    tr.set_comm(None)
    del tr
    cb.synchronize()
    cb.lib.ctk_comm_destroy(comm)
    cp.close()


if __name__ == "__main__":
    main()
