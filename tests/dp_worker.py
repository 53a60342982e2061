"""Worker of the data-parallel tests (one process per rank; started by the tests, not collected).

mode "cpu": gloo only -- each rank computes the oracle's gradient on its own shard, the ranks sum
            them, and rank 0 writes the sum (the host-side logic of the data-parallel step).
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
    import ctorch_b200 as cb
    from ctorch_b200 import frontend as F
    cb.check(cb.lib.ctk_set_device(cp.local_rank))
    F.set_quiet(True)
    comm = dp.make_comm(cb, cp)
    tr = F.MlpTrainer(DIMS, p, LR)
    tr.set_comm(comm)
    losses, grads = [], []
    for s in range(STEPS):
        bi = s % NB
        losses.append(tr.step_host(x[cp.rank, bi], lab[cp.rank, bi]))
        grads.append(tr.grads())
    params = tr.params()
    all_losses = cp.sum_over_ranks(np.eye(cp.world, dtype=np.float32)[cp.rank][:, None] * np.asarray(losses, np.float32)[None, :])
    if cp.rank == 0:
        np.savez(out, losses=all_losses.T, grads=np.stack(grads), params=params, status=cb.ops.matmul_status())
    tr.set_comm(None)
    del tr
    cb.synchronize()
    cb.lib.ctk_comm_destroy(comm)
    cp.close()


if __name__ == "__main__":
    main()
