"""Data-parallel path: N ranks, each on its own shard, gradients summed element-wise, identical update
everywhere.  The oracle for N ranks is N reference replicas with summed gradients
(orc_mlp_train(replicas=N)), not one big-batch run: the reference's bias gradient is row 0 of the
upstream gradient, which is not additive across rows.

CPU: world_size 2 over gloo (host-side logic).  GPU: 2 ranks over NCCL, when the box has 2 GPUs."""
import ctypes
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from conftest import assert_close, assert_matmul_close

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _launch(mode, world, out, extra_env=None):
    procs = []
    port = str(_free_port())
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1", MASTER_PORT=port)
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "dp_worker.py"), mode, out], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        logs.append(o)
    assert all(p.returncode == 0 for p in procs), "\n".join(logs)


def test_two_gloo_ranks_sum_their_replica_gradients(tmp_path, orc):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import dp_worker as W
    out = str(tmp_path / "cpu.npz")
    _launch("cpu", 2, out)
    r = np.load(out)
    assert int(r["world"]) == 2 and bool(r["token_ok"]) and float(r["slowest"]) == 2.0
    x, lab, p = W.case(W.DIMS, W.BATCH, W.NB, 2)
    ref = orc.mlp_train(W.DIMS, x, lab, p, W.LR, 1, grad_steps=(0,))
    assert_close(r["gsum"], ref["grads"][0], 1e-6, 1e-7, "sum over ranks of per-shard gradients == 2-replica oracle")
    # and it is NOT the big-batch gradient for the biases (row 0 of each shard, summed)
    xb = np.concatenate([x[0], x[1]], axis=1)[None]
    lb = np.concatenate([lab[0], lab[1]], axis=1)[None]
    big = orc.mlp_train(W.DIMS, xb, lb, p, W.LR, 1, grad_steps=(0,))
    assert np.abs(big["grads"][0] - ref["grads"][0]).max() > 1e-3


def test_shards_differ_per_rank():
    from ctorch_b200.dp import shard_seed
    assert len({shard_seed(1234, r) for r in range(8)}) == 8


@pytest.mark.gpu
def test_two_gpus_nccl_allreduce_matches_two_replica_oracle(tmp_path, orc, cb):
    n = ctypes.c_int()
    cb.check(cb.lib.ctk_device_count(ctypes.byref(n)))
    if n.value < 2:
        pytest.skip("needs 2 GPUs")
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import dp_worker as W
    out = str(tmp_path / "gpu.npz")
    _launch("gpu", 2, out, {"NCCL_NVLS_ENABLE": "0"})
    r = np.load(out)
    x, lab, p = W.case(W.DIMS, W.BATCH, W.NB, 2)
    ref = orc.mlp_train(W.DIMS, x, lab, p, W.LR, W.STEPS, grad_steps=tuple(range(W.STEPS)))
    assert int(r["status"]) == 0
    assert_close(r["losses"], ref["losses"], 1e-4, 1e-3, "per-rank losses at every step")
    for s in range(W.STEPS):
        assert_matmul_close(r["grads"][s], ref["grads"][s], 1e-4, f"all-reduced gradients at step {s}")
    assert_matmul_close(r["params"], ref["params"], 1e-4, "final weights")
