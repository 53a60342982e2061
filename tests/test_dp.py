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


def test_bounded_wait_gives_up_when_a_rank_never_contributes(tmp_path):
    """Failure detection on the host: the loop behind ctk_comm_wait (poll the work, poll the
    communicator's health, stop at a deadline, abort once) over gloo ranks.  With every rank present it
    returns 0; with rank 1 absent from the collective the others get CTK_ERR_NCCL at the deadline
    instead of waiting for ever."""
    out = str(tmp_path / "wd.npz")
    _launch("watchdog", 2, out)
    r = np.load(out)
    assert int(r["rc_ok"]) == 0 and bool(r["sum_ok"])
    assert int(r["rc_bad"]) == 3, "CTK_ERR_NCCL expected"
    assert int(r["aborts"]) == 1
    assert 0.6 <= float(r["waited"]) <= 2.0, float(r["waited"])
    assert "did not take part" in str(r["msg"])


def test_bounded_wait_reports_errors_at_once():
    """An error of the awaited work or of the communicator ends the wait immediately (no ranks needed)."""
    import time
    import ctorch_b200 as cb
    from ctorch_b200.dp import Watchdog
    wd = Watchdog(cb)
    aborted = []
    t0 = time.perf_counter()
    assert wd.wait(lambda: 0, health=lambda: 6, abort=lambda: aborted.append(1), timeout_ms=60000) == 3
    assert time.perf_counter() - t0 < 1.0 and aborted == [1]
    assert b"asynchronous error (6)" in cb.lib.ctk_last_error()
    assert wd.wait(lambda: -700, timeout_ms=60000) == 3
    assert b"reported an error (-700)" in cb.lib.ctk_last_error()
    assert wd.wait(lambda: 1, health=lambda: 6, timeout_ms=0) == 0    # done wins over everything
    polls = []
    assert wd.wait(lambda: polls.append(1) or (1 if len(polls) > 50 else 0), timeout_ms=60000) == 0


def test_shards_differ_per_rank():
    from ctorch_b200.dp import shard_seed
    assert len({shard_seed(1234, r) for r in range(8)}) == 8


@pytest.mark.gpu
@pytest.mark.parametrize("dp_mode", ["inplace", "arena", "serial", "sharded"])
def test_two_gpus_nccl_allreduce_matches_two_replica_oracle(tmp_path, orc, cb, dp_mode):
    n = ctypes.c_int()
    cb.check(cb.lib.ctk_device_count(ctypes.byref(n)))
    if n.value < 2:
        pytest.skip("needs 2 GPUs")
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import dp_worker as W
    out = str(tmp_path / "gpu.npz")
    _launch("gpu", 2, out, {"NCCL_NVLS_ENABLE": "0", "CTORCH_TEST_DP_MODE": dp_mode})
    r = np.load(out)
    x, lab, p = W.case(W.DIMS, W.BATCH, W.NB, 2)
    ref = orc.mlp_train(W.DIMS, x, lab, p, W.LR, W.STEPS, grad_steps=tuple(range(W.STEPS)))
    assert int(r["status"]) == 0
    assert_close(r["losses"], ref["losses"], 1e-4, 1e-3, "per-rank losses at every step")
    if dp_mode != "sharded":   # (sharded: a rank holds the summed gradient of its own shard only)
        for s in range(W.STEPS):
            assert_matmul_close(r["grads"][s], ref["grads"][s], 1e-4, f"all-reduced gradients at step {s}")
    assert_matmul_close(r["params"], ref["params"], 1e-4, "final weights")
    assert float(r["spread"]) == 0.0, "every rank must end with the same weights, bit for bit"
