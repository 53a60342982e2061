#!/usr/bin/env python
"""Benchmark of the B200 CUDA backend for CTorch.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (the headline): the data-parallel MLP training step -- 784-4096-4096-4096-10,
fp32, ReLU, Softmax+CrossEntropy (summed), SGD lr 0.01, 8192 synthetic rows per GPU (pixels k/255,
labels 0..9), Kaiming-uniform weights from a fixed seed, one process per GPU, gradients all-reduced
with NCCL while backward runs.  Prints ONE JSON line (rank 0).

  value   samples/s of the whole job with the step's inputs already resident on the device
  e2e     the same step through the public call that takes HOST buffers: the host-to-device copy of
          the batch (from page-locked memory) and the device-to-host read of the loss are inside
          the timed region
  roofline  the dominant kernel (the tcgen05 MatMul): algorithmic flops (2*M*N*K per product) over
          its launch durations, timed with CUDA events on the launching stream during the timed steps;
          `peak` is the nominal dense TF32 rate / 3 (three TF32 products per fp32 product), and
          `ceilings` lists the measured alternatives (a TF32 GEMM of the vendor library timed in this
          run as a comparator, the driver-measured bf16 figures) with the fraction against each
  cpu_baseline  the reference's own CPU path (single-threaded by construction) on a bounded sample
          of the same workload, N=1 only
  parity_check  (N=1) after timing: logits of sampled rows of the full-size step against the oracle
  dp_check  (N>1) before timing: one reduced-width step against the N-replica oracle; after timing:
          the largest difference between any two ranks' weights (must be 0)
  extras  (N=1) the single-op metrics of the other benchmark configurations, each with achieved rate,
          roofline fraction and the reference's CPU rate on a bounded sample

`--impl reference` times that CPU path alone (rank 0; other ranks exit).
Other workloads (single GPU): elementwise, rowwise, matmul -- the single-op sweeps of the other
benchmark configs, one JSON line each with achieved GB/s or TFLOP/s; mlp_small -- the 784-128-10,
batch-64, 100-step configuration the reference itself can run, timed next to the reference's CPU
path; mnist -- the reference application (IDX files, 784-128-64-10, batch 128, 5 epochs, accuracy)
on a synthetic data set in the same file format.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DIMS = [784, 4096, 4096, 4096, 10]
BATCH = 8192
LR = 0.01
WORKLOAD = "dp-mlp-784-4096-4096-4096-10_batch8192-per-gpu_fp32_sgd"
CPU_SAMPLE_BATCH = 4  # rows per reference step: the reference's cost is linear in rows (~0.2 GFLOP/s)
DEFAULT_DP_MODE, DEFAULT_MAX_CTAS = "arena", 0
DEFAULT_CORRECTION = "bf16"
DEFAULT_NCCL_ALGO = "auto"
NOMINAL_TF32 = 1125.0  # TFLOP/s, dense, the part's data sheet
NOMINAL_HBM = 7700.0   # GB/s
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant shape from one ncu capture
# (not re-measured by a benchmark run; the summary and its command are the named file)
QUOTED_TRAFFIC = dict(bytes=1.2244e9 + 0.3656e9, launch="forward 8192x4096x4096 + bias + ReLU + split, correction terms on the bf16 path (algorithmic: 402 MB of operands and their small terms read, 268 MB of result + its small terms written)",
                      **{"from": "profiles/tcgen05_matmul_pair_tf32_2xbf16_8192x4096x4096.md"})


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


def make_params(seed=42):
    rng = np.random.default_rng(seed)
    parts = []
    for i, j in zip(DIMS[:-1], DIMS[1:]):
        lim = np.sqrt(6.0 / i)
        parts.append(rng.uniform(-lim, lim, (i, j)).astype(np.float32).ravel())
        parts.append(np.zeros(j, np.float32))
    return np.concatenate(parts)


def make_batch(rank, rows=BATCH, seed=1234):
    from ctorch_b200.dp import shard_seed
    rng = np.random.default_rng(shard_seed(seed, rank))
    x = rng.integers(0, 256, (rows, DIMS[0])).astype(np.float32) / np.float32(255.0)
    labels = rng.integers(0, DIMS[-1], rows).astype(np.float32)
    return x, labels


def measure_library_tf32(device_index):
    """A TF32 GEMM of the vendor library (torch.matmul with TF32 allowed, 8192^3) timed with CUDA events:
    best of 10 (burst) and back to back for ~1.5 s (sustained).  A comparator for the roofline only --
    nothing in the product path uses it.  Returns None where torch or its CUDA build is unavailable."""
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        dev = torch.device("cuda", device_index)
        torch.backends.cuda.matmul.allow_tf32 = True
        n = 8192
        a = torch.randn(n, n, device=dev)
        b = torch.randn(n, n, device=dev)
        c = torch.empty(n, n, device=dev)
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize(dev)
        fl = 2.0 * n ** 3
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b, out=c)
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        reps = max(10, int(1500.0 / best))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            torch.matmul(a, b, out=c)
        e1.record()
        e1.synchronize()
        sustained = e0.elapsed_time(e1) / reps
        del a, b, c
        torch.cuda.empty_cache()
        return dict(burst_tflops=fl / (best * 1e-3) / 1e12, sustained_tflops=fl / (sustained * 1e-3) / 1e12,
                    how=f"torch.matmul fp32 with TF32 allowed, {n}^3, CUDA events: best of 10 and {reps} back to back")
    except Exception as e:  # a comparator only: its absence must not fail the benchmark
        return dict(error=repr(e)[:200])


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def wait_first_sample(self, limit_s=10.0):
        t0 = time.time()
        while self.proc and not self.lines and time.time() - t0 < limit_s:
            time.sleep(0.05)

    def stop(self):
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [v.strip() for v in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        return dict(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), power_w_max=max(power), samples=len(sm), reasons=sorted(reasons))


# ------------------------------------------------------------------------------------------------
# the reference arm: the reference's own CPU implementation, single-threaded by construction
# ------------------------------------------------------------------------------------------------
def cpu_reference_step_time(steps, warmup, batch=CPU_SAMPLE_BATCH):
    """Times `steps` training steps of the same architecture at `batch` rows on one host core.
    Uses the unmodified reference library when it was built, else the plain-C port."""
    import oracle
    # the reference prints a banner and log lines on stdout: keep stdout for the one JSON line
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    try:
        return _cpu_reference_step_time(oracle, steps, warmup, batch)
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)


def _cpu_reference_step_time(oracle, steps, warmup, batch):
    if oracle.Reference.available():
        impl = oracle.Reference()
    else:
        impl = oracle.Oracle()
    p = make_params()
    x, lab = make_batch(0, batch)
    x4 = x.reshape(1, 1, batch, DIMS[0])
    l4 = lab.reshape(1, 1, batch)
    times = []
    # every call rebuilds the model from `p`, so each call is timed as setup + n steps and the setup
    # (a zero-step call) is subtracted
    t0 = time.perf_counter(); impl.mlp_train(DIMS, x4, l4, p, LR, 0, want_logits=False); setup = time.perf_counter() - t0
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        impl.mlp_train(DIMS, x4, l4, p, LR, 1, want_logits=False)
        dt = max(time.perf_counter() - t0 - setup, 1e-9)
        if i >= warmup:
            times.append(dt)
    return impl.kind, statistics.median(times), sum(times), batch


def reference_sample_batch(n_steps):
    """Rows per reference step such that warm-up + timed steps end in roughly 2-3 minutes: a step of the
    reference at this width costs about 0.6 s + 1.5 s per row on one core."""
    per_step = 150.0 / max(1, n_steps)
    return int(min(CPU_SAMPLE_BATCH, max(1, (per_step - 0.6) // 1.5)))


def run_reference(args, rank):
    if rank != 0:
        return
    kind, t_step, total, batch = cpu_reference_step_time(args.steps, args.warmup, batch=reference_sample_batch(args.steps + args.warmup))
    v = batch / t_step
    cpu = dict(value=v, unit="samples/s", cores=1, kind=kind,
               sample=f"{args.steps} timed steps of the same 784-4096-4096-4096-10 training step at batch {batch} (cost is linear in rows), median step {t_step:.3f} s, host {host_cpu()}")
    print(json.dumps(dict(impl="reference", metric="mlp_train_samples_per_s", value=v, unit="samples/s", n_gpus=args.gpus, steps=args.steps,
                          warmup=args.warmup, ms_per_step=t_step * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32",
                          data="synthetic", config=dict(workload=WORKLOAD, sample_batch=batch, threads=1),
                          cpu_baseline=cpu, e2e=dict(value=v, unit="samples/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))))


def host_cpu():
    try:
        for ln in open("/proc/cpuinfo"):
            if ln.startswith("model name"):
                return ln.split(":", 1)[1].strip() + f" x{os.cpu_count()}"
    except Exception:
        pass
    return f"unknown x{os.cpu_count()}"


# ------------------------------------------------------------------------------------------------
# checks that ride along with the timed run (the oracle is the checker here, never the thing timed)
# ------------------------------------------------------------------------------------------------
def _quiet_oracle(fn):
    """Runs fn with stdout pointed at stderr: the reference library prints a banner and log lines."""
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    try:
        return fn()
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)


def parity_check_full_size(F, params, x, labels, rows=(0, 1, 4095, 4096, 8191, 777, 5000, 6001)):
    """One full-size step of a freshly initialised network with the logits kept; the logits of a few rows
    against the oracle's forward pass on those rows with the same weights (forward is row-independent).
    (The timed trainer is not used: at the specified learning rate on a summed loss its weights have
    long left the range where a comparison says anything -- the reference diverges the same way.)"""
    import oracle
    rows = np.asarray(rows)
    tr = F.MlpTrainer(DIMS, params, LR)
    tr.keep_logits(True)
    loss = tr.step_host(x, labels)
    got = tr.logits(x.shape[0])[rows]
    del tr
    ref = _quiet_oracle(lambda: oracle.Oracle().mlp_train(DIMS, x[rows][None, None], labels[rows][None, None], params, LR, 1))
    err = float(np.abs(got - ref["logits"][0]).max() / max(np.abs(ref["logits"][0]).max(), 1e-30))
    return dict(what="logits of 8 sampled rows of one full-size step (fresh weights) vs the oracle's forward pass on those rows", rows=[int(r) for r in rows],
                normwise_err=err, tolerance=1e-4, ok=bool(err <= 1e-4), loss=float(loss))


DP_CHECK_DIMS, DP_CHECK_BATCH = [784, 128, 64, 10], 64


def dp_check_before(cb, F, cp, comm, dp_mode):
    """One step of a reduced-width network through the same communicator and exchange mode, against the
    oracle run as `world` replicas with summed gradients (rank 0 evaluates the oracle on every shard)."""
    import oracle
    from ctorch_b200.dp import shard_seed
    dims, batch = DP_CHECK_DIMS, DP_CHECK_BATCH
    rw = np.random.default_rng(4242)
    parts = []
    for i, j in zip(dims[:-1], dims[1:]):
        lim = np.sqrt(6.0 / i)
        parts += [rw.uniform(-lim, lim, (i, j)).astype(np.float32).ravel(), np.zeros(j, np.float32)]
    p0 = np.concatenate(parts)

    def shard(r):
        rng = np.random.default_rng(shard_seed(99, r))
        return (rng.integers(0, 256, (batch, dims[0])).astype(np.float32) / np.float32(255.0), rng.integers(0, dims[-1], batch).astype(np.float32))

    x, lab = shard(cp.rank)
    tr = F.MlpTrainer(dims, p0, 0.001)
    tr.set_dp_mode(dp_mode)
    tr.set_comm(comm)
    tr.step_host(x, lab)
    grads, params = tr.grads(), tr.params()
    tr.set_comm(None)
    del tr
    cb.synchronize()
    out = None
    if cp.rank == 0:
        xs = np.stack([shard(r)[0] for r in range(cp.world)])[:, None]
        ls = np.stack([shard(r)[1] for r in range(cp.world)])[:, None]
        ref = _quiet_oracle(lambda: oracle.Oracle().mlp_train(dims, xs, ls, p0, 0.001, 1, grad_steps=(0,), want_logits=False))
        pe = float(np.abs(params - ref["params"]).max() / np.abs(ref["params"]).max())
        out = dict(what=f"one step of {'-'.join(map(str, dims))} at batch {batch} per rank vs the oracle run as {cp.world} replicas with summed gradients",
                   param_normwise_err=pe, tolerance=1e-4, ok=bool(pe <= 1e-4))
        if dp_mode != "sharded":   # (sharded: a rank holds the summed gradient of its own shards only)
            ge = float(np.abs(grads - ref["grads"][0]).max() / np.abs(ref["grads"][0]).max())
            out.update(grad_normwise_err=ge, ok=bool(pe <= 1e-4 and ge <= 1e-4))
    cp.barrier()
    return out


def weights_spread(cp, params):
    """Largest difference between any two ranks' weights after the timed steps: 0 when every rank holds
    the same bits (compared through a hash; the element-wise difference is only formed if they differ)."""
    bits = params.view(np.uint32)
    h = float(int(np.bitwise_xor.reduce(bits)) % (1 << 24)) + float(int(bits[::4097].astype(np.uint64).sum()) % (1 << 24)) * 2.0 ** -24
    same = cp.max_over_ranks(h) == -cp.max_over_ranks(-h)
    if same:
        return 0.0
    import torch
    hi = torch.from_numpy(params.copy()); lo = torch.from_numpy(params.copy())
    cp.dist.all_reduce(hi, op=cp.dist.ReduceOp.MAX)
    cp.dist.all_reduce(lo, op=cp.dist.ReduceOp.MIN)
    return float((hi - lo).abs().max())


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_mlp(args, cp):
    rank, world, local_rank = cp.rank, cp.world, cp.local_rank
    import ctorch_b200 as cb
    from ctorch_b200 import frontend as F
    from ctorch_b200.device import PinnedArray
    cb.check(cb.lib.ctk_set_device(local_rank))
    cb.ops.set_matmul_pairing(args.pairing)
    cb.ops.set_matmul_correction(1 if args.correction == "bf16" else 0)
    F.set_quiet(True)
    peaks = measured_peaks()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    comm = None
    dp_before = None
    algo_used = ""
    if world > 1:
        from ctorch_b200 import dp
        # NVLS (the reduction done inside the NVSwitch) from 4 GPUs up unless told otherwise; with fewer ranks NCCL's own choice
        algo = args.nccl_algo if args.nccl_algo != "auto" else ("NVLS" if world >= 4 else "")
        comm, algo_used = dp.make_comm(cb, cp, max_ctas=args.max_ctas, nvls_ctas=args.nvls_ctas, algo=algo)
        if not args.no_checks:
            dp_before = dp_check_before(cb, F, cp, comm, args.dp_mode)

    params = make_params()
    x, labels = make_batch(rank)
    onehot = np.zeros((BATCH, DIMS[-1]), np.float32)
    onehot[np.arange(BATCH), labels.astype(int)] = 1
    lr = LR / BATCH if args.stable_lr else LR
    trainer = F.MlpTrainer(DIMS, params, lr)
    if comm is not None:
        trainer.set_dp_mode(args.dp_mode)
        trainer.set_comm(comm)
    X, Y = F.Tensor.from_numpy(x), F.Tensor.from_numpy(onehot)
    px, pl = PinnedArray(x.shape), PinnedArray(labels.shape)
    px.array[...] = x
    pl.array[...] = labels

    def barrier():
        cb.synchronize()
        cp.barrier()

    max_over_ranks = cp.max_over_ranks

    def timed(step_fn, profile):
        for _ in range(args.warmup):
            step_fn()
        barrier()
        if profile:
            cb.check(cb.lib.ctk_matmul_profile_enable(1))
        e0, e1 = cb.Event(), cb.Event()
        l0 = cb.launch_count()
        e0.record()
        loss = None
        for _ in range(args.steps):
            loss = step_fn()
        e1.record()
        e1.sync()
        cb.synchronize()
        launches = cb.launch_count() - l0
        ms = e0.elapsed_ms(e1)
        prof = None
        if profile:
            n, tms, fl = ctypes.c_int64(), ctypes.c_double(), ctypes.c_double()
            cb.check(cb.lib.ctk_matmul_profile_read(ctypes.byref(n), ctypes.byref(tms), ctypes.byref(fl)))
            cb.check(cb.lib.ctk_matmul_profile_enable(0))
            prof = (n.value, tms.value, fl.value)
        barrier()
        return max_over_ranks(ms), launches, loss, prof

    # nvidia-smi takes a few hundred ms to come up (and holds driver locks while it does): it was started
    # before the model was built, and timing begins only once it has delivered its first sample
    if rank == 0:
        sampler.wait_first_sample()
    ms_dev, launches, loss_dev, prof = timed(lambda: trainer.step_device(X, Y), True)
    clocks = sampler.stop() if rank == 0 else None
    # End to end, from HOST buffers.  Plain form: upload, step, loss read-back, one after the other.
    ms_e2e_serial, _, loss_e2e, _ = timed(lambda: trainer.step_host(px.array, pl.array), False)
    # As an input pipeline runs it: the upload of batch k+1 is started (copy stream) before step k is
    # issued, so it overlaps the compute; every timed step still does one upload (25.7 MB from
    # page-locked memory) and one loss read-back inside the timed region.
    trainer.stage_host(px.array, pl.array)

    def pipelined_step():
        trainer.stage_host(px.array, pl.array)
        return trainer.step_staged()

    ms_e2e, _, loss_e2e, _ = timed(pipelined_step, False)
    status = cb.ops.matmul_status()

    # The specified learning rate (0.01 on a loss SUMMED over 8192 rows) drives the weights away within a
    # few steps -- in the reference too -- so the timed steps above run on saturated activations.  The same
    # step with the rate scaled to the mean loss keeps every operand well conditioned; it is timed beside
    # the headline so that a reader can see whether the operands' values (through power and clocks) matter.
    stable = None
    if world == 1 and not args.no_checks:
        t2 = F.MlpTrainer(DIMS, params, LR / BATCH)
        ms_st, _, loss_st, _ = timed(lambda: t2.step_device(X, Y), False)
        stable = dict(lr=LR / BATCH, ms_per_step=ms_st / args.steps, value=BATCH / (ms_st / args.steps * 1e-3), loss_last=float(loss_st),
                      what="the same step on device-resident inputs with lr / batch (no divergence)")
        del t2

    parity = dp_after = None
    if not args.no_checks:
        if world == 1:
            parity = parity_check_full_size(F, params, x, labels)
        else:
            spread = weights_spread(cp, trainer.params())
            dp_after = dict(what=f"largest difference between any two ranks' weights after {3 * (args.warmup + args.steps)} steps", max_abs_diff=spread, ok=bool(spread == 0.0))
    extras = None
    if rank == 0 and world == 1 and not args.no_extras:
        del X, Y
        extras = run_extras(cb, peaks, with_cpu=not args.no_cpu_baseline, correction=args.correction)
    # last: its seconds-long loop leaves the chip hot and power-throttled for whatever follows
    lib_tf32 = measure_library_tf32(local_rank) if rank == 0 and not args.no_comparator else None
    if extras and lib_tf32 and "burst_tflops" in lib_tf32:
        for e in extras:
            if e.get("bound") == "tensor":
                e["frac_of_library_tf32_gemm"] = e["value"] / (lib_tf32["burst_tflops"] / e["tf32_units"])

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        kind, t_step, total, b = cpu_reference_step_time(2, 0)
        cpu = dict(value=b / t_step, unit="samples/s", cores=1, kind=kind,
                   sample=f"2 steps of the same training step at batch {b} (cost linear in rows), median step {t_step:.2f} s, single thread (the reference has no threading), host {host_cpu()}")

    if rank == 0:
        per_step = ms_dev / args.steps
        value = BATCH * world / (per_step * 1e-3)
        e2e_v = BATCH * world / (ms_e2e / args.steps * 1e-3)
        n, tms, fl = prof
        achieved = fl / (tms * 1e-3) / 1e12 if tms > 0 else 0.0
        # Ceilings.  `peak` is the nominal dense TF32 rate of the part (1125 TFLOP/s) / 3: three TF32 products
        # are issued per fp32 product, and nothing can exceed it.  Beside it: a TF32 GEMM of the vendor
        # library timed in this run, and the driver-measured bf16 GEMM halved (TF32 issues at half the bf16
        # rate) -- library kernels that a hand-written kernel can pass, so a fraction above 1 against them
        # is possible and says how far the library itself is from the hardware.
        at_max = clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz") and clocks["sm_mhz"] >= 0.95 * clocks["sm_max_mhz"]
        bf16_key, bf16_val = ("bf16_tflops (burst)", peaks["bf16"]) if at_max else ("bf16_tflops_sustained", peaks["bf16_sustained"])
        # units of TF32-rate tensor work per fp32 product: three TF32 products, or one TF32 + two bf16 (each at twice the TF32 rate)
        units = 3.0 if args.correction == "tf32" else 2.0
        peak = NOMINAL_TF32 / units
        ceilings = {f"nominal_tf32_over_{units:g}": dict(peak=peak, frac=achieved / peak),
                    f"measured_bf16_over_{2 * units:g}": dict(peak=bf16_val / (2 * units), frac=achieved / (bf16_val / (2 * units)), source=f"{peaks['source']}: {bf16_key} {bf16_val}")}
        if lib_tf32 and "burst_tflops" in lib_tf32:
            lib_peak = (lib_tf32["burst_tflops"] if at_max else lib_tf32["sustained_tflops"]) / units
            ceilings[f"library_tf32_gemm_over_{units:g}"] = dict(peak=lib_peak, frac=achieved / lib_peak, measured=lib_tf32)
        elif lib_tf32:
            ceilings[f"library_tf32_gemm_over_{units:g}"] = lib_tf32
        flops_step = sum(2.0 * BATCH * i * j for i, j in zip(DIMS[:-1], DIMS[1:])) * 2 + sum(2.0 * BATCH * i * j for i, j in zip(DIMS[1:-1], DIMS[2:]))
        out = dict(
            metric="mlp_train_samples_per_s", value=value, unit="samples/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
            ms_per_step=per_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
            config=dict(workload=WORKLOAD, global_batch=BATCH * world, parallelism=f"dp{world}", matmul_mode="3xtf32" if args.correction == "tf32" else "tf32 + 2 x bf16 correction terms",
                        lr=lr, gradient_exchange=(args.dp_mode if world > 1 else None), nccl_max_ctas=args.max_ctas or None, nccl_algo=(algo_used or "NCCL's choice") if world > 1 else None,
                        l2="per-step working set (weights 147 MB + activations 3x134 MB per layer pass) exceeds the 126 MB L2",
                        loss_last=float(loss_dev) if loss_dev is not None else None, matmul_status=status, stable_lr_run=stable),
            clocks=clocks,
            e2e=dict(value=e2e_v, unit="samples/s", ms_per_step=ms_e2e / args.steps,
                     h2d_bytes_per_step=int(x.nbytes + labels.nbytes), d2h_bytes_per_step=4,
                     call="cth_mlp_stage_host(batch k+1) + cth_mlp_step_staged(batch k): the upload overlaps the previous step's compute",
                     serial_value=BATCH * world / (ms_e2e_serial / args.steps * 1e-3), serial_ms_per_step=ms_e2e_serial / args.steps,
                     serial_call="cth_mlp_step_host: upload, step and loss read-back in sequence"),
            gpu_launches=int(launches),
            roofline=dict(bound="tensor", achieved=achieved, peak=peak, unit="TFLOP/s", frac=achieved / peak,
                          peak_source=f"nominal dense TF32 rate 1125 TFLOP/s / {units:g} ({'three TF32 products' if units == 3 else 'one TF32 product + two bf16 products at twice the TF32 rate = two units of TF32-rate work'} per fp32 product); algorithmic flops 2*M*N*K; measured alternatives under `ceilings`",
                          ceilings=ceilings,
                          # not measured in this run: one ncu capture of one launch of the dominant shape, kept under profiles/
                          traffic=QUOTED_TRAFFIC["bytes"], traffic_quoted_from=QUOTED_TRAFFIC["from"], traffic_launch=QUOTED_TRAFFIC["launch"],
                          kernel=f"tcgen05_matmul_pair_kernel / tcgen05_matmul_kernel (fp32-accurate mode, correction terms on the {args.correction} path)", launches=int(n), avg_launch_ms=tms / n if n else None,
                          step_model_flops=flops_step, step_tflops=flops_step / (per_step * 1e-3) / 1e12, step_frac=flops_step / (per_step * 1e-3) / 1e12 / peak),
            parity_check=parity, dp_check=dict(before=dp_before, after=dp_after) if world > 1 else None, extras=extras,
            cpu_baseline=cpu,
        )
        print(json.dumps(out))
    if comm is not None:
        trainer.set_comm(None)
        del trainer
        cb.synchronize()
        cb.lib.ctk_comm_destroy(comm)


def run_extras(cb, peaks, with_cpu=True, correction="bf16"):
    """The single-op metrics of the other benchmark configurations, bounded to a few tens of seconds:
    elementwise Add / Mul-backward / Tanh at 2^28, softmax and cross entropy at C in {10, 1000, 32000},
    Sum at 2^28, and the three products at 8192^3 and 65536 x 784 x 4096 in both tensor-core modes.
    Every entry: achieved rate, fraction of the measured (HBM) or nominal (tensor) ceiling, and the
    reference's own CPU rate on a bounded sample of the same operation (one thread: it has no others).
    Operands are larger than the 126 MB L2 (C = 10 runs on 4 Mi rows for that reason)."""
    import oracle
    ref = None
    if with_cpu:
        ref = _quiet_oracle(lambda: oracle.Reference() if oracle.Reference.available() else oracle.Oracle())
    hbm = peaks["hbm_gbs"]
    i64 = ctypes.c_int64
    out = []

    def gpu_ms(fn, iters, warm=3):
        for _ in range(warm):
            fn()
        e0, e1 = cb.Event(), cb.Event()
        cb.synchronize()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        e1.sync()
        return e0.elapsed_ms(e1) / iters

    def cpu_rate(fn, work, unit, sample, warm=True):
        if ref is None:
            return None
        def run():
            if warm:
                fn()   # once untimed: page faults, the library's first-call set-up
            t0 = time.perf_counter()
            fn()
            return time.perf_counter() - t0
        dt = _quiet_oracle(run)
        return dict(value=work / dt / (1e9 if unit == "GB/s" else 1e12), unit=unit, cores=1, kind=ref.kind, sample=sample)

    def add(name, ms, work, unit, cpu, **extra):
        ach = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
        d = dict(name=name, value=ach, unit=unit, ms=ms)
        if unit == "GB/s":
            d.update(bound="hbm", peak=hbm, frac=ach / hbm, frac_of_nominal=ach / NOMINAL_HBM, peak_source=peaks["source"] + " hbm_gbs")
        d.update(extra)
        d["cpu_baseline"] = cpu
        out.append(d)

    rng = np.random.default_rng(0)
    # ---- elementwise, 2^28 (1 GiB per array; inputs U(-4, 4), second operand U(0.5, 4), generated on the device)
    n = 1 << 28
    a = cb.ops.rand_uniform((n,), seed=1); cb.ops.scalar(0, a, 8.0, out=a); cb.ops.scalar(1, a, -4.0, out=a)
    b = cb.ops.rand_uniform((n,), seed=2); cb.ops.scalar(0, b, 3.5, out=b); cb.ops.scalar(1, b, 0.5, out=b)
    g = cb.ops.rand_uniform((n,), seed=3)
    o, o2 = cb.empty((n,)), cb.empty((n,))
    ns = 1 << 22
    ha, hb, hg = (v.view(0, (ns,)).numpy() for v in (a, b, g))
    add("Add_fwd_2^28", gpu_ms(lambda: cb.ops.binary("Add", a, b, out=o), 10), 12 * n, "GB/s",
        cpu_rate(lambda: ref.binary("Add", ha, hb), 12 * ns, "GB/s", "the same op on 2^22 elements"))
    add("Mul_bwd_2^28", gpu_ms(lambda: lib_binary_bwd(cb, "Mul", a, b, g, o, o2), 10), 20 * n, "GB/s",
        cpu_rate(lambda: ref.grad_binary("Mul", ha, hb, hg), 20 * ns, "GB/s", "the Mul rule of AutoDiff::backward on 2^22 elements"))
    add("Tanh_fwd_2^28", gpu_ms(lambda: cb.ops.unary("Tanh", a, out=o), 10), 8 * n, "GB/s",
        cpu_rate(lambda: ref.unary("Tanh", ha), 8 * ns, "GB/s", "the same op on 2^22 elements"))
    s24 = a.view(0, (1 << 24,)).numpy()
    add("Sum_2^28", gpu_ms(lambda: cb.ops.sum(a), 10), 4 * n, "GB/s",
        cpu_rate(lambda: ref.sum(s24), 4 * (1 << 24), "GB/s", "Tensor::sum on 2^24 elements"))
    del a, b, g, o, o2
    # ---- row-wise
    for C in (10, 1000, 32000):
        rows = (1 << 22) if C == 10 else 65536
        block = (2 * rng.standard_normal((64, C))).astype(np.float32)          # logits N(0, 2^2)
        x = cb.ops.tile(cb.to_device(block), rows * C).reshape(rows, C)
        y = cb.empty((rows, C))
        labels = rng.integers(0, C, rows).astype(np.float32)
        lab = cb.to_device(labels)
        rs = max(32, (1 << 20) // C)
        hx = np.tile(block, (rs // 64 + 1, 1))[:rs]
        it = 10 if C < 32000 else 3
        add(f"softmax_fwd_{rows}x{C}", gpu_ms(lambda: cb.ops.softmax(x, out=y), it), 8 * rows * C, "GB/s",
            cpu_rate(lambda: ref.softmax(hx), 8 * rs * C, "GB/s", f"Tensor::softmax on [{rs}, {C}]"))
        add(f"ce_index_fwd_{rows}x{C}", gpu_ms(lambda: cb.ops.cross_entropy(x, lab), it), 4 * rows * C + 4 * rows, "GB/s",
            cpu_rate(lambda: ref.ce(hx, labels[:rs]), 4 * rs * C + 4 * rs, "GB/s", f"CrossEntropy_BASIC_kernel (index labels) on [{rs}, {C}]"))
        add(f"ce_fused_fwd_bwd_{rows}x{C}", gpu_ms(lambda: lib_ce_fused(cb, x, lab, y, rows, C), it), 8 * rows * C + 4 * rows, "GB/s", None,
            note="forward + gradient in one pass; the reference runs them as separate passes (its backward needs one-hot labels)")
        del x, y, lab
        _scratch.clear()
    # ---- products (operands N(0, 1): one 2^24 block tiled on the device)
    blk = cb.to_device(rng.standard_normal(1 << 24).astype(np.float32))
    hblk = blk.numpy()

    def mat(rows_, cols_, shift):
        return cb.ops.tile(blk.view(shift, ((1 << 24) - shift,)), rows_ * cols_).reshape(rows_, cols_)

    def host_rows(shift, nrows, cols_):        # the first rows of mat(., cols_, shift) as a host array
        return np.resize(hblk[shift:], nrows * cols_).reshape(nrows, cols_)

    def host_cols(shift, nrows, cols_, r):     # the first r columns of mat(nrows, cols_, shift)
        idx = (np.arange(nrows, dtype=np.int64)[:, None] * cols_ + np.arange(r)[None, :]) % ((1 << 24) - shift) + shift
        return np.ascontiguousarray(hblk[idx])

    from ctorch_b200 import frontend as F
    for (m, k, nn) in ((8192, 8192, 8192), (65536, 784, 4096)):
        A, B, dC = mat(m, k, 0), mat(k, nn, 1237), mat(m, nn, 40961)
        Cc, dA, dB = cb.empty((m, nn)), cb.empty((m, k)), cb.empty((k, nn))
        fl = 2.0 * m * nn * k
        r = 4
        cpus = {}
        if ref is not None:
            hB = host_rows(1237, k, nn)
            a_rows, dc_rows = host_rows(0, r, k), host_rows(40961, r, nn)
            cpus["fwd"] = cpu_rate(lambda: ref.matmul(a_rows, hB), 2.0 * r * k * nn, "TFLOP/s", f"{r} rows of C (MatMul_BASIC_kernel, cost linear in rows)", warm=False)
            cpus["dA"] = cpu_rate(lambda: ref.matmul(dc_rows, hB, False, True), 2.0 * r * k * nn, "TFLOP/s", f"{r} rows of dA = dC.B^T", warm=False)
            # rows of dB = A^T.dC: columns of A against all of dC
            rb = r if m == 8192 else 1
            a_cols, hdC = host_cols(0, m, k, rb), host_rows(40961, m, nn)
            cpus["dB"] = cpu_rate(lambda: ref.matmul(a_cols, hdC, True, False), 2.0 * rb * m * nn, "TFLOP/s", f"{rb} row(s) of dB = A^T.dC", warm=False)
            del a_cols, hdC, hB
        units = 3.0 if correction == "tf32" else 2.0
        for mode, nominal in (("3xtf32", NOMINAL_TF32 / units), ("tf32", NOMINAL_TF32)):
            for which, fn in (("fwd", lambda: cb.ops.matmul(A, B, mode=mode, out=Cc)),
                              ("dA", lambda: cb.ops.matmul(dC, B, tb=True, mode=mode, out=dA)),
                              ("dB", lambda: cb.ops.matmul(A, dC, ta=True, mode=mode, out=dB))):
                ms = gpu_ms(fn, 5)
                # the tensor-core kernel alone (without the operand-split passes of a 3xTF32 call), by the library's own events
                cb.check(cb.lib.ctk_matmul_profile_enable(1))
                fn(); fn()
                cnt, tms, tfl = ctypes.c_int64(), ctypes.c_double(), ctypes.c_double()
                cb.check(cb.lib.ctk_matmul_profile_read(ctypes.byref(cnt), ctypes.byref(tms), ctypes.byref(tfl)))
                cb.check(cb.lib.ctk_matmul_profile_enable(0))
                kern = tfl.value / (tms.value * 1e-3) / 1e12 if tms.value > 0 else None
                ach = fl / (ms * 1e-3) / 1e12
                d = dict(bound="tensor", tf32_units=(units if mode == "3xtf32" else 1.0), peak=nominal, frac=ach / nominal, peak_source="nominal dense TF32 1125 TFLOP/s" + (f" / {units:g} (correction terms on the {correction} path)" if mode == "3xtf32" else ""),
                         kernel_alone_tflops=kern, kernel_alone_frac=(kern / nominal if kern else None),
                         call="ctk_matmul_f32, operands split inside the call (3xTF32)" if mode == "3xtf32" else "ctk_matmul_f32, operands read in place")
                add(f"matmul_{which}_{mode}_{m}x{k}x{nn}", ms, fl, "TFLOP/s", cpus.get(which), **d)
        del Cc, dA, dB
        # the three products as user code gets them: C = A.matmul(B); backward(C, dC) through Tensor / AutoDiff,
        # where every operand's split is made once and kept for the second product that reads it
        tA, tB, tG = (F.Tensor.from_numpy(v.numpy()) for v in (A, B, dC))
        del A, B, dC
        with F.AutoDiff() as ctx:
            ctx.make_leaf(tA, True); ctx.make_leaf(tB, True)
            tA.requires_grad(); tB.requires_grad()

            def fwd_bwd():
                ctx.zero_grad(tA); ctx.zero_grad(tB)
                F.backward(tA.matmul(tB), tG)
                ctx.release_step_nodes()
            ms = gpu_ms(fwd_bwd, 5)
        add(f"matmul_fwd_bwd_frontend_{m}x{k}x{nn}", ms, 3 * fl, "TFLOP/s", None, bound="tensor", tf32_units=units, peak=NOMINAL_TF32 / units,
            frac=3 * fl / (ms * 1e-3) / 1e12 / (NOMINAL_TF32 / units),
            call="Tensor::matmul + backward(C, dC): C, dA and dB in the fp32-accurate mode, each operand split once")
        del tA, tB, tG
    out.append(dict(name="matmul_status", value=cb.ops.matmul_status()))
    return out


def run_single_op(args):
    """The single-op sweeps (one GPU): prints one JSON line per measurement."""
    import ctorch_b200 as cb
    cb.check(cb.lib.ctk_set_device(0))
    cb.ops.set_matmul_pairing(args.pairing)
    cb.ops.set_matmul_correction(1 if args.correction == "bf16" else 0)
    peaks = measured_peaks()

    def timeit(fn, iters, warm=3):
        for _ in range(warm):
            fn()
        e0, e1 = cb.Event(), cb.Event()
        cb.synchronize()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        e1.sync()
        return e0.elapsed_ms(e1) / iters

    def emit(name, ms, work, unit, peak, extra=None):
        ach = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
        d = dict(metric=name, value=ach, unit=unit, n_gpus=1, ms=ms, higher_is_better=True, data="synthetic",
                 roofline=dict(bound="hbm" if unit == "GB/s" else "tensor", achieved=ach, peak=peak, unit=unit, frac=ach / peak, traffic=None,
                               peak_source=peaks["source"]))
        if extra:
            d["config"] = extra
        print(json.dumps(d), flush=True)

    rng = np.random.default_rng(0)
    if args.workload == "elementwise":
        for logn in (20, 24, 28):
            n = 1 << logn
            # two rotating buffer sets larger than L2 at 2^24 and above
            a = cb.to_device(rng.uniform(-4, 4, n).astype(np.float32)); b = cb.to_device(rng.uniform(0.5, 4, n).astype(np.float32))
            g = cb.to_device(rng.standard_normal(n).astype(np.float32)); o, o2 = cb.empty((n,)), cb.empty((n,))
            row = cb.to_device(rng.uniform(0.5, 4, 1024).astype(np.float32))
            it = 20
            for op in ("Add", "Sub", "Mul", "Div"):
                emit(f"{op}_fwd_2^{logn}", timeit(lambda: cb.ops.binary(op, a, b, out=o), it), 12 * n, "GB/s", peaks["hbm_gbs"])
                emit(f"{op}_scalar_2^{logn}", timeit(lambda: cb.ops.binary(op, a, b.view(0, (1,)), cb.ops.B_SCALAR, out=o), it), 8 * n, "GB/s", peaks["hbm_gbs"])
                emit(f"{op}_row1024_2^{logn}", timeit(lambda: cb.ops.binary(op, a, row, cb.ops.B_ROW, out=o), it), 8 * n + 4096, "GB/s", peaks["hbm_gbs"])
                bwd_bytes = 12 * n if op in ("Add", "Sub") else 20 * n
                emit(f"{op}_bwd_2^{logn}", timeit(lambda: lib_binary_bwd(cb, op, a, b, g, o, o2), it), bwd_bytes, "GB/s", peaks["hbm_gbs"])
            for op in ("Neg", "ReLU", "Sigmoid", "Tanh", "Sin", "Cos"):
                emit(f"{op}_fwd_2^{logn}", timeit(lambda: cb.ops.unary(op, a, out=o), it), 8 * n, "GB/s", peaks["hbm_gbs"])
                emit(f"{op}_bwd_2^{logn}", timeit(lambda: lib_unary_bwd(cb, op, a, g, o), it), (8 if op == "Neg" else 12) * n, "GB/s", peaks["hbm_gbs"])
            # comparisons (float -> bool bytes), conversions out of float, uniform random numbers
            ob = cb.DeviceArray((n,), np.uint8)
            emit(f"cmp_gt_tensor_2^{logn}", timeit(lambda: cb.check(cb.lib.ctk_compare_f32(0, 0, a.p, b.p, ctypes.c_float(0), ob.p, ctypes.c_int64(n), None)), it), 9 * n, "GB/s", peaks["hbm_gbs"])
            emit(f"cmp_gt_scalar_2^{logn}", timeit(lambda: cb.check(cb.lib.ctk_compare_f32(0, 1, a.p, None, ctypes.c_float(1.0), ob.p, ctypes.c_int64(n), None)), it), 5 * n, "GB/s", peaks["hbm_gbs"])
            for code, name, size in ((1, "f64", 8), (2, "i32", 4), (3, "i64", 8), (4, "bool", 1)):
                od = ob if size == 1 else (o if size == 4 else None)
                if od is None:
                    od = cb.DeviceArray((n,), np.float64)
                emit(f"cast_f32_{name}_2^{logn}", timeit(lambda: cb.check(cb.lib.ctk_cast_f32(code, a.p, od.p, ctypes.c_int64(n), None)), it), (4 + size) * n, "GB/s", peaks["hbm_gbs"])
                del od
            emit(f"rand_uniform_2^{logn}", timeit(lambda: cb.check(cb.lib.ctk_rand_uniform_f32(o.p, ctypes.c_int64(n), ctypes.c_uint64(1), ctypes.c_uint64(0), None)), it), 4 * n, "GB/s", peaks["hbm_gbs"])
            del a, b, g, o, o2, ob
    elif args.workload == "rowwise":
        for C in (10, 1000, 32000):
            rows = (1 << 22) if C == 10 else 65536  # every operand larger than the 126 MB L2
            x = cb.empty((rows, C)); cb.ops.fill(x, 0.0)
            xs = cb.to_device((2 * rng.standard_normal((rows, min(C, 1000)))).astype(np.float32)) if C <= 1000 else None
            if xs is not None:
                x = xs
            else:
                tile = cb.to_device((2 * rng.standard_normal(C * 64)).astype(np.float32))
                x = cb.ops.tile(tile, rows * C).reshape(rows, C)
            y = cb.empty((rows, C))
            lab = cb.to_device(rng.integers(0, C, rows).astype(np.float32))
            it = 10 if C < 32000 else 3
            emit(f"softmax_fwd_C{C}", timeit(lambda: cb.ops.softmax(x, out=y), it), 8 * rows * C, "GB/s", peaks["hbm_gbs"])
            emit(f"softmax_bwd_C{C}", timeit(lambda: lib_softmax_bwd(cb, y, x, rows, C), it), 12 * rows * C, "GB/s", peaks["hbm_gbs"])
            emit(f"ce_index_fwd_C{C}", timeit(lambda: cb.ops.cross_entropy(x, lab), it), 4 * rows * C + 4 * rows, "GB/s", peaks["hbm_gbs"])
            emit(f"ce_fused_fwd_bwd_C{C}", timeit(lambda: lib_ce_fused(cb, x, lab, y, rows, C), it), 8 * rows * C + 4 * rows, "GB/s", peaks["hbm_gbs"])
            del x, y
        n = 65536 * 1024
        a = cb.to_device(rng.standard_normal(n).astype(np.float32)); b = cb.to_device(rng.standard_normal(n).astype(np.float32)); o = cb.empty((n,))
        emit("mse_fwd_65536x1024", timeit(lambda: cb.ops.mse(a, b), 10), 8 * n, "GB/s", peaks["hbm_gbs"])
        emit("mae_fwd_65536x1024", timeit(lambda: cb.ops.mae(a, b), 10), 8 * n, "GB/s", peaks["hbm_gbs"])
        emit("mse_bwd_65536x1024", timeit(lambda: cb.check(cb.lib.ctk_mse_backward_f32(a.p, b.p, None, o.p, ctypes.c_int64(n), None)), 10), 12 * n, "GB/s", peaks["hbm_gbs"])
        del a, b, o
        n = 1 << 28
        a = cb.ops.tile(cb.to_device(rng.uniform(-4, 4, 1 << 20).astype(np.float32)), n)
        emit("sum_2^28", timeit(lambda: cb.ops.sum(a), 10), 4 * n, "GB/s", peaks["hbm_gbs"])
    elif args.workload == "matmul":
        units = 2.0 if args.correction == "bf16" else 3.0   # TF32-rate units of tensor work per fp32 product
        for mode, peak in (("tf32", NOMINAL_TF32), ("3xtf32", NOMINAL_TF32 / units)):
            for (m, k, n) in ((512, 512, 512), (1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192), (65536, 784, 4096)):
                A = cb.to_device(rng.standard_normal((m, k)).astype(np.float32)); B = cb.to_device(rng.standard_normal((k, n)).astype(np.float32))
                dC = cb.to_device(rng.standard_normal((m, n)).astype(np.float32))
                C, dA, dB = cb.empty((m, n)), cb.empty((m, k)), cb.empty((k, n))
                it = 20 if m <= 2048 else 5
                fl = 2.0 * m * n * k
                cfg = dict(m=m, n=n, k=k, mode=mode, correction=args.correction if mode == "3xtf32" else None,
                           peak_source="nominal dense TF32 1125 TFLOP/s" + (f" / {units:g}" if mode == "3xtf32" else ""))
                emit(f"matmul_fwd_{mode}_{m}x{k}x{n}", timeit(lambda: cb.ops.matmul(A, B, mode=mode, out=C), it), fl, "TFLOP/s", peak, cfg)
                emit(f"matmul_dA_{mode}_{m}x{k}x{n}", timeit(lambda: cb.ops.matmul(dC, B, tb=True, mode=mode, out=dA), it), fl, "TFLOP/s", peak, cfg)
                emit(f"matmul_dB_{mode}_{m}x{k}x{n}", timeit(lambda: cb.ops.matmul(A, dC, ta=True, mode=mode, out=dB), it), fl, "TFLOP/s", peak, cfg)
                del A, B, dC, C, dA, dB
        print(json.dumps(dict(matmul_status=cb.ops.matmul_status())))
    elif args.workload == "mnist":
        run_mnist_app(cb, args, rng)
    elif args.workload == "mlp_small":
        run_mlp_small(cb, args)
    elif args.workload == "kernel":
        run_one_kernel(cb, args.case, rng)
    else:
        raise SystemExit("unknown workload " + args.workload)


def run_mlp_small(cb, args):
    """Benchmark config 1, the reference's own CPU-runnable case: 784-128-10, batch 64, SGD lr 0.01, a fixed
    seeded sequence of 100 batches, 100 steps (launch-bound on a GPU: reported as samples/s and us per step).
    The reference's CPU path runs the same 100 steps on one host core next to it."""
    from ctorch_b200 import frontend as F
    from ctorch_b200.device import PinnedArray
    F.set_quiet(True)
    dims, batch, steps, lr = [784, 128, 10], 64, 100, 0.01
    rng = np.random.default_rng(1234)
    xs = (rng.integers(0, 256, (steps, batch, 784)) / 255.0).astype(np.float32)
    labs = rng.integers(0, 10, (steps, batch)).astype(np.float32)
    wr = np.random.default_rng(42)
    parts = []
    for i, j in zip(dims[:-1], dims[1:]):
        lim = np.sqrt(6.0 / i)
        parts += [wr.uniform(-lim, lim, (i, j)).astype(np.float32).ravel(), np.zeros(j, np.float32)]
    p0 = np.concatenate(parts)
    px, pl = PinnedArray(xs.shape), PinnedArray(labs.shape)
    px.array[...] = xs
    pl.array[...] = labs

    def run(graph):
        tr = F.MlpTrainer(dims, p0, lr)
        step = tr.step_graph_host if graph else tr.step_host
        t0 = time.perf_counter()   # wall clock: the graph path runs on a stream of its own
        cb.synchronize()
        loss = 0.0
        for s in range(steps):
            loss = step(px.array[s], pl.array[s])
        cb.synchronize()
        return time.perf_counter() - t0, loss

    for _ in range(3):
        run(False)
        run(True)
    t_eager, loss_eager = run(False)
    t, loss = run(True)   # steps 0-1 of the run are eager, step 2 is the recording; 97 replays follow
    assert loss == loss_eager, (loss, loss_eager)
    cpu = None
    if not args.no_cpu_baseline:
        import oracle
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)   # the reference prints a banner on stdout
        try:
            impl = oracle.Reference() if oracle.Reference.available() else oracle.Oracle()
            n_cpu = 10
            t0 = time.perf_counter()
            impl.mlp_train(dims, xs[:n_cpu].reshape(1, n_cpu, batch, 784), labs[:n_cpu].reshape(1, n_cpu, batch), p0, lr, n_cpu, want_logits=False)
            t_cpu = (time.perf_counter() - t0) / n_cpu
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
        cpu = dict(value=batch / t_cpu, unit="samples/s", cores=1, kind=impl.kind, sample=f"{n_cpu} steps of the same run, {t_cpu * 1e3:.1f} ms per step, host {host_cpu()}")
    print(json.dumps(dict(metric="mlp_small_train_samples_per_s", value=steps * batch / t, unit="samples/s", n_gpus=1, steps=steps, higher_is_better=True,
                          dtype="f32", data="synthetic", config=dict(workload="mlp-784-128-10_batch64_100-steps_from-host-batches", us_per_step=t / steps * 1e6, final_loss=float(loss),
                                      call="cth_mlp_step_graph_host (steps 0-1 eager, step 2 recorded into a CUDA graph, 97 replays; all 100 timed)",
                                      eager_us_per_step=t_eager / steps * 1e6, eager_samples_per_s=steps * batch / t_eager),
                          e2e=dict(value=steps * batch / t, unit="samples/s", h2d_bytes_per_step=int(xs[0].nbytes + labs[0].nbytes), d2h_bytes_per_step=4),
                          cpu_baseline=cpu)))


def run_mnist_app(cb, args, rng):
    """The reference application (mnist/mnist.cpp:218-275): 784-128-64-10, batch 128, lr 0.01, 5 epochs over
    60000 training images in file order, then accuracy on the training and the 10000 test images.  The
    MNIST image files are not available here: a synthetic set in the same IDX format stands in (dim
    noise plus a bright band whose position encodes the class, shifted at random), read by the
    product's IDX loader.  The data set lives in HBM; an epoch is 468 steps on views of it."""
    import tempfile
    from ctorch_b200 import frontend as F
    F.set_quiet(True)
    # lr: the application's 0.01 acts on a loss SUMMED over the 128 rows of a batch; on this synthetic set
    # that diverges (it is the reference's behaviour too), so the run uses 0.01 / 128, i.e. the same step
    # on the mean loss, and says so in its config
    dims, batch, epochs, lr = [784, 128, 64, 10], 128, 5, 0.01 / 128

    def synth(n):
        lab = rng.integers(0, 10, n).astype(np.uint8)
        px = rng.integers(0, 64, (n, 28, 28)).astype(np.uint8)
        shift = rng.integers(0, 3, n)
        for c in range(10):
            for sft in range(3):
                idx = np.nonzero((lab == c) & (shift == sft))[0]
                px[idx, 2 * c + sft: 2 * c + sft + 3, 2 + 2 * c: 8 + 2 * c] = 255   # rows shift, columns name the class
        return px, lab

    with tempfile.TemporaryDirectory() as d:
        for names, n in ((("train-images-idx3-ubyte", "train-labels-idx1-ubyte"), 60000), (("t10k-images-idx3-ubyte", "t10k-labels-idx1-ubyte"), 10000)):
            px, lab = synth(n)
            with open(os.path.join(d, names[0]), "wb") as f:   # IDX3: big-endian magic 2051, n, rows, cols, then the bytes
                f.write(np.asarray([2051, n, 28, 28], ">i4").tobytes() + px.tobytes())
            with open(os.path.join(d, names[1]), "wb") as f:   # IDX1: magic 2049, n, then the bytes
                f.write(np.asarray([2049, n], ">i4").tobytes() + lab.tobytes())
        t0 = time.perf_counter()
        train_x, train_y = F.mnist_load(d, "train")
        test_x, test_y = F.mnist_load(d, "test")
        cb.synchronize()
        load_s = time.perf_counter() - t0
    parts = []
    for i, j in zip(dims[:-1], dims[1:]):
        lim = np.sqrt(6.0 / i)
        parts += [rng.uniform(-lim, lim, (i, j)).astype(np.float32).ravel(), np.zeros(j, np.float32)]
    tr = F.MlpTrainer(dims, np.concatenate(parts), lr)
    tr.train_epoch(train_x.narrow_rows(0, 10 * batch), train_y.narrow_rows(0, 10 * batch), batch)   # warm-up: 10 untimed steps
    tr = F.MlpTrainer(dims, np.concatenate(parts), lr)
    cb.synchronize()
    t0 = time.perf_counter()   # wall clock: the graph-replayed steps run on a stream of their own
    losses = [tr.train_epoch_graph(train_x, train_y, batch) for _ in range(epochs)]
    cb.synchronize()
    train_s = time.perf_counter() - t0
    t0 = time.perf_counter()
    acc_train, acc_test = tr.accuracy(train_x, train_y), tr.accuracy(test_x, test_y)
    eval_s = time.perf_counter() - t0
    steps = epochs * (60000 // batch)
    print(json.dumps(dict(metric="mnist_app_train_samples_per_s", value=steps * batch / train_s, unit="samples/s", n_gpus=1, higher_is_better=True,
                          data="synthetic IDX files (60000 + 10000 images of 28x28 bytes)", dtype="f32",
                          config=dict(workload="mnist-app-784-128-64-10_batch128_5epochs", lr=lr, steps=steps, us_per_step=train_s / steps * 1e6,
                                      call="cth_mlp_train_epoch_graph: every step a replay of one recorded CUDA graph"),
                          load_s=load_s, train_s=train_s, eval_s=eval_s, epoch_mean_loss=[float(v) for v in losses],
                          accuracy_train=float(acc_train), accuracy_test=float(acc_test))))


def run_one_kernel(cb, case, rng):
    """A few launches of ONE kernel on a small case (inputs larger than L2, a few hundred MB on the
    device): the command profiler captures are taken from.  Cases: matmul_<mode>_<m>x<k>x<n>[_dA|_dB|_fwdfused|_dAfused]
    (mode 3xtf32, tf32 or simt), add_<log2n>, relu_<log2n>, sum_<log2n>, cmp_<log2n>, cast_<log2n>, rand_<log2n>,
    u8_<log2n>, sgdsplit_<rows>x<cols>, colsum_<rows>x<cols>, softmax_<rows>x<cols>, softmaxcols_<rows>x<cols>,
    ce_<rows>x<cols>, argmax_<rows>x<cols>, gather_<rows>x<cols>."""
    parts = case.split("_")
    kind = parts[0]
    if kind == "matmul":
        mode = "fp32_simt" if parts[1] == "simt" else parts[1]
        m, k, n = (int(v) for v in parts[2].split("x"))
        which = parts[3] if len(parts) > 3 else "fwd"
        A = cb.to_device(rng.standard_normal((m, k)).astype(np.float32)); B = cb.to_device(rng.standard_normal((k, n)).astype(np.float32))
        dC = cb.to_device(rng.standard_normal((m, n)).astype(np.float32))
        ws = cb.empty((cb.lib.ctk_matmul_workspace_bytes(max(m, n), max(m, n), max(k, m), cb.ops.MODES[mode]) // 4 + 64,))
        outs = dict(fwd=cb.empty((m, n)), dA=cb.empty((m, k)), dB=cb.empty((k, n)))
        fn = dict(fwd=lambda: cb.ops.matmul(A, B, mode=mode, out=outs["fwd"], workspace=ws),
                  dA=lambda: cb.ops.matmul(dC, B, tb=True, mode=mode, out=outs["dA"], workspace=ws),
                  dB=lambda: cb.ops.matmul(A, dC, ta=True, mode=mode, out=outs["dB"], workspace=ws)).get(which)
        if which in ("fwdfused", "dAfused"):
            # the products of the training step with their epilogues: forward + bias + ReLU + split of the
            # result; dX = dC.B^T with the ReLU-backward mask + split of the result
            bias = cb.to_device(rng.standard_normal(n).astype(np.float32))
            act = cb.to_device(np.maximum(rng.standard_normal((m, k)), 0).astype(np.float32))
            fn = (lambda: cb.ops.matmul_fused(A, B, bias=bias, relu=True, want_split=False, keep_split=True)) if which == "fwdfused" else \
                 (lambda: cb.ops.matmul_fused(dC, B, mask=act, tb=True, keep_split=True))
        work, unit = 2.0 * m * n * k, "TFLOP/s"
        if n <= 16 and which in ("fwd", "dB"):
            work, unit = 4.0 * m * k, "GB/s"   # a narrow output: the product is a pass over A's bytes
    elif kind in ("add", "relu", "sum"):
        n = 1 << int(parts[1])
        a = cb.to_device(rng.uniform(-4, 4, n).astype(np.float32)); b = cb.to_device(rng.uniform(-4, 4, n).astype(np.float32)); o = cb.empty((n,))
        fn = dict(add=lambda: cb.ops.binary("Add", a, b, out=o), relu=lambda: cb.ops.unary("ReLU", a, out=o), sum=lambda: cb.ops.sum(a))[kind]
        work, unit = dict(add=12, relu=8, sum=4)[kind] * n, "GB/s"
    elif kind in ("cmp", "cast", "rand"):
        n = 1 << int(parts[1])
        a = cb.to_device(rng.uniform(-4, 4, n).astype(np.float32)); b = cb.to_device(rng.uniform(-4, 4, n).astype(np.float32))
        ob, od, of = cb.DeviceArray((n,), np.uint8), cb.DeviceArray((n,), np.float64), cb.empty((n,))
        i64 = ctypes.c_int64
        fn = dict(cmp=lambda: cb.check(cb.lib.ctk_compare_f32(0, 0, a.p, b.p, ctypes.c_float(0), ob.p, i64(n), None)),
                  cast=lambda: cb.check(cb.lib.ctk_cast_f32(1, a.p, od.p, i64(n), None)),
                  rand=lambda: cb.check(cb.lib.ctk_rand_uniform_f32(of.p, i64(n), ctypes.c_uint64(1), ctypes.c_uint64(0), None)))[kind]
        work, unit = dict(cmp=9, cast=12, rand=4)[kind] * n, "GB/s"
    elif kind in ("sgdsplit", "colsum"):
        rows, cols = (int(v) for v in parts[1].split("x"))
        p_ = cb.to_device(rng.standard_normal((rows, cols)).astype(np.float32)); g = cb.to_device(rng.standard_normal((rows, cols)).astype(np.float32))
        split = cb.empty((int(cb.lib.ctk_matmul_split_bytes(cols, rows)) // 4,))
        i64 = ctypes.c_int64
        fn = dict(sgdsplit=lambda: cb.check(cb.lib.ctk_sgd_update_split_f32(p_.p, g.p, ctypes.c_float(1e-3), i64(rows), i64(cols), i64(cols), split.p, None)),
                  colsum=lambda: cb.ops.colsum(p_))[kind]
        work, unit = dict(sgdsplit=16, colsum=4)[kind] * rows * cols, "GB/s"   # p and g read, p and the 4-byte small terms of its split written
    elif kind == "u8":
        n = 1 << int(parts[1])
        src = cb.to_device(rng.integers(0, 256, n).astype(np.uint8), dtype=np.uint8); o = cb.empty((n,))
        fn = lambda: cb.ops.u8_to_f32(src, 255.0, out=o)
        work, unit = 5 * n, "GB/s"
    elif kind in ("softmaxcols", "argmax", "gather"):
        rows, cols = (int(v) for v in parts[1].split("x"))
        x = cb.to_device((2 * rng.standard_normal((rows, cols))).astype(np.float32)); y = cb.empty((rows, cols))
        i64 = ctypes.c_int64
        if kind == "softmaxcols":
            fn = lambda: cb.check(cb.lib.ctk_softmax_cols_f32(x.p, y.p, i64(rows), i64(cols), None))
            work = 8 * rows * cols
        elif kind == "argmax":
            out = cb.empty((rows,))
            fn = lambda: cb.check(cb.lib.ctk_argmax_rows_f32(x.p, i64(rows), i64(cols), ctypes.c_float(-1.0), out.p, None))
            work = 4 * rows * cols + 4 * rows
        else:
            # the general gather of the gradient-shape adjustment: [rows, cols] -> [rows, 1], index 0 on the dimension the target has as 1
            out = cb.empty((rows,))
            dshape = (ctypes.c_int64 * 2)(rows, 1)
            sstride = (ctypes.c_int64 * 2)(cols, 0)
            fn = lambda: cb.check(cb.lib.ctk_gather_nd_f32(x.p, out.p, 2, dshape, sstride, None))
            work = 8 * rows
        unit = "GB/s"
    elif kind in ("softmax", "ce"):
        rows, cols = (int(v) for v in parts[1].split("x"))
        x = cb.to_device((2 * rng.standard_normal((rows, cols))).astype(np.float32)); y = cb.empty((rows, cols))
        lab = cb.to_device(rng.integers(0, cols, rows).astype(np.float32))
        fn = (lambda: cb.ops.softmax(x, out=y)) if kind == "softmax" else (lambda: cb.ops.cross_entropy(x, lab))
        work, unit = (8 if kind == "softmax" else 4) * rows * cols, "GB/s"
    else:
        raise SystemExit("unknown case " + case)
    fn()
    cb.synchronize()
    e0, e1 = cb.Event(), cb.Event()
    e0.record()
    for _ in range(3):
        fn()
    e1.record()
    e1.sync()
    ms = e0.elapsed_ms(e1) / 3
    print(json.dumps(dict(case=case, ms=ms, value=work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12), unit=unit)))


def lib_binary_bwd(cb, op, a, b, g, da, db):
    cb.check(cb.lib.ctk_binary_backward_f32(cb.ops.OP[op], a.p, b.p, g.p, da.p, db.p, ctypes.c_int64(a.size), 0, ctypes.c_int64(1), None))


def lib_unary_bwd(cb, op, x, g, dx):
    cb.check(cb.lib.ctk_unary_backward_f32(cb.ops.OP[op], x.p, g.p, dx.p, ctypes.c_int64(x.size), None))


def lib_softmax_bwd(cb, y, g, rows, C):
    dx = _scratch_like(cb, y)
    cb.check(cb.lib.ctk_softmax_backward_rows_f32(y.p, g.p, dx.p, ctypes.c_int64(rows), ctypes.c_int64(C), None))


_scratch = {}


def _scratch_like(cb, t):
    key = t.size
    if key not in _scratch:
        _scratch.clear()
        _scratch[key] = cb.empty((t.size,))
    return _scratch[key]


def lib_ce_fused(cb, x, lab, d, rows, C):
    out = _scratch_like(cb, lab)
    cb.check(cb.lib.ctk_ce_fused_index_f32(x.p, lab.p, ctypes.c_int64(rows), ctypes.c_int64(C), out.p, d.p, None, None, None))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--pairing", type=int, default=0, choices=[0, 1], help="MatMul tile scheduling: 0 = CTA pairs where possible (default), 1 = single-CTA kernel only")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mlp", choices=["mlp", "mlp_small", "mnist", "elementwise", "rowwise", "matmul", "kernel"])
    ap.add_argument("--case", default="matmul_3xtf32_4096x4096x4096", help="for --workload kernel")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the single-op metrics that ride along with the default N=1 run")
    ap.add_argument("--no-checks", action="store_true", help="skip parity_check / dp_check")
    ap.add_argument("--no-comparator", action="store_true", help="skip the vendor-library TF32 GEMM timed for the roofline's `ceilings`")
    ap.add_argument("--dp-mode", default=DEFAULT_DP_MODE, choices=["inplace", "arena", "serial", "sharded"], help="how gradients cross the ranks (N > 1)")
    ap.add_argument("--max-ctas", type=int, default=DEFAULT_MAX_CTAS, help="upper bound on the CTAs of one collective (0: NCCL's choice)")
    ap.add_argument("--correction", default=DEFAULT_CORRECTION, choices=["tf32", "bf16"],
                    help="which tensor-core path carries the two correction terms of the fp32-accurate MatMul mode")
    ap.add_argument("--stable-lr", action="store_true", help="time the headline run itself at lr / batch (weights do not diverge); recorded in config")
    ap.add_argument("--nccl-algo", default=DEFAULT_NCCL_ALGO, help="NCCL_ALGO for the gradient exchange's communicator: a name, '' for NCCL's own choice, or 'auto' (NVLS from 4 ranks up, with a fall-back if a rank cannot run it)")
    ap.add_argument("--nvls-ctas", type=int, default=0, help="CTAs of a collective's in-switch part (0: NCCL's choice)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours" and args.workload == "mlp":
        args.warmup = 3  # timing rule: at least three warm-up steps

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload != "mlp":
        if rank == 0:
            run_single_op(args)
        return

    # control plane only (barrier, id broadcast, max over ranks) over gloo; gradients travel over the
    # library's own NCCL communicator
    from ctorch_b200 import dp
    cp = dp.ControlPlane(rank, world)
    try:
        run_mlp(args, cp)
    finally:
        cp.close()


if __name__ == "__main__":
    main()
