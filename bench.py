"""Benchmark of the training-step hot path: fwd + bwd + Adam steps/s of the data-parallel
wide MLP (4096 -> 8192 -> 8192 -> 4096, f32, global batch 65536, MSE, TF32 tensor-core
GEMMs) on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--precision tf32|fp32|tf32x3]

N > 1 is launched by torchrun (one process per GPU); torch.distributed (gloo) carries only
the rendezvous, barriers and the max-over-ranks of the timings, the gradients travel through
the library's own NCCL communicator.  Rank 0 prints one JSON line.

Keys beyond the base contract:
  roofline      dominant kernel (the tcgen05 GEMM): algorithmic flop / event-timed duration,
                against the measured dense peak in MEASURED_PEAKS.json (bf16/2 for TF32), with the
                vendor library's TF32 GEMM timed on the same box beside it (tf32_measured)
  cpu_baseline  the CPU oracle (a restatement of the reference's single-threaded AVX2 path)
                timed on bounded row slices of the same workload and extrapolated; `value` is
                the reference as written (with its operand copies and element-wise layout
                walks), `math_only` the same arithmetic without them
  e2e           the same step including, every step, the upload of that step's batch from
                pinned host memory and the read-back of the loss
  configs       (N = 1) short runs of the other BASELINE configurations and precisions:
                C1, C2, C3, C4, and C5 in the FP32-accurate modes
  dp_check      (N > 1) replicas bit-identical after the timed steps; the data-parallel gradient
                against the same batch on one GPU
"""
from __future__ import annotations

import argparse
import ctypes as C
import hashlib
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

DIMS = [4096, 8192, 8192, 4096]
GLOBAL_BATCH = 65536
SEED = 4
BLOCK_ROWS = 8192     # the synthetic batch is generated in blocks of rows, so that it is the same global batch for every N
METRIC = "fwd+bwd+Adam steps/s (MLP 4096-8192-8192-4096, global batch 65536)"
# DRAM bytes per flop of the tcgen05 GEMM, from an ncu capture of a 16384 x 8192 x 8192 product of the same kernel, a quarter of
# a C5 layer product (dram__bytes_read.sum + dram__bytes_write.sum = 4.64 + 0.53 GB per launch, divided by its 2.199e12 flop;
# the 8192^3 case gives the same ratio, 2.55 GB per 1.0995e12 flop, so traffic grows in proportion to the flop)
GEMM_DRAM_BYTES_PER_FLOP_8192 = 5.17e9 / 2.199e12
# Learning rates.  BASELINE.json fixes one for C1 only (1e-3, the reference's default).  On the wide networks that default
# kills the workload: Adam's first steps are sign-like, so every pre-activation of an 8192-wide layer moves by about
# 8192 * 1e-3 * E|h| = +-4 at once, and with random targets (best prediction: zero) the ReLUs of the second hidden layer
# are ALL dead after a few steps.  The step then multiplies zeros, which the tensor cores do at lower power and 11 % faster
# under the power cap (measured: 72 against 80 ms) - not the workload the metric names.  The rates below keep about
# half of every hidden layer's activations non-zero through the timed steps; each line reports the fraction it ended with.
C5_LR = 1e-6
CONFIG_LR = {"c1": 1e-3, "c3": 1e-6, "c4": 1e-4}


def flop_per_step(batch: int) -> float:
    """2*M*N*K for forward and dW of every layer, dX for every layer but the first."""
    fwd = sum(2.0 * batch * DIMS[i] * DIMS[i + 1] for i in range(3))
    dx = sum(2.0 * batch * DIMS[i] * DIMS[i + 1] for i in range(1, 3))
    return 2.0 * fwd + dx


def n_params() -> int:
    return sum(DIMS[i] * DIMS[i + 1] + DIMS[i + 1] for i in range(3))


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


def init_params(rng):
    """Kaiming-uniform weights U(-sqrt(6/fan_in), sqrt(6/fan_in)), zero biases (synthetic, seed 4)."""
    ws, bs = [], []
    for i in range(3):
        bound = np.sqrt(6.0 / DIMS[i])
        ws.append(rng.uniform(-bound, bound, (DIMS[i], DIMS[i + 1])).astype(np.float32))
        bs.append(np.zeros(DIMS[i + 1], np.float32))
    return ws, bs


class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons during the timed region (read-only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.proc, self.path = device, None, None
        self.t_begin = self.t_end = None

    def start(self):
        """Started before the warm-up (nvidia-smi needs a few hundred ms to come up); the samples used are those whose
        timestamps fall between mark_begin() and mark_end(), i.e. inside the timed region."""
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu=timestamp,{self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.device)], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def mark_begin(self):
        import datetime
        self.t_begin = datetime.datetime.now()

    def mark_end(self):
        import datetime
        self.t_end = datetime.datetime.now()

    def stop(self):
        import datetime
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "window": None}
        if not self.proc:
            return out
        self.proc.terminate()   # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        try:
            for line in open(self.path):
                c = [x.strip() for x in line.split(",")]
                if len(c) < 10:
                    continue
                try:
                    when = datetime.datetime.strptime(c[0], "%Y/%m/%d %H:%M:%S.%f")
                    rows.append((when, float(c[2]), float(c[3]), [v.lower() == "active" for v in c[6:10]]))
                except ValueError:
                    continue
            os.unlink(self.path)
        except Exception:
            pass
        inside = [r for r in rows if self.t_begin and self.t_end and self.t_begin <= r[0] <= self.t_end]
        use, out["window"] = (inside, "timed region") if inside else (rows[-25:], "last samples before the end of the timed region")
        if use:
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            reasons = sorted({n for r in use for n, a in zip(names, r[3]) if a})
            out.update(sm_mhz=float(np.median([r[1] for r in use])), sm_max_mhz=float(max(r[2] for r in use)),
                       reasons=reasons, samples=len(use))
        return out


class Dist:
    """Rendezvous and host-side reductions for N > 1 (torch.distributed, gloo backend)."""

    def __init__(self, n_gpus: int):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            import torch.distributed as dist
            dist.init_process_group(backend="gloo", rank=self.rank, world_size=self.world)
            self.dist = dist
        if n_gpus != self.world:
            raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE is {self.world}: launch N > 1 with torch.distributed.run")

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def max(self, v: float) -> float:
        if not self.dist:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t[0])

    def sum(self, v: float) -> float:
        if not self.dist:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t[0])

    def close(self):
        if self.dist:
            self.dist.destroy_process_group()


# ------------------------------------------------------------------------ CPU arm
def batch_rows(r0: int, r1: int):
    """Rows [r0, r1) of the synthetic global batch (inputs and targets ~ N(0,1)).  Generated block by block with
    one seed per block, so every world size trains on the same 65536 rows."""
    xs, ts_ = [], []
    for blk in range(r0 // BLOCK_ROWS, (r1 + BLOCK_ROWS - 1) // BLOCK_ROWS):
        rng = np.random.default_rng([SEED, 1, blk])
        x = rng.standard_normal((BLOCK_ROWS, DIMS[0]), dtype=np.float32)
        t = rng.standard_normal((BLOCK_ROWS, DIMS[-1]), dtype=np.float32)
        lo, hi = max(r0, blk * BLOCK_ROWS) - blk * BLOCK_ROWS, min(r1, (blk + 1) * BLOCK_ROWS) - blk * BLOCK_ROWS
        xs.append(x[lo:hi]); ts_.append(t[lo:hi])
    return np.concatenate(xs), np.concatenate(ts_)


def _cpu_step(ora, ws, bs, x, t, loss_kind, relu_last, want_gx, rows, as_written):
    kind = {"sum": ora.LOSS_SUM, "mean": ora.LOSS_MEAN, "mse": ora.LOSS_MSE}[loss_kind]
    st = ora.MlpState(ws, bs)
    t0 = time.perf_counter()
    ora.mlp_step(st, x[:rows], None if t is None else t[:rows], loss_kind=kind, relu_last=relu_last, do_adam=False,
                 want_gx=want_gx, as_written=as_written)
    return time.perf_counter() - t0, st


def cpu_baseline_for(ws, bs, x, t, loss_kind, relu_last, want_gx, batch, sample_rows, what):
    """Both CPU figures for one configuration: the reference as written and its arithmetic alone, one thread (the
    reference is single-threaded, tensor/ops/matmul/mod.rs:3-4), plus one full Adam update.

    With sample_rows < batch the step is timed on that many rows (a whole number of the reference's 128-row GEMM
    blocks) and the arithmetic is scaled by rows.  What the reference does around the arithmetic has a part that does
    not grow with the batch (deep copies and element-by-element transposes of the WEIGHTS), which a one-row step
    isolates, and a part that does (the same for activations and gradients); each is extended separately."""
    ora = entry.load_oracle()
    args = (ora, ws, bs, x, t, loss_kind, relu_last, want_gx)
    t_m, st = _cpu_step(*args, sample_rows, False)
    t_w, _ = _cpu_step(*args, sample_rows, True)
    spent = t_m + t_w
    if sample_rows < batch:
        t_m1, _ = _cpu_step(*args, 1, False)
        t_w1, _ = _cpu_step(*args, 1, True)
        spent += t_m1 + t_w1
        fixed = max(t_w1 - t_m1, 0.0)
        per_row_extra = max((t_w - t_m - fixed) / sample_rows, 0.0)
        sec_m = t_m * batch / sample_rows
        sec_w = sec_m + fixed + per_row_extra * batch
        how = (f"fwd+bwd on {sample_rows} of {batch} batch rows, arithmetic scaled by rows; the reference's copies and layout walks "
               f"split into a per-step part ({fixed:.1f} s, from a one-row step) and a per-row part")
    else:
        sec_m, sec_w, how = t_m, t_w, f"fwd+bwd on all {batch} rows"
    t0 = time.perf_counter()
    for l in range(len(ws)):
        ora.adam_update(st.w[l].reshape(-1), st.gw[l].reshape(-1), st.mw[l].reshape(-1), st.vw[l].reshape(-1), 1)
        ora.adam_update(st.b[l], st.gb[l], st.mb[l], st.vb[l], 1)
    t_adam = time.perf_counter() - t0
    return {"value": 1.0 / (sec_w + t_adam), "unit": "steps/s", "cores": 1, "kind": "port", "cpu_model": host_cpu_model(),
            "math_only": 1.0 / (sec_m + t_adam),
            "sample": f"{what}: {how} ({spent:.1f} s of CPU time) + one full Adam ({t_adam:.2f} s); `value` is the reference as written "
                      f"(operand deep copies, element-by-element broadcast of the bias, coordinate-walk transposes), `math_only` its "
                      f"arithmetic alone"}


def host_cpu_model() -> str:
    """The host CPU the one-thread baseline ran on (first `model name` of /proc/cpuinfo)."""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.lower().startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def cpu_baseline(sample_rows: int = 128):
    """The C5 step on the CPU oracle."""
    rng = np.random.default_rng(SEED)
    ws, bs = init_params(rng)
    x, t = batch_rows(0, sample_rows)
    return cpu_baseline_for(ws, bs, x, t, "mse", False, False, GLOBAL_BATCH, sample_rows, "C5")


def run_reference(args, d: Dist):
    if d.rank != 0:
        return
    vals = []
    for _ in range(max(1, min(args.steps, 2))):
        vals.append(cpu_baseline())
    base = vals[-1]
    v = float(np.median([b["value"] for b in vals]))
    base["value"] = v
    line = {"metric": METRIC, "value": v, "unit": "steps/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 / v, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "impl": "reference",
            "config": {"workload": "C5 data-parallel wide MLP 4096-8192-8192-4096 f32, Kaiming-uniform init, ReLU, MSE, Adam",
                       "global_batch": GLOBAL_BATCH, "seed": SEED,
                       "note": "the reference is single-threaded CPU code with no multi-device path; timed on one host core"},
            "cpu_baseline": base, "e2e": {"value": v, "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------ GPU arm
def _prof(lib, cls):
    n, t, w = C.c_ulonglong(), C.c_double(), C.c_double()
    lib.ts_profile_get(cls, C.byref(n), C.byref(t), C.byref(w))
    return int(n.value), float(t.value), float(w.value)


def library_tf32_yardstick(m=8192, burst_reps=10, seconds=2.0):
    """Not the product path: the vendor library's TF32 GEMM (torch.matmul on f32 with TF32 allowed) on 8192^3, timed on
    this box as a measured stand-in for the TF32 tensor-pipe peak (the driver-written peaks file holds bf16 only).
    Best single launch (burst) and back-to-back for about two seconds (sustained, under the power cap)."""
    import torch
    torch.backends.cuda.matmul.allow_tf32 = True
    dev = torch.device("cuda", torch.cuda.current_device())
    a, b = torch.randn(m, m, device=dev), torch.randn(m, m, device=dev)
    c = torch.empty(m, m, device=dev)
    for _ in range(3):
        torch.matmul(a, b, out=c)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(burst_reps):
        e0.record(); torch.matmul(a, b, out=c); e1.record(); torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    reps = max(20, int(seconds * 1e3 / best))
    e0.record()
    for _ in range(reps):
        torch.matmul(a, b, out=c)
    e1.record(); torch.cuda.synchronize()
    flop = 2.0 * m ** 3
    out = {"library": "torch.matmul f32, allow_tf32 (cuBLAS)", "case": f"{m}^3", "burst": flop / (best * 1e-3) / 1e12,
           "sustained": flop / (e0.elapsed_time(e1) / reps * 1e-3) / 1e12, "sustained_launches": reps, "unit": "TFLOP/s"}
    del a, b, c
    torch.cuda.empty_cache()
    return out


def run_gpu(args, d: Dist):
    ts = entry.load_package()
    lib = ts._ffi.lib()
    ts.set_default_device(d.local_rank)
    prec = {"tf32": ts.TF32, "fp32": ts.FP32, "tf32x3": ts.TF32X3}[args.precision]
    ts.set_matmul_precision(prec)
    if d.world > 1:
        ids = [ts.distributed.get_unique_id() if d.rank == 0 else None]
        d.dist.broadcast_object_list(ids, src=0)
        ts.distributed.init(ids[0], d.rank, d.world)

    r0, r1 = ts.distributed.shard_rows(GLOBAL_BATCH, d.rank, d.world)
    local = r1 - r0
    rng = np.random.default_rng(SEED)
    ws, bs = init_params(rng)                      # identical on every rank
    W = [ts.Tensor.from_slice(w, w.shape).with_requires_grad() for w in ws]
    B = [ts.Tensor.from_slice(b, b.shape).with_requires_grad() for b in bs]
    del ws, bs
    params = [p for pair in zip(W, B) for p in pair]
    opt = ts.Adam.with_learning_rate(args.lr)
    opt.add_parameters(params)
    if d.world > 1:
        ts.distributed.register_parameters(params)
        # per-rank mean losses -> gradient of the global mean
        assert GLOBAL_BATCH % d.world == 0, "equal shards: a rank's mean loss then weighs 1/world in the global mean"
        opt.grad_scale = 1.0 / d.world

    # this rank's rows of the synthetic batch, in pinned host memory (two slots for the prefetching e2e loop)
    pins_x = [ts.PinnedBuffer(local * DIMS[0]) for _ in range(2)]
    pins_t = [ts.PinnedBuffer(local * DIMS[-1]) for _ in range(2)]
    hx, ht = batch_rows(r0, r1)
    for px, pt in zip(pins_x, pins_t):
        px.array[:] = hx.reshape(-1)
        pt.array[:] = ht.reshape(-1)
    del hx, ht

    def forward(X, T):
        h = X
        for i in range(3):
            h = h.matmul(W[i]).add_tensor(B[i])
            if i < 2:
                h = h.relu()
        return h.sub_tensor(T).pow_scalar(2.0).mean()

    def step(X, T):
        loss = forward(X, T)
        loss.backward(None)
        opt.step(params)
        opt.zero_grad(params)
        return loss

    X = ts.Tensor.from_pinned_async(pins_x[0], [local, DIMS[0]])
    T = ts.Tensor.from_pinned_async(pins_t[0], [local, DIMS[-1]])

    sampler = ClockSampler(d.local_rank)
    sampler.start()
    for _ in range(args.warmup):
        loss = step(X, T)
    ts.synchronize()

    # ---- timed region 1: inputs resident in HBM
    ev0, ev1 = lib.ts_event_create(), lib.ts_event_create()
    lib.ts_profile_reset()
    lib.ts_profile_enable(1)
    d.barrier(); ts.synchronize()
    sampler.mark_begin()
    launches0 = int(lib.ts_launch_count())
    lib.ts_event_record(ev0, None)
    for _ in range(args.steps):
        loss = step(X, T)
    lib.ts_event_record(ev1, None)
    ts.synchronize(); d.barrier()
    sampler.mark_end()
    ms = float(lib.ts_event_elapsed_ms(ev0, ev1))
    launches = int(lib.ts_launch_count()) - launches0
    clocks = sampler.stop()
    lib.ts_profile_enable(0)
    ts._ffi.check(lib.ts_profile_collect(), "profile")
    final_loss = loss.value()
    ms = d.max(ms)
    ms_per_step = ms / args.steps
    value = 1000.0 / ms_per_step

    peaks = measured_peaks()
    cls = 1 if prec == ts.FP32 else 0
    gl, gms, gwork = _prof(lib, cls)
    # no TF32 entry is measured: half the measured sustained bf16 rate (a sixth for the three sweeps of 3xTF32)
    tf32_peak = peaks["bf16_sustained"] / (6.0 if prec == ts.TF32X3 else 2.0)
    roof = {"bound": "tensor", "kernel": "gemm_tf32_2cta_kernel / gemm_tf32_kernel (tcgen05)" if cls == 0 else "sgemm_kernel (FFMA)",
            "achieved": (gwork / (gms * 1e-3) / 1e12) if gms > 0 else None, "peak": tf32_peak, "unit": "TFLOP/s",
            "frac": None, "traffic": None, "launches": gl, "avg_launch_ms": gms / gl if gl else None,
            "peak_source": f"{peaks['source']}: bf16_tflops_sustained / 2 (derived; TF32 runs at half the bf16 rate)",
            "share_of_step": gms / ms if ms > 0 else None}
    if roof["achieved"]:
        roof["frac"] = roof["achieved"] / roof["peak"]
    if cls == 0 and gl:
        roof["traffic"] = GEMM_DRAM_BYTES_PER_FLOP_8192 * (gwork / gl)
        roof["traffic_note"] = ("scaled, not measured in this run: DRAM bytes per flop from an ncu capture of a 16384 x 8192 x 8192 "
                                "product of the same kernel (dram__bytes_read.sum + dram__bytes_write.sum = 5.17 GB for 2.199e12 flop; "
                                "8192^3 gives the same ratio) times the flop of an average launch here; the bench's own GEMMs are too "
                                "large to capture under ncu; algorithmic bytes (operands and result once) are about a quarter of it")
    al, ams, awork = _prof(lib, 4)
    el, ems, ework = _prof(lib, 2)
    rl, rms, rwork = _prof(lib, 3)
    other = {"adam": {"launches": al, "GBps": awork / (ams * 1e-3) / 1e9 if ams > 0 else None, "frac_of_hbm": None,
                      "ms_per_step": ams / args.steps},
             "elementwise": {"launches": el, "GBps": ework / (ems * 1e-3) / 1e9 if ems > 0 else None, "ms_per_step": ems / args.steps},
             "reduce": {"launches": rl, "GBps": rwork / (rms * 1e-3) / 1e9 if rms > 0 else None, "ms_per_step": rms / args.steps},
             "hbm_peak_GBps": peaks["hbm_gbs"]}
    if other["adam"]["GBps"]:
        other["adam"]["frac_of_hbm"] = other["adam"]["GBps"] / peaks["hbm_gbs"]

    # ---- timed region 2: end to end, each step's batch uploaded from pinned memory, loss read back
    h2d = 4 * local * (DIMS[0] + DIMS[-1])
    d.barrier(); ts.synchronize()
    t0 = time.perf_counter()
    prev = None
    lib.ts_event_record(ev0, None)
    # every step's upload lies inside the timed region, the first one included (nothing hides it); from then on the
    # upload of step s + 1 is issued before step s is enqueued and runs on the copy stream beside it
    nxt = (ts.Tensor.from_pinned_async(pins_x[1], [local, DIMS[0]]), ts.Tensor.from_pinned_async(pins_t[1], [local, DIMS[-1]]))
    for s in range(args.steps):
        cur = nxt
        slot = s % 2   # the slot the step before last used is free again: its upload has been consumed
        if s + 1 < args.steps:
            nxt = (ts.Tensor.from_pinned_async(pins_x[slot], [local, DIMS[0]]),
                   ts.Tensor.from_pinned_async(pins_t[slot], [local, DIMS[-1]]))
        l = step(*cur)
        # device -> host read of every step's loss, one step behind: the next step is already queued while the host
        # waits for this value, so the GPU never idles on the read-back
        if prev is not None:
            _ = prev.value()
        prev = l
    _ = prev.value()
    lib.ts_event_record(ev1, None)
    ts.synchronize(); d.barrier()
    e2e_ms = d.max(float(lib.ts_event_elapsed_ms(ev0, ev1)))
    e2e = {"value": 1000.0 * args.steps / e2e_ms, "unit": "steps/s", "h2d_bytes_per_step": h2d * d.world,
           "d2h_bytes_per_step": 4 * d.world, "wall_ms_per_step_rank0": 1000.0 * (time.perf_counter() - t0) / args.steps}
    del cur, nxt, prev, l

    # ---- host side of the uploads: what one rank gets alone and what every rank gets when all upload at once
    def upload_GBps():
        dst = ts.Tensor.new([local, DIMS[0]])
        ptr = dst.data_ptr()
        lib.ts_event_record(ev0, None)
        for _ in range(3):
            ts._ffi.check(lib.ts_memcpy_async(ptr, pins_x[0].ptr, local * DIMS[0], 0, None), "upload")
        lib.ts_event_record(ev1, None)
        ts.synchronize()
        return 3 * 4.0 * local * DIMS[0] / (float(lib.ts_event_elapsed_ms(ev0, ev1)) * 1e-3) / 1e9
    d.barrier()
    together = upload_GBps()
    d.barrier()
    alone = upload_GBps() if d.rank == 0 else 0.0
    d.barrier()
    e2e["h2d_GBps"] = {"rank0_alone": alone if d.rank == 0 else None, "per_rank_all_together_min": -d.max(-together),
                       "aggregate_all_together": d.sum(together),
                       "note": "pinned host memory to HBM, 3 copies of this rank's input shard back to back"}

    # Are the hidden layers alive?  A network whose ReLUs have all died computes on zeros, which the tensor cores do at
    # lower power (and therefore higher clocks) than on real data: the fraction of non-zero hidden activations on the
    # first rows of the batch says whether the timed steps were representative.
    with ts.NoGradTrack():
        rows = min(512, local)
        hh = ts.Tensor.from_slice(np.array(pins_x[0].array[:rows * DIMS[0]]).reshape(rows, DIMS[0]), [rows, DIMS[0]])
        alive = []
        for i in range(2):
            hh = hh.matmul(W[i]).add_tensor(B[i]).relu()
            alive.append(float((hh.data() > 0).mean()))
        del hh

    stats = ts.allocator_stats()
    line = {"metric": METRIC, "value": value, "unit": "steps/s", "n_gpus": d.world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": args.precision if prec != ts.FP32 else "f32", "data": "synthetic",
            "config": {"workload": "C5 data-parallel wide MLP 4096-8192-8192-4096 f32, Kaiming-uniform init, ReLU, MSE, Adam",
                       "global_batch": GLOBAL_BATCH, "rows_per_gpu": local, "parallelism": f"dp{d.world}", "seed": SEED, "adam_lr": args.lr,
                       "gemm_precision": args.precision, "l2": "inputs and activations (>= 1 GiB each) are larger than the 126 MB L2",
                       "allreduce": ts.distributed.describe() if d.world > 1 else "none"},
            "tflops_per_gpu": flop_per_step(local) / (ms_per_step * 1e-3) / 1e12,
            "tflops_total": flop_per_step(GLOBAL_BATCH) / (ms_per_step * 1e-3) / 1e12,
            "loss": final_loss, "hidden_nonzero_fraction": alive, "roofline": roof, "other_kernels": other, "e2e": e2e, "gpu_launches": launches,
            "launches_per_step": launches / args.steps, "clocks": clocks, "peak_device_bytes": stats["peak_bytes_in_use"]}

    if d.world > 1 and not args.no_dp_check:
        line["dp_check"] = dp_check(ts, d, W, B, params, forward, X, T)
    if d.world == 1 and not args.no_extras:
        extras = {}
        # C5 in the two FP32-accurate modes, on the tensors already resident
        for name, mode, n_steps in (("c5_tf32x3", ts.TF32X3, 3), ("c5_fp32", ts.FP32, 2)):
            if mode == prec:
                continue
            ts.set_matmul_precision(mode)
            extras[name] = _timed_steps(ts, lib, lambda: step(X, T), 1, n_steps, mode, flop_per_step(local), peaks)
        ts.set_matmul_precision(prec)
    del X, T, W, B, params, opt, pins_x, pins_t
    ts.clear_gradients()
    ts.release_cached_memory()
    if d.world == 1 and not args.no_extras:
        for cfg, precs in (("c1", ("fp32", "tf32")), ("c4", ("tf32", "fp32")), ("c3", ("tf32", "tf32x3", "fp32"))):
            for pname in precs:
                extras[f"{cfg}_{pname}"] = run_config(cfg, pname, steps={"c1": 200, "c4": 100, "c3": 5}[cfg], warmup=3,
                                                      with_cpu=(pname == precs[0]), compact=True)
                ts.release_cached_memory()
        extras["c2"] = run_c2(steps=5, warmup=2, sizes=(20, 24, 28), compact=True)
        ts.release_cached_memory()
        line["configs"] = extras
        try:
            y = library_tf32_yardstick()
            line["roofline"]["tf32_measured"] = y
            if roof["achieved"] and cls == 0:
                line["roofline"]["frac_of_tf32_measured_sustained"] = roof["achieved"] / y["sustained"] / (3.0 if prec == ts.TF32X3 else 1.0)
        except Exception as exc:   # the yardstick is context, never a reason to lose the line
            line["roofline"]["tf32_measured"] = {"unavailable": repr(exc)[:200]}
    if d.rank == 0:
        if d.world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line), flush=True)
    if d.world > 1:
        ts.distributed.finalize()


def _timed_steps(ts, lib, step_fn, warmup, steps, mode, flop, peaks):
    """`steps` calls of step_fn between two events: a compact record.  The step time comes from a first pass without
    instrumentation; a second pass of the same length brackets every GEMM launch with events for the GEMM rate and its
    share of that pass (on steps of a few hundred microseconds the brackets themselves cost several per cent)."""
    for _ in range(warmup):
        step_fn()
    ts.synchronize()
    ev0, ev1 = lib.ts_event_create(), lib.ts_event_create()
    launches0 = int(lib.ts_launch_count())
    lib.ts_event_record(ev0, None)
    for _ in range(steps):
        out = step_fn()
    lib.ts_event_record(ev1, None)
    ts.synchronize()
    ms = float(lib.ts_event_elapsed_ms(ev0, ev1)) / steps
    launches = int(lib.ts_launch_count()) - launches0
    lib.ts_profile_reset(); lib.ts_profile_enable(1)
    lib.ts_event_record(ev0, None)
    for _ in range(steps):
        out = step_fn()
    lib.ts_event_record(ev1, None)
    ts.synchronize()
    ms_profiled = float(lib.ts_event_elapsed_ms(ev0, ev1)) / steps
    lib.ts_profile_enable(0)
    ts._ffi.check(lib.ts_profile_collect(), "profile")
    tc_n, tc_ms, tc_w = _prof(lib, 0)
    fp_n, fp_ms, fp_w = _prof(lib, 1)
    peak = {ts.TF32: peaks["bf16_sustained"] / 2, ts.TF32X3: peaks["bf16_sustained"] / 6, ts.FP32: None}[mode]
    gemm_ms, gemm_w = tc_ms + fp_ms, tc_w + fp_w
    rec = {"steps": steps, "ms_per_step": ms, "steps_per_s": 1000.0 / ms, "step_tflops": flop / (ms * 1e-3) / 1e12,
           "gemm_tflops": gemm_w / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None,
           "gemm_launches": {"tensor_core": tc_n, "fp32": fp_n}, "gemm_share_of_step": gemm_ms / (ms_profiled * steps) if ms_profiled > 0 else None,
           "ms_per_step_with_gemm_brackets": ms_profiled,
           "launches_per_step": launches / steps, "peak_tflops": peak, "frac": None}
    if tc_ms > 0 and peak:
        rec["frac"] = tc_w / (tc_ms * 1e-3) / 1e12 / peak      # tensor-core launches only, against the derived peak
    try:
        rec["loss"] = out.value()
    except Exception:
        pass
    return rec


def dp_check(ts, d: Dist, W, B, params, forward, X, T):
    """After the timed steps: (1) every rank holds bit-identical parameters; (2) the data-parallel gradient of the first
    layer's weights (sum over ranks of the shard gradients, times 1/world) equals, within TF32 rounding, the gradient one
    GPU computes on the whole batch with the same parameters."""
    out = {}
    h = hashlib.blake2b(digest_size=16)
    for p in params:
        h.update(p.data().tobytes())
    digests = [None] * d.world
    d.dist.all_gather_object(digests, h.hexdigest())
    out["replicas_identical"] = len(set(digests)) == 1
    loss = forward(X, T)
    loss.backward(None)
    g_dp = W[0].grad_by_value().data().astype(np.float64) * (1.0 / d.world)
    shard_loss = loss.value()
    ts.clear_gradients()
    out["loss_mean_over_shards"] = d.sum(shard_loss) / d.world
    d.barrier()
    err = None
    if d.rank == 0:
        try:
            ts.distributed.register_parameters([])      # nothing registered: this backward runs no collective
            hx, ht = batch_rows(0, GLOBAL_BATCH)
            Xf, Tf = ts.Tensor.from_slice(hx, hx.shape), ts.Tensor.from_slice(ht, ht.shape)
            del hx, ht
            lf = forward(Xf, Tf)
            lf.backward(None)
            g1 = W[0].grad_by_value().data().astype(np.float64)
            out["loss_single_gpu"] = lf.value()
            out["grad_w1_rel_diff_vs_single_gpu"] = float(np.linalg.norm(g_dp - g1) / np.linalg.norm(g1))
            ts.clear_gradients()
            del Xf, Tf, lf
        except Exception as exc:
            err = repr(exc)[:300]
        finally:
            ts.distributed.register_parameters(params)
    d.barrier()
    if err:
        out["error"] = err
    return out


# ------------------------------------------------------------------------ the smaller BASELINE configurations
CONFIGS = {
    # name: (layer dims, batch, loss, relu after last layer, input requires grad, description)
    "c1": ([784, 128], 32, "sum", True, False, "C1 README step: y = relu(x.w + b), loss = sum(y), Adam; x[32,784], w[784,128]; seed 0"),
    "c3": ([8192, 8192], 8192, "mean", True, True, "C3 dense layer 8192^3: Y = relu(X.W + b), loss = mean(Y), dX dW db, Adam; seed 2"),
    "c4": ([784, 1024, 1024, 10], 4096, "mse", False, False, "C4 MLP 784-1024-1024-10, batch 4096, one-hot targets, MSE, Adam; seed 3"),
}


def _config_inputs(name):
    dims, batch, loss_kind, relu_last, x_grad, desc = CONFIGS[name]
    seed = {"c1": 0, "c3": 2, "c4": 3}[name]
    rng = np.random.default_rng(seed)
    L = len(dims) - 1
    if name == "c1":
        ws = [rng.standard_normal((dims[0], dims[1]), dtype=np.float32)]
    elif name == "c3":
        ws = [(rng.standard_normal((dims[0], dims[1]), dtype=np.float32) * np.float32(np.sqrt(1.0 / dims[0]))).astype(np.float32)]   # variance 1/8192
    else:
        ws = [rng.uniform(-np.sqrt(6 / dims[i]), np.sqrt(6 / dims[i]), (dims[i], dims[i + 1])).astype(np.float32) for i in range(L)]
    bs = [np.zeros(dims[i + 1], np.float32) for i in range(L)]
    x = rng.standard_normal((batch, dims[0]), dtype=np.float32)
    t = np.eye(dims[-1], dtype=np.float32)[rng.integers(0, dims[-1], batch)] if loss_kind == "mse" else None
    return ws, bs, x, t, seed


def run_config(name, precision, steps, warmup, with_cpu=True, compact=False):
    """One of the single-GPU configurations C1, C3, C4 through the public API: steps/s, GEMM rate, CPU port beside it."""
    dims, batch, loss_kind, relu_last, x_grad, desc = CONFIGS[name]
    ws, bs, x, t, seed = _config_inputs(name)
    L = len(dims) - 1
    ts = entry.load_package()
    lib = ts._ffi.lib()
    ts.set_default_device(0)
    prec = {"tf32": ts.TF32, "fp32": ts.FP32, "tf32x3": ts.TF32X3}[precision]
    ts.set_matmul_precision(prec)

    W = [ts.Tensor.from_slice(w, w.shape).with_requires_grad() for w in ws]
    B = [ts.Tensor.from_slice(b, b.shape).with_requires_grad() for b in bs]
    params = [p for pair in zip(W, B) for p in pair]
    opt = ts.Adam.with_learning_rate(CONFIG_LR[name])
    opt.add_parameters(params)
    pin_x = ts.PinnedBuffer(x.size); pin_x.array[:] = x.reshape(-1)
    pin_t = None
    if t is not None:
        pin_t = ts.PinnedBuffer(t.size); pin_t.array[:] = t.reshape(-1)

    def upload():
        X = ts.Tensor.from_pinned_async(pin_x, x.shape)
        if x_grad:
            X = X.with_requires_grad()
        return X, (ts.Tensor.from_pinned_async(pin_t, t.shape) if pin_t else None)

    def step(X, T):
        h = X
        for i in range(L):
            h = h.matmul(W[i]).add_tensor(B[i])
            if i + 1 < L or relu_last:
                h = h.relu()
        loss = h.sum() if loss_kind == "sum" else h.mean() if loss_kind == "mean" else h.sub_tensor(T).pow_scalar(2.0).mean()
        loss.backward(None)
        opt.step(params)
        opt.zero_grad(params)
        return loss

    flop = 0.0
    for i in range(L):
        mnk = 2.0 * batch * dims[i] * dims[i + 1]
        flop += 2 * mnk + (mnk if (i > 0 or x_grad) else 0.0)
    peaks = measured_peaks()
    X, T = upload()
    sampler = ClockSampler(0)
    if not compact:
        sampler.start()
    sampler.mark_begin()
    rec = _timed_steps(ts, lib, lambda: step(X, T), warmup, steps, prec, flop, peaks)
    sampler.mark_end()
    clocks = sampler.stop() if not compact else None
    # end to end: every step's inputs uploaded from pinned memory (the upload of step s + 1 is issued before step s is
    # enqueued and runs on the copy stream beside it; the first one is exposed), every step's loss read back one step
    # behind the queue.  A few untimed steps first, so that the allocator already holds the blocks this loop cycles through.
    prefetch = 4 * (x.size + (t.size if t is not None else 0)) >= (1 << 20)   # a 100 KB batch is cheaper to upload in line

    def e2e_loop(count):
        nxt, prev = (upload() if prefetch else None), None
        for s in range(count):
            cur = nxt if prefetch else upload()
            if prefetch and s + 1 < count:
                nxt = upload()
            l = step(*cur)
            if prev is not None:
                _ = prev.value()
            prev = l
        _ = prev.value()
    e2e_loop(min(3, steps))
    ts.synchronize()
    ev0, ev1 = lib.ts_event_create(), lib.ts_event_create()
    lib.ts_event_record(ev0, None)
    e2e_loop(steps)
    lib.ts_event_record(ev1, None)
    ts.synchronize()
    e2e_ms = float(lib.ts_event_elapsed_ms(ev0, ev1)) / steps
    h2d = 4 * (x.size + (t.size if t is not None else 0))
    rec["e2e_steps_per_s"] = 1000.0 / e2e_ms
    rec["precision"] = precision
    rec["adam_lr"] = CONFIG_LR[name]
    with ts.NoGradTrack():      # fraction of non-zero activations per ReLU layer on the first rows, after the timed steps
        rows = min(512, batch)
        hh = ts.Tensor.from_slice(x[:rows], [rows, dims[0]])
        alive = []
        for i in range(L):
            hh = hh.matmul(W[i]).add_tensor(B[i])
            if i + 1 < L or relu_last:
                hh = hh.relu()
                alive.append(round(float((hh.data() > 0).mean()), 4))
        del hh
    rec["relu_nonzero_fraction"] = alive
    cpu = None
    if with_cpu:
        # CPU port: the full step where that takes seconds, a 64-row slice for the 8192^3 layer
        cpu = cpu_baseline_for(ws, bs, x, t, loss_kind, relu_last, x_grad, batch, 64 if name == "c3" else batch, name.upper())
    del X, T, W, B, params, opt, pin_x, pin_t
    ts.clear_gradients()
    if compact:
        if cpu:
            rec["cpu_steps_per_s"] = {"as_written": cpu["value"], "math_only": cpu["math_only"], "cores": 1}
        return rec
    return {"metric": f"fwd+bwd+Adam steps/s ({name.upper()})", "value": rec["steps_per_s"], "unit": "steps/s", "n_gpus": 1,
            "steps": steps, "warmup": warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "none",
            "vs_baseline": None, "dtype": precision, "data": "synthetic",
            "config": {"workload": desc, "gemm_precision": precision, "seed": seed},
            "tflops": rec["step_tflops"], "loss": rec.get("loss"),
            "roofline": {"bound": "tensor" if prec != ts.FP32 else "fp32 pipe", "achieved": rec["gemm_tflops"], "peak": rec["peak_tflops"],
                         "unit": "TFLOP/s", "frac": rec["frac"], "traffic": None, "launches": rec["gemm_launches"],
                         "share_of_step": rec["gemm_share_of_step"],
                         "note": "achieved covers every GEMM of the step; frac is the tensor-core launches alone against the derived "
                                 "peak; GEMMs the tensor-core kernel cannot take run on the FP32 kernel"},
            "e2e": {"value": 1000.0 / e2e_ms, "unit": "steps/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": int(round(rec["launches_per_step"] * steps)), "launches_per_step": rec["launches_per_step"], "clocks": clocks,
            "cpu_baseline": cpu}


def run_c2(steps, warmup, sizes=(20, 24, 28), compact=False):
    """C2: add/sub/mul/div of two f32 tensors (a ~ N(0,1), b ~ U[0.5,2)), loss = sum(out), backward to both operands.
    Reports achieved GB/s of the whole forward+backward sequence per op and size against its algorithmic bytes."""
    ts = entry.load_package()
    lib = ts._ffi.lib()
    ts.set_default_device(0)
    peaks = measured_peaks()
    rng = np.random.default_rng(1)
    base_a = rng.standard_normal(1 << 24, dtype=np.float32)
    base_b = (rng.random(1 << 24, dtype=np.float32) * 1.5 + 0.5).astype(np.float32)
    out = []
    for logn in sizes:
        n = 1 << logn
        # larger sizes repeat a 2^24-element block of the random data: the kernels' speed does not depend on the values
        ha = np.tile(base_a, n >> 24) if logn > 24 else base_a[:n]
        hb = np.tile(base_b, n >> 24) if logn > 24 else base_b[:n]
        a = ts.Tensor.from_slice(ha, [n]).with_requires_grad()
        b = ts.Tensor.from_slice(hb, [n]).with_requires_grad()
        del ha, hb
        for op, bwd_bytes in (("add", 0), ("sub", 8), ("mul", 20), ("div", 20)):
            # forward 12 B/elem, sum 4, seed fill 4 (written once, then read by the op's backward where it has one)
            algo = (12 + 4 + 4 + bwd_bytes) * n

            def once():
                o = getattr(a, f"{op}_tensor")(b)
                o.sum().backward(None)
                ts.clear_gradients()
            for _ in range(warmup):
                once()
            ts.synchronize()
            ev0, ev1 = lib.ts_event_create(), lib.ts_event_create()
            lib.ts_event_record(ev0, None)
            for _ in range(steps):
                once()
            lib.ts_event_record(ev1, None)
            ts.synchronize()
            ms = float(lib.ts_event_elapsed_ms(ev0, ev1)) / steps
            out.append({"op": op, "n": n, "ms": ms, "GBps": algo / (ms * 1e-3) / 1e9, "frac_of_hbm": algo / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]})
        del a, b
        ts.release_cached_memory()
    big = [r for r in out if r["n"] == 1 << max(sizes)]
    if compact:
        return {"metric": "elementwise fwd+bwd HBM GB/s of algorithmic bytes", "hbm_peak_GBps": peaks["hbm_gbs"],
                "results": [{k: (round(v, 4) if isinstance(v, float) else v) for k, v in r.items()} for r in out]}
    return {"metric": "elementwise fwd+bwd HBM GB/s (C2)", "value": float(np.mean([r["GBps"] for r in big])), "unit": "GB/s",
            "n_gpus": 1, "steps": steps, "warmup": warmup, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "C2 elementwise sweep 2^20/2^24/2^28, out = op(a,b), loss = sum(out), backward; seed 1",
                       "bytes": "algorithmic: forward 12 B/elem, sum 4, seed fill 4, backward 0 (add: gradients alias), 8 (sub), 20 (mul, div)"},
            "roofline": {"bound": "hbm", "peak": peaks["hbm_gbs"], "unit": "GB/s", "peak_source": peaks["source"]},
            "results": out}


# ------------------------------------------------------------------------ single-kernel cases
MICRO_CASES = ("gemm_nn", "gemm_nt", "gemm_tn", "gemm_nn_fp32", "gemm_nt_fp32", "gemm_tn_fp32", "gemm_nn_tf32x3", "adam", "add", "mul_backward", "relu_backward_colsum",
               "colsum", "sum", "fill", "library_tf32", "exp", "tanh", "sigmoid", "sigmoid_backward", "softmax_rows", "softmax_classes",
               "softmax_inner", "transpose", "permute_021", "permute_gather", "reduce_rows", "reduce_cols", "reduce_all_max",
               "reduce_middle", "broadcast_row", "broadcast_col", "broadcast_outer", "broadcast_mul_backward",
               "matmul_batched_fp32", "matmul_batched_tf32")


def run_micro(args):
    """One kernel on a case that is larger than L2 but holds about a gigabyte on the device: the
    case the ncu captures under profiles/ are taken on, and a quick per-kernel roofline check."""
    ts = entry.load_package()
    lib, chk = ts._ffi.lib(), ts._ffi.check
    ts.set_default_device(0)
    rng = np.random.default_rng(0)
    peaks = measured_peaks()
    vp = C.c_void_p

    def dev(a):
        a = np.ascontiguousarray(a, np.float32)
        p = lib.cuda_malloc(a.size)
        chk(p, "cuda_malloc")
        chk(lib.cuda_memcpy(p, a.ctypes.data, a.size, 0), "upload")
        return p

    def empty(n):
        p = lib.cuda_malloc(n)
        chk(p, "cuda_malloc")
        return p

    name, n = args.micro, args.micro_size
    if name == "library_tf32":
        # Yardstick, not the product path: the vendor library's TF32 GEMM on the same 8192^3 case, timed the same way,
        # as a measured stand-in for the TF32 tensor-pipe peak (the driver-written peaks file holds bf16 only).
        import torch
        m = n or 8192
        torch.backends.cuda.matmul.allow_tf32 = True
        a = torch.randn(m, m, device="cuda:0")
        b = torch.randn(m, m, device="cuda:0")
        c = torch.empty(m, m, device="cuda:0")
        for _ in range(args.warmup):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        best = float("inf")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(args.steps):      # burst: best single launch
            e0.record(); torch.matmul(a, b, out=c); e1.record(); torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        reps = max(args.steps, 200)      # sustained: back to back for a few seconds
        e0.record()
        for _ in range(reps):
            torch.matmul(a, b, out=c)
        e1.record(); torch.cuda.synchronize()
        sustained_ms = e0.elapsed_time(e1) / reps
        flop = 2.0 * m * m * m
        print(json.dumps({"micro": name, "size": m, "library": "torch.matmul f32 with allow_tf32 (cuBLAS)",
                          "burst_tflops": flop / (best * 1e-3) / 1e12, "sustained_tflops": flop / (sustained_ms * 1e-3) / 1e12,
                          "sustained_launches": reps, "derived_peak_burst": peaks["bf16_burst"] / 2.0,
                          "derived_peak_sustained": peaks["bf16_sustained"] / 2.0}), flush=True)
        return
    if name.startswith("gemm"):
        m = nn = k = n or 8192
        if args.shape:      # M,N,K of a rectangular case, e.g. the C5 layer products 65536,8192,8192 (nn, nt) and 8192,8192,65536 (tn)
            m, nn, k = (int(v) for v in args.shape.split(","))
        block = rng.standard_normal(1 << 24, dtype=np.float32)     # large operands repeat a 2^24-element block of random data
        fill = lambda count: np.resize(block, count)
        a, b, c = dev(fill(m * k)), dev(fill(k * nn)), empty(m * nn)
        ta, tb = {"gemm_nn": (0, 0), "gemm_nt": (0, 1), "gemm_tn": (1, 0), "gemm_nn_fp32": (0, 0), "gemm_nt_fp32": (0, 1),
                  "gemm_tn_fp32": (1, 0), "gemm_nn_tf32x3": (0, 0)}[name]
        prec = 0 if name.endswith("fp32") else 2 if name.endswith("x3") else 1
        launch = lambda: chk(lib.launch_gemm_kernel(a, b, c, m, nn, k, ta, tb, None, 0, None, prec, None), name)
        # 3xTF32 does three tensor-core sweeps (plus the operand split) for the same algorithmic flop: its roofline is a third
        peak = {0: None, 1: peaks["bf16_burst"] / 2.0, 2: peaks["bf16_burst"] / 6.0}[prec]
        work, unit = 2.0 * m * nn * k, "TFLOP/s"
    elif name == "adam":
        n = n or (1 << 26)
        bufs = [dev(rng.standard_normal(n, dtype=np.float32)) for _ in range(2)] + [dev(np.zeros(n, np.float32)) for _ in range(2)]
        tab = lambda p: (vp * 1)(p)
        sizes = (C.c_ulonglong * 1)(n)
        launch = lambda: chk(lib.launch_adam_multi_tensor_kernel(tab(bufs[0]), tab(bufs[1]), tab(bufs[2]), tab(bufs[3]), sizes, 1,
                                                                 1e-3, 0.9, 0.999, 1e-8, 0.0, 10.0, 1000.0, 1.0, None), name)
        work, unit, peak = 28.0 * n, "GB/s", peaks["hbm_gbs"]
    elif name in ("add", "mul_backward"):
        n = n or (1 << 26)
        x, y, g = (dev(rng.standard_normal(n, dtype=np.float32)) for _ in range(3))
        o1, o2 = empty(n), empty(n)
        if name == "add":
            launch = lambda: chk(lib.launch_add_kernel(x, y, o1, n, None), name)
            work = 12.0 * n
        else:
            launch = lambda: chk(lib.launch_mul_backward_kernel(x, y, g, o1, o2, n, None), name)
            work = 20.0 * n
        unit, peak = "GB/s", peaks["hbm_gbs"]
    elif name == "fill":
        # write-only: the ceiling for kernels that read (almost) nothing, such as a column plus a row broadcast to a matrix
        n = n or (1 << 26)
        o1 = empty(n)
        launch = lambda: chk(lib.launch_fill_kernel(o1, 1.5, n, None), name)
        work, unit, peak = 4.0 * n, "GB/s", peaks["hbm_gbs"]
    elif name in ("exp", "tanh", "sigmoid", "sigmoid_backward"):
        n = n or (1 << 26)
        x, g, o1 = dev(rng.standard_normal(n, dtype=np.float32)), dev(rng.standard_normal(n, dtype=np.float32)), empty(n)
        code = {"exp": 0, "tanh": 3, "sigmoid": 4, "sigmoid_backward": 4}[name]     # enum ts_unary_op
        if name.endswith("backward"):
            launch = lambda: chk(lib.launch_unary_backward_kernel(code, x, g, o1, n, 0.0, None), name)
            work = 12.0 * n
        else:
            launch = lambda: chk(lib.launch_unary_kernel(code, x, o1, n, 0.0, None), name)
            work = 8.0 * n
        unit, peak = "GB/s", peaks["hbm_gbs"]
    elif name in ("softmax_rows", "softmax_classes", "softmax_inner"):
        # long rows (one warp per row), 10-class rows (one thread per row), and a middle axis (one thread per line)
        outer, reduce, inner = {"softmax_rows": (16384, 4096, 1), "softmax_classes": (1 << 22, 10, 1),
                                "softmax_inner": (64, 256, 4096)}[name]
        n = outer * reduce * inner
        x, o1 = dev(rng.standard_normal(n, dtype=np.float32)), empty(n)
        launch = lambda: chk(lib.launch_softmax_kernel(x, o1, outer, reduce, inner, None), name)
        work, unit, peak = 8.0 * n, "GB/s", peaks["hbm_gbs"]
    elif name in ("transpose", "permute_021", "permute_gather"):
        # [8192, 8192] -> transposed; [64, 1024, 1024] with the last two axes swapped; [256, 512, 512] -> axes (2, 0, 1)
        shape, perm = {"transpose": ((8192, 8192), (1, 0)), "permute_021": ((64, 1024, 1024), (0, 2, 1)),
                       "permute_gather": ((256, 512, 512), (2, 0, 1))}[name]
        n = int(np.prod(shape))
        x, o1 = dev(rng.standard_normal(n, dtype=np.float32)), empty(n)
        dims = (C.c_ulonglong * len(shape))(*shape)
        pm = (C.c_int * len(shape))(*perm)
        launch = lambda: chk(lib.launch_permute_kernel(x, o1, dims, pm, len(shape), None), name)
        work, unit, peak = 8.0 * n, "GB/s", peaks["hbm_gbs"]
    elif name in ("reduce_rows", "reduce_cols", "reduce_all_max", "reduce_middle"):
        # sum over the last axis, over the first axis, max of everything, sum over the middle axis of [64, 256, 4096]
        shape, axes, op = {"reduce_rows": ((16384, 4096), (1,), 0), "reduce_cols": ((16384, 4096), (0,), 0),
                           "reduce_all_max": ((1 << 26,), (0,), 1), "reduce_middle": ((64, 256, 4096), (1,), 0)}[name]
        n = int(np.prod(shape))
        x, o1 = dev(rng.standard_normal(n, dtype=np.float32)), empty(n)
        sc = empty(int(lib.ts_reduce_dims_scratch_elems()))
        dims = (C.c_ulonglong * len(shape))(*shape)
        ax = (C.c_ulonglong * len(axes))(*axes)
        launch = lambda: chk(lib.launch_reduce_dims_kernel(op, x, None, o1, dims, len(shape), ax, len(axes), sc, None), name)
        work, unit, peak = 4.0 * n, "GB/s", peaks["hbm_gbs"]
    elif name in ("matmul_batched_fp32", "matmul_batched_tf32"):
        # the batched pair of the reference's own matmul benchmark (64 x 128 x 128 times 64 x 128 x 128,
        # libtorch-validation/examples/benches/matmul_performance.rs:22-46) through Tensor::matmul; the result tensor of
        # each call is dropped at once, so the caching allocator hands the same block back every time
        ts.set_matmul_precision(ts.FP32 if name.endswith("fp32") else ts.TF32)
        bt, mm = 64, 128
        ta = ts.Tensor.from_slice(rng.standard_normal((bt, mm, mm), dtype=np.float32), [bt, mm, mm])
        tb = ts.Tensor.from_slice(rng.standard_normal((bt, mm, mm), dtype=np.float32), [bt, mm, mm])
        n = bt * mm * mm

        def launch():
            with ts.NoGradTrack():
                ta.matmul(tb).data_ptr()
        work, unit, peak = 2.0 * bt * mm * mm * mm, "TFLOP/s", None
    elif name in ("broadcast_row", "broadcast_col", "broadcast_outer", "broadcast_mul_backward"):
        # [16384, 4096] with a row [4096], with a column [16384, 1]; a column times a row; both gradients of the column case
        sa, sb = {"broadcast_row": ((16384, 4096), (4096,)), "broadcast_col": ((16384, 4096), (16384, 1)),
                  "broadcast_outer": ((16384, 1), (1, 4096)), "broadcast_mul_backward": ((16384, 4096), (16384, 1))}[name]
        so = np.broadcast_shapes(sa, sb)
        n = int(np.prod(so))
        a, b, o1 = dev(rng.standard_normal(sa, dtype=np.float32)), dev(rng.standard_normal(sb, dtype=np.float32)), empty(n)
        da, db = (C.c_ulonglong * len(sa))(*sa), (C.c_ulonglong * len(sb))(*sb)
        if name.endswith("backward"):
            g, o2 = dev(rng.standard_normal(so, dtype=np.float32)), empty(n)
            launch = lambda: chk(lib.launch_binary_broadcast_backward_kernel(2, a, da, len(sa), b, db, len(sb), g, o1, o2, None), name)
            work = 4.0 * (3 * n + int(np.prod(sa)) + int(np.prod(sb)))
        else:
            launch = lambda: chk(lib.launch_binary_broadcast_kernel(0, a, da, len(sa), b, db, len(sb), o1, None), name)
            work = 4.0 * (n + int(np.prod(sa)) + int(np.prod(sb)))
        unit, peak = "GB/s", peaks["hbm_gbs"]
    elif name in ("colsum", "relu_backward_colsum"):
        rows, cols = (n or 16384), 8192
        g, ref = dev(rng.standard_normal((rows, cols), dtype=np.float32)), dev(rng.standard_normal((rows, cols), dtype=np.float32))
        out, gi, sc = empty(cols), empty(rows * cols), empty(int(lib.ts_colsum_scratch_elems(rows, cols)))
        if name == "colsum":
            launch = lambda: chk(lib.launch_colsum_kernel(g, out, rows, cols, sc, None), name)
            work = 4.0 * rows * cols
        else:
            launch = lambda: chk(lib.launch_relu_backward_colsum_kernel(ref, g, gi, out, rows, cols, sc, None), name)
            work = 12.0 * rows * cols
        unit, peak = "GB/s", peaks["hbm_gbs"]
    else:
        n = n or (1 << 27)
        x, out, sc = dev(rng.standard_normal(n, dtype=np.float32)), empty(1), empty(int(lib.ts_reduce_scratch_elems()))
        launch = lambda: chk(lib.launch_sum_kernel(x, out, n, 0, sc, None), name)
        work, unit, peak = 4.0 * n, "GB/s", peaks["hbm_gbs"]

    for _ in range(args.warmup):
        launch()
    ts.synchronize()
    ev0, ev1 = lib.ts_event_create(), lib.ts_event_create()
    lib.ts_event_record(ev0, None)
    for _ in range(args.steps):
        launch()
    lib.ts_event_record(ev1, None)
    ts.synchronize()
    ms = float(lib.ts_event_elapsed_ms(ev0, ev1)) / args.steps
    rate = work / (ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9)
    print(json.dumps({"micro": name, "size": n, "launches": args.steps, "ms_per_launch": ms, "achieved": rate, "unit": unit,
                      "peak": peak, "frac": rate / peak if peak else None, "peak_source": peaks["source"]}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--micro", default=None, choices=MICRO_CASES, help="time one kernel on a small standalone case")
    ap.add_argument("--micro-size", type=int, default=0)
    ap.add_argument("--shape", default="", help="--micro gemm_*: M,N,K of a rectangular case")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="tf32", choices=["tf32", "fp32", "tf32x3"])
    ap.add_argument("--config", default="c5", choices=["c1", "c2", "c3", "c4", "c5"],
                    help="BASELINE configuration; c5 (default) is the headline data-parallel MLP, the others run on one GPU")
    ap.add_argument("--lr", type=float, default=C5_LR, help="Adam learning rate of the C5 run")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-dp-check", action="store_true", help="N > 1: skip the replica and gradient checks after the timed steps")
    ap.add_argument("--no-extras", action="store_true", help="C5 only: skip the short runs of the other configurations and the vendor TF32 yardstick")
    args = ap.parse_args()
    if args.micro:
        run_micro(args)
        return
    if args.config == "c2":
        print(json.dumps(run_c2(args.steps, args.warmup)), flush=True)
        return
    if args.config in CONFIGS:
        print(json.dumps(run_config(args.config, args.precision, args.steps, args.warmup)), flush=True)
        return
    d = Dist(args.gpus)
    try:
        if args.impl == "reference":
            run_reference(args, d)
        else:
            run_gpu(args, d)
    finally:
        d.close()


if __name__ == "__main__":
    main()
