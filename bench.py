#!/usr/bin/env python
"""Benchmark of the GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the hot path over one batch of synthetic input.  The
default workload is the large bf16 GEMM (M=32768, N=16384, K=8192, A row-major,
B column-major, fp32 accumulation, bf16 output), the configuration the metric
"GEMM TFLOP/s at 1/2/4/8 GPUs" is quoted on; with N > 1 ranks (torchrun, one
process per GPU) A and C are sharded by row blocks, B is broadcast once over
NCCL before the timed region, and no collective runs inside a step (strong
scaling: total work fixed).

One JSON line is printed by rank 0:
  value     whole-job TFLOP/s with operands resident in HBM (CUDA events, max over ranks)
  e2e       the same through the C ABI with pinned HOST buffers (H2D + kernel + D2H timed)
  roofline  algorithmic FLOPs per launch / measured launch time against the measured peak
  cpu_baseline  the reference's CPU kernel timed on this box's host cores (bounded sample)
  sweep     short timings of the other workloads (fp32 FFMA / 3xTF32 SGEMM, int8, conv)

--impl reference times the reference's own CPU implementation (its generated
AVX-512 C when available, else the C restatement) on all host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "gemm_tflops"
UNIT = "TFLOP/s"

BF16_SHAPE = (32768, 16384, 8192)
SUBBLOCK = 2048  # CPU sample: the 2048^3 sub-block of the bf16 problem, in fp32


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["source"] = "measured"
        return p
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def recorded_dram_traffic():
    """dram read + write bytes of one headline launch, from the ncu summary under profiles/."""
    path = os.path.join(ROOT, "profiles", "gemm_tc2t_bf16_dram_traffic.txt")
    vals = {}
    try:
        with open(path) as f:
            for line in f:
                if line.startswith("#") or ":" not in line:
                    continue
                k, v = line.split(":", 1)
                vals[k.strip()] = float(v)
        return vals["dram_bytes_read_per_launch"] + vals["dram_bytes_write_per_launch"]
    except (OSError, KeyError, ValueError):
        return None


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [l for (t, l) in self.lines if t0 <= t <= t1 + 0.2] or [l for (_, l) in self.lines]
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in rows:
            parts = [p.strip() for p in l.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------- CPU reference
def _cpu_inputs():
    """The 2048^3 sub-block of the bf16 problem as the reference sees it: bf16
    values N(0,1)*0.02 widened exactly to fp32, B transposed to row-major."""
    import numpy as np

    from tests import inputs

    A = inputs.bf16_bits_to_f32(inputs.normal_bf16(1, (SUBBLOCK, SUBBLOCK)))
    B = np.ascontiguousarray(inputs.bf16_bits_to_f32(inputs.normal_bf16(2, (SUBBLOCK, SUBBLOCK))).T)
    return A, B


_W = {}


def _worker_init(kind):
    import oracle

    _W["kind"] = kind
    _W["impl"] = oracle.ref() if kind == "reference" else oracle.port()


def _worker_run(args):
    import numpy as np

    r0, r1 = args
    A, B = _W["A"], _W["B"]
    C = np.zeros((r1 - r0, B.shape[1]), np.float32)
    _W["impl"].sgemm(np.ascontiguousarray(A[r0:r1]), B, C)
    return float(C[0, 0])


def cpu_reference_kind():
    import oracle

    return "reference" if oracle.ref_available() else "port"


def run_cpu_single_core(budget_s=10.0):
    """cpu_baseline leg: one host core (the generated sgemm_exo keeps its tiles in
    function statics, so it is single-threaded by construction)."""
    import numpy as np

    import oracle

    kind = cpu_reference_kind()
    impl = oracle.ref() if kind == "reference" else oracle.port()
    A, B = _cpu_inputs()
    C = np.zeros((SUBBLOCK, SUBBLOCK), np.float32)
    impl.sgemm(A, B, C)  # warm-up
    times = []
    t_start = time.perf_counter()
    while time.perf_counter() - t_start < budget_s and len(times) < 50:
        C[:] = 0
        t0 = time.perf_counter()
        impl.sgemm(A, B, C)
        times.append(time.perf_counter() - t0)
    times.sort()
    med = times[len(times) // 2]
    return {"value": 2.0 * SUBBLOCK ** 3 / med / 1e12, "unit": UNIT, "cores": 1, "kind": kind,
            "sample": f"{SUBBLOCK}^3 fp32 sub-block of the bf16 problem (bf16-rounded inputs), "
                      f"median of {len(times)} runs, {sum(times):.1f} s of CPU work"}


def run_reference_arm(args):
    """--impl reference: the reference CPU kernel on all host cores.  Rows are
    independent, so P processes each run sgemm_exo on a row block (processes, not
    threads: the generated code is not reentrant)."""
    import multiprocessing as mp

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind = cpu_reference_kind()
    cores = len(os.sched_getaffinity(0))
    A, B = _cpu_inputs()
    _W["A"], _W["B"] = A, B
    # load the checker library in this process too (the workers are forks and inherit the mapping),
    # so that a loader hook on the parent sees which shared object the arm runs
    _worker_init(kind)
    ctx = mp.get_context("fork")
    blocks = [(i * SUBBLOCK // cores, (i + 1) * SUBBLOCK // cores) for i in range(cores)]
    with ctx.Pool(cores, initializer=_worker_init, initargs=(kind,)) as pool:
        for _ in range(args.warmup):
            pool.map(_worker_run, blocks)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            pool.map(_worker_run, blocks)
        dt = time.perf_counter() - t0
    ms = dt / args.steps * 1e3
    value = 2.0 * SUBBLOCK ** 3 / (ms / 1e3) / 1e12
    sample = (f"each step = the {SUBBLOCK}^3 fp32 sub-block of the bf16 problem (bf16-rounded inputs), "
              f"row-sharded over {cores} processes")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config("bf16", args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------- workloads
def workload_config(name, gpus, shape=None):
    if shape is not None:
        return {"workload": f"{name} (profiling case, not the headline shape)", "shape": list(shape)}
    if name == "bf16":
        M, N, K = BF16_SHAPE
        return {"workload": f"bf16 GEMM M={M} N={N} K={K}, A row-major, B column-major, fp32 accumulate, bf16 out",
                "sharding": f"A/C row blocks over {gpus} GPU(s), B broadcast once (NCCL) outside the timed region",
                "l2": "inputs (768 MB) larger than L2; no flush needed",
                # the same text in both arms, so that their configs compare equal and neither claims more than it ran
                "reference_arm_sample": f"--impl reference times the {SUBBLOCK}^3 fp32 sub-block per step on the host "
                                        "cores (a rate comparison: the full problem is not run on the CPU)"}
    return {"workload": name}


class Workload:
    """flops per step, a device-resident step, and a host-buffer (e2e) step."""

    def __init__(self, name, lib, torch, rank, world, shape=None, dist=None):
        self.name, self.lib, self.torch, self.rank, self.world = name, lib, torch, rank, world
        self.launches_per_step = 1
        self.custom_shape = shape
        self.dist = dist
        getattr(self, f"_setup_{name}")()

    # -- bf16 headline
    def _setup_bf16(self):
        from exo_b200.shard import ShardedGemm

        t = self.torch
        M, N, K = self.custom_shape or BF16_SHAPE
        self.dtype = "bf16"
        self.sharded = ShardedGemm(self.dist, M, N, K)  # row blocks on CTA-tile boundaries
        rows = self.sharded.block.rows
        self.shape = (rows, N, K)
        g = t.Generator(device="cuda").manual_seed(1234 + self.rank)
        self.A = (t.randn((rows, K), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        self.B = t.empty((N, K), dtype=t.bfloat16, device="cuda")  # column-major K x N
        if self.rank == 0:
            gb = t.Generator(device="cuda").manual_seed(99)
            self.B.copy_((t.randn((N, K), generator=gb, device="cuda") * 0.02).to(t.bfloat16))
        self.C = t.empty((rows, N), dtype=t.bfloat16, device="cuda")
        self.flops_total = 2.0 * M * N * K
        self.flops_local = 2.0 * rows * N * K
        self.bound = "tensor"
        if self.custom_shape is None and self.world > 1 and any(b.rows != rows for b in self.sharded.blocks):
            raise SystemExit("row blocks must be equal for the scaling run")

    def step_bf16(self):
        self.sharded.step(self.A, self.B, self.C)

    def host_bf16(self):
        """Pinned host copies of this rank's operands.  Returns the bytes THIS rank moves per
        step: its rows of A and, with several ranks, only its 1/world slice of B (the rest
        arrives over NVLink, exo_b200/shard.py), and its rows of C back."""
        t = self.torch
        self.hA = t.empty(self.A.shape, dtype=self.A.dtype, pin_memory=True).copy_(self.A)
        self.hB = t.empty(self.B.shape, dtype=self.B.dtype, pin_memory=True).copy_(self.B)
        self.hC = t.empty(self.C.shape, dtype=self.C.dtype, pin_memory=True)
        lo, hi = self.sharded.b_slices(self.B.shape[0])[self.rank]
        b_rows = self.B.shape[0] if self.world == 1 else hi - lo
        return (self.hA.numel() + b_rows * self.B.shape[1]) * 2, self.hC.numel() * 2

    def verify_bf16(self, C, nrows=16):
        """Row sample of a result against an fp32 reference of the same rows (torch, on the
        GPU: a checker, not the product path): |delta| <= one bf16 ulp of the reference plus a
        floor near zero.  Returns the number of rows checked; raises on a mismatch."""
        t = self.torch
        rows = self.A.shape[0]
        pick = sorted({0, 1, 127, 128, 255, 256, 511, 512, rows // 2, rows - 129, rows - 2, rows - 1} |
                      {(i * 2654435761) % rows for i in range(4)})
        pick = [r for r in pick if 0 <= r < rows][:max(nrows, 1)]
        idx = t.tensor(pick, device=self.A.device)
        ref = self.A[idx].float() @ self.B.float().t()
        got = C[idx].float() if C.is_cuda else C[idx.cpu()].to(self.A.device).float()
        K = self.A.shape[1]
        tol = ref.abs() * 2.0 ** -7 + 1e-3 * K ** 0.5 * 4e-4
        bad = int(((got - ref).abs() > tol).sum().item())
        if bad:
            raise SystemExit(f"bench: {bad} elements of the verified rows are outside the bf16 tolerance")
        return len(pick)

    def e2e_bf16(self):
        self.sharded.step(self.hA, self.hB, self.hC)

    # -- fp32 SGEMM 8192^3 (FFMA exact / 3xTF32)
    def _setup_sgemm(self, n=8192):
        t = self.torch
        M, N, K = self.custom_shape or (n, n, n)
        self.dtype = "f32"
        self.shape = (M, N, K)
        g = t.Generator(device="cuda").manual_seed(5)
        self.A = t.rand((M, K), generator=g, device="cuda") * 2 - 1
        self.B = t.rand((K, N), generator=g, device="cuda") * 2 - 1
        self.C = t.zeros((M, N), device="cuda")
        self.flops_total = self.flops_local = 2.0 * M * N * K
        self.bound = "tensor"

    _setup_sgemm_ffma = _setup_sgemm

    def _setup_sgemm_3xtf32(self):
        self._setup_sgemm()
        self.launches_per_step = 3  # two split pre-passes + the GEMM

    def step_sgemm_ffma(self):
        M, N, K = self.shape
        self.lib.sgemm_exo_ffma(None, M, N, K, self.A, self.B, self.C)

    def step_sgemm_3xtf32(self):
        M, N, K = self.shape
        self.lib.sgemm_exo_3xtf32(None, M, N, K, self.A, self.B, self.C)

    def host_sgemm(self):
        t = self.torch
        self.hA = t.empty(self.A.shape, pin_memory=True).copy_(self.A)
        self.hB = t.empty(self.B.shape, pin_memory=True).copy_(self.B)
        self.hC = t.zeros(self.C.shape).pin_memory()
        return (self.hA.numel() + self.hB.numel() + self.hC.numel()) * 4, self.hC.numel() * 4

    host_sgemm_ffma = host_sgemm_3xtf32 = host_sgemm

    def e2e_sgemm_ffma(self):
        M, N, K = self.shape
        self.lib.sgemm_exo_ffma(None, M, N, K, self.hA, self.hB, self.hC)

    def e2e_sgemm_3xtf32(self):
        M, N, K = self.shape
        self.lib.sgemm_exo_3xtf32(None, M, N, K, self.hA, self.hB, self.hC)

    # -- int8 4096^3
    def _setup_i8(self, n=4096):
        t = self.torch
        if self.custom_shape:
            n = self.custom_shape[0]
        self.dtype = "i8"
        self.shape = (n, n, n)
        g = t.Generator(device="cuda").manual_seed(6)
        self.A = t.randint(-128, 128, (n, n), generator=g, device="cuda", dtype=t.int8)
        self.B = t.randint(-128, 128, (n, n), generator=g, device="cuda", dtype=t.int8)
        self.C = t.empty((n, n), dtype=t.int8, device="cuda")
        self.flops_total = self.flops_local = 2.0 * n ** 3
        self.bound = "tensor"
        self.launches_per_step = 1  # B is read MN-major in place: no pre-pass

    def _setup_i8_512(self):
        self._setup_i8(512)
        self.launches_per_step = 1

    def step_i8_512(self):
        self.step_i8()

    def step_i8(self):
        n = self.shape[0]
        self.lib.matmul_on_cpu(None, n, n, n, 1.0 / 256, False, self.A, self.B, self.C)

    def host_i8(self):
        t = self.torch
        self.hA = t.empty(self.A.shape, dtype=t.int8, pin_memory=True).copy_(self.A)
        self.hB = t.empty(self.B.shape, dtype=t.int8, pin_memory=True).copy_(self.B)
        self.hC = t.empty(self.C.shape, dtype=t.int8, pin_memory=True)
        return self.hA.numel() + self.hB.numel(), self.hC.numel()

    def e2e_i8(self):
        n = self.shape[0]
        self.lib.matmul_on_cpu(None, n, n, n, 1.0 / 256, False, self.hA, self.hB, self.hC)

    # -- fp32 conv: batch 4, 56x56, 64->64, 3x3, pad 1 (implicit GEMM, exact)
    def _setup_conv(self, cv=(4, 56, 56, 64, 64, 3, 1)):
        t = self.torch
        self.dtype = "f32"
        g = t.Generator(device="cuda").manual_seed(8)
        self.cv = cv
        b, h, w, ci, co, k, pad = self.cv
        self.A = t.rand((b, h, w, ci), generator=g, device="cuda") * 2 - 1
        self.B = t.rand((k, k, ci, co), generator=g, device="cuda") * 2 - 1
        self.bias = t.rand((co,), generator=g, device="cuda") * 2 - 1
        oh, ow = h + 2 * pad - k + 1, w + 2 * pad - k + 1
        self.C = t.empty((b, oh, ow, co), device="cuda")
        self.flops_total = self.flops_local = 2.0 * b * oh * ow * co * k * k * ci
        self.bound = "tensor"

    def step_conv(self):
        b, h, w, ci, co, k, pad = self.cv
        self.lib.conv_nhwc_exo(None, b, h, w, ci, co, k, pad, True, self.A, self.C, self.B, self.bias)

    # -- the same conv on the tensor cores (TMA implicit im2col, 3xTF32)
    def _setup_conv_3xtf32(self):
        self._setup_conv()
        self.launches_per_step = 2  # one pre-pass (input and weight split), the conv kernel

    def step_conv_3xtf32(self):
        b, h, w, ci, co, k, pad = self.cv
        self.lib.conv_nhwc_exo_3xtf32(None, b, h, w, ci, co, k, pad, True, self.A, self.C, self.B, self.bias)

    # -- the reference's own instance (apps/x86/conv/conv.py:49,55): batch 5, 82x102 -> 80x100, 128 -> 128, 3x3
    def _setup_conv_ref(self):
        self._setup_conv(cv=(5, 82, 102, 128, 128, 3, 0))

    step_conv_ref = step_conv

    def _setup_conv_ref_3xtf32(self):
        self._setup_conv(cv=(5, 82, 102, 128, 128, 3, 0))
        self.launches_per_step = 2

    step_conv_ref_3xtf32 = step_conv_3xtf32

    # -- the 1x1 conv: batch 8, 28x28, 256 -> 512 (exact FFMA and 3xTF32)
    def _setup_conv1x1(self):
        self._setup_conv(cv=(8, 28, 28, 256, 512, 1, 0))

    step_conv1x1 = step_conv

    def _setup_conv1x1_3xtf32(self):
        self._setup_conv(cv=(8, 28, 28, 256, 512, 1, 0))
        self.launches_per_step = 2

    step_conv1x1_3xtf32 = step_conv_3xtf32

    # -- Gemmini int8 conv_3: batch 4, 58 -> 56, 64 -> 64, 3x3 (tensor cores, bit-exact)
    def _setup_conv_i8(self):
        t = self.torch
        self.dtype = "i8"
        g = t.Generator(device="cuda").manual_seed(9)
        self.A = t.randint(-128, 128, (4, 58, 58, 64), generator=g, device="cuda", dtype=t.int8)
        self.B = t.randint(-128, 128, (3, 3, 64, 64), generator=g, device="cuda", dtype=t.int8)
        self.bias = t.randint(-1000, 1000, (1, 64), generator=g, device="cuda", dtype=t.int32)
        self.C = t.empty((4, 56, 56, 64), dtype=t.int8, device="cuda")
        self.flops_total = self.flops_local = 2.0 * 4 * 56 * 56 * 64 * 9 * 64
        self.bound = "tensor"

    def step_conv_i8(self):
        self.lib.conv_3(None, self.C, self.bias, self.A, self.B, True, 1.0 / 256)

    def step(self):
        getattr(self, f"step_{self.name}")()

    def host(self):
        return getattr(self, f"host_{self.name}")()

    def e2e_step(self):
        getattr(self, f"e2e_{self.name}")()


def time_steps(torch, fn, steps, warmup, dist=None):
    """CUDA events on the launching stream, barrier + synchronize on both sides,
    max over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.time()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        dist.barrier()
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps, t0, t1


def run_ours(args):
    import torch

    import exo_b200

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    lib = exo_b200.library()
    peaks = measured_peaks()

    shape = tuple(int(x) for x in args.shape.split("x")) if args.shape else None
    wl = Workload(args.workload, lib, torch, rank, world, shape=shape, dist=dist)
    bcast_ms = None
    if dist is not None:
        # the one exchange of the sharded GEMM: B from rank 0 to every GPU over NVLink
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        wl.sharded.broadcast_b(wl.B)
        e1.record()
        torch.cuda.synchronize()
        bcast_ms = e0.elapsed_time(e1)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    if args.workload == "bf16":
        wl.C.zero_()  # so that the check below cannot pass on a stale result
    ms, t0, t1 = time_steps(torch, wl.step, args.steps, args.warmup, dist)
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    lib.synchronize()
    value = wl.flops_total / (ms / 1e3) / 1e12
    verified_rows = wl.verify_bf16(wl.C) if args.workload == "bf16" else 0

    # the same launch back to back for a few seconds: the power-capped regime, with the SM clock it settles at
    sustained = None
    if args.workload == "bf16" and args.sustained_seconds > 0:
        n = max(args.steps, int(args.sustained_seconds * 1e3 / max(ms, 1e-3)) + 1)
        s2 = ClockSampler(local)
        if rank == 0:
            s2.start()
            time.sleep(0.2)
        sms, st0, st1 = time_steps(torch, wl.step, n, 1, dist)
        sclk = s2.stop(st0, st1) if rank == 0 else None
        sustained = {"value": wl.flops_total / (sms / 1e3) / 1e12, "unit": UNIT, "launches": n, "seconds": sms * n / 1e3,
                     "ms_per_step": sms, "clocks": sclk}
        if sclk and sclk.get("sm_mhz"):
            sustained["ms_times_sm_mhz"] = sms * sclk["sm_mhz"]

    # Optional same-GPU, same-minute denominator: the vendor library's GEMM (torch.matmul ->
    # cuBLAS) on the same buffers with the same timing loop.  A library call, reported for
    # comparison only; nothing of the product runs through it.
    library = None
    if args.library_gemm and args.workload == "bf16" and world == 1:
        time.sleep(1.0)
        lib_c = torch.empty_like(wl.C)
        sampler2 = ClockSampler(local)
        sampler2.start()
        time.sleep(0.3)
        lms, lt0, lt1 = time_steps(torch, lambda: torch.matmul(wl.A, wl.B.t(), out=lib_c), args.steps, args.warmup)
        library = {"impl": "torch.matmul (cuBLAS)", "tflops": wl.flops_total / (lms / 1e3) / 1e12, "ms_per_step": lms,
                   "clocks": sampler2.stop(lt0, lt1), "ours_over_library": lms / ms}
        del lib_c

    # end to end: pinned host buffers through the C ABI, copies inside the timed region
    if args.no_e2e:
        h2d = d2h = 0
        e2e_steps, e2e_ms, e2e_value = 0, None, None
    else:
        h2d, d2h = wl.host()
        if dist is not None:  # whole-job bytes: every rank's share
            tb = torch.tensor([h2d, d2h], device="cuda", dtype=torch.float64)
            dist.all_reduce(tb)
            h2d, d2h = int(tb[0].item()), int(tb[1].item())
        e2e_steps = max(1, min(args.steps, 5))
        if args.workload == "bf16":
            wl.hC.zero_()
        e2e_ms, _, _ = time_steps(torch, wl.e2e_step, e2e_steps, 1, dist)
        e2e_value = wl.flops_total / (e2e_ms / 1e3) / 1e12
        if args.workload == "bf16":
            verified_rows += wl.verify_bf16(wl.hC, 8)
    pcie = None
    if not args.no_e2e and args.workload == "bf16":
        hsave = wl.hC.clone()  # the copies below overwrite it
        pcie = pinned_copy_rates(torch, wl.hC, dist)
        wl.hC.copy_(hsave)
        del hsave

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peak = peaks["bf16_tflops"]
    per_launch_tflops = wl.flops_local / (ms / 1e3) / 1e12
    # DRAM bytes per launch of the headline shape: from the committed one-pass ncu capture of one
    # full-size launch (profiles/gemm_tc2t_bf16_dram_traffic.txt), scaled by the rows a rank owns
    traffic = None
    if args.workload == "bf16" and shape is None:
        per_launch = recorded_dram_traffic()
        traffic = per_launch * wl.shape[0] / BF16_SHAPE[0] if per_launch else None
    roofline = {"bound": "tensor", "achieved": per_launch_tflops, "peak": peak, "unit": "TFLOP/s",
                "frac": per_launch_tflops / peak, "traffic": traffic,
                "frac_of_sustained_peak": per_launch_tflops / peaks.get("bf16_tflops_sustained", peak),
                "peak_source": f"{peaks['source']} bf16 burst (sustained: {peaks.get('bf16_tflops_sustained')})",
                "kernel": "gemm_tc2t_kernel<bf16>" if args.workload == "bf16" else args.workload}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": workload_config(args.workload, world, shape), "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "steps": e2e_steps},
        "gpu_launches": wl.launches_per_step * args.steps,
        "roofline": roofline,
        "verified_rows": verified_rows,
    }
    if sustained is not None:
        line["sustained"] = sustained
    if e2e_ms and d2h and pcie:
        # The floor PCIe sets for the step: both directions busy at once, at the rates this box gave when
        # every rank copied both ways at the same time.  bound_frac near 1 = the step is the copies.
        line["e2e"]["pcie"] = pcie
        sfx = "_sum_over_ranks" if world > 1 else ""
        rate = pcie["bidir_each_way_gbs" + sfx]
        line["e2e"]["pcie_bound_ms"] = max(d2h, h2d) / (rate * 1e6)
        line["e2e"]["pcie_bound_frac"] = line["e2e"]["pcie_bound_ms"] / e2e_ms
        line["e2e"]["limiter"] = ("device-to-host copy of C" if d2h >= h2d else "host-to-device copy of A and B") + \
            " over PCIe with both directions busy"
    if bcast_ms is not None:
        line["b_broadcast_ms"] = bcast_ms
    if library is not None:
        line["library_gemm"] = library
    if world == 1:
        del wl
        torch.cuda.empty_cache()
        if not args.no_sweep:
            probes = probe_peaks(lib, torch)
            line["measured_peaks"] = probes
            line["sweep"] = run_sweep(lib, torch, peaks, args.workload, probes)
            try:
                line["sgemm_shapes"] = run_shapes(lib, torch, peaks, probes=probes)
                line["sgemm_aspect_k512"] = run_shapes(lib, torch, peaks, ASPECT_SHAPES, ("ffma",), probes)
                line["sgemm_squares"] = run_shapes(lib, torch, peaks, SQUARE_SHAPES, ("ffma",), probes)
                line["ssyrk"] = run_ssyrk(lib, torch, probes)
                line["conv_layers_exact"] = run_conv_layers(lib, torch, probes)
            except Exception as e:
                line["sgemm_shapes"] = {"error": str(e)[:200]}
        if not args.no_cpu:
            line["cpu_baseline"] = run_cpu_single_core()
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def pinned_copy_rates(torch, host_buf, dist=None):
    """GB/s of large pinned-memory copies on this box (CUDA events): one direction at a time, and both
    directions at once on two streams (what an end-to-end step does).  With several ranks all of them
    copy at the same time -- their links may share a PCIe switch or a host memory controller -- and the
    per-rank minimum and the sum over ranks are reported: the ceiling the end-to-end number sits under."""
    if host_buf is None:
        return None
    n = min(host_buf.numel(), 256 << 20)
    h = host_buf.view(-1)[:n]
    h2 = torch.empty(n, dtype=h.dtype, pin_memory=True)
    d = torch.empty(n, dtype=h.dtype, device="cuda")
    d2 = torch.empty(n, dtype=h.dtype, device="cuda")
    side = torch.cuda.Stream()
    nbytes = n * h.element_size()

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        return nbytes / (e0.elapsed_time(e1) * 1e6)

    def both():
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            h2.copy_(d2, non_blocking=True)
        d.copy_(h, non_blocking=True)
        torch.cuda.current_stream().wait_stream(side)

    out = {"h2d_gbs": timed(lambda: d.copy_(h, non_blocking=True)),
           "d2h_gbs": timed(lambda: h.copy_(d, non_blocking=True)),
           "bidir_each_way_gbs": timed(both)}
    if dist is not None:
        keys = sorted(out)
        t = torch.tensor([out[k] for k in keys], device="cuda", dtype=torch.float64)
        tmin = t.clone()
        dist.all_reduce(t)
        dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
        out = {"ranks_copy_concurrently": dist.get_world_size()}
        for i, k in enumerate(keys):
            out[k + "_sum_over_ranks"] = float(t[i].item())
            out[k + "_min_rank"] = float(tmin[i].item())
    return out


def probe_peaks(lib, torch):
    """Ceilings measured on this GPU by the library's probe kernels (packed fp32 FMA from registers;
    tcgen05.mma with operands resident in shared memory), ~40 ms each; the computed SIMT figure
    (SMs x 128 lanes x 2 x max clock) is kept beside the measured one."""
    sm_count = torch.cuda.get_device_properties(0).multi_processor_count
    out = {"fp32_simt_computed": sm_count * 128 * 2 * 1.965e9 / 1e12}
    for key, what in (("fp32_simt", 0), ("int8_tensor", 1), ("bf16_tensor", 2), ("tf32_tensor", 3)):
        v = lib.dll.exo_b200_measure_peak(what, 40)
        out[key] = v if v > 0 else None
    return out


def run_sweep(lib, torch, peaks, skip, probes=None):
    """Short device-resident timings of the other workloads (5 steps each)."""
    out = {}
    probes = probes or {}
    simt_peak = probes.get("fp32_simt") or probes.get("fp32_simt_computed")
    simt_name = "fp32 SIMT measured (packed FMA probe)" if probes.get("fp32_simt") else "fp32 SIMT at max SM clock (computed)"
    i8_peak = probes.get("int8_tensor") or peaks["bf16_tflops"] * 2
    i8_name = "int8 tensor measured (tcgen05.mma probe)" if probes.get("int8_tensor") else "2 x bf16 measured (nominal int8 ratio)"
    tf32_peak = probes.get("tf32_tensor") or peaks["bf16_tflops"] / 2
    flush, flush_ms = None, 0.0
    for name in ("sgemm_ffma", "sgemm_3xtf32", "i8", "i8_512", "conv", "conv_3xtf32", "conv1x1", "conv1x1_3xtf32", "conv_ref", "conv_ref_3xtf32",
                 "conv_i8", "bf16"):
        if name == skip:
            continue
        try:
            wl = Workload(name, lib, torch, 0, 1)
            ms, _, _ = time_steps(torch, wl.step, 5 if wl.flops_total > 1e12 else 50, 3)
            lib.synchronize()
            tf = wl.flops_total / (ms / 1e3) / 1e12
            if name in ("sgemm_ffma", "conv", "conv1x1", "conv_ref"):
                peak, pname = simt_peak, simt_name
            elif name in ("sgemm_3xtf32", "conv_3xtf32", "conv1x1_3xtf32", "conv_ref_3xtf32"):
                peak, pname = tf32_peak / 3, "tf32 tensor peak / 3 (three MMAs per product)"
            elif name in ("i8", "i8_512", "conv_i8"):
                peak, pname = i8_peak, i8_name
            else:
                peak, pname = peaks["bf16_tflops"], "bf16 measured"
            out[name] = {"tflops": tf, "ms": ms, "peak": peak, "frac": tf / peak, "peak_is": pname,
                         "launches_per_step": wl.launches_per_step}
            if ms < 0.2:
                # A step this short is paced by the host (a call through ctypes takes about as long): also time
                # it on the device alone, replayed from a CUDA graph with an L2 flush before every step.
                if flush is None:
                    flush = L2Flush(torch)
                    flush_ms = graph_replay_ms(torch, flush)

                def body():
                    flush()
                    wl.step()

                try:
                    dev_ms = max(graph_replay_ms(torch, body) - flush_ms, 1e-6)
                    out[name]["device_us"] = dev_ms * 1e3
                    out[name]["tflops_device"] = wl.flops_total / (dev_ms / 1e3) / 1e12
                    out[name]["frac_device"] = out[name]["tflops_device"] / peak
                except Exception as e:
                    out[name]["device_us_error"] = str(e)[:200]
                    torch.cuda.synchronize()
            del wl
            torch.cuda.empty_cache()
        except Exception as e:  # a failing side workload must not lose the headline line
            out[name] = {"error": str(e)[:200]}
    return out


SGEMM_SHAPES = [(256, 256, 256), (512, 512, 512), (1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096),
                (1000, 1000, 1000), (17, 4099, 513), (4096, 64, 4096), (1, 8192, 8192)]


# the K = 512 aspect-ratio sweep of the reference's SGEMM bench (apps/x86/sgemm/bench_sgemm.cpp:85-97)
ASPECT_SHAPES = [(32768, 8, 512), (16384, 16, 512), (8192, 32, 512), (4096, 64, 512), (2048, 128, 512),
                 (1024, 256, 512), (256, 1024, 512), (128, 2048, 512), (64, 4096, 512), (32, 8192, 512),
                 (16, 16384, 512), (8, 32768, 512)]


# the square sizes of the reference's SGEMM bench (apps/x86/sgemm/bench_sgemm.cpp:58-84: 64 .. 1984 in steps of 64 up
# to 512, then coarser), every fourth of them here to keep the sweep short
SQUARE_SHAPES = [(n, n, n) for n in (64, 128, 192, 256, 320, 384, 448, 512, 640, 768, 896, 1024, 1152, 1280, 1408, 1536,
                                     1664, 1792, 1920, 2048)]


# the layer list of the reference's convolution bench (apps/x86/conv/bench_conv.cpp:46-53):
# batch, in_h, in_w, in_chan, out_chan, kernel, pad, stride
CONV_LAYERS = [(4, 224, 224, 3, 64, 7, 3, 2), (4, 56, 56, 64, 64, 3, 1, 1), (4, 28, 28, 128, 128, 3, 1, 2),
               (4, 56, 56, 64, 64, 3, 0, 1), (5, 82, 102, 128, 128, 3, 0, 1)]


def run_conv_layers(lib, torch, probes):
    """Exact fp32 convolution (bias + ReLU) on the layers the reference's bench lists; the stride-2 ones
    go through conv_nhwc_strided_exo (the Exo procedure itself has no stride)."""
    out = []
    gen = torch.Generator(device="cuda").manual_seed(5)
    simt_peak = probes.get("fp32_simt") or probes.get("fp32_simt_computed")
    for (b, h, w, ci, co, k, pad, stride) in CONV_LAYERS:
        x = torch.rand((b, h, w, ci), generator=gen, device="cuda") * 2 - 1
        wt = torch.rand((k, k, ci, co), generator=gen, device="cuda") * 2 - 1
        bias = torch.rand((co,), generator=gen, device="cuda") * 2 - 1
        oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        y = torch.empty((b, oh, ow, co), device="cuda")

        def call():
            lib.conv_nhwc_strided_exo(None, b, h, w, ci, co, k, pad, stride, True, x, y, wt, bias)

        for _ in range(3):
            call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            call()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 20
        tf = 2.0 * b * oh * ow * co * k * k * ci / ms / 1e9
        out.append({"layer": [b, h, w, ci, co, k, pad, stride], "us": ms * 1e3, "tflops": tf, "frac_of_simt": tf / simt_peak})
    lib.synchronize()
    return out


def run_ssyrk(lib, torch, probes):
    """SSYRK at sizes of the reference's comparison benchmark (apps/x86/ssyrk/bench_ssyrk.cpp:60-65),
    flops counted its way: k n (n + 1)."""
    out = []
    gen = torch.Generator(device="cuda").manual_seed(4)
    simt_peak = probes.get("fp32_simt") or probes.get("fp32_simt_computed")
    for (n, k) in ((256, 256), (1024, 1024), (2048, 512), (2048, 2048)):
        A = torch.rand((n, k), generator=gen, device="cuda") * 2 - 1
        C = torch.zeros((n, n), device="cuda")
        row = {"shape": [n, k]}
        for path, fn in (("ffma", lib.ssyrk_exo_ffma), ("3xtf32", lib.ssyrk_exo_3xtf32)):
            for _ in range(3):
                fn(None, n, k, A, C)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                fn(None, n, k, A, C)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 20
            tf = k * n * (n + 1.0) / ms / 1e9
            row[path] = {"us": ms * 1e3, "tflops": tf}
            if path == "ffma":
                row[path]["frac_of_simt"] = tf / simt_peak
        out.append(row)
    lib.synchronize()
    return out


class L2Flush:
    """Flushes L2 between timed launches: a 256 MB write (larger than the 126 MB L2), then a 256 MB read of a
    second buffer.  The write alone leaves L2 full of dirty lines that are written back while the next kernel
    runs, which costs an HBM-bound kernel DRAM bandwidth that is not its own (1 x 8192 x 2048: 18.0 us after
    the write alone, 14.7 us after write + read, 13.7 us after a read-only flush, 11.8 us warm); after the read
    L2 holds clean lines of an unrelated buffer."""

    def __init__(self, torch):
        self.dirty = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        self.clean = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self):
        self.dirty.fill_(1)
        self.clean.max()


def graph_replay_ms(torch, body, R=10):
    """Device time of one `body`: R of them captured in a CUDA graph, median of 5 replays, per body."""
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(R):
            body()
    g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2] / R


def run_shapes(lib, torch, peaks, shapes=None, paths=("ffma", "3xtf32"), probes=None):
    """The SGEMM shape sweep (squares and ragged / skinny shapes) on both fp32
    paths, device time per launch.  Small shapes finish faster than the host can
    launch them, so launches are replayed from a CUDA graph: R x [L2 flush (a
    256 MB write, then a 256 MB read), GEMM], minus a graph of R flushes alone;
    median of 5 replays."""
    probes = probes or {}
    simt_peak = probes.get("fp32_simt") or probes.get("fp32_simt_computed")
    tf32_peak = probes.get("tf32_tensor") or peaks["bf16_tflops"] / 2
    hbm = peaks["hbm_gbs"]
    flush = L2Flush(torch)

    def replay_ms(body):
        return graph_replay_ms(torch, body)

    flush_ms = replay_ms(flush)
    out = []
    gen = torch.Generator(device="cuda").manual_seed(3)
    for (M, N, K) in (shapes or SGEMM_SHAPES):
        A = torch.rand((M, K), generator=gen, device="cuda") * 2 - 1
        B = torch.rand((K, N), generator=gen, device="cuda") * 2 - 1
        C = torch.zeros((M, N), device="cuda")
        flops = 2.0 * M * N * K
        nbytes = 4.0 * (M * K + K * N + 2 * M * N)
        row = {"shape": [M, N, K], "flop_per_byte": flops / nbytes}
        big = twin = None
        for path, fn in (("ffma", lib.sgemm_exo_ffma), ("3xtf32", lib.sgemm_exo_3xtf32)):
            if path not in paths:
                continue
            for _ in range(3):
                fn(None, M, N, K, A, B, C)  # warm-up: also sizes the scratch before capture
            torch.cuda.synchronize()
            # let the clocks recover: a small shape timed right after a power-capped large one inherits its
            # low clock (1000^3 measured 83.6 us directly after the 4096^3 rows, 63.1 us on its own)
            time.sleep(0.1)

            # operands larger than L2 (126 MB) need no flush: they evict themselves
            flushed = nbytes <= 1.5 * 126e6

            # ... but the tail of the previous launch's pass is still there, so those launches alternate
            # between two copies of the larger operand
            if not flushed and twin is None:
                big = A if A.numel() >= B.numel() else B
                twin = big.clone()
            toggle = [0]

            def body():
                if flushed:
                    flush()
                    fn(None, M, N, K, A, B, C)
                else:
                    toggle[0] ^= 1
                    a = twin if (toggle[0] and big is A) else A
                    b = twin if (toggle[0] and big is B) else B
                    fn(None, M, N, K, a, b, C)

            ms = max(replay_ms(body) - (flush_ms if flushed else 0.0), 1e-6)
            tf, gbs = flops / ms / 1e9, nbytes / ms / 1e6
            peak_tf = simt_peak if path == "ffma" else tf32_peak / 3
            # the roofline that binds: min(compute peak, bandwidth x arithmetic intensity)
            ceiling = min(peak_tf, hbm * row["flop_per_byte"] / 1e3)
            row[path] = {"us": ms * 1e3, "tflops": tf, "gbs": gbs, "bound": "hbm" if ceiling < peak_tf else "compute",
                         "frac_of_roofline": tf / ceiling, "l2": "flushed" if flushed else "operands larger than L2, two copies alternating"}
        out.append(row)
    lib.synchronize()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="bf16", choices=["bf16", "sgemm_ffma", "sgemm_3xtf32", "i8", "conv", "conv_3xtf32", "conv1x1", "conv1x1_3xtf32",
                             "conv_i8"])
    ap.add_argument("--shape", default=None, help="MxNxK override for small profiling cases")
    ap.add_argument("--library-gemm", action="store_true",
                    help="bf16, 1 GPU: also time torch.matmul (cuBLAS) on the same buffers, for comparison")
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="bf16: also time the launch back to back for about this long (0: skip)")
    ap.add_argument("--time-shapes", default=None,
                    help="comma-separated MxNxK list: time only sgemm_exo_ffma on these shapes (CUDA-graph replay, L2 "
                         "flushed) and print one JSON line; with EXOB200_FFMA_TILE this is how the tile cost table "
                         "of the FFMA engine was measured")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.time_shapes:
        import torch

        import exo_b200
        shapes = [tuple(int(x) for x in t.split("x")) for t in args.time_shapes.split(",")]
        rows = run_shapes(exo_b200.library(), torch, measured_peaks(), shapes, ("ffma",), {"fp32_simt_computed": 74.45})
        print(json.dumps({"forced_tile": os.environ.get("EXOB200_FFMA_TILE"),
                          "us": {"x".join(map(str, r["shape"])): round(r["ffma"]["us"], 2) for r in rows}}))
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
