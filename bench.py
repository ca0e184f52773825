"""Benchmark of the matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

Headline workload (default): configuration 2 of the benchmark list -- bf16 batched matmul
A[16,2048,2048] @ B[16,2048,2048], f32 accumulate, bf16 output, seeded synthetic operands
(N(0,1)/sqrt(2048), generated in f32 on the host, narrowed to bf16 on the device by this
library's cast kernel).  One step = one call of `hodu_b200_matmul` on that input.

With N > 1 ranks (torchrun, one per GPU) the ONE configuration is sharded over the ranks the way
the configurations name it: whole batches for config 2, rows of A / tokens for configs 3, 4, 5,
with B and the weights replicated on every GPU and no collective on the compute path.  The
whole-job value is the configuration's flops / the slowest rank's time ("strong" scaling).
`--scaling weak` runs the whole configuration on every rank instead.

Prints ONE JSON line on rank 0.  `value` = device-resident throughput of the headline workload,
`e2e` = the same metric through the host-buffer entry point (pinned host operands in, host result
out, copies inside the timed region), `roofline` = achieved / measured tensor peak for the GEMM
kernel, `cpu_baseline` = the reference's own CPU matmul (its C kernel over OpenBLAS sgemm,
compiled from the reference sources into oracle/_ref) timed on this box's host cores, and
`configs` = one sub-record per other configuration (config 1, 3, 4, 5 and the two input casts):
value, time per step over a region of at least 50 ms, roofline, clocks, and a sampled check of
the result against the CPU oracle made outside the timed region.

`--impl reference` times only that CPU implementation, on the same configuration.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {
    "c1": "f32 matmul A[512,1024] @ B[1024,768] (config 1)",
    "c2": "bf16 batched matmul A[16,2048,2048] @ B[16,2048,2048] -> bf16 (config 2)",
    "c3": "f8e4m3 matmul A[8192,8192] @ B[8192,8192], scales 1/64 -> bf16 (config 3)",
    "c4": "i8 matmul A[8192,8192] @ B[8192,8192] -> i32 (config 4)",
    "c5": "SwiGLU MLP X[16384,4096], W_gate/W_up [4096,14336], W_down [14336,4096] bf16 (config 5)",
    "cast_bf16": "cast f32 -> bf16 of 67,108,864 contiguous elements (input preparation of one config 2 operand)",
    "cast_e4m3": "cast f32 -> f8e4m3 of 67,108,864 contiguous elements (input preparation of one config 3 operand)",
}
# the widened rows (not BASELINE configs): one representative shape each
WIDENED = {
    "linear": "Linear with bias, X[8192,4096] . W[4096,4096]^T + b[4096], bf16 (hodu_nn::Linear forward, one launch)",
    "einsum_qk": "einsum bhqd,bhkd->bhqk, b=4 h=16 q=k=2048 d=128, bf16 (attention scores; 512 MiB written: HBM-bound)",
    "conv3x3": "conv2d NCHW batch 32, 64->64 channels, 56x56, 3x3, padding 1, bf16",
    "proj": "bf16 matmul X[1024,4096] . W[4096,1024] (a projection on 1024 tokens: 32 output tiles, K slices inside one launch)",
}
WORKLOADS.update(WIDENED)
CAST_WORKLOADS = {"cast_bf16": ("bf16", 2), "cast_e4m3": ("f8e4m3", 1)}  # destination dtype, its size
CAST_ELEMS = 67_108_864
# DRAM bytes per launch of the dominant kernel, from the ncu captures summarised in profiles/
# (None until a capture of that workload exists): bytes, the summary, the kernel's source file and
# the hash its code (comments stripped, see kernel_source_sha) had when the capture was made -- the
# line says whether it has changed since.
_PAIR512 = "profiles/gemm_tc_pair512_tma_tail_configs2_3_4_5.md"
_CAST = "profiles/cast_contig_f32_to_bf16_e4m3_67M_elements.md"
NCU_TRAFFIC = {
    "c2": (408.6e6, _PAIR512, "gemm_tc.cu", "e02de8ed4f31"),
    "c3": (496.5e6, _PAIR512, "gemm_tc.cu", "e02de8ed4f31"),
    "c4": (630.2e6, _PAIR512, "gemm_tc.cu", "e02de8ed4f31"),
    "c5": (3410.4e6, _PAIR512, "gemm_tc.cu", "e02de8ed4f31"),   # the SwiGLU launch (the dominant one)
    "c1": (5.27e6, "profiles/gemm_f32_fused_config1.md", "gemm_f32_fused.cu", "168a3092a7ed"),
    "proj": (16.85e6, "profiles/gemm_tc_1cta_k_slices_projection_1024x4096x1024.md", "gemm_tc.cu", "e02de8ed4f31"),
    "conv3x3": (12.95e6, "profiles/conv_implicit_3x3_64ch_56x56_batch32.md", "conv_implicit.cu", "731a333da663"),   # the GEMM launch
    "cast_bf16": (365.0e6, _CAST, "cast.cu", "ccade9e24509"),
    "cast_e4m3": (312.0e6, _CAST, "cast.cu", "ccade9e24509"),
}
NOMINAL_PEAK_TFLOPS = {"c1": 1100.0, "c2": 2250.0, "c3": 4500.0, "c4": 4500.0, "c5": 2250.0,
                       "linear": 2250.0, "einsum_qk": 2250.0, "conv3x3": 2250.0, "proj": 2250.0}
SUB_CONFIGS_1GPU = ["c1", "c3", "c4", "c5", "cast_bf16", "cast_e4m3", "proj"]
SUB_CONFIGS_SHARDED = ["c3", "c4", "c5"]     # config 1 does not shard (replicas only); casts are input preparation
MIN_REGION_MS = 50.0


def kernel_source_sha(file_name: str) -> str:
    """Hash of a kernel source without its // comments, blank lines and indentation: an edit of a
    comment does not make a capture stale, an edit of the code does."""
    p = os.path.join(ROOT, "hodu_b200", "csrc", file_name)
    if not os.path.exists(p):
        return "missing"
    h = hashlib.sha256()
    for line in open(p, encoding="utf-8", errors="replace"):
        code = line.split("//", 1)[0].strip()
        if code:
            h.update(code.encode() + b"\n")
    return h.hexdigest()[:12]


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return {"burst": float(d["bf16_tflops"]), "sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "hbm_gbs": float(d.get("hbm_gbs", 0)), "source": "measured"}
        except Exception:
            pass
    return {"burst": 1590.0, "sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with NVML while a timed region runs:
    back to back, so that even a region of a few milliseconds gets ten or more samples."""

    def __init__(self, uuid: str):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._first = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if isinstance(uuid, str) else uuid)
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._first.set()
            time.sleep(0.0001)

    def __enter__(self):
        if self.nv is not None:
            # a short switch interval, so that the sampling thread is not kept waiting for the
            # interpreter lock while the main thread issues launches
            self._switch = sys.getswitchinterval()
            sys.setswitchinterval(1e-4)
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
            self._first.wait(0.5)   # the region starts with the sampler already running
            self.samples.clear()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._t is not None:
            self._t.join()
            sys.setswitchinterval(self._switch)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_min_mhz": min(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------ reference CPU arm
def cpu_reference_rate(workload: str, budget_s: float):
    """Times the reference's CPU matmul (oracle/_ref: hodu_cpu_matmul_f32 / hodu_cpu_dot_f32 over
    OpenBLAS sgemm; falls back to the oracle restatement's sgemm form if _ref is absent) on a
    bounded sample of `workload`.  Returns (TFLOP/s, kind, cores, sample text, seconds)."""
    from hodu_b200.layout import Layout
    from hodu_b200.op_metadatas import dot_metadata, matmul_metadata
    from oracle import oracle as O

    ref = O.ref()
    have_blas = ref is not None and ref.blas is not None
    kind = "reference" if have_blas else "port"
    if have_blas:   # all host cores, whatever OMP_NUM_THREADS the launcher exported
        ref.set_blas_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    cores = ref.blas_info()["threads"] if have_blas else (os.cpu_count() or 1)

    def run(a, b, md, is_dot):
        out = np.empty(int(md[0]) * int(md[2]) if is_dot else int(md[0]), dtype=np.float32)
        t0 = time.perf_counter()
        if have_blas:
            ref.call("hodu_cpu_dot_f32" if is_dot else "hodu_cpu_matmul_f32", a, b, out, md)
        else:
            O.matmul(a, b, md, O.F32, is_dot=is_dot)
        return time.perf_counter() - t0

    rng = np.random.default_rng(0)
    if workload == "c2":
        d = 2048
        one = Layout.from_shape((1, d, d))
        a1 = (rng.standard_normal((1, d, d), dtype=np.float32) / 45.25).astype(np.float32)
        b1 = (rng.standard_normal((1, d, d), dtype=np.float32) / 45.25).astype(np.float32)
        t1 = run(a1, b1, matmul_metadata(one, one, one), False)            # warm-up + probe
        t1 = min(t1, run(a1, b1, matmul_metadata(one, one, one), False))
        nb = int(max(1, min(16, budget_s / max(t1, 1e-6))))
        lay = Layout.from_shape((nb, d, d))
        a = np.repeat(a1, nb, axis=0)
        b = np.repeat(b1, nb, axis=0)
        t = run(a, b, matmul_metadata(lay, lay, lay), False)
        flops = 2.0 * nb * d ** 3
        sample = f"{nb} of 16 batches of config 2 (operands widened to f32 beforehand, one hodu_cpu_matmul_f32 call)"
    else:
        # the widened rows are timed as the f32 product of their GEMM shape (the reference's CPU
        # conv2d / einsum kernels are scalar loops; its OpenBLAS build unfolds and calls sgemm too)
        shapes = {"c1": (512, 1024, 768), "c3": (8192, 8192, 8192), "c4": (8192, 8192, 8192), "c5": (16384, 4096, 14336),
                  "linear": (8192, 4096, 4096), "einsum_qk": (2048, 128, 2048), "conv3x3": (64, 576, 3136),
                  "proj": (1024, 4096, 1024)}
        m, k, n = shapes[workload]
        b = rng.standard_normal((k, n), dtype=np.float32)
        probe_rows = min(m, 512)
        a = rng.standard_normal((probe_rows, k), dtype=np.float32)
        md = dot_metadata(Layout.from_shape(a.shape), Layout.from_shape(b.shape))
        t1 = run(a, b, md, True)
        t1 = min(t1, run(a, b, md, True))
        rows = int(max(probe_rows, min(m, probe_rows * (budget_s / max(t1, 1e-6)))))
        rows = max(128, rows // 128 * 128) if rows >= 128 else rows
        a = rng.standard_normal((rows, k), dtype=np.float32)
        md = dot_metadata(Layout.from_shape(a.shape), Layout.from_shape(b.shape))
        t = run(a, b, md, True)
        flops = 2.0 * rows * k * n
        sample = f"{rows} of {m} rows of the {m}x{k}x{n} product (f32 operands, one hodu_cpu_dot_f32 call)"
    return flops / t / 1e12, kind, cores, sample, t


def cpu_reference_cast_rate(workload: str, budget_s: float):
    """Times the reference's CPU cast (oracle/_ref: hodu_cpu_cast_f32_to_{bf16,f8e4m3}; the oracle's
    numpy codec if _ref is absent) on a bounded sample.  Returns (GB/s, kind, cores, sample, seconds)."""
    from hodu_b200.layout import Layout
    from hodu_b200.op_metadatas import cast_metadata
    from oracle import oracle as O

    dst_name, dst_size = CAST_WORKLOADS[workload]
    ref = O.ref()
    n = 1 << 22
    x = np.random.default_rng(0).standard_normal(n, dtype=np.float32)
    out = np.empty(n, dtype=np.uint16 if dst_size == 2 else np.uint8)
    md = cast_metadata(Layout.from_shape((n,)))

    def run():
        t0 = time.perf_counter()
        if ref is not None:
            ref.cast(f"hodu_cpu_cast_f32_to_{dst_name}", x, out, md)
        else:
            O.narrow(x, O.BF16 if dst_name == "bf16" else O.F8E4M3)
        return time.perf_counter() - t0

    run()
    reps, total = 0, 0.0
    while total < min(budget_s, 5.0) and reps < 200:
        total += run()
        reps += 1
    secs = total / reps
    # the reference's cast spawns min(online CPUs, elements / 100000) pthreads per call
    cores = min(os.cpu_count() or 1, n // 100000) if ref is not None else 1
    return (n * (4 + dst_size) / secs / 1e9, "reference" if ref is not None else "port", cores,
            f"{n} of {CAST_ELEMS} elements, mean of {reps} calls", secs)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    per_step = max(0.05, min(3.0, 120.0 / max(1, args.steps + args.warmup)))
    is_cast = args.workload in CAST_WORKLOADS
    rate = cpu_reference_cast_rate if is_cast else cpu_reference_rate
    unit = "GB/s" if is_cast else "TFLOP/s"
    for _ in range(args.warmup):
        rate(args.workload, per_step)
    vals, secs = [], []
    sample = kind = ""
    cores = 1
    for _ in range(args.steps):
        v, kind, cores, sample, t = rate(args.workload, per_step)
        vals.append(v)
        secs.append(t)
    value = statistics.mean(vals)
    line = {
        "impl": "reference", "metric": "cast throughput" if is_cast else "matmul throughput", "value": value,
        "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(secs),
        "higher_is_better": True, "scaling": scaling_label(args, args.gpus), "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": config_dict(args.workload, args.scaling != "weak"),
        "note": ("reference CPU cast kernel (hodu_cpu_kernels ops_cast.c, its own pthreads) on host cores; each step is a bounded sample" if is_cast else
                 "reference CPU path (hodu_cpu_kernels C kernel over OpenBLAS sgemm) on host cores; each step is a bounded sample; "
                 "the CPU arm does not shard: rank 0 alone times it"),
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def config_dict(workload: str, strong: bool) -> dict:
    """The `config` object: the same for this library's arm and for the reference arm."""
    return {"workload": WORKLOADS[workload],
            "per_gpu": ("1/N of the configuration: whole batches (c2) or rows of A / tokens, B and weights replicated, no collective"
                        if strong else "the whole configuration on every GPU (independent batches / rows, no collective)"),
            "l2": ("operands + output exceed the 126 MB L2 (no flush needed)" if workload not in ("c1", "conv3x3")
                   else "fits in L2 (latency-bound case)" if workload == "c1"
                   else "input 12.8 MB fits in L2")}


def scaling_label(args, world: int) -> str:
    """auto = the sharding the configurations name (one fixed problem over the GPUs)."""
    return "weak" if args.scaling == "weak" else "strong"


# ------------------------------------------------------------------ GPU arm
class Workload:
    """Device-resident operands of one configuration plus the call that runs one step."""

    def __init__(self, name: str, dev, stream_ptr: int, shard=(0, 1)):
        """shard = (rank, world): with world > 1 this rank keeps only its slice of the fixed
        problem -- whole batches for c2, rows of A / tokens for c3, c4, c5 (B and the weights stay
        whole on every rank)."""
        import torch
        from hodu_b200 import DType, Layout
        from hodu_b200 import kernels as K
        from hodu_b200 import synthetic as S
        from hodu_b200.nn import Linear, SwiGluMlp
        from hodu_b200.op_metadatas import cast_metadata, dot_metadata, matmul_metadata
        from hodu_b200.tensor import Tensor

        self.name, self.K, self.torch, self.dev = name, K, torch, dev
        self.bound, self.alg_bytes, self.write_bytes = ("hbm" if name in CAST_WORKLOADS else "tensor"), None, None
        self.host = None     # host-side source values kept for the parity check
        self.units = "rows"
        d0 = dev.index or 0
        self.d0 = d0

        def cast_on_device(x32: np.ndarray, dt):
            t = torch.from_numpy(x32).pin_memory().to(dev, non_blocking=True)
            return Tensor.from_torch(t).to_dtype(dt).storage

        from hodu_b200.dist import shard_range
        rank, world = shard
        if name == "c2":
            c = S.config2()
            lo, hi = shard_range(c["a"].shape[0], rank, world)
            c = {"a": c["a"][lo:hi], "b": c["b"][lo:hi]}
            self.a, self.b = cast_on_device(c["a"], DType.BF16), cast_on_device(c["b"], DType.BF16)
            lay = Layout.from_shape(c["a"].shape)
            self.md = matmul_metadata(lay, lay, lay)
            self.out = torch.empty(lay.size(), dtype=torch.bfloat16, device=dev)
            self.flops, self.dtype, self.launches = float(S.FLOPS[2]) * (hi - lo) / 16.0, "bf16", 1
            self.in_dt, self.out_dt, self.scales, self.is_dot = DType.BF16, DType.BF16, (1.0, 1.0), False
            self.host = {"a0": c["a"][0], "b0": c["b"][0]} if hi > lo else None
            self.shard_text = f"batches [{lo},{hi}) of 16"
            self.step = lambda: K.call_ops_matmul(K.matmul.BF16, d0, self.a.data_ptr(), self.b.data_ptr(),
                                                  self.out.data_ptr(), self.md, stream_ptr)
        elif name in ("c3", "c4", "c1"):
            c = {"c3": S.config3, "c4": S.config4, "c1": S.config1}[name]()
            lo, hi = 0, c["a"].shape[0]
            if name != "c1":
                lo, hi = shard_range(c["a"].shape[0], rank, world)
                c["a"] = np.ascontiguousarray(c["a"][lo:hi])
            if name == "c3":
                self.a, self.b = cast_on_device(c["a"], DType.F8E4M3), cast_on_device(c["b"], DType.F8E4M3)
                self.in_dt, self.out_dt, self.scales, self.dtype = DType.F8E4M3, DType.BF16, (c["scale_a"], c["scale_b"]), "f8e4m3"
            elif name == "c4":
                self.a, self.b = torch.from_numpy(c["a"]).to(dev).reshape(-1), torch.from_numpy(c["b"]).to(dev).reshape(-1)
                self.in_dt, self.out_dt, self.scales, self.dtype = DType.I8, DType.I32, (1.0, 1.0), "i8"
            else:
                self.a, self.b = torch.from_numpy(c["a"]).to(dev).reshape(-1), torch.from_numpy(c["b"]).to(dev).reshape(-1)
                self.in_dt, self.out_dt, self.scales, self.dtype = DType.F32, DType.F32, (1.0, 1.0), "f32"
            m, k = c["a"].shape
            n = c["b"].shape[1]
            self.mkn = (m, k, n)
            self.md = dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n)))
            from hodu_b200.dtype import to_torch
            self.out = torch.empty(m * n, dtype=to_torch(self.out_dt), device=dev)
            self.flops, self.launches, self.is_dot = 2.0 * m * n * k, 1, True
            self.host = {"a": c["a"], "b": c["b"]}
            self.shard_text = f"rows [{lo},{hi}) of A"
            self.step = lambda: K.call_ops_matmul_ex(self.in_dt, self.out_dt, d0, self.a.data_ptr(), self.b.data_ptr(),
                                                     self.out.data_ptr(), self.md, self.scales[0], self.scales[1],
                                                     stream_ptr, is_dot=True)
        elif name == "c5":
            c = S.config5()
            lo, hi = shard_range(c["x"].shape[0], rank, world)
            c["x"] = np.ascontiguousarray(c["x"][lo:hi])
            x = Tensor(cast_on_device(c["x"], DType.BF16), Layout.from_shape(c["x"].shape))
            lin = lambda w: Linear(Tensor(cast_on_device(np.ascontiguousarray(w.T), DType.BF16), Layout.from_shape(w.T.shape)))
            self.mlp = SwiGluMlp(lin(c["w_gate"]), lin(c["w_up"]), lin(c["w_down"]))
            self.x = x
            self.flops, self.dtype, self.launches = float(S.FLOPS[5]) * (hi - lo) / 16384.0, "bf16", 2
            self.host = c
            self.shard_text = f"tokens [{lo},{hi})"
            self.y = None

            def step():
                self.y = self.mlp.forward(self.x)
            self.step = step
            self.md = None
        elif name == "linear":
            g = torch.Generator(device=dev).manual_seed(11)
            m, k, n = 8192, 4096, 4096
            x = Tensor.from_torch((torch.randn(m, k, generator=g, device=dev)).bfloat16())
            w = Tensor.from_torch((torch.randn(n, k, generator=g, device=dev) / 64).bfloat16())
            bias = Tensor.from_torch(torch.randn(n, generator=g, device=dev).bfloat16())
            self.layer = Linear(w, bias)
            self.flops, self.dtype, self.launches = 2.0 * m * n * k, "bf16", 1
            self.step = lambda: self.layer.forward(x)
        elif name == "proj":
            g = torch.Generator(device=dev).manual_seed(14)
            m, k, n = 1024, 4096, 1024
            self.a = (torch.randn(m * k, generator=g, device=dev) / 8).bfloat16()
            self.b = (torch.randn(k * n, generator=g, device=dev) / 8).bfloat16()
            self.out = torch.empty(m * n, dtype=torch.bfloat16, device=dev)
            self.md = dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n)))
            self.flops, self.dtype, self.launches = 2.0 * m * n * k, "bf16", 1
            # the wrapper's own call, output allocated once: a 15 us product would otherwise be
            # timed at the rate Python allocates tensors
            self.step = lambda: K.call_ops_dot(K.dot.BF16, d0, self.a.data_ptr(), self.b.data_ptr(),
                                               self.out.data_ptr(), self.md, stream_ptr)
        elif name == "einsum_qk":
            from hodu_b200.tensor import einsum
            g = torch.Generator(device=dev).manual_seed(12)
            b_, h_, q_, d_ = 4, 16, 2048, 128
            qt = Tensor.from_torch(torch.randn(b_, h_, q_, d_, generator=g, device=dev).bfloat16())
            kt = Tensor.from_torch(torch.randn(b_, h_, q_, d_, generator=g, device=dev).bfloat16())
            self.flops, self.dtype, self.launches = 2.0 * b_ * h_ * q_ * q_ * d_, "bf16", 1
            self.alg_bytes = 2.0 * (2 * b_ * h_ * q_ * d_ + b_ * h_ * q_ * q_)   # Q and K read, scores written
            self.write_bytes = 2.0 * b_ * h_ * q_ * q_
            self.bound = "hbm"
            self.step = lambda: einsum("bhqd,bhkd->bhqk", [qt, kt])
        elif name == "conv3x3":
            from hodu_b200.op_metadatas import conv2d_metadata
            g = torch.Generator(device=dev).manual_seed(13)
            b_, ci, co, hw = 32, 64, 64, 56
            self.a = torch.randn(b_ * ci * hw * hw, generator=g, device=dev).bfloat16()
            self.b = (torch.randn(co * ci * 9, generator=g, device=dev) / 24).bfloat16()
            self.md = conv2d_metadata(b_, ci, co, (hw, hw), (3, 3), (1, 1), (1, 1))
            self.out = torch.empty(self.md[0], dtype=torch.bfloat16, device=dev)
            self.flops, self.dtype, self.launches = 2.0 * self.md[0] * ci * 9, "bf16", 2
            # implicit GEMM: input read twice (re-laying pass, then the product: the second read is an
            # L2 hit when the input fits), re-laid copy written, weights, output written
            self.alg_bytes = 2.0 * (3 * b_ * ci * hw * hw + 2 * co * ci * 9 + self.md[0])
            self.write_bytes = 2.0 * (b_ * ci * hw * hw + self.md[0])
            self.bound = "tensor"
            self.step = lambda: K.call_ops_conv(K.conv2d.BF16, d0, self.a.data_ptr(), self.b.data_ptr(),
                                                self.out.data_ptr(), self.md, stream_ptr)
        elif name in CAST_WORKLOADS:
            # HBM-bound leg: algorithmic bytes per element = 4 (f32 read) + size of the destination.
            dst_name, dst_size = CAST_WORKLOADS[name]
            dst_dt = {"bf16": DType.BF16, "f8e4m3": DType.F8E4M3}[dst_name]
            g = torch.Generator(device=dev).manual_seed(7)
            self.a = torch.randn(CAST_ELEMS, generator=g, device=dev, dtype=torch.float32)
            from hodu_b200.dtype import to_torch
            self.out = torch.empty(CAST_ELEMS, dtype=to_torch(dst_dt), device=dev)
            self.md = cast_metadata(Layout.from_shape((CAST_ELEMS,)))
            kern = getattr(K.cast, f"F32_{dst_name.upper()}")
            self.flops, self.dtype, self.launches = float(CAST_ELEMS) * (4 + dst_size), f"f32->{dst_name}", 1
            self.write_bytes = float(CAST_ELEMS) * dst_size
            self.step = lambda: K.call_ops_cast(kern, d0, self.a.data_ptr(), self.out.data_ptr(), self.md, stream_ptr)
        else:
            raise SystemExit(f"unknown workload {name}")

    # ---- parity of the last step's result, sampled, against the CPU oracle ----------------------
    def check(self):
        """Compares a sample of what the last `step()` wrote with the CPU oracle (codecs and a
        float64 / f32 product in numpy).  Runs outside every timed region.  Returns a dict with
        `pass`, or None where this workload has no check here (the tests cover it)."""
        from oracle import oracle as O
        torch, dev = self.torch, self.dev
        rng = np.random.default_rng(12345)
        torch.cuda.synchronize(dev)
        try:
            if self.name == "c2" and self.host is not None:
                d = 2048
                rows = np.sort(rng.choice(d, 16, replace=False))
                a = O.bf16_to_f32(O.f32_to_bf16(self.host["a0"][rows]))
                b = O.bf16_to_f32(O.f32_to_bf16(self.host["b0"]))
                want = O.bf16_to_f32(O.f32_to_bf16((a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)))
                got = self.out.view(-1, d, d)[0][torch.from_numpy(rows).to(dev)].float().cpu().numpy()
                err, tol, what = O.rel_err(got, want), 1e-2, "16 rows of batch 0 of this rank's shard"
            elif self.name in ("c3", "c4", "c1"):
                m, k, n = self.mkn
                rows = np.sort(rng.choice(m, min(16, m), replace=False))
                cols = np.sort(rng.choice(n, min(512, n), replace=False))
                a, b = self.host["a"][rows], self.host["b"][:, cols]
                ridx, cidx = torch.from_numpy(rows).to(dev), torch.from_numpy(cols).to(dev)
                got_t = self.out.view(m, n)[ridx][:, cidx]
                what = f"{len(rows)} rows x {len(cols)} columns of this rank's output"
                if self.name == "c3":
                    af, bf = O.e4m3_to_f32(O.f32_to_e4m3(a)), O.e4m3_to_f32(O.f32_to_e4m3(b))
                    want = (af.astype(np.float64) @ bf.astype(np.float64)) * (self.scales[0] * self.scales[1])
                    want = O.bf16_to_f32(O.f32_to_bf16(want.astype(np.float32)))
                    err, tol = O.rel_err(got_t.float().cpu().numpy(), want), 6e-2
                elif self.name == "c4":
                    want = np.rint(a.astype(np.float64) @ b.astype(np.float64)).astype(np.int64)
                    err, tol = float(np.abs(got_t.cpu().numpy().astype(np.int64) - want).max()), 0.0
                    what += " (bit-exact)"
                else:
                    want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
                    err, tol = O.rel_err(got_t.cpu().numpy(), want), 1e-4
            elif self.name == "c5":
                c = self.host
                m = c["x"].shape[0]
                rows = np.sort(rng.choice(m, min(8, m), replace=False))
                cols = np.sort(rng.choice(c["w_down"].shape[1], 256, replace=False))
                rb = lambda x: O.bf16_to_f32(O.f32_to_bf16(np.ascontiguousarray(x)))
                xf, gf, uf, df = rb(c["x"][rows]), rb(c["w_gate"]), rb(c["w_up"]), rb(c["w_down"][:, cols])
                h = O.widen(O.swiglu_hidden(xf, gf, uf, O.BF16, round_each_op=True), O.BF16)
                want = rb(np.matmul(h, df).astype(np.float32))
                y = self.y.storage.view(m, -1)
                got = y[torch.from_numpy(rows).to(dev)][:, torch.from_numpy(cols).to(dev)].float().cpu().numpy()
                err, tol, what = O.rel_err(got, want), 1e-2, "8 tokens x 256 output features, op-by-op rounding form"
            elif self.name in CAST_WORKLOADS:
                n = 1 << 20
                src = self.a[:n].cpu().numpy()
                if self.name == "cast_bf16":
                    want = O.f32_to_bf16(src)
                    got = self.out[:n].view(torch.int16).cpu().numpy().view(np.uint16)
                else:
                    want = O.f32_to_e4m3(src)
                    got = self.out[:n].view(torch.uint8).cpu().numpy()
                err, tol, what = float((got != want).sum()), 0.0, f"first {n} elements (bit-exact)"
            elif self.name == "proj":
                m, k, n = 1024, 4096, 1024
                rows = np.sort(rng.choice(m, 16, replace=False))
                ridx = torch.from_numpy(rows).to(dev)
                a = self.a.view(m, k)[ridx].float().cpu().numpy()
                b = self.b.view(k, n).float().cpu().numpy()
                want = O.bf16_to_f32(O.f32_to_bf16((a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)))
                got = self.out.view(m, n)[ridx].float().cpu().numpy()
                err, tol, what = O.rel_err(got, want), 1e-2, "16 rows of the output"
            else:
                return None
        except Exception as e:   # a failed check must not lose the measurement: report it as such
            return {"pass": False, "error": f"{type(e).__name__}: {e}"}
        return {"pass": bool(err <= tol), "err": float(err), "tol": tol, "sample": what,
                "oracle": "numpy float64 product of the oracle-decoded operands, one rounding to the output dtype"}

    # ---- the end-to-end call: host buffers in, host result out ----------------------------------
    def e2e_call(self):
        """Returns (callable, h2d bytes, d2h bytes, api text) or None."""
        torch, K = self.torch, self.K
        if self.name in ("c1", "c2", "c3", "c4"):
            ha = self.a.view(torch.uint8).cpu().pin_memory()
            hb = self.b.view(torch.uint8).cpu().pin_memory()
            ho = torch.empty(self.out.numel() * self.out.element_size(), dtype=torch.uint8).pin_memory()
            self._pinned = (ha, hb, ho)
            call = lambda: K.call_ops_matmul_host(self.in_dt, self.out_dt, self.d0, ha.data_ptr(), hb.data_ptr(),
                                                  ho.data_ptr(), self.md, self.scales[0], self.scales[1],
                                                  is_dot=self.is_dot)
            return call, int(ha.numel() + hb.numel()), int(ho.numel()), (
                "hodu_b200_matmul_host / hodu_b200_dot_host (pinned host operands, host result; wall clock around the blocking call)")
        if self.name == "c5":
            hx = self.x.storage.view(torch.uint8).cpu().pin_memory()
            tokens = self.x.shape[0]
            hy = torch.empty(tokens * self.mlp.down.weight.shape[0] * 2, dtype=torch.uint8).pin_memory()
            self._pinned = (hx, hy)
            call = lambda: self.mlp.forward_host(hx.data_ptr(), hy.data_ptr(), tokens)
            return call, int(hx.numel()), int(hy.numel()), (
                "hodu_b200_swiglu_mlp_host (pinned host activations in, host result out, weights resident on the "
                "device as module parameters; wall clock around the blocking call)")
        return None


def timed_steps(wl, steps, stream, dev, uuid, barrier):
    """`steps` back-to-back calls between two CUDA events on the launching stream, clocks sampled
    while they run.  Returns (ms_total, clocks summary, launches)."""
    torch, K = wl.torch, wl.K
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches0 = K.launch_count()
    with ClockSampler(uuid) as clocks:
        e0.record(stream)
        for _ in range(steps):
            wl.step()
        e1.record(stream)
        torch.cuda.synchronize(dev)
    barrier()
    return e0.elapsed_time(e1), clocks.summary(), K.launch_count() - launches0


def roofline_of(name, wl, ms_step, timed_s, clk, peaks):
    """The roofline object for one rank's launch group."""
    hbm_bound = wl.bound == "hbm"
    is_cast = name in CAST_WORKLOADS
    per_unit = 1e9 if is_cast else 1e12
    if hbm_bound:
        peak, peak_src = peaks["hbm_gbs"], (f"{peaks['source']} copy bandwidth (MEASURED_PEAKS.json)"
                                            if peaks["source"] == "measured" else "fallback 6650 GB/s")
    elif name in ("c2", "c5", "linear"):
        # cuBLAS burst for a short region at full clocks; its sustained figure once the region is
        # long or the power cap was seen active while it ran
        peak_kind = "sustained" if (timed_s >= 1.0 or "sw_power_cap" in clk["reasons"]) else "burst"
        peak, peak_src = peaks[peak_kind], (f"{peaks['source']} cuBLAS bf16 {peak_kind} (MEASURED_PEAKS.json)"
                                            if peaks["source"] == "measured" else "fallback 1590 burst / 1400 sustained")
    else:
        peak, peak_src = NOMINAL_PEAK_TFLOPS[name], "nominal dense peak for this dtype (no measured figure for it)"
    achieved = wl.flops / (ms_step * 1e-3) / per_unit
    if hbm_bound and not is_cast:   # a product whose algorithmic bytes, not flops, bound it
        achieved = wl.alg_bytes / (ms_step * 1e-3) / 1e9
    traffic, traffic_src, kernel_file, sha_then = NCU_TRAFFIC.get(name, (None, None, None, None))
    r = {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": "GB/s" if hbm_bound else "TFLOP/s",
         "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src}
    if traffic is not None:
        sha = kernel_source_sha(kernel_file)
        r["traffic_source"] = traffic_src
        r["traffic_kernel_sha"] = {"file": kernel_file, "captured": sha_then, "now": sha,
                                   "kernel_changed_since_capture": sha != sha_then}
    if not hbm_bound:
        r["frac_of_nominal"] = achieved / NOMINAL_PEAK_TFLOPS[name]
    else:
        r["algorithmic_bytes_per_step"] = wl.flops if is_cast else wl.alg_bytes
    return r


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=20)
    ap.add_argument("--scaling", default="auto", choices=["auto", "weak", "strong"],
                    help="auto / strong: the one configuration is sharded over the GPUs as the configurations name it; "
                         "weak: every GPU runs the whole configuration")
    ap.add_argument("--configs", default="auto",
                    help="sub-records beside the headline: auto (the other configurations when the headline is c2), "
                         "none, or a comma list such as c3,c4")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--all-gather", action="store_true",
                    help="N > 1: also time an NCCL all-gather of the outputs (reported separately)")
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="after the timed region: per-step best/median and a back-to-back run of this length (0 = skip)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import torch.distributed as dist
    from hodu_b200 import _lib
    from hodu_b200 import kernels as K

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    _lib.lib()  # fails loudly if libhodu_b200.so is missing
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    warmup = max(3, args.warmup)
    stream = torch.cuda.current_stream(dev)
    strong = args.scaling != "weak"
    shard = (rank, world) if strong else (0, 1)
    uuid = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    peaks = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize(dev)

    def reduce_max(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def reduce_sum(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    def run_e2e(wl, total_units, n_steps):
        got = wl.e2e_call()
        if got is None:
            return None
        call, h2d, d2h, api = got
        for _ in range(3):
            call()
        barrier()
        t0 = time.perf_counter()
        for _ in range(n_steps):
            call()  # returns when the result is complete in host memory
        torch.cuda.synchronize(dev)
        e2e_ms = reduce_max((time.perf_counter() - t0) * 1e3) / n_steps
        wl._pinned = None
        return {"value": total_units / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": n_steps, "api": api}

    # =================================================================== headline workload
    wl = Workload(args.workload, dev, stream.cuda_stream, shard=shard)
    for _ in range(warmup):
        wl.step()
    torch.cuda.synchronize(dev)
    K.last_status(local)
    ms_total, clk, launches = timed_steps(wl, args.steps, stream, dev, uuid, barrier)
    K.last_status(local)
    ms_per_step = reduce_max(ms_total) / args.steps
    total_flops = reduce_sum(wl.flops)   # units all ranks process per step
    is_cast = args.workload in CAST_WORKLOADS
    per_unit = 1e9 if is_cast else 1e12   # casts count bytes (GB/s), products count flops (TFLOP/s)
    value = total_flops / (ms_per_step * 1e-3) / per_unit
    parity = wl.check()
    parity_all = reduce_sum(0.0 if (parity is None or parity.get("pass")) else 1.0) == 0.0

    # ---- optional: all-gather of the output over NCCL, timed separately (N > 1) -----------------
    gather = None
    if world > 1 and args.all_gather and hasattr(wl, "out"):
        flat = wl.out.reshape(-1)
        full = torch.empty(flat.numel() * world, dtype=flat.dtype, device=dev)
        for _ in range(2):
            dist.all_gather_into_tensor(full, flat)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 5
        g0.record(stream)
        for _ in range(reps):
            dist.all_gather_into_tensor(full, flat)
        g1.record(stream)
        torch.cuda.synchronize(dev)
        g_ms = reduce_max(g0.elapsed_time(g1) / reps)
        nbytes = flat.numel() * flat.element_size()
        gather = {"ms": g_ms, "bytes_per_rank": int(nbytes),
                  "bus_gbs": nbytes * (world - 1) / (g_ms * 1e-3) / 1e9,
                  "note": "ncclAllGather of every rank's output into a full copy on every rank; not part of `value`"}

    # ---- spread and a sustained figure (1 GPU only; outside the timed region above) -------------
    detail = None
    if world == 1 and args.sustained_seconds > 0:
        n_d = max(5, min(args.steps, 100))
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(n_d + 1)]
        evs[0].record(stream)
        for i in range(n_d):
            wl.step()
            evs[i + 1].record(stream)
        torch.cuda.synchronize(dev)
        per = sorted(evs[i].elapsed_time(evs[i + 1]) for i in range(n_d))
        to_rate = lambda ms: wl.flops / (ms * 1e-3) / per_unit
        n_s = int(min(200000, max(args.steps, args.sustained_seconds * 1e3 / max(ms_per_step, 1e-3))))
        s_ms, sclk, _ = timed_steps(wl, n_s, stream, dev, uuid, barrier)
        detail = {"per_step": {"steps": n_d, "best": to_rate(per[0]), "median": to_rate(per[n_d // 2]),
                               "note": "one CUDA event per step; includes the gap to the previous launch"},
                  "sustained": {"value": to_rate(s_ms / n_s), "seconds": s_ms * 1e-3, "steps": n_s,
                                "frac_of_sustained_peak": (to_rate(s_ms / n_s) / peaks["sustained"]
                                                           if args.workload in ("c2", "c5", "linear") else None),
                                "clocks": sclk}}
        K.last_status(local)

    # ---- e2e through the host-buffer entry point ------------------------------------------------
    e2e = run_e2e(wl, total_flops, max(1, min(args.steps, args.e2e_steps))) if args.e2e_steps > 0 else None
    headline_roof = roofline_of(args.workload, wl, ms_total / args.steps, ms_total * 1e-3, clk, peaks)
    headline_write = None
    if wl.bound == "hbm":
        # HBM takes pure writes more slowly than a copy's mix of reads and writes: time a plain fill of
        # 512 MiB here and now, and say how the bytes this workload WRITES compare with that rate
        buf = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
        for _ in range(3):
            buf.fill_(1)
        w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0.record(stream)
        for _ in range(10):
            buf.fill_(1)
        w1.record(stream)
        torch.cuda.synchronize(dev)
        write_peak = 10 * buf.numel() / (w0.elapsed_time(w1) * 1e-3) / 1e9
        written = wl.write_bytes / (ms_total / args.steps * 1e-3) / 1e9
        headline_write = {"write_peak_gbs": write_peak, "written_gbs": written,
                          "written_frac_of_write_peak": written / write_peak,
                          "write_peak_source": "torch fill_ of 512 MiB timed in this run"}
        del buf
    shard_text = getattr(wl, "shard_text", None)
    del wl
    torch.cuda.empty_cache()

    # =================================================================== the other configurations
    if args.configs == "auto":
        subs = (SUB_CONFIGS_1GPU if world == 1 else SUB_CONFIGS_SHARDED) if args.workload == "c2" else []
    elif args.configs == "none":
        subs = []
    else:
        subs = [s for s in args.configs.split(",") if s in WORKLOADS and s != args.workload]
    configs = {}
    for name in subs:
        rec = {"workload": WORKLOADS[name]}
        try:
            sub_shard = shard if name in SUB_CONFIGS_SHARDED or name == "c2" else (0, 1)
            sw = Workload(name, dev, stream.cuda_stream, shard=sub_shard)
            for _ in range(3):
                sw.step()
            torch.cuda.synchronize(dev)
            probe_ms, _, _ = timed_steps(sw, 5, stream, dev, uuid, barrier)
            est = reduce_max(probe_ms) / 5
            n_steps = int(max(10, min(20000, math.ceil(1.25 * MIN_REGION_MS / max(est, 1e-4)))))
            s_ms, s_clk, s_launches = timed_steps(sw, n_steps, stream, dev, uuid, barrier)
            K.last_status(local)
            ms_step = reduce_max(s_ms) / n_steps
            sub_cast = name in CAST_WORKLOADS
            unit_div = 1e9 if sub_cast else 1e12
            units_total = reduce_sum(sw.flops) if sub_shard != (0, 1) else sw.flops
            rec.update({
                "value": units_total / (ms_step * 1e-3) / unit_div,
                "unit": "GB/s" if sub_cast else ("TOP/s" if name == "c4" else "TFLOP/s"),
                "ms_per_step": ms_step, "steps": n_steps, "timed_region_ms": s_ms, "dtype": sw.dtype,
                "gpu_launches": int(s_launches),
                "sharding": (f"this rank: {sw.shard_text}; B / weights whole on every GPU" if sub_shard != (0, 1) and world > 1
                             else "whole configuration on one GPU"),
                "roofline": roofline_of(name, sw, s_ms / n_steps, s_ms * 1e-3, s_clk, peaks),
                "clocks": s_clk,
            })
            par = sw.check()
            ok_everywhere = reduce_sum(0.0 if (par is None or par.get("pass")) else 1.0) == 0.0
            if par is not None:
                par["pass_on_every_rank"] = ok_everywhere
                rec["parity"] = par
            if world == 1 and args.e2e_steps > 0:
                e = run_e2e(sw, units_total, 5)
                if e is not None:
                    rec["e2e"] = e
            del sw
        except Exception as ex:  # one configuration failing must not lose the headline line
            rec["error"] = f"{type(ex).__name__}: {ex}"
        torch.cuda.empty_cache()
        configs[name] = rec

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    unit = "GB/s" if is_cast else ("TFLOP/s" if args.workload != "c4" else "TOP/s")
    line = {
        "metric": "cast throughput" if is_cast else "matmul throughput", "value": value, "unit": unit,
        "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
        "dtype": {"c1": "f32", "c2": "bf16", "c3": "f8e4m3", "c4": "i8", "c5": "bf16"}.get(args.workload, "bf16"),
        "data": "synthetic",
        "config": config_dict(args.workload, strong),
        "timing": "CUDA events on the launching stream around all timed steps, max over ranks",
        "rank0_shard": shard_text,
        "clocks": clk,
        "gpu_launches": int(launches),
        "roofline": headline_roof,
    }
    if is_cast:
        line["dtype"] = f"f32->{CAST_WORKLOADS[args.workload][0]}"
    if headline_write is not None:
        line["roofline"].update(headline_write)
    if parity is not None:
        parity["pass_on_every_rank"] = parity_all
        line["parity"] = parity
    if e2e is not None:
        line["e2e"] = e2e
    if detail is not None:
        line["spread"] = detail
    if gather is not None:
        line["all_gather"] = gather
    if configs:
        line["configs"] = configs
    if world == 1 and not args.no_cpu_baseline:
        v, kind, cores, sample, secs = (cpu_reference_cast_rate if is_cast else cpu_reference_rate)(args.workload, 15.0)
        line["cpu_baseline"] = {"value": v, "unit": "GB/s" if is_cast else "TFLOP/s", "cores": cores, "kind": kind,
                                "sample": sample, "seconds": secs}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
