#!/usr/bin/env python
"""Benchmark of the dense-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one pass of the hot path over one batch of seeded synthetic input. The headline
workload (default) is BASELINE config 2: fp32 NCHW conv2d N=64 C=64 56x56 -> 64, 3x3, stride 1,
pad 1, with bias, one kernel launch per step. With N GPUs every rank convolves its own batch of
64 images (batch-sharded, no data-path collective, weak scaling). Rank 0 prints ONE JSON line.

Timing: CUDA events on the launching stream around exactly K steps after W warm-up steps,
barrier + synchronize on both sides, max over ranks. Inputs and outputs rotate over several
buffer sets whose total size exceeds the 126 MB L2, so no step finds its operands cached.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time


def _reference_arm_environment():
    """The CPU arm (--impl reference) wants every host core, in the OpenMP runtime of the oracle
    and in the host BLAS alike. Their thread pools are sized when the libraries are loaded, and
    torchrun exports OMP_NUM_THREADS=1, so the variables are set here, before anything that links
    an OpenMP runtime or a BLAS is imported, and the interpreter is started again with them. Idle
    OpenMP workers must sleep (passive wait policy): spinning ones take the cores from the BLAS
    threads that run between two parallel regions."""
    if "--impl" not in sys.argv or os.environ.get("DLF_B200_BENCH_ENV") == "1":
        return
    i = sys.argv.index("--impl")
    if i + 1 >= len(sys.argv) or sys.argv[i + 1] != "reference":
        return
    n = str(os.cpu_count() or 1)
    os.environ.update({"OMP_NUM_THREADS": n, "OPENBLAS_NUM_THREADS": n, "MKL_NUM_THREADS": n,
                       "OMP_WAIT_POLICY": "passive", "GOMP_SPINCOUNT": "0", "DLF_B200_BENCH_ENV": "1"})
    os.execv(sys.executable, [sys.executable] + sys.argv)


_reference_arm_environment()

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
NOMINAL = {"f16": 2250.0, "bf16": 2250.0, "f32": 1125.0 / 3.0}  # dense TFLOP/s; f32 = 3xTF32


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


# ------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------
class Workload:
    """One configuration of BASELINE.json: seeded inputs, a launch per step, algorithmic work."""
    name = ""
    dtype = "f32"
    launches_per_step = 1

    def torch_dtype(self):
        return {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[self.dtype]

    def tensor_peak(self, peaks):
        """Measured dense tensor roof for this dtype: cuBLAS bf16 burst for 16-bit inputs; tf32
        runs at half the bf16 rate and 3xTF32 issues three MMAs per product."""
        return peaks["bf16_tflops"] if self.dtype != "f32" else peaks["bf16_tflops"] / 6.0


class ConvC2(Workload):
    """Config 2: fp32 conv2d NCHW 64x64x56x56 -> 64 channels, 3x3 s1 p1, bias."""
    name = "conv2d_f32_n64_c64_56x56_k3"
    dtype = "f32"
    shape = dict(N=64, C=64, H=56, W=56, Co=64, KH=3, KW=3, pad=1, stride=1, group=1)

    def __init__(self, shape=None, dtype=None):
        if shape:
            self.shape = dict(self.shape, **shape)
        if dtype:
            self.dtype = dtype
        s = self.shape
        self.OH = (s["H"] + 2 * s["pad"] - s["KH"]) // s["stride"] + 1
        self.OW = (s["W"] + 2 * s["pad"] - s["KW"]) // s["stride"] + 1
        es = 4 if self.dtype == "f32" else 2
        self.flops = 2.0 * s["N"] * s["Co"] * self.OH * self.OW * (s["C"] // s["group"]) * s["KH"] * s["KW"]
        self.x_bytes = es * s["N"] * s["C"] * s["H"] * s["W"]
        self.y_bytes = es * s["N"] * s["Co"] * self.OH * self.OW
        self.bytes = self.x_bytes + self.y_bytes + es * s["Co"] * (s["C"] // s["group"]) * s["KH"] * s["KW"] + es * s["Co"]

    def host_inputs(self, seed):
        s = self.shape
        rng = np.random.default_rng(seed)
        X = rng.normal(size=(s["N"], s["C"], s["H"], s["W"])).astype(np.float32)
        std = math.sqrt(2.0 / (s["C"] // s["group"] * s["KH"] * s["KW"]))
        W = (std * rng.normal(size=(s["Co"], s["C"] // s["group"], s["KH"], s["KW"]))).astype(np.float32)
        b = rng.uniform(-0.1, 0.1, s["Co"]).astype(np.float32)
        return X, W, b

    def setup(self, device, seed, sets):
        from dlf_b200 import gdnn
        s = self.shape
        X, W, b = self.host_inputs(seed)
        td = self.torch_dtype()
        self.filt = gdnn.Filter2D(X.shape, W.shape, s["group"]).pads(s["pad"], s["pad"]).strides(s["stride"], s["stride"])
        self.W = torch.from_numpy(W).to(td).to(device)
        self.b = torch.from_numpy(b).to(td).to(device)
        x0 = torch.from_numpy(X).to(td)
        self.host_x = x0.pin_memory()
        self.X = [x0.to(device) for _ in range(sets)]
        self.Y = [torch.empty(self.filt.output_shape(), dtype=td, device=device) for _ in range(sets)]
        self.host_y = torch.empty(self.filt.output_shape(), dtype=td).pin_memory()
        self.sets = sets

    def sets_needed(self):
        return max(2, int(math.ceil(2.0 * L2_BYTES / (self.x_bytes + self.y_bytes))))

    def step(self, i):
        from dlf_b200 import gdnn
        j = i % self.sets
        gdnn.conv2d_filter(self.X[j], self.W, self.Y[j], self.filt, bias=self.b)

    def step_fused(self, i):
        """The same convolution followed by the residual Add and ReLU of a bottleneck's last layer,
        in one launch (profiling aid: --workload conv --residual)."""
        from dlf_b200 import gdnn
        j = i % self.sets
        if not hasattr(self, "R"):
            g = torch.Generator(device=self.Y[0].device).manual_seed(3)
            self.R = [torch.randn(self.Y[0].shape, generator=g, device=self.Y[0].device).to(self.Y[0].dtype)
                      for _ in range(self.sets)]
        gdnn.conv2d_filter(self.X[j], self.W, self.Y[j], self.filt, bias=self.b, residual=self.R[j], activation="relu")

    def step_nhwc(self, i, residual=False):
        """The same convolution between channels-last tensors (profiling aid: --workload conv --layout
        channels_last [--residual]); the copies and the filter packing are made once, outside the step."""
        from dlf_b200 import gdnn
        j = i % self.sets
        if not hasattr(self, "Xn"):
            self.Xn = [gdnn.nchw_to_nhwc(x) for x in self.X]
            self.Wp = gdnn.pack_filters_nhwc(self.W)
            o = self.filt.output_shape()
            self.Yn = [torch.empty((o[0], o[2], o[3], o[1]), dtype=self.Y[0].dtype, device=self.Y[0].device) for _ in range(self.sets)]
            g = torch.Generator(device=self.Y[0].device).manual_seed(3)
            self.Rn = [torch.randn(self.Yn[0].shape, generator=g, device=self.Y[0].device).to(self.Y[0].dtype)
                       for _ in range(self.sets)]
        gdnn.conv2d_nhwc(self.Xn[j], self.Wp, self.Yn[j], self.filt, bias=self.b,
                         residual=self.Rn[j] if residual else None, activation="relu" if residual else None)

    def step_no_workspace(self, i):
        """The same convolution through the C ABI with workspace = NULL (the filter bank is then
        gathered inside the main loop instead of being packed first)."""
        import ctypes
        import dlf_b200
        f = self.filt
        j = i % self.sets
        prec = 32 if self.dtype == "f32" else (16 if self.dtype == "f16" else 1600)
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        rc = dlf_b200.lib().dlf_b200_conv2d(
            prec, f.batches, f.channels, f.height, f.width, f.output_h, f.output_w, f.num_kernels, f.group,
            f.kernel_h, f.kernel_w, f.pad_top, f.pad_left, f.pad_bottom, f.pad_right, f.stride_h, f.stride_w,
            f.dilation_h, f.dilation_w, p(self.X[j]), p(self.W), p(self.b), p(self.Y[j]), None, 0,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError(dlf_b200.status_string(rc))

    def e2e_step(self, i):
        """Public API with host buffers: H2D of the step's input from pinned memory, the
        convolution, D2H of Y into pinned memory - every step. The three run on their own streams
        and rotate over the buffer sets, so the upload of step i + 1 and the download of step
        i - 1 overlap the convolution of step i (PCIe is full duplex), as a serving loop would."""
        from dlf_b200 import tensor as dt
        if not hasattr(self, "_e2e"):
            mk = lambda: [torch.cuda.Event() for _ in range(self.sets)]
            self._e2e = dict(s_in=torch.cuda.Stream(), s_c=torch.cuda.Stream(), s_out=torch.cuda.Stream(),
                             ev_in=mk(), ev_done=mk(), ev_out=mk(), n=0,
                             host_y=[torch.empty_like(self.host_y).pin_memory() for _ in range(self.sets)])
            for st in (self._e2e["s_in"], self._e2e["s_c"], self._e2e["s_out"]):
                st.wait_stream(torch.cuda.current_stream())
        e = self._e2e
        j = e["n"] % self.sets
        reuse = e["n"] >= self.sets
        e["n"] += 1
        with torch.cuda.stream(e["s_in"]):
            if reuse:
                e["s_in"].wait_event(e["ev_done"][j])  # the convolution that read X[j] last
            self.X[j].copy_(self.host_x, non_blocking=True)
            e["ev_in"][j].record(e["s_in"])
        with torch.cuda.stream(e["s_c"]):
            e["s_c"].wait_event(e["ev_in"][j])
            if reuse:
                e["s_c"].wait_event(e["ev_out"][j])   # the download that read Y[j] last
            dt.conv2d(self.X[j], self.W, self.Y[j], self.filt, bias=self.b)
            e["ev_done"][j].record(e["s_c"])
        with torch.cuda.stream(e["s_out"]):
            e["s_out"].wait_event(e["ev_done"][j])
            e["host_y"][j].copy_(self.Y[j], non_blocking=True)
            e["ev_out"][j].record(e["s_out"])

    def e2e_bytes(self):
        return self.x_bytes, self.y_bytes

    def check(self):
        """Spot check of the last output against the oracle (two images)."""
        import oracle
        X, W, b = self.host_inputs(self.seed_used)
        td = self.torch_dtype()
        if td != torch.float32:
            X = torch.from_numpy(X).to(td).float().numpy()
            W = torch.from_numpy(W).to(td).float().numpy()
            b = torch.from_numpy(b).to(td).float().numpy()
        s = self.shape
        ref = oracle.conv2d(X[:2], W, group=s["group"], pads=(s["pad"],) * 4,
                            strides=(s["stride"],) * 2, bias=b, wide=True)
        got = self.Y[0][:2].float().cpu().numpy()
        return float(np.linalg.norm(got - ref) / np.linalg.norm(ref))

    def cpu_reference(self, budget_s):
        """The reference's CPU schedule (dlf/include/tensor/dnn_detail.h:123-152: per image im2col
        then sgemm, serial over the batch; bias as a second pass) with the host BLAS. The thread
        counts of the OpenMP runtime (im2col, bias) and of the BLAS are tried at {1, all cores}
        each, once, and the fastest pair is the one that is timed."""
        import oracle
        X, W, b = self.host_inputs(0)
        fn, desc = oracle.find_host_cblas()
        cb = oracle.host_sgemm_nn_callback(fn) if fn is not None else None
        s = self.shape
        kw = dict(group=s["group"], pads=(s["pad"],) * 4, strides=(s["stride"],) * 2, bias=b, sgemm_nn=cb)
        n_img = min(s["N"], 8)
        cores = os.cpu_count() or 1
        try:
            import threadpoolctl
        except ImportError:
            threadpoolctl = None

        def limited(omp, blas):
            if threadpoolctl is None:
                import contextlib
                return contextlib.nullcontext()
            stack = contextlib_stack()
            stack.enter_context(threadpoolctl.threadpool_limits(limits=omp, user_api="openmp"))
            stack.enter_context(threadpoolctl.threadpool_limits(limits=blas, user_api="blas"))
            return stack

        def contextlib_stack():
            import contextlib
            return contextlib.ExitStack()

        if getattr(self, "_cpu_threads", None) is None:
            best = None
            combos = [(cores, cores), (1, cores), (cores, 1), (1, 1)] if threadpoolctl is not None else [(cores, cores)]
            for omp, blas in combos:
                with limited(omp, blas):
                    oracle.conv2d(X[:2], W, **kw)  # warm-up of the pools at this size
                    dt = None
                    for _ in range(3):
                        t0 = time.perf_counter()
                        oracle.conv2d(X[:4], W, **kw)
                        d = time.perf_counter() - t0
                        dt = d if dt is None or d < dt else dt
                if best is None or dt < best[0]:
                    best = (dt, omp, blas)
            self._cpu_threads = (best[1], best[2])
        omp, blas = self._cpu_threads
        with limited(omp, blas):
            oracle.conv2d(X[:n_img], W, **kw)  # warm-up
            t0 = time.perf_counter()
            reps = 0
            while True:
                oracle.conv2d(X[:n_img], W, **kw)
                reps += 1
                if time.perf_counter() - t0 > budget_s or reps >= 200:
                    break
            dt_s = (time.perf_counter() - t0) / reps
        flops = self.flops * n_img / s["N"]
        return dict(value=flops / dt_s / 1e12, seconds_per_sample=dt_s,
                    seconds_per_full_step=dt_s * s["N"] / n_img, cores=max(omp, blas),
                    sample="%d of %d images per pass, %d passes; im2col (%d OpenMP threads) + %s (%d threads) per "
                           "image, fastest of {1, %d} x {1, %d} threads" % (
                               n_img, s["N"], reps, omp, desc if fn is not None else "oracle sgemm (no host BLAS found)",
                               blas, cores, cores),
                    blas=desc)


class GemmWorkload(Workload):
    """Single or strided-batched GEMM; row-major."""

    def __init__(self, name, dtype, m, n, k, batch=1, ta=False, tb=False, alpha=1.0, beta=0.0, dist="normal"):
        self.name, self.dtype = name, dtype
        self.m, self.n, self.k, self.batch, self.ta, self.tb = m, n, k, batch, ta, tb
        self.alpha, self.beta, self.dist = alpha, beta, dist
        es = 4 if dtype == "f32" else 2
        self.flops = 2.0 * m * n * k * batch
        self.bytes = es * batch * (m * k + k * n + m * n * (2 if beta != 0 else 1))
        self.in_bytes = es * batch * (m * k + k * n)
        self.out_bytes = es * batch * m * n

    def sets_needed(self):
        per = self.bytes
        return max(2, min(8, int(math.ceil(2.0 * L2_BYTES / per))))

    def setup(self, device, seed, sets):
        g = torch.Generator(device=device).manual_seed(seed)
        td = self.torch_dtype()
        self.sets = sets
        mk = (lambda *s: torch.randn(*s, generator=g, device=device, dtype=torch.float32)) if self.dist == "normal" \
            else (lambda *s: torch.rand(*s, generator=g, device=device, dtype=torch.float32) * 2 - 1)
        scale = 0.1 if self.dist == "normal" else 1.0
        self.A = [(mk(self.batch * self.m * self.k) * scale).to(td) for _ in range(sets)]
        self.B = [(mk(self.batch * self.k * self.n) * scale).to(td) for _ in range(sets)]
        self.C = [torch.randn(self.batch * self.m * self.n, generator=g, device=device, dtype=torch.float32).to(td)
                  for _ in range(sets)]

    def step_abi(self, i):
        """The same step straight through the C ABI with arguments converted once (a single GEMM
        only): for products of a few microseconds, where the Python mirror's argument checks would
        set the rate. Scratch for the K-split comes from the workload, as a dlf caller's pool would."""
        import ctypes
        import dlf_b200
        L = dlf_b200.lib()
        if not hasattr(self, "_abi"):
            dt = {"f32": 32, "f16": 16, "bf16": 1600}[self.dtype]
            td = self.torch_dtype()
            self._al = torch.tensor([self.alpha], dtype=td).numpy().tobytes() if td == torch.float32 else \
                torch.tensor([self.alpha], dtype=td).view(torch.int16).numpy().tobytes()
            self._be = torch.tensor([self.beta], dtype=td).numpy().tobytes() if td == torch.float32 else \
                torch.tensor([self.beta], dtype=td).view(torch.int16).numpy().tobytes()
            need = L.dlf_b200_gemm_workspace_bytes(dt, self.m, self.n, self.k)
            self._ws = torch.empty(max(int(need), 1), dtype=torch.uint8, device=self.A[0].device)
            lda = self.m if self.ta else self.k
            ldb = self.k if self.tb else self.n
            P = lambda t: ctypes.c_void_p(t.data_ptr())
            self._abi = [(dt, 101, 112 if self.ta else 111, 112 if self.tb else 111, self.m, self.n, self.k,
                          ctypes.c_char_p(self._al), P(self.A[j]), lda, P(self.B[j]), ldb, ctypes.c_char_p(self._be),
                          P(self.C[j]), self.n, P(self._ws) if need else None, int(need)) for j in range(self.sets)]
        rc = L.dlf_b200_gemm_ex(*self._abi[i % self.sets], ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError("dlf_b200_gemm_ex: %d" % rc)

    def step_sharded(self, i, world, rank):
        """One large GEMM over `world` GPUs: rank r computes its block of rows of C, then the row
        blocks are all-gathered (NCCL) so that every rank holds all of C. Operands are replicated."""
        from dlf_b200 import gblas, shard
        j = i % self.sets
        ta = gblas.Transpose.Trans if self.ta else gblas.Transpose.NoTrans
        tb = gblas.Transpose.Trans if self.tb else gblas.Transpose.NoTrans
        A = self.A[j].view(self.k, self.m) if self.ta else self.A[j].view(self.m, self.k)
        B = self.B[j].view(self.n, self.k) if self.tb else self.B[j].view(self.k, self.n)
        C = self.C[j].view(self.m, self.n)
        if getattr(self, "overlap_gather", False) and self.m % (world * 4 * 128) == 0:
            # four panels: the all-gather of a finished panel overlaps the next panel's GEMM
            shard.gemm_row_sharded_overlapped(ta, tb, self.alpha, A, B, self.beta, C, world, rank, 4)
        else:
            shard.gemm_row_sharded(ta, tb, self.alpha, A, B, self.beta, C, world, rank)

    def step(self, i):
        from dlf_b200 import gblas
        j = i % self.sets
        ta = gblas.Transpose.Trans if self.ta else gblas.Transpose.NoTrans
        tb = gblas.Transpose.Trans if self.tb else gblas.Transpose.NoTrans
        lda = self.m if self.ta else self.k
        ldb = self.k if self.tb else self.n
        if self.batch == 1:
            gblas.gemm(gblas.Layout.RowMajor, ta, tb, self.m, self.n, self.k, self.alpha, self.A[j], 0, lda,
                       self.B[j], 0, ldb, self.beta, self.C[j], 0, self.n)
        else:
            gblas.gemmStridedBatched(gblas.Layout.RowMajor, ta, tb, self.m, self.n, self.k, self.alpha,
                                     self.A[j], 0, lda, self.m * self.k, self.B[j], 0, ldb, self.k * self.n,
                                     self.beta, self.C[j], 0, self.n, self.m * self.n, self.batch)


class GemmBatchedOffsets(GemmWorkload):
    """gemmBatched (per-batch offset tables and scalars, gblas.h:661-671) on the config 4 (i)
    shape with the batch entries visited in a shuffled order; called through the C ABI with the
    host tables built once, as a caller that reuses its tables would."""

    def setup(self, device, seed, sets):
        import ctypes
        super().setup(device, seed, sets)
        rng = np.random.default_rng(seed)
        perm = rng.permutation(self.batch)
        arr = ctypes.c_size_t * self.batch
        self.ao = arr(*[int(i) * self.m * self.k for i in perm])
        self.bo = arr(*[int(i) * self.k * self.n for i in perm])
        self.co = arr(*[int(i) * self.m * self.n for i in perm])
        self.al = torch.full((self.batch,), self.alpha, dtype=self.torch_dtype())
        self.be = torch.full((self.batch,), self.beta, dtype=self.torch_dtype())
        import dlf_b200
        self.L = dlf_b200.lib()
        self.ws = torch.empty(self.L.dlf_b200_gemm_batched_workspace_bytes(self.batch), dtype=torch.uint8, device=device)

    def step(self, i):
        import ctypes
        j = i % self.sets
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        rc = self.L.dlf_b200_gemm_batched(16, 101, 111, 111, self.m, self.n, self.k, p(self.al), p(self.A[j]), self.ao,
                                          self.k, p(self.B[j]), self.bo, self.n, p(self.be), p(self.C[j]), self.co,
                                          self.n, self.batch, p(self.ws), self.ws.numel(),
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError("dlf_b200_gemm_batched: %d" % rc)


RESNET50_SHAPES = [
    # Cin, H, Cout, k, stride, pad, count   (ResNet-50 v1: stride on the first 1x1 of a stage)
    (3, 224, 64, 7, 2, 3, 1), (64, 56, 64, 1, 1, 0, 1), (64, 56, 64, 3, 1, 1, 3), (64, 56, 256, 1, 1, 0, 4),
    (256, 56, 64, 1, 1, 0, 2), (256, 56, 128, 1, 2, 0, 1), (128, 28, 128, 3, 1, 1, 4), (128, 28, 512, 1, 1, 0, 4),
    (256, 56, 512, 1, 2, 0, 1), (512, 28, 128, 1, 1, 0, 3), (512, 28, 256, 1, 2, 0, 1), (256, 14, 256, 3, 1, 1, 6),
    (256, 14, 1024, 1, 1, 0, 6), (512, 28, 1024, 1, 2, 0, 1), (1024, 14, 256, 1, 1, 0, 5), (1024, 14, 512, 1, 2, 0, 1),
    (512, 7, 512, 3, 1, 1, 3), (512, 7, 2048, 1, 1, 0, 3), (1024, 14, 2048, 1, 2, 0, 1), (2048, 7, 512, 1, 1, 0, 2),
]


# ------------------------------------------------------------------------------------------
# measurement helpers
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.t = threading.Thread(target=self._read, daemon=True)
        self.t.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0, t1):
        rows = [r for (t, r) in self.rows if t0 <= t <= t1] or [r for (_, r) in self.rows]
        sm, mx, reasons = [], [], set()
        for r in rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


NUMA_INFO = {}
ORIGINAL_AFFINITY = set()


def bind_to_gpu_numa_node(local):
    """Runs this rank on the CPUs of the NUMA node its GPU hangs off, before any pinned host buffer
    exists: pinned pages are placed where the allocating thread runs, and the end-to-end leg moves
    100 MB per step and rank between them and the GPU - through the socket interconnect when they
    sit on the other node. Only reads sysfs and sets this process's CPU affinity; any failure leaves
    the process as it was. What was done is reported in the JSON line (`numa`)."""
    info = {"bound": False}
    try:
        prop = torch.cuda.get_device_properties(local)
        bus = "%04x:%02x:%02x.0" % (prop.pci_domain_id, prop.pci_bus_id, prop.pci_device_id)
        info["pci"] = bus
        with open("/sys/bus/pci/devices/%s/numa_node" % bus) as f:
            node = int(f.read().strip())
        info["gpu_node"] = node
        if node < 0:
            return info
        with open("/sys/devices/system/node/node%d/cpulist" % node) as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        use = cpus & allowed
        info["node_cpus"], info["allowed_cpus"] = len(cpus), len(allowed)
        if use and use != allowed:
            ORIGINAL_AFFINITY.update(allowed)  # the CPU baseline's own process gets all of them back
            os.sched_setaffinity(0, use)
            info["bound"] = True
        info["cpus_used"] = len(use or allowed)
    except Exception as e:  # no sysfs entry, no permission, an older torch: run unbound
        info["error"] = repr(e)[:120]
    return info


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        NUMA_INFO.update(bind_to_gpu_numa_node(local))
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
        NUMA_INFO.update(bind_to_gpu_numa_node(0))
    return rank, world, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x, world):
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_steps(fn, steps, warmup, world):
    """W untimed + exactly K timed steps; returns milliseconds for the K steps (max over ranks)."""
    for i in range(warmup):
        fn(i)
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s = torch.cuda.current_stream()
    t0 = time.time()
    e0.record(s)
    for i in range(steps):
        fn(warmup + i)
    e1.record(s)
    barrier(world)
    t1 = time.time()
    return max_over_ranks(e0.elapsed_time(e1), world), t0, t1


def time_steps_graph(fn, steps, warmup, per_graph=20):
    """For steps of a few microseconds, whose rate would otherwise be set by the host's call
    overhead: `per_graph` consecutive steps are captured in a CUDA graph once and the graph is
    replayed; returns milliseconds for `steps` steps (rounded up to whole graphs), or None when the
    capture is not possible."""
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(max(warmup, 3)):
                fn(i)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(per_graph):
                fn(i)
        reps = max(1, (steps + per_graph - 1) // per_graph)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * steps / (reps * per_graph)
    except Exception as e:
        sys.stderr.write("graph timing not possible: %r\n" % (e,))
        torch.cuda.synchronize()
        return None


def run_extra(w, device, peaks, steps, warmup, graph=False):
    """Kernel-only numbers for a further BASELINE configuration (reported under "workloads")."""
    w.setup(device, 0, w.sets_needed())
    direct = bool(graph and hasattr(w, "step_abi") and w.batch == 1)
    step = w.step_abi if direct else w.step
    ms = time_steps_graph(step, steps, warmup) if graph else None
    timed = "cuda graph replay (20 steps per graph)" if ms is not None else \
        ("stream launches through the C ABI" if direct else "stream launches")
    if ms is None:
        ms, _, _ = time_steps(step, steps, warmup, 1)
    sec = ms / 1e3 / steps
    tf = w.flops / sec / 1e12
    return {"tflops": round(tf, 2), "us_per_step": round(sec * 1e6, 2), "dtype": w.dtype,
            "frac_of_measured_tensor_peak": round(tf / w.tensor_peak(peaks), 4),
            "frac_of_nominal_tensor_peak": round(tf / NOMINAL[w.dtype], 4),
            "hbm_gbs_algorithmic": round(w.bytes / sec / 1e9, 1),
            "frac_of_measured_hbm": round(w.bytes / sec / 1e9 / peaks["hbm_gbs"], 4),
            "out_gbs": round(getattr(w, "out_bytes", 0) / sec / 1e9, 1), "timed": timed}


def resnet_sweep(device, peaks, batch, reps):
    """Config 3: fp16 ResNet-50 v1 conv shapes at 224x224 (53 layers = 20 unique shapes), inputs as
    the configuration states them (activations |N(0,1)|, He-normal weights, bias U(-0.1, 0.1)),
    generated on the device from a seed per layer. Every layer's first image is compared with the
    oracle (wide accumulator): `max_rel_err` is the worst layer's maximum relative error
    (relative to max(|y|, 0.01 max|y|); tolerance 2e-2)."""
    import oracle
    from dlf_b200 import gdnn
    total_flops, total_s, rows, worst = 0.0, 0.0, [], 0.0
    for idx, (cin, h, cout, k, s, p, count) in enumerate(RESNET50_SHAPES):
        g = torch.Generator(device=device).manual_seed(idx)
        X = [torch.randn((batch, cin, h, h), generator=g, device=device).abs_().half() for _ in range(2)]
        W = (torch.randn((cout, cin, k, k), generator=g, device=device) * math.sqrt(2.0 / (cin * k * k))).half()
        b = (torch.rand(cout, generator=g, device=device) * 0.2 - 0.1).half()
        filt = gdnn.Filter2D(X[0].shape, W.shape).pads(p, p).strides(s, s)
        Y = [torch.empty(filt.output_shape(), dtype=torch.float16, device=device) for _ in range(2)]
        step = lambda i: gdnn.conv2d_filter(X[i % 2], W, Y[i % 2], filt, bias=b)
        ms, _, _ = time_steps(step, reps, 3, 1)
        sec = ms / 1e3 / reps
        flops = 2.0 * batch * cout * filt.output_h * filt.output_w * cin * k * k
        ref = oracle.conv2d(X[0][:1].float().cpu().numpy(), W.float().cpu().numpy(), pads=(p,) * 4, strides=(s, s),
                            bias=b.float().cpu().numpy(), wide=True)
        step(0)
        got = Y[0][:1].float().cpu().numpy()
        den = np.maximum(np.abs(ref), 1e-2 * np.abs(ref).max())
        err = float((np.abs(got - ref) / den).max())
        worst = max(worst, err)
        rows.append({"shape": [cin, h, cout, k, s], "count": count, "tflops": round(flops / sec / 1e12, 1),
                     "us": round(sec * 1e6, 1), "err": float("%.2g" % err)})
        total_flops += flops * count
        total_s += sec * count
        del X, Y, W, b
        torch.cuda.empty_cache()
    tf = total_flops / total_s / 1e12
    summary = {"tflops": round(tf, 1), "ms_per_sweep": round(total_s * 1e3, 3), "batch": batch, "dtype": "f16",
               "frac_of_measured_tensor_peak": round(tf / peaks["bf16_tflops"], 4),
               "frac_of_nominal_tensor_peak": round(tf / NOMINAL["f16"], 4),
               "max_rel_err_vs_oracle": float("%.3g" % worst), "tolerance": 2e-2}
    return summary, rows


def resnet50_graph(batch, size=224, classes=1000, seed=0):
    """ResNet-50 v1 (stride on the first 1x1 of a stage) as a graph for dlf_b200.predict: the 53
    convolutions of RESNET50_SHAPES with a bias each (batch normalisation already folded), ReLU and
    residual Add nodes as an exporter writes them, 3x3 max pool, global average pool, Flatten and
    the 2048 -> classes Gemm. Weights are seeded He-normal draws - no checkpoint is involved."""
    from dlf_b200 import predict as P
    rng = np.random.default_rng(seed)
    g = P.Graph()

    def conv(x, cin, cout, k, stride, pad, name):
        n = g.append("Conv", kernel_shape=[k, k], strides=[stride, stride], pads=[pad] * 4)
        n.addInput(x)
        n.addInput(g.addInitializer(name + ".W", (math.sqrt(2.0 / (cin * k * k)) *
                                    rng.standard_normal((cout, cin, k, k), dtype=np.float32))))
        n.addInput(g.addInitializer(name + ".B", rng.uniform(-0.1, 0.1, cout).astype(np.float32)))
        return n.addOutput(name)

    def relu(x, name):
        n = g.append("Relu")
        n.addInput(x)
        return n.addOutput(name)

    t = relu(conv(g.addInput("image", P.DataType.FLOAT, (batch, 3, size, size)), 3, 64, 7, 2, 3, "conv1"), "relu1")
    mp = g.append("MaxPool", kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1])
    mp.addInput(t)
    t, cin = mp.addOutput("pool1"), 64
    for stage, (blocks, width, stride) in enumerate(((3, 64, 1), (4, 128, 2), (6, 256, 2), (3, 512, 2))):
        for b in range(blocks):
            nm = "s%db%d" % (stage + 1, b)
            st = stride if b == 0 else 1
            a = relu(conv(t, cin, width, 1, st, 0, nm + ".c1"), nm + ".r1")
            a = relu(conv(a, width, width, 3, 1, 1, nm + ".c2"), nm + ".r2")
            a = conv(a, width, 4 * width, 1, 1, 0, nm + ".c3")
            sc = conv(t, cin, 4 * width, 1, st, 0, nm + ".down") if b == 0 else t
            add = g.append("Add")
            add.addInput(a).addInput(sc)
            t, cin = relu(add.addOutput(nm + ".add"), nm + ".out"), 4 * width
    gap = g.append("GlobalAveragePool")
    gap.addInput(t)
    fl = g.append("Flatten", axis=1)
    fl.addInput(gap.addOutput("gap"))
    fc = g.append("Gemm", transB=1)
    fc.addInput(fl.addOutput("flat"))
    fc.addInput(g.addInitializer("fc.W", rng.standard_normal((classes, cin), dtype=np.float32) / math.sqrt(cin)))
    fc.addInput(g.addInitializer("fc.B", rng.uniform(-0.1, 0.1, classes).astype(np.float32)))
    g.addOutput(fc.addOutput("logits"))
    return g


def oracle_forward(graph, image, rnd):
    """An optimized graph (convolutions carrying their residual / ReLU marks) evaluated operator by
    operator with the CPU oracle on one batch; ``rnd`` rounds every operator's result to the
    storage type, as the device does when it stores it."""
    import oracle
    env = {}
    for v in graph.inputs:
        env[id(v)] = rnd(np.asarray(v.initializer, dtype=np.float32)) if v.has_initializer() else rnd(image)
    for n in graph.nodes:
        a = [env.get(id(v)) if v is not None else None for v in n.inputs]
        if n.kind == "Conv":
            res = env[id(n.get("residual"))] if n.get("residual") is not None else None
            y = oracle.conv2d_fused(a[0], a[1], residual=res, relu=bool(n.get("relu")), bias=a[2] if len(a) > 2 else None,
                                    pads=tuple(n.get("pads", (0,) * 4)), strides=tuple(n.get("strides", (1, 1))), wide=True)
        elif n.kind == "MaxPool":
            y = oracle.pool2d(a[0], tuple(n.get("kernel_shape")), "max", tuple(n.get("pads", (0,) * 4)),
                              tuple(n.get("strides", (1, 1))))
        elif n.kind == "GlobalAveragePool":
            y = oracle.global_pool(a[0], "avg", wide=True)
        elif n.kind == "Flatten":
            y = a[0].reshape(a[0].shape[0], -1)
        elif n.kind == "Gemm":
            B = a[1].T if n.get("transB", 0) else a[1]
            y = (a[0].astype(np.float64) @ B.astype(np.float64) + a[2].astype(np.float64)).astype(np.float32)
        else:
            raise RuntimeError("oracle_forward: " + n.kind)
        env[id(n.output(0))] = rnd(y)
    return env[id(graph.outputs[0])]


def resnet_forward(device, peaks, batch, reps, layouts="both"):
    """A whole ResNet-50 v1 forward (fp16, 224x224) as an operator list of this library
    (dlf_b200.predict): 53 fused convolutions, max pool, global average pool, the FC Gemm - with the
    tensors between the operators kept channels-last (the default) and with every tensor NCHW as the
    reference's operators have them, each timed launch by launch and as a CUDA-graph replay. The
    logits of one image are compared with the oracle evaluating the same operator list on the CPU
    (relative Frobenius error)."""
    from dlf_b200 import predict as P
    flops = sum(2.0 * batch * co * (h // s) ** 2 * ci * k * k * cnt for ci, h, co, k, s, _, cnt in RESNET50_SHAPES)
    flops += 2.0 * batch * 1000 * 2048
    out = {"batch": batch, "dtype": "f16"}
    rnd = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).half().float().numpy()
    g = torch.Generator(device=device).manual_seed(7)
    images = torch.randn((batch, 3, 224, 224), generator=g, device=device).half()
    want = None
    for key, channels_last in (("nchw", False), ("channels_last", True)):
        if layouts != "both" and layouts != key:
            continue
        pred = P.Predictor(resnet50_graph(batch), dtype=torch.float16, device=device, cuda_graph=False,
                           channels_last=channels_last)
        pred.input(0).copy_(images)
        step = lambda i: pred.predict()
        ms_stream, _, _ = time_steps(step, reps, 3, 1)
        row = {"operators": len(pred.operators), "launching_operators": pred.launches_per_predict(),
               "stream_launches": {"ms_per_forward": round(ms_stream / reps, 3),
                                   "images_per_s": round(batch * reps / (ms_stream / 1e3), 1)}}
        pred._want_graph = True  # the next predict() captures the list, later ones replay it
        pred.predict()
        if pred._cuda_graph is not None:
            ms_graph, _, _ = time_steps(step, reps, 3, 1)
            sec = ms_graph / 1e3 / reps
            row["cuda_graph_replay"] = {"ms_per_forward": round(sec * 1e3, 3), "images_per_s": round(batch / sec, 1),
                                        "tflops": round(flops / sec / 1e12, 1),
                                        "frac_of_measured_tensor_peak": round(flops / sec / 1e12 / peaks["bf16_tflops"], 4)}
        # parity of the whole chain on one image: a batch-1 predictor with the same weights
        small = P.Predictor(resnet50_graph(1), dtype=torch.float16, device=device, cuda_graph=False,
                            channels_last=channels_last)
        image = images[:1].float().cpu().numpy()
        small.set(0, image)
        small.predict()
        if want is None:
            want = oracle_forward(small.graph, image, rnd)
        got = small.get(0)
        row["logits_rel_fro_err_vs_oracle"] = float("%.3g" % (np.linalg.norm(got - want) / np.linalg.norm(want)))
        row["logits_batch_vs_single_image_max_abs_diff"] = float(
            "%.3g" % np.abs(pred.output(0)[:1].float().cpu().numpy() - got).max())
        out[key] = row
        del pred, small
        torch.cuda.empty_cache()
    return out


def multi_gpu_workloads(table, device, peaks, world, rank):
    """The two other ways the path shards, measured on every rank (max over ranks):
    * config 5, one large fp32 GEMM: rows of C per rank, then the NCCL all-gather of the row
      blocks (the only collective of the design) - strong scaling, the all-gather timed by itself
      as well;
    * config 4 (i), strided-batched fp16 GEMM: batch entries per rank, no collective - weak
      scaling (every rank multiplies its own 1024 matrices)."""
    from dlf_b200 import shard
    out = {}
    try:
        w = table["sgemm_16384"]()
        w.setup(device, 0, 2)
        fn = lambda i: w.step_sharded(i, world, rank)
        ms, _, _ = time_steps(fn, 5, 2, world)
        sec = ms / 1e3 / 5
        C = w.C[0].view(w.m, w.n)
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            shard.all_gather_rows(C, world, rank)
        e1.record()
        barrier(world)
        ag_ms = max_over_ranks(e0.elapsed_time(e1), world) / 5
        out[w.name] = {"tflops": round(w.flops / sec / 1e12, 1), "ms_per_step": round(sec * 1e3, 3),
                       "tflops_per_gpu": round(w.flops / world / sec / 1e12, 1), "scaling": "strong",
                       "sharding": "rows of C per rank + NCCL all-gather of the row blocks",
                       "all_gather_ms": round(ag_ms, 3),
                       "all_gather_gbs_bus": round(4.0 * w.m * w.n * (world - 1) / world / (ag_ms / 1e3) / 1e9, 1)}
        del w, C
        torch.cuda.empty_cache()
    except Exception as e:
        out["sgemm_f32_16384_tn"] = {"error": repr(e)[:200]}
    try:
        w = table["batched_c4_a"]()
        w.setup(device, rank, w.sets_needed())
        ms, _, _ = time_steps(w.step, 100, 5, world)
        sec = ms / 1e3 / 100
        out[w.name] = {"tflops": round(w.flops * world / sec / 1e12, 1), "us_per_step": round(sec * 1e6, 2),
                       "tflops_per_gpu": round(w.flops / sec / 1e12, 1), "scaling": "weak",
                       "sharding": "batch entries per rank, no collective",
                       "hbm_gbs_algorithmic_per_gpu": round(w.bytes / sec / 1e9, 1)}
        del w
        torch.cuda.empty_cache()
    except Exception as e:
        out["bgemm_f16_b1024_512x512x64"] = {"error": repr(e)[:200]}
    return out


def pooling_extras(device, peaks):
    """The two pooling layers of ResNet-50 at batch 256, fp16: HBM-bound, reported against the
    measured copy bandwidth (bytes = input read once + output written once)."""
    from dlf_b200 import gdnn
    out = {}
    for name, shape, k, s, p, kind in (("maxpool_3x3_s2_64x112x112", (256, 64, 112, 112), 3, 2, 1, "max"),
                                       ("global_avgpool_2048x7x7", (256, 2048, 7, 7), 7, 7, 0, "avg")):
        X = [torch.randn(shape, device=device).abs().half() for _ in range(2)]
        f = gdnn.Filter2D(shape, k, k).pads(p, p).strides(s, s)
        Y = [torch.empty((shape[0], shape[1], f.output_h, f.output_w), dtype=torch.float16, device=device)
             for _ in range(2)]
        if kind == "max":
            fn = lambda i: gdnn.max_pooling(X[i % 2], Y[i % 2], f)
        else:
            fn = lambda i: gdnn.average_pooling(X[i % 2], Y[i % 2], f, False)
        ms, _, _ = time_steps(fn, 50, 5, 1)
        sec = ms / 1e3 / 50
        nbytes = 2 * (X[0].numel() + Y[0].numel())
        out[name] = {"us_per_step": round(sec * 1e6, 2), "hbm_gbs_algorithmic": round(nbytes / sec / 1e9, 1),
                     "frac_of_measured_hbm": round(nbytes / sec / 1e9 / peaks["hbm_gbs"], 4)}
        del X, Y
        torch.cuda.empty_cache()
    return out


def reference_arm(args, rank):
    """--impl reference: the reference's CPU implementation of the path (oracle port; the
    reference itself needs TBB + MKL, which are absent) timed on the host cores. A step is a
    bounded sample (8 of the 64 images) of the workload; ms_per_step is scaled to the full batch."""
    if rank != 0:
        return
    w = ConvC2()
    steps = max(1, args.steps if args.steps_given else 3)
    per_step_budget = min(20.0, 120.0 / (steps + args.warmup))
    vals = []
    info = None
    for i in range(args.warmup + steps):
        info = w.cpu_reference(per_step_budget)
        if i >= args.warmup:
            vals.append(info["value"])
    value = float(np.mean(vals))
    line = {"impl": "reference", "metric": "gemm_conv_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
            "ms_per_step": info["seconds_per_full_step"] * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w.name, "note": "reference CPU schedule: per-image im2col + sgemm, serial over "
                                                   "batch; ms_per_step = sample time scaled to the 64-image step"},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": info["cores"], "kind": "port",
                             "sample": info["sample"], "host_cores": os.cpu_count() or 1},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def cpu_baseline_subprocess():
    """The cpu_baseline leg of the default run: the reference arm in a process of its own, so that
    its OpenMP / BLAS thread pools are sized by its own environment (this process has long loaded
    its OpenMP runtime with whatever the launcher exported)."""
    env = {k: v for k, v in os.environ.items() if k not in ("OMP_NUM_THREADS", "DLF_B200_BENCH_ENV")}
    orig = set(ORIGINAL_AFFINITY)
    res = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, env=env, timeout=600,
                         preexec_fn=(lambda: os.sched_setaffinity(0, orig)) if orig else None)
    for ln in reversed(res.stdout.splitlines()):
        if ln.startswith("{"):
            return json.loads(ln)["cpu_baseline"]
    raise RuntimeError("reference arm printed no line: " + res.stderr[-300:])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--workload", default="conv_c2")
    ap.add_argument("--headline-only", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=None, help="images per GPU for conv_c2 (profiling: a small case)")
    ap.add_argument("--shape", default="64,56,64,3,1,1", help="--workload conv: Cin,H,Cout,k,stride,pad")
    ap.add_argument("--dtype", default="f16", help="--workload conv: f16, bf16 or f32")
    ap.add_argument("--layout", default="both", choices=["both", "nchw", "channels_last"],
                    help="--workload resnet_forward: which tensor layout between the operators to run; --workload conv: "
                         "channels_last times the channels-last entry")
    ap.add_argument("--residual", action="store_true", help="--workload conv: fuse a residual Add and ReLU")
    ap.add_argument("--tuning", type=lambda x: int(x, 0), default=0,
                    help="experiments: second argument of dlf_b200_set_tuning for the whole run")
    ap.add_argument("--overlap-gather", action="store_true",
                    help="row-sharded GEMM: all-gather finished panels while the next panel is computed")
    ap.add_argument("--kernel-only", action="store_true",
                    help="only the timed kernel loop: no end-to-end leg, parity check, CPU baseline or extras")
    args = ap.parse_args()
    args.steps_given = args.steps is not None
    if args.impl == "reference":
        if args.warmup is None:
            args.warmup = 1
        reference_arm(args, int(os.environ.get("RANK", "0")))
        return
    steps = args.steps if args.steps is not None else 4000
    warmup = max(3, args.warmup if args.warmup is not None else 200)

    import dlf_b200
    dlf_b200.lib()  # fail loudly when the CUDA library is missing
    if args.tuning:
        dlf_b200.set_tuning(0, args.tuning)
    rank, world, local = dist_setup(args.gpus)
    device = torch.device("cuda", local)
    peaks = measured_peaks()

    table = {
        "conv_c2": lambda: ConvC2(shape=dict(N=args.batch) if args.batch else None),
        "gemm_f16_4096": lambda: GemmWorkload("gemm_f16_4096", "f16", 4096, 4096, 4096),
        "sgemm_1024": lambda: GemmWorkload("sgemm_f32_1024", "f32", 1024, 1024, 1024, dist="uniform"),
        "sgemm_16384": lambda: GemmWorkload("sgemm_f32_16384_tn", "f32", 16384, 16384, 16384, ta=True, alpha=0.5,
                                            beta=0.5, dist="uniform"),
        # config 5's operand layout and K at a size that an ncu capture can hold (profiling aid)
        "sgemm_4096_k16384": lambda: GemmWorkload("sgemm_f32_4096x4096x16384_tn", "f32", 4096, 4096, 16384, ta=True,
                                                  alpha=0.5, beta=0.5, dist="uniform"),
        "batched_c4_a": lambda: GemmWorkload("bgemm_f16_b1024_512x512x64", "f16", 512, 512, 64, batch=1024, alpha=0.125),
        "batched_c4_b": lambda: GemmWorkload("bgemm_f16_b1024_512x64x512", "f16", 512, 64, 512, batch=1024, alpha=0.125),
        "fc_c3": lambda: GemmWorkload("resnet50_fc_f16_256x1000x2048", "f16", 256, 1000, 2048),
        "gemm_batched_offsets": lambda: GemmBatchedOffsets("gemm_batched_offsets_f16_b1024_512x512x64", "f16", 512, 512,
                                                           64, batch=1024, alpha=0.125),
    }
    for tag, ta, tb in (("tn", True, False), ("nt", False, True), ("tt", True, True)):
        table["batched_c4_a_" + tag] = (lambda tag=tag, ta=ta, tb=tb: GemmWorkload(
            "bgemm_f16_b1024_512x512x64_" + tag, "f16", 512, 512, 64, batch=1024, ta=ta, tb=tb, alpha=0.125))
        table["batched_c4_b_" + tag] = (lambda tag=tag, ta=ta, tb=tb: GemmWorkload(
            "bgemm_f16_b1024_512x64x512_" + tag, "f16", 512, 64, 512, batch=1024, ta=ta, tb=tb, alpha=0.125))
    if args.workload == "conv":  # profiling aid: one convolution layer, e.g. --shape 64,56,64,3,1,1 --batch 16 --dtype f16
        cin, h, cout, k, st_, pd = [int(x) for x in args.shape.split(",")]
        w = ConvC2(shape=dict(N=args.batch or 16, C=cin, H=h, W=h, Co=cout, KH=k, KW=k, pad=pd, stride=st_, group=1),
                   dtype=args.dtype)
        w.setup(device, 0, w.sets_needed())
        n = steps if args.steps is not None else 20
        if args.layout == "channels_last":
            fn = lambda i: w.step_nhwc(i, args.residual)
        else:
            fn = w.step_fused if args.residual else w.step
        ms, _, _ = time_steps(fn, n, warmup, 1)
        sec = ms / 1e3 / n
        print(json.dumps({"workload": "conv", "shape": args.shape, "batch": w.shape["N"], "dtype": args.dtype,
                          "residual_relu": bool(args.residual), "layout": args.layout if args.layout != "both" else "nchw",
                          "us_per_step": sec * 1e6, "tflops": w.flops / sec / 1e12,
                          "algorithmic_bytes": w.bytes, "device_status": dlf_b200.device_status()}), flush=True)
        return
    if args.workload == "resnet_forward":  # the whole network as an operator list
        print(json.dumps({"resnet50_v1_forward_f16": resnet_forward(device, peaks, args.batch or 256,
                                                                   steps if args.steps is not None else 10, args.layout),
                          "device_status": dlf_b200.device_status()}), flush=True)
        return
    if args.workload == "resnet_sweep":  # development aid: config 3 alone, per layer
        summary, rows = resnet_sweep(device, peaks, args.batch or 256, steps if args.steps is not None else 10)
        print(json.dumps({"resnet50_v1_convs_f16": summary, "layers": rows, "device_status": dlf_b200.device_status()}), flush=True)
        return
    w = table[args.workload]()
    w.overlap_gather = args.overlap_gather
    sets = w.sets_needed()
    # a single (unbatched) GEMM is sharded by rows of C with an all-gather: strong scaling, and
    # every rank must hold the same operands
    row_sharded = world > 1 and isinstance(w, GemmWorkload) and w.batch == 1
    w.seed_used = 0 if row_sharded else rank
    w.setup(device, w.seed_used, sets)
    step_fn = (lambda i: w.step_sharded(i, world, rank)) if row_sharded else w.step

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(warmup):  # warm-up happens here so that the launch counter brackets the timed steps only
        step_fn(i)
    l0 = dlf_b200.launch_count()
    ms, t0, t1 = time_steps(step_fn, steps, 0, world)
    launches = dlf_b200.launch_count() - l0
    if rank == 0:
        sampler.stop()
    launches_timed = launches
    status = dlf_b200.device_status()
    sec_per_step = ms / 1e3 / steps
    value = (w.flops if row_sharded else w.flops * world) / sec_per_step / 1e12

    # end to end through the public API with host buffers
    e2e = None
    if hasattr(w, "e2e_step") and not args.kernel_only:
        e_steps = max(3, min(steps, 60))
        for i in range(6):
            w.e2e_step(i)
        torch.cuda.synchronize()
        barrier(world)
        t_0 = time.perf_counter()
        for i in range(e_steps):
            w.e2e_step(i)
        torch.cuda.synchronize()
        dt_e = max_over_ranks(time.perf_counter() - t_0, world) / e_steps
        h2d, d2h = w.e2e_bytes()
        e2e = {"value": w.flops * world / dt_e / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": dt_e * 1e3}

    parity = w.check() if hasattr(w, "check") and not args.kernel_only else None

    multi_gpu_extras = None
    if world > 1 and args.workload == "conv_c2" and not args.headline_only and not args.kernel_only:
        multi_gpu_extras = multi_gpu_workloads(table, device, peaks, world, rank)

    numa_ranks = None
    if world > 1:  # every rank's GPU node and whether it was bound, for the line rank 0 prints
        import torch.distributed as dist
        numa_ranks = [None] * world
        dist.all_gather_object(numa_ranks, [NUMA_INFO.get("gpu_node"), NUMA_INFO.get("bound")])

    if rank != 0:
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()
        return

    tf_per_gpu = (w.flops / world if row_sharded else w.flops) / sec_per_step / 1e12
    peak = w.tensor_peak(peaks)
    roofline = {"bound": "tensor", "achieved": tf_per_gpu, "peak": peak, "unit": "TFLOP/s",
                "frac": tf_per_gpu / peak, "traffic": None,
                "peak_basis": ("%s bf16 cuBLAS burst %.0f TFLOP/s" % (peaks["source"], peaks["bf16_tflops"])) +
                              ("; fp32 runs as 3xTF32: tf32 rate = bf16/2, three MMAs per product => /6"
                               if w.dtype == "f32" else ""),
                "frac_of_nominal": tf_per_gpu / NOMINAL[w.dtype],
                "hbm_gbs_algorithmic": w.bytes / sec_per_step / 1e9,
                "hbm_frac_of_measured": w.bytes / sec_per_step / 1e9 / peaks["hbm_gbs"],
                "kernel": ("contraction_ts_kernel (row-form implicit GEMM); the step also launches "
                           "pack_weights_kernel once, its time is inside the measured step") if isinstance(w, ConvC2)
                          else ("contraction_ts_kernel" if w.dtype == "f32" else "contraction_kernel<2,true>"),
                "avg_launch_us": sec_per_step * 1e6}
    prof = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(prof):
        with open(prof) as f:
            entry = json.load(f).get(w.name)
            if isinstance(entry, dict):
                roofline["traffic"] = entry.get("bytes_per_launch")
                roofline["traffic_note"] = entry.get("captured")

    line = {"metric": "gemm_conv_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": sec_per_step * 1e3, "higher_is_better": True,
            "scaling": "strong" if row_sharded else "weak",
            "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
            "config": {"workload": w.name, "per_gpu_batch": getattr(w, "shape", {}).get("N"),
                       "sharding": (("rows of C per rank in four panels; the NCCL all-gather of a panel overlaps the next panel's GEMM"
                                     if args.overlap_gather else "rows of C per rank + NCCL all-gather of the row blocks") if row_sharded else
                                    "batch per rank, no collective") if world > 1 else "single GPU",
                       "l2": "rotating %d input/output buffer sets (%.0f MB > 126 MB L2)" % (
                           sets, sets * (getattr(w, "x_bytes", w.bytes) + getattr(w, "y_bytes", 0)) / 1e6),
                       "arithmetic": "3xTF32 tcgen05, fp32 accumulate" if w.dtype == "f32" else "tcgen05 f16, fp32 accumulate"},
            "roofline": roofline, "gpu_launches": int(launches_timed), "launches_per_step": launches / steps,
            "device_status": status, "clocks": sampler.summary(t0, t1), "parity_rel_fro_vs_oracle": parity}
    if e2e:
        line["e2e"] = e2e
    line["numa"] = dict(NUMA_INFO)
    if numa_ranks is not None:
        line["numa"]["ranks"] = numa_ranks

    if world == 1 and not args.no_cpu_baseline and not args.kernel_only and hasattr(w, "cpu_reference"):
        try:
            line["cpu_baseline"] = cpu_baseline_subprocess()
        except Exception as e:  # the baseline must never lose the headline line
            line["cpu_baseline"] = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "port",
                                    "sample": "failed: " + repr(e)[:200]}

    if world == 1 and not args.headline_only and not args.kernel_only and args.workload == "conv_c2":
        # Key order matters to readers that keep only the end of the line: the per-layer list of
        # the ResNet sweep comes first, the three north-star numbers (ResNet summary, fp16 4096^3
        # GEMM, fp32 16384^3 GEMM) last.
        extras = {}
        # sustained figure of the headline: at least two seconds back to back, with the clocks seen
        try:
            smp = ClockSampler(local)
            smp.start()
            n_sus = max(steps, int(2.2 / sec_per_step))
            ms_s, ts0, ts1 = time_steps(step_fn, n_sus, 50, 1)
            smp.stop()
            tf_s = w.flops / (ms_s / 1e3 / n_sus) / 1e12
            peak_s = peaks["bf16_tflops_sustained"] / (6.0 if w.dtype == "f32" else 1.0)
            line["sustained"] = {"steps": n_sus, "seconds": round(ms_s / 1e3, 3), "tflops": round(tf_s, 2),
                                 "frac_of_measured_sustained_peak": round(tf_s / peak_s, 4),
                                 "peak": round(peak_s, 1), "clocks": smp.summary(ts0, ts1)}
        except Exception as e:
            line["sustained"] = {"error": repr(e)[:200]}
        # what omitting the optional scratch costs: the same convolution with workspace = NULL
        try:
            ms_n, _, _ = time_steps(w.step_no_workspace, 50, 5, 1)
            extras["conv_c2_without_workspace"] = {"us_per_step": round(ms_n / 50 * 1e3, 2),
                                                   "tflops": round(w.flops / (ms_n / 1e3 / 50) / 1e12, 2)}
        except Exception as e:
            extras["conv_c2_without_workspace"] = {"error": repr(e)[:200]}
        del w
        torch.cuda.empty_cache()
        resnet_summary = None
        try:
            resnet_summary, rows = resnet_sweep(device, peaks, 256, 10)
            extras["resnet50_v1_convs_f16_b256_layers"] = rows
        except Exception as e:
            resnet_summary = {"error": repr(e)[:200]}
        try:
            extras["resnet50_v1_forward_f16_b256"] = resnet_forward(device, peaks, 256, 10)
        except Exception as e:
            extras["resnet50_v1_forward_f16_b256"] = {"error": repr(e)[:200]}
        torch.cuda.empty_cache()
        try:  # write-only HBM rate (memset of 1 GiB): the roof of the output-dominated workloads
            z = torch.empty(1 << 30, dtype=torch.uint8, device=device)
            ms, _, _ = time_steps(lambda i: z.zero_(), 10, 3, 1)
            extras["hbm_write_gbs_memset"] = round((1 << 30) * 10 / (ms / 1e3) / 1e9, 1)
            del z
            torch.cuda.empty_cache()
        except Exception as e:
            extras["hbm_write_gbs_memset"] = {"error": repr(e)[:200]}
        try:
            extras["pooling_f16_b256"] = pooling_extras(device, peaks)
        except Exception as e:
            extras["pooling_f16_b256"] = {"error": repr(e)[:200]}
        for key, reps in (("batched_c4_a_tn", 50), ("batched_c4_a_nt", 50), ("batched_c4_a_tt", 50),
                          ("batched_c4_b_tn", 50), ("batched_c4_b_nt", 50), ("batched_c4_b_tt", 50),
                          ("batched_c4_a", 100), ("batched_c4_b", 100), ("gemm_batched_offsets", 100),
                          ("sgemm_1024", 500), ("fc_c3", 200), ("gemm_f16_4096", 200), ("sgemm_16384", 5)):
            try:
                ww = table[key]()
                extras[ww.name] = run_extra(ww, device, peaks, reps, 5, graph=key in ("sgemm_1024", "fc_c3"))
                del ww
                torch.cuda.empty_cache()
            except Exception as e:  # an extra must never lose the headline line
                extras[key] = {"error": repr(e)[:200]}
        extras["device_status"] = dlf_b200.device_status()
        extras["resnet50_v1_convs_f16_b256"] = resnet_summary
        for key in ("gemm_f16_4096", "sgemm_f32_16384_tn"):  # north-star numbers: last keys of the line
            if key in extras:
                extras[key] = extras.pop(key)
        line["workloads"] = extras
    elif world > 1 and args.workload == "conv_c2" and not args.headline_only and not args.kernel_only:
        line["workloads"] = multi_gpu_extras

    print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
