#!/usr/bin/env python
"""Benchmark of the matmul / Linear path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Prints ONE JSON line (rank 0).  A "step" is one pass of the hot path over one batch of seeded
synthetic input.  The default workload is the large fp32 GEMM (M = N = K = 8192, Y = X.W^T, W
stored [out, in]); with N GPUs the output is cut into a pr x pc grid of blocks, a rank holding one
row-slab of X and one row-slab of W (= output columns), and no collective is on the data path.

  value      whole-job TFLOP/s (2.M.N.K per GEMM, split products not counted), inputs resident in
             HBM, timed with CUDA events over exactly K steps, max over ranks.
  e2e        the same work through the C ABI with HOST buffers: every step copies the inputs from
             pinned host memory, runs the GEMM and copies the result back.
  roofline   the tensor-core GEMM kernel alone (CUDA events recorded by the library around that
             kernel during the timed steps) against the accuracy-preserving tensor peak =
             measured dense TF32 rate / 3 MMAs per product.
  cpu_baseline  the reference's own CPU matmul (compiled from its sources, else the C port) on a
             bounded row-slab of the same workload, on this machine's host cores.

--impl reference times only that CPU implementation, on all host threads (independent row slabs).
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "fp32-accurate GEMM TFLOP/s"
UNIT = "TFLOP/s"
NOMINAL_TF32_DENSE = 1125.0  # TFLOP/s, B200 data sheet (half of the 2:4-sparse figure)


# ---------------------------------------------------------------------------------------------
# workloads: name -> description of one step
# ---------------------------------------------------------------------------------------------
def workload_spec(name: str, world: int) -> dict:
    if name == "gemm8192":
        return dict(kind="gemm_nt", M=8192, N=8192, K=8192, shard="MN",
                    desc="config 4: fp32 GEMM M=N=K=8192, A row-major, B [N,K] (transpose flag), U[-1,1); "
                         "over several GPUs N-column-sharded with X replicated (--shard blocks: a 2-D grid of output "
                         "blocks); config.partition says what this rank computed",
                    flops=2.0 * 8192 ** 3)
    if name.startswith("gemm_nt:"):  # e.g. gemm_nt:4096x4096x4096 -- profiling-sized cases of the same kernel
        m, n, k = (int(v) for v in name.split(":", 1)[1].split("x"))
        return dict(kind="gemm_nt", M=m, N=n, K=k, shard="MN",
                    desc=f"fp32 GEMM Y=X.W^T M={m} N={n} K={k}, U[-1,1); partitioned like config 4 over several GPUs",
                    flops=2.0 * m * n * k)
    if name == "gemm512":
        return dict(kind="gemm_nn", M=512, N=512, K=512, shard=None,
                    desc="config 1: fp32 GEMM M=N=K=512 row-major no transpose (latency regime); replicas",
                    flops=2.0 * 512 ** 3)
    if name == "linear_step":
        return dict(kind="linear_step", M=8192, N=4096, K=4096, shard="tokens",
                    desc="config 5: Linear 4096->4096, 8192 tokens: Y=X.W^T+b, dX=dY.W, dW=dY^T.X; tokens sharded, "
                         "dW all-reduced (NCCL) when world > 1",
                    flops=3 * 2.0 * 8192 * 4096 * 4096)
    if name.startswith(("attention:", "attention_train:", "attention_fused:")):   # profiling-sized: <name>:<nbat>
        base, nb = name.split(":", 1)
        spec = workload_spec(base, world)
        scale = int(nb) / spec["nbat"]
        return dict(spec, nbat=int(nb), flops=spec["flops"] * scale, desc=spec["desc"] + f" [nbat={int(nb)}]")
    if name == "attention":
        return dict(kind="attention", nbat=32, ntimes=512, nhead=8, npiece=64, shard="batch",
                    desc="config 3: S=QK^T/8, softmax, O=PV; 32x8 heads, seq 512, head_dim 64; batch sharded",
                    flops=2 * 2.0 * 32 * 8 * 512 * 512 * 64)
    if name == "attention_fused":
        return dict(kind="attention", fused=True, nbat=32, ntimes=512, nhead=8, npiece=64, shard="batch",
                    desc="config 3 through the fused forward call (kai_mh_attention_forward: probs never written to "
                         "memory); 32x8 heads, seq 512, head_dim 64; batch sharded",
                    flops=2 * 2.0 * 32 * 8 * 512 * 512 * 64)
    if name == "attention_train":
        return dict(kind="attention", backward=True, nbat=32, ntimes=512, nhead=8, npiece=64, shard="batch",
                    desc="config 3 forward + backward: the attention trio, then mix_values_backward_prop/value, "
                         "softmax_direct_on_axis_backward and mult_on_heads_backward for K and Q "
                         "(the engine's call order); batch sharded",
                    flops=6 * 2.0 * 32 * 8 * 512 * 512 * 64)
    if name == "conv2d" or name.startswith("conv2d:"):
        nd = int(name.split(":", 1)[1]) if ":" in name else 32
        return dict(kind="conv", ndat=nd, xchn=64, ychn=64, h=56, w=56, kh=3, kw=3, shard="batch",
                    desc=f"3x3 convolution 64->64 channels on {nd}x56x56 images (NCHW, padding 1): conv2d, "
                         "conv2d_backward_x, conv2d_backward_k; images sharded over GPUs",
                    flops=3 * 2.0 * nd * 64 * 56 * 56 * 64 * 9)
    if name == "rnn_gates":
        return dict(kind="rnn", ntimes=32, ndat=64, ninp=512, nrec=512, ngates=4, shard=None,
                    desc="recurrent-layer call pattern: 32 timesteps x (state matmul, input matmul with acc on the same "
                         "interior slice, add_bias, activate), batch 64, 512 inputs, 4 x 512 gates; latency regime; "
                         "replicas",
                    flops=32 * 2.0 * 64 * 2048 * (512 + 512))
    if name == "mlp":
        return dict(kind="mlp", shard=None,
                    desc="config 2: Linear(784->512)+ReLU -> Linear(512->10), batch 128, softmax-CE on int labels, "
                         "forward+backward as the reference's 15 math calls; latency regime; replicas",
                    flops=2.0 * 128 * (784 * 512 + 512 * 10) * 3 - 2.0 * 128 * 784 * 512)
    if name.startswith("skinny"):
        m = int(name[6:] or 1)
        return dict(kind="skinny", M=m, N=4096, K=4096, shard=None,
                    desc=f"config 5 skinny inference: Y[{m},4096]=X.W^T, HBM-bound; replicas",
                    flops=2.0 * m * 4096 * 4096, bytes=4.0 * (m * 4096 + 4096 * 4096 + m * 4096))
    raise SystemExit(f"unknown workload {name!r}")


# ---------------------------------------------------------------------------------------------
# clocks sampler (nvidia-smi in the background during the timed region)
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows: list[list[str]] = []
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1])); power.append(float(r[2]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------
# CPU baseline (the oracle is only ever the thing compared against / timed beside, never the product)
# ---------------------------------------------------------------------------------------------
def cpu_reference_gemm(spec: dict, threads: int, rows_per_thread: int, repeats: int = 1):
    """Times the reference's CPU matmul on `threads` independent row slabs of the workload's GEMM.
    Every output row is independent in the reference loop (support/vmath.cu:2962, 3008, 3052), so a
    slab of rows costs exactly rows/M of the whole problem."""
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    orc = oracle.Oracle("ref" if kind == "reference" else "port")
    K = spec["K"]
    N = spec["N"]
    rng = np.random.default_rng(0)
    w = rng.uniform(-1, 1, (N, K)).astype(np.float32)
    xs = [rng.uniform(-1, 1, (rows_per_thread, K)).astype(np.float32) for _ in range(threads)]
    ys = [np.empty((rows_per_thread, N), np.float32) for _ in range(threads)]
    nn = spec["kind"] == "gemm_nn"

    def one(i):
        if nn:   # C = A.B row-major, no transpose: matmul_backward_x(pgx=C, pgy=A, pw=B)
            orc._call("matmul_backward_x", oracle._ptr(ys[i]), oracle._ptr(xs[i]), oracle._ptr(w),
                      oracle._I64(K), oracle._I64(rows_per_thread), oracle._I64(N), oracle._B(False))
        else:
            orc.matmul_into(ys[i], w, xs[i], N, rows_per_thread, K)

    times = []
    with ThreadPoolExecutor(max_workers=threads) as ex:
        for _ in range(repeats):
            t0 = time.perf_counter()
            list(ex.map(one, range(threads)))
            times.append(time.perf_counter() - t0)
    flops = 2.0 * threads * rows_per_thread * N * K
    return kind, flops, times


def cpu_reference_attention(spec: dict, threads: int, repeats: int = 1):
    """The reference's attention steps (support/vmath.cu:6729-7129, host loops) on one batch item per thread;
    batch items are independent, so one item costs 1/nbat of the workload."""
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    orc = oracle.Oracle("ref" if kind == "reference" else "port")
    T, H, P = spec["ntimes"], spec["nhead"], spec["npiece"]
    rng = np.random.default_rng(0)
    items = [[rng.standard_normal((1, T, H * P)).astype(np.float32) for _ in range(3)] for _ in range(threads)]
    gys = [rng.standard_normal((1, T, H, P)).astype(np.float32) for _ in range(threads)]
    coef = float(P) ** -0.5

    def one(i):
        q, k, v = items[i]
        probs = orc.softmax_direct_on_axis(orc.mult_on_heads(k, q, H, coef))
        orc.mix_values(probs, v, H)
        if spec.get("backward"):
            gp = orc.mix_values_backward_prop(gys[i], v, H)
            orc.mix_values_backward_value(gys[i], probs, H)
            gs = orc.softmax_direct_on_axis_backward(gp, probs, coef)
            orc.mult_on_heads_backward(gs, q, H)
            orc.mult_on_heads_backward(gs, k, H)

    times = []
    with ThreadPoolExecutor(max_workers=threads) as ex:
        for _ in range(repeats):
            t0 = time.perf_counter()
            list(ex.map(one, range(threads)))
            times.append(time.perf_counter() - t0)
    flops = spec["flops"] / spec["nbat"] * threads
    return kind, flops, times


def cpu_reference_conv(spec: dict, threads: int, repeats: int = 1):
    """The reference's conv2d, conv2d_backward_x host loops and the kernel gradient on one image per thread
    (images are independent in the first two; the kernel gradient of one image is 1/ndat of the sum)."""
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    orc = oracle.Oracle("ref" if kind == "reference" else "port")
    port = oracle.Oracle("port")      # kernel gradient: the restated loop (the compiled host loop has a wrong column offset)
    cx, cy, hh, ww, kh, kw = spec["xchn"], spec["ychn"], spec["h"], spec["w"], spec["kh"], spec["kw"]
    rng = np.random.default_rng(0)
    k = rng.standard_normal((cy, cx, kh, kw)).astype(np.float32)
    xs = [rng.standard_normal((1, cx, hh, ww)).astype(np.float32) for _ in range(threads)]
    gys = [rng.standard_normal((1, cy, hh, ww)).astype(np.float32) for _ in range(threads)]

    def one(i):
        orc.conv2d(xs[i], k, hh, ww, kh // 2, kw // 2)
        orc.conv2d_backward_x(gys[i], k, hh, ww, kh // 2, kw // 2)
        port.conv2d_backward_k(gys[i], xs[i], kh, kw, kh // 2, kw // 2)

    times = []
    with ThreadPoolExecutor(max_workers=threads) as ex:
        for _ in range(repeats):
            t0 = time.perf_counter()
            list(ex.map(one, range(threads)))
            times.append(time.perf_counter() - t0)
    return kind, spec["flops"] / spec["ndat"] * threads, times


def cpu_reference_mlp(spec: dict, repeats: int = 1):
    """The reference's 15 math calls of the config-2 training step, host loops, one thread."""
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    orc = oracle.Oracle("ref" if kind == "reference" else "port")
    wl = importlib.import_module("deep-learning-framework_b200.workloads")
    d = wl.mlp(seed=0)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        h1 = orc.add_bias(orc.matmul(d["w1"], d["x"]), d["b1"])
        h2 = orc.activate(h1, 1, 0.1)
        l1 = orc.add_bias(orc.matmul(d["w2"], h2), d["b2"])
        ce = orc.softmax_idx_crossentropy(l1, d["labels"])
        orc.sum(ce)
        gl = orc.softmax_idx_crossentropy_backward_x(orc.sum_backward(ce.size), l1, d["labels"])
        orc.add_bias_backward_b(gl)
        gh2 = orc.matmul_backward_x(gl, d["w2"])
        orc.matmul_backward_w(gl, h2, *d["w2"].shape)
        gh1 = orc.activate_backward(gh2, h1, 1, 0.1)
        orc.add_bias_backward_b(gh1)
        orc.matmul_backward_w(gh1, d["x"], *d["w1"].shape)
        times.append(time.perf_counter() - t0)
    return kind, spec["flops"], times


def run_reference_arm(args, spec):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    if spec["kind"] == "attention":
        threads = min(threads, spec["nbat"])
        kind, flops, times = cpu_reference_attention(spec, threads, repeats=args.warmup + args.steps)
        sample = (f"{threads} threads x 1 batch item of {spec['nbat']} per step (batch items are independent); the "
                  "fused call has no reference counterpart and is compared with the reference's separate steps")
    elif spec["kind"] == "conv":
        threads = min(threads, spec["ndat"])
        kind, flops, times = cpu_reference_conv(spec, threads, repeats=args.warmup + args.steps)
        sample = f"{threads} threads x 1 image of {spec['ndat']} per step (forward, input gradient, kernel gradient)"
    elif spec["kind"] == "mlp":
        threads = 1
        kind, flops, times = cpu_reference_mlp(spec, repeats=args.warmup + args.steps)
        sample = "the whole 15-call step, 1 thread (the reference's host loops are single-threaded)"
    else:
        if spec["kind"] == "linear_step":
            spec = dict(spec, kind="gemm_nt")
        rows = 8 if spec["K"] * spec["N"] >= 1 << 24 else 64
        rows = min(rows, max(1, spec["M"]))
        kind, flops, times = cpu_reference_gemm(spec, threads, rows, repeats=args.warmup + args.steps)
        sample = (f"{threads} threads x {rows} output rows of the {spec['M']}x{spec['N']}x{spec['K']} GEMM per step "
                  f"({threads * rows / spec['M']:.4%} of the rows; rows are independent in the reference loop)")
    timed = times[args.warmup:]
    total = sum(timed)
    value = flops * len(timed) / total / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(timed),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": spec["desc"], "cpu": "reference VMath host loop (device=-1), -O3 -ffp-contract=off"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# GPU arm: builders of one workload's step (device-resident), its host-buffer step, and its parity check
# ---------------------------------------------------------------------------------------------
class Ctx:
    """What every workload builder needs: the bindings, this rank's place in the job, a seeded generator."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.pkg = importlib.import_module("deep-learning-framework_b200")
        self.vm, self.capi = self.pkg.vmath, self.pkg.capi
        self.lib = self.pkg.load()
        self.sharding = importlib.import_module("deep-learning-framework_b200.sharding")
        self.dev = self.local_rank
        self.gen = None

    def fresh_gen(self):
        self.gen = self.torch.Generator(device="cuda")
        self.gen.manual_seed(1234)   # same values on every rank: replicated operands are identical
        return self.gen

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        t = self.torch.tensor([v], device="cuda", dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def set_option(self, name: str, value: int):
        self.capi.call("kai_set_option", name.encode(), int(value))


class Workload:
    """step(): one pass with inputs resident in HBM.  step_e2e(): the same from pinned host buffers.
    parity(): dict of error figures for this rank's share (or None).  close(): release handles."""
    step = step_e2e = None
    parity = None
    local_flops = 0.0
    h2d = d2h = 0
    notes: dict

    def __init__(self):
        self.notes = {}
        self.extra_e2e = {}
        self._closers = []

    def close(self):
        for c in self._closers:
            c()
        self._closers = []


def _rel_fro_dev(torch, got32, truth64) -> float:
    return float(torch.linalg.norm((got32.double() - truth64).flatten()) / torch.linalg.norm(truth64.flatten()))


def build_gemm(ctx: Ctx, spec: dict, shard_mode: str, prepared: bool) -> Workload:
    torch, vm, capi, dev = ctx.torch, ctx.vm, ctx.capi, ctx.dev
    gen = ctx.fresh_gen()
    W = Workload()
    kind = spec["kind"]
    M, N, K = spec["M"], spec["N"], spec["K"]
    if spec["shard"] == "MN" and ctx.world > 1:
        if shard_mode == "columns":        # W row-slabs = output columns, X replicated
            m0, m1 = 0, M
            n0, n1 = ctx.sharding.slab(N, ctx.world, ctx.rank)
        else:                              # most square pr x pc grid of output blocks
            m0, m1, n0, n1 = ctx.sharding.block2d(M, N, ctx.world, ctx.rank)
    else:
        m0, m1, n0, n1 = 0, M, 0, N
    nl = n1 - n0
    if kind == "gemm_nn":
        a = torch.rand((M, K), device="cuda", generator=gen) * 2 - 1
        b = torch.rand((K, N), device="cuda", generator=gen) * 2 - 1
        layout = capi.GEMM_NN
        ml = M
    else:
        a_full = torch.rand((M, K), device="cuda", generator=gen) * 2 - 1
        w_full = torch.rand((N, K), device="cuda", generator=gen) * 2 - 1
        a = a_full[m0:m1].contiguous()
        b = w_full[n0:n1].contiguous()
        del w_full, a_full
        ml = m1 - m0                                  # this rank's rows of X and Y
        layout = capi.GEMM_NT
    c = torch.empty((ml, nl), device="cuda")
    W.local_flops = 2.0 * ml * nl * K
    W.shape = (ml, nl, K)
    have_prep = layout == capi.GEMM_NT and kind == "gemm_nt"
    main_prepared = bool(prepared) and have_prep
    W.scheme_mixed = bool(capi.load().kai_get_option(b"tc_cross_bf16")) and K >= 2048 and K % 8 == 0
    wp = None

    def step_plain(stream=None):
        # the reference's own call: matmul(device, Y, W, X, ...) -- both operands are split inside the call
        vm.sgemm(dev, layout, c, a, b, ml, nl, K, stream=stream)

    step_prep = None
    if have_prep:
        # W as a layer's parameter: its planes are written once, outside the timed region (it changes only at an
        # optimiser step); X is split inside every step.
        wp = vm.PreparedOperand(dev, b, nl, K)
        W._closers.append(wp.release)

        def step_prep(stream=None):
            vm.linear_forward_prepared(dev, c, wp, a, None, ml, stream=stream)
    W.step = step_prep if main_prepared else step_plain
    W.step_other = (step_plain if main_prepared else step_prep) if have_prep else None
    W.other_name = "unprepared" if main_prepared else "prepared"
    W.other_note = ("the same step through kai_matmul: W's planes written inside every call as well" if main_prepared else
                    "the same step through kai_linear_forward_prepared: W's planes written once, outside the timed region")
    # the same step with three TF32 MMAs per K step
    W.step_pure = None
    if W.scheme_mixed:
        if main_prepared:
            wp_pure = vm.PreparedOperand(dev, b, nl, K, tf32_lo=True)   # such a handle makes its calls use that scheme
            W._closers.append(wp_pure.release)

            def step_pure(stream=None):
                vm.linear_forward_prepared(dev, c, wp_pure, a, None, ml, stream=stream)
        else:
            def step_pure(stream=None):
                ctx.set_option("tc_cross_bf16", 0)        # read on the host when the call is made
                try:
                    step_plain(stream)
                finally:
                    ctx.set_option("tc_cross_bf16", 1)
        W.step_pure = step_pure
    step = W.step

    host_a = torch.empty_like(a, device="cpu").pin_memory()
    host_b = torch.empty_like(b, device="cpu").pin_memory()
    host_a.copy_(a); host_b.copy_(b)
    host_out = torch.empty_like(c, device="cpu").pin_memory()
    W.host_bufs = (host_a, host_b, host_out)
    if layout == capi.GEMM_NT and ctx.world >= 4 and shard_mode == "columns" and spec["shard"] == "MN":
        # X is replicated: every rank uploads only its 1/world of the rows over its own PCIe link and the
        # ranks exchange the slabs over NVLink (all-gather), instead of world full uploads through the
        # host's memory system; then this rank's W slab goes up, the product runs, its columns of Y go down.
        # (With two ranks the chunk-pipelined kai_matmul_host on the full X measured faster: 120 vs 104 TFLOP/s.)
        r0, r1 = ctx.sharding.slab(M, ctx.world, ctx.rank)
        even = (M % ctx.world == 0)
        x_dev = torch.empty((M, K), device="cuda")
        w_dev = torch.empty_like(b)

        def step_e2e():
            if even:
                x_dev[r0:r1].copy_(host_a[r0:r1], non_blocking=True)
                ctx.dist.all_gather_into_tensor(x_dev, x_dev[r0:r1])
            else:
                x_dev.copy_(host_a, non_blocking=True)
            w_dev.copy_(host_b, non_blocking=True)
            vm.sgemm(dev, layout, c, x_dev, w_dev, ml, nl, K)
            host_out.copy_(c, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        W.h2d = ((r1 - r0) * K + b.numel()) * 4 if even else (a.numel() + b.numel()) * 4
        W.notes["e2e_path"] = ("each rank uploads 1/world of X's rows and its W slab from pinned memory, X is "
                               "all-gathered over NVLink (NCCL), product, this rank's columns of Y downloaded")
    elif layout == capi.GEMM_NT:
        def step_e2e():
            # the host-buffer entry point: upload / multiply / download pipelined over row chunks
            vm.matmul_host(dev, host_out, host_b, host_a, nl, ml, K)

        W.h2d = (a.numel() + b.numel()) * 4
        W.notes["e2e_path"] = "kai_matmul_host (chunked upload / multiply / download pipeline; X and W uploaded every step)"
        if wp is not None:
            def step_e2e_resident():
                vm.linear_forward_host(dev, host_out, wp, host_a, ml)
            W.extra_e2e["weights_resident"] = (step_e2e_resident, a.numel() * 4, c.numel() * 4,
                                               "kai_linear_forward_host: W stays on the device as a prepared operand "
                                               "(uploaded and split once); only X goes up and Y comes down")
    else:
        a2, b2 = torch.empty_like(a), torch.empty_like(b)

        def step_e2e():
            a2.copy_(host_a, non_blocking=True)
            b2.copy_(host_b, non_blocking=True)
            vm.sgemm(dev, layout, c, a2, b2, ml, nl, K)
            host_out.copy_(c, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        W.h2d = (a.numel() + b.numel()) * 4
    W.step_e2e = step_e2e
    W.d2h = c.numel() * 4

    def parity(with_oracle: bool):
        """Relative Frobenius error of this rank's block of the LAST timed result against fp64 computed on the GPU,
        and the reference loop's own error on a 16-row slab of the same block (rows are independent)."""
        truth = (a.double() @ b.double().T) if layout == capi.GEMM_NT else (a.double() @ b.double())
        if W.step_pure is not None:
            W.step_pure()
            torch.cuda.synchronize()
            W.pure_rel_fro = _rel_fro_dev(torch, c, truth)
        step()
        torch.cuda.synchronize()
        err = _rel_fro_dev(torch, c, truth)
        out = {"rel_fro_vs_fp64": err, "bound_1e-5_sqrtK": 1e-5 * float(np.sqrt(K)), "finite": bool(torch.isfinite(c).all())}
        if with_oracle:
            import oracle
            orc = oracle.Oracle("ref" if oracle.have_ref() else "port")
            rows = slice(ml // 2, min(ml, ml // 2 + 16))
            a_s = np.ascontiguousarray(a[rows].cpu().numpy())
            b_h = np.ascontiguousarray(b.cpu().numpy())
            ref = orc.matmul(b_h, a_s) if layout == capi.GEMM_NT else orc.matmul_backward_x(a_s, b_h)
            t_s = truth[rows].cpu().numpy()
            d = np.linalg.norm((ref.astype(np.float64) - t_s).ravel()) / np.linalg.norm(t_s.ravel())
            g = np.linalg.norm((c[rows].cpu().numpy().astype(np.float64) - t_s).ravel()) / np.linalg.norm(t_s.ravel())
            out.update({"oracle_rel_fro_vs_fp64_slab": float(d), "gpu_rel_fro_vs_fp64_same_slab": float(g),
                        "oracle_slab": f"rows {rows.start}..{rows.stop - 1} of this rank's block, reference loop on CPU"})
        del truth
        out["ok"] = bool(out["finite"] and err <= out["bound_1e-5_sqrtK"] and
                         (not with_oracle or out["gpu_rel_fro_vs_fp64_same_slab"] <= 2 * out["oracle_rel_fro_vs_fp64_slab"] + 6e-8))
        return out
    W.parity = parity
    W.notes["partition"] = ("single GPU" if ctx.world == 1 or spec["shard"] != "MN" else
                            (f"columns: W row-slab [{n0},{n1}) = output columns, X replicated" if shard_mode == "columns"
                             else f"blocks: X rows [{m0},{m1}) x W rows [{n0},{n1})"))
    W.notes["weights"] = (("W prepared once outside the timed region (kai_operand_prepare: a layer's weights change "
                           "only at the optimiser step); X is split inside every step") if main_prepared else
                          "the reference's call kai_matmul(Y, W, X): both operands are split into their planes inside every step")
    return W


def build_linear_step(ctx: Ctx, spec: dict) -> Workload:
    torch, vm, dev, dist = ctx.torch, ctx.vm, ctx.dev, ctx.dist
    gen = ctx.fresh_gen()
    W = Workload()
    M, N, K = spec["M"], spec["N"], spec["K"]
    t0, t1 = ctx.sharding.slab(M, ctx.world, ctx.rank)
    ml = t1 - t0
    x = torch.randn((ml, K), device="cuda", generator=gen)
    w = torch.randn((N, K), device="cuda", generator=gen) / 64
    dy = torch.randn((ml, N), device="cuda", generator=gen)
    bias = torch.randn(N, device="cuda", generator=gen)
    y = torch.empty((ml, N), device="cuda"); dx = torch.empty((ml, K), device="cuda")
    dw = torch.empty((N, K), device="cuda")
    W.local_flops = 3 * 2.0 * ml * N * K
    # Y and dX reduce over 4096 values (mixed scheme when the option is on); dW over this rank's tokens
    W.scheme_mixed = bool(ctx.capi.load().kai_get_option(b"tc_cross_bf16")) and K >= 2048 and N >= 2048
    nslabs = 4 if ctx.world > 1 else 1
    slabs = ctx.sharding.row_slabs(N, nslabs)
    # dW = dY^T.X from the K-major planes of dY^T and X^T: written once per step (refresh), then one product per
    # row slab of dW, each followed at once by its all-reduce.
    a_prep = vm.PreparedOperand(dev, dy, N, ml, transpose=True, left=True)
    b_prep = vm.PreparedOperand(dev, x, K, ml, transpose=True)
    W._closers += [a_prep.release, b_prep.release]
    sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
    reserve = 0
    if ctx.world > 1:
        # The collective's kernels need SMs of their own: a persistent GEMM grid that holds every SM's shared
        # memory would push them between the GEMM kernels instead of under them.
        # (measured: 2 ranks 423 vs 394 TFLOP/s with 8 vs 0 SMs left free, 4 ranks 705 vs 618, 8 ranks 865 vs 925 --
        # at eight ranks the per-rank GEMMs are small and the SMs given away cost more than the overlap returns)
        reserve = int(os.environ.get("KAI_BENCH_RESERVED_SMS", "16" if ctx.world <= 4 else "0"))
        ctx.set_option("tc_max_ctas", sm_count - reserve if reserve > 0 else 0)
        W._closers.append(lambda: ctx.set_option("tc_max_ctas", 0))
    W.notes["dw_reduce"] = (f"{len(slabs)} row slabs of dW, each all-reduced (NCCL, async) right after its product; "
                            f"{reserve} SMs left to the collective (tc_max_ctas)") if ctx.world > 1 else "single GPU: no collective"

    def step():
        a_prep.refresh(dy)
        b_prep.refresh(x)
        works = []
        for r0, r1 in slabs:
            vm.sgemm_prepared(dev, dw[r0:r1], a_prep, r0, r1 - r0, b_prep, 0, K)
            if ctx.world > 1:
                works.append(dist.all_reduce(dw[r0:r1], async_op=True))
        vm.linear_forward(dev, y, w, x, bias, N, ml, K)
        vm.matmul_backward_x(dev, dx, dy, w, N, ml, K)
        for wk in works:
            wk.wait()
    W.step = step

    host_in = [t.cpu().pin_memory() for t in (x, dy)]
    host_out = torch.empty_like(dw, device="cpu").pin_memory()

    def step_e2e():
        x.copy_(host_in[0], non_blocking=True)
        dy.copy_(host_in[1], non_blocking=True)
        step()
        host_out.copy_(dw, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    W.step_e2e = step_e2e
    W.h2d = (x.numel() + dy.numel()) * 4
    W.d2h = dw.numel() * 4

    def parity(with_oracle: bool):
        step()
        torch.cuda.synchronize()
        out = {}
        ty = x.double() @ w.double().T + bias.double()
        out["y_rel_fro_vs_fp64"] = _rel_fro_dev(torch, y, ty); del ty
        tx = dy.double() @ w.double()
        out["dx_rel_fro_vs_fp64"] = _rel_fro_dev(torch, dx, tx); del tx
        tw = dy.double().T @ x.double()
        if ctx.world > 1:
            dist.all_reduce(tw)
        out["dw_rel_fro_vs_fp64"] = _rel_fro_dev(torch, dw, tw); del tw
        out["bound_1e-5_sqrtK"] = 1e-5 * float(np.sqrt(K))
        out["ok"] = bool(max(out["y_rel_fro_vs_fp64"], out["dx_rel_fro_vs_fp64"]) <= out["bound_1e-5_sqrtK"] and
                         out["dw_rel_fro_vs_fp64"] <= 1e-5 * float(np.sqrt(M)))
        return out
    W.parity = parity
    return W


def build_attention(ctx: Ctx, spec: dict) -> Workload:
    torch, vm, dev = ctx.torch, ctx.vm, ctx.dev
    gen = ctx.fresh_gen()
    W = Workload()
    nb, T, H, P = spec["nbat"], spec["ntimes"], spec["nhead"], spec["npiece"]
    b0, b1 = ctx.sharding.slab(nb, ctx.world, ctx.rank)
    bl = b1 - b0
    q = torch.randn((bl, T, H * P), device="cuda", generator=gen)
    k = torch.randn((bl, T, H * P), device="cuda", generator=gen)
    v = torch.randn((bl, T, H * P), device="cuda", generator=gen)
    fused = bool(spec.get("fused"))
    bwd = bool(spec.get("backward"))
    probs = None if fused else torch.empty((bl, T, T, H), device="cuda")
    out = torch.empty((bl, T, H, P), device="cuda")
    coef_val = 1.0 / float(np.sqrt(P))
    coef = torch.tensor([coef_val], device="cuda")
    W.local_flops = (6 if bwd else 2) * 2.0 * bl * H * T * T * P
    W.dims = (bl, T, H, P)
    if bwd:
        gy = torch.randn((bl, T, H, P), device="cuda", generator=gen)
        gprobs = torch.empty_like(probs)
        gq, gk, gv = (torch.empty_like(q) for _ in range(3))

    def step():
        if fused:
            vm.mh_attention_forward(dev, out, k, q, v, bl, T, H * P, H, P, coef)
            return
        vm.mult_on_heads(dev, probs, k, q, bl, T, H * P, H, P, coef)
        vm.softmax_direct_on_axis(dev, probs, bl * T, T, H)
        vm.mix_values(dev, out, probs, v, bl, T, H * P, H, P)
        if bwd:   # api_objects/vtensor.cpp:3145-3154
            vm.mix_values_backward_prop(dev, gprobs, gy, v, bl, T, H * P, H, P)
            vm.mix_values_backward_value(dev, gv, gy, probs, bl, T, H * P, H, P)
            vm.softmax_direct_on_axis_backward(dev, gprobs, probs, bl, T, H, coef)
            vm.mult_on_heads_backward(dev, gk, gprobs, q, bl, T, H * P, H, P)
            vm.mult_on_heads_backward(dev, gq, gprobs, k, bl, T, H * P, H, P)
    W.step = step

    host_in = [t.cpu().pin_memory() for t in (q, k, v)]
    host_out = torch.empty_like(out, device="cpu").pin_memory()

    def step_e2e():
        for d, h in zip((q, k, v), host_in):
            d.copy_(h, non_blocking=True)
        step()
        host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    W.step_e2e = step_e2e
    W.h2d = 3 * q.numel() * 4
    W.d2h = out.numel() * 4

    def parity(with_oracle: bool):
        step()
        torch.cuda.synchronize()
        worst = 0.0
        for g0 in range(0, bl, 4):     # fp64 softmax attention on the GPU, four batch items at a time
            g1 = min(bl, g0 + 4)
            q4, k4, v4 = (t[g0:g1].double().view(g1 - g0, T, H, P).permute(0, 2, 1, 3) for t in (q, k, v))
            pr = torch.softmax((q4 @ k4.transpose(-1, -2)) * coef_val, dim=-1)
            o = (pr @ v4).permute(0, 2, 1, 3).contiguous()
            worst = max(worst, _rel_fro_dev(torch, out[g0:g1], o))
            del pr, o
        res = {"out_rel_fro_vs_fp64": worst, "bound_1e-5_sqrtK": 1e-5 * float(np.sqrt(T)),
               "finite": bool(torch.isfinite(out).all())}
        if with_oracle:
            import oracle
            orc = oracle.Oracle("ref" if oracle.have_ref() else "port")
            qh, kh, vh = (t[:1].cpu().numpy() for t in (q, k, v))
            ref = orc.mix_values(orc.softmax_direct_on_axis(orc.mult_on_heads(kh, qh, H, coef_val)), vh, H)
            q4, k4, v4 = (t[:1].double().view(1, T, H, P).permute(0, 2, 1, 3) for t in (q, k, v))
            o = (torch.softmax((q4 @ k4.transpose(-1, -2)) * coef_val, dim=-1) @ v4).permute(0, 2, 1, 3).cpu().numpy()
            res["oracle_rel_fro_vs_fp64_one_item"] = float(np.linalg.norm((ref - o).ravel()) / np.linalg.norm(o.ravel()))
        res["ok"] = bool(res["finite"] and worst <= res["bound_1e-5_sqrtK"] and
                         (not with_oracle or worst <= 2 * res["oracle_rel_fro_vs_fp64_one_item"] + 6e-8))
        return res
    W.parity = parity
    return W


def build_conv(ctx: Ctx, spec: dict) -> Workload:
    torch, vm, dev, dist = ctx.torch, ctx.vm, ctx.dev, ctx.dist
    gen = ctx.fresh_gen()
    W = Workload()
    n0, n1 = ctx.sharding.slab(spec["ndat"], ctx.world, ctx.rank)
    nl = n1 - n0
    cx, cy, hh, ww, kh, kw = spec["xchn"], spec["ychn"], spec["h"], spec["w"], spec["kh"], spec["kw"]
    x = torch.randn((nl, cx, hh, ww), device="cuda", generator=gen)
    kk = torch.randn((cy, cx, kh, kw), device="cuda", generator=gen) / (cx * kh * kw) ** 0.5
    gy = torch.randn((nl, cy, hh, ww), device="cuda", generator=gen)
    y, gx, gk = torch.empty_like(gy), torch.empty_like(x), torch.empty_like(kk)
    W.local_flops = spec["flops"] * nl / spec["ndat"]

    def step():
        vm.conv2d(dev, y, x, kk, nl, cy, hh, ww, cx, hh, ww, kh, kw, 1, kh // 2, kw // 2)
        vm.conv2d_backward_x(dev, gx, gy, kk, nl, cx, hh, ww, cy, hh, ww, kh, kw, 1, kh // 2, kw // 2)
        vm.conv2d_backward_k(dev, gk, gy, x, nl, cx, hh, ww, cy, hh, ww, kh, kw, 1, kh // 2, kw // 2)
        if ctx.world > 1:
            dist.all_reduce(gk)
    W.step = step
    host_in = [t_.cpu().pin_memory() for t_ in (x, gy)]
    host_out = torch.empty_like(gk, device="cpu").pin_memory()

    def step_e2e():
        x.copy_(host_in[0], non_blocking=True)
        gy.copy_(host_in[1], non_blocking=True)
        step()
        host_out.copy_(gk, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    W.step_e2e = step_e2e
    W.h2d = (x.numel() + gy.numel()) * 4
    W.d2h = gk.numel() * 4

    def parity(with_oracle: bool):
        step()
        torch.cuda.synchronize()
        F = torch.nn.functional
        x64 = x.double().requires_grad_(True)
        k64 = kk.double().requires_grad_(True)
        y64 = F.conv2d(x64, k64, padding=(kh // 2, kw // 2))
        y64.backward(gy.double())
        tgk = k64.grad
        if ctx.world > 1:
            dist.all_reduce(tgk)
        res = {"y_rel_fro_vs_fp64": _rel_fro_dev(torch, y, y64.detach()),
               "gx_rel_fro_vs_fp64": _rel_fro_dev(torch, gx, x64.grad),
               "gk_rel_fro_vs_fp64": _rel_fro_dev(torch, gk, tgk)}
        res["ok"] = bool(max(res["y_rel_fro_vs_fp64"], res["gx_rel_fro_vs_fp64"]) <= 1e-5 * np.sqrt(cx * kh * kw) and
                         res["gk_rel_fro_vs_fp64"] <= 1e-5 * np.sqrt(spec["ndat"] * hh * ww))
        return res
    W.parity = parity
    return W


def build_rnn(ctx: Ctx, spec: dict) -> Workload:
    torch, vm, dev = ctx.torch, ctx.vm, ctx.dev
    gen = ctx.fresh_gen()
    W = Workload()
    T, B, I, R, NG = spec["ntimes"], spec["ndat"], spec["ninp"], spec["nrec"], spec["ngates"]
    G = NG * R
    x = torch.randn((T, B, I), device="cuda", generator=gen)
    wi = torch.randn((G, I), device="cuda", generator=gen) / I ** 0.5
    wr = torch.randn((G, R), device="cuda", generator=gen) / R ** 0.5
    bb = torch.randn((G,), device="cuda", generator=gen)
    aff = torch.zeros((T, B, G), device="cuda")
    rec = torch.zeros((T, B, R), device="cuda")
    W.local_flops = spec["flops"]

    def step(stream=None, batched=False, grouped=False):
        # api_objects/vtensor.cpp:2456-2495; the cell update is stood in for by tanh of the first gate block
        if batched:
            vm.matmul(dev, aff, wi, x, G, T * B, I, False, stream=stream)
        elif grouped:      # all input products as ONE grouped launch (they do not depend on each other)
            vm.sgemm_grouped(dev, 0, [aff[t_] for t_ in range(T)], [x[t_] for t_ in range(T)], [wi] * T, B, G, I,
                             accumulate=False, stream=stream)
        for t_ in range(T):
            if t_ > 0:
                vm.matmul(dev, aff[t_], wr, rec[t_ - 1], G, B, R, batched or grouped, stream=stream)
            if not (batched or grouped):
                vm.matmul(dev, aff[t_], wi, x[t_], G, B, I, True, stream=stream)
            vm.add_bias(dev, aff[t_], aff[t_], bb, B, G, stream=stream)
            vm.activate(dev, rec[t_], aff[t_].view(-1)[: B * R].view(B, R), B, R, 4, None, stream=stream)
    W.step = step
    host_x = x.cpu().pin_memory()
    host_out = torch.empty((B, R)).pin_memory()

    def step_e2e():
        x.copy_(host_x, non_blocking=True)
        step()
        host_out.copy_(rec[T - 1], non_blocking=True)
        torch.cuda.current_stream().synchronize()
    W.step_e2e = step_e2e
    W.h2d = x.numel() * 4
    W.d2h = B * R * 4
    return W


def build_mlp(ctx: Ctx, spec: dict) -> Workload:
    torch, vm, dev = ctx.torch, ctx.vm, ctx.dev
    W = Workload()
    wl = importlib.import_module("deep-learning-framework_b200.workloads")
    d = wl.mlp(seed=0)
    t = {k: torch.from_numpy(v).cuda() for k, v in d.items()}
    B, D = d["x"].shape
    Hd, C = d["w1"].shape[0], d["w2"].shape[0]
    alpha = torch.tensor([0.1], device="cuda")
    z = lambda *sh: torch.empty(sh, device="cuda")  # noqa: E731
    h0, h1, h2, l0, l1 = z(B, Hd), z(B, Hd), z(B, Hd), z(B, C), z(B, C)
    ce, loss, gce, gl = z(B), z(1), z(B), z(B, C)
    gb2, gh2, gw2, gh1, gb1, gw1 = z(C), z(B, Hd), z(C, Hd), z(B, Hd), z(Hd), z(Hd, D)
    W.local_flops = spec["flops"]

    def step(stream=None):  # the reference's call list for this model (forward, loss, backward)
        vm.matmul(dev, h0, t["w1"], t["x"], Hd, B, D, False, stream=stream)
        vm.add_bias(dev, h1, h0, t["b1"], B, Hd, stream=stream)
        vm.activate(dev, h2, h1, B, Hd, 1, alpha, stream=stream)
        vm.matmul(dev, l0, t["w2"], h2, C, B, Hd, False, stream=stream)
        vm.add_bias(dev, l1, l0, t["b2"], B, C, stream=stream)
        vm.softmax_idx_crossentropy(dev, ce, l1, t["labels"], B, C, stream=stream)
        vm.sum(dev, loss, ce, B, stream=stream)
        vm.sum_backward(dev, gce, None, B, stream=stream)
        vm.softmax_idx_crossentropy_backward_x(dev, gl, gce, l1, t["labels"], B, C, stream=stream)
        vm.add_bias_backward_b(dev, gb2, gl, B, C, False, stream=stream)
        vm.matmul_backward_x(dev, gh2, gl, t["w2"], C, B, Hd, False, stream=stream)
        vm.matmul_backward_w(dev, gw2, gl, h2, C, B, Hd, False, stream=stream)
        vm.activate_backward(dev, gh1, gh2, h1, B, Hd, 1, alpha, stream=stream)
        vm.add_bias_backward_b(dev, gb1, gh1, B, Hd, False, stream=stream)
        vm.matmul_backward_w(dev, gw1, gh1, t["x"], Hd, B, D, False, stream=stream)
    W.step = step
    host_x = t["x"].cpu().pin_memory()
    host_loss = torch.empty(1).pin_memory()

    def step_e2e():
        t["x"].copy_(host_x, non_blocking=True)
        step()
        host_loss.copy_(loss, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    W.step_e2e = step_e2e
    W.h2d = host_x.numel() * 4
    W.d2h = 4

    def parity(with_oracle: bool):
        step()
        torch.cuda.synchronize()
        if not with_oracle:
            return None
        import oracle
        orc = oracle.Oracle("ref" if oracle.have_ref() else "port")
        hh1 = orc.add_bias(orc.matmul(d["w1"], d["x"]), d["b1"])
        hh2 = orc.activate(hh1, 1, 0.1)
        ll1 = orc.add_bias(orc.matmul(d["w2"], hh2), d["b2"])
        want = float(orc.sum(orc.softmax_idx_crossentropy(ll1, d["labels"]))[0])
        got = float(loss.item())
        ggl = orc.softmax_idx_crossentropy_backward_x(orc.sum_backward(B), ll1, d["labels"])
        ggh1 = orc.activate_backward(orc.matmul_backward_x(ggl, d["w2"]), hh1, 1, 0.1)
        want_gw1 = orc.matmul_backward_w(ggh1, d["x"], Hd, D)
        e = float(np.linalg.norm(gw1.cpu().numpy() - want_gw1) / np.linalg.norm(want_gw1))
        return {"loss": got, "oracle_loss": want, "loss_rel_diff": abs(got - want) / abs(want),
                "gW1_rel_fro_vs_oracle": e, "ok": bool(abs(got - want) <= 1e-5 * abs(want) and e <= 1e-5)}
    W.parity = parity
    return W


def build_workload(ctx: Ctx, spec: dict, shard_mode: str, prepared: bool) -> Workload:
    kind = spec["kind"]
    if kind in ("gemm_nt", "gemm_nn", "skinny"):
        return build_gemm(ctx, spec, shard_mode, prepared)
    if kind == "linear_step":
        return build_linear_step(ctx, spec)
    if kind == "attention":
        return build_attention(ctx, spec)
    if kind == "conv":
        return build_conv(ctx, spec)
    if kind == "rnn":
        return build_rnn(ctx, spec)
    if kind == "mlp":
        return build_mlp(ctx, spec)
    raise SystemExit(kind)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm8192")
    ap.add_argument("--shard", default="columns", choices=["columns", "blocks"],
                    help="partition of the large NT GEMM over GPUs: W row-slabs = output columns with X replicated "
                         "(the named configuration, default), or a pr x pc grid of output blocks")
    ap.add_argument("--unprepared", action="store_true",
                    help="time the reference's own call kai_matmul (W split inside every step as well) instead of "
                         "kai_linear_forward_prepared; the other one is reported beside it")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the sustained run, the other partition and the other configurations' lines")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="library tuning switch for this run (kai_set_option), e.g. tc_min_flops=0")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    spec = workload_spec(args.workload, int(os.environ.get("WORLD_SIZE", "1")))
    if args.impl == "reference":
        run_reference_arm(args, spec)
        return

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    # The collective of the Linear step runs beside the GEMM kernels on SMs left free for it (tc_max_ctas).
    default_reserve = "16" if int(os.environ.get("WORLD_SIZE", "1")) <= 4 else "0"
    if int(os.environ.get("KAI_BENCH_RESERVED_SMS", default_reserve)) > 0:
        os.environ.setdefault("NCCL_MAX_CTAS", os.environ.get("KAI_BENCH_RESERVED_SMS", default_reserve))
    ctx = Ctx(args)
    torch, dist, vm, capi, lib = ctx.torch, ctx.dist, ctx.vm, ctx.capi, ctx.lib
    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    for opt in args.option:
        name, _, val = opt.partition("=")
        ctx.set_option(name, int(val))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback for the GPU arm")
    torch.cuda.set_device(ctx.local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", ctx.local_rank))

    kind = spec["kind"]
    W = build_workload(ctx, spec, args.shard, not args.unprepared)
    scheme_mixed = bool(getattr(W, "scheme_mixed", False))
    step = W.step
    notes_main = dict(W.notes)

    # Small workloads live in L2: evict between steps by overwriting a buffer larger than L2.
    small = kind in ("gemm_nn", "skinny", "mlp", "rnn") or (kind == "gemm_nt" and spec["M"] * spec["K"] * 4 < (256 << 20))
    # L2 flush = overwrite a buffer larger than L2, then read a second one: the read pass pushes the dirty
    # lines of the write pass out to HBM before the timed call starts (otherwise their write-back competes
    # with the call's own traffic).
    flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda") if small else None
    flush_rd = torch.zeros(192 << 20, dtype=torch.uint8, device="cuda") if small else None

    def flush_l2():
        flush.fill_(1)
        flush_rd.max()

    lead_in = kind in ("skinny", "gemm_nn")      # single-kernel steps of a few microseconds

    def timed_loop(fn, steps, flush_between):
        """Device time of `steps` calls; with L2 flushing each call is bracketed by its own events."""
        if not flush_between:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1)
        total = 0.0
        for _ in range(steps):
            flush_l2()
            if lead_in:
                # a spin kernel ahead of the start event: the host queues the call while the GPU spins, so the events
                # bracket device time and not the host's launch path (a 10-20 us call would otherwise be timed together
                # with several microseconds of an idle GPU waiting for its launch)
                torch.cuda._sleep(200000)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total

    # ---- dense TF32 peak of this GPU, same method as the driver's bf16 figure -----------------
    tf32_peak = None
    if rank == 0 and kind in ("gemm_nt", "gemm_nn", "linear_step", "conv"):
        n = 8192
        pa = torch.randn(n, n, device="cuda"); pb = torch.randn(n, n, device="cuda")
        torch.backends.cuda.matmul.allow_tf32 = True
        for _ in range(3):
            torch.matmul(pa, pb)
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); torch.matmul(pa, pb); e1.record(); torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        torch.backends.cuda.matmul.allow_tf32 = False
        tf32_peak = 2.0 * n ** 3 / best / 1e9
        del pa, pb
        torch.cuda.empty_cache()

    # ---- warm-up, then the timed region --------------------------------------------------------
    for _ in range(args.warmup):
        step()
    ctx.barrier()
    sampler = ClockSampler(ctx.local_rank)
    if rank == 0:
        sampler.start()
    capi.call("kai_profile_enable", 1)
    launches0 = lib.kai_launch_count()
    ctx.barrier()
    ms = timed_loop(step, args.steps, small)
    ctx.barrier()
    launches = lib.kai_launch_count() - launches0
    import ctypes
    prof_ms = (ctypes.c_double * 3)(); prof_n = (ctypes.c_int64 * 3)()
    capi.call("kai_profile_read", prof_ms, prof_n)
    capi.call("kai_profile_enable", 0)
    clocks = sampler.stop() if rank == 0 else None
    ms_max = ctx.max_over_ranks(ms)
    total_flops = spec["flops"] if spec["shard"] else spec["flops"] * world  # replicas: every rank does it all
    value = total_flops * args.steps / (ms_max * 1e-3) / 1e12

    def quick_time(fn, steps=None, warm=2, like_main=False):
        """A short timed run of another step function (max over ranks), for the side figures of the line.
        `like_main`: as many steps and warm-up steps as the main region, so that a figure that is compared with
        the headline sees the same power state (a ten-step burst after a pause runs ~10 % faster than step 50)."""
        steps = steps or min(args.steps, 10)
        if like_main:
            steps, warm = args.steps, max(args.warmup, warm)
        for _ in range(warm):
            fn()
        ctx.barrier()
        t = timed_loop(fn, steps, small)
        ctx.barrier()
        return ctx.max_over_ranks(t) / steps

    other_path = None
    other_name = getattr(W, "other_name", "prepared")
    if getattr(W, "step_other", None) is not None:
        ums = quick_time(W.step_other, like_main=True)
        other_path = {"ms_per_step": ums, "value": total_flops / (ums * 1e-3) / 1e12, "note": W.other_note}

    pure = None
    if getattr(W, "step_pure", None) is not None:
        pms = quick_time(W.step_pure, like_main=True)
        pure = {"ms_per_step": pms, "value": total_flops / (pms * 1e-3) / 1e12,
                "note": "the same step with three TF32 MMAs per K step (hi.hi, hi.lo, lo.hi) instead of one TF32 MMA "
                        "plus one BF16 MMA for the two cross terms"}

    # ---- the same call list recorded once and replayed as one launch (latency-bound workloads) ----
    replay = None
    if kind in ("mlp", "gemm_nn", "skinny", "rnn"):
        with vm.Replay(dev) as rp:
            step(stream=rp.stream)
        for _ in range(3):
            rp.launch()
        rms = timed_loop(rp.launch, args.steps, True)
        # back to back without a flush: the launch-latency floor of the list
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(200):
            rp.launch()
        e1.record()
        torch.cuda.synchronize()
        replay = {"us_per_step": rms * 1e3 / args.steps, "us_per_step_call_by_call": ms * 1e3 / args.steps,
                  "us_per_step_back_to_back_warm_l2": e0.elapsed_time(e1) * 1e3 / 200,
                  "calls_recorded": int(launches / args.steps),
                  "note": "one cudaGraphLaunch per step (kai_replay_*); L2 flushed between steps except in the "
                          "back-to-back figure"}
        rp.close()
        if kind == "rnn":   # the input products of all timesteps as one GEMM / one grouped launch, recorded the same way
            for name, kw in (("batched_input_gemm", dict(batched=True)), ("grouped_input_products", dict(grouped=True))):
                step(**kw)
                with vm.Replay(dev) as rpb:
                    step(stream=rpb.stream, **kw)
                for _ in range(3):
                    rpb.launch()
                replay[f"us_per_step_{name}"] = timed_loop(rpb.launch, args.steps, True) * 1e3 / args.steps
                replay[f"us_per_step_{name}_call_by_call"] = timed_loop(lambda: step(**kw), args.steps, True) * 1e3 / args.steps
                rpb.close()

    # ---- end to end through the C ABI with host buffers ------------------------------------------
    e2e = None
    if not args.no_e2e:
        def time_e2e(fn, n):
            for _ in range(2):
                fn()
            ctx.barrier()
            t0 = time.perf_counter()
            for _ in range(n):
                fn()
            ctx.barrier()
            return ctx.max_over_ranks(time.perf_counter() - t0)

        e2e_steps = min(args.steps, 10)
        te = time_e2e(W.step_e2e, e2e_steps)
        e2e = {"value": total_flops * e2e_steps / te / 1e12, "unit": UNIT, "steps": e2e_steps,
               "ms_per_step": 1e3 * te / e2e_steps,
               "h2d_bytes_per_step": int(W.h2d), "d2h_bytes_per_step": int(W.d2h),
               "timing": "host clock around steps that each end with the result in pinned host memory; max over ranks",
               "path": W.notes.get("e2e_path", "torch copies from / to pinned memory around the device calls")}
        # Floor of the copies alone: every rank moves its bytes up and down at the same time, nothing else runs.
        if W.h2d + W.d2h >= (8 << 20):
            up = torch.empty(int(W.h2d), dtype=torch.uint8, device="cuda")
            dn = torch.empty(int(W.d2h), dtype=torch.uint8, device="cuda")
            hup = torch.empty(int(W.h2d), dtype=torch.uint8).pin_memory()
            hdn = torch.empty(int(W.d2h), dtype=torch.uint8).pin_memory()
            s2 = torch.cuda.Stream()

            def copies():
                up.copy_(hup, non_blocking=True)
                with torch.cuda.stream(s2):
                    hdn.copy_(dn, non_blocking=True)
                s2.synchronize()
                torch.cuda.current_stream().synchronize()
            tc = time_e2e(copies, 5)
            e2e["copy_floor_ms"] = 1e3 * tc / 5
            e2e["copy_floor_note"] = ("all ranks copy h2d_bytes up and d2h_bytes down concurrently from / to pinned "
                                      "memory, no compute: what the host's PCIe and memory system allow")
            del up, dn, hup, hdn
        for name, (fn, hb, db, note) in W.extra_e2e.items():
            tx = time_e2e(fn, e2e_steps)
            e2e[name] = {"value": total_flops * e2e_steps / tx / 1e12, "ms_per_step": 1e3 * tx / e2e_steps,
                         "h2d_bytes_per_step": int(hb), "d2h_bytes_per_step": int(db), "path": note}

    # ---- parity of the benchmarked launch itself ---------------------------------------------------
    parity = None
    if W.parity is not None:
        p = W.parity(with_oracle=(rank == 0 and not args.no_cpu_baseline))
        if p is not None:
            ok_all = ctx.max_over_ranks(0.0 if p.get("ok") else 1.0) == 0.0
            parity = dict(p, ok=bool(ok_all), ranks_checked=world)
    pure_rel_fro = getattr(W, "pure_rel_fro", None)

    # ---- sustained figure: the same step for >= 2 s (the board settles at its power limit) ---------
    sustained = None
    if not args.no_extras and kind in ("gemm_nt", "linear_step") and not small:
        per = ms_max / args.steps
        n_s = max(20, int(2500.0 / max(per, 1e-3)))
        s2 = ClockSampler(ctx.local_rank)
        ctx.barrier()
        if rank == 0:
            s2.start()
        t_s = timed_loop(step, n_s, False)
        ctx.barrier()
        c2 = s2.stop() if rank == 0 else None
        t_s = ctx.max_over_ranks(t_s)
        sustained = {"ms_per_step": t_s / n_s, "tflops": total_flops * n_s / (t_s * 1e-3) / 1e12,
                     "seconds": t_s * 1e-3, "steps": n_s, "clocks": c2}

    # ---- the other partition of the large GEMM, and the other configurations at this N ------------
    alt_partition = None
    other_configs = None
    main_was_default = args.workload == "gemm8192"
    if not args.no_extras and kind == "gemm_nt" and spec["shard"] == "MN" and world > 1:
        other = "blocks" if args.shard == "columns" else "columns"
        W.close(); del W, step
        torch.cuda.empty_cache()
        W2 = build_workload(ctx, spec, other, not args.unprepared)
        ams = quick_time(W2.step)
        alt_partition = {"partition": other, "ms_per_step": ams, "value": total_flops / (ams * 1e-3) / 1e12,
                         "note": W2.notes.get("partition")}
        W2.close(); del W2
        torch.cuda.empty_cache()
        W = None
    if not args.no_extras and main_was_default:
        if W is not None:
            W.close()
        W = None
        torch.cuda.empty_cache()
        other_configs = {}
        for name in ("linear_step", "attention", "attention_fused"):
            sp = workload_spec(name, world)
            Wo = build_workload(ctx, sp, args.shard, True)
            oms = quick_time(Wo.step)
            entry = {"ms_per_step": oms, "tflops": sp["flops"] / (oms * 1e-3) / 1e12, "n_gpus": world,
                     "workload": sp["desc"]}
            entry.update(Wo.notes)
            if Wo.parity is not None:
                pp = Wo.parity(with_oracle=False)
                if pp is not None:
                    entry["parity_ok"] = bool(ctx.max_over_ranks(0.0 if pp.get("ok") else 1.0) == 0.0)
            other_configs[name] = entry
            Wo.close(); del Wo
            torch.cuda.empty_cache()

    rc = lib.kai_device_status(dev, None)
    if rc != 0:
        raise SystemExit(f"device status {rc}: {lib.kai_last_error_string().decode()}")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel -----------------------------------------------------------
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except (OSError, ValueError):
        pass
    local_flops = spec["flops"] / world if spec["shard"] else spec["flops"]
    if kind == "skinny":
        hbm = peaks.get("hbm_gbs", 6650.0)
        achieved = spec["bytes"] * args.steps / (ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                    "traffic": TRAFFIC_BYTES.get(args.workload),
                    "kernel": "skinny_fma_kernel" if spec["M"] <= 4 else "skinny_mma_kernel",
                    "peak_source": "MEASURED_PEAKS.json hbm_gbs" if "hbm_gbs" in peaks else "fallback 6650 GB/s",
                    "algorithmic_bytes_per_launch": spec["bytes"]}
    elif kind == "conv":
        peak = (tf32_peak or 0.0) / 3.0
        achieved = local_flops * args.steps / (ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak if peak else None, "traffic": None,
                    "kernel": "whole step: pad_channels_last + conv_igemm_tma (forward, input gradient); im2col_t + gemm_3xtf32 + fixup (kernel gradient)",
                    "gemm_kernels_ms_per_step": prof_ms[0] / args.steps,
                    "split_kernels_ms_per_step": prof_ms[1] / args.steps,
                    "peak_source": f"dense TF32 measured in this run ({tf32_peak:.1f} TFLOP/s) / 3",
                    "algorithmic_flops_per_launch": local_flops}
    elif prof_n[0] > 0:
        gemm_ms = prof_ms[0] / prof_n[0]
        per_launch_flops = local_flops / (prof_n[0] / args.steps)
        achieved = per_launch_flops / (gemm_ms * 1e-3) / 1e12
        # MMA slots per 8-wide K step: three TF32 MMAs, or (reductions of 2048 and more) one TF32 MMA and one BF16
        # MMA of the same duration that forms both cross terms
        mixed = scheme_mixed
        slots = 2.0 if mixed else 3.0
        pair = bool(lib.kai_get_option(b"tc_pair"))
        peak = (tf32_peak or 0.0) / slots
        roofline = {
            "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak if peak else None, "traffic": TRAFFIC_BYTES.get(args.workload),
            "kernel": "gemm_3xtf32_pair_kernel<32>" if pair else "gemm_3xtf32_kernel<256,16>",
            "mma_per_k_step": "1 TF32 (hi.hi) + 1 BF16 (hi.lo + lo.hi)" if mixed else "3 TF32 (lo.hi, hi.lo, hi.hi)",
            "launches": int(prof_n[0]), "avg_ms": gemm_ms,
            "peak_source": f"dense TF32 measured in this run (torch.matmul 8192^3, best of 10: {tf32_peak:.1f} TFLOP/s) "
                           f"/ {slots:.0f} tcgen05.mma slots per product; MEASURED_PEAKS.json carries no TF32 figure "
                           f"(its bf16_tflops/{2 * slots:.0f} = {peaks.get('bf16_tflops', 0) / (2 * slots):.1f})",
            "frac_of_3xtf32_peak": achieved / ((tf32_peak or 0.0) / 3.0) if tf32_peak else None,
            "frac_of_bf16_measured_over_6": achieved / (peaks["bf16_tflops"] / 6.0) if "bf16_tflops" in peaks else None,
            "frac_of_nominal": achieved / (NOMINAL_TF32_DENSE / slots),
            "algorithmic_flops_per_launch": per_launch_flops,
            "split_kernels_ms_per_step": prof_ms[1] / args.steps,
        }
    elif kind == "attention":
        # Unfused trio in the reference layouts: Q,K read, probs written; probs read + written (softmax in
        # place); probs + V read, out written.  Batch-sharded: this rank's share.
        nb, T, H, P = spec["nbat"], spec["ntimes"], spec["nhead"], spec["npiece"]
        bl = nb // world if nb % world == 0 else -(-nb // world)
        qkv = bl * T * H * P * 4.0
        pr = bl * T * T * H * 4.0
        alg = (2 * qkv + pr) + (2 * pr) + (pr + qkv + qkv)
        kernel_names = "mult_on_heads_tc + softmax_axis_warp + mix_values_tc (whole step)"
        if spec.get("fused"):   # Q, K, V read once, O written once
            alg = 4 * qkv
            kernel_names = "mh_attention_fused_kernel + operand split kernels (whole step)"
        if spec.get("backward"):
            # gprobs written; probs + gy read, gV written; probs + gprobs read, gprobs written;
            # twice (gprobs + operand read, gradient written)
            alg += (2 * qkv + pr) + (pr + 2 * qkv) + (3 * pr) + 2 * (pr + 2 * qkv)
        hbm = peaks.get("hbm_gbs", 6650.0)
        achieved = alg * args.steps / (ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                    "traffic": TRAFFIC_BYTES.get(args.workload), "kernel": kernel_names,
                    "peak_source": "MEASURED_PEAKS.json hbm_gbs" if "hbm_gbs" in peaks else "fallback 6650 GB/s",
                    "algorithmic_bytes_per_launch": alg}
    else:
        roofline = {"bound": "latency", "achieved": None, "peak": None, "unit": "us", "frac": None,
                    "traffic": None, "note": "launch-latency regime: a few microseconds of work per call"}
    if sustained is not None and "bf16_tflops_sustained" in peaks and kind == "gemm_nt":
        sustained["frac_of_bf16_sustained_over_6"] = sustained["tflops"] / world / (peaks["bf16_tflops_sustained"] / 6.0)
        sustained["sm_mhz_median"] = (sustained["clocks"] or {}).get("sm_mhz")

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline and kind == "attention":
        ckind, cflops, ctimes = cpu_reference_attention(spec, 1, repeats=1)
        cpu_baseline = {"value": cflops / ctimes[0] / 1e12, "unit": UNIT, "cores": 1, "kind": ckind,
                        "host_cores": os.cpu_count(),
                        "sample": f"1 batch item of {spec['nbat']} ({ctimes[0]:.1f} s, 1 thread), the reference's "
                                  "separate steps"}
    elif world == 1 and not args.no_cpu_baseline and kind == "conv":
        ckind, cflops, ctimes = cpu_reference_conv(spec, 1, repeats=1)
        cpu_baseline = {"value": cflops / ctimes[0] / 1e12, "unit": UNIT, "cores": 1, "kind": ckind,
                        "host_cores": os.cpu_count(),
                        "sample": f"1 image of {spec['ndat']} ({ctimes[0]:.1f} s, 1 thread): forward, input gradient, "
                                  "kernel gradient"}
    elif world == 1 and not args.no_cpu_baseline and kind == "mlp":
        ckind, cflops, ctimes = cpu_reference_mlp(spec, repeats=3)
        cpu_baseline = {"value": cflops / min(ctimes) / 1e12, "unit": UNIT, "cores": 1, "kind": ckind,
                        "host_cores": os.cpu_count(), "us_per_step": min(ctimes) * 1e6,
                        "sample": "the whole 15-call step, best of 3, 1 thread"}
    elif world == 1 and not args.no_cpu_baseline and kind in ("gemm_nt", "gemm_nn", "linear_step", "skinny"):
        sp = dict(spec, kind="gemm_nt") if kind == "linear_step" else spec
        rows = min(128 if sp["K"] * sp["N"] >= 1 << 24 else 512, sp["M"])
        ckind, cflops, ctimes = cpu_reference_gemm(sp, 1, rows, repeats=1)
        cpu_baseline = {"value": cflops / ctimes[0] / 1e12, "unit": UNIT, "cores": 1, "kind": ckind,
                        "host_cores": os.cpu_count(),
                        "sample": f"{rows} output rows of the {sp['M']}x{sp['N']}x{sp['K']} GEMM "
                                  f"({ctimes[0]:.1f} s, 1 thread: the reference's host loop is single-threaded)"}

    notes = dict(notes_main)
    notes.pop("e2e_path", None)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_max / args.steps, "higher_is_better": True,
        "scaling": "strong" if spec["shard"] else "weak", "vs_baseline": None, "dtype": ("f32 (TF32 hi.hi + BF16 cross terms per K step, fp32 accumulate)" if scheme_mixed
                                                                                       else "f32 (3xTF32 split, fp32 accumulate)"),
        "data": "synthetic",
        "config": {"workload": spec["desc"], "sharding": spec["shard"] or "replicas",
                   "l2": ("L2 flushed between steps" + ("; a spin kernel queued ahead of the start event keeps the host's "
                                                         "launch path out of the device time" if lead_in else ""))
                   if small else "operands larger than L2 (no flush)",
                   "accumulation_chunk_k": int(lib.kai_get_option(b"tc_kc")) or "auto (<=128)",
                   **notes,
                   **({"options": args.option} if args.option else {})},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
        "cpu_baseline": cpu_baseline, "parity": parity,
    }
    if pure is not None and pure_rel_fro is not None:
        pure["rel_fro_vs_fp64"] = pure_rel_fro
    for key, val in ((other_name, other_path), ("pure_3xtf32", pure), ("sustained", sustained), ("alt_partition", alt_partition),
                     ("other_configs", other_configs), ("replay", replay)):
        if val is not None:
            line[key] = val
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel per launch, from the ncu captures
# summarised under profiles/ (None until one exists for the workload).
TRAFFIC_BYTES: dict = {
    # gemm_3xtf32_pair_kernel: 700.0 MB per launch measured at 4096^3 and 2147.7 MB at 6144^3 (traffic ~ n^2.77);
    # 8192^3 extrapolated with that exponent: 700.0 MB x 2^2.77 (too large to capture under ncu's size rule)
    "gemm8192": 700.0e6 * 2 ** 2.77,
    "gemm_nt:4096x4096x4096": 700.0e6,
    "gemm_nt:6144x6144x6144": 2147.7e6,
    # skinny kernels, L2 flushed before the launch: W is read once
    "skinny1": 67.15e6 + 0.2e3, "skinny2": 67.2e6, "skinny4": 67.3e6, "skinny8": 67.3e6, "skinny16": 67.39e6 + 0.7e3,
    # whole steps (all kernels of one step), captured at 16 batch items and scaled x2 (traffic grows with the batch)
    "attention": 2 * (67.3e6 + 76.7e6 + 134.2e6 + 74.5e6 + 169.3e6 + 6.7e6),
    "attention_fused": 2 * (100.7e6 + 3.7e6 + 33.6e6 + 0.2e6 + 16.8e6),
}

if __name__ == "__main__":
    main()
