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
                         "output blocks (X row-slab x W row-slab) sharded over a 2-D grid of GPUs",
                    flops=2.0 * 8192 ** 3)
    if name.startswith("gemm_nt:"):  # e.g. gemm_nt:4096x4096x4096 -- profiling-sized cases of the same kernel
        m, n, k = (int(v) for v in name.split(":", 1)[1].split("x"))
        return dict(kind="gemm_nt", M=m, N=n, K=k, shard="MN",
                    desc=f"fp32 GEMM Y=X.W^T M={m} N={n} K={k}, U[-1,1); output blocks sharded over a 2-D grid of GPUs",
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
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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
# GPU arm
# ---------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm8192")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="library tuning switch for this run (kai_set_option), e.g. tc_min_flops=0")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    spec = workload_spec(args.workload, world)

    if args.impl == "reference":
        run_reference_arm(args, spec)
        return

    import torch
    import torch.distributed as dist

    pkg = importlib.import_module("deep-learning-framework_b200")
    vm, capi = pkg.vmath, pkg.capi
    lib = pkg.load()
    for opt in args.option:
        name, _, val = opt.partition("=")
        capi.call("kai_set_option", name.encode(), int(val))
    sharding = importlib.import_module("deep-learning-framework_b200.sharding")

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback for the GPU arm")
    torch.cuda.set_device(local_rank)
    dev = local_rank
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- build the step ---------------------------------------------------------------------
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234)  # same values on every rank: replicated operands are identical
    kind = spec["kind"]
    h2d = d2h = 0
    if kind in ("gemm_nt", "gemm_nn", "skinny"):
        M, N, K = spec["M"], spec["N"], spec["K"]
        m0, m1, n0, n1 = sharding.block2d(M, N, world, rank) if spec["shard"] == "MN" else (0, M, 0, N)
        nl = n1 - n0
        if kind == "gemm_nn":
            a = torch.rand((M, K), device="cuda", generator=gen) * 2 - 1
            b = torch.rand((K, N), device="cuda", generator=gen) * 2 - 1
            layout = capi.GEMM_NN
        else:
            a_full = torch.rand((M, K), device="cuda", generator=gen) * 2 - 1
            w_full = torch.rand((N, K), device="cuda", generator=gen) * 2 - 1
            a = a_full[m0:m1].contiguous()
            b = w_full[n0:n1].contiguous()
            del w_full, a_full
            M = m1 - m0                                   # this rank's rows of X and Y
            layout = capi.GEMM_NT
        c = torch.empty((M, nl), device="cuda")
        local_flops = 2.0 * M * nl * K

        def step(stream=None):
            vm.sgemm(dev, layout, c, a, b, M, nl, K, stream=stream)

        host_in = [torch.empty_like(a, device="cpu").pin_memory(), torch.empty_like(b, device="cpu").pin_memory()]
        host_in[0].copy_(a); host_in[1].copy_(b)
        host_out = torch.empty_like(c, device="cpu").pin_memory()
        a2, b2 = torch.empty_like(a), torch.empty_like(b)

        def step_e2e():
            if layout == capi.GEMM_NT:
                # the host-buffer entry point: upload / multiply / download pipelined over row chunks
                vm.matmul_host(dev, host_out, host_in[1], host_in[0], nl, M, K)
                return
            a2.copy_(host_in[0], non_blocking=True)
            b2.copy_(host_in[1], non_blocking=True)
            vm.sgemm(dev, layout, c, a2, b2, M, nl, K)
            host_out.copy_(c, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        h2d = (a.numel() + b.numel()) * 4
        d2h = c.numel() * 4
    elif kind == "linear_step":
        M, N, K = spec["M"], spec["N"], spec["K"]
        t0, t1 = sharding.slab(M, world, rank)
        ml = t1 - t0
        x = torch.randn((ml, K), device="cuda", generator=gen)
        w = torch.randn((N, K), device="cuda", generator=gen) / 64
        dy = torch.randn((ml, N), device="cuda", generator=gen)
        bias = torch.randn(N, device="cuda", generator=gen)
        y = torch.empty((ml, N), device="cuda"); dx = torch.empty((ml, K), device="cuda")
        dw = torch.empty((N, K), device="cuda")
        local_flops = 3 * 2.0 * ml * N * K

        def step():
            # dW first: its all-reduce (the one collective of the path, NCCL over NVLink) then runs on
            # NCCL's stream while this rank computes Y and dX.
            vm.matmul_backward_w(dev, dw, dy, x, N, ml, K)
            work = dist.all_reduce(dw, async_op=True) if world > 1 else None
            vm.linear_forward(dev, y, w, x, bias, N, ml, K)
            vm.matmul_backward_x(dev, dx, dy, w, N, ml, K)
            if work is not None:
                work.wait()

        host_in = [t.cpu().pin_memory() for t in (x, dy)]
        host_out = torch.empty_like(dw, device="cpu").pin_memory()

        def step_e2e():
            x.copy_(host_in[0], non_blocking=True)
            dy.copy_(host_in[1], non_blocking=True)
            step()
            host_out.copy_(dw, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        h2d = (x.numel() + dy.numel()) * 4
        d2h = dw.numel() * 4
    elif kind == "attention":
        nb, T, H, P = spec["nbat"], spec["ntimes"], spec["nhead"], spec["npiece"]
        b0, b1 = sharding.slab(nb, world, rank)
        bl = b1 - b0
        q = torch.randn((bl, T, H * P), device="cuda", generator=gen)
        k = torch.randn((bl, T, H * P), device="cuda", generator=gen)
        v = torch.randn((bl, T, H * P), device="cuda", generator=gen)
        probs = torch.empty((bl, T, T, H), device="cuda")
        out = torch.empty((bl, T, H, P), device="cuda")
        coef = torch.tensor([1.0 / np.sqrt(P)], device="cuda")
        bwd = bool(spec.get("backward"))
        local_flops = (6 if bwd else 2) * 2.0 * bl * H * T * T * P
        if bwd:
            gy = torch.randn((bl, T, H, P), device="cuda", generator=gen)
            gprobs = torch.empty_like(probs)
            gq, gk, gv = (torch.empty_like(q) for _ in range(3))

        fused = bool(spec.get("fused"))

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

        host_in = [t.cpu().pin_memory() for t in (q, k, v)]
        host_out = torch.empty_like(out, device="cpu").pin_memory()

        def step_e2e():
            for d, h in zip((q, k, v), host_in):
                d.copy_(h, non_blocking=True)
            step()
            host_out.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        h2d = 3 * q.numel() * 4
        d2h = out.numel() * 4
    elif kind == "conv":
        n0, n1 = sharding.slab(spec["ndat"], world, rank)
        nl = n1 - n0
        cx, cy, hh, ww, kh, kw = spec["xchn"], spec["ychn"], spec["h"], spec["w"], spec["kh"], spec["kw"]
        x = torch.randn((nl, cx, hh, ww), device="cuda", generator=gen)
        kk = torch.randn((cy, cx, kh, kw), device="cuda", generator=gen) / (cx * kh * kw) ** 0.5
        gy = torch.randn((nl, cy, hh, ww), device="cuda", generator=gen)
        y, gx, gk = torch.empty_like(gy), torch.empty_like(x), torch.empty_like(kk)
        local_flops = spec["flops"] * nl / spec["ndat"]

        def step():
            vm.conv2d(dev, y, x, kk, nl, cy, hh, ww, cx, hh, ww, kh, kw, 1, kh // 2, kw // 2)
            vm.conv2d_backward_x(dev, gx, gy, kk, nl, cx, hh, ww, cy, hh, ww, kh, kw, 1, kh // 2, kw // 2)
            vm.conv2d_backward_k(dev, gk, gy, x, nl, cx, hh, ww, cy, hh, ww, kh, kw, 1, kh // 2, kw // 2)
            if world > 1:
                dist.all_reduce(gk)

        host_in = [t_.cpu().pin_memory() for t_ in (x, gy)]
        host_out = torch.empty_like(gk, device="cpu").pin_memory()

        def step_e2e():
            x.copy_(host_in[0], non_blocking=True)
            gy.copy_(host_in[1], non_blocking=True)
            step()
            host_out.copy_(gk, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        h2d = (x.numel() + gy.numel()) * 4
        d2h = gk.numel() * 4
    elif kind == "rnn":
        T, B, I, R, NG = spec["ntimes"], spec["ndat"], spec["ninp"], spec["nrec"], spec["ngates"]
        G = NG * R
        x = torch.randn((T, B, I), device="cuda", generator=gen)
        wi = torch.randn((G, I), device="cuda", generator=gen) / I ** 0.5
        wr = torch.randn((G, R), device="cuda", generator=gen) / R ** 0.5
        bb = torch.randn((G,), device="cuda", generator=gen)
        aff = torch.zeros((T, B, G), device="cuda")
        rec = torch.zeros((T, B, R), device="cuda")
        local_flops = spec["flops"]

        def step(stream=None, batched=False):
            # api_objects/vtensor.cpp:2456-2495; the cell update is stood in for by tanh of the first gate block
            if batched:
                vm.matmul(dev, aff, wi, x, G, T * B, I, False, stream=stream)
            for t_ in range(T):
                if t_ > 0:
                    vm.matmul(dev, aff[t_], wr, rec[t_ - 1], G, B, R, batched, stream=stream)
                if not batched:
                    vm.matmul(dev, aff[t_], wi, x[t_], G, B, I, True, stream=stream)
                vm.add_bias(dev, aff[t_], aff[t_], bb, B, G, stream=stream)
                vm.activate(dev, rec[t_], aff[t_].view(-1)[: B * R].view(B, R), B, R, 4, None, stream=stream)

        host_x = x.cpu().pin_memory()
        host_out = torch.empty((B, R)).pin_memory()

        def step_e2e():
            x.copy_(host_x, non_blocking=True)
            step()
            host_out.copy_(rec[T - 1], non_blocking=True)
            torch.cuda.current_stream().synchronize()

        h2d = x.numel() * 4
        d2h = B * R * 4
    elif kind == "mlp":
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
        local_flops = spec["flops"]

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

        host_x = t["x"].cpu().pin_memory()
        host_loss = torch.empty(1).pin_memory()

        def step_e2e():
            t["x"].copy_(host_x, non_blocking=True)
            step()
            host_loss.copy_(loss, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        h2d = host_x.numel() * 4
        d2h = 4
    else:
        raise SystemExit(kind)

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
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    capi.call("kai_profile_enable", 1)
    launches0 = lib.kai_launch_count()
    barrier()
    ms = timed_loop(step, args.steps, small)
    barrier()
    launches = lib.kai_launch_count() - launches0
    import ctypes
    prof_ms = (ctypes.c_double * 3)(); prof_n = (ctypes.c_int64 * 3)()
    capi.call("kai_profile_read", prof_ms, prof_n)
    capi.call("kai_profile_enable", 0)
    clocks = sampler.stop() if rank == 0 else None

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
        if kind == "rnn":   # the input products of all timesteps as one GEMM, recorded the same way
            step(batched=True)
            with vm.Replay(dev) as rpb:
                step(stream=rpb.stream, batched=True)
            for _ in range(3):
                rpb.launch()
            replay["us_per_step_batched_input_gemm"] = timed_loop(rpb.launch, args.steps, True) * 1e3 / args.steps
            replay["us_per_step_batched_call_by_call"] = timed_loop(lambda: step(batched=True), args.steps, True) * 1e3 / args.steps
            rpb.close()

    tms = torch.tensor([ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms_max = float(tms.item())
    total_flops = spec["flops"] if spec["shard"] else spec["flops"] * world  # replicas: every rank does it all
    value = total_flops * args.steps / (ms_max * 1e-3) / 1e12

    # ---- end to end through the C ABI with host buffers ------------------------------------------
    e2e = None
    if not args.no_e2e:
        for _ in range(2):
            step_e2e()
        barrier()
        e2e_steps = min(args.steps, 10)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            step_e2e()
        barrier()
        te = torch.tensor([time.perf_counter() - t0], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e = {"value": total_flops * e2e_steps / float(te.item()) / 1e12, "unit": UNIT, "steps": e2e_steps,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "timing": "host clock around steps that each end with the result in pinned host memory"
                         + ("; kai_matmul_host (chunked upload / multiply / download pipeline)"
                            if kind in ("gemm_nt", "skinny") else "")}

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
    if kind == "skinny":
        hbm = peaks.get("hbm_gbs", 6650.0)
        achieved = spec["bytes"] * args.steps / (ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                    "traffic": None, "kernel": "skinny_nt_kernel",
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
                    "algorithmic_flops_per_launch": local_flops,
                    "note": "forward and input gradient: TMA-fed implicit GEMM (operand tiles are boxes of a zero-padded "
                            "channels-last copy; N = 64 MMAs from four issuing warps); the kernel gradient still "
                            "writes the unfolded input (kh*kw times the input) to memory and reads it back"}
    elif prof_n[0] > 0:
        gemm_ms = prof_ms[0] / prof_n[0]
        per_launch_flops = local_flops / (prof_n[0] / args.steps)
        achieved = per_launch_flops / (gemm_ms * 1e-3) / 1e12
        peak = (tf32_peak or 0.0) / 3.0
        roofline = {
            "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak if peak else None, "traffic": TRAFFIC_BYTES.get(args.workload),
            "kernel": "gemm_3xtf32_kernel<256,16>", "launches": int(prof_n[0]), "avg_ms": gemm_ms,
            "peak_source": f"dense TF32 measured in this run (torch.matmul 8192^3, best of 10: {tf32_peak:.1f} TFLOP/s) "
                           "/ 3 tcgen05.mma per product (3xTF32); MEASURED_PEAKS.json carries no TF32 figure "
                           f"(its bf16_tflops/6 = {peaks.get('bf16_tflops', 0) / 6:.1f})",
            "frac_of_nominal": achieved / (NOMINAL_TF32_DENSE / 3.0),
            "algorithmic_flops_per_launch": per_launch_flops,
            "split_kernels_ms_per_step": prof_ms[1] / args.steps,
        }
    elif kind == "attention":
        # Unfused trio in the reference layouts: Q,K read, probs written; probs read + written (softmax in
        # place); probs + V read, out written.  Batch-sharded: this rank's share.
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

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_max / args.steps, "higher_is_better": True,
        "scaling": "strong" if spec["shard"] else "weak", "vs_baseline": None, "dtype": "f32 (3xTF32 split, fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": spec["desc"], "sharding": spec["shard"] or "replicas",
                   "l2": "L2 flushed between steps" if small else "operands larger than L2 (no flush)",
                   "accumulation_chunk_k": int(lib.kai_get_option(b"tc_kc")) or "auto (<=128)",
                   **({"options": args.option} if args.option else {})},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
        "cpu_baseline": cpu_baseline,
    }
    if replay is not None:
        line["replay"] = replay
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of the GEMM kernel per launch, from the ncu capture
# summarised under profiles/ (filled in from that capture; None until one exists for the workload).
TRAFFIC_BYTES: dict = {
    # 630.9 MB read + 66.6 MB written measured for gemm_nt:4096x4096x4096 (latest capture), x8 for 8192^3
    # (tiles x K-blocks both double per dimension) -- see profiles/
    "gemm8192": 8 * 0.6975e9,
    "gemm_nt:4096x4096x4096": 0.6975e9,
    # whole steps (all kernels of one step), captured at 16 batch items and scaled x2 (traffic grows with the batch)
    "attention": 2 * (67.3e6 + 76.7e6 + 134.2e6 + 74.5e6 + 169.3e6 + 6.7e6),
    "attention_fused": 2 * (100.7e6 + 3.7e6 + 33.6e6 + 0.2e6 + 16.8e6),
}

if __name__ == "__main__":
    main()
