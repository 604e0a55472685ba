#!/usr/bin/env python
"""Benchmark of the hot path on B200.

Headline workload: BASELINE config 2 -- batched bf16 matmul 8 x 4096^3 with a fused bias add,
through Graph.compile()/execute() of the CUDA backend. At N > 1 every configuration is sharded over
its outermost extent (matrices, images, batch, rows), one process per GPU; the only data-path
exchange is the cross-rank sum of the convolution weight gradients, which is inside config 4's
timed step. The whole job is the same at every N (strong scaling).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-side]
  python bench.py --op conv_fprop --n 64 --c 64 --hw 56 --kout 64 --r 3 --iters 2   # one operator

Prints ONE JSON line on rank 0. `value` is whole-job TFLOP/s with inputs resident in HBM; `e2e` is
the same metric through the public API with pinned HOST buffers (host->device copies of A, B, bias
and the device->host read of C inside the timed region); `roofline` is the dominant kernel against
the measured bf16 peak; `cpu_baseline` is the CPU oracle timed on a bounded sample of the same
workload, whose results also check the GPU outputs that were just timed; `all_configs` carries the
other BASELINE configs measured the same way, `checks` what was compared with the oracle.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

B_TOTAL, M, N, K = 8, 4096, 4096, 4096
L2_BYTES = 126 * 1024 * 1024
METRIC = "batched matmul bf16 8x4096^3 + bias throughput"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], tf_burst=p["bf16_tflops"], tf_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


def c2_sets(b_local: int):
    """Rotating input sets so that consecutive steps never find their operands in L2."""
    set_bytes = b_local * (M * K + K * N + M * N) * 2
    nsets = 1 if set_bytes > 2 * L2_BYTES else int(np.ceil(2.5 * L2_BYTES / set_bytes))
    return nsets, set_bytes


def config_dict(world: int) -> dict:
    """The workload description; identical for both arms at a given N."""
    b_local = B_TOTAL // world
    nsets, set_bytes = c2_sets(b_local)
    return {"workload": "C2 batched matmul bf16 B=8 M=N=K=4096 row-major, fp32 accumulate, fused bias add, bf16 out",
            "batch_per_gpu": b_local, "l2": f"{nsets} rotating input set(s), {set_bytes * nsets >> 20} MiB > L2",
            "parallelism": f"batch sharded over {world} GPU(s), no data-path collective"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---- CPU legs -----------------------------------------------------------------------------
def cpu_matmul_sample(a_rows: np.ndarray, b: np.ndarray, threads: int | None = None):
    """Oracle (CPU restatement) on `a_rows` [r, K] x `b` [K, N], float32 views of bf16 data.
    Returns (float32 result, TFLOP/s, seconds)."""
    from oracle import fusilli_oracle as orc
    # every host core, also under a launcher that exports OMP_NUM_THREADS=1 to its ranks
    orc.set_threads(threads or os.cpu_count() or 1)
    orc.matmul(a_rows[:8], b)  # load the library, warm caches
    t0 = time.perf_counter()
    c = orc.matmul(a_rows, b)
    dt = time.perf_counter() - t0
    return c, 2.0 * a_rows.shape[0] * b.shape[1] * b.shape[0] / dt / 1e12, dt


def cpu_torch_bmm():
    """A second CPU figure beside the oracle port: PyTorch's own bf16 matmul of ONE full 4096^3
    product on the host cores (what a tuned CPU library reaches; not the reference's code)."""
    import torch
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0x5EED + 1)
    a = (torch.randn(M, K, generator=g) * 0.02).to(torch.bfloat16)
    b = (torch.randn(K, N, generator=g) * 0.02).to(torch.bfloat16)
    torch.matmul(a[:256], b)
    t0 = time.perf_counter()
    torch.matmul(a, b)
    dt = time.perf_counter() - t0
    return {"value": 2.0 * M * N * K / dt / 1e12, "unit": "TFLOP/s", "cores": threads,
            "kind": "library (torch CPU bf16 matmul, not the reference)", "sample": f"one full 4096^3 product ({dt:.2f} s)"}


def host_seeded_c2(rows: int):
    """Host copy of config 2's distribution for the reference arm: `rows` rows of A and one B."""
    from fusilli_b200 import workloads as wl
    from oracle import fusilli_oracle as orc
    a = orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(wl.seeded_values(1, 0, rows * K, ("normal", 0.0, 0.02)))).reshape(rows, K)
    b = orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(wl.seeded_values(1, 1, K * N, ("normal", 0.0, 0.02)))).reshape(K, N)
    return a, b


def run_reference(args):
    """Reference arm: the CPU statement of the path on the host cores (the reference's own CPU
    backend needs the IREE compiler/runtime, which are not on this machine). Each step is a
    bounded sample of the workload: 1024 rows of one 4096^3 product."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    rows = 1024
    a, b = host_seeded_c2(rows)
    for _ in range(args.warmup):
        cpu_matmul_sample(a[:32], b)
    vals, times = [], []
    for _ in range(args.steps):
        _, v, dt = cpu_matmul_sample(a, b)
        vals.append(v)
        times.append(dt)
    v = float(np.mean(vals))
    sample = (f"{rows} rows of one 4096^3 product per step (the whole job is 8 x 4096 rows), CPU oracle, "
              "double accumulation, OpenMP")
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean(times)) * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_dict(max(1, args.gpus)),
        "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "cpu_baseline_torch": cpu_torch_bmm(),
        "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "each step is a row sample of the workload, not the whole 8 x 4096^3 job; throughput per step is "
                "what the whole job would reach at the same rate",
    }
    print(json.dumps(line))


# ---- GPU side -------------------------------------------------------------------------------
class Env:
    """What every configuration needs: torch, the front end, this rank's handle and its shard."""

    def __init__(self, torch, fz, wl, handle, rank, world, comm, pk):
        self.torch, self.fz, self.wl, self.handle = torch, fz, wl, handle
        self.rank, self.world, self.comm, self.pk = rank, world, comm, pk
        # L2 flush = READING a buffer four times the size of L2: a written buffer would leave L2 full
        # of dirty lines whose write-back lands inside the next (timed) kernel
        # (float32 on purpose: torch sums integers through a 64-bit copy of the whole buffer, a 1 GiB write)
        self.flush_src = torch.zeros(128 * 1024 * 1024, dtype=torch.float32, device="cuda")

    def flush(self):
        self.flush_sink = self.flush_src.sum()

    def seeded(self, config, index, shape, dist, dtype):
        """Tensor number `index` of configuration `config`, the same on every rank."""
        torch = self.torch
        g = torch.Generator(device="cuda").manual_seed(((0x5EED + config) << 8) + index)
        if dist[0] == "normal":
            t = torch.randn(*shape, device="cuda", generator=g) * dist[2] + dist[1]
        else:
            t = torch.rand(*shape, device="cuda", generator=g) * (dist[2] - dist[1]) + dist[1]
        return t.to(dtype)

    def shard(self, total):
        from fusilli_b200.sharding import shard_range
        return shard_range(total, self.rank, self.world)

    def buf(self, t):
        return self.fz.Buffer.importPointer(self.handle, t.data_ptr(), t.numel() * t.element_size())

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        import torch.distributed as dist
        t = self.torch.tensor([v], device="cuda", dtype=self.torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        self.torch.cuda.synchronize()


class Case:
    """One timed unit: graphs executed back to back (+ an optional trailing call)."""

    def __init__(self, env, name, unit, bound, peak, work, nbytes=None, flush=False, steps=10):
        self.env, self.name, self.unit, self.bound, self.peak = env, name, unit, bound, peak
        self.work, self.nbytes, self.flush, self.steps = work, nbytes, flush, steps
        self.items = []   # (graph, pack, workspace buffer)
        self.calls = []   # the same, marshalled for repeated execution (Graph.bind)
        self.after = None  # callable enqueued after the graphs (the weight-gradient exchange)
        self.keep = []
        self.bytes = 0    # device bytes this rank's step touches: decides whether L2 must be flushed

    def add(self, graph, ins, tensors, outs):
        env = self.env
        graph.compile(env.handle)
        wsz = graph.getWorkspaceSize()
        ws = None
        if wsz:
            wst = env.torch.empty(wsz, dtype=env.torch.uint8, device="cuda")
            self.keep.append(wst)
            ws = env.buf(wst)
        pack = {ins[k]: env.buf(tensors[k]) for k in ins}
        for t, tt in outs:
            pack[t] = tt if isinstance(tt, env.fz.Buffer) else env.buf(tt)
        self.keep += list(tensors.values()) + [tt for _, tt in outs]
        self.bytes += sum(b.size() for b in pack.values())
        self.items.append((graph, pack, ws))
        self.calls.append(graph.bind(env.handle, pack, ws))  # fixed buffers: marshalled once
        return self

    def run(self):
        for c in self.calls:
            c.run()
        if self.after:
            self.after()

    def launches(self):
        return sum(g.numLaunches() for g, _, _ in self.items) + (1 if self.after else 0)

    def time(self):
        env, torch = self.env, self.env.torch
        ms = []
        # A 512 MiB read precedes every timed iteration: it leaves L2 cold (and clean) and keeps the GPU
        # busy while the host enqueues the timed launches, so the events bracket device time only.
        flush = True
        for i in range(3 + self.steps):
            if env.world > 1 and self.after:
                env.barrier()  # ranks enter an exchanging step together
            if flush:
                env.flush()  # > L2; also covers the host's enqueue latency of what follows
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            self.run()
            b.record()
            torch.cuda.synchronize()
            if i >= 3:
                ms.append(a.elapsed_time(b))
        t = env.max_over_ranks(float(np.median(ms))) * 1e-3
        err = env.handle.kernelError()
        if err:
            raise SystemExit(f"bench.py: {self.name}: kernel error word {err:#x} (a bounded wait ran out)")
        n = env.world
        ach = self.work / t / (1e12 if self.unit == "TFLOP/s" else 1e9)
        out = {"ms": t * 1e3, "achieved": ach, "unit": self.unit, "bound": self.bound, "peak_per_gpu": self.peak,
               "frac": ach / (self.peak * n), "launches": self.launches(), "n_gpus": n,
               "l2": "flushed by a 512 MiB read before every iteration",
               "workspace_bytes": sum(g.getWorkspaceSize() or 0 for g, _, _ in self.items)}
        if self.nbytes is not None and self.unit == "TFLOP/s":
            # two-sided roofline: the slower of the tensor-core time and the HBM time of the
            # algorithmic bytes (each operand read once, the result written once), per GPU
            t_tensor, t_hbm = self.work / n / (self.peak * 1e12), self.nbytes / n / (env.pk["hbm"] * 1e9)
            out.update({"algorithmic_bytes": self.nbytes, "roofline_ms": max(t_tensor, t_hbm) * 1e3,
                        "roofline_bound": "hbm" if t_hbm > t_tensor else "tensor",
                        "frac_of_roofline": max(t_tensor, t_hbm) / t})
        return out


def nbytes(*ts):
    return float(sum(t.numel() * t.element_size() for t in ts))


def build_side_cases(env, shard=True):
    """Configurations 1, 3, 4, 5 for this rank's shard (or unsharded when shard=False).
    Returns (cases, outputs): outputs[name] = (local output tensor, total leading extent)."""
    torch, wl, pk = env.torch, env.wl, env.pk
    from fusilli_b200.graph import DataType
    bf = torch.bfloat16
    cases, outputs, inputs = [], {}, {}

    def span(total):
        return env.shard(total) if shard else (0, total)
    world = env.world if shard else 1

    # C5: LayerNorm / RMSNorm / row sum on X[32768, 8192] bf16, rows sharded
    R, C = 32768, 8192
    lo, hi = span(R)
    r = hi - lo
    x5 = env.seeded(4, 0, (R, C), ("normal", 0.0, 1.0), bf)[lo:hi]
    gam = env.seeded(4, 1, (C,), ("normal", 1.0, 0.02), torch.float32)
    bet = env.seeded(4, 2, (C,), ("normal", 0.0, 0.02), torch.float32)
    inputs["C5"] = (x5, gam, bet, lo)
    y_ln, y_rms = torch.empty_like(x5), torch.empty_like(x5)
    ysum = torch.empty(r, device="cuda", dtype=bf)
    g, ins, outs = wl.layernorm_infer(r, C)
    cases.append(Case(env, "C5_layernorm_bf16_32768x8192", "GB/s", "hbm", pk["hbm"], 2.0 * R * C * 2)
                 .add(g, ins, {"x": x5, "gamma": gam, "beta": bet}, [(outs[0], y_ln)]))
    outputs["C5_layernorm_bf16_32768x8192"] = (y_ln, R)
    g, ins, o = wl.rmsnorm_infer(r, C)
    cases.append(Case(env, "C5_rmsnorm_bf16_32768x8192", "GB/s", "hbm", pk["hbm"], 2.0 * R * C * 2)
                 .add(g, ins, {"x": x5, "gamma": gam}, [(o, y_rms)]))
    outputs["C5_rmsnorm_bf16_32768x8192"] = (y_rms, R)
    g, ins, o = wl.row_sum(r, C)
    cases.append(Case(env, "C5_rowsum_bf16_32768x8192", "GB/s", "hbm", pk["hbm"], 1.0 * R * C * 2 + R * 2)
                 .add(g, ins, {"x": x5}, [(o, ysum)]))
    outputs["C5_rowsum_bf16_32768x8192"] = (ysum, R)

    # C1: conv fprop fp32 16x56x56x64 -> 64, 3x3, bias + relu (images sharded)
    lo, hi = span(16)
    x1 = env.seeded(0, 0, (16, 56, 56, 64), ("uniform", -1.0, 1.0), torch.float32)[lo:hi]
    w1 = env.seeded(0, 1, (64, 3, 3, 64), ("uniform", -1.0, 1.0), torch.float32)
    b1 = env.seeded(0, 2, (64,), ("uniform", -0.1, 0.1), torch.float32)
    y1 = torch.empty(hi - lo, 56, 56, 64, device="cuda")
    inputs["C1"] = (x1, w1, b1, lo)
    g, ins, o = wl.conv_fprop_bias_relu(hi - lo, 64, 56, 56, 64, 3, 3, 1, DataType.Float)
    nm = "C1_conv_fprop_f32_16x56x56x64_k64_3x3_bias_relu"
    cases.append(Case(env, nm, "TFLOP/s", "fp32 FFMA (CUDA cores; nominal 148 SMs x 128 lanes x 2 x 1.965 GHz, "
                      "fp32 results to rtol 1e-5)", 148 * 128 * 2 * 1.965e-3, 2.0 * 16 * 56 * 56 * 64 * 64 * 9, flush=True)
                 .add(g, ins, {"x": x1, "w": w1, "bias": b1}, [(o, y1)]))
    outputs[nm] = (y1, 16)

    # C3: SDPA fwd bf16 B8 H32 S4096 D128 causal (batch sharded; heads stay together)
    B, H, S, D = 8, 32, 4096, 128
    lo, hi = span(B)
    q = env.seeded(2, 0, (B, H, S, D), ("normal", 0.0, 1.0), bf)[lo:hi]
    k = env.seeded(2, 1, (B, H, S, D), ("normal", 0.0, 1.0), bf)[lo:hi]
    v = env.seeded(2, 2, (B, H, S, D), ("normal", 0.0, 1.0), bf)[lo:hi]
    o3 = torch.empty_like(q)
    inputs["C3"] = (q, k, v, lo)
    g, ins, o = wl.sdpa_fwd(hi - lo, H, S, D)
    nm = "C3_sdpa_bf16_b8_h32_s4096_d128_causal"
    cases.append(Case(env, nm, "TFLOP/s", "tensor", pk["tf_burst"], 4.0 * B * H * D * S * (S + 1) / 2,
                      steps=3 if world == 1 else 5)
                 .add(g, ins, {"q": q, "k": k, "v": v}, [(o, o3)]))
    outputs[nm] = (o3, B)

    # C4: ResNet-50-shaped conv sweep bf16 N=256 (images sharded), fprop + dgrad + wgrad per layer.
    # Across ranks the weight gradients are fp32 partials in the communicator's buffer, summed and
    # rounded once by the fused exchange at the end of the step.
    n_total = 256
    lo, hi = span(n_total)
    n = hi - lo
    exchanging = shard and env.world > 1
    dw_elems = [kk * r_ * r_ * c for c, _, kk, r_, _ in wl.RESNET_LAYERS]
    dw_total = sum(dw_elems)
    step_case = Case(env, "C4_step_15_passes" + ("_and_wgrad_exchange" if exchanging else ""), "TFLOP/s", "tensor",
                     pk["tf_burst"], 0.0, flush=True, steps=5)
    c4 = {"dw": [], "layers": []}
    off = 0
    for li, (c, hw, kk, r_, pad) in enumerate(wl.RESNET_LAYERS):
        xx = env.seeded(3, 3 * li + 0, (n_total, hw, hw, c), ("normal", 0.0, 0.05), bf)[lo:hi]
        ww = env.seeded(3, 3 * li + 1, (kk, r_, r_, c), ("normal", 0.0, 0.05), bf)
        dy = env.seeded(3, 3 * li + 2, (n_total, hw, hw, kk), ("normal", 0.0, 0.01), bf)[lo:hi]
        yy = torch.empty(n, hw, hw, kk, device="cuda", dtype=bf)
        dx = torch.empty_like(xx)
        fl = 2.0 * n_total * hw * hw * c * kk * r_ * r_
        tag = f"C4_{hw}x{hw}_c{c}_k{kk}_{r_}x{r_}"
        scale = n_total / n  # algorithmic bytes of the whole job from this shard's tensors
        g, ins, o = wl.conv_fprop_bias_relu(n, c, hw, hw, kk, r_, r_, pad, DataType.BFloat16, bias=False, relu=False)
        cf = Case(env, tag + "_fprop", "TFLOP/s", "tensor", pk["tf_burst"], fl, flush=True, steps=5,
                  nbytes=(nbytes(xx, yy) * scale + nbytes(ww) * world)).add(g, ins, {"x": xx, "w": ww}, [(o, yy)])
        g, ins, o = wl.conv_dgrad(n, c, hw, hw, kk, r_, r_, pad)
        cd = Case(env, tag + "_dgrad", "TFLOP/s", "tensor", pk["tf_burst"], fl, flush=True, steps=5,
                  nbytes=(nbytes(dy, dx) * scale + nbytes(ww) * world)).add(g, ins, {"dy": dy, "w": ww}, [(o, dx)])
        # across ranks: fp32 partial into the exchange bucket, rounded once after the sum
        g, ins, o = wl.conv_wgrad(n, c, hw, hw, kk, r_, r_, pad, dw_dtype=DataType.Float if exchanging else None)
        if exchanging:
            dwb = env.comm.view(off * 4, dw_elems[li] * 4)
        else:
            dwb = torch.empty(kk, r_, r_, c, device="cuda", dtype=bf)
        cw = Case(env, tag + "_wgrad" + ("_partial" if exchanging else ""), "TFLOP/s", "tensor", pk["tf_burst"], fl,
                  flush=True, steps=5, nbytes=(nbytes(dy, xx) * scale + dw_elems[li] * 2.0 * world))
        cw.add(g, ins, {"dy": dy, "x": xx}, [(o, dwb)])
        cases += [cf, cd, cw]
        outputs[tag + "_fprop"] = (yy, n_total)
        outputs[tag + "_dgrad"] = (dx, n_total)
        c4["layers"].append((xx, ww, dy, lo))
        c4["dw"].append((dwb, off, dw_elems[li]))
        for cc in (cf, cd, cw):
            step_case.items += cc.items
            step_case.calls += cc.calls
            step_case.keep += cc.keep
            step_case.bytes += cc.bytes
        step_case.work += 3 * fl
        off += dw_elems[li]
    if exchanging:
        out_off = (dw_total * 4 + 255) // 256 * 256
        step_case.after = lambda: env.comm.sumFused(0, dw_total, out_off, DataType.BFloat16)
        c4["dw_sum"] = (out_off, dw_total)
        ex = Case(env, "C4_wgrad_exchange_fused_11.2MB_fp32_to_bf16", "GB/s", "nvlink", 770.0,
                  dw_total * 4.0 * (env.world - 1) / env.world + dw_total * 2.0 * (env.world - 1) / env.world, steps=10)
        ex.after = step_case.after
        # library route for comparison: ncclAllReduce in place on a private copy of the bucket, then a cast
        scratch = torch.zeros(dw_total, device="cuda", dtype=torch.float32)
        cast = torch.empty(dw_total, device="cuda", dtype=bf)
        exn = Case(env, "C4_wgrad_exchange_nccl_allreduce_plus_cast", "GB/s", "nvlink", 770.0, ex.work, steps=10)
        exn.after = lambda: env.comm.sumNccl(scratch.data_ptr(), dw_total, cast.data_ptr(), DataType.BFloat16)
        exn.keep += [scratch, cast]
        cases += [ex, exn]
    cases.append(step_case)
    return cases, outputs, inputs, c4


def as_np(t):
    """Device tensor -> host numpy storage array (bf16 as uint16 bit patterns)."""
    import torch
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).reshape(-1)
    return t.numpy().reshape(-1)


def oracle_checks(env, c2, outputs, inputs, c4):
    """The CPU leg of an N = 1 run: the oracle recomputes SAMPLES of what the GPU just produced
    from the same input bytes (the config 2 sample is also what `cpu_baseline` times). Returns
    (cpu_baseline, checks); a sample outside tolerance ends the run."""
    from fusilli_b200 import workloads as wl
    from fusilli_b200.graph import DataType
    from oracle import check as chk
    from oracle import fusilli_oracle as orc
    orc.set_threads(os.cpu_count() or 1)
    BF16 = DataType.BFloat16
    checks = {}

    def record(name, got, want, dtype, graph, sample):
        acc_len, chained = chk.graph_traits(graph)
        r = chk.mismatch(got, want, dtype, acc_len, chained)
        r["sample"] = sample
        checks[name] = r
        if r["bad"]:
            raise SystemExit(f"bench.py: {name}: {r['bad']} of {r['count']} sampled outputs differ from the oracle "
                             f"(max abs err {r['max_abs_err']:.3g}, atol {r.get('atol')}, rtol {r.get('rtol')})")

    # config 2: 256 rows of batch 0 + 16 rows of every other batch
    a, b, bias, c = c2
    rows0 = np.unique(np.concatenate([[0, 1, 127, 128, M - 2, M - 1], np.random.default_rng(1).integers(0, M, 250)]))[:256]
    b0 = orc.bf16_bits_to_f32(as_np(b[0])).reshape(K, N)
    a0 = orc.bf16_bits_to_f32(as_np(a[0][rows0])).reshape(len(rows0), K)
    acc, _, _ = cpu_matmul_sample(a0, b0)
    # the timed CPU baseline: one whole 4096^3 product of the eight (about a second on the host cores)
    a_full = orc.bf16_bits_to_f32(as_np(a[0])).reshape(M, K)
    _, v, dt = cpu_matmul_sample(a_full, b0)
    del a_full
    cpu = {"value": v, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
           "sample": f"one whole 4096^3 product of the eight ({dt:.2f} s), CPU oracle, double accumulation, OpenMP"}
    rb = lambda x: orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(x))  # noqa: E731
    bias_f = orc.bf16_bits_to_f32(as_np(bias))
    want = orc.f32_to_bf16_bits(rb(acc) + bias_f[None, :])
    r = chk.mismatch(as_np(c[0][rows0]), want.reshape(-1), BF16, K, True)  # matmul + bias add: chained
    r["sample"] = f"batch 0, {len(rows0)} rows incl. first/last tile rows"
    checks["C2_batch0"] = r
    rows = np.array([0, 127, 128, 2047, 2048, 4095] + list(np.random.default_rng(2).integers(0, M, 10)))
    gs, ins_s, cs = wl.matmul_bias(B_TOTAL - 1, len(rows), N, K, name="c2_rows")
    got = as_np(c[1:, rows, :])
    want = orc.execute(gs, {ins_s["a"]: as_np(a[1:, rows, :]), ins_s["b"]: as_np(b[1:]), ins_s["bias"]: as_np(bias)})[cs]
    r2 = chk.mismatch(got, want, BF16, K, True)
    r2["sample"] = "batches 1-7, 16 rows each incl. tile edges"
    checks["C2_batches1to7"] = r2
    for nm in ("C2_batch0", "C2_batches1to7"):
        if checks[nm]["bad"]:
            raise SystemExit(f"bench.py: {nm}: sampled outputs differ from the oracle: {checks[nm]}")

    # config 1: complete
    x1, w1, b1, _ = inputs["C1"]
    g, ins, o = wl.conv_fprop_bias_relu(16, 64, 56, 56, 64, 3, 3, 1, DataType.Float)
    want = orc.execute(g, {ins["x"]: as_np(x1), ins["w"]: as_np(w1), ins["bias"]: as_np(b1)})[o]
    record("C1", as_np(outputs["C1_conv_fprop_f32_16x56x56x64_k64_3x3_bias_relu"][0]), want, DataType.Float, g, "all outputs")

    # config 3: (batch, head) pairs (0,0), (3,17), (7,31); first, middle and last 128-query block
    q, k, v, _ = inputs["C3"]
    o3 = outputs["C3_sdpa_bf16_b8_h32_s4096_d128_causal"][0]
    S, D = 4096, 128
    pairs = [(0, 0), (3, 17), (7, 31)]
    rows = np.concatenate([np.arange(0, 128), np.arange(1984, 2112), np.arange(S - 128, S)])
    gs, ins_s, os_ = wl.sdpa_fwd(1, len(pairs), len(rows), D, causal=False, skv=S, mask=True, name="c3_rows")
    mask = np.where(np.arange(S)[None, :] <= rows[:, None], 0.0, -np.inf).astype(np.float32)
    rows_t = env.torch.as_tensor(rows, device="cuda")
    sel = lambda t, take_rows: np.concatenate(  # noqa: E731
        [as_np(t[bb, hh][rows_t] if take_rows else t[bb, hh]) for bb, hh in pairs])
    data = {ins_s["q"]: sel(q, True), ins_s["k"]: sel(k, False), ins_s["v"]: sel(v, False),
            ins_s["mask"]: orc.to_storage(mask.reshape(-1), BF16)}
    want = orc.execute(gs, data)[os_]
    record("C3", sel(o3, True), want, BF16, gs, "3 (batch, head) pairs x 384 query rows against all 4096 keys")

    # config 4: fprop / dgrad on the first and last image, wgrad on 8 output channels over all pixels
    n = 256
    for li, (c_, hw, kk, r_, pad) in enumerate(wl.RESNET_LAYERS):
        xx, ww, dy, _ = c4["layers"][li]
        tag = f"C4_{hw}x{hw}_c{c_}_k{kk}_{r_}x{r_}"
        imgs = [0, n - 1]
        gs, ins_s, ys = wl.conv_fprop_bias_relu(2, c_, hw, hw, kk, r_, r_, pad, BF16, bias=False, relu=False)
        want = orc.execute(gs, {ins_s["x"]: as_np(xx[imgs]), ins_s["w"]: as_np(ww)})[ys]
        record(tag + "_fprop", as_np(outputs[tag + "_fprop"][0][imgs]), want, BF16, gs, "images 0 and 255")
        gs, ins_s, dxs = wl.conv_dgrad(2, c_, hw, hw, kk, r_, r_, pad)
        want = orc.execute(gs, {ins_s["dy"]: as_np(dy[imgs]), ins_s["w"]: as_np(ww)})[dxs]
        record(tag + "_dgrad", as_np(outputs[tag + "_dgrad"][0][imgs]), want, BF16, gs, "images 0 and 255")
        ks = 8
        gs, ins_s, dws = wl.conv_wgrad(n, c_, hw, hw, ks, r_, r_, pad)
        want = orc.execute(gs, {ins_s["dy"]: as_np(dy[..., :ks]), ins_s["x"]: as_np(xx)})[dws]
        dwb = c4["dw"][li][0]
        record(tag + "_wgrad", as_np(dwb[:ks]), want, BF16, gs, "output channels 0-7, all 256 images")

    # config 5: first and last 1024 rows
    x5, gam, bet, _ = inputs["C5"]
    rsel = np.concatenate([np.arange(0, 1024), np.arange(32768 - 1024, 32768)])
    rs_t = env.torch.as_tensor(rsel, device="cuda")
    xs = as_np(x5[rs_t])
    g, ins, outs = wl.layernorm_infer(len(rsel), 8192)
    want = orc.execute(g, {ins["x"]: xs, ins["gamma"]: as_np(gam), ins["beta"]: as_np(bet)})[outs[0]]
    record("C5_layernorm", as_np(outputs["C5_layernorm_bf16_32768x8192"][0][rs_t]), want, BF16, g, "first and last 1024 rows")
    g, ins, o = wl.rmsnorm_infer(len(rsel), 8192)
    want = orc.execute(g, {ins["x"]: xs, ins["gamma"]: as_np(gam)})[o]
    record("C5_rmsnorm", as_np(outputs["C5_rmsnorm_bf16_32768x8192"][0][rs_t]), want, BF16, g, "first and last 1024 rows")
    g, ins, o = wl.row_sum(len(rsel), 8192)
    want = orc.execute(g, {ins["x"]: xs})[o]
    record("C5_rowsum", as_np(outputs["C5_rowsum_bf16_32768x8192"][0][rs_t]), want, BF16, g, "first and last 1024 rows")
    return cpu, checks


def sharded_checks(env, outputs, c4):
    """The N > 1 self-check: every rank's output slab is gathered (ncclAllGather) and rank 0 compares
    the gathered tensor with the unsharded run of the same graph on its own GPU; the exchanged
    weight gradients are compared with the full-batch ones."""
    torch, comm = env.torch, env.comm
    from fusilli_b200.graph import DataType
    res = {}
    gathered = {}
    for name, (t, total) in outputs.items():
        full = torch.empty((total,) + tuple(t.shape[1:]), device="cuda", dtype=t.dtype)
        comm.allGather(t.data_ptr(), full.data_ptr(), t.numel() * t.element_size())
        gathered[name] = full
    off, count = c4["dw_sum"]
    env.barrier()
    comm.sumFused(0, count, off, DataType.BFloat16)  # the buckets still hold the last step's partials
    env.barrier()
    dw_bits = comm.view(off, count * 2).read(env.handle, np.uint16)  # synchronises the stream
    dw_sum = torch.from_numpy(dw_bits.view(np.int16).copy()).view(torch.bfloat16).float()
    if env.rank == 0:
        cases, outs1, _, c41 = build_side_cases(env, shard=False)
        for cs in cases:
            cs.run()
        torch.cuda.synchronize()
        for name, (t, _) in outs1.items():
            same = bool(torch.equal(t, gathered[name]))
            res[name] = {"gathered_equals_unsharded": same}
            if not same:
                d = (t.float() - gathered[name].float()).abs().max().item()
                raise SystemExit(f"bench.py: {name}: gathered output differs from the unsharded run (max abs {d})")
        full = torch.cat([d[0].reshape(-1).float() for d in c41["dw"]]).cpu()
        got = dw_sum
        # fp32 partial sums added in another order, then one bf16 rounding: within one bf16 ulp
        tol = 2.0 ** -7 * full.abs().max().item()
        worst = (full - got).abs().max().item()
        res["C4_wgrad_exchanged_vs_full_batch"] = {"max_abs_diff": worst, "tolerance": tol, "elements": int(count)}
        if not worst <= tol:
            raise SystemExit(f"bench.py: exchanged weight gradients differ from the full-batch ones: {worst} > {tol}")
    env.barrier()
    return res


def run_ours(args):
    import torch
    import torch.distributed as dist

    import fusilli_b200 as fz
    from fusilli_b200 import workloads as wl
    from fusilli_b200.comm import Comm, torch_allgather_bytes

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    assert B_TOTAL % world == 0, "the batch of 8 matrices must divide across the ranks"
    b_local = B_TOTAL // world
    pk = peaks()

    # A dedicated (non-default) torch stream is handed to the backend as its external
    # stream, so the CUDA events below are recorded on the stream the kernels run on.
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    handle = fz.Handle.create(fz.Backend.CUDA, local, stream.cuda_stream)
    assert handle.stream() == stream.cuda_stream
    comm = None
    if world > 1:
        dw_total = sum(kk * r * r * c for c, _, kk, r, _ in wl.RESNET_LAYERS)
        comm = Comm.create(handle, rank, world, dw_total * 4 + dw_total * 2 + 4096, torch_allgather_bytes())
    env = Env(torch, fz, wl, handle, rank, world, comm, pk)

    graph, ins, out_t = wl.matmul_bias(b_local, M, N, K, name=f"bench_c2_b{b_local}")
    graph.compile(handle)
    wsz = graph.getWorkspaceSize()
    ws = None
    if wsz:
        ws_t = torch.empty(wsz, dtype=torch.uint8, device="cuda")
        ws = fz.Buffer.importPointer(handle, ws_t.data_ptr(), wsz)
    launches_per_step = graph.numLaunches()

    nsets, set_bytes = c2_sets(b_local)
    lo, hi = env.shard(B_TOTAL)
    sets, keep = [], []
    for si in range(nsets):
        # set 0 is the seeded configuration itself; further sets only rotate L2 contents
        a = env.seeded(1, 0 + 8 * si, (B_TOTAL, M, K), ("normal", 0.0, 0.02), torch.bfloat16)[lo:hi]
        b = env.seeded(1, 1 + 8 * si, (B_TOTAL, K, N), ("normal", 0.0, 0.02), torch.bfloat16)[lo:hi]
        bias = env.seeded(1, 2 + 8 * si, (N,), ("normal", 0.0, 0.02), torch.bfloat16)
        c = torch.empty(b_local, M, N, device="cuda", dtype=torch.bfloat16)
        keep.append((a, b, bias, c))
        sets.append({ins["a"]: env.buf(a), ins["b"]: env.buf(b), ins["bias"]: env.buf(bias), out_t: env.buf(c)})

    for i in range(args.warmup):
        graph.execute(handle, sets[i % nsets], ws)
    env.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    evs[0].record()
    for i in range(args.steps):
        graph.execute(handle, sets[i % nsets], ws)
        evs[i + 1].record()
    env.barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = env.max_over_ranks(evs[0].elapsed_time(evs[-1]))
    step_ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
    flops_job = 2.0 * B_TOTAL * M * N * K
    value = flops_job * args.steps / (total_ms * 1e-3) / 1e12
    kern_ms = float(np.mean(step_ms))
    achieved = 2.0 * b_local * M * N * K / (kern_ms * 1e-3) / 1e12
    err = handle.kernelError()
    if err:
        raise SystemExit(f"bench.py: kernel error word {err:#x}")
    if nsets > 1:  # leave set 0's result in place for the checks
        graph.execute(handle, sets[0], ws)
        torch.cuda.synchronize()

    # ---- end to end through the public API with pinned host buffers -------------------
    # Every step copies its A, B and bias from pinned host memory (Buffer h2d), executes the
    # plan and reads C back (Buffer d2h). Three host threads, each with its own Handle (own stream),
    # plan and buffers, take alternate steps, the way a serving loop would keep the PCIe link busy
    # in both directions: one step's read-back overlaps the next step's upload and the GEMM.
    lib = fz.runtime.lib()
    n_lanes = 3
    h2d = (b_local * M * K + b_local * K * N + N) * 2
    d2h = b_local * M * N * 2
    lanes = []
    for li in range(n_lanes):
        st_l = torch.cuda.Stream()
        h_l = fz.Handle.create(fz.Backend.CUDA, local, st_l.cuda_stream)
        g_l, ins_l, out_l = wl.matmul_bias(b_local, M, N, K, name=f"bench_c2_e2e{li}_b{b_local}")
        g_l.compile(h_l)
        g_l.getWorkspaceSize()
        dev_t = {"a": torch.empty(b_local, M, K, dtype=torch.bfloat16, device="cuda"),
                 "b": torch.empty(b_local, K, N, dtype=torch.bfloat16, device="cuda"),
                 "bias": torch.empty(N, dtype=torch.bfloat16, device="cuda"),
                 "c": torch.empty(b_local, M, N, dtype=torch.bfloat16, device="cuda")}
        pack_l = {ins_l[k_]: fz.Buffer.importPointer(h_l, dev_t[k_].data_ptr(), dev_t[k_].numel() * 2) for k_ in ("a", "b", "bias")}
        pack_l[out_l] = fz.Buffer.importPointer(h_l, dev_t["c"].data_ptr(), dev_t["c"].numel() * 2)
        host = {"a": torch.empty(b_local, M, K, dtype=torch.bfloat16).pin_memory(),
                "b": torch.empty(b_local, K, N, dtype=torch.bfloat16).pin_memory(),
                "bias": torch.empty(N, dtype=torch.bfloat16).pin_memory(),
                "c": torch.empty(b_local, M, N, dtype=torch.bfloat16).pin_memory()}
        host["a"].copy_(keep[0][0].cpu()); host["b"].copy_(keep[0][1].cpu()); host["bias"].copy_(keep[0][2].cpu())
        lanes.append((st_l, h_l, g_l, ins_l, out_l, dev_t, pack_l, host))

    def e2e_step(lane):
        _, h_l, g_l, ins_l, out_l, _, pack_l, host = lane
        for k_ in ("a", "b", "bias"):
            st = lib.fb_buffer_h2d(h_l._ptr, pack_l[ins_l[k_]]._ptr, host[k_].data_ptr(), host[k_].numel() * 2)
            assert st == 0
        g_l.execute(h_l, pack_l, None)
        st = lib.fb_buffer_d2h(h_l._ptr, pack_l[out_l]._ptr, host["c"].data_ptr(), d2h)
        assert st == 0

    e2e_steps = max(4, min(args.steps, 24))  # enough steps that filling and draining the pipeline is not the figure
    for lane in lanes:
        e2e_step(lane)
    # the pipelined path produces the bytes the device-resident path produced (which the oracle checks)
    assert torch.equal(lanes[0][7]["c"], keep[0][3].cpu()), "end-to-end result differs from the device-resident one"

    def worker(li):
        torch.cuda.set_device(local)
        for i in range(li, e2e_steps, n_lanes):
            e2e_step(lanes[li])

    env.barrier()
    t0 = time.perf_counter()
    threads = [threading.Thread(target=worker, args=(li,)) for li in range(n_lanes)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    env.barrier()
    e2e_s = env.max_over_ranks(time.perf_counter() - t0)
    e2e_value = flops_job * e2e_steps / e2e_s / 1e12
    del lanes

    # ---- output all-gather (reported separately; not part of `value`) ------------------
    allgather_ms = None
    if world > 1:
        c_local = keep[0][3]
        gathered = torch.empty(B_TOTAL, M, N, device="cuda", dtype=torch.bfloat16)
        comm.allGather(c_local.data_ptr(), gathered.data_ptr(), c_local.numel() * 2)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        comm.allGather(c_local.data_ptr(), gathered.data_ptr(), c_local.numel() * 2)
        e1.record()
        torch.cuda.synchronize()
        allgather_ms = env.max_over_ranks(e0.elapsed_time(e1))
        del gathered

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded on the device: one generator per configuration and tensor)",
        "config": config_dict(world),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk["tf_burst"], "unit": "TFLOP/s",
                     "frac": achieved / pk["tf_burst"],
                     # not measured in this run: dram__bytes_read + write of an ncu capture at
                     # 2 x 4096^3 (205.7 MB, profiles/gemm_pair_tcgen05_c2.md), scaled by the matrices
                     # one launch processes
                     "traffic": 205.7e6 * b_local / 2, "traffic_source": "ncu profile of 2 x 4096^3, scaled",
                     "traffic_algorithmic": 3.0 * b_local * M * N * 2,
                     "peak_source": pk["source"],
                     "kernel": "gemm_pair_tcgen05_kernel (CTA pairs, cta_group::2)", "kernel_ms": kern_ms,
                     "frac_of_sustained": achieved / pk["tf_sustained"]},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "pipeline": f"{n_lanes} host threads x (h2d, execute, d2h), one Handle each"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
        "allgather_ms": allgather_ms,
        "plan": json.loads(graph.statistics()),
    }
    if not args.no_side:
        sets_rest = sets[1:]
        del sets_rest
        while len(keep) > 1:
            keep.pop()
        torch.cuda.empty_cache()
        cases, outputs, inputs, c4 = build_side_cases(env)
        line["all_configs"] = {cs.name: cs.time() for cs in cases}
        if world == 1:
            cpu, checks = oracle_checks(env, keep[0], outputs, inputs, c4)
            line["cpu_baseline"] = cpu
            line["cpu_baseline_torch"] = cpu_torch_bmm()
            line["checks"] = checks
        else:
            line["checks"] = sharded_checks(env, outputs, c4)
    elif world == 1:
        from oracle import fusilli_oracle as orc
        a, b, _, _ = keep[0]
        _, v, dt = cpu_matmul_sample(orc.bf16_bits_to_f32(as_np(a[0][:256])).reshape(256, K),
                                     orc.bf16_bits_to_f32(as_np(b[0])).reshape(K, N))
        line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                                "sample": f"256 rows of one 4096^3 product ({dt:.2f} s), CPU oracle, double accumulation, OpenMP"}
    if rank == 0:
        print(json.dumps(line))
    if comm is not None:
        env.barrier()
        comm.close()
    if world > 1:
        dist.destroy_process_group()


# ---- one operator at a chosen size (the small, self-terminating command to put under ncu) ------
def run_op(a):
    import torch

    import fusilli_b200 as fz
    from fusilli_b200 import workloads as wl
    from fusilli_b200.graph import DataType

    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    handle = fz.Handle.create(fz.Backend.CUDA, 0, stream.cuda_stream)
    bf = torch.bfloat16

    def rnd(*shape, scale=1.0, dtype=bf):
        return (torch.randn(*shape, device="cuda") * scale).to(dtype)

    if a.op == "matmul":
        g, ins, out = wl.matmul_bias(a.b, a.m, a.n, a.k, DataType.BFloat16, not a.no_bias, a.trans_b)
        shape_b = (a.b, a.n, a.k) if a.trans_b else (a.b, a.k, a.n)
        tens = {"a": rnd(a.b, a.m, a.k, scale=0.02), "b": rnd(*shape_b, scale=0.02), "bias": rnd(a.n, scale=0.02)}
        if a.no_bias:
            tens.pop("bias")
        outs = [(out, torch.empty(a.b, a.m, a.n, device="cuda", dtype=bf))]
        work, unit = 2.0 * a.b * a.m * a.n * a.k, "TFLOP/s"
    elif a.op.startswith("conv"):
        pad = a.r // 2
        if a.op == "conv_fprop_f32":
            x = torch.rand(a.n, a.hw, a.hw, a.c, device="cuda") * 2 - 1
            w = torch.rand(a.kout, a.r, a.r, a.c, device="cuda") * 2 - 1
            g, ins, out = wl.conv_fprop_bias_relu(a.n, a.c, a.hw, a.hw, a.kout, a.r, a.r, pad, DataType.Float)
            tens = {"x": x, "w": w, "bias": torch.rand(a.kout, device="cuda") * 0.2 - 0.1}
            outs = [(out, torch.empty(a.n, a.hw, a.hw, a.kout, device="cuda"))]
        else:
            x = rnd(a.n, a.hw, a.hw, a.c, scale=0.05)
            w = rnd(a.kout, a.r, a.r, a.c, scale=0.05)
            dy = rnd(a.n, a.hw, a.hw, a.kout, scale=0.01)
            if a.op == "conv_fprop":
                g, ins, out = wl.conv_fprop_bias_relu(a.n, a.c, a.hw, a.hw, a.kout, a.r, a.r, pad, DataType.BFloat16,
                                                      bias=False, relu=False)
                tens, outs = {"x": x, "w": w}, [(out, torch.empty_like(dy))]
            elif a.op == "conv_dgrad":
                g, ins, out = wl.conv_dgrad(a.n, a.c, a.hw, a.hw, a.kout, a.r, a.r, pad)
                tens, outs = {"dy": dy, "w": w}, [(out, torch.empty_like(x))]
            else:
                g, ins, out = wl.conv_wgrad(a.n, a.c, a.hw, a.hw, a.kout, a.r, a.r, pad)
                tens, outs = {"dy": dy, "x": x}, [(out, torch.empty_like(w))]
        work, unit = 2.0 * a.n * a.hw * a.hw * a.c * a.kout * a.r * a.r, "TFLOP/s"
    elif a.op == "sdpa":
        d = 128
        g, ins, out = wl.sdpa_fwd(a.b, a.h, a.s, d, causal=not a.non_causal)
        tens = {k_: rnd(a.b, a.h, a.s, d) for k_ in ("q", "k", "v")}
        outs = [(out, torch.empty(a.b, a.h, a.s, d, device="cuda", dtype=bf))]
        work = 4.0 * a.b * a.h * d * (a.s * (a.s + 1) / 2 if not a.non_causal else a.s * a.s)
        unit = "TFLOP/s"
    elif a.op in ("layernorm", "rmsnorm", "rowsum"):
        x = rnd(a.rows, a.cols)
        gam = torch.ones(a.cols, device="cuda")
        bet = torch.zeros(a.cols, device="cuda")
        if a.op == "layernorm":
            g, ins, o = wl.layernorm_infer(a.rows, a.cols)
            tens, outs = {"x": x, "gamma": gam, "beta": bet}, [(o[0], torch.empty_like(x))]
            work = 2.0 * a.rows * a.cols * 2
        elif a.op == "rmsnorm":
            g, ins, o = wl.rmsnorm_infer(a.rows, a.cols)
            tens, outs = {"x": x, "gamma": gam}, [(o, torch.empty_like(x))]
            work = 2.0 * a.rows * a.cols * 2
        else:
            g, ins, o = wl.row_sum(a.rows, a.cols)
            tens, outs = {"x": x}, [(o, torch.empty(a.rows, device="cuda", dtype=bf))]
            work = 1.0 * a.rows * a.cols * 2
        unit = "GB/s"
    else:  # batchnorm_train / batchnorm_infer
        train = a.op == "batchnorm_train"
        g, ins, o = wl.batchnorm_fwd(a.n, a.c, [a.hw, a.hw], train=train, channels_last=True)
        x = rnd(a.n, a.hw, a.hw, a.c)
        tens = {"x": x, "gamma": torch.ones(a.c, device="cuda"), "beta": torch.zeros(a.c, device="cuda"),
                "mean": torch.zeros(a.c, device="cuda"), "var": torch.ones(a.c, device="cuda")}
        outs = [(o[0], torch.empty_like(x))]
        if train:
            outs += [(o[1], torch.empty(a.c, device="cuda")), (o[2], torch.empty(a.c, device="cuda"))]
        work, unit = (3.0 if train else 2.0) * x.numel() * 2, "GB/s"

    g.compile(handle)
    wsz = g.getWorkspaceSize()
    wst = torch.empty(max(wsz, 1), dtype=torch.uint8, device="cuda")
    ws = fz.Buffer.importPointer(handle, wst.data_ptr(), wst.numel()) if wsz else None
    pack = {ins[k_]: fz.Buffer.importPointer(handle, t.data_ptr(), t.numel() * t.element_size()) for k_, t in tens.items()}
    for t, tt in outs:
        pack[t] = fz.Buffer.importPointer(handle, tt.data_ptr(), tt.numel() * tt.element_size())
    flush = torch.zeros(128 * 1024 * 1024, dtype=torch.float32, device="cuda")  # float: summed without a widened copy
    ms = []
    for i in range(a.warmup + a.iters):
        sink = flush.sum()  # read > L2: no dirty lines left behind  # noqa: F841
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.execute(handle, pack, ws)
        e1.record()
        torch.cuda.synchronize()
        if i >= a.warmup:
            ms.append(e0.elapsed_time(e1))
    err = handle.kernelError()
    t = float(np.median(ms)) * 1e-3
    print(json.dumps({"op": a.op, "ms": t * 1e3, "achieved": work / t / (1e12 if unit == "TFLOP/s" else 1e9),
                      "unit": unit, "launches": g.numLaunches(), "kernel_error": err,
                      "plan": json.loads(g.statistics())}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-side", action="store_true", help="skip the other BASELINE configs")
    ap.add_argument("--op", default=None, help="run ONE operator at a chosen size instead of the benchmark",
                    choices=["matmul", "conv_fprop", "conv_fprop_f32", "conv_dgrad", "conv_wgrad", "sdpa", "layernorm",
                             "rmsnorm", "rowsum", "batchnorm_train", "batchnorm_infer"])
    for name, default in (("b", 1), ("m", 4096), ("n", 4096), ("k", 4096), ("c", 64), ("hw", 56), ("kout", 64),
                          ("r", 3), ("h", 8), ("s", 4096), ("rows", 8192), ("cols", 8192), ("iters", 3)):
        ap.add_argument("--" + name, type=int, default=default)
    ap.add_argument("--no-bias", action="store_true")
    ap.add_argument("--trans-b", action="store_true")
    ap.add_argument("--non-causal", action="store_true")
    args = ap.parse_args()
    if args.op:
        args.warmup = min(args.warmup, 2)
        run_op(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
