"""Runs one hot-path op at a chosen size a few times and prints its CUDA-event time:
the small, self-terminating command to put under `ncu` (one kernel, few launches).

  python -m fusilli_b200.probe matmul --b 1 --m 2048 --n 4096 --k 4096 --iters 3
  python -m fusilli_b200.probe conv_fprop --n 32 --c 64 --hw 56 --kout 64 --r 3 --iters 3
  python -m fusilli_b200.probe sdpa --b 1 --h 8 --s 4096 --iters 2
  python -m fusilli_b200.probe layernorm --rows 8192 --cols 8192 --iters 3
"""
from __future__ import annotations

import argparse
import json

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["matmul", "conv_fprop", "conv_dgrad", "conv_wgrad", "sdpa", "layernorm",
                                   "rmsnorm", "rowsum", "batchnorm_train", "batchnorm_infer"])
    for name, default in (("b", 1), ("m", 4096), ("n", 4096), ("k", 4096), ("c", 64), ("hw", 56), ("kout", 64),
                          ("r", 3), ("h", 8), ("s", 4096), ("rows", 8192), ("cols", 8192), ("iters", 3),
                          ("warmup", 1)):
        ap.add_argument("--" + name, type=int, default=default)
    ap.add_argument("--no-bias", action="store_true")
    ap.add_argument("--trans-b", action="store_true")
    ap.add_argument("--non-causal", action="store_true")
    a = ap.parse_args()

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
        outs = [(out, torch.empty(a.b, a.m, a.n, device="cuda", dtype=bf))]
        work, unit = 2.0 * a.b * a.m * a.n * a.k, "TFLOP/s"
    elif a.op.startswith("conv"):
        pad = a.r // 2
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
        g, ins, out = wl.sdpa_fwd(a.b, a.h, a.s, 128, causal=not a.non_causal)
        tens = {k: rnd(a.b, a.h, a.s, 128) for k in ("q", "k", "v")}
        outs = [(out, torch.empty(a.b, a.h, a.s, 128, device="cuda", dtype=bf))]
        pairs = a.s * (a.s + 1) / 2 if not a.non_causal else a.s * a.s
        work, unit = 4.0 * a.b * a.h * 128 * pairs, "TFLOP/s"
    elif a.op.startswith("batchnorm"):
        # channels-last bf16 [n, c, hw, hw]; algorithmic bytes: training reads x twice and writes y
        train = a.op == "batchnorm_train"
        g, ins, o = wl.batchnorm_fwd(a.n, a.c, [a.hw, a.hw], train=train, channels_last=True)
        x = rnd(a.n, a.hw, a.hw, a.c)
        tens = {"x": x, "gamma": torch.ones(a.c, device="cuda"), "beta": torch.zeros(a.c, device="cuda"),
                "mean": torch.zeros(a.c, device="cuda"), "var": torch.ones(a.c, device="cuda")}
        outs = [(o[0], torch.empty_like(x))]
        if train:
            outs += [(o[1], torch.empty(a.c, device="cuda")), (o[2], torch.empty(a.c, device="cuda"))]
        work, unit = (3.0 if train else 2.0) * x.numel() * 2, "GB/s"
    else:
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
            work = 1.0 * a.rows * a.cols * 2 + a.rows * 2
        unit = "GB/s"

    g.compile(handle)
    wsz = g.getWorkspaceSize()
    wst = torch.empty(max(wsz, 1), dtype=torch.uint8, device="cuda")
    ws = fz.Buffer.importPointer(handle, wst.data_ptr(), wst.numel()) if wsz else None
    pack = {t: fz.Buffer.importPointer(handle, tens[name].data_ptr(), tens[name].numel() * tens[name].element_size())
            for name, t in ins.items()}
    for t, tt in outs:
        pack[t] = fz.Buffer.importPointer(handle, tt.data_ptr(), tt.numel() * tt.element_size())
    for _ in range(a.warmup):
        g.execute(handle, pack, ws)
    torch.cuda.synchronize()
    ms = []
    for _ in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.execute(handle, pack, ws)
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    t = float(np.median(ms))
    err = handle.kernelError()
    print(json.dumps({"op": a.op, "ms": t, "achieved": work / (t * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9),
                      "unit": unit, "kernel_error": err, "plan": json.loads(g.statistics())}))
    if err:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
