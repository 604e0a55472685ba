"""Tolerances of the parity checks and the graph facts they depend on. TEST INFRASTRUCTURE
(like everything under oracle/): used by tests/ and by bench.py's CPU-baseline leg, where the
oracle's sampled results double as the checker of the timed GPU outputs."""
from __future__ import annotations

import math

import numpy as np

from fusilli_b200.graph import DataType

# Tolerances of the north-star contract: integers bit-exact, fp32 paths rtol 1e-5,
# 16-bit paths rtol/atol 2e-2.
TOL = {
    DataType.Float: dict(rtol=1e-5, atol=1e-5),
    DataType.Half: dict(rtol=2e-2, atol=2e-2),
    DataType.BFloat16: dict(rtol=2e-2, atol=2e-2),
}



# Largest spacing of representable values relative to the value: 8 significant bits for
# bfloat16, 11 for half, 24 for float.
ULP_REL = {DataType.BFloat16: 2.0 ** -7, DataType.Half: 2.0 ** -10, DataType.Float: 2.0 ** -23}


def graph_traits(graph) -> tuple:
    """(acc_len, chained) of a validated graph: the longest accumulation any node performs (terms
    summed per output element) and whether a rounded intermediate feeds a later node."""
    from fusilli_b200.graph import Op
    acc = 1
    for n in graph.nodes:
        if n.op == Op.CONV_FPROP:
            w = n.inputs[1]
            acc = max(acc, int(np.prod(w.dim[1:])))
        elif n.op == Op.CONV_DGRAD:
            w = n.inputs[1]
            acc = max(acc, int(w.dim[0] * np.prod(w.dim[2:])))
        elif n.op == Op.CONV_WGRAD:
            dy = n.inputs[0]
            acc = max(acc, int(dy.dim[0] * np.prod(dy.dim[2:])))
        elif n.op == Op.MATMUL:
            acc = max(acc, int(n.inputs[0].dim[-1]))
        elif n.op == Op.SDPA:
            acc = max(acc, int(n.inputs[1].dim[2]))
        elif n.op in (Op.LAYERNORM, Op.RMSNORM):
            acc = max(acc, int(np.prod(n.inputs[0].dim[1:])))
        elif n.op == Op.BATCHNORM:
            x = n.inputs[0]
            acc = max(acc, int(np.prod(x.dim)) // int(x.dim[1]))
        elif n.op == Op.REDUCTION:
            x, y = n.inputs[0], n.outputs[0]
            acc = max(acc, int(np.prod(x.dim)) // max(1, int(np.prod(y.dim))))
    return acc, len(graph.nodes) > 1


def tolerance(dtype: DataType, want: np.ndarray, acc_len: int = 1, chained: bool = False) -> dict:
    """rtol/atol for comparing a result of `dtype` with the oracle's `want` (float64 values).

    rtol is the contract's (2e-2 for 16-bit, 1e-5 for fp32). atol is the contract's too, scaled DOWN
    when the outputs are smaller than 1 (an absolute 2e-2 would accept anything on gradients of
    magnitude 1e-2), and raised only where arithmetic says an absolute error of that size is
    expected from a correct implementation:
      * fp32: the oracle accumulates in float64, the kernels in float32; summing `acc_len` terms in a
        different order moves a result by about sqrt(acc_len) * 2^-24 times the size of the partial
        sums, whatever the size of the result itself. atol = twice that at the largest output.
      * 16-bit graphs with more than one node: an intermediate rounded to 16 bits can land on the
        neighbouring value (float32 vs float64 accumulation under it), i.e. move by one ulp at its
        own magnitude, and a following add can cancel most of it. atol = one 16-bit ulp at the
        largest output magnitude."""
    t = dict(TOL[dtype])
    w = np.abs(want[np.isfinite(want)])
    m = float(w.max()) if w.size else 0.0
    t["atol"] = t["atol"] * min(1.0, m)
    if dtype == DataType.Float:
        t["atol"] = max(t["atol"], 2.0 * math.sqrt(max(1, acc_len)) * 2.0 ** -24 * m)
    elif chained:
        t["atol"] = max(t["atol"], ULP_REL[dtype] * m)
    return t


def mismatch(got: np.ndarray, want: np.ndarray, dtype: DataType, acc_len: int = 1, chained: bool = False) -> dict:
    """Compares storage arrays `got` and `want` of `dtype` under `tolerance`; returns the number of
    elements outside it and the largest absolute error instead of raising."""
    from . import fusilli_oracle as orc
    if dtype not in TOL:
        bad = int(np.count_nonzero(got.reshape(-1) != want.reshape(-1)))
        return {"bad": bad, "count": int(want.size), "max_abs_err": float(bad > 0), "exact": True}
    g = orc.from_storage(got.reshape(-1), dtype).astype(np.float64)
    w = orc.from_storage(want.reshape(-1), dtype).astype(np.float64)
    tol = tolerance(dtype, w, acc_len, chained)
    err = np.abs(g - w)
    ok = (err <= tol["atol"] + tol["rtol"] * np.abs(w)) | (np.isnan(g) & np.isnan(w)) | (g == w)
    return {"bad": int(np.count_nonzero(~ok)), "count": int(w.size),
            "max_abs_err": float(np.nanmax(err)) if err.size else 0.0, "rtol": tol["rtol"], "atol": tol["atol"]}
