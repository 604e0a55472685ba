"""CPU oracle for the Fusilli graph path: a graph interpreter over the C kernels
of ``fusilli_oracle.c``. TEST INFRASTRUCTURE ONLY -- imported by tests/,
__graft_entry__.smoke() and bench.py's cpu_baseline / reference arm as the
checker and the timed CPU baseline; nothing in the ``fusilli_b200`` package
imports it and the product path fails loudly without its CUDA library.

It walks the same validated graph object the CUDA path is compiled from
(``fusilli_b200.graph.GraphBase``): every node's inputs are viewed in logical
order through their strides (the physical->logical permute of
include/fusilli/support/asm_emitter.h:174-237), converted to float32 / int64,
handed to the C restatement, and the result is rounded to the tensor's declared
dtype -- including virtual tensors, which is where the reference rounds between
fused ops.

Parity status: pinned against the reference's closed-form samples and against
PyTorch-CPU golden vectors (tests/golden); seeded-random bf16 results at the
benchmark shapes are unpinned by the reference itself ("parity unpinned").
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Dict, Optional

import numpy as np

from fusilli_b200.graph import (DTYPE_SIZE, DataType, GraphBase, Node, NormFwdPhase, Op,
                                PointwiseMode, ReductionMode, TensorAttr)

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfusilli_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compiles fusilli_oracle.c with gcc (see oracle/Makefile)."""
    src = os.path.join(_HERE, "fusilli_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libfusilli_oracle.so"])
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def set_threads(n: int) -> int:
    """OpenMP threads of the C kernels (overrides an inherited OMP_NUM_THREADS); returns the count."""
    f = lib().orc_set_threads
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_int]
    return int(f(int(n)))


# ---- dtype helpers -----------------------------------------------------------
NP_DTYPE = {
    DataType.Half: np.float16, DataType.BFloat16: np.uint16, DataType.Float: np.float32,
    DataType.Double: np.float64, DataType.Uint8: np.uint8, DataType.Int8: np.int8,
    DataType.Int16: np.int16, DataType.Int32: np.int32, DataType.Int64: np.int64,
    DataType.Boolean: np.uint8,
    DataType.Int4: np.uint8,  # packed: element 2k in the low half of byte k (int_types.h:56-66)
}
_FLOAT_TYPES = (DataType.Half, DataType.BFloat16, DataType.Float, DataType.Double)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit pattern (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    nan = np.isnan(a)
    r = ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)
    r[nan] = 0x7FC0
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def pack_int4(values: np.ndarray) -> np.ndarray:
    """Signed 4-bit elements (clamped to [-8, 7]) -> packed bytes, element 2k in the low half of
    byte k (reference include/fusilli/support/int_types.h:32-66)."""
    v = np.clip(np.asarray(values).astype(np.int64).reshape(-1), -8, 7).astype(np.uint8) & 0x0F
    if v.size % 2:
        v = np.concatenate([v, np.zeros(1, np.uint8)])
    return (v[0::2] | (v[1::2] << 4)).astype(np.uint8)


def unpack_int4(raw: np.ndarray, count: int) -> np.ndarray:
    """Packed bytes -> int8 values with sign extension from bit 3 (int_types.h:37-41, 69-78)."""
    b = np.asarray(raw, dtype=np.uint8).reshape(-1)
    nib = np.empty(b.size * 2, np.uint8)
    nib[0::2] = b & 0x0F
    nib[1::2] = b >> 4
    v = nib[:count].astype(np.int8)
    return np.where(v >= 8, v - 16, v).astype(np.int8)


def to_storage(values: np.ndarray, dtype: DataType) -> np.ndarray:
    """Rounds a float / int array to ``dtype``'s storage representation."""
    if dtype == DataType.BFloat16:
        return f32_to_bf16_bits(values.astype(np.float32))
    if dtype == DataType.Boolean:
        return (values != 0).astype(np.uint8)
    if dtype == DataType.Int4:
        return pack_int4(values)
    return values.astype(NP_DTYPE[dtype])


def from_storage(raw: np.ndarray, dtype: DataType) -> np.ndarray:
    """Storage array -> float32 (floating types) or int64 (integral / bool)."""
    if dtype == DataType.BFloat16:
        return bf16_bits_to_f32(raw)
    if dtype in _FLOAT_TYPES:
        return raw.astype(np.float32)
    return raw.astype(np.int64)


def logical_view(flat: np.ndarray, t: TensorAttr) -> np.ndarray:
    item = flat.dtype.itemsize
    return np.lib.stride_tricks.as_strided(flat, shape=t.dim, strides=[s * item for s in t.stride])


def _p(a: Optional[np.ndarray], ct):
    return None if a is None else a.ctypes.data_as(ctypes.POINTER(ct))


def _i64(vals):
    return (ctypes.c_int64 * len(vals))(*[int(v) for v in vals])


def _f32c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


_PF = ctypes.c_float
_PI = ctypes.c_int64


# ---- op wrappers (logical, contiguous float32/int64 in and out) ------------------
def _pad5(dims, ns):
    return list(dims[:2]) + [1] * (3 - ns) + list(dims[2:])


def _pad3(v, ns, fill):
    return [fill] * (3 - ns) + list(v)


def conv(kind: str, a: np.ndarray, b: np.ndarray, xdim, wdim, ydim, pad, stride, dil) -> np.ndarray:
    """kind: fprop (a=x,b=w -> y), dgrad (a=dy,b=w -> dx), wgrad (a=dy,b=x -> dw)."""
    ns = len(xdim) - 2
    xd, wd, yd = _i64(_pad5(xdim, ns)), _i64(_pad5(wdim, ns)), _i64(_pad5(ydim, ns))
    p, s, d = _i64(_pad3(pad, ns, 0)), _i64(_pad3(stride, ns, 1)), _i64(_pad3(dil, ns, 1))
    a, b = _f32c(a), _f32c(b)
    out_dim = {"fprop": ydim, "dgrad": xdim, "wgrad": wdim}[kind]
    out = np.empty(out_dim, dtype=np.float32)
    fn = getattr(lib(), "orc_conv_" + kind)
    fn(_p(a, _PF), _p(b, _PF), _p(out, _PF), xd, wd, yd, p, s, d)
    return out


def matmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a, b = _f32c(a), _f32c(b)
    M, K = a.shape[-2:]
    N = b.shape[-1]
    bdims = [max(x, y) for x, y in zip(a.shape[:-2], b.shape[:-2])]
    nb = int(np.prod(bdims)) if bdims else 1
    a_off, b_off = [], []
    for lin in range(nb):
        idx = np.unravel_index(lin, bdims) if bdims else ()
        ai = [i % d for i, d in zip(idx, a.shape[:-2])]
        bi = [i % d for i, d in zip(idx, b.shape[:-2])]
        a_off.append((int(np.ravel_multi_index(ai, a.shape[:-2])) if bdims else 0) * M * K)
        b_off.append((int(np.ravel_multi_index(bi, b.shape[:-2])) if bdims else 0) * K * N)
    out = np.empty(bdims + [M, N], dtype=np.float32)
    lib().orc_matmul(_p(a, _PF), _p(b, _PF), _p(out, _PF), ctypes.c_int64(nb), _i64(a_off),
                     _i64(b_off), ctypes.c_int64(M), ctypes.c_int64(N), ctypes.c_int64(K))
    return out


def sdpa(q, k, v, mask, causal: bool, scale: Optional[float]) -> np.ndarray:
    q, k, v = _f32c(q), _f32c(k), _f32c(v)
    B, Hq, Sq, D = q.shape
    _, Hk, Skv, _ = k.shape
    _, Hv, _, Dv = v.shape
    if scale is None:
        scale = 1.0 / np.sqrt(np.float32(D))
    m = _f32c(mask) if mask is not None else None
    md = _i64(m.shape) if m is not None else None
    out = np.empty((B, Hq, Sq, Dv), dtype=np.float32)
    lib().orc_sdpa(_p(q, _PF), _p(k, _PF), _p(v, _PF), _p(m, _PF), md, _p(out, _PF),
                   *[ctypes.c_int64(x) for x in (B, Hq, Hk, Hv, Sq, Skv, D, Dv)],
                   ctypes.c_int32(1 if causal else 0), ctypes.c_double(float(scale)))
    return out


def layernorm(x, scale, bias, eps: float, training: bool):
    x = _f32c(x)
    B = x.shape[0]
    R = x.size // B
    s = _f32c(scale).reshape(-1) if scale is not None else None
    b = _f32c(bias).reshape(-1) if bias is not None else None
    y = np.empty_like(x)
    mean = np.empty(B, np.float32) if training else None
    rstd = np.empty(B, np.float32) if training else None
    lib().orc_layernorm(_p(x, _PF), _p(s, _PF), _p(b, _PF), ctypes.c_double(eps), _p(y, _PF),
                        _p(mean, _PF), _p(rstd, _PF), ctypes.c_int64(B), ctypes.c_int64(R))
    return y, mean, rstd


def rmsnorm(x, scale, eps: float):
    x = _f32c(x)
    B = x.shape[0]
    R = x.size // B
    s = _f32c(scale).reshape(-1) if scale is not None else None
    y = np.empty_like(x)
    lib().orc_rmsnorm(_p(x, _PF), _p(s, _PF), ctypes.c_double(eps), _p(y, _PF),
                      ctypes.c_int64(B), ctypes.c_int64(R))
    return y


def reduction(mode: int, x: np.ndarray, ydim, integral: bool) -> np.ndarray:
    xd, yd = _i64(x.shape), _i64(ydim)
    if integral:
        xi = np.ascontiguousarray(x, dtype=np.int64)
        out = np.empty(ydim, np.int64)
        lib().orc_reduce_i(ctypes.c_int32(mode), _p(xi, _PI), _p(out, _PI), ctypes.c_int32(x.ndim), xd, yd)
        return out
    xf = _f32c(x)
    out = np.empty(ydim, np.float32)
    trailing = list(ydim) == list(x.shape[:-1]) + [1]
    if mode in (ReductionMode.ADD, ReductionMode.SUM) and trailing:
        rows = xf.size // xf.shape[-1]
        lib().orc_rowsum_f(_p(xf, _PF), _p(out, _PF), ctypes.c_int64(rows), ctypes.c_int64(xf.shape[-1]))
    else:
        lib().orc_reduce_f(ctypes.c_int32(mode), _p(xf, _PF), _p(out, _PF), ctypes.c_int32(x.ndim), xd, yd)
    return out


def pointwise(mode: int, ins, out_shape, integral: bool, prm) -> np.ndarray:
    n = int(np.prod(out_shape))
    if integral:
        arrs = [np.ascontiguousarray(np.broadcast_to(a, out_shape), dtype=np.int64) if a is not None else None
                for a in ins]
        out = np.empty(out_shape, np.int64)
        rc = lib().orc_pointwise_i(ctypes.c_int32(mode), ctypes.c_int64(n), _p(arrs[0], _PI),
                                   _p(arrs[1], _PI), _p(arrs[2], _PI), _p(out, _PI))
        if rc != 0:
            raise ValueError(f"pointwise mode {mode} has no integer form")
        return out
    arrs = [_f32c(np.broadcast_to(a, out_shape)) if a is not None else None for a in ins]
    out = np.empty(out_shape, np.float32)
    lib().orc_pointwise_f(ctypes.c_int32(mode), ctypes.c_int64(n), _p(arrs[0], _PF), _p(arrs[1], _PF),
                          _p(arrs[2], _PF), _p(out, _PF), (ctypes.c_double * 4)(*prm))
    return out


def batchnorm(x, scale, bias, mean, var, eps: float, training: bool):
    """torch.aten.native_batch_norm on value tensors, the op the reference emits
    (include/fusilli/support/asm_emitter.h:1283-1284): per-channel statistics over every dim but 1.
    Training uses the batch's mean and biased variance and returns them as (mean, 1/sqrt(var+eps));
    inference uses the given running mean / var. No running statistics are returned, so momentum
    has no effect. float64 accumulation."""
    xd = np.asarray(x, dtype=np.float64)
    c = xd.shape[1]
    axes = tuple(i for i in range(xd.ndim) if i != 1)
    shape = [1, c] + [1] * (xd.ndim - 2)
    if training:
        m = xd.mean(axis=axes)
        v = xd.var(axis=axes)  # biased
    else:
        m = np.asarray(mean, dtype=np.float64).reshape(c)
        v = np.asarray(var, dtype=np.float64).reshape(c)
    inv = 1.0 / np.sqrt(v + eps)
    y = (xd - m.reshape(shape)) * inv.reshape(shape)
    if scale is not None:
        y = y * np.asarray(scale, dtype=np.float64).reshape(shape)
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64).reshape(shape)
    return y.astype(np.float32), m.astype(np.float32), inv.astype(np.float32)


# ---- graph interpreter -----------------------------------------------------------
def execute(graph: GraphBase, inputs: Dict[TensorAttr, np.ndarray]) -> Dict[TensorAttr, np.ndarray]:
    """Runs a validated graph. ``inputs`` maps each non-scalar graph input to its
    flat storage array (physical order, storage dtype). Returns flat storage
    arrays, physical order, for every non-virtual output."""
    vals: Dict[int, np.ndarray] = {}  # id(TensorAttr) -> logical float32/int64 array

    def get(t: Optional[TensorAttr]):
        if t is None:
            return None
        if id(t) in vals:
            return vals[id(t)]
        if t.isScalar():
            v = t.getScalarValue()
            arr = np.array([v], dtype=np.float32 if t.dataType in _FLOAT_TYPES else np.int64)
        else:
            flat = np.ascontiguousarray(inputs[t]).reshape(-1)
            if t.dataType == DataType.Int4:
                # only ever a matmul operand: unpack, then compute in float (values are exact)
                arr = logical_view(unpack_int4(flat, t.physicalVolume()), t).astype(np.float32)
            else:
                arr = from_storage(logical_view(flat, t), t.dataType)
        vals[id(t)] = arr
        return arr

    def put(t: TensorAttr, arr: np.ndarray):
        # round to the declared dtype right here, virtual or not
        vals[id(t)] = from_storage(to_storage(arr, t.dataType), t.dataType).reshape(t.dim)

    for n in graph.nodes:
        a = n.attr
        if n.op in (Op.CONV_FPROP, Op.CONV_DGRAD, Op.CONV_WGRAD):
            t0, t1 = n.inputs[:2]
            o = n.outputs[0]
            if n.op == Op.CONV_FPROP:
                xd, wd, yd, kind = t0.dim, t1.dim, o.dim, "fprop"
            elif n.op == Op.CONV_DGRAD:
                xd, wd, yd, kind = o.dim, t1.dim, t0.dim, "dgrad"
            else:
                xd, wd, yd, kind = t1.dim, o.dim, t0.dim, "wgrad"
            put(o, conv(kind, get(t0), get(t1), xd, wd, yd, a.padding, a.stride, a.dilation))
        elif n.op == Op.MATMUL:
            put(n.outputs[0], matmul(get(n.inputs[0]), get(n.inputs[1])))
        elif n.op == Op.SDPA:
            q, k, v, m = n.inputs
            put(n.outputs[0], sdpa(get(q), get(k), get(v), get(m), a.isCausal, a.scale))
        elif n.op == Op.LAYERNORM:
            x, s, b, e = n.inputs
            tr = a.forwardPhase == NormFwdPhase.TRAINING
            y, mean, rstd = layernorm(get(x), get(s), get(b), float(e.getScalarValue()), tr)
            put(n.outputs[0], y)
            if tr:
                put(n.outputs[1], mean)
                put(n.outputs[2], rstd)
        elif n.op == Op.BATCHNORM:
            x, sc, bi, mean, var, e, _momentum = n.inputs
            tr = a.forwardPhase == NormFwdPhase.TRAINING
            y, sm, si = batchnorm(get(x), get(sc), get(bi), get(mean), get(var), float(e.getScalarValue()), tr)
            put(n.outputs[0], y)
            if tr:
                put(n.outputs[1], sm)
                put(n.outputs[2], si)
        elif n.op == Op.RMSNORM:
            x, s, e = n.inputs
            put(n.outputs[0], rmsnorm(get(x), get(s), float(e.getScalarValue())))
        elif n.op == Op.REDUCTION:
            x = n.inputs[0]
            integral = x.dataType not in _FLOAT_TYPES
            put(n.outputs[0], reduction(int(a.mode), get(x), n.outputs[0].dim, integral))
        elif n.op == Op.POINTWISE:
            ins = [get(t) for t in n.inputs]
            integral = all(t is None or t.dataType not in _FLOAT_TYPES for t in n.inputs)
            prm = (a.eluAlpha, a.softplusBeta, a.softplusThreshold, a.swishBeta)
            put(n.outputs[0], pointwise(int(a.mode), ins, n.outputs[0].dim, integral, prm))
        else:
            raise NotImplementedError(n.op)

    results: Dict[TensorAttr, np.ndarray] = {}
    for t in graph.outputs:
        if t.isVirtual():
            continue
        flat = np.zeros(t.physicalVolume(), dtype=NP_DTYPE[t.dataType])
        logical_view(flat, t)[...] = to_storage(vals[id(t)], t.dataType)
        results[t] = flat
    return results
