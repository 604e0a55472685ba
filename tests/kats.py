"""Closed-form known-answer cases restated from the reference's samples (the only
numeric pins the reference holds for this path). Each case returns
(graph, {tensor: flat input array}, checker(outputs_by_tensor)). The CPU suite
runs them through the oracle; the GPU suite runs them through the CUDA path."""
from __future__ import annotations

import math

import numpy as np

import fusilli_b200 as fz
from fusilli_b200.graph import (DataType, PointwiseMode, ReductionMode, TensorAttr, channelsLastStride,
                                contiguousStride)
from oracle import fusilli_oracle as orc

F32, F16, I32 = DataType.Float, DataType.Half, DataType.Int32


def _fill(t: TensorAttr, value) -> np.ndarray:
    return orc.to_storage(np.full(t.physicalVolume(), value, np.float32), t.dataType)


def _f(arr, t):
    return orc.from_storage(arr, t.dataType)


def conv_fprop_1x1_bias_relu():
    """samples/convolution/conv_fprop_with_relu_and_bias.cpp:25,79-112: ones -> 129 exactly."""
    n, c, h, w, k = 16, 128, 64, 64, 256
    g = fz.Graph()
    g.setName("kat_conv_1x1").setIODataType(F16).setComputeDataType(F32)
    x = g.tensor(TensorAttr().setName("image").setDim([n, c, h, w]).setStride(channelsLastStride([n, c, h, w])))
    wt = g.tensor(TensorAttr().setName("filter").setDim([k, c, 1, 1]).setStride(channelsLastStride([k, c, 1, 1])))
    y = g.convFProp(x, wt, fz.ConvFPropAttr().setStride([1, 1]).setPadding([0, 0]).setDilation([1, 1]).setName("conv_fprop"))
    y.setName("conv_result").setDataType(F16)
    b = g.tensor(TensorAttr().setName("bias").setDim([1, k, 1, 1]).setStride([k, 1, k, k]))
    y = g.pointwise(y, b, fz.PointwiseAttr().setMode(PointwiseMode.ADD))
    y.setName("bias_result").setDataType(F16)
    y = g.pointwise(y, fz.PointwiseAttr().setMode(PointwiseMode.RELU_FWD))
    y.setName("result").setOutput(True)
    g.validate()
    ins = {x: _fill(x, 1.0), wt: _fill(wt, 1.0), b: _fill(b, 1.0)}
    return g, ins, lambda o: np.all(o[y] == np.float16(129.0))


def conv_fprop_3x3_pad():
    """samples/convolution/conv_fprop_nhwc_krsc_with_pad.cpp:24,94: corner = 4 taps x 128."""
    n, c, h, w, k = 4, 128, 16, 16, 32
    g = fz.Graph()
    g.setName("kat_conv_3x3").setIODataType(F16).setComputeDataType(F32)
    x = g.tensor(TensorAttr().setName("image").setDim([n, c, h, w]).setStride(channelsLastStride([n, c, h, w])))
    wt = g.tensor(TensorAttr().setName("filter").setDim([k, c, 3, 3]).setStride(channelsLastStride([k, c, 3, 3])))
    y = g.convFProp(x, wt, fz.ConvFPropAttr().setStride([1, 1]).setPadding([1, 1]).setDilation([1, 1]))
    y.setName("result").setOutput(True)
    g.validate()

    def check(o):
        v = _f(o[y], y).reshape(n, h, w, k)
        return v[0, 0, 0, 0] == 512 and v[0, 0, 1, 0] == 768 and v[0, 5, 5, 3] == 1152

    return g, {x: _fill(x, 1.0), wt: _fill(wt, 1.0)}, check


def conv_fprop_grouped_bias_relu():
    """samples/convolution/conv_fprop_grouped_with_relu_and_bias.cpp: max(fc*r*s + 1, 0)."""
    n, c, h, w, k, groups = 2, 32, 8, 8, 16, 8
    fc = c // groups
    g = fz.Graph()
    g.setName("kat_conv_grouped").setIODataType(F16).setComputeDataType(F32)
    x = g.tensor(TensorAttr().setName("image").setDim([n, c, h, w]).setStride(channelsLastStride([n, c, h, w])))
    wt = g.tensor(TensorAttr().setName("filter").setDim([k, fc, 1, 1]).setStride(channelsLastStride([k, fc, 1, 1])))
    y = g.convFProp(x, wt, fz.ConvFPropAttr().setStride([1, 1]).setPadding([0, 0]).setDilation([1, 1]))
    y.setDataType(F16)
    b = g.tensor(TensorAttr().setName("bias").setDim([1, k, 1, 1]).setStride([k, 1, k, k]))
    y = g.pointwise(y, b, fz.PointwiseAttr().setMode(PointwiseMode.ADD))
    y.setDataType(F16)
    y = g.pointwise(y, fz.PointwiseAttr().setMode(PointwiseMode.RELU_FWD))
    y.setName("result").setOutput(True)
    g.validate()
    return g, {x: _fill(x, 1.0), wt: _fill(wt, 1.0), b: _fill(b, 1.0)}, lambda o: np.all(_f(o[y], y) == fc + 1)


def conv_dgrad_1x1():
    """samples/convolution/conv_dgrad_nhwc_krsc.cpp:98: dx == k."""
    n, c, h, w, k = 4, 16, 8, 8, 32
    g = fz.Graph()
    g.setName("kat_dgrad").setIODataType(F32).setComputeDataType(F32)
    dy = g.tensor(TensorAttr().setName("dy").setDim([n, k, h, w]).setStride(channelsLastStride([n, k, h, w])))
    wt = g.tensor(TensorAttr().setName("w").setDim([k, c, 1, 1]).setStride(channelsLastStride([k, c, 1, 1])))
    dx = g.convDGrad(dy, wt, fz.ConvDGradAttr().setStride([1, 1]).setPadding([0, 0]).setDilation([1, 1]))
    dx.setDim([n, c, h, w]).setName("dx").setOutput(True)
    g.validate()
    return g, {dy: _fill(dy, 1.0), wt: _fill(wt, 1.0)}, lambda o: np.all(o[dx] == k)


def conv_wgrad_grouped_strided():
    """samples/convolution/conv_wgrad_nhwc_krsc_grouped_strided.cpp: dw == n*ho*wo."""
    n, c, h, w, k, groups = 4, 16, 8, 8, 32, 4
    ho = wo = 4
    g = fz.Graph()
    g.setName("kat_wgrad").setIODataType(F32).setComputeDataType(F32)
    dy = g.tensor(TensorAttr().setName("dy").setDim([n, k, ho, wo]).setStride(channelsLastStride([n, k, ho, wo])))
    x = g.tensor(TensorAttr().setName("x").setDim([n, c, h, w]).setStride(channelsLastStride([n, c, h, w])))
    dw = g.convWGrad(dy, x, fz.ConvWGradAttr().setStride([2, 2]).setPadding([0, 0]).setDilation([1, 1]))
    dw.setDim([k, c // groups, 1, 1]).setName("dw").setOutput(True)
    g.validate()
    return g, {dy: _fill(dy, 1.0), x: _fill(x, 1.0)}, lambda o: np.all(o[dw] == n * ho * wo)


def matmul_batched_bias():
    """samples/matmul/matmul_batched_with_bias.cpp:117-120: ones -> k + 2."""
    b, m, n, k = 16, 32, 64, 128
    g = fz.Graph()
    g.setName("kat_matmul").setIODataType(F32).setComputeDataType(F32).setIntermediateDataType(F32)
    a = g.tensor(TensorAttr().setName("a").setDim([b, m, k]).setStride(contiguousStride([b, m, k])))
    bt = g.tensor(TensorAttr().setName("b").setDim([b, k, n]).setStride(contiguousStride([b, k, n])))
    c = g.matmul(a, bt, fz.MatmulAttr())
    bias = g.tensor(TensorAttr().setName("bias").setDim([1, 1, n]).setStride([n, n, 1]))
    c = g.pointwise(c, bias, fz.PointwiseAttr().setMode(PointwiseMode.ADD))
    c.setName("c").setOutput(True)
    g.validate()
    return g, {a: _fill(a, 1.0), bt: _fill(bt, 1.0), bias: _fill(bias, 2.0)}, lambda o: np.all(o[c] == k + 2.0)


def matmul_transposed_b_f16():
    """samples/matmul/matmul_basic.cpp:112-113: B given with transposed strides; ones -> k."""
    m, n, k = 16, 32, 64
    g = fz.Graph()
    g.setName("kat_matmul_tb").setIODataType(F16).setComputeDataType(F32).setIntermediateDataType(F32)
    a = g.tensor(TensorAttr().setName("a").setDim([m, k]).setStride([k, 1]))
    bt = g.tensor(TensorAttr().setName("b").setDim([k, n]).setStride([1, k]))
    c = g.matmul(a, bt, fz.MatmulAttr())
    c.setName("c").setOutput(True)
    g.validate()
    return g, {a: _fill(a, 1.0), bt: _fill(bt, 1.0)}, lambda o: np.all(o[c] == np.float16(k))


def matmul_int4_fp16():
    """samples/matmul/matmul_int4_fp16.cpp:30-98: A si4 ones (packed nibbles), B f16 ones -> k."""
    b, m, k, n = 1, 4, 8, 4
    g = fz.Graph()
    g.setName("kat_matmul_int4").setIODataType(F16).setComputeDataType(F32).setIntermediateDataType(F32)
    a = g.tensor(TensorAttr().setName("a").setDim([b, m, k]).setStride([m * k, k, 1]).setDataType(DataType.Int4))
    bt = g.tensor(TensorAttr().setName("b").setDim([b, k, n]).setStride([k * n, n, 1]))
    c = g.matmul(a, bt, fz.MatmulAttr().setName("matmul"))
    c.setName("c").setOutput(True)
    g.validate()
    ones = orc.pack_int4(np.ones(b * m * k))
    assert ones.size == b * m * k // 2 and np.all(ones == 0x11)
    return g, {a: ones, bt: _fill(bt, 1.0)}, lambda o: np.all(o[c] == np.float16(k))


def batchnorm_infer_nchw_scale_bias():
    """samples/batchnorm/batchnorm_infer_nchw_scale_bias.cpp with batchnorm_utils.h:25-50: x = c + 1,
    running mean 0 and var 1 -> y = scale * x / sqrt(1 + eps) + bias."""
    n, c, h, w, eps, scale, bias = 2, 3, 4, 4, 1e-5, 2.0, 1.0
    g = fz.Graph()
    g.setName("kat_bn_infer").setIODataType(F32).setComputeDataType(F32)
    x = g.tensor(TensorAttr().setName("x").setDim([n, c, h, w]).setStride(contiguousStride([n, c, h, w])))
    ts = {k: g.tensor(TensorAttr().setName(k).setDim([c]).setStride([1])) for k in ("scale", "bias", "mean", "var")}
    attr = fz.BatchnormAttr().setForwardPhase(fz.NormFwdPhase.INFERENCE).setName("batchnorm")
    attr.setEpsilon(g.tensor(TensorAttr(eps).setName("epsilon"))).setMomentum(g.tensor(TensorAttr(0.1).setName("momentum")))
    y, _, _ = g.batchnorm(x, ts["scale"], ts["bias"], ts["mean"], ts["var"], attr)
    y.setName("y").setOutput(True)
    g.validate()
    xv = np.repeat(np.tile(np.arange(1, c + 1, dtype=np.float32), n), h * w)
    want = scale * xv / np.float32(math.sqrt(1.0 + eps)) + bias
    ins = {x: xv, ts["scale"]: _fill(ts["scale"], scale), ts["bias"]: _fill(ts["bias"], bias),
           ts["mean"]: _fill(ts["mean"], 0.0), ts["var"]: _fill(ts["var"], 1.0)}
    return g, ins, lambda o: np.max(np.abs(o[y] - want)) < 1e-4


def batchnorm_train_nchw_two_value():
    """samples/batchnorm/batchnorm_train_nchw.cpp with batchnorm_utils.h:58-91: half of every channel
    is -1 and half +1 -> mean 0, var 1, y = x / sqrt(1 + eps), saved statistics (0, 1/sqrt(1+eps))."""
    n, c, h, w, eps = 2, 3, 4, 4, 1e-5
    g = fz.Graph()
    g.setName("kat_bn_train").setIODataType(F32).setComputeDataType(F32)
    x = g.tensor(TensorAttr().setName("x").setDim([n, c, h, w]).setStride(contiguousStride([n, c, h, w])))
    attr = fz.BatchnormAttr().setForwardPhase(fz.NormFwdPhase.TRAINING).setName("batchnorm")
    attr.setEpsilon(g.tensor(TensorAttr(eps).setName("epsilon"))).setMomentum(g.tensor(TensorAttr(0.1).setName("momentum")))
    y, sm, si = g.batchnorm(x, None, None, None, None, attr)
    y.setName("y").setOutput(True)
    sm.setName("saved_mean").setOutput(True)
    si.setName("saved_inv_var").setOutput(True)
    g.validate()
    xv = np.empty((n, c, h, w), np.float32)
    for ni in range(n):
        for hi in range(h):
            for wi in range(w):
                xv[ni, :, hi, wi] = -1.0 if ni * h * w + hi * w + wi < n * h * w // 2 else 1.0
    inv = np.float32(1.0 / math.sqrt(1.0 + eps))

    def check(o):
        return (np.max(np.abs(o[y] - xv.reshape(-1) * inv)) < 1e-4 and np.max(np.abs(o[sm])) < 1e-4
                and np.max(np.abs(o[si] - inv)) < 1e-4)
    return g, {x: xv.reshape(-1)}, check


def _sdpa_case(name, causal=False, mask=False, hk=8, hv=8, sq=64, skv=64):
    """samples/sdpa/*.cpp against samples/sdpa_utils.cpp:49-102 (constant fills 0.01):
    softmax over equal scores is uniform, so every output element equals the V fill."""
    b, hq, d = 1, 8, 64
    g = fz.Graph()
    g.setName(name).setIODataType(F16).setComputeDataType(F32)
    q = g.tensor(TensorAttr().setName("q").setDim([b, hq, sq, d]).setStride(contiguousStride([b, hq, sq, d])))
    k = g.tensor(TensorAttr().setName("k").setDim([b, hk, skv, d]).setStride(contiguousStride([b, hk, skv, d])))
    v = g.tensor(TensorAttr().setName("v").setDim([b, hv, skv, d]).setStride(contiguousStride([b, hv, skv, d])))
    m = None
    if mask:
        m = g.tensor(TensorAttr().setName("mask").setDim([b, 1, sq, skv]).setStride(contiguousStride([b, 1, sq, skv])))
    o = g.sdpa(q, k, v, m, fz.SdpaAttr().setIsCausal(causal).setEnableGqa(hk != hq or hv != hq))
    o.setName("o").setOutput(True)
    g.validate()
    ins = {q: _fill(q, 0.01), k: _fill(k, 0.01), v: _fill(v, 0.01)}
    if mask:
        ins[m] = _fill(m, 0.5)
    return g, ins, lambda out: np.all(np.abs(_f(out[o], o) - 0.01) < 1e-2) and np.all(np.abs(_f(out[o], o) - 0.01) < 2e-4)


def layernorm_train_two_value(layout="NHWC", affine=True):
    """samples/layernorm/*.cpp + layernorm_utils.h:25-82: two-value rows -> +-scale/sqrt(1+eps)+bias,
    mean = x0+1, inv-variance = 1/sqrt(1+eps); abs tol 1e-4."""
    n, c, h, w = 2, 3, 32, 32
    scale, bias, eps = (2.0, 0.5, 1e-5) if affine else (1.0, 0.0, 1e-5)
    g = fz.Graph()
    g.setName("kat_ln_" + layout).setIODataType(F32).setComputeDataType(F32).setIntermediateDataType(F32)
    sf = contiguousStride if layout == "NCHW" else channelsLastStride
    x = g.tensor(TensorAttr().setName("x").setDim([n, c, h, w]).setStride(sf([n, c, h, w])))
    ins = {}
    st = bt = None
    if affine:
        st = g.tensor(TensorAttr().setName("scale").setDim([1, c, h, w]).setStride(sf([1, c, h, w])))
        bt = g.tensor(TensorAttr().setName("bias").setDim([1, c, h, w]).setStride(sf([1, c, h, w])))
    e = g.tensor(TensorAttr(eps).setName("eps"))
    y, mean, iv = g.layernorm(x, st, bt, fz.LayernormAttr().setForwardPhase(fz.NormFwdPhase.TRAINING).setEpsilon(e))
    for t in (y, mean, iv):
        t.setOutput(True)
    g.validate()
    if affine:
        ins[st] = _fill(st, scale)
        ins[bt] = _fill(bt, bias)
    row = c * h * w
    xin = np.zeros(n * row, np.float32)
    want = np.zeros(n * row, np.float32)
    div = math.sqrt(1.0 + eps)
    for b in range(n):
        xin[b * row: b * row + row // 2] = 2.0 * b
        xin[b * row + row // 2: (b + 1) * row] = 2.0 * b + 2
        want[b * row: b * row + row // 2] = scale * (-1.0 / div) + bias
        want[b * row + row // 2: (b + 1) * row] = scale * (1.0 / div) + bias
    ins[x] = xin

    def check(o):
        return (np.all(np.abs(o[y] - want) < 1e-4) and np.all(np.abs(o[mean] - np.array([1.0, 3.0])) < 1e-4)
                and np.all(np.abs(o[iv] - 1.0 / div) < 1e-4))

    return g, ins, check


def rmsnorm_two_value():
    """samples/rmsnorm/*.cpp + rmsnorm_utils.h:26-90; abs tol 1e-4."""
    n, c, h, w, scale, eps = 2, 3, 32, 32, 2.0, 1e-5
    g = fz.Graph()
    g.setName("kat_rms").setIODataType(F32).setComputeDataType(F32).setIntermediateDataType(F32)
    x = g.tensor(TensorAttr().setName("x").setDim([n, c, h, w]).setStride(channelsLastStride([n, c, h, w])))
    st = g.tensor(TensorAttr().setName("scale").setDim([1, c, h, w]).setStride(channelsLastStride([1, c, h, w])))
    e = g.tensor(TensorAttr(eps).setName("eps"))
    y, _ = g.rmsnorm(x, st, fz.RmsnormAttr().setForwardPhase(fz.NormFwdPhase.INFERENCE).setEpsilon(e))
    y.setOutput(True)
    g.validate()
    row = c * h * w
    xin = np.zeros(n * row, np.float32)
    want = np.zeros(n * row, np.float32)
    for b in range(n):
        x0, x1 = 2.0 * b + 1, 2.0 * b + 3
        rms = math.sqrt((x0 * x0 + x1 * x1) / 2 + eps)
        xin[b * row: b * row + row // 2] = x0
        xin[b * row + row // 2: (b + 1) * row] = x1
        want[b * row: b * row + row // 2] = scale * x0 / rms
        want[b * row + row // 2: (b + 1) * row] = scale * x1 / rms
    return g, {x: xin, st: _fill(st, scale)}, lambda o: np.all(np.abs(o[y] - want) < 1e-4)


def reduction_i32(mode):
    """samples/reduction/reduction_ops.cpp:83-273: values -50..49, [2,16,8,8] -> [2,16,1,1], exact."""
    g = fz.Graph()
    g.setName("kat_red_" + mode).setIODataType(I32).setComputeDataType(F32)
    x = g.tensor(TensorAttr().setName("x").setDim([2, 16, 8, 8]).setStride(contiguousStride([2, 16, 8, 8])))
    y = g.reduction(x, fz.ReductionAttr().setMode(ReductionMode[mode]))
    y.setDim([2, 16, 1, 1]).setStride([16, 1, 1, 1]).setName("y").setOutput(True)
    g.validate()
    xin = (np.arange(2 * 16 * 64) % 100 - 50).astype(np.int32)
    v = xin.reshape(32, 64).astype(np.int64)
    want = {"ADD": v.sum(1), "SUM": v.sum(1), "MIN": v.min(1), "MAX": v.max(1), "AMAX": np.abs(v).max(1),
            "NORM1": np.abs(v).sum(1)}[mode]
    return g, {x: xin}, lambda o: np.array_equal(o[y].astype(np.int64), want)


def pointwise_i32_div():
    """samples/pointwise/pointwise_binary_ops.cpp:129-131,176: i32 -50 / 13 == -3 (truncation)."""
    g = fz.Graph()
    g.setName("kat_div").setIODataType(I32).setComputeDataType(F32)
    a = g.tensor(TensorAttr().setName("a").setDim([2, 16, 64, 64]).setStride(contiguousStride([2, 16, 64, 64])))
    b = g.tensor(TensorAttr().setName("b").setDim([1, 16, 1, 1]).setStride([16, 1, 1, 1]))
    o = g.pointwise(a, b, fz.PointwiseAttr().setMode(PointwiseMode.DIV))
    o.setName("o").setOutput(True)
    g.validate()
    return (g, {a: np.full(a.getVolume(), -50, np.int32), b: np.full(16, 13, np.int32)},
            lambda out: np.all(out[o] == -3))


def aot_add_i32():
    """samples/aot/single_backend.cpp: 2 + 3 == 5."""
    g = fz.Graph()
    g.setName("kat_aot_add").setIODataType(I32).setComputeDataType(I32)
    a = g.tensor(TensorAttr().setName("a").setDim([4, 4]).setStride([4, 1]))
    b = g.tensor(TensorAttr().setName("b").setDim([4, 4]).setStride([4, 1]))
    o = g.pointwise(a, b, fz.PointwiseAttr().setMode(PointwiseMode.ADD))
    o.setName("o").setOutput(True)
    g.validate()
    return g, {a: np.full(16, 2, np.int32), b: np.full(16, 3, np.int32)}, lambda out: np.all(out[o] == 5)


CASES = {
    "conv_fprop_1x1_bias_relu": conv_fprop_1x1_bias_relu,
    "conv_fprop_3x3_pad": conv_fprop_3x3_pad,
    "conv_fprop_grouped_bias_relu": conv_fprop_grouped_bias_relu,
    "conv_dgrad_1x1": conv_dgrad_1x1,
    "conv_wgrad_grouped_strided": conv_wgrad_grouped_strided,
    "matmul_batched_bias": matmul_batched_bias,
    "matmul_transposed_b_f16": matmul_transposed_b_f16,
    "matmul_int4_fp16": matmul_int4_fp16,
    "batchnorm_infer_nchw_scale_bias": batchnorm_infer_nchw_scale_bias,
    "batchnorm_train_nchw_two_value": batchnorm_train_nchw_two_value,
    "sdpa_mha": lambda: _sdpa_case("kat_sdpa_mha"),
    "sdpa_causal": lambda: _sdpa_case("kat_sdpa_causal", causal=True),
    "sdpa_mask": lambda: _sdpa_case("kat_sdpa_mask", mask=True),
    "sdpa_gqa_8_2": lambda: _sdpa_case("kat_sdpa_gqa", hk=2, hv=2),
    "sdpa_gqa_8_4_2": lambda: _sdpa_case("kat_sdpa_gqa2", hk=4, hv=2),
    "sdpa_cross_32x128": lambda: _sdpa_case("kat_sdpa_cross", sq=32, skv=128),
    "layernorm_train_nhwc_affine": lambda: layernorm_train_two_value("NHWC", True),
    "layernorm_train_nchw_plain": lambda: layernorm_train_two_value("NCHW", False),
    "rmsnorm_two_value": rmsnorm_two_value,
    "reduction_i32_ADD": lambda: reduction_i32("ADD"),
    "reduction_i32_MIN": lambda: reduction_i32("MIN"),
    "reduction_i32_MAX": lambda: reduction_i32("MAX"),
    "reduction_i32_AMAX": lambda: reduction_i32("AMAX"),
    "reduction_i32_NORM1": lambda: reduction_i32("NORM1"),
    "pointwise_i32_div": pointwise_i32_div,
    "aot_add_i32": aot_add_i32,
}
