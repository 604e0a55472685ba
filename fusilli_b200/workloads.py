"""Graph builders for the benchmarked workloads, following the canonical graph
construction of the reference's benchmark driver (benchmarks/driver.cpp:
conv fprop :116, wgrad :249, dgrad :381, layernorm :513, sdpa :610, matmul :740):
where dtypes are set, how the bias is shaped, which layouts are used.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np

from .graph import (BatchnormAttr, ConvDGradAttr, ConvFPropAttr, ConvWGradAttr, DataType, LayernormAttr, MatmulAttr,
                    NormFwdPhase, PointwiseAttr, ReductionAttr, RmsnormAttr, SdpaAttr, TensorAttr,
                    channelsLastStride, contiguousStride)
from .runtime import Graph


# Seeds of the benchmarked configurations: one generator per (configuration, tensor), tensors
# numbered in declaration order, so any tensor can be regenerated alone and a rank can draw just
# its shard's source tensor. Configurations are numbered from 0 in the order the benchmark
# lists them (fp32 conv, batched matmul, attention, ResNet-50 layers, norms).
SEED_BASE = 0x5EED

RESNET_LAYERS = [  # (C, H = W, K, R = S, pad) of the bf16 convolution sweep at N = 256
    (64, 56, 64, 1, 0), (64, 56, 64, 3, 1), (128, 28, 128, 3, 1), (256, 14, 1024, 1, 0), (512, 7, 512, 3, 1)]


def seeded_values(config: int, tensor_index: int, count: int, dist) -> np.ndarray:
    """`count` float32 values of tensor number `tensor_index` of configuration `config`;
    dist = ("normal", mean, std) or ("uniform", lo, hi)."""
    rng = np.random.default_rng([SEED_BASE + int(config), int(tensor_index)])
    if dist[0] == "normal":
        v = rng.standard_normal(count, dtype=np.float32)
        v *= np.float32(dist[2])
        if dist[1]:
            v += np.float32(dist[1])
        return v
    if dist[0] == "uniform":
        v = rng.random(count, dtype=np.float32)
        v *= np.float32(dist[2] - dist[1])
        v += np.float32(dist[1])
        return v
    raise ValueError(dist)


def _new(name: str, io: DataType, inter: DataType = DataType.Float) -> Graph:
    g = Graph()
    g.setName(name).setIODataType(io).setComputeDataType(DataType.Float).setIntermediateDataType(inter)
    return g


def conv_fprop_bias_relu(n, c, h, w, k, r, s, pad, dtype=DataType.Float, stride=1, dilation=1,
                         bias=True, relu=True, name="conv_fprop"):
    """NHWC x, KRSC w, optional bias [1,K,1,1] + ReLU fused (driver.cpp:116-247)."""
    g = _new(name, dtype, dtype)
    x = g.tensor(TensorAttr().setName("x").setDim([n, c, h, w]).setStride(channelsLastStride([n, c, h, w])))
    wt = g.tensor(TensorAttr().setName("w").setDim([k, c, r, s]).setStride(channelsLastStride([k, c, r, s])))
    y = g.convFProp(x, wt, ConvFPropAttr().setPadding([pad, pad]).setStride([stride, stride])
                    .setDilation([dilation, dilation]).setName("conv"))
    ins = {"x": x, "w": wt}
    if bias:
        b = g.tensor(TensorAttr().setName("bias").setDim([1, k, 1, 1]).setStride([k, 1, k, k]))
        y = g.pointwise(y, b, PointwiseAttr().setMode(PointwiseAttr.Mode.ADD).setName("bias_add"))
        ins["bias"] = b
    if relu:
        y = g.pointwise(y, PointwiseAttr().setMode(PointwiseAttr.Mode.RELU_FWD).setName("relu"))
    y.setName("y").setOutput(True)
    g.validate()
    return g, ins, y


def conv_dgrad(n, c, h, w, k, r, s, pad, dtype=DataType.BFloat16, stride=1, name="conv_dgrad", dilation=1):
    g = _new(name, dtype, dtype)
    p = 1 + (h + 2 * pad - (r - 1) * dilation - 1) // stride
    q = 1 + (w + 2 * pad - (s - 1) * dilation - 1) // stride
    dy = g.tensor(TensorAttr().setName("dy").setDim([n, k, p, q]).setStride(channelsLastStride([n, k, p, q])))
    wt = g.tensor(TensorAttr().setName("w").setDim([k, c, r, s]).setStride(channelsLastStride([k, c, r, s])))
    dx = g.convDGrad(dy, wt, ConvDGradAttr().setPadding([pad, pad]).setStride([stride, stride])
                     .setDilation([dilation, dilation]).setName("dgrad"))
    dx.setName("dx").setDim([n, c, h, w]).setOutput(True)
    g.validate()
    return g, {"dy": dy, "w": wt}, dx


def conv_wgrad(n, c, h, w, k, r, s, pad, dtype=DataType.BFloat16, stride=1, name="conv_wgrad", dw_dtype=None,
               dilation=1):
    """dy, x NHWC of `dtype`; dw KRSC of `dw_dtype` (default `dtype`; Float keeps the fp32 sum, which
    is what a rank contributes to the cross-rank exchange before the one rounding)."""
    g = _new(name, dtype, dtype)
    p = 1 + (h + 2 * pad - (r - 1) * dilation - 1) // stride
    q = 1 + (w + 2 * pad - (s - 1) * dilation - 1) // stride
    dy = g.tensor(TensorAttr().setName("dy").setDim([n, k, p, q]).setStride(channelsLastStride([n, k, p, q])))
    x = g.tensor(TensorAttr().setName("x").setDim([n, c, h, w]).setStride(channelsLastStride([n, c, h, w])))
    dw = g.convWGrad(dy, x, ConvWGradAttr().setPadding([pad, pad]).setStride([stride, stride])
                     .setDilation([dilation, dilation]).setName("wgrad"))
    dw.setName("dw").setDim([k, c, r, s]).setOutput(True)
    if dw_dtype is not None:
        dw.setDataType(dw_dtype)
    g.validate()
    return g, {"dy": dy, "x": x}, dw


def matmul_bias(b, m, n, k, dtype=DataType.BFloat16, bias=True, trans_b=False, name="matmul"):
    """A[b,m,k] x B[b,k,n] row-major, bias [1,1,n]; the matmul's own (virtual) result
    takes the bias dtype and the ADD result the output dtype (driver.cpp:807-828)."""
    g = _new(name, dtype, dtype)
    ad = [b, m, k] if b > 1 else [m, k]
    bd = [b, k, n] if b > 1 else [k, n]
    a = g.tensor(TensorAttr().setName("a").setDim(ad).setStride(contiguousStride(ad)).setDataType(dtype))
    if trans_b:
        bs = [k * n, 1, k] if b > 1 else [1, k]
    else:
        bs = contiguousStride(bd)
    bt = g.tensor(TensorAttr().setName("b").setDim(bd).setStride(bs).setDataType(dtype))
    c = g.matmul(a, bt, MatmulAttr().setName("mm"))
    c.setDataType(dtype)
    ins = {"a": a, "b": bt}
    if bias:
        bdim = [1, 1, n] if b > 1 else [1, n]
        bi = g.tensor(TensorAttr().setName("bias").setDim(bdim).setStride(contiguousStride(bdim)).setDataType(dtype))
        c = g.pointwise(c, bi, PointwiseAttr().setMode(PointwiseAttr.Mode.ADD).setName("bias_add"))
        ins["bias"] = bi
    c.setName("c").setOutput(True).setDataType(dtype)
    g.validate()
    return g, ins, c


def sdpa_fwd(b, h, s, d, dtype=DataType.BFloat16, causal=True, skv=None, hkv=None, mask=False,
             scale=None, name="sdpa"):
    g = _new(name, dtype, dtype)
    skv = skv or s
    hkv = hkv or h
    qd, kd = [b, h, s, d], [b, hkv, skv, d]
    q = g.tensor(TensorAttr().setName("q").setDim(qd).setStride(contiguousStride(qd)))
    k = g.tensor(TensorAttr().setName("k").setDim(kd).setStride(contiguousStride(kd)))
    v = g.tensor(TensorAttr().setName("v").setDim(kd).setStride(contiguousStride(kd)))
    ins = {"q": q, "k": k, "v": v}
    m = None
    if mask:
        md = [b, 1, s, skv]
        m = g.tensor(TensorAttr().setName("mask").setDim(md).setStride(contiguousStride(md)))
        ins["mask"] = m
    attr = SdpaAttr().setIsCausal(causal).setEnableGqa(hkv != h).setName("attn")
    if scale is not None:
        attr.setScale(scale)
    o = g.sdpa(q, k, v, m, attr)
    o.setName("o").setOutput(True)
    g.validate()
    return g, ins, o


def layernorm_infer(rows, cols, dtype=DataType.BFloat16, param_dtype=DataType.Float, train=False, name="layernorm"):
    g = _new(name, dtype, dtype)
    xd = [rows, cols]
    x = g.tensor(TensorAttr().setName("x").setDim(xd).setStride(contiguousStride(xd)))
    sc = g.tensor(TensorAttr().setName("gamma").setDim([1, cols]).setStride([cols, 1]).setDataType(param_dtype))
    bi = g.tensor(TensorAttr().setName("beta").setDim([1, cols]).setStride([cols, 1]).setDataType(param_dtype))
    eps = g.tensor(TensorAttr(1e-5).setName("eps"))
    attr = LayernormAttr().setForwardPhase(NormFwdPhase.TRAINING if train else NormFwdPhase.INFERENCE)
    attr.setEpsilon(eps).setName("ln")
    y, mean, rstd = g.layernorm(x, sc, bi, attr)
    y.setName("y").setOutput(True)
    outs = [y]
    if train:
        mean.setName("mean").setOutput(True).setDataType(DataType.Float)
        rstd.setName("rstd").setOutput(True).setDataType(DataType.Float)
        outs += [mean, rstd]
    g.validate()
    return g, {"x": x, "gamma": sc, "beta": bi}, outs


def rmsnorm_infer(rows, cols, dtype=DataType.BFloat16, param_dtype=DataType.Float, name="rmsnorm"):
    g = _new(name, dtype, dtype)
    xd = [rows, cols]
    x = g.tensor(TensorAttr().setName("x").setDim(xd).setStride(contiguousStride(xd)))
    sc = g.tensor(TensorAttr().setName("gamma").setDim([1, cols]).setStride([cols, 1]).setDataType(param_dtype))
    eps = g.tensor(TensorAttr(1e-5).setName("eps"))
    attr = RmsnormAttr().setForwardPhase(NormFwdPhase.INFERENCE).setEpsilon(eps).setName("rms")
    y, _ = g.rmsnorm(x, sc, attr)
    y.setName("y").setOutput(True)
    g.validate()
    return g, {"x": x, "gamma": sc}, y


def row_sum(rows, cols, dtype=DataType.BFloat16, name="rowsum"):
    g = _new(name, dtype, dtype)
    xd = [rows, cols]
    x = g.tensor(TensorAttr().setName("x").setDim(xd).setStride(contiguousStride(xd)))
    y = g.reduction(x, ReductionAttr().setMode(ReductionAttr.Mode.SUM).setName("sum"))
    y.setName("y").setDim([rows, 1]).setStride([1, 1]).setOutput(True)
    g.validate()
    return g, {"x": x}, y


def batchnorm_fwd(n, c, spatial, dtype=DataType.BFloat16, param_dtype=DataType.Float, train=False,
                  channels_last=False, affine=True, running=True, name="batchnorm"):
    """x [n, c, *spatial] (contiguous or channels-last), per-channel [c] parameters, as the reference's
    samples/batchnorm/*.cpp build it."""
    g = _new(name, dtype, dtype)
    xd = [n, c] + list(spatial)
    xs = channelsLastStride(xd) if channels_last else contiguousStride(xd)
    x = g.tensor(TensorAttr().setName("x").setDim(xd).setStride(xs))
    ins = {"x": x}

    def per_channel(nm):
        t = g.tensor(TensorAttr().setName(nm).setDim([c]).setStride([1]).setDataType(param_dtype))
        ins[nm] = t
        return t
    sc = per_channel("gamma") if affine else None
    bi = per_channel("beta") if affine else None
    mean = per_channel("mean") if running else None
    var = per_channel("var") if running else None
    attr = BatchnormAttr().setForwardPhase(NormFwdPhase.TRAINING if train else NormFwdPhase.INFERENCE)
    attr.setEpsilon(g.tensor(TensorAttr(1e-5).setName("eps"))).setMomentum(g.tensor(TensorAttr(0.1).setName("momentum")))
    attr.setName("bn")
    y, sm, si = g.batchnorm(x, sc, bi, mean, var, attr)
    y.setName("y").setOutput(True)
    outs = [y]
    if train:
        sm.setName("saved_mean").setOutput(True).setDataType(DataType.Float)
        si.setName("saved_inv_var").setOutput(True).setDataType(DataType.Float)
        outs += [sm, si]
    g.validate()
    return g, ins, outs
