"""GPU parity: every op family of the hot path, CUDA (through the C ABI) against the
CPU oracle on identical seeded bytes. Tolerances are the contract's: integers
bit-exact, fp32 rtol 1e-5, 16-bit rtol/atol 2e-2."""
import numpy as np
import pytest

import fusilli_b200 as fz
from fusilli_b200 import workloads as wl
from fusilli_b200.graph import (DataType, PointwiseMode, ReductionMode, TensorAttr, channelsLastStride,
                                contiguousStride)
from helpers import check_graph, make_input

pytestmark = pytest.mark.gpu

F32, F16, BF16, I32 = DataType.Float, DataType.Half, DataType.BFloat16, DataType.Int32


def _inputs(ins, seed, dist=("uniform", -1.0, 1.0), per=None):
    rng = np.random.default_rng(seed)
    per = per or {}
    return {t: make_input(t, rng, per.get(name, dist)) for name, t in ins.items()}


# ---- convolution ------------------------------------------------------------------
def test_conv_fprop_c1_exact_config():
    """BASELINE config 1 at full size: fp32 NHWC 16x56x56x64 -> 64, 3x3 pad 1, bias + ReLU."""
    g, ins, y = wl.conv_fprop_bias_relu(16, 64, 56, 56, 64, 3, 3, 1, F32)
    data = _inputs(ins, 0x5EED + 0, per={"bias": ("uniform", -0.1, 0.1)})
    check_graph(g, data)
    # bf16 piece split of x and w, then ONE tensor-core kernel for conv + bias + relu
    assert "conv_fprop_split_f32_tcgen05" in g.statistics()
    assert g.numLaunches() == 2 and g.getWorkspaceSize() > 0


def test_conv_fprop_f32_tensor_core_path_beats_fp32_fma_accuracy():
    """The fp32 forward convolution on the tensor cores (three bf16 pieces per operand, TMEM
    accumulation restarted per filter tap, chunks added in fp32 registers) against the float64
    accumulating oracle: its worst error must stay below what a plain fp32 FMA chain of the same
    length gives (about 4e-5 on these inputs), i.e. it is an fp32-grade result, not a bf16 one."""
    from helpers import run_gpu
    from oracle import fusilli_oracle as orc
    g, ins, y = wl.conv_fprop_bias_relu(6, 128, 28, 36, 96, 3, 3, 1, F32)
    data = _inputs(ins, 0x5EED, per={"bias": ("uniform", -0.1, 0.1)})
    want = orc.execute(g, data)[y].astype(np.float64)
    got = run_gpu(g, data)[y].astype(np.float64)
    assert "conv_fprop_split_f32_tcgen05" in g.statistics()
    # K = 9 * 128 products of U[-1,1] values per output, |y| up to ~50
    assert np.abs(got - want).max() < 3e-5


@pytest.mark.parametrize("shape", [
    (2, 64, 56, 56, 64, 1, 1, 0), (2, 64, 56, 56, 64, 3, 3, 1), (2, 128, 28, 28, 128, 3, 3, 1),
    (4, 256, 14, 14, 1024, 1, 1, 0), (4, 512, 7, 7, 512, 3, 3, 1),
])
def test_conv_resnet_layers_bf16_fprop_dgrad_wgrad(shape):
    """BASELINE config 4's five layers at reduced batch: fprop, dgrad, wgrad in bf16."""
    n, c, h, w, k, r, s, pad = shape
    x_dist, dy_dist = ("normal", 0.0, 0.05), ("normal", 0.0, 0.01)
    g, ins, _ = wl.conv_fprop_bias_relu(n, c, h, w, k, r, s, pad, BF16, bias=False, relu=False)
    check_graph(g, _inputs(ins, 1, x_dist))
    g, ins, _ = wl.conv_dgrad(n, c, h, w, k, r, s, pad, BF16)
    check_graph(g, _inputs(ins, 2, per={"dy": dy_dist, "w": x_dist}))
    g, ins, _ = wl.conv_wgrad(n, c, h, w, k, r, s, pad, BF16)
    check_graph(g, _inputs(ins, 3, per={"dy": dy_dist, "x": x_dist}))
@pytest.mark.parametrize("shape", [
    (32, 512, 7, 7, 512, 3, 3, 1),    # one rank's shard of the 7x7 layer on 8 GPUs: 1568 pixels, 25 ragged patches
    (64, 512, 7, 7, 512, 3, 3, 1),    # ... on 4 GPUs
    (32, 256, 14, 14, 1024, 1, 1, 0),  # the 14x14 1x1 layer's shard on 8 GPUs
    (21, 64, 7, 7, 64, 3, 3, 1),      # 1029 pixels: just above the tensor-core kernel's threshold
])
def test_conv_wgrad_small_pixel_counts_on_tensor_cores(shape):
    """Weight gradients whose reduction is only a few thousand pixels (what a rank sees when the
    benchmark's batch is split over 4 or 8 GPUs) still take the tensor-core kernel."""
    n, c, h, w, k, r, s, pad = shape
    g, ins, _ = wl.conv_wgrad(n, c, h, w, k, r, s, pad, BF16)
    check_graph(g, _inputs(ins, 17, per={"dy": ("normal", 0.0, 0.01), "x": ("normal", 0.0, 0.05)}))
    assert "conv_wgrad_tcgen05" in g.statistics()
    g, ins, _ = wl.conv_wgrad(n, c, h, w, k, r, s, pad, BF16, dw_dtype=F32)   # the fp32 partial a rank contributes
    check_graph(g, _inputs(ins, 18, per={"dy": ("normal", 0.0, 0.01), "x": ("normal", 0.0, 0.05)}))


@pytest.mark.parametrize("n", [5, 6, 7])
@pytest.mark.parametrize("k", [128, 256, 192])
def test_conv_wide_layers_on_cta_pairs(n, k):
    """128- and 256-channel tiles with at least eight K blocks run on clusters of two CTAs (two neighbouring
    pixel tiles per 256-row MMA); batch sizes that give even and odd tile counts (an odd count leaves the last
    pair's second tile past the end of the tensor), a ragged channel tile (192), fused bias + ReLU, dgrad."""
    c, h, w, r, s, pad = 128, 14, 14, 3, 3, 1
    x_dist, dy_dist = ("normal", 0.0, 0.05), ("normal", 0.0, 0.01)
    g, ins, _ = wl.conv_fprop_bias_relu(n, c, h, w, k, r, s, pad, BF16)
    check_graph(g, _inputs(ins, 31, x_dist, per={"bias": ("uniform", -0.1, 0.1)}))
    assert "conv_fprop_tcgen05" in g.statistics()
    g, ins, _ = wl.conv_dgrad(n, c, h, w, k, r, s, pad, BF16)
    check_graph(g, _inputs(ins, 32, per={"dy": dy_dist, "w": x_dist}))


@pytest.mark.parametrize("shape", [
    (5, 64, 20, 12, 64, 3, 3, 1),     # ragged 8 x 8 patches, five images against stages of four
    (3, 128, 16, 24, 128, 3, 3, 1),   # two 64-channel tiles, 128 output channels (two dY boxes per image)
    (6, 64, 18, 18, 64, 3, 3, 0),     # no padding: 16 x 16 outputs
    (5, 64, 16, 16, 128, 1, 3, 0),    # one filter row: a column's single tap
    (9, 64, 16, 16, 64, 2, 2, 0),     # even filter: 15 x 15 outputs
    (2, 64, 24, 24, 192, 3, 3, 1),    # two output-channel tiles
])
@pytest.mark.parametrize("dtype", [BF16, F16])
def test_conv_wgrad_haloed_patches(shape, dtype):
    """Weight gradients of narrow R x S > 1 layers: one CTA per filter column reads the column's taps as
    shifted windows of one haloed X patch, several images per ring stage."""
    n, c, h, w, k, r, s, pad = shape
    per = {"dy": ("normal", 0.0, 0.01), "x": ("normal", 0.0, 0.05)}
    g, ins, _ = wl.conv_wgrad(n, c, h, w, k, r, s, pad, dtype)
    check_graph(g, _inputs(ins, 23, per=per))
    assert "conv_wgrad_tcgen05" in g.statistics()
    g, ins, _ = wl.conv_wgrad(n, c, h, w, k, r, s, pad, dtype, dw_dtype=F32)
    check_graph(g, _inputs(ins, 24, per=per))


@pytest.mark.parametrize("shape", [
    (2, 96, 30, 24, 160, 3, 3, 1),   # ragged channel block and ragged output-channel tile
    (1, 64, 32, 32, 64, 5, 5, 2),    # 5x5 taps, resident filter
    (1, 64, 34, 34, 128, 3, 3, 0),   # no padding: output 32x32
    (1, 64, 16, 16, 512, 3, 3, 1),   # two output-channel tiles, streamed filter
    (3, 128, 56, 56, 64, 3, 3, 1),   # several patch slots in flight per tile
])
@pytest.mark.parametrize("dtype", [BF16, F16])
def test_conv_halo_tiles(shape, dtype):
    """3x3 / 5x5 unit-stride layers large enough for the kernel that loads one haloed patch per
    channel block and reads every tap as a shifted window of it; fprop with fused bias + ReLU and
    dgrad."""
    n, c, h, w, k, r, s, pad = shape
    x_dist, dy_dist = ("normal", 0.0, 0.05), ("normal", 0.0, 0.01)
    g, ins, _ = wl.conv_fprop_bias_relu(n, c, h, w, k, r, s, pad, dtype)
    check_graph(g, _inputs(ins, 4, x_dist, per={"bias": ("uniform", -0.1, 0.1)}))
    g, ins, _ = wl.conv_dgrad(n, c, h, w, k, r, s, pad, dtype)
    check_graph(g, _inputs(ins, 5, per={"dy": dy_dist, "w": x_dist}))
@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("shape", [(2, 64, 40, 40, 64, 3, 3, 2, 2), (3, 128, 36, 28, 96, 3, 3, 3, 3), (2, 64, 33, 33, 128, 5, 5, 4, 2)])
def test_conv_dilated_on_tensor_cores(dtype, shape):
    """16-bit channels-last convolutions with dilation > 1 and >= 64 channels take the tensor-core
    kernels (per-tap loads step by the dilation): fprop, dgrad and wgrad against the oracle."""
    n, c, h, w, k, r, s, pad, dil = shape
    x_dist, dy_dist = ("normal", 0.0, 0.05), ("normal", 0.0, 0.01)
    g, ins, _ = wl.conv_fprop_bias_relu(n, c, h, w, k, r, s, pad, dtype, dilation=dil)
    check_graph(g, _inputs(ins, 14, x_dist, per={"bias": ("uniform", -0.1, 0.1)}))
    assert "tcgen05" in g.statistics()
    g, ins, _ = wl.conv_dgrad(n, c, h, w, k, r, s, pad, dtype, dilation=dil)
    check_graph(g, _inputs(ins, 15, per={"dy": dy_dist, "w": x_dist}))
    assert "tcgen05" in g.statistics()
    g, ins, _ = wl.conv_wgrad(n, c, h, w, k, r, s, pad, dtype, dilation=dil)
    check_graph(g, _inputs(ins, 16, per={"dy": dy_dist, "x": x_dist}))


@pytest.mark.parametrize("dtype", [F16, F32])
@pytest.mark.parametrize("case", ["grouped_strided", "nchw", "dilated", "conv1d", "conv3d"])
def test_conv_variants(dtype, case):
    g = fz.Graph()
    g.setName("conv_" + case).setIODataType(dtype).setComputeDataType(F32).setIntermediateDataType(dtype)
    if case == "grouped_strided":
        xd, wd, pad, st, dl, cl = [2, 16, 13, 12], [24, 4, 3, 3], [1, 1], [2, 2], [1, 1], True
    elif case == "nchw":
        xd, wd, pad, st, dl, cl = [3, 6, 10, 9], [8, 6, 3, 3], [1, 0], [1, 1], [1, 1], False
    elif case == "dilated":
        xd, wd, pad, st, dl, cl = [1, 8, 15, 14], [8, 8, 3, 2], [2, 1], [1, 1], [2, 2], True
    elif case == "conv1d":
        xd, wd, pad, st, dl, cl = [2, 8, 40], [12, 8, 5], [2], [1], [1], True
    else:
        xd, wd, pad, st, dl, cl = [2, 4, 5, 9, 8], [6, 4, 2, 3, 3], [0, 1, 1], [1, 1, 1], [1, 1, 1], True
    sf = channelsLastStride if cl else contiguousStride
    x = g.tensor(TensorAttr().setName("x").setDim(xd).setStride(sf(xd)))
    w = g.tensor(TensorAttr().setName("w").setDim(wd).setStride(sf(wd)))
    y = g.convFProp(x, w, fz.ConvFPropAttr().setPadding(pad).setStride(st).setDilation(dl))
    y.setName("y").setOutput(True)
    g.validate()
    data = _inputs({"x": x, "w": w}, 7)
    check_graph(g, data)
    for kind in ("dgrad", "wgrad"):
        g2 = fz.Graph()
        g2.setName(f"conv_{case}_{kind}").setIODataType(dtype).setComputeDataType(F32).setIntermediateDataType(dtype)
        dy = g2.tensor(TensorAttr().setName("dy").setDim(y.dim).setStride(sf(y.dim)))
        if kind == "dgrad":
            w2 = g2.tensor(TensorAttr().setName("w").setDim(wd).setStride(sf(wd)))
            o = g2.convDGrad(dy, w2, fz.ConvDGradAttr().setPadding(pad).setStride(st).setDilation(dl))
            o.setDim(xd).setName("dx").setOutput(True)
            ins = {"dy": dy, "w": w2}
        else:
            x2 = g2.tensor(TensorAttr().setName("x").setDim(xd).setStride(sf(xd)))
            o = g2.convWGrad(dy, x2, fz.ConvWGradAttr().setPadding(pad).setStride(st).setDilation(dl))
            o.setDim(wd).setName("dw").setOutput(True)
            ins = {"dy": dy, "x": x2}
        g2.validate()
        check_graph(g2, _inputs(ins, 8))
@pytest.mark.parametrize("geom", [
    # x dims (NCHW logical), w dims, pad, stride, dilation
    ([3, 32, 19, 23], [24, 32, 3, 3], [1, 1], [1, 1], [1, 1]),   # ragged pixel and output-channel tiles
    ([2, 48, 17, 17], [40, 48, 3, 3], [2, 2], [2, 2], [2, 2]),   # stride and dilation
    ([2, 64, 12, 12], [32, 16, 3, 3], [1, 1], [1, 1], [1, 1]),   # four groups of 16 channels
    ([1, 16, 9, 30], [16, 16, 1, 5], [0, 2], [1, 1], [1, 1]),    # 1x5 taps
])
def test_conv_fprop_f32_channels_last(geom):
    """fp32 channels-last forward convolutions whose channel count per group is a multiple of 16: the
    CUDA-core kernel with the hoisted index arithmetic; results to the fp32 tolerance."""
    xd, wd, pad, st, dl = geom
    g = fz.Graph()
    g.setName("conv_f32_cl").setIODataType(F32).setComputeDataType(F32).setIntermediateDataType(F32)
    x = g.tensor(TensorAttr().setName("x").setDim(xd).setStride(channelsLastStride(xd)))
    w = g.tensor(TensorAttr().setName("w").setDim(wd).setStride(channelsLastStride(wd)))
    y = g.convFProp(x, w, fz.ConvFPropAttr().setPadding(pad).setStride(st).setDilation(dl))
    y.setName("y").setOutput(True)
    g.validate()
    check_graph(g, _inputs({"x": x, "w": w}, 9))
@pytest.mark.parametrize("cfg", [
    # b, m, n, k, dtype, bias, trans_b
    (2, 256, 512, 384, BF16, True, False),   # row-major B (MN-major operand), tensor cores
    (2, 256, 512, 384, BF16, True, True),    # transposed B (K-major operand)
    (1, 384, 256, 512, F16, False, False),
    (3, 200, 264, 136, BF16, True, False),   # ragged tiles: zero-filled loads, clipped stores
    (1, 128, 64, 32, BF16, False, False),    # smallest shape the tensor-core kernel takes
    (2, 96, 80, 72, F32, True, False),       # fp32: CUDA-core kernel
    (4, 16, 32, 64, F16, True, False),       # tiny: CUDA-core kernel
    (1, 2048, 2560, 128, BF16, True, False),  # 160 tiles on 148 SMs: whole tiles, then 12 split into halves
    (1, 2048, 2560, 128, F16, False, True),   # the same with a K-major B (two 128-row boxes per tile)
    (1, 1024, 1152, 192, BF16, True, False),  # 40 tiles, all split; the last column tile has one half out of range
])
def test_matmul(cfg):
    b, m, n, k, dtype, bias, trans_b = cfg
    g, ins, _ = wl.matmul_bias(b, m, n, k, dtype, bias, trans_b)
    data = _inputs(ins, 11, ("normal", 0.0, 0.5))
    check_graph(g, data)
    assert g.numLaunches() == 1


def test_matmul_c2_tile_sized_slice():
    """BASELINE config 2's distribution (normal(0, 0.02)) and K = 4096 on one 512x512 output."""
    g, ins, _ = wl.matmul_bias(1, 512, 512, 4096, BF16, True)
    check_graph(g, _inputs(ins, 0x5EED + 1, ("normal", 0.0, 0.02)))
def test_matmul_batch_broadcast_and_transposed_a():
    g = fz.Graph()
    g.setName("mm_bcast").setIODataType(F16).setComputeDataType(F32).setIntermediateDataType(F16)
    a = g.tensor(TensorAttr().setName("a").setDim([4, 64, 48]).setStride([64 * 48, 1, 64]))  # A stored transposed
    b = g.tensor(TensorAttr().setName("b").setDim([1, 48, 72]).setStride(contiguousStride([1, 48, 72])))
    c = g.matmul(a, b, fz.MatmulAttr())
    c.setName("c").setOutput(True)
    g.validate()
    check_graph(g, _inputs({"a": a, "b": b}, 12))
@pytest.mark.parametrize("dtype,m,n,k", [(BF16, 256, 192, 128), (F32, 40, 24, 56)])
@pytest.mark.parametrize("a_batch,b_batch", [(4, 2), (2, 6)])
def test_matmul_batch_broadcast_by_a_divisor(dtype, m, n, k, a_batch, b_batch):
    """Batch dims that divide one another (reference matmul_node.h:140-150 accepts them): the operand
    with fewer matrices is read modulo its own batch extent, on the tensor-core and the CUDA-core path."""
    g = fz.Graph()
    g.setName("mm_div").setIODataType(dtype).setComputeDataType(F32).setIntermediateDataType(dtype)
    a = g.tensor(TensorAttr().setName("a").setDim([a_batch, m, k]).setStride(contiguousStride([a_batch, m, k])))
    b = g.tensor(TensorAttr().setName("b").setDim([b_batch, k, n]).setStride(contiguousStride([b_batch, k, n])))
    c = g.matmul(a, b, fz.MatmulAttr())
    c.setName("c").setOutput(True)
    g.validate()
    assert c.dim[0] == max(a_batch, b_batch)
    check_graph(g, _inputs({"a": a, "b": b}, 13, ("normal", 0.0, 0.5)))
    assert ("gemm_tcgen05" in g.statistics()) == (dtype == BF16)


def _int4_matmul(b, m, k, n, other, a_int4=True, bias=False, odd_k=False):
    """si4 x f16/bf16 matmul (the reference's samples/matmul/matmul_int4_fp16.cpp pattern); mixed
    element types need rank 3 with equal batch (matmul_node.h:155-177)."""
    g = fz.Graph()
    g.setName("mm_int4").setIODataType(other).setComputeDataType(F32).setIntermediateDataType(F32)
    a = g.tensor(TensorAttr().setName("a").setDim([b, m, k]).setStride(contiguousStride([b, m, k])))
    bt = g.tensor(TensorAttr().setName("b").setDim([b, k, n]).setStride(contiguousStride([b, k, n])))
    (a if a_int4 else bt).setDataType(DataType.Int4)
    c = g.matmul(a, bt, fz.MatmulAttr().setName("mm"))
    ins = {"a": a, "b": bt}
    if bias:
        bi = g.tensor(TensorAttr().setName("bias").setDim([1, 1, n]).setStride([n, n, 1]))
        c = g.pointwise(c, bi, fz.PointwiseAttr().setMode(PointwiseMode.ADD).setName("bias_add"))
        ins["bias"] = bi
    c.setName("c").setOutput(True)
    g.validate()
    return g, ins


@pytest.mark.parametrize("cfg", [
    dict(b=1, m=4, k=8, n=4, other=F16),                       # the reference sample's shape
    dict(b=3, m=33, k=96, n=40, other=F16, bias=True),
    dict(b=2, m=17, k=63, n=25, other=BF16),                   # odd K: rows start in the middle of a byte
    dict(b=2, m=24, k=64, n=31, other=F16, a_int4=False),      # quantised B, odd N
    dict(b=1, m=128, k=512, n=256, other=BF16, bias=True),     # large enough for tensor cores, stays on CUDA cores
])
def test_matmul_int4_operand(cfg):
    g, ins = _int4_matmul(**cfg)
    data = _inputs(ins, 21, ("normal", 0.0, 0.5))
    check_graph(g, data)
    assert g.numLaunches() == 1
    assert "gemm_tcgen05" not in g.statistics()


# ---- batch normalisation -------------------------------------------------------------
@pytest.mark.parametrize("cfg", [
    dict(n=4, c=8, spatial=[5, 6], dtype=F32, train=False),
    dict(n=4, c=8, spatial=[5, 6], dtype=F32, train=True),
    dict(n=4, c=8, spatial=[5, 6], dtype=F32, train=True, channels_last=True),
    dict(n=16, c=64, spatial=[28, 28], dtype=BF16, train=True, channels_last=True),   # several slices per channel block
    dict(n=16, c=64, spatial=[28, 28], dtype=BF16, train=True),
    dict(n=8, c=48, spatial=[14, 14], dtype=F16, train=False, channels_last=True),
    dict(n=2, c=3, spatial=[4, 5, 6], dtype=F32, train=True),                         # 5-D
    dict(n=2, c=3, spatial=[4, 5, 6], dtype=F32, train=True, channels_last=True),
    dict(n=64, c=40, spatial=[], dtype=F32, train=True),                              # [N, C]
    dict(n=8, c=16, spatial=[7, 7], dtype=F32, train=True, affine=False, running=False),
    dict(n=8, c=16, spatial=[7, 7], dtype=BF16, train=False, affine=False),
    dict(n=32, c=256, spatial=[56, 56], dtype=BF16, train=True, channels_last=True),  # 51 M elements
])
def test_batchnorm(cfg):
    g, ins, outs = wl.batchnorm_fwd(**cfg)
    data = _inputs(ins, 31, ("uniform", -1.0, 3.0), per={"var": ("uniform", 0.25, 2.0)})
    check_graph(g, data)
    assert g.numLaunches() == (3 if cfg["train"] else 1)


# ---- sdpa ---------------------------------------------------------------------------
@pytest.mark.parametrize("cfg", [
    dict(b=1, h=8, s=64, d=64, dtype=F16, causal=False),
    dict(b=1, h=8, s=64, d=64, dtype=F16, causal=True),
    dict(b=2, h=8, s=64, d=64, dtype=F16, causal=False, mask=True),
    dict(b=1, h=8, s=64, d=64, dtype=F16, causal=False, hkv=2),
    dict(b=1, h=4, s=32, d=64, dtype=F16, causal=False, skv=128),
    dict(b=1, h=2, s=50, d=40, dtype=F32, causal=True),
    dict(b=1, h=2, s=64, d=64, dtype=F16, causal=False, scale=0.25),
    dict(b=2, h=4, s=512, d=128, dtype=BF16, causal=True),
    dict(b=1, h=2, s=384, d=128, dtype=BF16, causal=False),
    dict(b=1, h=2, s=200, d=128, dtype=BF16, causal=True),
    dict(b=1, h=4, s=1024, d=128, dtype=BF16, causal=True, hkv=2),
    dict(b=1, h=2, s=640, d=128, dtype=F16, causal=False),
    dict(b=1, h=2, s=300, d=128, dtype=BF16, causal=False, skv=1000),
    dict(b=1, h=1, s=1280, d=128, dtype=BF16, causal=True, scale=0.5),
])
def test_sdpa(cfg):
    g, ins, _ = wl.sdpa_fwd(**cfg)
    data = _inputs(ins, 21, ("normal", 0.0, 1.0))
    check_graph(g, data)


def test_sdpa_growing_row_maximum():
    """Scores whose row maximum keeps rising along the key axis (keys scaled by their index), so the
    accumulator rescaling in the tensor-core kernel runs on many blocks, not only on the first."""
    g, ins, _ = wl.sdpa_fwd(b=1, h=2, s=1024, d=128, dtype=BF16, causal=False)
    data = _inputs(ins, 22, ("normal", 0.0, 1.0))
    from oracle import fusilli_oracle as orc
    k = ins["k"]
    kv = orc.from_storage(data[k], BF16).reshape(1, 2, 1024, 128)
    ramp = np.linspace(0.2, 4.0, 1024, dtype=np.float32).reshape(1, 1, 1024, 1)
    data[k] = orc.to_storage((kv * ramp).reshape(-1).astype(np.float32), BF16)
    check_graph(g, data)


# ---- norms ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,rows,cols,pdt", [(BF16, 64, 8192, F32), (F16, 33, 4096, F16), (F32, 17, 1024, F32),
                                                 (BF16, 9, 1000, F32), (F32, 5, 30000, F32)])
@pytest.mark.parametrize("train", [False, True])
def test_layernorm_rows(dtype, rows, cols, pdt, train):
    g, ins, _ = wl.layernorm_infer(rows, cols, dtype, pdt, train)
    data = _inputs(ins, 31, ("normal", 0.0, 1.0), per={"gamma": ("normal", 1.0, 0.02), "beta": ("normal", 0.0, 0.02)})
    check_graph(g, data)
@pytest.mark.parametrize("kind,dtype,rows,cols,pdt,train", [
    ("ln", BF16, 1500, 8192, F32, False), ("ln", BF16, 1201, 8192, F32, True), ("rms", BF16, 1500, 8192, F32, False),
    ("ln", F16, 1333, 4096, F16, False), ("ln", F32, 1250, 4096, F32, True), ("rms", F32, 1400, 2048, F32, False),
])
def test_norm_many_rows(kind, dtype, rows, cols, pdt, train):
    """Enough rows for the persistent, bulk-copy-staged row kernel (several rows per CTA, uneven
    split over the grid)."""
    if kind == "ln":
        g, ins, _ = wl.layernorm_infer(rows, cols, dtype, pdt, train)
        per = {"gamma": ("normal", 1.0, 0.02), "beta": ("normal", 0.0, 0.02)}
    else:
        g, ins, _ = wl.rmsnorm_infer(rows, cols, dtype)
        per = {"gamma": ("normal", 1.0, 0.02)}
    data = _inputs(ins, 33, ("normal", 0.5, 1.0), per=per)
    check_graph(g, data)
@pytest.mark.parametrize("dtype,rows,cols", [(BF16, 64, 8192), (F32, 7, 333)])
def test_rmsnorm_rows(dtype, rows, cols):
    g, ins, _ = wl.rmsnorm_infer(rows, cols, dtype)
    data = _inputs(ins, 32, ("normal", 0.0, 1.0), per={"gamma": ("normal", 1.0, 0.02)})
    check_graph(g, data)
@pytest.mark.parametrize("layout", ["NCHW", "NHWC"])
@pytest.mark.parametrize("affine", [True, False])
def test_layernorm_4d_train(layout, affine):
    """Shapes of the reference's layernorm samples: f32 [2,3,32,32], mean / inv-variance outputs."""
    g = fz.Graph()
    g.setName("ln4d").setIODataType(F32).setComputeDataType(F32).setIntermediateDataType(F32)
    xd = [2, 3, 32, 32]
    sf = contiguousStride if layout == "NCHW" else channelsLastStride
    x = g.tensor(TensorAttr().setName("x").setDim(xd).setStride(sf(xd)))
    sc = bi = None
    ins = {"x": x}
    if affine:
        sc = g.tensor(TensorAttr().setName("scale").setDim([1, 3, 32, 32]).setStride(sf([1, 3, 32, 32])))
        bi = g.tensor(TensorAttr().setName("bias").setDim([1, 3, 32, 32]).setStride(sf([1, 3, 32, 32])))
        ins.update(scale=sc, bias=bi)
    eps = g.tensor(TensorAttr(1e-5).setName("eps"))
    y, m, v = g.layernorm(x, sc, bi, fz.LayernormAttr().setForwardPhase(fz.NormFwdPhase.TRAINING).setEpsilon(eps))
    for t in (y, m, v):
        t.setOutput(True)
    g.validate()
    check_graph(g, _inputs(ins, 33, ("normal", 0.5, 2.0)))
@pytest.mark.parametrize("dtype", [I32, F16, F32])
@pytest.mark.parametrize("mode", ["ADD", "SUM", "MIN", "MAX", "AMAX", "AVG", "NORM1", "NORM2", "MUL", "MUL_NO_ZEROS"])
def test_reduction_modes(dtype, mode):
    """The reference's reduction sample: [2,16,8,8] -> [2,16,1,1], ten modes x three dtypes."""
    if dtype == I32 and mode == "AVG":
        pytest.skip("AVG is rejected for integer tensors at validation")
    g = fz.Graph()
    g.setName("red").setIODataType(dtype).setComputeDataType(F32).setIntermediateDataType(dtype)
    xd = [2, 16, 8, 8]
    x = g.tensor(TensorAttr().setName("x").setDim(xd).setStride(contiguousStride(xd)))
    y = g.reduction(x, fz.ReductionAttr().setMode(ReductionMode[mode]))
    y.setDim([2, 16, 1, 1]).setStride([16, 1, 1, 1]).setName("y").setOutput(True)
    g.validate()
    rng = np.random.default_rng(41)
    if dtype == I32:
        if mode in ("MUL", "MUL_NO_ZEROS"):
            vals = rng.integers(-2, 3, 2 * 16 * 64)
            vals[rng.random(vals.size) < 0.7] = 1  # keep products inside int32
        else:
            vals = rng.integers(-50, 50, 2 * 16 * 64)
        data = {x: vals.astype(np.int32)}
    else:
        lo, hi = (0.8, 1.2) if mode.startswith("MUL") else (-2.0, 2.0)
        data = {x: make_input(x, rng, ("uniform", lo, hi))}
    if dtype == I32 and mode == "NORM2":
        from helpers import run_gpu
        from oracle import fusilli_oracle as orc
        got = run_gpu(g, data)[y].astype(np.int64)
        want = orc.execute(g, data)[y].astype(np.int64)
        assert np.all(np.abs(got - want) <= 1)  # the reference allows +-1 for integer sqrt
    else:
        check_graph(g, data)
@pytest.mark.parametrize("dtype,rows,cols", [(BF16, 128, 8192), (F32, 37, 2048), (F16, 16, 1000)])
def test_row_sum(dtype, rows, cols):
    g, ins, _ = wl.row_sum(rows, cols, dtype)
    check_graph(g, _inputs(ins, 42, ("normal", 0.0, 1.0)))
def test_reduction_leading_and_middle_dims():
    g = fz.Graph()
    g.setName("red2").setIODataType(F32).setComputeDataType(F32).setIntermediateDataType(F32)
    xd = [6, 5, 7, 9]
    x = g.tensor(TensorAttr().setName("x").setDim(xd).setStride(channelsLastStride(xd)))
    y = g.reduction(x, fz.ReductionAttr().setMode(ReductionMode.SUM))
    y.setDim([1, 5, 1, 9]).setStride([45, 9, 9, 1]).setName("y").setOutput(True)
    g.validate()
    check_graph(g, _inputs({"x": x}, 43))
_UNARY = ["ABS", "CEIL", "FLOOR", "NEG", "EXP", "ERF", "SIN", "TAN", "TANH_FWD", "SIGMOID_FWD", "RELU_FWD",
          "IDENTITY", "ELU_FWD", "GELU_FWD", "GELU_APPROX_TANH_FWD", "SOFTPLUS_FWD", "SWISH_FWD"]
_UNARY_POS = ["LOG", "SQRT", "RSQRT", "RECIPROCAL"]
_BINARY = ["ADD", "SUB", "MUL", "DIV", "MAX_OP", "MIN_OP", "ADD_SQUARE", "RELU_BWD", "TANH_BWD", "GELU_BWD",
           "GELU_APPROX_TANH_BWD", "SWISH_BWD"]
_CMP = ["CMP_EQ", "CMP_NEQ", "CMP_LT", "CMP_LE", "CMP_GT", "CMP_GE"]


def _pw_graph(mode, dtype, nin, second=None, dims=(2, 16, 64, 64)):
    g = fz.Graph()
    g.setName("pw_" + mode).setIODataType(dtype).setComputeDataType(F32).setIntermediateDataType(dtype)
    xd = list(dims)
    ts = {"in0": g.tensor(TensorAttr().setName("in0").setDim(xd).setStride(contiguousStride(xd)))}
    if nin >= 2:
        d1 = second or xd
        ts["in1"] = g.tensor(TensorAttr().setName("in1").setDim(d1).setStride(contiguousStride(d1)))
    attr = fz.PointwiseAttr().setMode(PointwiseMode[mode]).setEluAlpha(0.7).setSwishBeta(1.3)
    out = g.pointwise(*ts.values(), attr)
    out.setName("out").setOutput(True)
    g.validate()
    return g, ts, out


@pytest.mark.parametrize("mode", _UNARY + _UNARY_POS)
def test_pointwise_unary_f16(mode):
    g, ts, _ = _pw_graph(mode, F16, 1)
    dist = ("uniform", 0.2, 3.0) if mode in _UNARY_POS else ("uniform", -1.4, 1.4)
    check_graph(g, _inputs(ts, 51, dist))


@pytest.mark.parametrize("mode", _BINARY)
@pytest.mark.parametrize("dtype", [F16, F32])
def test_pointwise_binary_float(mode, dtype):
    g, ts, _ = _pw_graph(mode, dtype, 2)
    data = _inputs(ts, 52, ("uniform", -2.0, 2.0))
    if mode == "DIV":
        data[ts["in1"]] = make_input(ts["in1"], np.random.default_rng(5), ("uniform", 0.5, 2.0))
    check_graph(g, data)
@pytest.mark.parametrize("mode", ["ADD", "SUB", "MUL", "DIV", "MAX_OP", "MIN_OP"] + _CMP)
def test_pointwise_binary_int32_exact(mode):
    g, ts, _ = _pw_graph(mode, I32, 2, second=[1, 16, 1, 1])  # broadcast second operand
    data = _inputs(ts, 53)
    data[ts["in1"]] = np.array([13, -7, 3, 5, -2, 9, 11, -13, 4, 6, -5, 8, 1, -1, 2, 7], np.int32)
    check_graph(g, data)


@pytest.mark.parametrize("mode", ["ABS", "NEG", "RELU_FWD", "IDENTITY"])
def test_pointwise_unary_int32_exact(mode):
    g, ts, _ = _pw_graph(mode, I32, 1)
    check_graph(g, _inputs(ts, 54))


def test_pointwise_logical_and_select():
    g = fz.Graph()
    g.setName("pw_logic").setIODataType(F16).setComputeDataType(F32).setIntermediateDataType(F16)
    d = [2, 8, 16, 16]
    a = g.tensor(TensorAttr().setName("a").setDim(d).setStride(contiguousStride(d)))
    b = g.tensor(TensorAttr().setName("b").setDim(d).setStride(contiguousStride(d)))
    gt = g.pointwise(a, b, fz.PointwiseAttr().setMode(PointwiseMode.CMP_GT))
    lt0 = g.pointwise(a, g.tensor(TensorAttr(0.0).setName("zero")), fz.PointwiseAttr().setMode(PointwiseMode.CMP_LT))
    both = g.pointwise(gt, lt0, fz.PointwiseAttr().setMode(PointwiseMode.LOGICAL_OR))
    neg = g.pointwise(both, fz.PointwiseAttr().setMode(PointwiseMode.LOGICAL_NOT))
    sel = g.pointwise(neg, a, b, fz.PointwiseAttr().setMode(PointwiseMode.BINARY_SELECT))
    sel.setName("sel").setOutput(True)
    both.setName("both").setOutput(True)
    g.validate()
    check_graph(g, _inputs({"a": a, "b": b}, 55))
    assert g.getWorkspaceSize() > 0  # virtual booleans cross kernels through the workspace


def test_pointwise_transposed_operand_and_scalar():
    g = fz.Graph()
    g.setName("pw_tr").setIODataType(F32).setComputeDataType(F32).setIntermediateDataType(F32)
    a = g.tensor(TensorAttr().setName("a").setDim([48, 40]).setStride([40, 1]))
    b = g.tensor(TensorAttr().setName("b").setDim([48, 40]).setStride([1, 48]))  # stored transposed
    s = g.pointwise(a, b, fz.PointwiseAttr().setMode(PointwiseMode.ADD))
    o = g.pointwise(s, g.tensor(TensorAttr(2.5).setName("alpha")), fz.PointwiseAttr().setMode(PointwiseMode.MUL))
    o.setName("o").setOutput(True)
    g.validate()
    check_graph(g, _inputs({"a": a, "b": b}, 56))


# ---- multi-node graphs -----------------------------------------------------------------------
def test_wgrad_with_bias_gradient_in_one_graph():
    """The reference's wgrad sample also reduces dY to the bias gradient in the same graph."""
    n, c, h, w, k = 4, 16, 8, 8, 32
    g = fz.Graph()
    g.setName("wgrad_db").setIODataType(F32).setComputeDataType(F32).setIntermediateDataType(F32)
    dy = g.tensor(TensorAttr().setName("dy").setDim([n, k, h, w]).setStride(channelsLastStride([n, k, h, w])))
    x = g.tensor(TensorAttr().setName("x").setDim([n, c, h, w]).setStride(channelsLastStride([n, c, h, w])))
    dw = g.convWGrad(dy, x, fz.ConvWGradAttr().setPadding([0, 0]).setStride([1, 1]).setDilation([1, 1]))
    dw.setDim([k, c, 1, 1]).setName("dw").setOutput(True)
    db = g.reduction(dy, fz.ReductionAttr().setMode(ReductionMode.SUM))
    db.setDim([1, k, 1, 1]).setStride([k, 1, k, k]).setName("db").setOutput(True)
    g.validate()
    data = {dy: make_input(dy, np.random.default_rng(1), ("const", 1.0)),
            x: make_input(x, np.random.default_rng(1), ("const", 1.0))}
    got, _ = check_graph(g, data)
    assert np.all(got[dw] == n * h * w) and np.all(got[db] == n * h * w)  # closed form of the sample
    assert g.numLaunches() >= 2
