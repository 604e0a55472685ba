"""Host-side checks that need no GPU: the C-ABI library loads and exports every
symbol the header declares, plan building / artifact validation, front-end
validation and the execute() protocol errors the reference's unit tests pin."""
import ctypes
import json
import os
import re

import numpy as np
import pytest

import fusilli_b200 as fz
from fusilli_b200 import runtime
from fusilli_b200 import workloads as wl
from fusilli_b200.graph import (DataType, ErrorCode, FusilliError, PointwiseMode, ReductionMode, TensorAttr,
                                channelsLastStride, contiguousStride)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "fusilli_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(fb_[a-z0-9_]+)\s*\(", header))
    lib = ctypes.CDLL(runtime.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in fusilli_b200.h but not exported"
    bound = {n for n, _, _ in runtime.ABI_SYMBOLS}
    assert declared == bound, (declared - bound, bound - declared)
    assert runtime.lib().fb_abi_version() == 3


def test_status_codes_match_error_codes():
    header = open(os.path.join(ROOT, "include", "fusilli_b200.h")).read()
    for name, val in re.findall(r"FB_([A-Z_]+) = (\d+)", header):
        camel = "".join(p.capitalize() for p in name.split("_"))
        if camel == "Ok":
            camel = "OK"
        if hasattr(ErrorCode, camel):
            assert int(ErrorCode[camel]) == int(val)


def _has_gpu():
    return runtime.lib().fb_device_count() > 0


def test_no_cpu_execution_path():
    with pytest.raises(FusilliError) as e:
        fz.Handle.create(fz.Backend.CPU)
    assert e.value.code == ErrorCode.NotImplemented
    with pytest.raises(FusilliError) as e:
        fz.Handle.create(fz.Backend.CPU, 0, 1234)
    assert e.value.code == ErrorCode.InvalidArgument  # stream on a non-device backend (handle.h:96-98)
    if not _has_gpu():
        with pytest.raises(FusilliError) as e:
            fz.Handle.create(fz.Backend.CUDA)
        assert e.value.code == ErrorCode.RuntimeFailure
        assert "no CPU execution path" in e.value.message


def test_plan_build_fuses_conv_bias_relu_into_one_kernel():
    g, _, _ = wl.conv_fprop_bias_relu(2, 64, 16, 16, 64, 3, 3, 1, DataType.BFloat16)
    blob = g.compileToArtifact()
    assert runtime.lib().fb_plan_check(blob, len(blob)) == 0
    assert blob[:7] == b"FB2PLAN"


def test_artifact_is_deterministic_and_portable_between_graphs():
    g1, _, _ = wl.matmul_bias(2, 128, 128, 64)
    g2, _, _ = wl.matmul_bias(2, 128, 128, 64)
    assert g1.compileToArtifact() == g2.compileToArtifact()


@pytest.mark.parametrize("damage", ["magic", "version", "truncate", "flip", "trailing"])
def test_corrupt_artifacts_are_rejected(damage):
    g, _, _ = wl.row_sum(8, 64, DataType.Float)
    blob = bytearray(g.compileToArtifact())
    if damage == "magic":
        blob[0] ^= 0xFF
    elif damage == "version":
        blob[8] = 99
    elif damage == "truncate":
        blob = blob[:-5]
    elif damage == "flip":
        blob[len(blob) // 2] ^= 0x01
    else:
        blob += b"\0\0"
    lib = runtime.lib()
    assert lib.fb_plan_check(bytes(blob), len(blob)) == int(ErrorCode.RuntimeFailure)
    assert lib.fb_last_error()


def test_compile_requires_validation():
    g = fz.Graph()
    g.setName("nv").setIODataType(DataType.Float).setComputeDataType(DataType.Float)
    a = g.tensor(TensorAttr().setName("a").setDim([4, 4]).setStride([4, 1]))
    o = g.pointwise(a, fz.PointwiseAttr().setMode(PointwiseMode.RELU_FWD))
    o.setOutput(True)
    with pytest.raises(FusilliError) as e:
        g.compileToArtifact()
    assert e.value.code == ErrorCode.NotValidated
    assert e.value.message == "Graph must be validated before being compiled"


def test_execute_before_compile_is_not_compiled():
    g, ins, out = wl.row_sum(8, 64, DataType.Float)
    with pytest.raises(FusilliError) as e:
        g.execute(None, {}, None)
    assert e.value.code == ErrorCode.NotCompiled
    assert g.getWorkspaceSize() is None  # nullopt before load (runtime.h:317-327)


def test_unsupported_patterns_fail_at_build_time():
    g = fz.Graph()
    g.setName("f64").setIODataType(DataType.Double).setComputeDataType(DataType.Double)
    a = g.tensor(TensorAttr().setName("a").setDim([4, 4]).setStride([4, 1]))
    o = g.pointwise(a, fz.PointwiseAttr().setMode(PointwiseMode.RELU_FWD))
    o.setOutput(True)
    g.validate()
    with pytest.raises(FusilliError) as e:
        g.compileToArtifact()
    assert e.value.code == ErrorCode.NotImplemented

    g, _, _ = wl.sdpa_fwd(1, 2, 64, 64, DataType.Half, causal=False)
    g.nodes[0].attr.setDropout(0.1)
    with pytest.raises(FusilliError) as e:
        g.compileToArtifact()
    assert e.value.code == ErrorCode.NotImplemented


# ---- front-end behaviour pinned by the reference's unit tests ------------------------------
def test_auto_names_and_virtual_outputs():
    g = fz.Graph()
    g.setName("names").setIODataType(DataType.Half).setComputeDataType(DataType.Float).setIntermediateDataType(DataType.Float)
    x = g.tensor(TensorAttr().setDim([2, 8, 4, 4]).setStride(channelsLastStride([2, 8, 4, 4])))
    w = g.tensor(TensorAttr().setDim([8, 8, 1, 1]).setStride(channelsLastStride([8, 8, 1, 1])))
    y = g.convFProp(x, w, fz.ConvFPropAttr().setPadding([0, 0]).setStride([1, 1]).setDilation([1, 1]))
    assert (x.getName(), w.getName(), y.getName()) == ("conv_fprop_0_X", "conv_fprop_0_W", "conv_fprop_0_Y")
    assert y.isVirtual()
    r = g.pointwise(y, fz.PointwiseAttr().setMode(PointwiseMode.RELU_FWD))
    assert r.getName() == "pointwise_1_OUT_0"
    r.setOutput(True)
    assert not r.isVirtual()
    g.validate()
    assert y.getDim() == [2, 8, 4, 4] and y.getStride() == channelsLastStride([2, 8, 4, 4])
    assert y.getDataType() == DataType.Float and r.getDataType() == DataType.Half  # intermediate vs IO default


def test_validation_errors():
    g = fz.Graph()
    with pytest.raises(FusilliError) as e:
        g.validate()
    assert e.value.code == ErrorCode.AttributeNotSet and e.value.message == "Graph name not set"

    g = fz.Graph()
    g.setName("dup").setIODataType(DataType.Float).setComputeDataType(DataType.Float)
    a = g.tensor(TensorAttr().setName("t").setDim([4]).setStride([1]))
    b = g.tensor(TensorAttr().setName("t").setDim([4]).setStride([1]))
    g.pointwise(a, b, fz.PointwiseAttr().setMode(PointwiseMode.ADD)).setOutput(True)
    with pytest.raises(FusilliError) as e:
        g.validate()
    assert e.value.message == "Symbol name 't' already in use"

    g = fz.Graph()
    g.setName("mm").setIODataType(DataType.Float).setComputeDataType(DataType.Float)
    a = g.tensor(TensorAttr().setName("a").setDim([4, 8]).setStride([8, 1]))
    b = g.tensor(TensorAttr().setName("b").setDim([9, 4]).setStride([4, 1]))
    g.matmul(a, b, fz.MatmulAttr()).setOutput(True)
    with pytest.raises(FusilliError) as e:
        g.validate()
    assert e.value.code == ErrorCode.InvalidAttribute and "incompatible inner dimensions" in e.value.message

    g = fz.Graph()
    g.setName("red").setIODataType(DataType.Int32).setComputeDataType(DataType.Float)
    x = g.tensor(TensorAttr().setName("x").setDim([4, 8]).setStride([8, 1]))
    y = g.reduction(x, fz.ReductionAttr().setMode(ReductionMode.AVG))
    y.setDim([4, 1]).setStride([1, 1]).setOutput(True)
    with pytest.raises(FusilliError) as e:
        g.validate()
    assert "AVG is not supported for integral" in e.value.message

    g = fz.Graph()
    g.setName("sdpa").setIODataType(DataType.Half).setComputeDataType(DataType.Float)
    q = g.tensor(TensorAttr().setName("q").setDim([1, 8, 16, 32]).setStride(contiguousStride([1, 8, 16, 32])))
    k = g.tensor(TensorAttr().setName("k").setDim([1, 3, 16, 32]).setStride(contiguousStride([1, 3, 16, 32])))
    v = g.tensor(TensorAttr().setName("v").setDim([1, 3, 16, 32]).setStride(contiguousStride([1, 3, 16, 32])))
    g.sdpa(q, k, v, None, fz.SdpaAttr().setEnableGqa(True)).setOutput(True)
    with pytest.raises(FusilliError) as e:
        g.validate()
    assert "multiple of K heads" in e.value.message

    g = fz.Graph()
    g.setName("rms").setIODataType(DataType.Float).setComputeDataType(DataType.Float)
    x = g.tensor(TensorAttr().setName("x").setDim([2, 8]).setStride([8, 1]))
    eps = g.tensor(TensorAttr(1e-5).setName("eps"))
    g.rmsnorm(x, None, fz.RmsnormAttr().setForwardPhase(fz.NormFwdPhase.TRAINING).setEpsilon(eps))
    with pytest.raises(FusilliError) as e:
        g.validate()
    assert e.value.code == ErrorCode.NotImplemented


def test_tensor_layout_algebra():
    t = TensorAttr().setDim([2, 3, 4, 5]).setStride([60, 1, 15, 3])
    assert t.isChannelsLast() and not t.isContiguous()
    assert t.getPhysicalDim() == [2, 4, 5, 3]
    assert t.getLogicalToPhysicalPermuteOrder() == [0, 2, 3, 1]
    b = TensorAttr().setDim([8, 2, 64, 128]).setStride([0, 0, 128, 1])
    assert b.hasBroadcastDims() and b.getPhysicalDim() == [1, 1, 64, 128]
    assert not TensorAttr().setDim([2, 3]).setStride([4, 1]).hasValidPhysicalRepresentation()
    assert fz.graph.computeBroadcastShape([[64, 16, 1, 1], [1, 32, 1]]) == [64, 16, 32, 1]
    assert fz.graph.getConvInferredOutputShape([16, 64, 56, 56], [64, 64, 3, 3], [1, 1], [1, 1], [1, 1]) == [16, 64, 56, 56]


def _int4_graph(as_pointwise_input=False, as_output=False):
    g = fz.Graph()
    g.setName("int4_host").setIODataType(DataType.Half).setComputeDataType(DataType.Float)
    g.setIntermediateDataType(DataType.Float)
    a = g.tensor(TensorAttr().setName("a").setDim([1, 4, 8]).setStride([32, 8, 1]).setDataType(DataType.Int4))
    if as_pointwise_input:
        o = g.pointwise(a, fz.PointwiseAttr().setMode(PointwiseMode.RELU_FWD))
    else:
        b = g.tensor(TensorAttr().setName("b").setDim([1, 8, 4]).setStride([32, 4, 1]))
        o = g.matmul(a, b, fz.MatmulAttr().setName("mm"))
    o.setName("o").setOutput(True)
    if as_output:
        o.setDataType(DataType.Int4)
    g.validate()
    return g


def test_int4_is_a_matmul_operand_and_nothing_else():
    """Int4 x f16 matmul builds a plan (reference samples/matmul/matmul_int4_fp16.cpp); every other
    use of the sub-byte type is refused when the plan is built."""
    blob = _int4_graph().compileToArtifact()
    assert runtime.lib().fb_plan_check(blob, len(blob)) == 0
    for kwargs in (dict(as_pointwise_input=True), dict(as_output=True)):
        with pytest.raises(FusilliError) as e:
            _int4_graph(**kwargs).compileToArtifact()
        assert e.value.code == ErrorCode.NotImplemented
        assert "si4" in e.value.message


def test_mixed_precision_matmul_needs_rank_3_and_equal_batch():
    g = fz.Graph()
    g.setName("int4_rank2").setIODataType(DataType.Half).setComputeDataType(DataType.Float)
    a = g.tensor(TensorAttr().setName("a").setDim([4, 8]).setStride([8, 1]).setDataType(DataType.Int4))
    b = g.tensor(TensorAttr().setName("b").setDim([8, 4]).setStride([4, 1]))
    g.matmul(a, b, fz.MatmulAttr().setName("mm")).setOutput(True)
    with pytest.raises(FusilliError) as e:
        g.validate()
    assert e.value.code == ErrorCode.InvalidAttribute
    assert "Mixed precision matmul is only supported when input tensors A and B are of rank 3" in e.value.message


def test_matmul_batch_broadcast_by_a_divisor_builds_a_plan():
    """The reference's validation lets a batch dim divide the other operand's (matmul_node.h:140-150);
    the plan accepts it (the smaller operand is read modulo its batch extent) and the result has the
    larger batch."""
    g = fz.Graph()
    g.setName("mm_divisor").setIODataType(DataType.Float).setComputeDataType(DataType.Float)
    g.setIntermediateDataType(DataType.Float)
    a = g.tensor(TensorAttr().setName("a").setDim([4, 8, 16]).setStride([128, 16, 1]))
    b = g.tensor(TensorAttr().setName("b").setDim([2, 16, 8]).setStride([128, 8, 1]))
    c = g.matmul(a, b, fz.MatmulAttr().setName("mm"))
    c.setName("c").setOutput(True)
    g.validate()
    assert c.dim == [4, 8, 8]
    assert runtime.lib().fb_plan_check(g.compileToArtifact(), len(g.compileToArtifact())) == 0


def test_norm_on_a_batch_inner_or_padded_tensor_is_refused_at_plan_build():
    """The row kernels walk a sample as one dense run of prod(dims[1:]) elements. The front ends only
    admit contiguous or channels-last tensors; a graph that reaches the C ABI with another layout (here:
    strides changed after validation) is refused when the plan is built, not run on the wrong bytes."""
    for strides in ([1, 64], [1024 + 8, 1]):   # batch innermost; padded rows
        g, ins, y = wl.rmsnorm_infer(64, 1024, DataType.Float)
        ins["x"].stride = list(strides)
        with pytest.raises(FusilliError) as e:
            g.compileToArtifact()
        assert e.value.code == ErrorCode.NotImplemented
        assert "dense with the batch dim outermost" in e.value.message
