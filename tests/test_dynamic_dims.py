"""Dynamic dims (TensorAttr::setDynamicDims, reference tensor_attributes.h:71-84, 512-570): one plan,
built for representative extents, executed with the extents of each call's buffers.

Reference behaviour being reproduced: samples/dynamic_shapes/conv_fprop_dynamic_batch.cpp (one
compile, runtime batch 1, 2, 4), sdpa_basic_dynamic_sequence.cpp (runtime sequence 16, 32, 64) and
reduction_min_max_dynamic_batch.cpp. CPU tests check the shape derivation without a device: the plan
specialised for extents E must be byte-identical to the plan built from a graph declared with E.
GPU tests compare each runtime shape with the oracle run on a static graph of that shape.
"""
import ctypes

import numpy as np
import pytest

import fusilli_b200 as fz
from fusilli_b200 import runtime, workloads as wl
from fusilli_b200.graph import (DataType, ErrorCode, FusilliError, PointwiseAttr, ReductionAttr, TensorAttr,
                                contiguousStride)
from oracle import fusilli_oracle as orc

import helpers as H

FB_MAX_RANK = runtime.FB_MAX_RANK


def flag_dynamic(graph, axis, static=(), revalidate=True):
    """Marks `axis` dynamic on every tensor of the graph (virtual ones too) except `static` names
    and scalars, then validates again (not for a comparison twin, whose extent may be 1, which
    validation only accepts as a runtime extent, not as a representative one)."""
    for t in graph.inputs + graph.outputs:
        if t.isScalar() or t.name in static or len(t.dim) <= axis:
            continue
        t.setDynamicDim(axis)
    if revalidate:
        graph.validate()
    return graph


def reduction_min(n, dtype=DataType.Int32):
    """x [n,16,8,8] -> min over the two inner dims (the reference's dynamic reduction sample)."""
    g = fz.Graph()
    g.setName("dyn_min").setIODataType(dtype).setComputeDataType(dtype).setIntermediateDataType(dtype)
    xd, yd = [n, 16, 8, 8], [n, 16, 1, 1]
    x = g.tensor(TensorAttr().setName("x").setDim(xd).setStride(contiguousStride(xd)))
    y = g.reduction(x, ReductionAttr().setMode(ReductionAttr.Mode.MIN).setName("min"))
    y.setName("y").setDim(yd).setStride(contiguousStride(yd)).setOutput(True)
    g.validate()
    return g, {"x": x}, y


def add_bias_rows(n, dtype=DataType.Float):
    """x [n,32,6] + bias [1,32,1] -> relu, two standalone pointwise kernels with a virtual between."""
    g = fz.Graph()
    g.setName("dyn_pw").setIODataType(dtype).setComputeDataType(DataType.Float).setIntermediateDataType(dtype)
    xd = [n, 32, 6]
    x = g.tensor(TensorAttr().setName("x").setDim(xd).setStride(contiguousStride(xd)))
    b = g.tensor(TensorAttr().setName("bias").setDim([1, 32, 1]).setStride([32, 1, 1]))
    s = g.pointwise(x, b, PointwiseAttr().setMode(PointwiseAttr.Mode.ADD).setName("add"))
    e = g.pointwise(s, PointwiseAttr().setMode(PointwiseAttr.Mode.EXP).setName("exp"))
    y = g.pointwise(e, s, PointwiseAttr().setMode(PointwiseAttr.Mode.MUL).setName("mul"))
    y.setName("y").setOutput(True)
    g.validate()
    return g, {"x": x, "bias": b}, y


# (id, builder(extent), dynamic axis, names that stay static, representative, runtime extents)
CASES = [
    ("conv_nchw_batch_f16", lambda n: _conv_nchw(n), 0, ("w",), 4, [1, 2, 4]),
    ("conv_nhwc_bias_relu_batch_bf16",
     lambda n: wl.conv_fprop_bias_relu(n, 64, 16, 16, 64, 3, 3, 1, DataType.BFloat16), 0, ("w", "bias"), 8, [1, 3, 8]),
    ("conv_nhwc_height_bf16",
     lambda h: wl.conv_fprop_bias_relu(2, 64, h, 16, 128, 3, 3, 1, DataType.BFloat16), 2, ("w", "bias"), 16, [8, 12, 16]),
    ("conv_f32_batch", lambda n: wl.conv_fprop_bias_relu(n, 16, 9, 9, 24, 3, 3, 1, DataType.Float), 0, ("w", "bias"),
     4, [1, 2, 4]),
    ("dgrad_batch_bf16", lambda n: wl.conv_dgrad(n, 64, 14, 14, 64, 3, 3, 1), 0, ("w",), 8, [2, 5, 8]),
    ("wgrad_batch_bf16", lambda n: wl.conv_wgrad(n, 64, 14, 14, 64, 3, 3, 1), 0, ("dw",), 8, [2, 5, 8]),
    ("matmul_rows_bf16", lambda m: wl.matmul_bias(2, m, 256, 128), 1, ("b", "bias"), 512, [128, 200, 512]),
    ("matmul_batch_f32", lambda b: wl.matmul_bias(b, 48, 40, 24, DataType.Float), 0, ("bias",), 4, [2, 3, 4]),
    ("sdpa_sequence_f16", lambda s: wl.sdpa_fwd(1, 8, s, 64, DataType.Half, causal=False), 2, (), 64, [16, 32, 64]),
    ("sdpa_sequence_causal_bf16", lambda s: wl.sdpa_fwd(2, 4, s, 128, DataType.BFloat16, causal=True), 2, (), 512,
     [128, 320, 512]),
    ("layernorm_rows_train", lambda r: wl.layernorm_infer(r, 512, train=True), 0, ("gamma", "beta"), 64, [8, 33, 64]),
    ("rmsnorm_rows", lambda r: wl.rmsnorm_infer(r, 1024), 0, ("gamma",), 64, [8, 33, 64]),
    ("rowsum_rows", lambda r: wl.row_sum(r, 384), 0, (), 64, [8, 33, 64]),
    ("reduction_min_batch_i32", lambda n: reduction_min(n), 0, (), 2, [1, 2, 5]),
    ("batchnorm_train_batch_nhwc", lambda n: wl.batchnorm_fwd(n, 32, [6, 5], DataType.Float, train=True,
                                                               channels_last=True, running=False),
     0, ("gamma", "beta", "saved_mean", "saved_inv_var"), 8, [2, 5, 8]),
    ("pointwise_chain_batch", lambda n: add_bias_rows(n), 0, ("bias",), 6, [1, 4, 6]),
]


def _conv_nchw(n):
    """The reference's dynamic-batch sample: NCHW image, KCRS filter, 1x1, f16."""
    g = fz.Graph()
    g.setName("dyn_conv_nchw").setIODataType(DataType.Half).setComputeDataType(DataType.Float)
    g.setIntermediateDataType(DataType.Float)
    xd, wd = [n, 4, 4, 4], [4, 4, 1, 1]
    x = g.tensor(TensorAttr().setName("x").setDim(xd).setStride(contiguousStride(xd)))
    w = g.tensor(TensorAttr().setName("w").setDim(wd).setStride(contiguousStride(wd)))
    y = g.convFProp(x, w, fz.ConvFPropAttr().setPadding([0, 0]).setStride([1, 1]).setDilation([1, 1]).setName("conv"))
    y.setName("y").setOutput(True)
    g.validate()
    return g, {"x": x, "w": w}, y


def _arg_dims(dynamic_graph, static_graph):
    """Row-per-argument logical dims of `static_graph`'s tensors in `dynamic_graph`'s argument order."""
    by_name = {t.name: t for t in static_graph.inputs + static_graph.outputs}
    _, args, _keep = dynamic_graph._flatten()
    dims = (ctypes.c_int64 * (len(args) * FB_MAX_RANK))(*([1] * (len(args) * FB_MAX_RANK)))
    for i, t in enumerate(args):
        for k, v in enumerate(by_name[t.name].dim):
            dims[i * FB_MAX_RANK + k] = v
    return dims, len(args)


def _specialize(blob, dims, n):
    lib = runtime.lib()
    out = ctypes.POINTER(ctypes.c_uint8)()
    size = ctypes.c_size_t()
    st = lib.fb_plan_specialize(blob, len(blob), dims, n, ctypes.byref(out), ctypes.byref(size))
    if st != 0:
        return st, (lib.fb_last_error() or b"").decode()
    data = ctypes.string_at(out, size.value)
    lib.fb_bytes_free(out)
    return 0, data


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_specialised_plan_equals_plan_built_for_that_shape(case):
    _, build, axis, static, rep, extents = case
    base = flag_dynamic(build(rep)[0], axis, static)
    blob = base.compileToArtifact()
    assert runtime.lib().fb_plan_check(blob, len(blob)) == 0
    for e in extents:
        twin = flag_dynamic(build(e)[0], axis, static, revalidate=False)
        dims, n = _arg_dims(base, twin)
        st, got = _specialize(blob, dims, n)
        assert st == 0, got
        assert got == twin.compileToArtifact(), f"extent {e}"


def test_static_dim_mismatch_and_wrong_output_shape_are_refused():
    base = flag_dynamic(wl.conv_fprop_bias_relu(8, 64, 16, 16, 64, 3, 3, 1, DataType.BFloat16)[0], 0, ("w", "bias"))
    blob = base.compileToArtifact()
    twin = wl.conv_fprop_bias_relu(4, 64, 16, 16, 64, 3, 3, 1, DataType.BFloat16)[0]
    dims, n = _arg_dims(base, twin)
    _, args, _keep = base._flatten()
    names = [t.name for t in args]
    # a static dim (image width) that differs from the plan's
    bad = (ctypes.c_int64 * len(dims))(*dims)
    bad[names.index("x") * FB_MAX_RANK + 3] = 20
    st, msg = _specialize(blob, bad, n)
    assert st == int(ErrorCode.InvalidArgument) and "static" in msg
    # an output buffer whose batch is not the input's
    bad = (ctypes.c_int64 * len(dims))(*dims)
    bad[names.index("y") * FB_MAX_RANK + 0] = 3
    st, msg = _specialize(blob, bad, n)
    assert st == int(ErrorCode.InvalidArgument) and "imply" in msg
    # a zero extent
    bad = (ctypes.c_int64 * len(dims))(*dims)
    bad[names.index("x") * FB_MAX_RANK + 0] = 0
    st, msg = _specialize(blob, bad, n)
    assert st == int(ErrorCode.InvalidArgument)
    # wrong number of buffers
    st, msg = _specialize(blob, dims, n - 1)
    assert st == int(ErrorCode.VariantPackError)


def test_unflagged_dependent_tensor_is_refused_not_overrun():
    # y depends on the batch but is not marked: the concrete shapes disagree and nothing is lowered
    g, _, _ = wl.conv_fprop_bias_relu(8, 64, 16, 16, 64, 3, 3, 1, DataType.BFloat16, bias=False, relu=False)
    next(t for t in g.inputs if t.name == "x").setDynamicDim(0)
    g.validate()
    blob = g.compileToArtifact()
    twin = wl.conv_fprop_bias_relu(4, 64, 16, 16, 64, 3, 3, 1, DataType.BFloat16, bias=False, relu=False)[0]
    dims, n = _arg_dims(g, twin)
    _, args, _keep = g._flatten()
    yi = [t.name for t in args].index("y")
    dims[yi * FB_MAX_RANK] = 8  # the static extent the plan holds for y
    st, msg = _specialize(blob, dims, n)
    assert st == int(ErrorCode.InvalidArgument) and "batch" in msg


def test_sdpa_key_value_lengths_must_agree():
    g = flag_dynamic(wl.sdpa_fwd(1, 8, 64, 64, DataType.Half, causal=False)[0], 2)
    blob = g.compileToArtifact()
    twin = wl.sdpa_fwd(1, 8, 32, 64, DataType.Half, causal=False)[0]
    dims, n = _arg_dims(g, twin)
    _, args, _keep = g._flatten()
    vi = [t.name for t in args].index("v")
    dims[vi * FB_MAX_RANK + 2] = 48
    st, msg = _specialize(blob, dims, n)
    assert st == int(ErrorCode.InvalidArgument) and "key and value" in msg


def test_tensor_validation_of_dynamic_dims():
    def tensor():
        return TensorAttr().setName("t").setDataType(DataType.Float).setDim([4, 1, 8]).setStride([8, 8, 1])
    t = tensor().setDynamicDims([2, 0, 2])
    assert t.getDynamicDims() == [0, 2] and t.isDynamicDim(2) and not t.isDynamicDim(1)
    t.validate()
    with pytest.raises(FusilliError) as e:
        tensor().setDynamicDim(3).validate()
    assert "has dynamic dim index 3 out of range for rank 3" in e.value.message
    with pytest.raises(FusilliError) as e:
        tensor().setDynamicDim(1).validate()
    assert "with representative size 1" in e.value.message
    with pytest.raises(FusilliError) as e:
        tensor().setStride([8, 8, 0]).setDynamicDim(2).validate()
    assert "with stride 0 (broadcast stride)" in e.value.message
    with pytest.raises(FusilliError) as e:
        tensor().setStride([0, 8, 1]).setDynamicDim(2).validate()
    assert "dynamic dimensions on a tensor with broadcast strides" in e.value.message
    assert not tensor().setDynamicDim(0).clearDynamicDims().hasDynamicDims()


# ---- on the device ---------------------------------------------------------------

def _run_extent(handle, dyn, ws_buf, ws_rep, build, extent, rng, seed_dist):
    twin, ins, _ = build(extent)
    inputs = {t: H.make_input(t, rng, seed_dist) for t in ins.values()}
    want = orc.execute(twin, inputs)
    by_name = {t.name: t for t in dyn.inputs + dyn.outputs}
    pack, outs = {}, {}
    for t, arr in inputs.items():
        pack[by_name[t.name]] = fz.Buffer.allocate(handle, t.getPhysicalDim(), arr)
    for t in twin.outputs:
        if t.isVirtual():
            continue
        init = np.zeros(t.physicalVolume(), dtype=orc.NP_DTYPE[t.dataType])
        pack[by_name[t.name]] = fz.Buffer.allocate(handle, t.getPhysicalDim(), init)
        outs[t] = pack[by_name[t.name]]
    assert dyn.getWorkspaceSizeFor(pack) <= ws_rep
    dyn.execute(handle, pack, ws_buf)
    for t, b in outs.items():
        H.compare(b.read(handle, orc.NP_DTYPE[t.dataType]), want[t], t.dataType, f"{t.name} at extent {extent}")
    assert handle.kernelError() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_one_plan_many_shapes(case):
    name, build, axis, static, rep, extents = case
    dyn = flag_dynamic(build(rep)[0], axis, static)
    handle = fz.Handle.create(fz.Backend.CUDA)
    dyn.compile(handle)
    ws_rep = dyn.getWorkspaceSize()
    ws_buf = fz.Buffer.allocateRaw(handle, ws_rep) if ws_rep else None
    rng = np.random.default_rng(0x5EED + len(name))
    dist = ("uniform", -1.0, 1.0) if "sdpa" not in name else ("normal", 0.0, 1.0)
    # every extent twice, in two orders: the second pass is served from the plan's shape cache
    for e in extents + extents[::-1]:
        _run_extent(handle, dyn, ws_buf, ws_rep, build, e, rng, dist)


@pytest.mark.gpu
def test_dynamic_plan_runs_unshaped_at_its_representative_extent():
    # fb_plan_execute (no shapes) on a dynamic plan = the representative shape
    g, ins, y = wl.layernorm_infer(64, 512)
    flag_dynamic(g, 0, ("gamma", "beta"))
    rng = np.random.default_rng(7)
    inputs = {t: H.make_input(t, rng) for t in ins.values()}
    handle = fz.Handle.create(fz.Backend.CUDA)
    g.compile(handle)
    assert g.getWorkspaceSize() == 0
    pack = {t: fz.Buffer.allocate(handle, t.getPhysicalDim(), arr) for t, arr in inputs.items()}
    out_t = y[0]
    pack[out_t] = fz.Buffer.allocate(handle, out_t.getPhysicalDim(),
                                     np.zeros(out_t.physicalVolume(), orc.NP_DTYPE[out_t.dataType]))
    n = len(g._arg_tensors)
    ptrs = (ctypes.c_void_p * n)(*[pack[t].ptr() for t in g._arg_tensors])
    sizes = (ctypes.c_size_t * n)(*[pack[t].size() for t in g._arg_tensors])
    assert runtime.lib().fb_plan_execute(g._plan, handle._ptr, ptrs, sizes, n, None, 0) == 0
    ref = orc.execute(g, inputs)
    H.compare(pack[out_t].read(handle, orc.NP_DTYPE[out_t.dataType]), ref[out_t], out_t.dataType, "y")


@pytest.mark.gpu
def test_buffer_without_shape_and_short_buffer_are_refused():
    g, ins, y = wl.rmsnorm_infer(64, 1024)
    flag_dynamic(g, 0, ("gamma",))
    handle = fz.Handle.create(fz.Backend.CUDA)
    g.compile(handle)
    g.getWorkspaceSize()
    x, gamma = ins["x"], ins["gamma"]
    xb = fz.Buffer.allocate(handle, [16, 1024], np.zeros(16 * 1024, np.uint16))
    gb = fz.Buffer.allocate(handle, [1, 1024], np.ones(1024, np.float32))
    raw = fz.Buffer.allocateRaw(handle, 16 * 1024 * 2)
    with pytest.raises(FusilliError) as e:
        g.execute(handle, {x: xb, gamma: gb, y: raw}, None)
    assert e.value.code == ErrorCode.InvalidArgument and "carries no shape" in e.value.message
    # an output declared as 16 rows but backed by 8 rows of memory
    short = fz.Buffer.allocateRaw(handle, 8 * 1024 * 2)
    short.shape = [16, 1024]
    with pytest.raises(FusilliError) as e:
        g.execute(handle, {x: xb, gamma: gb, y: short}, None)
    assert e.value.code == ErrorCode.InvalidArgument and "needs" in e.value.message


@pytest.mark.gpu
def test_workspace_of_the_representative_shape_bounds_larger_shapes():
    # exp(x + bias) * (x + bias): the sum crosses kernels through the workspace
    g = flag_dynamic(add_bias_rows(4)[0], 0, ("bias",))
    handle = fz.Handle.create(fz.Backend.CUDA)
    g.compile(handle)
    ws_rep = g.getWorkspaceSize()
    assert ws_rep > 0
    ws = fz.Buffer.allocateRaw(handle, ws_rep)
    big, ins, y = add_bias_rows(64)
    by_name = {t.name: t for t in g.inputs + g.outputs}
    pack = {by_name[t.name]: fz.Buffer.allocate(handle, t.getPhysicalDim(), np.zeros(t.physicalVolume(), np.float32))
            for t in list(ins.values()) + [y]}
    assert g.getWorkspaceSizeFor(pack) > ws_rep
    with pytest.raises(FusilliError) as e:
        g.execute(handle, pack, ws)
    assert e.value.code == ErrorCode.InvalidArgument and "Workspace buffer too small" in e.value.message


@pytest.mark.gpu
def test_shape_cache_eviction_under_concurrent_callers():
    """More distinct shapes than the per-plan cache holds (64), from several threads at once: a caller
    keeps its specialised plan alive while another thread's new shape drops the cached set, so every
    query returns the size a fresh specialisation of that shape gives (ctypes releases the GIL: the
    calls really overlap)."""
    import threading
    g, ins, y = wl.rmsnorm_infer(64, 1024)
    flag_dynamic(g, 0, ("gamma",))
    handle = fz.Handle.create(fz.Backend.CUDA)
    g.compile(handle)
    lib = runtime.lib()
    n = len(g._arg_tensors)
    names = [t.name for t in g._arg_tensors]
    errors = []

    def dims_for(rows):
        d = (ctypes.c_int64 * (n * 8))(*([1] * (n * 8)))
        for i, t in enumerate(g._arg_tensors):
            logical = list(t.dim)
            if t.hasDynamicDims():
                logical[0] = rows
            for k, v in enumerate(logical):
                d[i * 8 + k] = v
        return d

    def worker(seed):
        rng = np.random.default_rng(seed)
        for _ in range(400):
            rows = int(rng.integers(1, 200))
            out = ctypes.c_size_t(12345)
            st = lib.fb_plan_workspace_size_shaped(g._plan, dims_for(rows), n, ctypes.byref(out))
            if st != 0 or out.value != 0:   # a row norm needs no workspace at any batch size
                errors.append((rows, st, out.value))

    threads = [threading.Thread(target=worker, args=(s,)) for s in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:5]
    assert names  # the plan is still usable afterwards
    assert g.getWorkspaceSize() == 0
