"""fb_conv_wgrad_static: the weight-gradient entry point for callers that cannot
allocate (allocator hooks, no-allocation real-time loops, plugins that only get raw
pointers and a stream). Its split-reduction scratch is a fixed array inside the
library instead of a caller-provided workspace.

Checked against the CPU oracle AND against the existing planned path
(Graph.compile/execute with a workspace) on the same bytes, on two calls in a row so
the second call runs over whatever the first left in the shared array. Collected last
on purpose."""
import ctypes

import numpy as np
import pytest

import fusilli_b200 as fz
from fusilli_b200 import runtime
from fusilli_b200.graph import DataType, ErrorCode, TensorAttr, channelsLastStride
from helpers import compare, graph_traits, make_input, run_gpu
from oracle import fusilli_oracle as orc


def test_static_entry_point_is_exported_and_sized():
    lib = runtime.lib()
    assert lib.fb_conv_wgrad_static_scratch_bytes() == 8 << 20


def _wgrad_graph(dtype, n, c, h, w, k, r, s, pad, stride, groups):
    g = fz.Graph()
    g.setName("wgrad_static_ref").setIODataType(dtype).setComputeDataType(DataType.Float).setIntermediateDataType(dtype)
    p = 1 + (h + 2 * pad - (r - 1) - 1) // stride
    q = 1 + (w + 2 * pad - (s - 1) - 1) // stride
    dy = g.tensor(TensorAttr().setName("dy").setDim([n, k, p, q]).setStride(channelsLastStride([n, k, p, q])))
    x = g.tensor(TensorAttr().setName("x").setDim([n, c, h, w]).setStride(channelsLastStride([n, c, h, w])))
    dw = g.convWGrad(dy, x, fz.ConvWGradAttr().setPadding([pad, pad]).setStride([stride, stride]).setDilation([1, 1]))
    dw.setName("dw").setDim([k, c // groups, r, s]).setOutput(True)
    g.validate()
    return g, dy, x, dw


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,shape", [
    # n, c, h, w, k, r, s, pad, stride, groups
    (DataType.BFloat16, (8, 64, 28, 28, 64, 3, 3, 1, 1, 1)),   # split reduction through the static array
    (DataType.Float, (4, 32, 14, 14, 48, 1, 1, 0, 1, 1)),
    (DataType.Float, (4, 16, 8, 8, 32, 1, 1, 0, 2, 4)),       # the reference's grouped, strided wgrad sample geometry
    (DataType.Half, (6, 32, 17, 17, 48, 3, 3, 1, 2, 2)),      # grouped + stride 2 + padding, odd extent
])
def test_static_wgrad_matches_oracle_and_planned_path_twice(dtype, shape):
    n, c, h, w, k, r, s, pad, stride, groups = shape
    g, dy_t, x_t, dw_t = _wgrad_graph(dtype, n, c, h, w, k, r, s, pad, stride, groups)
    rng = np.random.default_rng(99)
    data = {dy_t: make_input(dy_t, rng, ("normal", 0.0, 0.1)), x_t: make_input(x_t, rng, ("normal", 0.0, 0.5))}
    want = orc.execute(g, data)[dw_t]                 # the CPU oracle
    acc_len, chained = graph_traits(g)
    handle = fz.Handle.create(fz.Backend.CUDA)
    planned = run_gpu(g, data, handle)[dw_t]           # existing entry point (workspace scratch)
    compare(planned, want, dtype, "planned path vs oracle", acc_len, chained)

    lib = runtime.lib()
    dy = fz.Buffer.allocate(handle, [data[dy_t].size], data[dy_t])
    x = fz.Buffer.allocate(handle, [data[x_t].size], data[x_t])
    np_dt = want.dtype
    for call in range(2):
        out = fz.Buffer.allocate(handle, [want.size], np.full(want.size, 0x7F7F if np_dt == np.uint16 else 3.0, np_dt))
        st = lib.fb_conv_wgrad_static(ctypes.c_void_p(handle.stream()), dy.ptr(), x.ptr(), out.ptr(), int(dtype),
                                      n, c, h, w, k, r, s, pad, pad, stride, stride, 1, 1, groups)
        assert st == 0, lib.fb_last_error().decode()
        got = out.read(handle, np_dt)
        compare(got, want, dtype, f"static entry point vs oracle, call {call}", acc_len, chained)
        compare(got, planned, dtype, f"static entry point vs planned path, call {call}", acc_len, chained)


@pytest.mark.gpu
def test_static_wgrad_rejects_oversized_filter_gradient():
    lib = runtime.lib()
    handle = fz.Handle.create(fz.Backend.CUDA)
    buf = fz.Buffer.allocateRaw(handle, 1024)
    # 2048 x 2048 x 3 x 3 fp32 partials = 144 MiB > 8 MiB: must be refused before any launch
    st = lib.fb_conv_wgrad_static(None, buf.ptr(), buf.ptr(), buf.ptr(), int(DataType.Float),
                                  1, 2048, 8, 8, 2048, 3, 3, 1, 1, 1, 1, 1, 1, 1)
    assert st == int(ErrorCode.InvalidArgument)
    assert b"static scratch" in lib.fb_last_error()
