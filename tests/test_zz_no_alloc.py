"""fb_conv_wgrad_static: the weight-gradient entry point for callers that cannot
allocate (allocator hooks, no-allocation real-time loops, plugins that only get raw
pointers and a stream). Its split-reduction scratch is a fixed array inside the
library instead of a caller-provided workspace.

Checked against the existing planned path (Graph.compile/execute with a workspace)
on the same bytes, on two calls in a row so the second call runs over whatever the
first left in the shared array. Collected last on purpose."""
import ctypes

import numpy as np
import pytest

import fusilli_b200 as fz
from fusilli_b200 import runtime
from fusilli_b200 import workloads as wl
from fusilli_b200.graph import DataType, ErrorCode
from helpers import compare, make_input, run_gpu


def test_static_entry_point_is_exported_and_sized():
    lib = runtime.lib()
    assert lib.fb_conv_wgrad_static_scratch_bytes() == 8 << 20


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,shape", [
    (DataType.BFloat16, (8, 64, 28, 28, 64, 3, 3, 1)),   # split reduction through the static array
    (DataType.Float, (4, 32, 14, 14, 48, 1, 1, 0)),
])
def test_static_wgrad_matches_planned_path_twice(dtype, shape):
    n, c, h, w, k, r, s, pad = shape
    g, ins, dw_t = wl.conv_wgrad(n, c, h, w, k, r, s, pad, dtype)
    rng = np.random.default_rng(99)
    data = {ins["dy"]: make_input(ins["dy"], rng, ("normal", 0.0, 0.1)),
            ins["x"]: make_input(ins["x"], rng, ("normal", 0.0, 0.5))}
    handle = fz.Handle.create(fz.Backend.CUDA)
    want = run_gpu(g, data, handle)[dw_t]           # existing entry point (workspace scratch)

    lib = runtime.lib()
    dy = fz.Buffer.allocate(handle, [data[ins["dy"]].size], data[ins["dy"]])
    x = fz.Buffer.allocate(handle, [data[ins["x"]].size], data[ins["x"]])
    np_dt = want.dtype
    for call in range(2):
        out = fz.Buffer.allocate(handle, [want.size], np.full(want.size, 0x7F7F if np_dt == np.uint16 else 3.0, np_dt))
        st = lib.fb_conv_wgrad_static(ctypes.c_void_p(handle.stream()), dy.ptr(), x.ptr(), out.ptr(), int(dtype),
                                      n, c, h, w, k, r, s, pad, pad, 1, 1, 1, 1, 1)
        assert st == 0, lib.fb_last_error().decode()
        got = out.read(handle, np_dt)
        compare(got, want, dtype, f"call {call}", scale_atol=0.5)


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
