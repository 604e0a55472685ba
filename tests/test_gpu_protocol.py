"""Device-side protocol of the boundary on a real GPU: execute() guards and error codes
(reference include/fusilli/backend/runtime.h:389-491, tests/test_graph.cpp), artifact
round trips between graphs, external stream + imported device pointers (the pattern of
the reference's tests/hip_tests), buffer checks (tests/test_buffer.cpp)."""
import numpy as np
import pytest

import fusilli_b200 as fz
from fusilli_b200 import workloads as wl
from fusilli_b200.graph import DataType, ErrorCode, FusilliError
from helpers import make_input, run_gpu
from oracle import fusilli_oracle as orc

pytestmark = pytest.mark.gpu


def _setup(handle):
    g, ins, out = wl.matmul_bias(2, 64, 64, 64, DataType.Float)
    rng = np.random.default_rng(3)
    data = {t: make_input(t, rng) for t in ins.values()}
    g.compile(handle)
    pack = {t: fz.Buffer.allocate(handle, [a.size], a) for t, a in data.items()}
    pack[out] = fz.Buffer.allocate(handle, [out.physicalVolume()], np.zeros(out.physicalVolume(), np.float32))
    return g, ins, out, data, pack


def test_execute_guards():
    h = fz.Handle.create(fz.Backend.CUDA)
    g, ins, out, data, pack = _setup(h)
    with pytest.raises(FusilliError) as e:
        g.execute(h, pack, None)
    assert e.value.code == ErrorCode.InvalidArgument
    assert "requires getWorkspaceSize() to be called" in e.value.message
    assert g.getWorkspaceSize() == 0
    g.execute(h, pack, None)
    missing = dict(pack)
    del missing[ins["a"]]
    with pytest.raises(FusilliError) as e:
        g.execute(h, missing, None)
    assert e.value.code == ErrorCode.VariantPackError and e.value.message == "Input tensor missing from variantPack"
    missing = dict(pack)
    del missing[out]
    with pytest.raises(FusilliError) as e:
        g.execute(h, missing, None)
    assert e.value.message == "Output tensor missing from variantPack"
    small = dict(pack)
    small[out] = fz.Buffer.allocateRaw(h, 16)
    with pytest.raises(FusilliError) as e:
        g.execute(h, small, None)
    assert e.value.code == ErrorCode.InvalidArgument


def test_workspace_required_and_size_checked():
    h = fz.Handle.create(fz.Backend.CUDA)
    g, ins, dw = wl.conv_wgrad(8, 64, 28, 28, 64, 3, 3, 1, DataType.BFloat16)
    rng = np.random.default_rng(4)
    g.compile(h)
    need = g.getWorkspaceSize()
    assert need > 0
    pack = {t: fz.Buffer.allocate(h, [t.physicalVolume()], make_input(t, rng)) for t in ins.values()}
    pack[dw] = fz.Buffer.allocateRaw(h, dw.physicalVolume() * 2)
    with pytest.raises(FusilliError) as e:
        g.execute(h, pack, None)
    assert e.value.code == ErrorCode.InvalidArgument and "Workspace buffer required" in e.value.message
    with pytest.raises(FusilliError) as e:
        g.execute(h, pack, fz.Buffer.allocateRaw(h, need // 2))
    assert "Workspace buffer too small" in e.value.message
    g.execute(h, pack, fz.Buffer.allocateRaw(h, need))
    h.synchronize()


def test_artifact_from_one_graph_loads_into_another():
    h = fz.Handle.create(fz.Backend.CUDA)
    g1, ins1, out1 = wl.matmul_bias(2, 64, 64, 64, DataType.Float)
    blob = g1.compileToArtifact()
    assert g1.getWorkspaceSize() is None  # compileToArtifact does not touch the loaded state
    g2, ins2, out2 = wl.matmul_bias(2, 64, 64, 64, DataType.Float)
    g2.loadFromArtifact(h, blob)
    rng = np.random.default_rng(5)
    data = {ins2[k]: make_input(ins2[k], rng) for k in ins2}
    pack = {t: fz.Buffer.allocate(h, [a.size], a) for t, a in data.items()}
    pack[out2] = fz.Buffer.allocateRaw(h, out2.physicalVolume() * 4)
    g2.getWorkspaceSize()
    g2.execute(h, pack, None)
    got = pack[out2].read(h, np.float32)
    want = orc.execute(g2, data)[out2]
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
    # a failed load leaves the graph not loaded (tests/test_graph.cpp:469-488)
    with pytest.raises(FusilliError) as e:
        g2.loadFromArtifact(h, b"not an artifact")
    assert e.value.code == ErrorCode.RuntimeFailure
    assert g2.getWorkspaceSize() is None
    with pytest.raises(FusilliError) as e:
        g2.execute(h, pack, None)
    assert e.value.code == ErrorCode.NotCompiled


def test_buffer_checks():
    h = fz.Handle.create(fz.Backend.CUDA)
    with pytest.raises(FusilliError) as e:
        fz.Buffer.allocate(h, [2, 3], np.zeros(10, np.float32))
    assert e.value.message == ("Buffer::allocate failed: bufferData size (10) does not match product of "
                               "bufferShape dimensions (6)")
    with pytest.raises(FusilliError) as e:
        fz.Buffer.allocate(h, [0], np.zeros(0, np.float32))
    assert e.value.message == "Buffer::allocate failed: cannot allocate a buffer with zero size"
    with pytest.raises(FusilliError) as e:
        fz.Buffer.allocateRaw(h, 0)
    assert e.value.message == "Buffer::allocateRaw failed: cannot allocate zero-size buffer"
    with pytest.raises(FusilliError) as e:
        fz.Buffer.importPointer(h, 0, 16)
    assert e.value.message == "Buffer::import failed as externalBufferView* is NULL"
    b = fz.Buffer.allocate(h, [4], np.arange(4, dtype=np.int32))
    assert b.read(h, np.int32).tolist() == [0, 1, 2, 3]
    bad = None
    with pytest.raises(FusilliError):
        bad = fz.Handle.create(fz.Backend.CUDA, 4096)
    assert bad is None


def test_buffers_may_outlive_their_handle():
    h = fz.Handle.create(fz.Backend.CUDA)
    b = fz.Buffer.allocate(h, [8], np.ones(8, np.float32))
    h.close()
    b.release()  # must not touch a destroyed stream


def test_external_stream_and_imported_pointers():
    """Handle on a caller-owned stream, buffers imported from caller-owned device memory,
    stream-ordered read (tests/hip_tests/test_handle.cpp:53-141, test_buffer.cpp:84-205)."""
    torch = pytest.importorskip("torch")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        h = fz.Handle.create(fz.Backend.CUDA, 0, stream.cuda_stream)
        assert h.stream() == stream.cuda_stream
        g, ins, out = wl.layernorm_infer(32, 2048)
        g.compile(h)
        g.getWorkspaceSize()
        x = torch.randn(32, 2048, device="cuda").to(torch.bfloat16)
        gamma = torch.ones(2048, device="cuda")
        beta = torch.zeros(2048, device="cuda")
        y = torch.empty_like(x)
        pack = {
            ins["x"]: fz.Buffer.importPointer(h, x.data_ptr(), x.numel() * 2),
            ins["gamma"]: fz.Buffer.importPointer(h, gamma.data_ptr(), gamma.numel() * 4),
            ins["beta"]: fz.Buffer.importPointer(h, beta.data_ptr(), beta.numel() * 4),
            out[0]: fz.Buffer.importPointer(h, y.data_ptr(), y.numel() * 2),
        }
        g.execute(h, pack, None)          # asynchronous on the caller's stream
        ref = torch.nn.functional.layer_norm(x.float(), (2048,)).to(torch.bfloat16)
    stream.synchronize()
    assert torch.allclose(y.float(), ref.float(), rtol=2e-2, atol=2e-2)
    del pack                               # importing never takes ownership
    assert float(x.float().abs().sum()) > 0


def test_reexecution_is_stable():
    h = fz.Handle.create(fz.Backend.CUDA)
    g, ins, out = wl.sdpa_fwd(1, 2, 256, 128)
    rng = np.random.default_rng(6)
    data = {t: make_input(t, rng, ("normal", 0.0, 1.0)) for t in ins.values()}
    first = run_gpu(g, data, h, repeat=1)[out]
    again = run_gpu(g, data, h, repeat=3)[out]
    assert np.array_equal(first, again)  # deterministic kernels: bitwise repeatable


@pytest.mark.gpu
def test_padded_leading_stride_needs_a_buffer_that_covers_the_padding():
    """A matmul operand whose leading stride exceeds its row length (rows padded to 136 elements for a
    128-wide A; reachable through the C ABI only): the size check counts one past the last element's offset, so a buffer of just
    prod(dims) elements is refused and the padded one computes the right product."""
    import ctypes
    from fusilli_b200.graph import DataType, ErrorCode, FusilliError, TensorAttr, contiguousStride
    from oracle import fusilli_oracle as orc
    m, k, n, lda = 256, 128, 192, 136
    g = fz.Graph()
    g.setName("mm_padded").setIODataType(DataType.BFloat16).setComputeDataType(DataType.Float).setIntermediateDataType(DataType.Float)
    a = g.tensor(TensorAttr().setName("a").setDim([m, k]).setStride([k, 1]))
    b = g.tensor(TensorAttr().setName("b").setDim([k, n]).setStride(contiguousStride([k, n])))
    c = g.matmul(a, b, fz.MatmulAttr().setName("mm"))
    c.setName("c").setOutput(True)
    g.validate()
    a.stride = [lda, 1]   # the front ends only admit dense layouts; the C ABI takes padded rows
    handle = fz.Handle.create(fz.Backend.CUDA)
    g.compile(handle)
    g.getWorkspaceSize()
    rng = np.random.default_rng(5)
    a_pad = orc.to_storage(rng.normal(0, 0.5, m * lda).astype(np.float32), DataType.BFloat16)
    b_val = orc.to_storage(rng.normal(0, 0.5, k * n).astype(np.float32), DataType.BFloat16)
    need = (m - 1) * lda + k
    bb = fz.Buffer.allocate(handle, [b_val.size], b_val)
    cb = fz.Buffer.allocate(handle, [m * n], np.zeros(m * n, np.uint16))
    short = fz.Buffer.allocate(handle, [m * k], a_pad[: m * k])
    with pytest.raises(FusilliError) as e:
        g.execute(handle, {a: short, b: bb, c: cb}, None)
    assert e.value.code == ErrorCode.InvalidArgument and "needs" in e.value.message
    ab = fz.Buffer.allocate(handle, [need], a_pad[:need])
    g.execute(handle, {a: ab, b: bb, c: cb}, None)
    got = orc.from_storage(cb.read(handle, np.uint16), DataType.BFloat16).reshape(m, n)
    a_log = orc.from_storage(a_pad, DataType.BFloat16).reshape(m, lda)[:, :k].astype(np.float64)
    want = a_log @ orc.from_storage(b_val, DataType.BFloat16).reshape(k, n).astype(np.float64)
    np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2 * min(1.0, np.abs(want).max()))


@pytest.mark.gpu
def test_bound_graph_runs_like_execute():
    """Graph.bind marshals the buffers once; run() must produce what execute() produces, apply the
    same variant-pack checks at bind time, and stay valid over repeated runs."""
    g, ins, out = wl.matmul_bias(2, 128, 128, 64)
    rng = np.random.default_rng(9)
    data = {t: make_input(t, rng, ("normal", 0.0, 0.5)) for t in ins.values()}
    handle = fz.Handle.create(fz.Backend.CUDA)
    want = run_gpu(g, data, handle)[out]
    pack = {t: fz.Buffer.allocate(handle, [a.size], a) for t, a in data.items()}
    pack[out] = fz.Buffer.allocate(handle, [want.size], np.zeros(want.size, want.dtype))
    bound = g.bind(handle, pack, None)
    for _ in range(3):
        bound.run()
    assert np.array_equal(pack[out].read(handle, want.dtype), want)
    missing = dict(pack)
    del missing[out]
    with pytest.raises(FusilliError) as e:
        g.bind(handle, missing, None)
    assert e.value.code == ErrorCode.VariantPackError
