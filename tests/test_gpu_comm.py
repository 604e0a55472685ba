"""The cross-rank sum of the weight gradients (fb_comm_*) and the failure path of the bounded
waits.

On one GPU the fused exchange kernel is exercised for 2, 4 and 8 VIRTUAL ranks inside one cooperative
launch (kernels that wait on one another are never separate launches on one GPU); with two or more
GPUs the real thing runs as child processes, one per GPU, bootstrapped through files. Sums are added
in rank order, so the expected bits are computable exactly on the host."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

import fusilli_b200 as fz
from fusilli_b200 import runtime
from fusilli_b200.graph import DataType, ErrorCode
from oracle import fusilli_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_VP = ctypes.c_void_p


def _expected(parts: np.ndarray, dtype: DataType) -> np.ndarray:
    acc = parts[0].copy()
    for r in range(1, parts.shape[0]):
        acc = acc + parts[r]  # float32, rank order: what the kernel does
    return acc if dtype == DataType.Float else orc.to_storage(acc, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("dtype,count", [(DataType.BFloat16, 2_801_664), (DataType.Float, 4096), (DataType.Half, 36_868)])
def test_fused_exchange_virtual_ranks(world, dtype, count):
    """count = 2,801,664 is the five ResNet-50 filter gradients of the benchmark in one bucket."""
    lib = runtime.lib()
    handle = fz.Handle.create(fz.Backend.CUDA)
    rng = np.random.default_rng(world * 1000 + count)
    parts = rng.normal(0, 1.0, (world, count)).astype(np.float32)
    src = fz.Buffer.allocate(handle, [parts.size], parts.reshape(-1))
    esz = 4 if dtype == DataType.Float else 2
    out = fz.Buffer.allocateRaw(handle, world * count * esz)
    st = lib.fb_comm_selftest_emulated(handle._ptr, world, _VP(src.ptr()), count, _VP(out.ptr()), int(dtype), 3)
    assert st == 0, lib.fb_last_error().decode()
    assert handle.kernelError() == 0
    got = out.read(handle, orc.NP_DTYPE[dtype]).reshape(world, count)
    want = _expected(parts, dtype)
    for r in range(world):
        assert np.array_equal(got[r], want), f"rank {r}'s copy of the sum differs"


@pytest.mark.gpu
def test_single_rank_comm_is_a_cast():
    handle = fz.Handle.create(fz.Backend.CUDA)
    count = 4096
    comm = fz.Comm.create(handle, 0, 1, count * 4 + count * 2)
    vals = np.random.default_rng(3).normal(0, 2.0, count).astype(np.float32)
    comm.view(0, count * 4).write(handle, vals)
    comm.sumFused(0, count, count * 4, DataType.BFloat16)
    got = comm.view(count * 4, count * 2).read(handle, np.uint16)
    assert np.array_equal(got, orc.to_storage(vals, DataType.BFloat16))
    with pytest.raises(fz.FusilliError) as e:
        comm.sumFused(0, count, count * 2, DataType.BFloat16)  # output inside the input range
    assert e.value.code == ErrorCode.InvalidArgument
    with pytest.raises(fz.FusilliError):
        comm.sumFused(0, count + 2, count * 4 + 64, DataType.BFloat16)  # not a multiple of 4
    comm.close()


@pytest.mark.gpu
def test_bounded_wait_runs_out_and_reports():
    """A wait nothing will ever satisfy gives up after its poll limit, the kernel ends normally with
    the code in the device's error word, and the device keeps working afterwards."""
    lib = runtime.lib()
    handle = fz.Handle.create(fz.Backend.CUDA)
    assert handle.kernelError() == 0
    assert lib.fb_device_selftest_wait_timeout(handle._ptr, 1000, 0x10) == 0
    assert handle.kernelError() == 0x10
    assert lib.fb_device_selftest_wait_timeout(handle._ptr, 500, 0x1) == 0
    assert handle.kernelError() == 0x11          # codes accumulate until cleared
    handle.clearKernelError()
    assert handle.kernelError() == 0
    buf = fz.Buffer.allocate(handle, [4], np.arange(4, dtype=np.int32))   # the context is still usable
    assert np.array_equal(buf.read(handle, np.int32), np.arange(4))


_CHILD = r"""
import os, sys, time, numpy as np
sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests"))
import fusilli_b200 as fz
from fusilli_b200 import workloads as wl
from fusilli_b200.graph import DataType
from fusilli_b200.sharding import shard_range
rank, world, tmp = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]

def allgather(b):
    with open(os.path.join(tmp, f"blk_{{rank}}.tmp"), "wb") as f: f.write(b)
    os.rename(os.path.join(tmp, f"blk_{{rank}}.tmp"), os.path.join(tmp, f"blk_{{rank}}"))
    out = []
    for r in range(world):
        p = os.path.join(tmp, f"blk_{{r}}")
        t0 = time.time()
        while not os.path.exists(p):
            if time.time() - t0 > 60: raise SystemExit("peer never wrote its block")
            time.sleep(0.01)
        out.append(open(p, "rb").read())
    return out

def barrier(tag):
    open(os.path.join(tmp, f"{{tag}}_{{rank}}"), "w").close()
    t0 = time.time()
    while not all(os.path.exists(os.path.join(tmp, f"{{tag}}_{{r}}")) for r in range(world)):
        if time.time() - t0 > 60: raise SystemExit("barrier timed out")
        time.sleep(0.002)

handle = fz.Handle.create(fz.Backend.CUDA, rank)
n, c, hw, k, r_, pad = 16, 64, 28, 64, 3, 1
elems = k * r_ * r_ * c
comm = fz.Comm.create(handle, rank, world, elems * 4 + elems * 2, allgather)
lo, hi = shard_range(n, rank, world)
x = np.load(os.path.join(tmp, "x.npy")).reshape(n, -1)[lo:hi].reshape(-1)
dy = np.load(os.path.join(tmp, "dy.npy")).reshape(n, -1)[lo:hi].reshape(-1)
g, ins, dw = wl.conv_wgrad(hi - lo, c, hw, hw, k, r_, r_, pad, dw_dtype=DataType.Float)
g.compile(handle)
ws = fz.Buffer.allocateRaw(handle, g.getWorkspaceSize()) if g.getWorkspaceSize() else None
pack = {{ins["x"]: fz.Buffer.allocate(handle, [x.size], x), ins["dy"]: fz.Buffer.allocate(handle, [dy.size], dy),
        dw: comm.view(0, elems * 4)}}
for step in range(3):                       # repeated steps reuse the flags and the buckets
    g.execute(handle, pack, ws)
    barrier(f"s{{step}}")
    comm.sumFused(0, elems, elems * 4, DataType.BFloat16)
    handle.synchronize()
fused = comm.view(elems * 4, elems * 2).read(handle, np.uint16)
part = comm.view(0, elems * 4).read(handle, np.float32)
scratch = fz.Buffer.allocate(handle, [elems], part)
out = fz.Buffer.allocateRaw(handle, elems * 2)
comm.sumNccl(scratch.ptr(), elems, out.ptr(), DataType.BFloat16)
nccl = out.read(handle, np.uint16)
gathered = fz.Buffer.allocateRaw(handle, world * elems * 4)
comm.allGather(comm.bufferPtr(), gathered.ptr(), elems * 4)
parts = gathered.read(handle, np.float32)
err = handle.kernelError()
np.savez(os.path.join(tmp, f"res_{{rank}}.npz"), fused=fused, nccl=nccl, parts=parts, err=err)
barrier("done")
comm.close()
"""


@pytest.mark.gpu
def test_wgrad_exchange_across_real_gpus(tmp_path):
    """Two (or four) processes, one GPU each: sharded wgrad -> fp32 partials in the exchange buffer ->
    fused sum -> bf16. Every rank must hold the bits of the rank-ordered sum of the gathered partials,
    the NCCL route must agree within one bf16 ulp, and the result must match the oracle's full-batch
    weight gradient."""
    ndev = runtime.lib().fb_device_count()
    if ndev < 2:
        pytest.skip("needs at least two GPUs")
    world = 4 if ndev >= 4 else 2
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from fusilli_b200 import workloads as wl
    from helpers import make_input
    n, c, hw, k, r_, pad = 16, 64, 28, 64, 3, 1
    g, ins, dw = wl.conv_wgrad(n, c, hw, hw, k, r_, r_, pad)
    rng = np.random.default_rng(77)
    x = make_input(ins["x"], rng, ("normal", 0.0, 0.05))
    dy = make_input(ins["dy"], rng, ("normal", 0.0, 0.01))
    np.save(tmp_path / "x.npy", x)
    np.save(tmp_path / "dy.npy", dy)
    script = tmp_path / "child.py"
    script.write_text(_CHILD.format(root=ROOT))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(world), str(tmp_path)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append(o)
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    res = [np.load(tmp_path / f"res_{r}.npz") for r in range(world)]
    assert all(int(r["err"]) == 0 for r in res)
    elems = k * r_ * r_ * c
    parts = res[0]["parts"].reshape(world, elems)
    want_bits = _expected(parts, DataType.BFloat16)
    for r in range(world):
        assert np.array_equal(res[r]["fused"], want_bits), f"rank {r}: fused sum is not the rank-ordered sum"
    f = orc.from_storage(res[0]["fused"], DataType.BFloat16).astype(np.float64)
    nc = orc.from_storage(res[0]["nccl"], DataType.BFloat16).astype(np.float64)
    assert np.all(np.abs(f - nc) <= 2.0 ** -7 * np.abs(f).max())
    from helpers import compare
    want = orc.execute(g, {ins["x"]: x, ins["dy"]: dy})[dw]
    compare(res[0]["fused"], want, DataType.BFloat16, "exchanged wgrad vs full-batch oracle", acc_len=n * hw * hw)
