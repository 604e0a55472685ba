"""Shared machinery of the parity tests: seeded inputs, run a validated graph on the
GPU through the C ABI, run the same graph through the CPU oracle, compare."""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np

import fusilli_b200 as fz
from fusilli_b200.graph import DataType, TensorAttr
from oracle import fusilli_oracle as orc

def gpu_available() -> bool:
    try:
        from fusilli_b200 import runtime
        return runtime.lib().fb_device_count() > 0
    except Exception:
        return False


def make_input(t: TensorAttr, rng: np.random.Generator, dist=("uniform", -1.0, 1.0)) -> np.ndarray:
    """Flat storage array (physical order) for tensor ``t`` drawn from ``dist``."""
    n = t.physicalVolume()
    if t.dataType in (DataType.Half, DataType.BFloat16, DataType.Float):
        if dist[0] == "uniform":
            vals = rng.uniform(dist[1], dist[2], n).astype(np.float32)
        elif dist[0] == "normal":
            vals = rng.normal(dist[1], dist[2], n).astype(np.float32)
        elif dist[0] == "const":
            vals = np.full(n, dist[1], np.float32)
        else:
            raise ValueError(dist)
        return orc.to_storage(vals, t.dataType)
    if t.dataType == DataType.Boolean:
        return rng.integers(0, 2, n).astype(np.uint8)
    if t.dataType == DataType.Int4:
        return orc.pack_int4(rng.integers(-8, 8, n))
    if dist[0] == "const":
        return np.full(n, int(dist[1]), orc.NP_DTYPE[t.dataType])
    return rng.integers(-50, 50, n).astype(orc.NP_DTYPE[t.dataType])


def run_gpu(graph: fz.Graph, inputs: Dict[TensorAttr, np.ndarray], handle: Optional[fz.Handle] = None,
            repeat: int = 1) -> Dict[TensorAttr, np.ndarray]:
    """validate()d graph -> compile -> execute on cuda:0 -> flat storage arrays of the outputs."""
    own = handle is None
    if own:
        handle = fz.Handle.create(fz.Backend.CUDA)
    graph.compile(handle)
    ws_size = graph.getWorkspaceSize()
    ws = fz.Buffer.allocateRaw(handle, ws_size) if ws_size else None
    pack = {}
    outs = {}
    for t, arr in inputs.items():
        pack[t] = fz.Buffer.allocate(handle, [arr.size], arr)  # Int4 arrives packed: bytes, not elements
    for t in graph.outputs:
        if t.isVirtual():
            continue
        init = np.zeros(t.physicalVolume(), dtype=orc.NP_DTYPE[t.dataType])
        pack[t] = fz.Buffer.allocate(handle, [init.size], init)
        outs[t] = pack[t]
    for _ in range(repeat):
        graph.execute(handle, pack, ws)
    res = {t: b.read(handle, orc.NP_DTYPE[t.dataType]) for t, b in outs.items()}
    err = handle.kernelError()
    assert err == 0, f"kernel error word {err:#x} (a bounded wait ran out)"
    return res


def as_float(flat: np.ndarray, dtype: DataType) -> np.ndarray:
    return orc.from_storage(flat, dtype)


from oracle.check import TOL, ULP_REL, graph_traits, tolerance  # noqa: E402,F401


def compare(got: np.ndarray, want: np.ndarray, dtype: DataType, what: str = "", acc_len: int = 1,
            chained: bool = False):
    """Bit-exact for integral types; `tolerance` for floating types. Large arrays are walked in
    chunks so a full-size benchmark tensor never needs several float64 copies at once."""
    if dtype not in TOL:
        assert np.array_equal(got, want), f"{what}: integer/bool outputs differ"
        return
    got, want = got.reshape(-1), want.reshape(-1)
    assert got.size == want.size, f"{what}: {got.size} elements, expected {want.size}"
    step = 1 << 24
    peak = 0.0
    for i in range(0, want.size, step):
        w = as_float(want[i:i + step], dtype)
        w = np.abs(w[np.isfinite(w)])
        if w.size:
            peak = max(peak, float(w.max()))
    tol = tolerance(dtype, np.array([peak]), acc_len, chained)
    for i in range(0, want.size, step):
        g = as_float(got[i:i + step], dtype).astype(np.float64)
        w = as_float(want[i:i + step], dtype).astype(np.float64)
        np.testing.assert_allclose(g, w, err_msg=f"{what} [elements {i}..]", **tol)


def check_graph(graph: fz.Graph, inputs: Dict[TensorAttr, np.ndarray], handle: Optional[fz.Handle] = None):
    """GPU vs oracle on identical bytes, every non-virtual output."""
    want = orc.execute(graph, inputs)
    got = run_gpu(graph, inputs, handle)
    assert set(got) == set(want)
    acc_len, chained = graph_traits(graph)
    for t in want:
        compare(got[t], want[t], t.dataType, t.name, acc_len, chained)
    return got, want
