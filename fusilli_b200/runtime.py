"""ctypes binding of libfusilli_b200.so plus the device-facing half of the graph
API (Handle, Buffer, Graph.compile/execute), mirroring the reference's
include/fusilli/backend/{handle,buffer}.h and include/fusilli/graph/graph.h.

There is no fallback: if the CUDA library is missing the import of this module
raises, and every device call fails with RuntimeFailure when no B200 is present.
"""
from __future__ import annotations

import ctypes
import enum
import os
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import graph as G
from .graph import (DTYPE_SIZE, DataType, ErrorCode, FusilliError, GraphBase, NormFwdPhase, Op,
                    TensorAttr)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FUSILLI_B200_LIB", os.path.join(_HERE, "libfusilli_b200.so"))

FB_MAX_RANK = 8


class fb_tensor_desc(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("dtype", ctypes.c_int32), ("role", ctypes.c_int32),
                ("rank", ctypes.c_int32), ("arg_index", ctypes.c_int32),
                ("dims", ctypes.c_int64 * FB_MAX_RANK), ("strides", ctypes.c_int64 * FB_MAX_RANK),
                ("scalar_value", ctypes.c_double), ("dynamic_mask", ctypes.c_uint32),
                ("reserved", ctypes.c_int32)]


class fb_node_desc(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("op", ctypes.c_int32), ("mode", ctypes.c_int32),
                ("flags", ctypes.c_int32), ("num_spatial", ctypes.c_int32),
                ("inputs", ctypes.c_int32 * 6), ("outputs", ctypes.c_int32 * 3),
                ("reserved", ctypes.c_int32), ("padding", ctypes.c_int64 * 3),
                ("stride", ctypes.c_int64 * 3), ("dilation", ctypes.c_int64 * 3),
                ("fparams", ctypes.c_float * 4)]


class fb_graph_desc(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("num_tensors", ctypes.c_int32),
                ("num_nodes", ctypes.c_int32), ("tensors", ctypes.POINTER(fb_tensor_desc)),
                ("nodes", ctypes.POINTER(fb_node_desc))]


# Every symbol include/fusilli_b200.h declares: (name, restype, argtypes)
_VP, _SZ, _I32 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int32
ABI_SYMBOLS = [
    ("fb_abi_version", _I32, []),
    ("fb_last_error", ctypes.c_char_p, []),
    ("fb_device_count", _I32, []),
    ("fb_device_open", _I32, [_I32, _VP, ctypes.POINTER(_VP)]),
    ("fb_device_close", _I32, [_VP]),
    ("fb_device_sync", _I32, [_VP]),
    ("fb_device_stream", _VP, [_VP]),
    ("fb_device_ordinal", _I32, [_VP]),
    ("fb_device_kernel_error", _I32, [_VP, ctypes.POINTER(ctypes.c_uint32)]),
    ("fb_buffer_alloc", _I32, [_VP, _SZ, ctypes.POINTER(_VP)]),
    ("fb_buffer_wrap", _I32, [_VP, _VP, _SZ, ctypes.POINTER(_VP)]),
    ("fb_buffer_retain", _I32, [_VP]),
    ("fb_buffer_release", _I32, [_VP]),
    ("fb_buffer_h2d", _I32, [_VP, _VP, _VP, _SZ]),
    ("fb_buffer_d2h", _I32, [_VP, _VP, _VP, _SZ]),
    ("fb_buffer_ptr", _VP, [_VP]),
    ("fb_buffer_size", _SZ, [_VP]),
    ("fb_plan_build", _I32, [ctypes.POINTER(fb_graph_desc), ctypes.POINTER(ctypes.POINTER(ctypes.c_uint8)),
                             ctypes.POINTER(_SZ)]),
    ("fb_bytes_free", None, [ctypes.POINTER(ctypes.c_uint8)]),
    ("fb_plan_load", _I32, [_VP, ctypes.c_char_p, _SZ, ctypes.POINTER(_VP)]),
    ("fb_plan_free", _I32, [_VP]),
    ("fb_plan_check", _I32, [ctypes.c_char_p, _SZ]),
    ("fb_plan_workspace_size", _I32, [_VP, ctypes.POINTER(_SZ)]),
    ("fb_plan_num_args", _I32, [_VP, ctypes.POINTER(_I32)]),
    ("fb_plan_num_launches", _I32, [_VP, ctypes.POINTER(_I32)]),
    ("fb_plan_stats_json", _I32, [_VP, ctypes.c_char_p, _SZ, ctypes.POINTER(_SZ)]),
    ("fb_plan_execute", _I32, [_VP, _VP, ctypes.POINTER(_VP), ctypes.POINTER(_SZ), _I32, _VP, _SZ]),
    ("fb_plan_execute_shaped", _I32, [_VP, _VP, ctypes.POINTER(_VP), ctypes.POINTER(_SZ),
                                      ctypes.POINTER(ctypes.c_int64), _I32, _VP, _SZ]),
    ("fb_plan_specialize", _I32, [ctypes.c_char_p, _SZ, ctypes.POINTER(ctypes.c_int64), _I32,
                                  ctypes.POINTER(ctypes.POINTER(ctypes.c_uint8)), ctypes.POINTER(_SZ)]),
    ("fb_plan_workspace_size_shaped", _I32, [_VP, ctypes.POINTER(ctypes.c_int64), _I32, ctypes.POINTER(_SZ)]),
    ("fb_device_selftest_wait_timeout", _I32, [_VP, ctypes.c_uint32, ctypes.c_uint32]),
    ("fb_device_clear_kernel_error", _I32, [_VP]),
    ("fb_comm_create", _I32, [_VP, _I32, _I32, _SZ, ctypes.POINTER(_VP)]),
    ("fb_comm_local_handle", _I32, [_VP, ctypes.c_char_p]),
    ("fb_comm_connect", _I32, [_VP, ctypes.c_char_p]),
    ("fb_comm_close", _I32, [_VP]),
    ("fb_comm_buffer", _VP, [_VP]),
    ("fb_comm_buffer_bytes", _SZ, [_VP]),
    ("fb_comm_rank", _I32, [_VP]),
    ("fb_comm_world", _I32, [_VP]),
    ("fb_comm_sum_fused", _I32, [_VP, _SZ, _SZ, _SZ, _I32]),
    ("fb_comm_sum_nccl", _I32, [_VP, _VP, _SZ, _VP, _I32]),
    ("fb_comm_allgather", _I32, [_VP, _VP, _VP, _SZ]),
    ("fb_comm_selftest_emulated", _I32, [_VP, _I32, _VP, _SZ, _VP, _I32, _I32]),
    ("fb_conv_wgrad_static_scratch_bytes", _SZ, []),
    ("fb_conv_wgrad_static", _I32, [_VP, _VP, _VP, _VP] + [_I32] * 15),
]

_lib = None


def lib():
    """Loads the CUDA library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FusilliError(ErrorCode.RuntimeFailure,
                               f"{LIB_PATH} not found: build it with `python -m fusilli_b200.build` "
                               "(there is no CPU fallback)")
        _lib = ctypes.CDLL(LIB_PATH)
        for name, res, args in ABI_SYMBOLS:
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


def _check(status: int) -> None:
    if status != 0:
        msg = lib().fb_last_error().decode("utf-8", "replace")
        raise FusilliError(ErrorCode(status), msg)


class Backend(enum.IntEnum):
    """Backend enum of the reference (backend.h:42) plus the value this build adds."""
    CPU = 0
    AMDGPU = 1
    CUDA = 2


class Handle:
    """fusilli::Handle (handle.h:35-176): one device + one stream."""

    def __init__(self, ptr, backend):
        self._ptr = ptr
        self.backend = backend

    @staticmethod
    def create(backend: Backend, deviceId: int = 0, stream: Optional[int] = None) -> "Handle":
        if backend != Backend.CUDA:
            code = ErrorCode.InvalidArgument if stream is not None else ErrorCode.NotImplemented
            raise FusilliError(code, f"Backend {Backend(backend).name} is not available in this build; "
                                     "use Backend.CUDA")
        out = _VP()
        _check(lib().fb_device_open(int(deviceId), _VP(stream) if stream else None, ctypes.byref(out)))
        return Handle(out, backend)

    def getBackend(self):
        return self.backend

    def stream(self) -> int:
        return lib().fb_device_stream(self._ptr) or 0

    def synchronize(self) -> None:
        _check(lib().fb_device_sync(self._ptr))

    def kernelError(self) -> int:
        w = ctypes.c_uint32(0)
        _check(lib().fb_device_kernel_error(self._ptr, ctypes.byref(w)))
        return w.value

    def clearKernelError(self) -> None:
        _check(lib().fb_device_clear_kernel_error(self._ptr))

    def close(self):
        if self._ptr:
            lib().fb_device_close(self._ptr)
            self._ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Buffer:
    """fusilli::Buffer (buffer.h:31-81)."""

    def __init__(self, ptr, handle=None, shape=None):
        self._ptr = ptr
        self._handle = handle  # keeps the device alive as long as the buffer
        # dims of the dense (physical order) array; graphs with dynamic dims read them at execute
        self.shape: Optional[List[int]] = [int(v) for v in shape] if shape is not None else None
        self._dptr: Optional[int] = None
        self._bytes: Optional[int] = None

    @staticmethod
    def allocate(handle: Handle, shape: Sequence[int], data: np.ndarray) -> "Buffer":
        expected = int(np.prod(shape)) if len(shape) else 0
        if expected == 0:
            raise FusilliError(ErrorCode.RuntimeFailure,
                               "Buffer::allocate failed: cannot allocate a buffer with zero size")
        data = np.ascontiguousarray(data)
        if data.size != expected:
            raise FusilliError(ErrorCode.RuntimeFailure,
                               f"Buffer::allocate failed: bufferData size ({data.size}) does not match "
                               f"product of bufferShape dimensions ({expected})")
        buf = Buffer.allocateRaw(handle, data.nbytes)
        buf.shape = [int(v) for v in shape]
        _check(lib().fb_buffer_h2d(handle._ptr, buf._ptr, data.ctypes.data_as(_VP), data.nbytes))
        return buf

    @staticmethod
    def allocateRaw(handle: Handle, sizeInBytes: int) -> "Buffer":
        if sizeInBytes == 0:
            raise FusilliError(ErrorCode.RuntimeFailure,
                               "Buffer::allocateRaw failed: cannot allocate zero-size buffer")
        out = _VP()
        _check(lib().fb_buffer_alloc(handle._ptr, sizeInBytes, ctypes.byref(out)))
        return Buffer(out, handle)

    @staticmethod
    def importPointer(handle: Handle, devicePtr: int, sizeInBytes: int, shape=None) -> "Buffer":
        """Buffer::import of caller-owned device memory (e.g. a torch tensor)."""
        if not devicePtr:
            raise FusilliError(ErrorCode.RuntimeFailure,
                               "Buffer::import failed as externalBufferView* is NULL")
        out = _VP()
        _check(lib().fb_buffer_wrap(handle._ptr, _VP(devicePtr), sizeInBytes, ctypes.byref(out)))
        return Buffer(out, handle, shape)

    def write(self, handle: Handle, data: np.ndarray) -> None:
        data = np.ascontiguousarray(data)
        _check(lib().fb_buffer_h2d(handle._ptr, self._ptr, data.ctypes.data_as(_VP), data.nbytes))

    def read(self, handle: Handle, dtype=np.uint8) -> np.ndarray:
        n = self.size()
        out = np.empty(n // np.dtype(dtype).itemsize, dtype=dtype)
        _check(lib().fb_buffer_d2h(handle._ptr, self._ptr, out.ctypes.data_as(_VP), n))
        return out

    def read_into(self, handle: Handle, out: np.ndarray) -> None:
        _check(lib().fb_buffer_d2h(handle._ptr, self._ptr, out.ctypes.data_as(_VP), out.nbytes))

    def ptr(self) -> int:
        if self._dptr is None:  # fixed at creation: asked once
            self._dptr = lib().fb_buffer_ptr(self._ptr) or 0
        return self._dptr

    def size(self) -> int:
        if self._bytes is None:
            self._bytes = lib().fb_buffer_size(self._ptr)
        return self._bytes

    def release(self):
        if self._ptr:
            lib().fb_buffer_release(self._ptr)
            self._ptr = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class Graph(GraphBase):
    """fusilli::Graph (graph.h:75-468) on the CUDA backend."""

    def __init__(self):
        super().__init__()
        self._plan = None
        self._artifact: Optional[bytes] = None
        self._workspace: Optional[int] = None
        self._ws_queried = False
        self._arg_tensors: List[TensorAttr] = []
        self._keep = None

    # -- flattening ------------------------------------------------------------
    def _flatten(self):
        """Validated graph -> fb_graph_desc. Argument order = non-virtual outputs
        sorted by name, then non-scalar inputs sorted by name (runtime.h:426-457)."""
        tensors: List[TensorAttr] = []
        index: Dict[int, int] = {}

        def tid(t: Optional[TensorAttr]) -> int:
            if t is None:
                return -1
            if id(t) not in index:
                index[id(t)] = len(tensors)
                tensors.append(t)
            return index[id(t)]

        nodes = (fb_node_desc * len(self.nodes))()
        keep = []
        for i, n in enumerate(self.nodes):
            d = nodes[i]
            nm = n.name.encode()
            keep.append(nm)
            d.name = nm
            d.op = int(n.op)
            node_ins = list(n.inputs)
            if n.op == Op.BATCHNORM:
                node_ins = node_ins[:6]  # momentum is not a kernel operand: it goes into fparams
                d.fparams[0] = float(n.inputs[6].getScalarValue())
            ins = node_ins + [None] * (6 - len(node_ins))
            outs = list(n.outputs) + [None] * (3 - len(n.outputs))
            for k in range(6):
                d.inputs[k] = tid(ins[k])
            for k in range(3):
                d.outputs[k] = tid(outs[k])
            a = n.attr
            if n.op in (Op.CONV_FPROP, Op.CONV_DGRAD, Op.CONV_WGRAD):
                d.num_spatial = len(a.padding)
                for k in range(len(a.padding)):
                    d.padding[k], d.stride[k], d.dilation[k] = a.padding[k], a.stride[k], a.dilation[k]
            elif n.op == Op.POINTWISE:
                d.mode = int(a.mode)
                d.fparams[0], d.fparams[1], d.fparams[2], d.fparams[3] = (
                    a.eluAlpha, a.softplusBeta, a.softplusThreshold, a.swishBeta)
            elif n.op == Op.REDUCTION:
                d.mode = int(a.mode)
            elif n.op == Op.SDPA:
                d.flags = (G.FLAG_SDPA_CAUSAL if a.isCausal else 0) | (G.FLAG_SDPA_GQA if a.enableGqa else 0)
                if a.scale is not None:
                    d.flags |= G.FLAG_SDPA_HAS_SCALE
                    d.fparams[0] = float(a.scale)
                d.fparams[1] = float(a.dropout)
            elif n.op in (Op.LAYERNORM, Op.RMSNORM, Op.BATCHNORM):
                if a.forwardPhase == NormFwdPhase.TRAINING:
                    d.flags |= G.FLAG_NORM_TRAINING
        outs_sorted = sorted((t for t in self.outputs if not t.isVirtual()), key=lambda t: t.name)
        ins_sorted = sorted((t for t in self.inputs if not t.isScalar() and id(t) in index),
                            key=lambda t: t.name)
        args = outs_sorted + ins_sorted
        arg_index = {id(t): i for i, t in enumerate(args)}
        tdesc = (fb_tensor_desc * len(tensors))()
        for i, t in enumerate(tensors):
            d = tdesc[i]
            nm = t.name.encode()
            keep.append(nm)
            d.name = nm
            d.dtype = int(t.dataType)
            d.rank = len(t.dim)
            for k in range(len(t.dim)):
                d.dims[k] = t.dim[k]
                d.strides[k] = t.stride[k]
            for k in t.getDynamicDims():
                d.dynamic_mask |= 1 << k
            if t.isScalar():
                d.role = 3
                d.scalar_value = float(t.getScalarValue())
                d.arg_index = -1
            elif t.isVirtual():
                d.role = 2
                d.arg_index = -1
            else:
                d.role = 1 if id(t) in {id(o) for o in self.outputs} else 0
                d.arg_index = arg_index[id(t)]
        gname = self.getName().encode()
        keep += [gname, nodes, tdesc]
        desc = fb_graph_desc(gname, len(tensors), len(self.nodes), tdesc, nodes)
        return desc, args, keep

    # -- compile / load ----------------------------------------------------------
    def compileToArtifact(self, backend: Backend = Backend.CUDA, remove: bool = False) -> bytes:
        if not self._validated:
            raise FusilliError(ErrorCode.NotValidated, "Graph must be validated before being compiled")
        if backend != Backend.CUDA:
            raise FusilliError(ErrorCode.NotImplemented,
                               f"Backend {Backend(backend).name} is not available in this build")
        desc, args, keep = self._flatten()
        out = ctypes.POINTER(ctypes.c_uint8)()
        n = _SZ(0)
        _check(lib().fb_plan_build(ctypes.byref(desc), ctypes.byref(out), ctypes.byref(n)))
        try:
            blob = ctypes.string_at(out, n.value)
        finally:
            lib().fb_bytes_free(out)
        self._arg_tensors = args
        return blob

    def loadFromArtifact(self, handle: Handle, artifact: bytes) -> None:
        if not self._validated:
            raise FusilliError(ErrorCode.NotValidated,
                               "Graph must be validated before loading a compiled artifact")
        self._clear()
        out = _VP()
        _check(lib().fb_plan_load(handle._ptr, artifact, len(artifact), ctypes.byref(out)))
        self._plan = out
        self._artifact = bytes(artifact)
        self._loaded_backend = handle.getBackend()
        if not self._arg_tensors:
            _, self._arg_tensors, _ = self._flatten()

    def compile(self, handle: Handle, remove: bool = False) -> None:
        blob = self.compileToArtifact(handle.getBackend(), remove)
        self.loadFromArtifact(handle, blob)

    def _clear(self):
        if self._plan:
            lib().fb_plan_free(self._plan)
        self._plan = None
        self._artifact = None
        self._workspace = None
        self._ws_queried = False

    def getWorkspaceSize(self) -> Optional[int]:
        if not self._plan:
            return None
        n = _SZ(0)
        _check(lib().fb_plan_workspace_size(self._plan, ctypes.byref(n)))
        self._workspace = n.value
        self._ws_queried = True
        return n.value

    def numLaunches(self) -> int:
        n = _I32(0)
        _check(lib().fb_plan_num_launches(self._plan, ctypes.byref(n)))
        return n.value

    def statistics(self) -> str:
        need = _SZ(0)
        _check(lib().fb_plan_stats_json(self._plan, None, 0, ctypes.byref(need)))
        buf = ctypes.create_string_buffer(need.value)
        _check(lib().fb_plan_stats_json(self._plan, buf, need.value, ctypes.byref(need)))
        return buf.value.decode()

    # -- execute (runtime.h:383-529) ------------------------------------------------
    def execute(self, handle: Handle, variantPack: Dict[TensorAttr, Buffer],
                workspace: Optional[Buffer]) -> None:
        if not self._plan:
            raise FusilliError(ErrorCode.NotCompiled, "Graph must be compiled before being executed")
        if not self._ws_queried:
            raise FusilliError(ErrorCode.InvalidArgument,
                               "Graph::execute requires getWorkspaceSize() to be called before "
                               "workspace allocation and execution")
        for t in self.outputs:
            if t.isVirtual() and t in variantPack:
                raise FusilliError(ErrorCode.VariantPackError, "Virtual output tensor found in variantPack")
        for t in self.inputs:
            if t.isScalar() and t in variantPack:
                raise FusilliError(ErrorCode.VariantPackError, "Scalar constant tensor found in variantPack")
        n = len(self._arg_tensors)
        ptrs = (_VP * n)()
        sizes = (_SZ * n)()
        out_ids = {id(o) for o in self.outputs}
        for i, t in enumerate(self._arg_tensors):
            if t not in variantPack:
                which = "Output" if id(t) in out_ids else "Input"
                raise FusilliError(ErrorCode.VariantPackError, f"{which} tensor missing from variantPack")
            b = variantPack[t]
            ptrs[i] = b.ptr()
            sizes[i] = b.size()
        ws_ptr, ws_size = (workspace.ptr(), workspace.size()) if workspace is not None else (None, 0)
        if any(t.hasDynamicDims() for t in self._arg_tensors):
            dims = self._runtime_dims(variantPack)
            _check(lib().fb_plan_execute_shaped(self._plan, handle._ptr, ptrs, sizes, dims, n, ws_ptr, ws_size))
            return
        _check(lib().fb_plan_execute(self._plan, handle._ptr, ptrs, sizes, n, ws_ptr, ws_size))

    def bind(self, handle: Handle, variantPack: Dict[TensorAttr, Buffer], workspace: Optional[Buffer]) -> "BoundGraph":
        """Marshals `variantPack` and `workspace` once and returns an object whose `run()` enqueues the
        plan with them again and again. `execute` walks the pack, checks it and builds the C argument
        arrays on every call (tens of microseconds of Python); a loop over fixed buffers pays that once
        here and a single C call per iteration afterwards. The same checks apply as in `execute`; the
        buffers must stay alive and unchanged while the bound object is in use. (A convenience of this
        Python front end; the reference's C++ `Graph::execute` has no such cost to hide.)"""
        if not self._plan:
            raise FusilliError(ErrorCode.NotCompiled, "Graph must be compiled before being executed")
        if not self._ws_queried:
            raise FusilliError(ErrorCode.InvalidArgument,
                               "Graph::execute requires getWorkspaceSize() to be called before "
                               "workspace allocation and execution")
        if any(t.hasDynamicDims() for t in self._arg_tensors):
            raise FusilliError(ErrorCode.NotImplemented, "Graph.bind: graphs with dynamic dims go through execute()")
        for t in self.outputs:
            if t.isVirtual() and t in variantPack:
                raise FusilliError(ErrorCode.VariantPackError, "Virtual output tensor found in variantPack")
        for t in self.inputs:
            if t.isScalar() and t in variantPack:
                raise FusilliError(ErrorCode.VariantPackError, "Scalar constant tensor found in variantPack")
        n = len(self._arg_tensors)
        ptrs = (_VP * n)()
        sizes = (_SZ * n)()
        out_ids = {id(o) for o in self.outputs}
        keep = []
        for i, t in enumerate(self._arg_tensors):
            if t not in variantPack:
                which = "Output" if id(t) in out_ids else "Input"
                raise FusilliError(ErrorCode.VariantPackError, f"{which} tensor missing from variantPack")
            b = variantPack[t]
            ptrs[i] = b.ptr()
            sizes[i] = b.size()
            keep.append(b)
        ws_ptr, ws_size = (workspace.ptr(), workspace.size()) if workspace is not None else (None, 0)
        return BoundGraph(self, handle, ptrs, sizes, n, ws_ptr, ws_size, keep + [workspace])

    def _runtime_dims(self, variantPack):
        """FB_MAX_RANK logical extents per argument: a tensor's own dims, or for one with dynamic
        dims the shape of this call's buffer (physical order, as the reference's buffer views)."""
        n = len(self._arg_tensors)
        dims = (ctypes.c_int64 * (n * FB_MAX_RANK))(*([1] * (n * FB_MAX_RANK)))
        for i, t in enumerate(self._arg_tensors):
            logical = list(t.dim)
            if t.hasDynamicDims():
                shape = variantPack[t].shape
                if shape is None or len(shape) != len(logical):
                    raise FusilliError(ErrorCode.InvalidArgument,
                                       f"Buffer for tensor '{t.name}' carries no shape of rank {len(logical)}")
                for pos, src in enumerate(t.getLogicalToPhysicalPermuteOrder()):
                    logical[src] = int(shape[pos])
            for k, v in enumerate(logical):
                dims[i * FB_MAX_RANK + k] = v
        return dims

    def getWorkspaceSizeFor(self, variantPack) -> int:
        """Workspace bytes for the shapes of `variantPack`'s buffers (dynamic graphs)."""
        if not self._plan:
            raise FusilliError(ErrorCode.NotCompiled, "Graph must be compiled before being executed")
        out = _SZ()
        _check(lib().fb_plan_workspace_size_shaped(self._plan, self._runtime_dims(variantPack),
                                                   len(self._arg_tensors), ctypes.byref(out)))
        return out.value

    def __del__(self):
        try:
            self._clear()
        except Exception:
            pass


class BoundGraph:
    """A compiled graph with its buffers already marshalled (see Graph.bind)."""

    def __init__(self, graph, handle, ptrs, sizes, n, ws_ptr, ws_size, keep):
        self._graph, self._handle = graph, handle
        self._ptrs, self._sizes, self._n, self._ws_ptr, self._ws_size = ptrs, sizes, n, ws_ptr, ws_size
        self._keep = keep
        self._call = lib().fb_plan_execute

    def run(self) -> None:
        st = self._call(self._graph._plan, self._handle._ptr, self._ptrs, self._sizes, self._n, self._ws_ptr,
                        self._ws_size)
        if st != 0:
            _check(st)
