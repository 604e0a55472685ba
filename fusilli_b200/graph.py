"""Python mirror of the Fusilli graph front end (builders, validation, inference).

The C++ headers under ``include/fusilli`` are the primary host side; this module
gives Python callers (tests, bench) the same surface with the same names and
the same error behaviour, and flattens a validated graph into the POD
descriptor that ``fb_plan_build`` consumes. It never computes anything.

Reference: include/fusilli/graph/graph.h:75-468 (Graph), :756-1193 (builders),
include/fusilli/attributes/tensor_attributes.h:374-809 (TensorAttr),
include/fusilli/node/*.h (validation and shape/stride inference).
"""
from __future__ import annotations

import enum
import math
from typing import Dict, List, Optional, Sequence


class ErrorCode(enum.IntEnum):
    """fusilli::ErrorCode (include/fusilli/support/logging.h:58-71)."""
    OK = 0
    NotImplemented = 1
    NotValidated = 2
    NotCompiled = 3
    AttributeNotSet = 4
    InternalError = 5
    InvalidAttribute = 6
    InvalidArgument = 7
    VariantPackError = 8
    CompileFailure = 9
    RuntimeFailure = 10
    FileSystemFailure = 11


class FusilliError(Exception):
    """Python stand-in for a non-OK fusilli::ErrorObject."""

    def __init__(self, code: ErrorCode, message: str):
        super().__init__(f"{code.name}: {message}")
        self.code = ErrorCode(code)
        self.message = message


def _require(cond: bool, code: ErrorCode, message: str) -> None:
    if not cond:
        raise FusilliError(code, message)


class DataType(enum.IntEnum):
    """fusilli::DataType (include/fusilli/attributes/types.h:27-47)."""
    NotSet = 0
    Half = 1
    BFloat16 = 2
    Float = 3
    Double = 4
    Uint8 = 5
    Int4 = 6
    Int8 = 7
    Int16 = 8
    Int32 = 9
    Int64 = 10
    Boolean = 11
    FP8E5M2 = 12


DTYPE_SIZE = {
    DataType.Half: 2, DataType.BFloat16: 2, DataType.Float: 4,
    DataType.Double: 8, DataType.Uint8: 1, DataType.Int8: 1,
    DataType.Int16: 2, DataType.Int32: 4, DataType.Int64: 8,
    DataType.Boolean: 1, DataType.FP8E5M2: 1,
}


def isIntegralOrBoolType(t: DataType) -> bool:
    return t in (DataType.Uint8, DataType.Int4, DataType.Int8, DataType.Int16,
                 DataType.Int32, DataType.Int64, DataType.Boolean)


class NormFwdPhase(enum.IntEnum):
    NOT_SET = 0
    TRAINING = 1
    INFERENCE = 2


class Op(enum.IntEnum):
    CONV_FPROP = 1
    CONV_DGRAD = 2
    CONV_WGRAD = 3
    MATMUL = 4
    SDPA = 5
    LAYERNORM = 6
    RMSNORM = 7
    REDUCTION = 8
    POINTWISE = 9
    BATCHNORM = 10


_PW_NAMES = (
    "NOT_SET ABS ADD ADD_SQUARE BINARY_SELECT CEIL CMP_EQ CMP_GE CMP_GT CMP_LE "
    "CMP_LT CMP_NEQ DIV ELU_FWD ERF EXP FLOOR GELU_APPROX_TANH_BWD "
    "GELU_APPROX_TANH_FWD GELU_BWD GELU_FWD IDENTITY LOG LOGICAL_AND LOGICAL_NOT "
    "LOGICAL_OR MAX_OP MIN_OP MUL NEG RECIPROCAL RELU_BWD RELU_FWD RSQRT "
    "SIGMOID_FWD SIN SOFTPLUS_FWD SQRT SUB SWISH_BWD SWISH_FWD TAN TANH_BWD "
    "TANH_FWD").split()
PointwiseMode = enum.IntEnum("PointwiseMode", {n: i for i, n in enumerate(_PW_NAMES)})
_RED_NAMES = "NOT_SET ADD SUM MUL MIN MAX AMAX AVG NORM1 NORM2 MUL_NO_ZEROS".split()
ReductionMode = enum.IntEnum("ReductionMode", {n: i for i, n in enumerate(_RED_NAMES)})

_PW_ARITY = {m: 1 for m in PointwiseMode}
for _n in ("ADD ADD_SQUARE CMP_EQ CMP_GE CMP_GT CMP_LE CMP_LT CMP_NEQ DIV "
           "GELU_APPROX_TANH_BWD GELU_BWD LOGICAL_AND LOGICAL_OR MAX_OP MIN_OP "
           "MUL RELU_BWD SUB SWISH_BWD TANH_BWD").split():
    _PW_ARITY[PointwiseMode[_n]] = 2
_PW_ARITY[PointwiseMode.BINARY_SELECT] = 3
_PW_BOOL_OUT = {PointwiseMode[n] for n in
                "CMP_EQ CMP_NEQ CMP_LT CMP_LE CMP_GT CMP_GE LOGICAL_AND LOGICAL_NOT LOGICAL_OR".split()}

FLAG_SDPA_CAUSAL, FLAG_SDPA_GQA, FLAG_SDPA_HAS_SCALE, FLAG_NORM_TRAINING = 1, 2, 4, 8


# --------------------------------------------------------------------------
# stride helpers (tensor_attributes.h:159-254)
# --------------------------------------------------------------------------
def getContiguousStrideOrder(n: int) -> List[int]:
    return [n - 1 - i for i in range(n)]


def getChannelsLastStrideOrder(n: int) -> List[int]:
    order = [0] * n
    nxt = 1
    for i in range(n - 1, 1, -1):
        order[i] = nxt
        nxt += 1
    order[0] = nxt
    return order


def generateStrideFromDim(dim: Sequence[int], order: Sequence[int]) -> List[int]:
    n = len(dim)
    by_rank = sorted(range(n), key=lambda i: order[i])
    stride = [0] * n
    acc = 1
    for i in by_rank:
        stride[i] = acc
        acc *= dim[i]
    return stride


def generateStrideOrderPreservingFormat(in_stride: Sequence[int], out_rank: int) -> List[int]:
    idx = sorted(range(len(in_stride)), key=lambda i: in_stride[i])
    order = [0] * len(in_stride)
    for rank, i in enumerate(idx):
        order[i] = rank
    order += list(range(len(in_stride), out_rank))
    return order


def contiguousStride(dim: Sequence[int]) -> List[int]:
    return generateStrideFromDim(dim, getContiguousStrideOrder(len(dim)))


def channelsLastStride(dim: Sequence[int]) -> List[int]:
    return generateStrideFromDim(dim, getChannelsLastStrideOrder(len(dim)))


def computeBroadcastShape(shapes: Sequence[Sequence[int]]) -> List[int]:
    shapes = [list(s) for s in shapes if len(s)]
    _require(bool(shapes), ErrorCode.InvalidAttribute, "All input shapes are empty")
    rank = max(len(s) for s in shapes)
    out = [1] * rank
    for s in shapes:
        for off in range(len(s)):
            ci, si = rank - 1 - off, len(s) - 1 - off
            if out[ci] == 1:
                out[ci] = s[si]
            _require(s[si] == 1 or out[ci] == s[si], ErrorCode.InvalidAttribute,
                     "Cannot broadcast two non unit dimensions")
    return out


class TensorAttr:
    """fusilli::TensorAttr (tensor_attributes.h:374-809)."""

    def __init__(self, scalar=None, dtype: Optional[DataType] = None):
        self.name = ""
        self.dataType = DataType.NotSet
        self.dim: List[int] = []
        self.stride: List[int] = []
        self._virtual = False
        self._scalar = False
        self.scalarValue = None
        self._dynamic: List[int] = []  # sorted, unique logical dim indices (tensor_attributes.h:512-570)
        if scalar is not None:
            self._scalar = True
            self.scalarValue = scalar
            self.dim = [1]
            self.stride = [1]
            if dtype is None:
                dtype = DataType.Float if isinstance(scalar, float) else DataType.Int32
            self.dataType = dtype

    # chainable setters -----------------------------------------------------
    def setName(self, name): self.name = name; return self
    def setDataType(self, t): self.dataType = DataType(t); return self
    def setDim(self, d): self.dim = [int(v) for v in d]; return self
    def setStride(self, s): self.stride = [int(v) for v in s]; return self
    def setIsVirtual(self, v): self._virtual = bool(v); return self
    def setOutput(self, v): return self.setIsVirtual(not v)
    def setIsScalar(self, v): self._scalar = bool(v); return self
    def setDynamicDim(self, index): return self.setDynamicDims(self._dynamic + [int(index)])
    def setDynamicDims(self, indices): self._dynamic = sorted({int(i) for i in indices}); return self
    def clearDynamicDims(self): self._dynamic = []; return self

    # getters -----------------------------------------------------------------
    def getName(self): return self.name
    def getDataType(self): return self.dataType
    def getDim(self): return self.dim
    def getStride(self): return self.stride
    def isVirtual(self): return self._virtual
    def isScalar(self): return self._scalar
    def getScalarValue(self): return self.scalarValue
    def getDynamicDims(self): return self._dynamic
    def hasDynamicDims(self): return bool(self._dynamic)
    def isDynamicDim(self, index): return int(index) in self._dynamic

    def getVolume(self) -> int:
        return math.prod(self.dim)

    def isContiguous(self) -> bool:
        return self.stride == contiguousStride(self.dim)

    def isChannelsLast(self) -> bool:
        return len(self.dim) >= 3 and self.stride == channelsLastStride(self.dim)

    def hasBroadcastDims(self) -> bool:
        return any(d > 1 and s == 0 for d, s in zip(self.dim, self.stride))

    def hasValidPhysicalRepresentation(self) -> bool:
        if len(self.dim) != len(self.stride):
            return False
        if any(s < 0 for s in self.stride):
            return False
        expected = 1
        for s, d in sorted(zip(self.stride, self.dim), key=lambda p: p[0]):
            if d == 1 or s == 0:
                continue
            if s != expected:
                return False
            expected = s * d
        return True

    def getLogicalToPhysicalPermuteOrder(self) -> List[int]:
        n = len(self.dim)
        perm = list(range(n))
        movable = [i for i in range(n) if self.dim[i] != 1 and self.stride[i] != 0]
        by_stride = sorted(movable, key=lambda i: -self.stride[i])
        for slot, src in zip(movable, by_stride):
            perm[slot] = src
        return perm

    def getPhysicalDim(self) -> List[int]:
        perm = self.getLogicalToPhysicalPermuteOrder()
        return [1 if (self.dim[p] > 1 and self.stride[p] == 0) else self.dim[p] for p in perm]

    def physicalVolume(self) -> int:
        return math.prod(self.getPhysicalDim())

    def fillFromContext(self, ctx: "Context"):
        if self.dataType == DataType.NotSet:
            self.dataType = ctx.intermediateDataType if self._virtual else ctx.ioDataType
        return self

    def validate(self) -> None:
        n = f"Tensor '{self.name}'"
        _require(bool(self.dim), ErrorCode.AttributeNotSet, n + " dims not set")
        _require(bool(self.stride), ErrorCode.AttributeNotSet, n + " strides not set")
        _require(len(self.dim) == len(self.stride), ErrorCode.InvalidAttribute,
                 n + " uses dim and stride of different dimensionality")
        for d in self._dynamic:
            _require(d < len(self.dim), ErrorCode.InvalidAttribute,
                     n + f" has dynamic dim index {d} out of range for rank {len(self.dim)}")
            _require(self.stride[d] != 0, ErrorCode.InvalidAttribute,
                     n + f" has dynamic dim at index {d} with stride 0 (broadcast stride), which "
                         "is not supported")
            _require(self.dim[d] != 1, ErrorCode.InvalidAttribute,
                     n + f" has dynamic dim at index {d} with representative size 1, which is "
                         "not supported")
        _require(not (self.hasBroadcastDims() and self.hasDynamicDims()), ErrorCode.InvalidAttribute,
                 n + " has dynamic dimensions on a tensor with broadcast strides, which is not supported")
        _require(self.hasValidPhysicalRepresentation(), ErrorCode.InvalidAttribute,
                 n + " has invalid physical representation. It must be a valid "
                     "permutation of the logical dimensions")
        _require(self.dataType != DataType.NotSet, ErrorCode.AttributeNotSet,
                 n + " data type not set")
        _require(not (self._virtual and self._scalar), ErrorCode.InvalidAttribute,
                 n + " cannot be both virtual (intermediate) and a scalar constant")
        _require(not (self.scalarValue is not None and not self._scalar),
                 ErrorCode.InvalidAttribute,
                 n + " has a scalar value set but is not marked as a scalar")
        _require(not (self.scalarValue is None and self._scalar), ErrorCode.InvalidAttribute,
                 n + " is marked as a scalar but does not have a scalar value set")


class Context:
    def __init__(self):
        self.name = ""
        self.ioDataType = DataType.NotSet
        self.computeDataType = DataType.NotSet
        self.intermediateDataType = DataType.NotSet


class _Attr:
    def __init__(self):
        self.name = ""
        self.computeDataType = DataType.NotSet

    def setName(self, n): self.name = n; return self
    def getName(self): return self.name
    def setComputeDataType(self, t): self.computeDataType = DataType(t); return self


class _ConvAttr(_Attr):
    def __init__(self):
        super().__init__()
        self.padding: List[int] = []
        self.stride: List[int] = []
        self.dilation: List[int] = []

    def setPadding(self, p): self.padding = list(p); return self
    def setStride(self, s): self.stride = list(s); return self
    def setDilation(self, d): self.dilation = list(d); return self
    def getPadding(self): return self.padding
    def getStride(self): return self.stride
    def getDilation(self): return self.dilation


class ConvFPropAttr(_ConvAttr): pass
class ConvDGradAttr(_ConvAttr): pass
class ConvWGradAttr(_ConvAttr): pass
class MatmulAttr(_Attr): pass


class SdpaAttr(_Attr):
    def __init__(self):
        super().__init__()
        self.dropout = 0.0
        self.isCausal = False
        self.scale: Optional[float] = None
        self.enableGqa = False

    def setDropout(self, p): self.dropout = float(p); return self
    def setIsCausal(self, v): self.isCausal = bool(v); return self
    def setScale(self, s): self.scale = s; return self
    def setEnableGqa(self, v): self.enableGqa = bool(v); return self


class _NormAttr(_Attr):
    def __init__(self):
        super().__init__()
        self.forwardPhase = NormFwdPhase.NOT_SET
        self.epsilon: Optional[TensorAttr] = None

    def setForwardPhase(self, p): self.forwardPhase = NormFwdPhase(p); return self
    def setEpsilon(self, e): self.epsilon = e; return self
    def getEpsilon(self): return self.epsilon
    def getForwardPhase(self): return self.forwardPhase


class LayernormAttr(_NormAttr): pass
class RmsnormAttr(_NormAttr): pass


class BatchnormAttr(_NormAttr):
    """attributes/batchnorm_attributes.h:27-90: epsilon and momentum are scalar tensors."""

    def __init__(self):
        super().__init__()
        self.momentum: Optional[TensorAttr] = None

    def setMomentum(self, m): self.momentum = m; return self
    def getMomentum(self): return self.momentum


class ReductionAttr(_Attr):
    Mode = ReductionMode

    def __init__(self):
        super().__init__()
        self.mode = ReductionMode.NOT_SET

    def setMode(self, m): self.mode = ReductionMode(m); return self
    def getMode(self): return self.mode


class PointwiseAttr(_Attr):
    Mode = PointwiseMode

    def __init__(self):
        super().__init__()
        self.mode = PointwiseMode.NOT_SET
        self.eluAlpha = 1.0
        self.softplusBeta = 1.0
        self.softplusThreshold = 20.0
        self.swishBeta = 1.0

    def setMode(self, m): self.mode = PointwiseMode(m); return self
    def getMode(self): return self.mode
    def setEluAlpha(self, a): self.eluAlpha = float(a); return self
    def setSoftplusBeta(self, b): self.softplusBeta = float(b); return self
    def setSoftplusThreshold(self, t): self.softplusThreshold = float(t); return self
    def setSwishBeta(self, b): self.swishBeta = float(b); return self


class Node:
    """One appended op: kind, attribute bag, input and output tensors."""

    def __init__(self, op: Op, attr: _Attr, inputs, outputs):
        self.op = op
        self.attr = attr
        self.inputs: List[Optional[TensorAttr]] = list(inputs)
        self.outputs: List[Optional[TensorAttr]] = list(outputs)

    @property
    def name(self): return self.attr.name


def getConvInferredOutputShape(xDim, wDim, dilation, padding, stride):
    """node/conv_node.h:38-56."""
    y = [xDim[0], wDim[0]]
    for i in range(2, len(xDim)):
        j = i - 2
        y.append(1 + (xDim[i] - (wDim[i] - 1) * dilation[j] + 2 * padding[j] - 1) // stride[j])
    return y


def getMatmulInferredOutputShape(aDim, bDim):
    """node/matmul_node.h:40-66."""
    r = len(aDim)
    return [max(aDim[i], bDim[i]) for i in range(r - 2)] + [aDim[r - 2], bDim[r - 1]]


def _layout_ok(t: TensorAttr) -> bool:
    return t.isContiguous() or t.isChannelsLast()


def _not_cl(t: TensorAttr) -> str:
    return (f"Tensor '{t.name}' is neither contiguous nor channels-last as defined by its stride")


class GraphBase:
    """Builders + validation; the device-facing half lives in fusilli_b200.runtime.Graph."""

    def __init__(self):
        self.context = Context()
        self.nodes: List[Node] = []
        self.inputs: List[TensorAttr] = []
        self.outputs: List[TensorAttr] = []
        self._validated = False

    # context ----------------------------------------------------------------
    def setName(self, n): self.context.name = n; return self
    def getName(self): return self.context.name
    def setIODataType(self, t): self.context.ioDataType = DataType(t); return self
    def setComputeDataType(self, t): self.context.computeDataType = DataType(t); return self
    def setIntermediateDataType(self, t): self.context.intermediateDataType = DataType(t); return self

    # builders (graph.h:756-1193) ---------------------------------------------
    def tensor(self, t: TensorAttr) -> TensorAttr:
        self.inputs.append(t)
        return t

    def _out(self, name: str) -> TensorAttr:
        t = TensorAttr().setName(name).setIsVirtual(True)
        self.outputs.append(t)
        return t

    def _auto(self, attr: _Attr, prefix: str, named: Dict[str, Optional[TensorAttr]]):
        if not attr.name:
            attr.setName(f"{prefix}_{len(self.nodes)}")
        for suffix, t in named.items():
            if t is not None and not t.name:
                t.setName(f"{attr.name}_{suffix}")

    def convFProp(self, x, w, attr: ConvFPropAttr):
        self._auto(attr, "conv_fprop", {"X": x, "W": w})
        y = self._out(attr.name + "_Y")
        self.nodes.append(Node(Op.CONV_FPROP, attr, [x, w], [y]))
        return y

    def convWGrad(self, dy, x, attr: ConvWGradAttr):
        self._auto(attr, "conv_wgrad", {"DY": dy, "X": x})
        dw = self._out(attr.name + "_DW")
        self.nodes.append(Node(Op.CONV_WGRAD, attr, [dy, x], [dw]))
        return dw

    def convDGrad(self, dy, w, attr: ConvDGradAttr):
        self._auto(attr, "conv_dgrad", {"DY": dy, "W": w})
        dx = self._out(attr.name + "_DX")
        self.nodes.append(Node(Op.CONV_DGRAD, attr, [dy, w], [dx]))
        return dx

    def matmul(self, a, b, attr: MatmulAttr):
        self._auto(attr, "matmul", {"A": a, "B": b})
        c = self._out(attr.name + "_C")
        self.nodes.append(Node(Op.MATMUL, attr, [a, b], [c]))
        return c

    def sdpa(self, q, k, v, mask, attr: SdpaAttr):
        self._auto(attr, "sdpa", {"Q": q, "K": k, "V": v, "MASK": mask})
        o = self._out(attr.name + "_O")
        self.nodes.append(Node(Op.SDPA, attr, [q, k, v, mask], [o]))
        return o

    def layernorm(self, x, scale, bias, attr: LayernormAttr):
        self._auto(attr, "layernorm", {"X": x, "SCALE": scale, "BIAS": bias,
                                       "EPSILON": attr.epsilon})
        y = self._out(attr.name + "_Y")
        m = v = None
        if attr.forwardPhase == NormFwdPhase.TRAINING:
            m = self._out(attr.name + "_MEAN")
            v = self._out(attr.name + "_INV_VARIANCE")
        self.nodes.append(Node(Op.LAYERNORM, attr, [x, scale, bias, attr.epsilon], [y, m, v]))
        return y, m, v

    def batchnorm(self, x, scale, bias, mean, var, attr: BatchnormAttr):
        """graph.h:857-912: Y always; SAVED_MEAN and SAVED_INV_VARIANCE in the training phase."""
        self._auto(attr, "batchnorm", {"X": x, "SCALE": scale, "BIAS": bias, "MEAN": mean, "VAR": var,
                                       "EPSILON": attr.epsilon, "MOMENTUM": attr.momentum})
        y = self._out(attr.name + "_Y")
        sm = si = None
        if attr.forwardPhase == NormFwdPhase.TRAINING:
            sm = self._out(attr.name + "_SAVED_MEAN")
            si = self._out(attr.name + "_SAVED_INV_VARIANCE")
        self.nodes.append(Node(Op.BATCHNORM, attr, [x, scale, bias, mean, var, attr.epsilon, attr.momentum],
                               [y, sm, si]))
        return y, sm, si

    def rmsnorm(self, x, scale, attr: RmsnormAttr):
        self._auto(attr, "rmsnorm", {"X": x, "SCALE": scale, "EPSILON": attr.epsilon})
        y = self._out(attr.name + "_Y")
        r = None
        if attr.forwardPhase == NormFwdPhase.TRAINING:
            r = self._out(attr.name + "_INV_RMS")
        self.nodes.append(Node(Op.RMSNORM, attr, [x, scale, attr.epsilon], [y, r]))
        return y, r

    def reduction(self, x, attr: ReductionAttr):
        self._auto(attr, "reduction", {"X": x})
        y = self._out(attr.name + "_Y")
        self.nodes.append(Node(Op.REDUCTION, attr, [x], [y]))
        return y

    def pointwise(self, in0, *rest):
        *more, attr = rest
        ins = [in0] + list(more)
        self._auto(attr, "pointwise", {f"IN_{i}": t for i, t in enumerate(ins)})
        out = self._out(attr.name + "_OUT_0")
        self.nodes.append(Node(Op.POINTWISE, attr, ins + [None] * (3 - len(ins)), [out]))
        return out

    # validation (graph.h:80-113, node.h:84-91) ---------------------------------
    def validate(self) -> None:
        _require(bool(self.context.name), ErrorCode.AttributeNotSet, "Graph name not set")
        used = set()
        for t in self.inputs + self.outputs:
            _require(t.name not in used, ErrorCode.InvalidAttribute,
                     f"Symbol name '{t.name}' already in use")
            used.add(t.name)
        for n in self.nodes:
            _require(n.name not in used, ErrorCode.InvalidAttribute,
                     f"Symbol name '{n.name}' already in use")
            used.add(n.name)
        for n in self.nodes:
            _VALIDATORS[n.op](self, n)
        for t in self.inputs:
            t.validate()
        for t in self.outputs:
            t.validate()
            _require(not t.hasBroadcastDims(), ErrorCode.InvalidAttribute,
                     f"Tensor '{t.name}' has broadcast strides (stride=0) on an operation "
                     "output, which is not yet supported")
        self._validated = True

    def _fill(self, n: Node) -> None:
        if n.attr.computeDataType == DataType.NotSet:
            n.attr.computeDataType = self.context.computeDataType
        for t in n.inputs + n.outputs:
            if t is not None:
                t.fillFromContext(self.context)


# ---- per-node validation + inference ---------------------------------------
def _v_conv_common(nm, attr, rank):
    _require(bool(attr.padding), ErrorCode.AttributeNotSet, f"{nm} padding not set")
    _require(bool(attr.stride), ErrorCode.AttributeNotSet, f"{nm} stride not set")
    _require(bool(attr.dilation), ErrorCode.AttributeNotSet, f"{nm} dilation not set")
    ns = rank - 2
    _require(len(attr.padding) == ns, ErrorCode.InvalidAttribute,
             f"{nm} padding size does not match number of spatial dimensions")
    _require(len(attr.stride) == ns, ErrorCode.InvalidAttribute,
             f"{nm} stride size does not match number of spatial dimensions")
    _require(len(attr.dilation) == ns, ErrorCode.InvalidAttribute,
             f"{nm} dilation size does not match number of spatial dimensions")


def _v_groups(nm, inC, outC, fC, in_name="input", out_name="output"):
    filt = "filter" if in_name == "input" else "filter (W)"
    _require(inC % fC == 0, ErrorCode.InvalidAttribute,
             f"{nm} {in_name} channels must be divisible by the {filt} channels")
    g = inC // fC
    _require(0 < g <= inC and g <= outC, ErrorCode.InvalidAttribute,
             f"{nm} group count must be greater than 0 and less than or equal to the "
             "numbers of input and outputs channels")
    _require(outC % g == 0, ErrorCode.InvalidAttribute,
             f"{nm} {out_name} channels must be divisible by the group count")


def _v_conv_fprop(g: GraphBase, n: Node):
    x, w = n.inputs[:2]
    y = n.outputs[0]
    a = n.attr
    _require(x is not None, ErrorCode.AttributeNotSet, "Conv input tensor X not set")
    _require(w is not None, ErrorCode.AttributeNotSet, "Conv weight tensor W not set")
    _require(len(x.dim) >= 3, ErrorCode.InvalidAttribute,
             "Conv input tensor X must have a rank of at least 3")
    _require(len(x.dim) == len(w.dim), ErrorCode.InvalidAttribute,
             "Conv input tensor X and weight tensor W have different ranks")
    _v_conv_common("Conv", a, len(x.dim))
    _require(_layout_ok(x), ErrorCode.NotImplemented, _not_cl(x))
    _require(_layout_ok(w), ErrorCode.NotImplemented, _not_cl(w))
    _v_groups("Conv", x.dim[1], w.dim[0], w.dim[1])
    g._fill(n)
    if not y.dim:
        y.setDim(getConvInferredOutputShape(x.dim, w.dim, a.dilation, a.padding, a.stride))
    if not y.stride:
        y.setStride(contiguousStride(y.dim) if x.isContiguous() else channelsLastStride(y.dim))
    _require(y.dim == getConvInferredOutputShape(x.dim, w.dim, a.dilation, a.padding, a.stride),
             ErrorCode.InvalidAttribute,
             "Conv output tensor Y dimensions do not match the expected shapes inferred "
             "based on the input and weight dimensions")
    _require(_layout_ok(y), ErrorCode.NotImplemented, _not_cl(y))


def _v_conv_wgrad(g: GraphBase, n: Node):
    dy, x = n.inputs[:2]
    dw = n.outputs[0]
    a = n.attr
    _require(dy is not None, ErrorCode.AttributeNotSet, "ConvWGrad gradient tensor DY not set")
    _require(x is not None, ErrorCode.AttributeNotSet, "ConvWGrad input tensor X not set")
    _require(len(dy.dim) >= 3 and len(x.dim) >= 3, ErrorCode.InvalidAttribute,
             "ConvWGrad input tensors DY/X must have a rank of at least 3")
    _require(len(dy.dim) == len(x.dim), ErrorCode.InvalidAttribute,
             "ConvWGrad tensors DY and X have different ranks")
    _v_conv_common("ConvWGrad", a, len(x.dim))
    _require(_layout_ok(dy), ErrorCode.NotImplemented, _not_cl(dy))
    _require(_layout_ok(x), ErrorCode.NotImplemented, _not_cl(x))
    _require(len(dw.dim) >= 3, ErrorCode.InvalidAttribute,
             "ConvWGrad weight gradient tensor DW must have a rank of at least 3")
    _v_groups("ConvWGrad", x.dim[1], dy.dim[1], dw.dim[1], "input (X)", "output (DY)")
    g._fill(n)
    if not dw.stride:
        dw.setStride(contiguousStride(dw.dim) if dy.isContiguous() else channelsLastStride(dw.dim))
    _require(dy.dim == getConvInferredOutputShape(x.dim, dw.dim, a.dilation, a.padding, a.stride),
             ErrorCode.InvalidAttribute,
             "ConvWGrad output DW dimensions do not match the expected shapes inferred "
             "based on input dimensions")
    _require(_layout_ok(dw), ErrorCode.NotImplemented, _not_cl(dw))


def _v_conv_dgrad(g: GraphBase, n: Node):
    dy, w = n.inputs[:2]
    dx = n.outputs[0]
    a = n.attr
    _require(dy is not None, ErrorCode.AttributeNotSet, "ConvDGrad gradient tensor DY not set")
    _require(w is not None, ErrorCode.AttributeNotSet, "ConvDGrad input tensor W not set")
    _require(len(dy.dim) >= 3, ErrorCode.InvalidAttribute,
             "ConvDGrad input tensors DY/W must have a rank of at least 3")
    _require(len(dy.dim) == len(w.dim), ErrorCode.InvalidAttribute,
             "ConvDGrad tensors DY and W have different ranks")
    _v_conv_common("ConvDGrad", a, len(dy.dim))
    _require(_layout_ok(dy), ErrorCode.NotImplemented, _not_cl(dy))
    _require(_layout_ok(w), ErrorCode.NotImplemented, _not_cl(w))
    _require(len(dx.dim) >= 3, ErrorCode.InvalidAttribute,
             "ConvDGrad input gradient DX must have a rank of at least 3")
    _v_groups("ConvDGrad", dx.dim[1], w.dim[0], w.dim[1], "input (DX)", "output (DY)")
    g._fill(n)
    if not dx.stride:
        dx.setStride(contiguousStride(dx.dim) if dy.isContiguous() else channelsLastStride(dx.dim))
    _require(len(dy.dim) == len(dx.dim), ErrorCode.InvalidAttribute,
             "ConvDGrad tensors DY and DX have different ranks")
    _require(dy.dim == getConvInferredOutputShape(dx.dim, w.dim, a.dilation, a.padding, a.stride),
             ErrorCode.InvalidAttribute,
             "ConvDGrad DY dimensions do not match the expected shapes inferred based on DX and W")
    _require(_layout_ok(dx), ErrorCode.NotImplemented, _not_cl(dx))


def _batch_outermost(t: TensorAttr, nm: str):
    perm = t.getLogicalToPhysicalPermuteOrder()
    for i in range(len(t.dim) - 2):
        _require(perm[i] == i, ErrorCode.InvalidAttribute,
                 f"Matmul tensor {nm} has batch dimensions that are not outermost or are transposed")


def _v_matmul(g: GraphBase, n: Node):
    a, b = n.inputs[:2]
    c = n.outputs[0]
    _require(a is not None, ErrorCode.AttributeNotSet, "Matmul input tensor A not set")
    _require(b is not None, ErrorCode.AttributeNotSet, "Matmul input tensor B not set")
    ra, rb = len(a.dim), len(b.dim)
    _require(ra >= 2, ErrorCode.InvalidAttribute, "Matmul input tensor A must have a rank of at least 2")
    _require(rb >= 2, ErrorCode.InvalidAttribute, "Matmul input tensor B must have a rank of at least 2")
    _require(ra == rb, ErrorCode.InvalidAttribute,
             f"Matmul input tensors A and B must have the same rank: A has rank={ra}, B has rank={rb}")
    _require(a.dim[-1] == b.dim[-2], ErrorCode.InvalidAttribute,
             "Matmul input tensors A and B have incompatible inner dimensions (K): "
             f"A has K={a.dim[-1]}, B has K={b.dim[-2]}")
    for i in range(ra - 2):
        _require(a.dim[i] % b.dim[i] == 0 or b.dim[i] % a.dim[i] == 0, ErrorCode.InvalidAttribute,
                 "Matmul input tensors A and B have incompatible batch dimensions for "
                 f"broadcasting at index {i}: A has dim={a.dim[i]}, B has dim={b.dim[i]}")
    _batch_outermost(a, "A")
    _batch_outermost(b, "B")
    g._fill(n)
    if a.dataType != b.dataType:
        _require(ra == 3, ErrorCode.InvalidAttribute,
                 "Mixed precision matmul is only supported when input tensors A and B "
                 f"are of rank 3 (single batch dim): A and B have rank={ra}")
        _require(a.dim[0] == b.dim[0], ErrorCode.InvalidAttribute,
                 "Mixed precision matmul input tensors A and B must have exactly equal "
                 "batch dimensions (no broadcast)")
    if not c.dim:
        c.setDim(getMatmulInferredOutputShape(a.dim, b.dim))
    if not c.stride:
        c.setStride(contiguousStride(c.dim))
    _require(c.dim == getMatmulInferredOutputShape(a.dim, b.dim), ErrorCode.InvalidAttribute,
             "Matmul output tensor C dimensions do not match the expected shapes inferred "
             "based on the input dimensions")
    _batch_outermost(c, "C")


def _v_sdpa(g: GraphBase, n: Node):
    q, k, v, mask = n.inputs
    o = n.outputs[0]
    a: SdpaAttr = n.attr
    _require(q is not None, ErrorCode.AttributeNotSet, "SDPA input tensor Q not set")
    _require(k is not None, ErrorCode.AttributeNotSet, "SDPA input tensor K not set")
    _require(v is not None, ErrorCode.AttributeNotSet, "SDPA input tensor V not set")
    for t, nm, hd in ((q, "Q", "heads_q, seq_q"), (k, "K", "heads_kv, seq_kv"), (v, "V", "heads_kv, seq_kv")):
        _require(len(t.dim) == 4, ErrorCode.InvalidAttribute,
                 f"SDPA input tensor {nm} must be rank 4 [batch, {hd}, head_dim]")
    _require(q.dim[0] == k.dim[0] == v.dim[0], ErrorCode.InvalidAttribute,
             "SDPA input tensors Q, K, V must have matching batch dimension")
    _require(q.dim[3] == k.dim[3], ErrorCode.InvalidAttribute,
             "SDPA input tensors Q and K must have matching head_dim")
    _require(k.dim[2] == v.dim[2], ErrorCode.InvalidAttribute,
             "SDPA input tensors K and V must have matching sequence length")
    hq, hk, hv = q.dim[1], k.dim[1], v.dim[1]
    if a.enableGqa:
        _require(hq % hk == 0, ErrorCode.InvalidAttribute,
                 f"SDPA with GQA requires Q heads ({hq}) to be a multiple of K heads ({hk})")
        _require(hq % hv == 0, ErrorCode.InvalidAttribute,
                 f"SDPA with GQA requires Q heads ({hq}) to be a multiple of V heads ({hv})")
    else:
        _require(hq == hk, ErrorCode.InvalidAttribute,
                 f"SDPA without GQA requires Q heads ({hq}) to equal K heads ({hk})")
        _require(hq == hv, ErrorCode.InvalidAttribute,
                 f"SDPA without GQA requires Q heads ({hq}) to equal V heads ({hv})")
    _require(not (mask is not None and a.isCausal), ErrorCode.InvalidAttribute,
             "SDPA attention mask and is_causal are mutually exclusive")
    if mask is not None:
        _require(len(mask.dim) == 4, ErrorCode.InvalidAttribute, "SDPA attention mask must be rank 4")
        full = [q.dim[0], hq, q.dim[2], k.dim[2]]
        what = ["batch dim", "heads dim", "seq_q dim", "seq_kv dim"]
        match = ["input batch", "Q heads", "Q sequence length", "KV sequence length"]
        for i in range(4):
            _require(mask.dim[i] in (1, full[i]), ErrorCode.InvalidAttribute,
                     f"SDPA attention mask {what[i]} ({mask.dim[i]}) must be 1 or match {match[i]} ({full[i]})")
    _require(0.0 <= a.dropout < 1.0, ErrorCode.InvalidAttribute,
             "SDPA dropout probability must be in [0, 1)")
    g._fill(n)
    odim = [q.dim[0], q.dim[1], q.dim[2], v.dim[3]]
    if not o.dim:
        o.setDim(odim)
    if not o.stride:
        o.setStride(contiguousStride(odim))
    _require(o.dim == odim, ErrorCode.InvalidAttribute,
             "SDPA output tensor O dimensions do not match expected shape "
             "[batch, headsQ, seqQ, headDim]")


def _scale_bias_infer(t: TensorAttr, x: TensorAttr):
    if not t.dim:
        t.setDim([1] + list(x.dim[1:]))
    if not t.stride:
        t.setStride(generateStrideFromDim(t.dim, generateStrideOrderPreservingFormat(x.stride, len(t.dim))))


def _v_norm(g: GraphBase, n: Node, nm: str):
    a: _NormAttr = n.attr
    x = n.inputs[0]
    y = n.outputs[0]
    _require(a.forwardPhase != NormFwdPhase.NOT_SET, ErrorCode.AttributeNotSet,
             f"{nm} forward phase not set")
    _require(x is not None, ErrorCode.AttributeNotSet, f"{nm} input tensor X not set")
    _require(len(x.dim) >= 2, ErrorCode.InvalidAttribute,
             f"{nm} input tensor X must have a rank of at least 2")
    _require(_layout_ok(x), ErrorCode.NotImplemented, _not_cl(x))
    affine = n.inputs[1:3] if n.op == Op.LAYERNORM else n.inputs[1:2]
    for t, tn in zip(affine, ("SCALE", "BIAS")):
        if t is None:
            continue
        if t.dim:
            _require(t.dim == [1] + list(x.dim[1:]), ErrorCode.InvalidAttribute,
                     f"{nm} input tensor {tn} must have shape as tensor X with single batch")
        if t.stride:
            _require(_layout_ok(t), ErrorCode.NotImplemented, _not_cl(t))
    eps = a.epsilon
    _require(eps is not None, ErrorCode.AttributeNotSet, f"{nm} epsilon not set")
    _require(eps.isScalar(), ErrorCode.InvalidAttribute, f"{nm} epsilon must be a scalar constant")
    if n.op == Op.RMSNORM:
        _require(a.forwardPhase != NormFwdPhase.TRAINING, ErrorCode.NotImplemented,
                 "RmsNorm training mode is not yet supported: torch-mlir does not lower the "
                 "training variant")
    g._fill(n)
    for t in affine:
        if t is not None:
            _scale_bias_infer(t, x)
    if not y.dim:
        y.setDim(x.dim)
    if not y.stride:
        y.setStride(x.stride)
    _require(y.dim == x.dim, ErrorCode.InvalidAttribute,
             f"{nm} output Y tensor must have the same shape as input X tensor")
    _require(_layout_ok(y), ErrorCode.NotImplemented, _not_cl(y))
    if n.op == Op.LAYERNORM and a.forwardPhase == NormFwdPhase.TRAINING:
        sd = [x.dim[0]] + [1] * (len(x.dim) - 1)
        ss = contiguousStride(sd)
        for t, tn in zip(n.outputs[1:3], ("MEAN", "INV_VARIANCE")):
            if not t.dim:
                t.setDim(sd)
            if not t.stride:
                t.setStride(ss)
            _require(t.dim == sd, ErrorCode.InvalidAttribute,
                     f"{nm} output {tn} tensor must have shape [B, 1, ..., 1]")
            _require(t.stride == ss, ErrorCode.InvalidAttribute,
                     f"{nm} output {tn} tensor must have unit strides")


def _v_reduction(g: GraphBase, n: Node):
    a: ReductionAttr = n.attr
    x = n.inputs[0]
    y = n.outputs[0]
    _require(a.mode != ReductionMode.NOT_SET, ErrorCode.AttributeNotSet, "Reduction mode not set")
    _require(x is not None, ErrorCode.AttributeNotSet, "Reduction operation requires X input")
    _require(bool(x.dim), ErrorCode.AttributeNotSet, "Reduction input X dimensions not set")
    g._fill(n)
    if not y.dim:
        y.setDim(x.dim)
    if not y.stride:
        y.setStride(contiguousStride(y.dim))
    _require(len(x.dim) == len(y.dim), ErrorCode.InvalidAttribute,
             "Reduction input and output must have the same rank")
    _require(not (a.mode == ReductionMode.AVG and
                  (isIntegralOrBoolType(x.dataType) or isIntegralOrBoolType(y.dataType))),
             ErrorCode.InvalidAttribute,
             "Reduction AVG is not supported for integral or boolean tensors")
    for i, (xd, yd) in enumerate(zip(x.dim, y.dim)):
        _require(yd == 1 or yd == xd, ErrorCode.InvalidAttribute,
                 f"Reduction output dimension {i} must be 1 or match input dimension")
    _require(any(yd == 1 and xd > 1 for xd, yd in zip(x.dim, y.dim)), ErrorCode.InvalidAttribute,
             "Reduction requires at least one dimension to reduce (Y[i] == 1 where X[i] > 1)")


def _v_pointwise(g: GraphBase, n: Node):
    a: PointwiseAttr = n.attr
    _require(a.mode != PointwiseMode.NOT_SET, ErrorCode.AttributeNotSet, "Pointwise mode not set")
    need = _PW_ARITY[a.mode]
    for i in range(3):
        has = n.inputs[i] is not None
        if i < need:
            _require(has, ErrorCode.AttributeNotSet, f"{a.mode.name} mode requires IN_{i} input")
        else:
            _require(not has, ErrorCode.InvalidAttribute,
                     f"{a.mode.name} mode should not have IN_{i} input set")
    out = n.outputs[0]
    if a.mode in _PW_BOOL_OUT:
        out.setDataType(DataType.Boolean)
    g._fill(n)
    ins = [t for t in n.inputs if t is not None]
    if not out.dim:
        out.setDim(computeBroadcastShape([t.dim for t in ins]))
    if not out.stride:
        for t in ins:
            if t.dim == out.dim:
                out.setStride(t.stride)
                break
        if not out.stride and out.isVirtual():
            out.setStride(generateStrideFromDim(
                out.dim, generateStrideOrderPreservingFormat(ins[0].stride, len(out.dim))))
        _require(bool(out.stride), ErrorCode.InvalidAttribute,
                 "Pointwise output strides could not be computed")


def _v_batchnorm(g: GraphBase, n: Node):
    """node/batchnorm_node.h:52-236."""
    a: BatchnormAttr = n.attr
    x, scale, bias, mean, var = n.inputs[:5]
    y, sm, si = n.outputs
    training = a.forwardPhase == NormFwdPhase.TRAINING
    _require(a.forwardPhase != NormFwdPhase.NOT_SET, ErrorCode.AttributeNotSet, "BatchNorm forward phase not set")
    _require(x is not None, ErrorCode.AttributeNotSet, "BatchNorm input tensor X not set")
    _require(y is not None, ErrorCode.AttributeNotSet, "BatchNorm output tensor Y not set")
    _require(len(x.dim) >= 2, ErrorCode.InvalidAttribute, "BatchNorm input tensor X must have a rank of at least 2")
    _require(_layout_ok(x), ErrorCode.NotImplemented, _not_cl(x))
    if not training:
        _require(mean is not None, ErrorCode.AttributeNotSet, "BatchNorm inference requires running MEAN")
        _require(var is not None, ErrorCode.AttributeNotSet, "BatchNorm inference requires running VAR")
        _require(sm is None, ErrorCode.InvalidAttribute, "BatchNorm SAVED_MEAN should not be set in inference mode")
        _require(si is None, ErrorCode.InvalidAttribute,
                 "BatchNorm SAVED_INV_VARIANCE should not be set in inference mode")
    else:
        _require(sm is not None, ErrorCode.AttributeNotSet, "BatchNorm training requires SAVED_MEAN output")
        _require(si is not None, ErrorCode.AttributeNotSet, "BatchNorm training requires SAVED_INV_VARIANCE output")
    _require(a.epsilon is not None, ErrorCode.AttributeNotSet, "BatchNorm epsilon not set")
    _require(a.epsilon.isScalar(), ErrorCode.InvalidAttribute, "BatchNorm epsilon must be a scalar constant")
    _require(a.momentum is not None, ErrorCode.AttributeNotSet, "BatchNorm momentum not set")
    _require(a.momentum.isScalar(), ErrorCode.InvalidAttribute, "BatchNorm momentum must be a scalar constant")
    g._fill(n)
    per_channel = [(scale, "SCALE"), (bias, "BIAS"), (mean, "MEAN"), (var, "VAR")]
    if training:
        per_channel += [(sm, "SAVED_MEAN"), (si, "SAVED_INV_VARIANCE")]
    for t, _ in per_channel:
        if t is None:
            continue
        if not t.dim:
            t.setDim([x.dim[1]])
        if not t.stride:
            t.setStride([1])
    if not y.dim:
        y.setDim(x.dim)
    if not y.stride:
        y.setStride(x.stride)
    _require(y.dim == x.dim, ErrorCode.InvalidAttribute,
             "BatchNorm output Y tensor must have the same shape as input X tensor")
    _require(_layout_ok(y), ErrorCode.NotImplemented, _not_cl(y))
    for t, tn in per_channel:
        if t is None:
            continue
        _require(t.dim == [x.dim[1]], ErrorCode.InvalidAttribute,
                 f"BatchNorm tensor {tn} must be 1D with size equal to channel dimension C")
        _require(t.stride == [1], ErrorCode.InvalidAttribute, f"BatchNorm tensor {tn} must have unit stride")


_VALIDATORS = {
    Op.CONV_FPROP: _v_conv_fprop,
    Op.CONV_DGRAD: _v_conv_dgrad,
    Op.CONV_WGRAD: _v_conv_wgrad,
    Op.MATMUL: _v_matmul,
    Op.SDPA: _v_sdpa,
    Op.LAYERNORM: lambda g, n: _v_norm(g, n, "LayerNorm"),
    Op.RMSNORM: lambda g, n: _v_norm(g, n, "RmsNorm"),
    Op.REDUCTION: _v_reduction,
    Op.POINTWISE: _v_pointwise,
    Op.BATCHNORM: _v_batchnorm,
}
