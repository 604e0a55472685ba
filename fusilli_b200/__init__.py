"""fusilli_b200: B200 (sm_100a) execution backend behind the Fusilli graph API.

Python surface = the reference's C++ surface with the same names
(Graph, TensorAttr, *Attr, Handle, Buffer, DataType, ErrorCode); all compute runs
in libfusilli_b200.so through the C ABI declared in include/fusilli_b200.h.
"""
from .graph import (ConvDGradAttr, ConvFPropAttr, ConvWGradAttr, DataType, ErrorCode, FusilliError,
                    BatchnormAttr, LayernormAttr, MatmulAttr, NormFwdPhase, PointwiseAttr, ReductionAttr, RmsnormAttr,
                    SdpaAttr, TensorAttr, channelsLastStride, contiguousStride)
from .comm import Comm
from .runtime import Backend, Buffer, Graph, Handle

__all__ = [
    "Backend", "Buffer", "Comm", "ConvDGradAttr", "ConvFPropAttr", "ConvWGradAttr", "DataType", "ErrorCode",
    "BatchnormAttr", "FusilliError", "Graph", "Handle", "LayernormAttr", "MatmulAttr", "NormFwdPhase", "PointwiseAttr",
    "ReductionAttr", "RmsnormAttr", "SdpaAttr", "TensorAttr", "channelsLastStride", "contiguousStride",
]
