"""Data-type and reduction-operator tables under the reference's module name
(necklace/cuda/ncclwrp.py:48-81).  The reference maps names to ``pynccl`` enum values; the
numeric values are NCCL's own ``ncclDataType_t`` / ``ncclRedOp_t`` and are kept, and a second
pair of tables maps the same names to what this framework's collectives take (torch dtypes
and the operator strings of ``comm.fns``).  Environment defaults follow the reference
(``NCCL_DEBUG=WARN`` unless set)."""
from __future__ import annotations

import os

import torch

if not os.environ.get("NCCL_DEBUG"):
    os.environ["NCCL_DEBUG"] = "WARN"

# ncclDataType_t
ncclInt8 = ncclChar = 0
ncclUint8 = 1
ncclInt32 = ncclInt = 2
ncclUint32 = 3
ncclInt64 = 4
ncclUint64 = 5
ncclFloat16 = ncclHalf = 6
ncclFloat32 = ncclFloat = 7
ncclFloat64 = ncclDouble = 8
ncclBfloat16 = 9
# ncclRedOp_t
ncclSum, ncclProd, ncclMax, ncclMin = 0, 1, 2, 3

PYNCCL_DTYPE_MAP = {
    "char": ncclChar, "int8": ncclInt8, "uint8": ncclUint8, "int": ncclInt, "int32": ncclInt32,
    "uint32": ncclUint32, "long": ncclInt64, "int64": ncclInt64, "uint64": ncclUint64,
    "float16": ncclFloat16, "half": ncclHalf, "float": ncclFloat, "float32": ncclFloat32,
    "float64": ncclFloat64, "double": ncclDouble, "bfloat16": ncclBfloat16,
}
PYNCCL_REDUCE_OP_MAP = {"sum": ncclSum, "prod": ncclProd, "max": ncclMax, "min": ncclMin}

TORCH_DTYPE_MAP = {
    "char": torch.int8, "int8": torch.int8, "uint8": torch.uint8, "int": torch.int32,
    "int32": torch.int32, "uint32": torch.int32, "long": torch.int64, "int64": torch.int64,
    "uint64": torch.int64, "float16": torch.float16, "half": torch.float16,
    "float": torch.float32, "float32": torch.float32, "float64": torch.float64,
    "double": torch.float64, "bfloat16": torch.bfloat16,
}
REDUCE_OP_MAP = {"sum": "sum", "prod": "prod", "max": "max", "min": "min"}


def torch_dtype(name_or_code):
    """torch dtype for a reference dtype name or NCCL enum value."""
    if isinstance(name_or_code, str):
        return TORCH_DTYPE_MAP[name_or_code]
    for k, v in PYNCCL_DTYPE_MAP.items():
        if v == name_or_code:
            return TORCH_DTYPE_MAP[k]
    raise KeyError(name_or_code)
