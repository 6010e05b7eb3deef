"""dtype tables: torch <-> numpy, torch <-> integer ids used when tensor
structures are exchanged between workers.  NumPy-2 safe and bf16-aware (the
reference maps bf16 to a dummy ``np.uint32`` and uses the removed
``np.bool8``, ``src/distdl/utilities/dtype.py:31-55``)."""
from __future__ import annotations

import numpy as np
import torch

torch_to_numpy_dtype_dict = {
    torch.bool: np.bool_,
    torch.uint8: np.uint8,
    torch.int8: np.int8,
    torch.int16: np.int16,
    torch.int32: np.int32,
    torch.int64: np.int64,
    torch.float16: np.float16,
    torch.float32: np.float32,
    torch.float64: np.float64,
    torch.complex64: np.complex64,
    torch.complex128: np.complex128,
}
numpy_to_torch_dtype_dict = {np.dtype(v): k for k, v in torch_to_numpy_dtype_dict.items()}

# Stable integer ids (never renumber: they travel in structure handshakes).
_ID_ORDER = [torch.bool, torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64, torch.float16,
             torch.float32, torch.float64, torch.complex64, torch.complex128, torch.bfloat16]
torch_to_intID_dtype_dict = {dt: i + 1 for i, dt in enumerate(_ID_ORDER)}
intID_to_torch_dtype_dict = {i: dt for dt, i in torch_to_intID_dtype_dict.items()}
# id 0 means "no tensor here"
intID_to_torch_dtype_dict[0] = None

# dtypes the gloo transport cannot reduce natively are widened for the wire
gloo_wire_dtype = {torch.bfloat16: torch.float32, torch.float16: torch.float32, torch.bool: torch.uint8}


def torch_dtype_to_id(dtype) -> int:
    return 0 if dtype is None else torch_to_intID_dtype_dict[dtype]


def id_to_torch_dtype(i: int):
    return intID_to_torch_dtype_dict[int(i)]
