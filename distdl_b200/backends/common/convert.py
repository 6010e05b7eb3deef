"""dtype conversion between torch and the "model" array library of the active
backend (``src/distdl/backends/common/convert.py:6-47``).  Every backend here
keeps tensors as torch tensors, so the model dtype *is* the torch dtype; the
integer-id maps are used in structure handshakes."""
from ...utilities.dtype import id_to_torch_dtype, torch_dtype_to_id


def convert_torch_to_model_dtype(dtype):
    return dtype


def convert_model_to_torch_dtype(dtype):
    return dtype


def convert_intID_to_model_dtype_dict(intID):
    return id_to_torch_dtype(intID)


def convert_model_to_intID_dtype_dict(dtype):
    return torch_dtype_to_id(dtype)
