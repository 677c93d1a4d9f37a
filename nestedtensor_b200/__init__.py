"""nestedtensor_b200 — B200 (sm_100a) implementation of nestedtensor's ragged<->dense, mask and
varlen self-attention path behind the reference's Python surface
(nestedtensor/__init__.py:3-22).

    import nestedtensor_b200 as nestedtensor
    nt = nestedtensor.nested_tensor(list_of_tensors, device="cuda", dtype=torch.bfloat16)
    dense = nt.to_padded_tensor(padding=0)
    data, mask = nt.to_tensor_mask(mask_dim=2)
    back = nestedtensor.nested_tensor_from_padded_tensor(dense, padding=0)

All compute runs in hand-written CUDA kernels reached through the C ABI of
``lib/libntb200.so`` (include/ntb200.h); there is no CPU or eager fallback.
"""
from .nested import NestedTensor
from .creation import nested_tensor, as_nested_tensor
from .masking import (nested_tensor_from_tensor_mask, nested_tensor_from_padded_tensor, nt_from_tensor_mask,
                      merge_tensor_mask, TensorMask)
from . import nn
from .sharding import token_balanced_partition
from .host_pipeline import (to_padded_tensor_host, from_padded_tensor_host, multi_head_attention_host,
                            transformer_encoder_layer_host)

__version__ = "0.1.0"

# Register torch.ops.nestedtensor.* at import when the native libraries are built, like the reference's
# `import nestedtensor` does.  If they are not, the first operator call raises with the build command.
import os as _os
from . import _build as _b, _ops as _o
if _os.path.exists(_b.CABI_LIB) and _os.path.exists(_b.DISPATCH_LIB):
    _o.load()
del _os, _b, _o


def device_error_flags():
    """Bit mask of device-side conditions recorded since the last call (0 = none): a bounded wait of a tcgen05
    kernel that ran out (projection: bits 0-2, attention: bits 8-10; the affected output tiles were left unwritten)
    or an embedding index out of range (bit 16).  Synchronises the device.  The torch operators do not read it on
    every call; a caller that wants the check after each of them sets ``NTB200_CHECK_DEVICE_ERRORS=1``."""
    from . import _cabi
    return int(_cabi.load().ntb200_device_error_flags())


def is_nested_tensor(obj):
    return isinstance(obj, NestedTensor)


def to_mask(nt, mask_dim=None):
    """``torch.ops.nestedtensor.to_mask`` (nestedtensor/csrc/masking.cpp:408-457) as a function."""
    from . import _ops
    return _ops.ops().to_mask(nt, mask_dim)


def from_padded_tensor(padded, target):
    """Remove the padding of ``padded`` using the sizes of the nested tensor ``target``
    (nestedtensor/csrc/masking.cpp:459-533; C++-internal in the reference)."""
    from .nested import _op_from_padded_tensor
    return _op_from_padded_tensor(padded, target)
