"""torch.ops namespace of the package.

Same naming rule as the reference's generated glue
(finegrained-fp8-helion/finegrained-fp8-helion/build/torch-cuda/_ops.py:21-36):
``_<package>_<backend>_<sha1(package)[:7]>``, so code that reaches the op through
``torch.ops._finegrained_fp8_helion_cuda_b0d7177`` keeps working.
"""
import hashlib

import torch

_KERNEL_NAME = "finegrained_fp8_helion"
_OPS_NAME = f"_{_KERNEL_NAME}_cuda_{hashlib.sha1(_KERNEL_NAME.encode()).hexdigest()[:7]}"


def add_op_namespace_prefix(op_name: str) -> str:
    return f"{_OPS_NAME}::{op_name}"


class _Ops:
    def __getattr__(self, name):
        return getattr(getattr(torch.ops, _OPS_NAME), name)


ops = _Ops()
