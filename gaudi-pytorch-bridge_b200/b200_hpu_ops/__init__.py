"""b200_hpu_ops -- the quantized-inference operators of the Gaudi PyTorch bridge
(``torch.ops.hpu.cast_to_fp8_v2 / cast_from_fp8 / fp8_gemm_v2 / convert_from_int4 /
convert_from_uint4``) for CUDA tensors on B200.

Importing this package loads two in-tree shared libraries:

* ``lib/libb200q.so``        -- the sm_100a kernels behind a C ABI (``include/b200q.h``)
* ``lib/b200_hpu_ops_ext.so`` -- the C++ torch extension that registers the ``hpu::*`` schemas

There is no fallback: if either library is missing the import fails and says how to build.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(os.path.dirname(_HERE), "lib")
KERNEL_LIB = os.path.join(LIB_DIR, "libb200q.so")
TORCH_EXT = os.path.join(LIB_DIR, "b200_hpu_ops_ext.so")


def _load():
    for p in (KERNEL_LIB, TORCH_EXT):
        if not os.path.exists(p):
            raise ImportError(
                f"{p} is missing: build the native libraries first "
                f"(python {os.path.join(os.path.dirname(_HERE), 'build.py')}); there is no fallback path")
    ctypes.CDLL(KERNEL_LIB, mode=ctypes.RTLD_GLOBAL)
    torch.ops.load_library(TORCH_EXT)


_load()

from . import abi  # noqa: E402
from .abi import device_status, launch_count  # noqa: E402


def set_sr_seed(seed: int) -> None:
    """Seed of the Philox stream used by stochastic rounding; also rewinds the per-call offset
    (each stochastic cast_to_fp8_v2 call consumes one offset so repeated calls differ)."""
    torch.ops.b200q.set_sr_seed(int(seed))


def set_cast_mul_in_fp32(on: bool) -> None:
    """False (default): input*scale is formed in the input dtype, as the reference's tests
    expect.  True: formed in fp32 with the unrounded fp32 scale."""
    torch.ops.b200q.set_cast_mul_in_fp32(bool(on))
