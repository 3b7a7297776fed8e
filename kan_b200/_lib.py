"""ctypes binding of libchebykan_b200.so (the C ABI in include/chebykan_b200.h).

There is no fallback: if the shared library has not been built the import of
any compute entry point raises, and every non-zero status from the library
becomes a RuntimeError.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libchebykan_b200.so")

MODE_FP32, MODE_TF32, MODE_BF16, MODE_FP32X3 = 0, 1, 2, 3
MODES = {"fp32": MODE_FP32, "tf32": MODE_TF32, "bf16": MODE_BF16, "fp32x3": MODE_FP32X3}
OP_FWD, OP_BWD_DCOEFF, OP_BWD_DX = 0, 1, 2
FAMILY_CHEBYSHEV, FAMILY_JACOBI, FAMILY_HERMITE, FAMILY_HERMITE_PROB = 0, 1, 2, 3


class Family(ctypes.Structure):
    """chebykan_family of the C header: a polynomial family described on the host."""
    _fields_ = [("kind", c_int32), ("alpha", c_float), ("beta", c_float), ("affine", c_int32),
                ("scale", c_float), ("shift", c_float), ("offset", c_float)]


_FAM = ctypes.POINTER(Family)

# name -> (restype, argtypes); every symbol declared in include/chebykan_b200.h
SIGNATURES = {
    "chebykan_abi_version": (c_int, []),
    "chebykan_strerror": (c_char_p, [c_int]),
    "chebykan_last_cuda_error": (c_int, []),
    "chebykan_packed_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int]),
    "chebykan_pack_coeffs": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "chebykan_workspace_bytes": (c_int64, [c_int, c_int64, c_int64, c_int64, c_int64, c_int]),
    "chebykan_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int,
                             c_void_p, c_void_p]),
    "chebykan_fwd_ln": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int,
                                c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p]),
    "chebykan_bwd_dcoeff": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                    c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "chebykan_bwd_dcoeff_static": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                           c_int, c_void_p]),
    "chebykan_bwd_dx": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "chebykan_jacobian": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "chebykan_normalize_input": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "chebykan_basis_functions": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "chebykan_family_table": (c_int, [_FAM, c_int64, c_void_p, c_void_p, c_void_p]),
    "chebykan_family_fwd": (c_int, [_FAM, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int,
                                    c_void_p, c_void_p]),
    "chebykan_family_workspace_bytes": (c_int64, [c_int, c_int64, c_int64, c_int64, c_int64, c_int]),
    "chebykan_family_bwd_dcoeff": (c_int, [_FAM, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                           c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "chebykan_family_bwd_dx": (c_int, [_FAM, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                       c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "chebykan_family_normalize": (c_int, [_FAM, c_void_p, c_void_p, c_int64, c_void_p]),
    "chebykan_family_basis": (c_int, [_FAM, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "chebykan_mse_workspace_bytes": (c_int64, []),
    "chebykan_mse_loss_grad": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                       c_float, c_void_p]),
    "chebykan_scale_by_device_scalar": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "chebykan_sgd_step": (c_int, [c_void_p, c_void_p, c_int64, c_float, c_float, c_void_p]),
    "chebykan_adam_step": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_float, c_float,
                                   c_float, c_float, c_int64, c_float, c_void_p]),
    "chebykan_adam_step_graph": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_float, c_float,
                                         c_float, c_float, c_void_p, c_float, c_void_p]),
    "chebykan_small_train_step_supported": (c_int, [c_int64, c_int64, c_int64, c_int64]),
    "chebykan_small_train_step": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_int64, c_int64, c_int64, c_int64, c_int, c_float, c_float, c_float, c_float,
                                          c_void_p]),
    "chebykan_selftest_bounded_wait": (c_int, [c_void_p, c_int64, c_int, c_void_p]),
    "chebykan_fwd_host_scratch_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int64, c_int]),
    "chebykan_fwd_host": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                  c_int64, c_int64, c_int, c_void_p]),
    "chebykan_fwd_host_packed_scratch_bytes": (c_int64, [c_int64, c_int64, c_int64]),
    "chebykan_fwd_host_packed": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                         c_int64, c_int64, c_int, c_int64, c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (once) and attach the C signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m kan_b200.build`. "
            "kan_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.chebykan_abi_version() != 7:
        raise RuntimeError("libchebykan_b200.so ABI version mismatch; rebuild it")
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().chebykan_strerror(code).decode()


def check(code: int, what: str) -> None:
    """Turn a negative library status into a RuntimeError."""
    if code < 0:
        lib = load()
        extra = ""
        if code == -4:
            extra = f" (cudaError {lib.chebykan_last_cuda_error()})"
        raise RuntimeError(f"{what}: {strerror(code)}{extra}")
