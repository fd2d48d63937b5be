"""ctypes binding of ``libvsa_b200.so`` (the C ABI declared in ``include/vsa_b200.h``).

The library is the only compute path of this package: if it has not been built
the import fails with instructions, never falling back to anything else.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvsa_b200.so")

VSA_BF16, VSA_F32, VSA_F16 = 0, 1, 2
ERR_BAD_ARGUMENT, ERR_UNSUPPORTED, ERR_LAUNCH, ERR_DEVICE_TIMEOUT = -1, -2, -3, -4

P, I, L, F = c_void_p, c_int, c_int64, c_float

# name -> argument types, in the order of include/vsa_b200.h
SIGNATURES = {
    "vsa_block_mean3_fwd": [P, P, P, P, P, P, P, P, L, L, L, I, I, I, P],
    "vsa_block_mean_fwd": [P, P, P, L, L, I, I, I, P],
    "vsa_block_mean_bwd_accumulate": [P, P, P, L, L, I, I, I, P],
    "vsa_block_mean_bwd": [P, P, P, L, L, I, I, I, P],
    "vsa_coarse_fwd": [P, P, P, P, P, P, L, I, I, I, F, I, P],
    "vsa_topk": [P, P, L, I, I, I, P],
    "vsa_coarse_bwd": [P, P, P, P, P, P, P, P, P, P, P, L, I, I, I, F, I, P],
    "vsa_sparse_fwd": [P, P, P, P, P, P, P, L, L, L, I, I, I, F, I, P],
    "vsa_sparse_fwd_combine": [P, P, P, P, P, P, P, P, P, P, L, L, L, I, I, I, F, I, P],
    "vsa_route_invert": [P, P, P, P, P, L, I, I, I, P],
    "vsa_route_invert_static": [P, P, P, P, L, I, I, I, P],
    "vsa_sparse_bwd_dq": [P, P, P, P, P, P, P, P, P, P, L, L, L, I, I, I, F, I, P],
    "vsa_sparse_bwd_dkdv": [P, P, P, P, P, P, P, P, P, P, P, P, L, L, L, I, I, I, F, I, P],
    "vsa_sparse_bwd_dq_fused": [P, P, P, P, P, P, P, P, P, P, P, P, L, L, L, I, I, I, F, I, P],
    "vsa_sparse_bwd_dkdv_fused": [P, P, P, P, P, P, P, P, P, P, P, P, P, P, L, L, L, I, I, I, F, I, P],
    "vsa_route_invert_edges": [P, P, P, P, P, L, I, I, I, P],
    "vsa_sparse_bwd_delta": [P, P, P, L, L, I, I, P],
    "vsa_sparse_bwd_dkdv_ds": [P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, L, L, L, I, I, I, F, I, P],
    "vsa_sparse_bwd_dq_from_ds": [P, P, P, P, P, P, P, L, L, L, I, I, I, F, I, P],
    "vsa_sparse_fwd_combine_sharded": [P, P, P, P, P, P, P, P, P, P, L, L, L, L, I, I, I, F, I, P],
    "vsa_sparse_bwd_dq_sharded": [P, P, P, P, P, P, P, P, P, P, P, P, L, L, L, L, I, I, I, F, I, P],
    "vsa_sparse_bwd_dkdv_sharded": [P, P, P, P, P, P, P, P, P, P, P, P, P, P, L, L, L, L, I, I, I, F, I, P],
    "vsa_combine_fwd": [P, P, P, P, L, L, I, I, I, P],
    "vsa_gather_rows": [P, P, P, L, L, L, L, P],
    "vsa_gather_rows_heads": [P, P, P, L, I, L, L, L, I, P],
    "vsa_sparse_fwd_combine_raster": [P, P, P, P, P, P, P, P, P, P, P, L, I, L, L, L, I, I, I, F, I, P],
    "vsa_combine_bwd_raster": [P, P, P, P, P, P, P, L, I, L, L, I, I, I, P],
    "vsa_sparse_bwd_dq_raster": [P, P, P, P, P, P, P, P, P, P, P, P, P, L, I, L, L, L, I, I, I, F, I, P],
    "vsa_sparse_bwd_dkdv_raster": [P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, L, I, L, L, L, I, I, I, F, I, P],
    "vsa_selftest_umma": [P, P, P, I, P],
    "vsa_device_status": [P],
    "vsa_selftest_wait_timeout": [L, P, P],
    "vsa_combine_bwd": [P, P, P, P, P, L, L, I, I, I, P],
}
PLAIN = {"vsa_last_error_string": ([], c_char_p), "vsa_version": ([], c_int),
         "vsa_launch_count": ([], c_int64),
         "vsa_workspace_bytes": ([I, L, L, L, I, I, I, I], c_int64),
         "vsa_sparse_bwd_ds_supported": ([I, I, I, I], c_int),
         "vsa_sparse_sharded_supported": ([I, I, I, I], c_int),
         "vsa_sparse_raster_supported": ([I, I, I, I], c_int),
         "vsa_sparse_kernel_family": ([I, I, I, I], c_int),
         "vsa_sparse_bwd_ds_workspace_bytes": ([L, L, I, I], c_int64)}


class VsaError(RuntimeError):
    """A kernel launch failed or a device-side wait ran out."""


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python simple_vsa_b200/build.py` "
            "(needs nvcc with sm_100a support). This package has no other compute path.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    for name, (argtypes, restype) in PLAIN.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    return lib


lib = _load()


def device_status() -> int:
    """Fetch and clear the device status word (synchronises): 0 or the code of a timed-out wait."""
    out = ctypes.c_int(0)
    rc = lib.vsa_device_status(ctypes.byref(out))
    if rc:
        raise VsaError(f"vsa_device_status: {last_error()}")
    return out.value


def raise_on_device_timeout(where: str) -> None:
    """For callers that have just synchronised: raise if a bounded device-side wait ran out since the last check.

    After a time-out every tcgen05 kernel returns without writing its outputs until the word is cleared, so the
    results produced since then are not valid; the word is cleared by this call."""
    code = device_status()
    if code:
        raise VsaError(f"{where}: a bounded device-side wait ran out (code {code}, status {ERR_DEVICE_TIMEOUT}); "
                       "results since the last check are not valid")


def last_error() -> str:
    return lib.vsa_last_error_string().decode("utf-8", "replace")


# Optional timing hook: when set to a callable, ``call`` brackets every entry point with
# ``recorder(name, "start", stream)`` / ``recorder(name, "stop", stream)``.  The stream is the
# last argument of every entry point.  Used by the benchmark to time kernels with CUDA events.
recorder = None


def call(name: str, *args) -> None:
    """Invoke an entry point; a bad-argument status becomes ValueError, the rest VsaError."""
    if recorder is not None:
        recorder(name, "start", args[-1])
        rc = getattr(lib, name)(*args)
        recorder(name, "stop", args[-1])
    else:
        rc = getattr(lib, name)(*args)
    if rc == 0:
        return
    msg = f"{name}: {last_error()} (status {rc})"
    if rc in (ERR_BAD_ARGUMENT, ERR_UNSUPPORTED):
        raise ValueError(msg)
    raise VsaError(msg)
