"""ctypes binding of libsbk.so (the C ABI declared in include/sbk.h).

There is no fallback: if the library is missing or does not export a symbol the
import of this module raises, and every caller above it fails with it.
"""
import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libsbk.so")

SBK_BF16, SBK_F32 = 0, 1
PREFILL_AUTO, PREFILL_TCGEN05, PREFILL_MMA_SYNC, PREFILL_TCGEN05_PAIR = 0, 1, 2, 3
SBK_OK, SBK_E_ARG, SBK_E_ALIGN, SBK_E_WORKSPACE, SBK_E_LAUNCH = 0, -1, -2, -3, -4
ST_BAD_SLOT, ST_BAD_BLOCK, ST_WAIT_TIMEOUT, ST_RETIRE_OVERFLOW, ST_BAD_POSITION = 1, 2, 4, 8, 16
ST_OUT_OF_BLOCKS, ST_TABLE_FULL, ST_VALUE_RANGE = 32, 64, 128
ABI_VERSION = 5

# name -> (restype, argtypes); must list every function include/sbk.h declares
SIGNATURES = {
    "sbk_abi_version": (c_int, []),
    "sbk_last_error": (c_char_p, []),
    "sbk_kv_append": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64,
        c_int64, c_int, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p,
        c_int, c_void_p, c_void_p]),
    "sbk_kv_gather": (c_int, [
        c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int,
        c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "sbk_swa_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "sbk_swa_copy_mode": (c_int, []),
    "sbk_swa_decode": (c_int, [
        c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
        c_int, c_int64, c_int, c_int64, c_int, c_float, c_void_p, c_int, c_int64, c_void_p,
        c_void_p, c_size_t, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "sbk_swa_prefill": (c_int, [
        c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
        c_int, c_int, c_int, c_int64, c_int, c_int64, c_int, c_float, c_void_p, c_int64, c_void_p,
        c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "sbk_gla_scan_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "sbk_gla_scan": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int64, c_void_p,
        c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int, c_float, c_void_p, c_float,
        c_int, c_void_p, c_size_t, c_void_p, c_void_p]),
    "sbk_swa_static_scratch_bytes": (c_size_t, []),
    "sbk_swa_decode_static": (c_int, [
        c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
        c_int, c_int64, c_int, c_int64, c_int, c_float, c_void_p, c_int, c_int64, c_void_p,
        c_int, c_int, c_void_p, c_void_p]),
    "sbk_swa_decode_gather": (c_int, [
        c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
        c_int, c_int64, c_int, c_int64, c_int, c_float, c_void_p, c_int64, c_void_p, c_size_t,
        c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int32, c_void_p, c_void_p,
        c_void_p]),
    "sbk_gla_step_gather": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int,
        c_float, c_void_p, c_int64, c_int, c_float, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int,
        c_int32, c_void_p, c_void_p, c_void_p]),
    "sbk_peer_alloc": (c_int, [c_size_t, c_void_p]),
    "sbk_peer_free": (c_int, [c_void_p]),
    "sbk_peer_handle_bytes": (c_int, []),
    "sbk_peer_export": (c_int, [c_void_p, c_void_p, c_int]),
    "sbk_peer_open": (c_int, [c_void_p, c_int, c_void_p]),
    "sbk_peer_close": (c_int, [c_void_p]),
    "sbk_peer_wait": (c_int, [c_void_p, c_int, c_int, c_int32, c_void_p, c_int32, c_int, c_void_p, c_void_p]),
    "sbk_peer_signal": (c_int, [c_void_p, c_int, c_int32, c_void_p, c_void_p]),
    "sbk_rope_kv_append": (c_int, [
        c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
        c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int, c_int64,
        c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "sbk_pool_init": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "sbk_plan_step": (c_int, [
        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "sbk_release_rows": (c_int, [
        c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p,
        c_void_p]),
    "sbk_swa_prefill_dense": (c_int, [
        c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int, c_int, c_int,
        c_int, c_int, c_int, c_int, c_float, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "sbk_gla_step": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_void_p, c_int, c_int,
        c_int, c_int, c_float, c_void_p, c_int, c_int, c_float, c_void_p, c_float, c_void_p,
        c_void_p]),
}


class SbkError(RuntimeError):
    """A C-ABI entry point returned a non-zero code."""

    def __init__(self, fn: str, code: int, msg: str):
        super().__init__(f"{fn} failed with code {code}: {msg}")
        self.code = code


def load(path: str = LIB_PATH) -> ctypes.CDLL:
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python spikingbrain-7b_b200/build.py` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this path.")
    lib = ctypes.CDLL(path)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    got = lib.sbk_abi_version()
    if got != ABI_VERSION:
        raise ImportError(f"{path} has ABI version {got}, binding expects {ABI_VERSION}")
    return lib


lib = load()


def check(fn: str, code: int) -> None:
    if code != SBK_OK:
        raise SbkError(fn, code, lib.sbk_last_error().decode("utf-8", "replace"))
