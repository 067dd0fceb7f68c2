"""ctypes binding of the C ABI declared in include/puff_advantage.h.

This is the stub a maintainer of the reference would add to reach the library
without going through torch's dispatcher; the torch operator
(`pufferlib_b200._C`) calls the same entry points from C++.  There is no CPU
path behind any of these functions: when the shared library has not been built
the import raises, and on a machine without an sm_100 GPU every launch returns
an error code that `check()` turns into a RuntimeError.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# PUFF_ADV_LIB names another build of the same library (a sanitizer or debug build) to load instead
LIB_PATH = os.environ.get("PUFF_ADV_LIB") or os.path.join(_HERE, "libpuff_advantage_sm100.so")

# error codes / variants / kernels of include/puff_advantage.h
OK = 0
ERR_NULL, ERR_SHAPE, ERR_VARIANT, ERR_ALIGN, ERR_ALIAS = -1, -2, -3, -4, -5
ERR_ARCH, ERR_DRIVER, ERR_DEVICE_WAIT, ERR_WORKSPACE, ERR_SIZE, ERR_DEVICE_BOUNDS = -6, -7, -8, -9, -10, -11
NOALLOC_MAX_SEGMENTS = 524288
EXCHANGE_HANDLE_BYTES = 64
FLAG_ZERO_LAST_COLUMN = 1
VARIANT_AUTO, VARIANT_SERIAL, VARIANT_SCAN, VARIANT_GENERIC = 0, 1, 2, 3
KERNEL_NONE, KERNEL_TMA2D, KERNEL_BULK1D, KERNEL_SCAN, KERNEL_GENERIC = 0, 1, 2, 3, 4
VARIANTS = {"auto": VARIANT_AUTO, "serial": VARIANT_SERIAL, "scan": VARIANT_SCAN, "generic": VARIANT_GENERIC}
KERNEL_NAMES = {KERNEL_NONE: "none", KERNEL_TMA2D: "tma2d", KERNEL_BULK1D: "bulk1d",
                KERNEL_SCAN: "scan", KERNEL_GENERIC: "generic"}

# every symbol the header declares, with its ctypes signature
_P = ctypes.c_void_p
_F = ctypes.c_float
_LL = ctypes.c_longlong
_I = ctypes.c_int
SIGNATURES = {
    "puff_advantage_sm100_launch": (_I, [_P] * 6 + [_F] * 4 + [_LL, _LL, _I, _P]),
    "puff_advantage_sm100_launch_ex": (_I, [_P] * 6 + [_F] * 4 + [_LL, _LL, _I, ctypes.c_uint, _P]),
    "puff_advantage_sm100_host": (_I, [_P] * 6 + [_F] * 4 + [_LL, _LL, _I, _I]),
    "puff_advantage_sm100_host_release": (_I, [_I]),
    "puff_advantage_sm100_host_copies_only": (_I, [_P] * 6 + [_LL, _LL, _I]),
    "puff_priorities_sm100_scratch_bytes": (ctypes.c_size_t, [_LL]),
    "puff_priorities_sm100_weights": (_I, [_P, _P, _P, _F, _LL, _P, ctypes.c_size_t, _P]),
    "puff_priorities_sm100_probs": (_I, [_P, _P, _P, _LL, _P]),
    "puff_exchange_sm100_create": (_I, [_I, _I, _P, ctypes.POINTER(_P)]),
    "puff_exchange_sm100_connect": (_I, [_P, _P]),
    "puff_exchange_sm100_connect_pointers": (_I, [_P, ctypes.POINTER(_P)]),
    "puff_exchange_sm100_mailbox": (_P, [_P]),
    "puff_exchange_sm100_set_wait_ns": (_I, [_P, ctypes.c_ulonglong]),
    "puff_exchange_sm100_destroy": (_I, [_P]),
    "puff_priorities_sm100_weights_push": (_I, [_P, _P, _F, _LL, _P, ctypes.c_size_t, _P, _P]),
    "puff_priorities_sm100_probs_gathered": (_I, [_P, _P, _P, _LL, _P, _P]),
    "puff_minibatch_sm100_scratch_bytes": (ctypes.c_size_t, [_LL]),
    "puff_minibatch_sm100_gather": (_I, [_P] * 9 + [_F, _LL, _LL, _LL, _P, ctypes.c_size_t, _P]),
    "puff_minibatch_sm100_gather_ex": (_I, [_P] * 9 + [_F, _LL, _LL, _LL, _LL, _P, ctypes.c_size_t, _P]),
    "puff_minibatch_sm100_bad_index": (_I, []),
    "puff_rollout_sm100_write": (_I, [_P] * 6 + [_LL] * 5 + [_F, _P]),
    "puff_priorities_sm100_weights_noalloc": (_I, [_P, _P, _P, _F, _LL, _P]),
    "puff_advantage_sm100_strerror": (ctypes.c_char_p, [_I]),
    "puff_advantage_sm100_last_kernel": (_I, []),
    "puff_advantage_sm100_launch_count": (_LL, []),
    "puff_advantage_sm100_device_status": (_I, []),
    "puff_advantage_sm100_inject_status": (_I, [_I]),
    "puff_advantage_sm100_set_tuning": (_I, [_I, _I]),
    "puff_advantage_sm100_version": (ctypes.c_char_p, []),
}

_lib = None


def load():
    """The loaded library (ctypes.CDLL) with argument types set."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} has not been built; run `python -m pufferlib_b200.build` "
                "(needs nvcc with sm_100a support)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


TUNE = {"force_kernel": 0, "stages": 1, "ws_stages": 2, "ctas_per_sm": 3, "load_group": 4, "scan_threads": 5,
        "reserve_sms": 6, "tile_rows": 7, "pdl": 8, "scan_wide": 9, "b1_warp_teams": 10}


def set_tuning(**knobs):
    """Set tuning knobs by name (see PUFF_TUNE_* in the header); None or -1
    restores the automatic choice.  Returns the previous values."""
    lib = load()
    return {k: lib.puff_advantage_sm100_set_tuning(TUNE[k], -1 if v is None else int(v)) for k, v in knobs.items()}


def reset_tuning():
    set_tuning(**{k: None for k in TUNE})


def strerror(code):
    return load().puff_advantage_sm100_strerror(int(code)).decode()


def check(code, what="puff_advantage"):
    if code != OK:
        raise RuntimeError(f"{what}: {strerror(code)} (code {code})")


def last_kernel():
    return KERNEL_NAMES.get(load().puff_advantage_sm100_last_kernel(), "?")


def launch_count():
    return int(load().puff_advantage_sm100_launch_count())


def device_status():
    return int(load().puff_advantage_sm100_device_status())
