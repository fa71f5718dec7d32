"""ctypes binding of libcusig.so, the sm_100a signature library.

Mirrors the part of pySigLib's loader that serves ``sig`` / ``sig_backprop``
(``pysiglib/load_siglib.py:76-130,484-494``): same symbol names, same argument
types.  There is no CPU library behind it and no fallback: if the shared library
has not been built, every operation raises.
"""
import atexit
import ctypes
import os
from ctypes import POINTER, c_bool, c_char_p, c_double, c_float, c_int, c_uint64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_HERE, "lib", "libcusig.so")

DTYPES = {"float32": c_float, "float64": c_double}

_lib = None


class CusigNotBuiltError(RuntimeError):
    pass


def library():
    """The loaded CDLL; raises CusigNotBuiltError when libcusig.so is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIBRARY_PATH):
            raise CusigNotBuiltError(
                "pysiglib_b200: %s not found. Build the CUDA library first with "
                "`python -m pysiglib_b200._build`; there is no CPU fallback." % LIBRARY_PATH)
        lib = ctypes.CDLL(LIBRARY_PATH)
        _bind(lib)
        atexit.register(lib.cusig_shutdown)
        _lib = lib
    return _lib


def _bind(lib):
    lib.cusig_last_error_message.argtypes = ()
    lib.cusig_last_error_message.restype = c_char_p
    lib.cusig_shutdown.argtypes = ()
    lib.cusig_shutdown.restype = None
    lib.prepare_log_sig_cuda.argtypes = (c_uint64, c_uint64, c_int, c_bool)
    lib.prepare_log_sig_cuda.restype = c_int
    lib.sigb200_sig_length.argtypes = (c_uint64, c_uint64)
    lib.sigb200_sig_length.restype = c_uint64
    lib.sigb200_set_kernel_policy.argtypes = (c_int,)
    lib.sigb200_set_kernel_policy.restype = None
    lib.sigb200_set_tile_preference.argtypes = (c_int,)
    lib.sigb200_set_tile_preference.restype = None
    lib.sigb200_kernel_family.argtypes = (c_uint64, c_uint64, c_bool, c_bool, c_int, c_int)
    lib.sigb200_kernel_family.restype = c_char_p
    lib.sigb200_describe_plan.argtypes = (ctypes.c_char_p, c_uint64, c_uint64, c_uint64, c_uint64, c_uint64, c_bool,
                                          c_bool, c_int, c_int)
    lib.sigb200_describe_plan.restype = c_int
    lib.sigb200_noalloc_scratch_bytes.argtypes = ()
    lib.sigb200_noalloc_scratch_bytes.restype = c_uint64
    lib.sigb200_set_forced_plan.argtypes = (c_int, c_int, c_int, c_int)
    lib.sigb200_set_forced_plan.restype = None
    lib.sigb200_inject_alloc_failures.argtypes = (c_int,)
    lib.sigb200_inject_alloc_failures.restype = None
    lib.sigb200_pool_reserved_bytes.argtypes = (c_int,)
    lib.sigb200_pool_reserved_bytes.restype = c_uint64
    lib.sigb200_launch_count.argtypes = ()
    lib.sigb200_launch_count.restype = c_uint64
    for suffix, real in (("f", c_float), ("d", c_double)):
        ptr = POINTER(real)
        # reference-compatible symbols
        f = getattr(lib, "signature_cuda_" + suffix)
        f.argtypes = (ptr, ptr, c_uint64, c_uint64, c_uint64, c_uint64, c_bool, c_bool, real, c_bool, c_bool,
                      ptr, c_uint64, c_uint64, c_uint64)
        f.restype = c_int
        f = getattr(lib, "sig_combine_cuda_" + suffix)
        f.argtypes = (ptr, ptr, ptr, c_uint64, c_uint64, c_uint64, c_bool)
        f.restype = c_int
        f = getattr(lib, "sig_combine_backprop_cuda_" + suffix)
        f.argtypes = (ptr, ptr, ptr, ptr, ptr, c_uint64, c_uint64, c_uint64, c_bool)
        f.restype = c_int
        f = getattr(lib, "sig_backprop_cuda_" + suffix)
        f.argtypes = (ptr, ptr, ptr, ptr, c_uint64, c_uint64, c_uint64, c_uint64, c_bool, c_bool, real, c_bool,
                      ptr, c_uint64, c_uint64, c_uint64)
        f.restype = c_int
        f = getattr(lib, "linear_sig_cuda_" + suffix)
        f.argtypes = (ptr, ptr, c_uint64, c_uint64, c_uint64, c_bool)
        f.restype = c_int
        f = getattr(lib, "sig_join_cuda_" + suffix)
        f.argtypes = (ptr, ptr, ptr, c_uint64, c_uint64, c_uint64, c_bool, c_bool)
        f.restype = c_int
        f = getattr(lib, "sig_join_backprop_cuda_" + suffix)
        f.argtypes = (ptr, ptr, ptr, ptr, ptr, c_uint64, c_uint64, c_uint64, c_bool, c_bool)
        f.restype = c_int
        u64p = POINTER(c_uint64)
        f = getattr(lib, "sig_coef_cuda_" + suffix)
        f.argtypes = (ptr, ptr, u64p, c_uint64, u64p, c_uint64, c_uint64, c_uint64, c_bool)
        f.restype = c_int
        f = getattr(lib, "sig_coef_backprop_cuda_" + suffix)
        f.argtypes = (ptr, ptr, ptr, ptr, u64p, c_uint64, u64p, c_uint64, c_uint64, c_uint64)
        f.restype = c_int
        f = getattr(lib, "sig_to_log_sig_cuda_" + suffix)
        f.argtypes = (ptr, ptr, c_uint64, c_uint64, c_uint64, c_int, c_bool)
        f.restype = c_int
        f = getattr(lib, "sig_to_log_sig_backprop_cuda_" + suffix)
        f.argtypes = (ptr, ptr, ptr, c_uint64, c_uint64, c_uint64, c_int, c_bool)
        f.restype = c_int
        for name in ("transform_path_cuda_", "transform_path_backprop_cuda_"):
            f = getattr(lib, name + suffix)
            f.argtypes = (ptr, ptr, c_uint64, c_uint64, c_uint64, c_bool, c_bool, real)
            f.restype = c_int
        # extensions
        f = getattr(lib, "sigb200_signature_" + suffix)
        f.argtypes = (ptr, ptr, c_uint64, c_uint64, c_uint64, c_uint64, c_bool, c_bool, real, c_bool,
                      c_void_p, c_int, POINTER(c_int))
        f.restype = c_int
        f = getattr(lib, "sigb200_sig_backprop_" + suffix)
        f.argtypes = (ptr, ptr, ptr, ptr, c_uint64, c_uint64, c_uint64, c_uint64, c_bool, c_bool, real, c_bool,
                      c_void_p, c_int)
        f.restype = c_int
        f = getattr(lib, "sigb200_log_sig_" + suffix)
        f.argtypes = (ptr, ptr, c_uint64, c_uint64, c_uint64, c_uint64, c_bool, c_bool, real, c_int, c_bool,
                      c_void_p, c_int, POINTER(c_int))
        f.restype = c_int
        f = getattr(lib, "sigb200_sig_backprop_noalloc_" + suffix)
        f.argtypes = (ptr, ptr, ptr, ptr, c_uint64, c_uint64, c_uint64, c_uint64, c_bool, c_bool, real, c_bool,
                      c_void_p, c_int)
        f.restype = c_int
        f = getattr(lib, "sigb200_signature_sharded_" + suffix)
        f.argtypes = (ptr, ptr, c_uint64, c_uint64, c_uint64, c_uint64, c_bool, c_bool, real, c_bool,
                      POINTER(c_int), c_int)
        f.restype = c_int
        f = getattr(lib, "sigb200_sig_backprop_sharded_" + suffix)
        f.argtypes = (ptr, ptr, ptr, ptr, c_uint64, c_uint64, c_uint64, c_uint64, c_bool, c_bool, real, c_bool,
                      POINTER(c_int), c_int)
        f.restype = c_int


def fn(name, dtype):
    """Native function ``name`` for dtype "float32" / "float64"."""
    return getattr(library(), name + ("_f" if dtype == "float32" else "_d"))


def last_error_message():
    msg = library().cusig_last_error_message()
    return msg.decode("utf-8", errors="replace") if msg else ""


def launch_count():
    return int(library().sigb200_launch_count())


def set_kernel_policy(policy):
    """0: automatic choice between the register-tile and the generic kernels; 1: generic only."""
    library().sigb200_set_kernel_policy(int(policy))


def describe_plan(batch, dimension, length, degree, *, time_aug=False, lead_lag=False, dtype="float32",
                  backward=False):
    """Kernel variant a call of this shape would run on the current CUDA device."""
    buf = ctypes.create_string_buffer(256)
    code = library().sigb200_describe_plan(buf, 256, batch, dimension, length, degree, time_aug, lead_lag,
                                           1 if dtype == "float64" else 0, 1 if backward else 0)
    return buf.value.decode() if code == 0 else "error %d: %s" % (code, last_error_message())


def set_tile_preference(preference):
    """0 automatic, 1 biggest register tile, 2 smallest, 3 automatic without time segmentation,
    4 biggest tile with forced time segmentation of the forward sweep."""
    library().sigb200_set_tile_preference(int(preference))


def set_forced_plan(backward, chain_length, group, segments=1):
    """Test hook: pin the register-tile variant (chain length, group) and time-segment count of the
    forward / backward sweep; ``chain_length < 0`` clears it."""
    library().sigb200_set_forced_plan(1 if backward else 0, int(chain_length), int(group), int(segments))


def inject_alloc_failures(count):
    """Test hook: the next ``count`` scratch / staging requests fail as if the GPU were out of memory."""
    library().sigb200_inject_alloc_failures(int(count))


def pool_reserved_bytes(device=0):
    return int(library().sigb200_pool_reserved_bytes(int(device)))


def kernel_family(dimension, degree, *, time_aug=False, lead_lag=False, dtype="float32", backward=False):
    return library().sigb200_kernel_family(dimension, degree, time_aug, lead_lag,
                                           1 if dtype == "float64" else 0, 1 if backward else 0).decode()
