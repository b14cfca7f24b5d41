"""ctypes binding of libmega_b200.so (declared in include/mega_b200.h).

There is no CPU or PyTorch fallback: if the shared library is missing, loading raises, and
every op raises when handed a non-CUDA tensor.
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libmega_b200.so")

c_p = ctypes.c_void_p
c_i = ctypes.c_int
c_u = ctypes.c_uint
c_l = ctypes.c_int64
c_d = ctypes.c_double

# name -> argument types, in the order of include/mega_b200.h
SIGNATURES = {
    "mega_ema_coeffs": [c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_p, c_p, c_p, c_p],
    "mega_ema_kernel": [c_p, c_p, c_p, c_i, c_i, c_i, c_p, c_p],
    "mega_ema_bias": [c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_p, c_p],
    "mega_ema_fwd": [c_p, c_p, c_i, c_i, c_i, c_i, c_l, c_l, c_l, c_l, c_l, c_l, c_p, c_p, c_p, c_p, c_i,
                     c_p, c_p, c_p, c_u, c_i, c_p],
    "mega_ema_step": [c_p, c_p, c_i, c_i, c_i, c_p, c_p, c_p, c_p, c_i, c_p, c_p, c_u, c_p],
    "mega_timestep_norm_fwd": [c_p, c_p, c_i, c_i, c_i, c_i, c_l, c_l, c_l, c_l, c_l, c_l, c_p, c_p, c_p,
                               c_p, c_p, c_p, c_i, c_d, c_p, c_p, c_p, c_p],
    "mega_sequence_norm_fwd": [c_p, c_p, c_i, c_i, c_i, c_i, c_l, c_l, c_l, c_l, c_l, c_l, c_p, c_p, c_p,
                               c_i, c_d, c_p, c_p, c_p, c_p],
    "mega_tsn_ema_fwd": [c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_l, c_l, c_l, c_l, c_l, c_l, c_p, c_p, c_p,
                         c_p, c_p, c_d, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_p, c_p, c_p, c_u, c_p],
    "mega_tsn_ema_fwd_runs": [c_p, c_p, c_i, c_i, c_i, c_i, c_l, c_l, c_l, c_l, c_l, c_l, c_p, c_p, c_p,
                              c_p, c_p, c_d, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_p, c_p, c_u, c_i, c_p],
    "mega_sqn_ema_fwd": [c_p, c_p, c_i, c_i, c_i, c_i, c_l, c_l, c_l, c_l, c_l, c_l, c_p, c_p, c_d, c_p, c_p, c_p,
                         c_p, c_p, c_p, c_p, c_i, c_p, c_u, c_p],
    "mega_tsn_ema_step": [c_p, c_p, c_p, c_i, c_i, c_i, c_p, c_p, c_p, c_p, c_p, c_p, c_d, c_p, c_p, c_p, c_p, c_i,
                          c_p, c_u, c_p],
    "mega_tsn_cema_step": [c_p, c_p, c_p, c_i, c_i, c_i, c_p, c_p, c_p, c_p, c_p, c_p, c_d, c_p, c_p, c_p, c_p, c_i,
                           c_p, c_u, c_p],
    "mega_gate_silu": [c_p, c_l, c_p, c_l, c_p, c_l, c_i, c_l, c_i, c_p],
    "mega_gate_mul_silu": [c_p, c_l, c_p, c_l, c_p, c_l, c_i, c_l, c_i, c_p],
    "mega_gate_output": [c_p, c_l, c_p, c_l, c_p, c_l, c_p, c_l, c_p, c_l, c_i, c_l, c_i, c_p],
    "mega_gate_qk": [c_p, c_l, c_p, c_p, c_p, c_l, c_p, c_l, c_i, c_l, c_i, c_d, c_p],
    "mega_gate_qk_rotary": [c_p, c_l, c_p, c_p, c_p, c_i, c_i, c_i, c_p, c_l, c_p, c_l, c_i, c_l, c_i, c_d, c_p],
    "mega_timestep_norm_fwd_train": [c_p, c_p, c_i, c_i, c_i, c_i, c_l, c_l, c_l, c_l, c_l, c_l, c_p, c_p, c_p,
                                     c_p, c_p, c_p, c_i, c_d, c_p, c_p, c_p, c_p, c_p, c_p, c_p],
    "mega_timestep_norm_bwd": [c_p, c_p, c_p, c_i, c_i, c_i, c_i] + [c_l] * 9 + [c_p] * 9 + [c_i] + [c_p] * 5,
    "mega_sequence_norm_bwd": [c_p, c_p, c_p, c_i, c_i, c_i, c_i] + [c_l] * 9 + [c_p] * 5 + [c_i] + [c_p] * 3,
    "mega_ema_bwd": [c_p, c_p, c_p, c_i, c_i, c_i, c_i] + [c_l] * 9 + [c_p] * 4 + [c_i] + [c_p] * 3 + [c_u, c_i]
                    + [c_p] * 6,
    "mega_ema_coeffs_bwd": [c_p] * 6 + [c_i, c_i] + [c_p] * 5,
    "mega_cema_coeffs": [c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_p, c_p, c_p, c_p],
    "mega_cema_kernel": [c_p, c_p, c_p, c_i, c_i, c_i, c_p, c_p],
    "mega_cema_fwd": [c_p, c_p, c_i, c_i, c_i, c_i, c_l, c_l, c_l, c_l, c_l, c_l, c_p, c_p, c_p, c_p, c_i,
                      c_p, c_p, c_p, c_u, c_i, c_p],
    "mega_cema_step": [c_p, c_p, c_i, c_i, c_i, c_p, c_p, c_p, c_p, c_i, c_p, c_p, c_u, c_p],
    "mega_cema_bwd": [c_p, c_p, c_p, c_i, c_i, c_i, c_i] + [c_l] * 9 + [c_p] * 4 + [c_i, c_p, c_u, c_i] + [c_p] * 5,
    "mega_cema_coeffs_bwd": [c_p] * 7 + [c_i, c_i] + [c_p] * 5,
    "mega_attention_softmax_fwd": [c_p, c_p, c_i, c_l, c_l, c_i, c_i, c_p],
    "mega_attention_softmax_bwd": [c_p, c_p, c_p, c_i, c_l, c_l, c_i, c_i, c_p],
    "mega_attention_dropkey_softmax_fwd": [c_p, c_p, c_i, c_l, c_l, c_i, c_i, c_d, ctypes.c_uint64, ctypes.c_uint64,
                                           c_p],
    "mega_tsn_cema_fwd": [c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_l, c_l, c_l, c_l, c_l, c_l, c_p, c_p, c_p,
                          c_p, c_p, c_d, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_p, c_p, c_p, c_u, c_p],
    "mega_set_option": [c_i, c_i],
    "mega_debug_device_error": [ctypes.POINTER(c_i), c_i],
}
OTHER = {
    "mega_status_string": ([c_i], ctypes.c_char_p),
    "mega_last_cuda_error": ([], ctypes.c_char_p),
    "mega_abi_version": ([], c_i),
    "mega_launch_count": ([], ctypes.c_uint64),
    "mega_debug_last_kernel": ([], ctypes.c_char_p),
}

_lib = None


class MegaError(RuntimeError):
    pass


def lib():
    """The loaded library; raises if it was never built (python fairseq-apollo_b200/build.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "libmega_b200.so is missing at %s: build it with `python fairseq-apollo_b200/build.py` "
                "(there is no CPU fallback)" % LIB_PATH)
        l = ctypes.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            f = getattr(l, name)
            f.argtypes = args
            f.restype = c_i
        for name, (args, res) in OTHER.items():
            f = getattr(l, name)
            f.argtypes = args
            f.restype = res
        _lib = l
    return _lib


def check(status, what):
    if status != 0:
        l = lib()
        msg = l.mega_status_string(status).decode()
        if status == 8:
            msg += " (%s)" % l.mega_last_cuda_error().decode()
        raise MegaError("%s: %s" % (what, msg))


def launch_count():
    return int(lib().mega_launch_count())


def last_kernel():
    """Kernel family of the most recent launch of this process (test aid)."""
    return lib().mega_debug_last_kernel().decode()


def set_option(key, value):
    check(lib().mega_set_option(int(key), int(value)), "set_option")


def device_error(reset=False):
    """Synchronising read of the device-side error word (0 = no bounded wait ever gave up)."""
    v = c_i(0)
    check(lib().mega_debug_device_error(ctypes.byref(v), 1 if reset else 0), "device_error")
    return v.value
