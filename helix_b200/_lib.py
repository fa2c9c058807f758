"""ctypes binding of ``libhelix_b200.so`` (declared in ``include/helix_b200.h``).

The library is the only compute path: if it is missing or fails to load, every
operator raises -- there is no CPU or PyTorch fallback.
"""
import ctypes
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libhelix_b200.so")

OP_GEMM_F16, OP_GEMV_F16, OP_CONV_F16, OP_GEMM_F32, OP_CONV_F32, OP_GEMV_F32 = 0, 1, 2, 3, 4, 5

STATUS_TEXT = {
    0: "ok", -1: "invalid argument", -2: "pointer or leading dimension not 16-byte aligned",
    -3: "workspace missing or too small", -4: "CUDA call failed", -5: "bounded device-side wait ran out",
    -6: "configuration not built into the library", -7: "no sm_100 device is current",
    -8: "problem exceeds the capacity of a fixed built-in buffer",
}


class HelixError(RuntimeError):
    def __init__(self, status, what=""):
        self.status = int(status)
        super().__init__(f"{what}: helix status {self.status} ({STATUS_TEXT.get(self.status, 'unknown')})")


class DevInfo(ctypes.Structure):
    _fields_ = [("sm_count", ctypes.c_int), ("cc_major", ctypes.c_int), ("cc_minor", ctypes.c_int),
                ("clock_khz", ctypes.c_int), ("mem_clock_khz", ctypes.c_int),
                ("l2_bytes", ctypes.c_int64), ("smem_per_sm", ctypes.c_int64),
                ("smem_per_block_optin", ctypes.c_int64), ("total_mem", ctypes.c_int64),
                ("name", ctypes.c_char * 64)]


class Cfg(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int), ("tile_m", ctypes.c_int), ("tile_n", ctypes.c_int),
                ("tile_k", ctypes.c_int), ("stages", ctypes.c_int), ("cta_group", ctypes.c_int),
                ("split_k", ctypes.c_int), ("swap_ab", ctypes.c_int), ("raster", ctypes.c_int),
                ("thread_m", ctypes.c_int), ("thread_n", ctypes.c_int), ("load_group", ctypes.c_int),
                ("stream_k", ctypes.c_int), ("conv_gather", ctypes.c_int), ("max_ctas", ctypes.c_int), ("probe", ctypes.c_int)]

    def key(self):
        """Hashable identity used as the prof_dict key."""
        return (self.op, self.tile_m, self.tile_n, self.tile_k, self.stages, self.cta_group,
                self.split_k, self.swap_ab, self.load_group, self.stream_k, self.conv_gather)

    def copy(self):
        c = Cfg()
        ctypes.memmove(ctypes.byref(c), ctypes.byref(self), ctypes.sizeof(Cfg))
        return c


class Launch(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int), ("cfg", Cfg),
                ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("c", ctypes.c_void_p),
                ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldc", ctypes.c_int64),
                ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int), ("batch", ctypes.c_int),
                ("stride_a", ctypes.c_int64), ("stride_b", ctypes.c_int64), ("stride_c", ctypes.c_int64),
                ("conv", ctypes.c_int * 9), ("trans_a", ctypes.c_int), ("ldc_inner", ctypes.c_int64),
                ("ws", ctypes.c_void_p), ("ws_bytes", ctypes.c_size_t), ("flags", ctypes.c_uint32)]


LAUNCH_INDEPENDENT = 1
LAUNCH_STATIC_A = 2


# name -> (restype, argtypes); every symbol include/helix_b200.h declares
_P, _I, _L, _Z = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t
_PD = ctypes.POINTER(ctypes.c_double)
SIGNATURES = {
    "helix_version": (_I, []),
    "helix_status_string": (ctypes.c_char_p, [_I]),
    "helix_device_info": (_I, [_I, ctypes.POINTER(DevInfo)]),
    "helix_num_configs": (_I, [_I]),
    "helix_get_config": (_I, [_I, _I, ctypes.POINTER(Cfg)]),
    "helix_default_config": (_I, [ctypes.POINTER(Launch), ctypes.POINTER(Cfg)]),
    "helix_workspace_bytes": (_Z, [ctypes.POINTER(Launch)]),
    "helix_launch": (_I, [ctypes.POINTER(Launch), _P, _P]),
    "helix_gemm_f16": (_I, [ctypes.POINTER(Cfg), _P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _L, _L, _L, _P, _Z, _P, _P]),
    "helix_gemv_f16": (_I, [ctypes.POINTER(Cfg), _P, _L, _P, _L, _P, _L, _L, _I, _I, _I, _P, _Z, _P, _P]),
    "helix_gemv_f32": (_I, [ctypes.POINTER(Cfg), _P, _L, _P, _L, _P, _L, _L, _I, _I, _I, _P, _Z, _P, _P]),
    "helix_conv2d_f16_nhwc": (_I, [ctypes.POINTER(Cfg), _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _Z, _P, _P]),
    "helix_gemm_f32": (_I, [ctypes.POINTER(Cfg), _P, _L, _I, _P, _L, _P, _L, _I, _I, _I, _P, _P]),
    "helix_conv2d_f32_nhwc": (_I, [ctypes.POINTER(Cfg), _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _Z, _P, _P]),
    "helix_time_launches": (_I, [ctypes.POINTER(Launch), _I, _I, _I, _I, _PD, _PD, _PD]),
    "helix_gemm_f16_host": (_I, [_P, _P, _P, _I, _I, _I]),
    "helix_gemv_f16_host": (_I, [_P, _P, _P, _I, _I, _I]),
    "helix_gemm_f32_host": (_I, [_P, _P, _P, _I, _I, _I]),
    "helix_conv2d_f16_nhwc_host": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I]),
    "helix_gemv_f16_static": (_I, [_P, _L, _P, _L, _P, _L, _L, _I, _I, _I, _I, _P]),
    "helix_selftest_bounded_wait": (_I, [ctypes.c_uint64, _P, _P]),
    "helix_launch_count": (_L, []),
    "helix_trace_buffer": (_I, [_P, _Z]),
    "helix_trace_words_per_cta": (_I, []),
}

_lib = None


def load():
    """Load the shared library (building nothing); raises if it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m helix_b200.build` "
                "(nvcc, sm_100a).  There is no fallback path.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status, what):
    if status != 0:
        raise HelixError(status, what)
