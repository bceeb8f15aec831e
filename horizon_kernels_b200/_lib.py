"""ctypes binding of the C ABI in include/hkv.h. There is no fallback: if the CUDA library is missing or does not
load, every kernel entry point raises."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libhkv.so")

EXPORTS = ("hkv_version", "hkv_error_string", "hkv_last_cuda_error", "hkv_write", "hkv_decode_workspace_bytes",
           "hkv_decode", "hkv_combine", "hkv_workspace_status", "hkv_decode_noalloc", "hkv_decode_noalloc_status",
           "hkv_set_option", "hkv_dequant", "hkv_write_rot",
           "hkv_decode_rot", "hkv_write_k8", "hkv_decode_k8", "hkv_dequant_k8",
           "hkv_selftest_wait_timeout", "hkv_selftest_codec", "hkv_probe_issue_rates")

_lib = None


class HkvError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        L = load()
        msg = L.hkv_error_string(code).decode()
        extra = f" (cuda error {L.hkv_last_cuda_error()})" if code == -7 else ""
        super().__init__(f"{where}: {msg}{extra} [{code}]")


def load():
    """the loaded library; raises if it has not been built (python -m horizon_kernels_b200.build)"""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m horizon_kernels_b200.build`; "
                               "there is no CPU or PyTorch fallback for these kernels")
        L = C.CDLL(LIB_PATH)
        i64, i32, vp, f32 = C.c_int64, C.c_int, C.c_void_p, C.c_float
        L.hkv_version.restype = i32
        L.hkv_error_string.restype = C.c_char_p
        L.hkv_error_string.argtypes = [i32]
        L.hkv_last_cuda_error.restype = i32
        L.hkv_write.restype = i32
        L.hkv_write.argtypes = [vp, vp, i64, i64, i64, i64, vp, vp, vp, vp, C.POINTER(i64), i32, vp, i64, vp, vp, i32,
                                i32, i32, vp]
        L.hkv_decode_workspace_bytes.restype = C.c_size_t
        L.hkv_decode_workspace_bytes.argtypes = [i32, i32, i32, i32, i32]
        L.hkv_decode.restype = i32
        L.hkv_decode.argtypes = [vp, vp, vp, vp, vp, C.POINTER(i64), i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, f32,
                                 f32, vp, vp, vp, C.c_size_t, i32, vp, vp]
        L.hkv_combine.restype = i32
        L.hkv_combine.argtypes = [vp, C.c_size_t, vp, i32, i32, i32, i32, i32, f32, vp, vp]
        L.hkv_decode_noalloc.restype = i32
        L.hkv_decode_noalloc.argtypes = [vp, vp, vp, vp, vp, C.POINTER(i64), i32, vp, i32, vp, vp, i32, i32, i32, i32, i32,
                                         f32, f32, vp, vp, i32, vp, vp]
        L.hkv_decode_noalloc_status.restype = i32
        L.hkv_decode_noalloc_status.argtypes = [C.POINTER(i32), vp]
        L.hkv_write_rot.restype = i32
        L.hkv_write_rot.argtypes = L.hkv_write.argtypes[:-1] + [vp, vp]
        L.hkv_decode_rot.restype = i32
        L.hkv_decode_rot.argtypes = L.hkv_decode.argtypes[:-2] + [vp, vp, vp]
        L.hkv_dequant.restype = i32
        L.hkv_dequant.argtypes = [vp, vp, vp, vp, C.POINTER(i64), i32, vp, i32, vp, vp, i32, i64, i64, vp, vp, i32, i32,
                                  i32, vp]
        L.hkv_write_k8.restype = i32
        L.hkv_write_k8.argtypes = [vp, vp, i64, i64, i64, i64, vp, vp, vp, C.POINTER(i64), i32, vp, i64, vp, vp, i32, i32,
                                   i32, vp]
        L.hkv_decode_k8.restype = i32
        L.hkv_decode_k8.argtypes = [vp, vp, vp, vp, C.POINTER(i64), i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, f32,
                                    f32, vp, vp, vp, C.c_size_t, i32, vp, vp]
        L.hkv_dequant_k8.restype = i32
        L.hkv_dequant_k8.argtypes = [vp, vp, vp, C.POINTER(i64), i32, vp, i32, vp, vp, i32, i64, i64, vp, vp, i32, i32,
                                     i32, vp]
        L.hkv_selftest_wait_timeout.restype = i32
        L.hkv_selftest_wait_timeout.argtypes = [vp, i64, vp]
        L.hkv_selftest_codec.restype = i32
        L.hkv_selftest_codec.argtypes = [vp, C.c_size_t, vp]
        L.hkv_probe_issue_rates.restype = i32
        L.hkv_probe_issue_rates.argtypes = [vp, C.c_size_t, i32, vp]
        L.hkv_set_option.restype = i32
        L.hkv_set_option.argtypes = [i32, i32]
        L.hkv_workspace_status.restype = i32
        L.hkv_workspace_status.argtypes = [vp, C.POINTER(i32), vp]
        _lib = L
    return _lib


def check(code: int, where: str):
    if code != 0:
        raise HkvError(code, where)
