"""ctypes binding of ``libjvpattn.so`` (the C ABI declared in ``include/jvpattn.h``).

The shared library is built in-tree with ``nvcc`` for sm_100a by :func:`build` and loaded from this
package's directory.  There is no fallback of any kind: if the library cannot be loaded, or the
device is not a B200, every compute call raises.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import threading

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG_DIR, "csrc")
LIB_PATH = os.path.join(_PKG_DIR, "libjvpattn.so")
SOURCES = ["jvpattn_api.cu", "jvpattn_simt.cu", "jvpattn_sm100_fwd.cu", "jvpattn_sm100_bwd.cu",
           "sm100_tensormap.cu", "rotary.cu", "dual_pointwise.cu", "vocab_head.cu", "vocab_loss.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]

BF16, FP16 = 0, 1
KERNELS_AUTO, KERNELS_SIMT, KERNELS_TCGEN05 = 0, 1, 2

EXPORTS = (
    "jvpattn_fwd", "jvpattn_bwd", "jvpattn_bwd_workspace_bytes", "jvpattn_selected_kernels",
    "jvpattn_launch_count", "jvpattn_device_status", "jvpattn_strerror", "jvpattn_last_cuda_error",
    "jvpattn_abi_version", "jvpattn_profile_begin", "jvpattn_profile_end", "jvpattn_kernel_name",
    "jvpattn_bwd_static", "jvpattn_rotary_cast", "jvpattn_stream_check", "jvpattn_debug_set",
    "jvpattn_ln_modulate", "jvpattn_gated_residual", "jvpattn_flow_map_head", "jvpattn_gelu_dual", "jvpattn_vocab_op",
    "jvpattn_gated_residual_dual", "jvpattn_ln_finalize", "jvpattn_rotary_qkv",
)
DEBUG_WAIT_CYCLES, DEBUG_STALL_NEXT_FWD = 0, 1
STATIC_SCRATCH_ROWS = 262144
NUM_KERNELS = 9


class Dropout(ctypes.Structure):
    """``jvpattn_dropout``: device pointer to the step's 64-bit seed, the call's number within the step, drop probability."""
    _fields_ = [("seed", ctypes.c_void_p), ("call", ctypes.c_uint32), ("p", ctypes.c_float)]


class Tensor4(ctypes.Structure):
    """``jvpattn_tensor``: device pointer + element strides in (batch, head, position, channel) order."""
    _fields_ = [("ptr", ctypes.c_void_p), ("stride", ctypes.c_int64 * 4)]


class Problem(ctypes.Structure):
    """``jvpattn_problem``."""
    _fields_ = [
        ("batch", ctypes.c_int32), ("heads", ctypes.c_int32),
        ("len_q", ctypes.c_int32), ("len_k", ctypes.c_int32),
        ("head_dim", ctypes.c_int32), ("stat_len", ctypes.c_int32),
        ("dtype", ctypes.c_int32), ("kernels", ctypes.c_int32),
        ("scale", ctypes.c_float),
    ]


class JvpAttnError(RuntimeError):
    def __init__(self, code: int, where: str, detail: str = ""):
        self.code = code
        super().__init__(f"{where} failed with code {code}: {detail}")


def _sources_newer_than_lib() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(_CSRC, f) for f in os.listdir(_CSRC)] + [
        os.path.join(os.path.dirname(_PKG_DIR), "include", "jvpattn.h")]
    return any(os.path.getmtime(d) > t for d in deps if os.path.isfile(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile ``libjvpattn.so`` for sm_100a with nvcc (cross-compiles without a GPU)."""
    if not force and not _sources_newer_than_lib():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libjvpattn.so")
    cmd = [nvcc, *NVCC_FLAGS, "-o", LIB_PATH + ".tmp", *[os.path.join(_CSRC, s) for s in SOURCES]]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    if verbose:
        print(proc.stderr)
    return LIB_PATH


_lib = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """Load the library (once) and declare the prototypes.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(or semicat_b200._lib.build()).  There is no CPU or PyTorch fallback for these kernels.")
        lib = ctypes.CDLL(LIB_PATH)
        T = ctypes.POINTER(Tensor4)
        P = ctypes.POINTER(Problem)
        F = ctypes.c_void_p  # float* device pointers are passed as integers
        lib.jvpattn_fwd.argtypes = [P] + [T] * 8 + [F, F, F, ctypes.c_void_p]
        lib.jvpattn_fwd.restype = ctypes.c_int
        lib.jvpattn_bwd.argtypes = [P] + [T] * 10 + [F, F] + [T] * 6 + [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
        lib.jvpattn_bwd.restype = ctypes.c_int
        lib.jvpattn_bwd_static.argtypes = [P] + [T] * 10 + [F, F] + [T] * 6 + [ctypes.c_void_p]
        lib.jvpattn_bwd_static.restype = ctypes.c_int
        lib.jvpattn_rotary_cast.argtypes = ([ctypes.c_void_p] + [ctypes.c_int64] * 3 + [ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                            ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 5 + [ctypes.c_void_p])
        lib.jvpattn_rotary_cast.restype = ctypes.c_int
        lib.jvpattn_bwd_workspace_bytes.argtypes = [P]
        lib.jvpattn_bwd_workspace_bytes.restype = ctypes.c_size_t
        lib.jvpattn_selected_kernels.argtypes = [P, ctypes.c_int]
        lib.jvpattn_selected_kernels.restype = ctypes.c_int
        lib.jvpattn_launch_count.argtypes = []
        lib.jvpattn_launch_count.restype = ctypes.c_uint64
        lib.jvpattn_device_status.argtypes = []
        lib.jvpattn_device_status.restype = ctypes.c_int
        V, I64, I = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
        lib.jvpattn_ln_modulate.argtypes = [I] + [V] * 8 + [I64, I64] + [V] * 7 + [I, I, I, ctypes.c_float, I, I, V]
        lib.jvpattn_ln_modulate.restype = ctypes.c_int
        lib.jvpattn_gated_residual.argtypes = [V] * 4 + [I64, V, I, I, I, I, ctypes.POINTER(Dropout), V]
        lib.jvpattn_gated_residual.restype = ctypes.c_int
        lib.jvpattn_flow_map_head.argtypes = [I, V, V, I64, I64] + [V] * 8 + [I, I, I, I, V]
        lib.jvpattn_flow_map_head.restype = ctypes.c_int
        P3, S9 = ctypes.POINTER(ctypes.c_void_p * 3), ctypes.POINTER(ctypes.c_int64 * 9)
        lib.jvpattn_rotary_qkv.argtypes = [P3, S9, I, P3, S9, I, V, V, I, I, I, I, I, V]
        lib.jvpattn_rotary_qkv.restype = ctypes.c_int
        lib.jvpattn_gelu_dual.argtypes = [I] + [V] * 6 + [I64, I, V]
        lib.jvpattn_gated_residual_dual.argtypes = [I] + [V] * 7 + [I64, I64] + [V] * 7 + [I, I, I, I, ctypes.POINTER(Dropout), V]
        lib.jvpattn_gated_residual_dual.restype = ctypes.c_int
        lib.jvpattn_ln_finalize.argtypes = [V] * 6 + [I64, I64] + [V] * 6 + [I, I, I, V]
        lib.jvpattn_ln_finalize.restype = ctypes.c_int
        lib.jvpattn_gelu_dual.restype = ctypes.c_int
        lib.jvpattn_vocab_op.argtypes = [I, V, V, V, I64, V, I64] + [V] * 9 + [I64, ctypes.c_float, I, I, I, I, V]
        lib.jvpattn_vocab_op.restype = ctypes.c_int
        lib.jvpattn_stream_check.argtypes = [ctypes.c_void_p]
        lib.jvpattn_stream_check.restype = ctypes.c_int
        lib.jvpattn_debug_set.argtypes = [ctypes.c_int, ctypes.c_longlong]
        lib.jvpattn_debug_set.restype = ctypes.c_int
        lib.jvpattn_strerror.argtypes = [ctypes.c_int]
        lib.jvpattn_strerror.restype = ctypes.c_char_p
        lib.jvpattn_last_cuda_error.argtypes = []
        lib.jvpattn_last_cuda_error.restype = ctypes.c_char_p
        lib.jvpattn_abi_version.argtypes = []
        lib.jvpattn_abi_version.restype = ctypes.c_int
        lib.jvpattn_profile_begin.argtypes = []
        lib.jvpattn_profile_begin.restype = ctypes.c_int
        lib.jvpattn_profile_end.argtypes = [ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_uint64)]
        lib.jvpattn_profile_end.restype = ctypes.c_int
        lib.jvpattn_kernel_name.argtypes = [ctypes.c_int]
        lib.jvpattn_kernel_name.restype = ctypes.c_char_p
        if lib.jvpattn_abi_version() != 1:
            raise RuntimeError("libjvpattn.so ABI version mismatch; rebuild it")
        _lib = lib
    return _lib


def check(code: int, where: str) -> None:
    if code == 0:
        return
    lib = load()
    detail = lib.jvpattn_strerror(code).decode()
    if code == -8:
        detail += " [" + lib.jvpattn_last_cuda_error().decode() + "]"
    raise JvpAttnError(code, where, detail)


def launch_count() -> int:
    return int(load().jvpattn_launch_count())


def device_status() -> int:
    return int(load().jvpattn_device_status())


def stream_check(stream: int | None = None) -> None:
    """Wait for ``stream`` (default: the legacy default stream) and raise ``JvpAttnError(-9)`` if a device-side wait of
    one of the kernels has run out; :func:`device_status` then tells which."""
    check(load().jvpattn_stream_check(stream), "jvpattn_stream_check")


def debug_set(knob: int, value: int) -> None:
    """Test hooks of the failure path (``DEBUG_WAIT_CYCLES``, ``DEBUG_STALL_NEXT_FWD``); see include/jvpattn.h."""
    check(load().jvpattn_debug_set(knob, value), "jvpattn_debug_set")


def profile_begin() -> None:
    check(load().jvpattn_profile_begin(), "jvpattn_profile_begin")


def profile_end() -> dict:
    """Stop per-kernel timing; returns {kernel name: (total_ms, launches)} for kernels that ran."""
    lib = load()
    ms = (ctypes.c_double * NUM_KERNELS)()
    n = (ctypes.c_uint64 * NUM_KERNELS)()
    check(lib.jvpattn_profile_end(ms, n), "jvpattn_profile_end")
    return {lib.jvpattn_kernel_name(i).decode(): (float(ms[i]), int(n[i])) for i in range(NUM_KERNELS) if n[i]}
