"""ctypes binding of ``libvq_b200.so`` (the C ABI declared in ``include/vq_b200.h``).

The library is built in-tree by ``build()`` (``nvcc`` for sm_100a) and loaded
lazily.  There is no fallback: if the library is missing, every operator
raises.
"""

import ctypes
import glob
import os
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG, "csrc")
_LIBDIR = os.path.join(_PKG, "lib")
LIB_PATH = os.path.join(_LIBDIR, "libvq_b200.so")
INCLUDE_DIR = os.path.join(os.path.dirname(_PKG), "include")

VQ_BF16, VQ_F16, VQ_F32 = 0, 1, 2
(ROUND_NONE, ROUND_TABLE, ROUND_INT, ROUND_MINIFLOAT, ROUND_STEPS, ROUND_SEARCH,
 ROUND_STOCHASTIC) = range(7)
MAX_STEPS = 32
MAX_DIMS = 5

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


class VqRound(ctypes.Structure):
    _fields_ = [
        ("mode", ctypes.c_int32),
        ("table", ctypes.c_void_p),
        ("lo", ctypes.c_float),
        ("hi", ctypes.c_float),
        ("emin", ctypes.c_int32),
        ("mbits", ctypes.c_int32),
        ("max_norm", ctypes.c_float),
        ("is_signed", ctypes.c_int32),
        ("n_steps", ctypes.c_int32),
        ("steps", ctypes.c_void_p),
        ("nan_value", ctypes.c_uint16),
        ("edges", ctypes.c_void_p),
        ("levels", ctypes.c_void_p),
        ("n_edges", ctypes.c_int32),
        ("n_levels", ctypes.c_int32),
        ("seed", ctypes.c_void_p),
    ]


class VqBroadcast(ctypes.Structure):
    _fields_ = [
        ("ndim", ctypes.c_int32),
        ("size", ctypes.c_int64 * MAX_DIMS),
        ("div", ctypes.c_int64 * MAX_DIMS),
        ("stride", ctypes.c_int64 * MAX_DIMS),
    ]


class VqBlocks(ctypes.Structure):
    _fields_ = [
        ("O", ctypes.c_int64), ("A", ctypes.c_int64), ("M", ctypes.c_int64),
        ("B", ctypes.c_int64), ("I", ctypes.c_int64),
        ("block_a", ctypes.c_int32), ("block_b", ctypes.c_int32),
    ]


class VqGemmEpilogue(ctypes.Structure):
    _fields_ = [
        ("alpha_cols", ctypes.c_void_p), ("alpha_cols_dtype", ctypes.c_int32),
        ("residual", ctypes.c_void_p), ("ldr", ctypes.c_int64), ("strideR", ctypes.c_int64),
        ("causal_mode", ctypes.c_int32), ("causal_period", ctypes.c_int64),
        ("gate_scale", ctypes.c_void_p), ("gate_scale_dtype", ctypes.c_int32),
        ("round_acc", ctypes.c_int32),
    ]


class VqScaleRule(ctypes.Structure):
    _fields_ = [
        ("quant_max", ctypes.c_float),
        ("power_of_two", ctypes.c_int32),
        ("global_scale", ctypes.c_void_p),
        ("global_scale_dtype", ctypes.c_int32),
        ("scale_round", VqRound),
    ]


_P = ctypes.c_void_p
_I = ctypes.c_int
_I64 = ctypes.c_int64
_F = ctypes.c_float

# name -> argtypes; every function returns int except where noted below.
SIGNATURES = {
    "vq_version": [],
    "vq_vmap": [_P, _P, _I, ctypes.POINTER(VqRound), _I64, _P],
    "vq_quantize": [_P, _P, _P, _P, _I, _I, ctypes.POINTER(VqBroadcast), ctypes.POINTER(VqRound), _P],
    "vq_dequantize": [_P, _P, _P, _P, _I, _I, ctypes.POINTER(VqBroadcast), ctypes.POINTER(VqRound),
                      ctypes.POINTER(VqRound), _P],
    "vq_mx_qparam": [_P, _P, _I, ctypes.POINTER(VqBlocks), ctypes.POINTER(VqScaleRule), _P],
    "vq_quantize_mx": [_P, _P, _P, _I, ctypes.POINTER(VqBlocks), ctypes.POINTER(VqScaleRule),
                       ctypes.POINTER(VqRound), _P],
    "vq_quantize_affine": [_P, _P, _P, _P, _I, ctypes.POINTER(VqBlocks), _F, _F, ctypes.POINTER(VqRound),
                           ctypes.POINTER(VqRound), _P],
    "vq_dequantize_mx": [_P, _P, _P, ctypes.c_int32, _P, _I, _P, _I, ctypes.POINTER(VqBroadcast), _P],
    "vq_amax": [_P, _I, _I64, _P, _P],
    "vq_amax_history_update": [_P, _I, _I64, _I64, _P, _P, _I, _I64, _F, _I, _P, _P],
    "vq_pack_codes": [_P, _I, _P, _I, _I64, _P],
    "vq_outlier_count": [_P, _I, _P, _I64, _I64, _F, _P],
    "vq_outlier_fill": [_P, _I, _P, _P, _P, _P, _I64, _I64, _I64, _F, _I64, _P],
    "vq_spmm_csr": [_P, _I, _P, _P, _P, _I, _P, _I, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _P],
    "vq_unpack_dequantize": [_P, _I, _P, _P, _P, _I, _I, ctypes.POINTER(VqBroadcast), ctypes.POINTER(VqRound), _P],
    "vq_gemm_tn": [_P, _P, _P, _I, _I, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _P, _I, _P, _I, _P],
    "vq_gemm_tn_ex": [_P, _P, _P, _I, _I, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _P, _I, _P, _I,
                      ctypes.POINTER(VqGemmEpilogue), _P],
    "vq_gemm_mx": [_P, _P, _P, _P, _I64, _P, _I, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _P, _I, _P, _I,
                   _P],
    "vq_peer_max": [_P, _I64, _P, _P],
    "vq_peer_gather": [_P, _I64, _I64, _P, _P],
    "vq_peer_reduce_rows": [_P, _I64, _I64, _I64, _P, _P],
    "vq_gemm_status": [_I],
    "vq_nvfp4_scale_bytes": [_I64, _I64],
    "vq_quantize_nvfp4": [_P, _P, _I, _P, _P, _I64, _I64, _P],
    "vq_pack_nvfp4": [_P, _P, _P, _P, _I64, _I64, _P, _P],
    "vq_gemm_nvfp4": [_P, _P, _P, _P, _P, _I, _I64, _I64, _I64, _I64, _I64, _I64, _P, _I, _P, _I, _P],
    "vq_gemm_nvfp4_ex": [_P, _P, _P, _P, _P, _I, _I64, _I64, _I64, _I64, _I64, _I64, _P, _I, _P, _I, _P, _I, _P],
    "vq_gemm_lut4_workspace_floats": [_I64, _I64, _I64],
    "vq_gemm_lut4_counters": [_I64],
    "vq_gemm_lut4": [_P, _I64, _P, _P, _I, _I64, _P, _P, _P, _I, _P, _I, _I64, _I64, _P, _I, _P, _I, _P, _P, _P],
    "vq_pack_lut4": [_P, _P, _I64, _I64, _P, _P],
    "vq_kivi_decode_attention": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _F, _P],
    "vq_kivi_read_2bit": [_P, _P, _P, _P, _I64, _I64, _I64, _I, _I64, _P],
    "vq_gptq_block": [_P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I, _F, _F, _I, ctypes.POINTER(VqRound),
                      ctypes.POINTER(VqRound), _P],
    "vq_gptq_update": [_P, _P, _P, _I64, _I64, _I64, _I64, _P],
    "vq_gptq_block_step_static": [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _I, _F, _F, _I, ctypes.POINTER(VqRound),
                                  ctypes.POINTER(VqRound), _P],
    "vq_hadamard_rotate": [_P, _P, _I, _P, _I64, _I64, _I64, _P],
    "vq_quantize_fp8": [_P, _P, _I, _P, _I, _I64, _I64, _P],
    "vq_softmax_quantize_fp8": [_P, _P, _I64, _I64, _F, _P, _I64, _I64, _P, _I, _I, _P],
    "vq_silu_mul_amax": [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _P],
    "vq_rope_heads_bf16": [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _P],
    "vq_rope_decode_append": [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _P],
    "vq_fp8_roundtrip_add": [_P, _P, _P, _I64, _P, _I, _P],
    "vq_attention_bf16": [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _F, _I, _P],
    "vq_attention_fp8": [_P, _P, _P, _P, _I64, _P, _I64, _I64, _I64, _I64, _P, _I, _F, _P, _I, _P, _I, _P, _I, _I, _P],
    "vq_attention_status": [_I],
    "vq_rmsnorm_backward_programs": [_I64, _I64],
    "vq_rmsnorm_backward": [_P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _P],
    "vq_rmsnorm_quantize_fp8": [_P, _P, _P, _I64, _I64, _F, _P, _I, _P],
    "vq_silu_mul_quantize_fp8": [_P, _P, _P, _I64, _I64, _I64, _I64, _P, _I, _P],
    "vq_qkv_post_fp8": [_P, _P, _P, _I64, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _P, _I, _P, _I, _P, _I, _P],
    "vq_rope_quantize_fp8": [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _P, _I, _P],
    "vq_transpose_quantize_fp8": [_P, _P, _P, _P, _I, _I64, _I64, _I64, _I64, _P, _I, _P],
}
IN_BF16, IN_F16, IN_E4M3, IN_E5M2 = range(4)
_INT64_RESULTS = ("vq_nvfp4_scale_bytes", "vq_rmsnorm_backward_programs", "vq_gemm_lut4_workspace_floats",
                  "vq_gemm_lut4_counters")


def sources():
    return sorted(glob.glob(os.path.join(_CSRC, "*.cu")))


def _stale():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = sources() + glob.glob(os.path.join(_CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE_DIR, "*.h"))
    return any(os.path.getmtime(d) > built for d in deps)


def build(force=False, verbose=False):
    """Compile every ``csrc/*.cu`` into ``lib/libvq_b200.so`` for sm_100a."""
    if not force and not _stale():
        return LIB_PATH
    os.makedirs(_LIBDIR, exist_ok=True)
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(_LIBDIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        cmd = ["nvcc", *NVCC_FLAGS, "-I", INCLUDE_DIR, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose and out:
            print(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
    link = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH, *objs]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    return LIB_PATH


_lib = None


def lib():
    """The loaded library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`. "
                "There is no fallback implementation.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = ctypes.c_int64 if name in _INT64_RESULTS else ctypes.c_int
        handle.vq_last_error.restype = ctypes.c_char_p
        handle.vq_last_error.argtypes = []
        _lib = handle
    return _lib


def _cuda_device_of(values, found):
    for v in values:
        if isinstance(v, (list, tuple)):
            found = _cuda_device_of(v, found)
        elif hasattr(v, "is_cuda") and v.is_cuda:
            if found is None:
                found = v.device
            elif v.device != found:
                raise ValueError(f"operands live on different devices: {found} and {v.device}")
    return found


def device_guarded(fn):
    """Run ``fn`` with the device of its CUDA tensor arguments current, so that kernels launch on
    that device's current stream whatever device the caller had selected (a model whose layers are
    placed on several GPUs in one process calls operators with tensors of each of them).  Operands
    spread over different devices are refused."""
    import functools

    import torch

    @functools.wraps(fn)
    def call(*args, **kwargs):
        device = _cuda_device_of(args, None)
        device = _cuda_device_of(kwargs.values(), device)
        if device is None or device.index == torch.cuda.current_device():
            return fn(*args, **kwargs)
        with torch.cuda.device(device):
            return fn(*args, **kwargs)

    return call


def check(rc, what=""):
    if rc != 0:
        msg = lib().vq_last_error().decode(errors="replace")
        raise RuntimeError(f"{what or 'libvq_b200'} failed ({rc}): {msg}")
