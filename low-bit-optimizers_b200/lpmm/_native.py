"""ctypes binding of the C-ABI CUDA library (``include/lpmm_b200.h``).

The library is the only implementation of the optimizer-step arithmetic in this package: if it
cannot be loaded, importing this module raises, and nothing falls back to torch ops or the CPU.
"""
import ctypes
import os

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_lib", "liblpmm_b200.so")

c_float_p = ctypes.c_void_p
c_void_p = ctypes.c_void_p


class Tensor(ctypes.Structure):
    """``lpmm_b200_tensor``"""
    _fields_ = [
        ("p", ctypes.c_void_p),
        ("g", ctypes.c_void_p),
        ("m", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("m_scale", ctypes.c_void_p),
        ("v_scale", ctypes.c_void_p),
        ("numel", ctypes.c_int64),
        ("kind", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
    ]


class Hyper(ctypes.Structure):
    """``lpmm_b200_hyper``"""
    _fields_ = [(n, ctypes.c_float) for n in ("beta1", "beta2", "lr", "weight_decay", "eps", "step")]


class StepTensor(ctypes.Structure):
    """``lpmm_b200_step_tensor``"""
    _fields_ = [
        ("p", ctypes.c_void_p),
        ("g", ctypes.c_void_p),
        ("numel", ctypes.c_int64),
        ("ndim", ctypes.c_int32),
        ("first", ctypes.c_int32),
        ("shape", ctypes.c_int64 * 8),
        ("m_mode", ctypes.c_int32),
        ("v_mode", ctypes.c_int32),
        ("m", ctypes.c_void_p),
        ("m_max1", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("v_max1", ctypes.c_void_p),
        ("v_max_dims_old", ctypes.c_void_p * 8),
        ("v_max_dims_new", ctypes.c_void_p * 8),
        ("row", ctypes.c_void_p),
        ("col", ctypes.c_void_p),
        ("m_bits", ctypes.c_int32),
        ("v_bits", ctypes.c_int32),
        ("m_group", ctypes.c_int32),
        ("v_group", ctypes.c_int32),
    ]


STATE_FP32, STATE_GROUP4, STATE_RANK1_4, STATE_FACTORED = 0, 1, 2, 3
KIND_Q4 = 0
KIND_FP32 = 1
DTYPE_BF16 = 1
DTYPE_FP16 = 2
FLAG_PARAMS_WITHIN_TOLERANCE = 1
GROUP = 128
PACK_GROUP = 2048
STATIC_SCRATCH_BYTES = 8 * 1024 * 1024


class NativeError(RuntimeError):
    pass


def _load():
    if not os.path.exists(_LIB_PATH):
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python low-bit-optimizers_b200/build.py` "
            "(needs nvcc; there is no non-CUDA implementation)")
    lib = ctypes.CDLL(_LIB_PATH)
    f, i64, i32, vp, d = ctypes.c_float, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_double
    sigs = {
        "lpmm_b200_strerror": (ctypes.c_char_p, [i32]),
        "lpmm_b200_last_cuda_error": (ctypes.c_char_p, []),
        "lpmm_b200_abi_version": (i32, []),
        "lpmm_b200_adamw4bit_single_tensor": (i32, [vp] * 8 + [f] * 6 + [i64, vp]),
        "lpmm_b200_adamw_single_tensor": (i32, [vp] * 4 + [f] * 6 + [i64, vp]),
        "lpmm_b200_adamw4bit_multi_tensor": (i32, [ctypes.POINTER(Tensor), i32, vp, vp, Hyper, i64, i64, vp]),
        "lpmm_b200_adamw4bit_multi_tensor_flags": (i32, [ctypes.POINTER(Tensor), i32, vp, vp, Hyper, i64, i64,
                                                         ctypes.c_uint32, vp]),
        "lpmm_b200_adamw4bit_multi_tensor_16bit": (i32, [ctypes.POINTER(Tensor), i32, i32, vp, vp, Hyper, i64, i64, vp]),
        "lpmm_b200_adamw4bit_multi_tensor_16bit_flags": (i32, [ctypes.POINTER(Tensor), i32, i32, vp, vp, Hyper, i64, i64,
                                                               ctypes.c_uint32, vp]),
        "lpmm_b200_adamw4bit_multi_tensor_16bit_peers": (i32, [ctypes.POINTER(Tensor), i32, i32, vp, vp, Hyper, i64, i64,
                                                               ctypes.POINTER(i64), i32, ctypes.c_uint32, vp]),
        "lpmm_b200_adamw4bit_multi_tensor_peers_flags": (i32, [ctypes.POINTER(Tensor), i32, vp, vp, Hyper, i64, i64,
                                                               ctypes.POINTER(i64), i32, ctypes.c_uint32, vp]),
        "lpmm_b200_adamw4bit_multi_tensor_peers": (i32, [ctypes.POINTER(Tensor), i32, vp, vp, Hyper, i64, i64,
                                                         ctypes.POINTER(i64), i32, vp]),
        "lpmm_b200_adamw4bit_multi_tensor_zero1": (i32, [ctypes.POINTER(Tensor), i32, vp, vp, Hyper, i64, i64,
                                                         ctypes.POINTER(i64), i32, ctypes.POINTER(i64), i32, f, vp]),
        "lpmm_b200_count_groups": (i64, [ctypes.POINTER(Tensor), i32]),
        "lpmm_b200_bias_corrections": (i32, [f, f, f, vp, vp]),
        "lpmm_b200_packed_len": (i64, [i64]),
        "lpmm_b200_pack_nonlinear4": (i32, [vp, i64, vp, vp, vp]),
        "lpmm_b200_unpack_nonlinear4": (i32, [vp, vp, i64, vp, vp]),
        "lpmm_b200_quant_group4": (i32, [vp, i64, vp, vp, vp, vp]),
        "lpmm_b200_dequant_group4": (i32, [vp, vp, vp, i64, vp, vp]),
        "lpmm_b200_axis_absmax": (i32, [vp, ctypes.POINTER(i64), i32, ctypes.POINTER(vp), vp]),
        "lpmm_b200_quant_rank1_4": (i32, [vp, ctypes.POINTER(i64), i32, vp, ctypes.POINTER(vp), vp, vp]),
        "lpmm_b200_dequant_rank1_4": (i32, [vp, vp, ctypes.POINTER(vp), ctypes.POINTER(i64), i32, vp, vp]),
        "lpmm_b200_packed_len_bits": (i64, [i64, i32]),
        "lpmm_b200_pack_nonlinear": (i32, [vp, i64, vp, i32, vp, vp]),
        "lpmm_b200_unpack_nonlinear": (i32, [vp, vp, i32, i64, vp, vp]),
        "lpmm_b200_quant_group": (i32, [vp, i64, vp, i32, i64, vp, vp, vp]),
        "lpmm_b200_dequant_group": (i32, [vp, vp, i32, i64, vp, i64, vp, vp]),
        "lpmm_b200_quant_rank1": (i32, [vp, ctypes.POINTER(i64), i32, vp, i32, ctypes.POINTER(vp), vp, vp]),
        "lpmm_b200_dequant_rank1": (i32, [vp, vp, i32, ctypes.POINTER(vp), ctypes.POINTER(i64), i32, vp, vp]),
        "lpmm_b200_pack_nonlinear_sr": (i32, [vp, i64, vp, i32, vp, ctypes.c_uint64, ctypes.c_uint64, vp]),
        "lpmm_b200_quant_group_sr": (i32, [vp, i64, vp, i32, i64, vp, vp, ctypes.c_uint64, ctypes.c_uint64, vp]),
        "lpmm_b200_quant_rank1_sr": (i32, [vp, ctypes.POINTER(i64), i32, vp, i32, ctypes.POINTER(vp), vp, ctypes.c_uint64,
                                           ctypes.c_uint64, vp]),
        "lpmm_b200_sgd_lowbit_step": (i32, [vp, vp, i64, vp, vp, i32, i32, i64, i32, vp, d, d, d, d, i32, i32, vp]),
        "lpmm_b200_sgd4bit_multi_tensor": (i32, [ctypes.POINTER(Tensor), i32, vp, d, d, d, d, i32, i32, i64, i64, vp]),
        "lpmm_b200_adamw4bit_unfused_step": (i32, [ctypes.POINTER(StepTensor), vp, vp] + [d] * 6 + [vp, i64, vp]),
        "lpmm_b200_adamw4bit_unfused_multi_tensor": (i32, [ctypes.POINTER(Tensor), i32, vp, vp] + [d] * 6
                                                     + [i64, i64, vp]),
        "lpmm_b200_unfused_step_many_scratch_bytes": (i64, [ctypes.POINTER(vp), i32]),
        "lpmm_b200_adamw4bit_unfused_step_many": (i32, [ctypes.POINTER(vp), i32, vp, vp] + [d] * 5
                                                  + [ctypes.POINTER(d), vp, i64, vp]),
        "lpmm_b200_adamw4bit_unfused_step_many_flags": (i32, [ctypes.POINTER(vp), i32, vp, vp] + [d] * 5
                                                        + [ctypes.POINTER(d), vp, i64, vp, ctypes.c_uint32]),
        "lpmm_b200_adamw4bit_fused_arith_step_many_flags": (i32, [ctypes.POINTER(vp), i32, vp, vp] + [d] * 5
                                                            + [ctypes.POINTER(d), vp, i64, vp, ctypes.c_uint32]),
        "lpmm_b200_adamw4bit_fused_arith_step": (i32, [ctypes.POINTER(StepTensor), vp, vp] + [d] * 6 + [vp]),
        "lpmm_b200_adamw4bit_fused_arith_step_many": (i32, [ctypes.POINTER(vp), i32, vp, vp] + [d] * 5
                                                      + [ctypes.POINTER(d), vp, i64, vp]),
        "lpmm_b200_factored_scratch_bytes": (i64, [ctypes.POINTER(i64), i32]),
        "lpmm_b200_adamw4bit_factored_step_noalloc": (i32, [ctypes.POINTER(StepTensor), vp] + [d] * 6 + [vp]),
        "lpmm_b200_narrow_fp32": (i32, [vp, vp, i64, i32, vp]),
        "lpmm_b200_test_exactness": (i32, [i32, vp, ctypes.c_uint64, i64, vp, vp]),
        "lpmm_b200_sgd4bit_step": (i32, [vp, vp, i64, vp, vp, i32, i32, vp, d, d, d, d, i32, i32, vp]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib, sigs


lib, SIGNATURES = _load()


def check(status):
    """Raise ``NativeError`` (a RuntimeError, like the reference's TORCH_CHECK failures) on a
    non-zero status."""
    if status != 0:
        msg = lib.lpmm_b200_strerror(int(status)).decode()
        if status == -4:
            msg += ": " + lib.lpmm_b200_last_cuda_error().decode()
        raise NativeError(f"lpmm_b200 status {status}: {msg}")


def current_stream_handle():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
