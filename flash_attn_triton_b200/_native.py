"""ctypes binding of libfa_b200.so (the C ABI declared in include/fa_b200.h).

There is no CPU fallback: if the library is missing or a call fails, an exception is
raised.  Build it with `python -m flash_attn_triton_b200.build`.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# FA_B200_LIB selects another build of the same library (e.g. a variant made with FA_BUILD_TAG)
LIB_PATH = os.environ.get("FA_B200_LIB") or os.path.join(_HERE, "libfa_b200.so")

FA_F16, FA_BF16, FA_F32 = 0, 1, 2
IMPL_AUTO, IMPL_MMA, IMPL_TCGEN05 = 0, 1, 2
_I64x3 = C.c_int64 * 3


class AttnArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("device", C.c_int32), ("impl", C.c_int32),
        ("batch", C.c_int32), ("seqlen_q", C.c_int32), ("seqlen_k", C.c_int32),
        ("heads_q", C.c_int32), ("heads_kv", C.c_int32), ("head_dim", C.c_int32),
        ("total_q", C.c_int32), ("total_k", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
        ("q_stride", _I64x3), ("k_stride", _I64x3), ("v_stride", _I64x3), ("o_stride", _I64x3),
        ("lse2", C.c_void_p), ("lse_stride", _I64x3),
        ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_k", C.c_void_p),
        ("softmax_scale", C.c_float), ("softcap", C.c_float), ("alibi_slopes", C.c_void_p),
        ("causal", C.c_int32), ("window_left", C.c_int32), ("window_right", C.c_int32),
        ("q_pos_offset", C.c_int32),
        ("dout", C.c_void_p), ("do_stride", _I64x3), ("delta", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("dq_stride", _I64x3), ("dk_stride", _I64x3), ("dv_stride", _I64x3),
        ("seqused_q", C.c_void_p), ("seqused_k", C.c_void_p),
        ("attn_bias", C.c_void_p), ("bias_stride", C.c_int64 * 4),
        ("dropout_p", C.c_float), ("dropout_row_stride", C.c_int32), ("dropout_seed", C.c_uint64),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("device", C.c_int32),
        ("batch", C.c_int32), ("seqlen_q", C.c_int32), ("heads_q", C.c_int32),
        ("heads_kv", C.c_int32), ("head_dim", C.c_int32),
        ("q", C.c_void_p), ("o", C.c_void_p), ("q_stride", _I64x3), ("o_stride", _I64x3),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("kc_stride", _I64x3), ("vc_stride", _I64x3),
        ("page_size", C.c_int32), ("num_pages", C.c_int32),
        ("block_table", C.c_void_p), ("block_table_stride", C.c_int32),
        ("cache_batch_idx", C.c_void_p), ("cache_seqlens", C.c_void_p),
        ("cache_leftpad", C.c_void_p),
        ("k_new", C.c_void_p), ("v_new", C.c_void_p), ("kn_stride", _I64x3), ("vn_stride", _I64x3),
        ("seqlen_new", C.c_int32),
        ("rotary_cos", C.c_void_p), ("rotary_sin", C.c_void_p),
        ("rotary_dim", C.c_int32), ("rotary_seqlen", C.c_int32), ("rotary_interleaved", C.c_int32),
        ("softmax_scale", C.c_float), ("alibi_slopes", C.c_void_p),
        ("causal", C.c_int32), ("window_left", C.c_int32), ("window_right", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("num_splits", C.c_int32),
    ]


class Int8Args(C.Structure):
    _fields_ = [
        ("device", C.c_int32), ("impl", C.c_int32),
        ("batch", C.c_int32), ("heads", C.c_int32), ("seqlen", C.c_int32), ("head_dim", C.c_int32),
        ("q", C.c_void_p), ("k8", C.c_void_p), ("s_k", C.c_void_p), ("v", C.c_void_p),
        ("o", C.c_void_p), ("lse2", C.c_void_p),
        ("softmax_scale", C.c_float), ("causal", C.c_int32),
        ("q8_scratch", C.c_void_p), ("sq_scratch", C.c_void_p),
        ("seqlen_k_valid", C.c_int32), ("q_pos_offset", C.c_int32),
    ]


class RotaryArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("device", C.c_int32),
        ("batch", C.c_int32), ("seqlen", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("x", C.c_void_p), ("out", C.c_void_p), ("x_stride", _I64x3), ("out_stride", _I64x3),
        ("cos", C.c_void_p), ("sin", C.c_void_p),
        ("rotary_dim", C.c_int32), ("rotary_seqlen", C.c_int32),
        ("interleaved", C.c_int32), ("conjugate", C.c_int32),
        ("seqlen_offset", C.c_int32), ("seqlen_offsets", C.c_void_p), ("cu_seqlens", C.c_void_p),
    ]


EXPORTS = {
    "fa_fwd": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "fa_bwd_preprocess": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "fa_bwd_dq": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "fa_bwd_dkdv": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "fa_attn_probs": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p, C.POINTER(C.c_int64 * 4), C.c_void_p, C.c_int64,
                                C.c_void_p]),
    "fa_varlen_fwd": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "fa_varlen_bwd_dq": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "fa_varlen_bwd_dkdv": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "fa_decode_paged": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "fa_decode_workspace_bytes": (C.c_size_t, [C.POINTER(DecodeArgs)]),
    "fa_decode_paged_static": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "fa_decode_static_scratch_bytes": (C.c_size_t, []),
    "fa_quantize_k_int8": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                     C.c_int32, C.c_void_p]),
    "fa_fwd_int8": (C.c_int, [C.POINTER(Int8Args), C.c_void_p]),
    "fa_rotary": (C.c_int, [C.POINTER(RotaryArgs), C.c_void_p]),
    "fa_gather_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                 C.c_int32, C.c_void_p]),
    "fa_scatter_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                  C.c_int32, C.c_int32, C.c_void_p]),
    "fa_version": (C.c_char_p, []),
    "fa_last_error": (C.c_char_p, []),
    "fa_fwd_uses_tcgen05": (C.c_int, [C.POINTER(AttnArgs)]),
    "fa_device_wait_status": (C.c_int, [C.c_int]),
    "fa_device_wait_clear": (C.c_int, [C.c_int]),
    "fa_wait_probe": (C.c_int, [C.c_int32, C.c_int64, C.c_void_p]),
    "fa_debug_set_wait_status": (C.c_int, [C.c_int32, C.c_int32]),
    "fa_mma_peak_probe": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "fa_sizeof_args": (C.c_size_t, [C.c_int]),
}

_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the CUDA extension with "
                "`python -m flash_attn_triton_b200.build` (there is no CPU fallback)")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        for which, st in ((0, AttnArgs), (1, DecodeArgs), (2, Int8Args), (3, RotaryArgs)):
            if l.fa_sizeof_args(which) != C.sizeof(st):
                raise RuntimeError(f"ABI mismatch for {st.__name__}: library "
                                   f"{l.fa_sizeof_args(which)} vs binding {C.sizeof(st)}")
        _lib = l
    return _lib


class DeviceWaitError(RuntimeError):
    """A bounded wait inside a kernel ran out earlier on this device (FA_ERR_DEVICE_WAIT): the
    kernel that hit it left its outputs incomplete and the tcgen05 kernels refuse to launch
    until `lib().fa_device_wait_clear(device)`."""


def check(status, what):
    if status != 0:
        msg = lib().fa_last_error().decode(errors="replace")
        if status == -1:
            raise ValueError(f"{what}: {msg}")
        if status == -5:
            raise DeviceWaitError(f"{what}: {msg}")
        raise RuntimeError(f"{what} failed (status {status}): {msg}")


def dtype_code(t: torch.dtype) -> int:
    if t == torch.float16:
        return FA_F16
    if t == torch.bfloat16:
        return FA_BF16
    raise ValueError(f"unsupported dtype {t}")


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t):
    return None if t is None else t.data_ptr()


def strides3(t, dims):
    """Element strides of tensor `t` in (batch,row,head) order; `dims` gives the tensor's
    dimension index of each (None -> 0)."""
    return _I64x3(*[0 if d is None else t.stride(d) for d in dims])


def kernel_ready(t) -> bool:
    """True when `t` can be handed to the kernels as is: unit inner stride, 16-byte rows."""
    return (t.stride(-1) == 1 and t.data_ptr() % 16 == 0
            and all(s % 8 == 0 for s in t.stride()[:-1]))
