"""ctypes binding of libniti_b200.so (the C ABI declared in include/niti_b200.h).

There is no other implementation behind these calls: if the library has not been built
(``python -m niti_b200.build``) importing this module raises, and every non-zero status
code becomes a ``RuntimeError`` carrying the library's own message.
"""
import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libniti_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: the CUDA kernels of niti_b200 have not been built. "
        "Run `python -m niti_b200.build` (needs nvcc); there is no CPU or PyTorch fallback.")

lib = C.CDLL(LIB_PATH)

_p, _i, _i64, _u64, _u32, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_uint32, C.c_size_t

SIGNATURES = {
    "niti_set_option": (_i, [_i, _i]),
    "niti_version": (_i, []),
    "niti_strerror": (C.c_char_p, [_i]),
    "niti_last_cuda_error": (C.c_char_p, []),
    "niti_conv_fprop_scratch_bytes": (_sz, [_i] * 7),
    "niti_conv_fprop_i8": (_i, [_p, _p, _p, _p, _p, _sz] + [_i] * 9 + [_p, _p]),
    "niti_conv_fprop_i4_scratch_bytes": (_sz, [_i] * 7),
    "niti_conv_fprop_i4": (_i, [_p, _p, _p, _p, _p, _sz] + [_i] * 8 + [_p, _p]),
    "niti_conv_fprop_requant_supported": (_i, [_i] * 5),
    "niti_conv_dgrad_requant_supported": (_i, [_i] * 5),
    "niti_conv_fprop_requant_i8": (_i, [_p, _p, _p, _p, _p, _sz] + [_i] * 8 + [_i, _p, _u32, _u64, _i, _p, _p, _p, _p, _p, _p]),
    "niti_conv_fprop_requant_pool_supported": (_i, [_i] * 8),
    "niti_conv_fprop_requant_pool_i8": (_i, [_p, _p, _p, _p, _p] + [_i] * 8 + [_i, _p, _u32, _u64, _i, _p, _p, _p, _p, _p, _p]),
    "niti_conv_dgrad_requant_i8": (_i, [_p, _p, _p, _p] + [_i] * 8 + [_i, _p, _u32, _u64, _p, _p, _p, _p, _p, _p, _p]),
    "niti_conv_dgrad_requant_side_bytes": (_sz, [_i] * 8),
    "niti_conv_dgrad_requant_side_i8": (_i, [_p, _p, _p, _p, _p, _sz] + [_i] * 8 + [_i, _p, _u32, _u64, _p, _p, _p, _p, _p, _p, _p]),
    "niti_conv_dgrad_i8": (_i, [_p, _p, _p, _p] + [_i] * 8 + [_p, _p]),
    "niti_conv_wgrad_scratch_bytes": (_sz, [_i] * 7),
    "niti_conv_wgrad_i8": (_i, [_p, _p, _p, _p, _p, _sz] + [_i] * 8 + [_p, _p]),
    "niti_conv_wgrad_accumulate_multi_max": (_i, []),
    "niti_conv_wgrad_accumulate_multi_i8": (_i, [_p, _i, _p, _p]),
    "niti_conv_wgrad_patches_scratch_bytes": (_sz, [_i] * 7),
    "niti_conv_wgrad_patches_i8": (_i, [_p, _p, _p, _p, _p, _sz] + [_i] * 7 + [_p, _p]),
    "niti_conv_wgrad_builtin_scratch_i8": (_i, [_p, _p, _p, _p] + [_i] * 8 + [_p, _p]),
    "niti_gemm_i8": (_i, [_p, _p, _p, _p] + [_i] * 5 + [_p, _p]),
    "niti_requant_i8": (_i, [_p, _p, _p, _i64, _i, _i, _i, _p, _u32, _u64, _i, _p, _p, _p, _p, _p]),
    "niti_absmax_i32": (_i, [_p, _i64, _p, _p]),
    "niti_group_conv1_i8": (_i, [_p, _p, _p] + [_i] * 7 + [_p]),
    "niti_maxpool_fwd_i8": (_i, [_p, _p] + [_i] * 6 + [_p]),
    "niti_maxpool_bwd_i8": (_i, [_p, _p, _p] + [_i] * 7 + [_p]),
    "niti_relu_fwd_i8": (_i, [_p, _p, _i64, _p]),
    "niti_relu_bwd_i8": (_i, [_p, _p, _p, _i64, _p]),
    "niti_dropout_i8": (_i, [_p, _p, _i64, _i64, _p, _u32, _p]),
    "niti_loss_i8": (_i, [_p, _p, _p, _p, _i, _i, _p, _u32, _u64, _p]),
    "niti_update_i8": (_i, [_p, _p, _p, _i64, _i, _i, _p, _u32, _p]),
    "niti_quantize_input_f32": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _p]),
    "niti_selftest_barrier_timeout": (_i, [_p, _p, _p]),
    "niti_absmax_f32": (_i, [_p, _i64, _p, _p]),
    "niti_quantize_input_with_max_f32": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _p]),
    "niti_update_multi_scratch_bytes": (_sz, []),
    "niti_update_multi_i8": (_i, [_p, _i, _i, _i, _i, _p, _p, _sz, _p, _p]),
    "niti_conv_wgrad_accumulate_supported": (_i, [_i] * 5),
    "niti_conv_wgrad_accumulate_i8": (_i, [_p, _p, _p] + [_i] * 8 + [_p, _p]),
    "niti_fc_head_supported": (_i, [_i, _i, _i]),
    "niti_fc_head_scratch_bytes": (_sz, [_i, _i, _i]),
    "niti_fc_head_train_i8": (_i, [_p, _p]),
    "niti_dp_exchange_bytes": (_sz, []),
    "niti_peer_copy": (_i, [_p, _p, _sz, _p]),
    "niti_peer_arena_create": (_i, [_sz, _p, _p]),
    "niti_peer_arena_open": (_i, [_p, _p]),
    "niti_peer_arena_close": (_i, [_p]),
    "niti_peer_arena_destroy": (_i, [_p]),
    "niti_dp_update_i8": (_i, [_p, _p]),
}


class UpdateItem(C.Structure):
    """niti_update_item of include/niti_b200.h"""
    _fields_ = [("w", _p), ("g32", _p), ("maxabs", _p), ("n", _i64), ("rng_stream", _u32)]


class WgradItem(C.Structure):
    """niti_wgrad_item of include/niti_b200.h"""
    _fields_ = [("x", _p), ("err", _p), ("g32", _p)] + [(n, C.c_int32) for n in ("N", "H", "W", "C", "K", "R", "S", "pad")]


class DpItem(C.Structure):
    """niti_dp_item of include/niti_b200.h"""
    _fields_ = [("w_offset", _i64), ("g_offset", _i64), ("n", _i64), ("rng_stream", _u32), ("staged", _p * 8)]


class DpUpdateArgs(C.Structure):
    """niti_dp_update_args of include/niti_b200.h"""
    _fields_ = [("items", _p), ("count", C.c_int32), ("rank", C.c_int32), ("world", C.c_int32),
                ("weights", _p), ("grads", _p), ("exchange", _p), ("mu", C.c_int32), ("round_mode", C.c_int32),
                ("seed", _p), ("maxabs", _p), ("status", _p)]


class FcHeadArgs(C.Structure):
    """niti_fc_head_args of include/niti_b200.h"""
    _fields_ = [("x", _p), ("exp_x", _p), ("w", _p), ("exp_w", _p), ("target", _p), ("out8", _p), ("exp_out", _p),
                ("err8", _p), ("e8", _p), ("exp_err", _p), ("g32", _p), ("grad_maxabs", _p),
                ("scratch", _p), ("scratch_bytes", _sz), ("B", C.c_int32), ("F", C.c_int32), ("J", C.c_int32),
                ("dropout", C.c_int32), ("bits", C.c_int32), ("act_round", C.c_int32), ("err_round", C.c_int32),
                ("grad_round", C.c_int32), ("mu", C.c_int32), ("update", C.c_int32), ("seed", _p),
                ("layer_stream", _u32), ("dropout_stream", _u32), ("loss_stream", _u32), ("sample_offset", _u64),
                ("status", _p)]



for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


class NitiError(RuntimeError):
    pass


def check(code, what):
    if code != 0:
        msg = lib.niti_strerror(code).decode()
        if code == -3:
            msg += ": " + lib.niti_last_cuda_error().decode()
        raise NitiError(f"{what} failed with status {code}: {msg}")
