"""ctypes binding of the C-ABI declared in include/nn_b200.h."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))


class NnbError(RuntimeError):
    """A C-ABI call returned a non-zero nnb_status."""


def lib_path() -> str:
    return os.path.join(_HERE, "libnn-b200.so")


_lib = None

_P = C.c_void_p
_SZ = C.c_size_t
_I = C.c_int

# name -> (restype, argtypes); status-returning unless noted
_SIGNATURES = {
    "nnb_last_error": (C.c_char_p, []),
    "nnb_engine_create": (_I, [_I, C.POINTER(_P)]),
    "nnb_engine_destroy": (None, [_P]),
    "nnb_engine_describe": (_I, [_P, C.c_char_p, _SZ]),
    "nnb_engine_sync": (_I, [_P]),
    "nnb_engine_set_stream": (_I, [_P, _P]),
    "nnb_engine_stream": (_P, [_P]),
    "nnb_engine_launch_count": (C.c_ulonglong, [_P]),
    "nnb_alloc": (_I, [_P, _SZ, C.POINTER(_P)]),
    "nnb_free": (_I, [_P, _P]),
    "nnb_upload": (_I, [_P, _P, _P, _SZ]),
    "nnb_download": (_I, [_P, _P, _P, _SZ]),
    "nnb_zero": (_I, [_P, _P, _SZ]),
    "nnb_tensor_create": (_I, [_P, _SZ, _SZ, C.POINTER(_P)]),
    "nnb_tensor_destroy": (None, [_P]),
    "nnb_tensor_rows": (_SZ, [_P]),
    "nnb_tensor_cols": (_SZ, [_P]),
    "nnb_tensor_data": (_P, [_P]),
    "nnb_tensor_write_epoch": (C.c_ulonglong, [_P]),
    "nnb_tensor_mark_written": (_I, [_P]),
    "nnb_tensor_upload": (_I, [_P, _P, _SZ]),
    "nnb_tensor_download": (_I, [_P, _P, _SZ]),
    "nnb_t_zero": (_I, [_P]),
    "nnb_t_clone": (_I, [_P, C.POINTER(_P)]),
    "nnb_t_copy_into": (_I, [_P, _P]),
    "nnb_t_transpose": (_I, [_P, C.POINTER(_P)]),
    "nnb_t_slice_rows": (_I, [_P, _SZ, _SZ, C.POINTER(_P)]),
    "nnb_t_insert_rows": (_I, [_P, _SZ, _P]),
    "nnb_t_gather_rows": (_I, [_P, _P, C.POINTER(_P)]),
    "nnb_t_scatter_add_rows": (_I, [_P, _P, _P]),
    "nnb_t_rearrange_3d": (_I, [_P, _SZ, _SZ, _SZ, _I, C.POINTER(_P)]),
    "nnb_t_scale_inplace": (_I, [_P, C.c_float]),
    "nnb_t_accumulate": (_I, [_P, _P]),
    "nnb_t_col_reduce_max": (_I, [_P, C.POINTER(_P)]),
    "nnb_t_row_reduce_sum": (_I, [_P, C.POINTER(_P)]),
    "nnb_t_absmean_tau": (_I, [_P, C.POINTER(_P)]),
    "nnb_t_trit_pack": (_I, [_P, _P, C.POINTER(_P)]),
    "nnb_t_trit_pack_into": (_I, [_P, _P, _P]),
    "nnb_t_matmul_q": (_I, [_P, _P, _P, C.POINTER(_P)]),
    "nnb_t_matmul_q_t": (_I, [_P, _P, _P, _SZ, C.POINTER(_P)]),
    "nnb_t_quantize_i8": (_I, [_P, _P, _I, C.POINTER(_P)]),
    "nnb_t_unpack_i8": (_I, [_P, _SZ, C.POINTER(_P)]),
    "nnb_t_matmul_q_i8": (_I, [_P, _P, _P, _P, C.POINTER(_P)]),
    "nnb_t_abs": (_I, [_P, C.POINTER(_P)]),
    "nnb_t_add_row_broadcast": (_I, [_P, _P]),
    "nnb_t_bitlinear_dw_accumulate": (_I, [_P, _P, _P, _P, _P]),
    "nnb_rmsnorm_fwd": (_I, [_P, _P, _P, _SZ, _SZ, _P]),
    "nnb_rmsnorm_bwd": (_I, [_P, _P, _P, _P, _SZ, _SZ, _P, _P]),
    "nnb_rope_tables": (_I, [_P, _SZ, _SZ, _P, _P]),
    "nnb_rope_apply": (_I, [_P, _P, _P, _P, _SZ, _SZ, _SZ, _SZ, _I]),
    "nnb_rope_step": (_I, [_P, _P, _P, _P, _SZ, _SZ, _SZ, _SZ]),
    "nnb_absmean_tau": (_I, [_P, _P, _SZ, _SZ, _P]),
    "nnb_trit_pack": (_I, [_P, _P, _P, _SZ, _SZ, _P]),
    "nnb_col_absmax_scale": (_I, [_P, _P, _SZ, _SZ, _P]),
    "nnb_quantize_i8": (_I, [_P, _P, _SZ, _SZ, _P, _I, _P]),
    "nnb_unpack_i8": (_I, [_P, _P, _SZ, _SZ, _P]),
    "nnb_matmul_q_i8": (_I, [_P, _P, _P, _P, _P, _SZ, _SZ, _SZ, _P, _P]),
    "nnb_matmul_q": (_I, [_P, _P, _P, _P, _SZ, _SZ, _SZ, _P]),
    "nnb_matmul_q_t": (_I, [_P, _P, _P, _P, _SZ, _SZ, _SZ, _P]),
    "nnb_actq_bytes": (_SZ, [_SZ, _SZ]),
    "nnb_act_quant_tm": (_I, [_P, _P, _I, _SZ, _SZ, _P, _P, _P]),
    "nnb_actq_to_plain": (_I, [_P, _P, _SZ, _SZ, _P]),
    "nnb_bitlinear_fwd_tm": (_I, [_P, _P, _P, _P, _P, _P, _P, _SZ, _SZ, _SZ, _P, _I, _P]),
    "nnb_bitlinear_fwd_tm_stack": (_I, [_P, _P, _SZ, _P, _P, _P, _P, _P, _SZ, _SZ, _SZ, _SZ, _P, _SZ, _I]),
    "nnb_bitlinear_dx_tm": (_I, [_P, _P, _P, _P, _SZ, _SZ, _SZ, _P, _I, _I]),
    "nnb_bitlinear_dw_tm": (_I, [_P, _P, _P, _P, _P, _SZ, _SZ, _SZ, _P, _I]),
    "nnb_expand_weights": (_I, [_P, _P, _SZ, _SZ, _P, _P]),
    "nnb_tc_set_forward_tile": (_I, [_I]),
    "nnb_bitlinear_fwd_tc": (_I, [_P, _P, _P, _P, _P, _P, _P, _SZ, _SZ, _SZ, _P]),
    "nnb_bitlinear_bwd_tc": (_I, [_P, _P, _P, _P, _P, _P, _SZ, _SZ, _SZ, _P, _P, _P, _I, _P]),
    "nnb_lmhead_logprob_entropy_fwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _SZ, _SZ, _SZ, _P, _P, _P]),
    "nnb_lmhead_logprob_entropy_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _SZ, _SZ, _SZ, _P, _P]),
    "nnb_engine_check": (_I, [_P]),
    "nnb_attention_fwd": (_I, [_P, _P, _P, _P, _SZ, _SZ, _SZ, _SZ, _I, _P, _P]),
    "nnb_attention_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _SZ, _SZ, _SZ, _SZ, _I, _P, _P, _P, _P]),
    "nnb_attention_decode": (_I, [_P, _P, _P, _P, _SZ, _P, _P, _SZ, _SZ, _SZ, _P, _P, _P, _SZ, _SZ, _SZ, _I, _P, _P, _P, _P]),
    "nnb_attention_rope_fwd": (_I, [_P, _P, _P, _P, _P, _P, _SZ, _SZ, _SZ, _SZ, _I, _P, _P]),
    "nnb_attention_rope_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _SZ, _SZ, _SZ, _SZ, _I, _P, _P, _P, _P]),
    "nnb_bitlinear_fwd_host": (_I, [_P, _P, _P, _P, _P, _SZ, _SZ, _SZ, _P]),
    "nnb_policy_create": (_I, [_P, _P, C.POINTER(_P)]),
    "nnb_policy_destroy": (None, [_P]),
    "nnb_policy_param_count": (_SZ, [_P]),
    "nnb_policy_params": (_P, [_P]),
    "nnb_policy_tensor_count": (_SZ, [_P]),
    "nnb_policy_tensor_info": (_I, [_P, _SZ, C.c_char_p, _SZ, C.POINTER(_SZ), C.POINTER(_SZ), C.POINTER(_SZ)]),
    "nnb_policy_upload_params": (_I, [_P, _P]),
    "nnb_policy_requantize": (_I, [_P]),
    "nnb_policy_save": (_I, [_P, C.c_char_p, _I]),
    "nnb_policy_load": (_I, [_P, C.c_char_p]),
    "nnb_trit_base3_bytes_per_row": (_SZ, [_SZ]),
    "nnb_trit_pack_row_base3": (None, [_P, _SZ, _P]),
    "nnb_trit_unpack_row_base3": (None, [_P, _SZ, _P]),
    "nnb_trit_latent_row_scale": (C.c_float, [_P, _SZ, C.c_float]),
    "nnb_trit_dequant_row": (None, [_P, _SZ, C.c_float, _P]),
    "nnb_policy_linear": (_I, [_P, _I, _I, C.POINTER(_P), C.POINTER(_P), C.POINTER(_SZ), C.POINTER(_SZ)]),
    "nnb_rollout": (_I, [_P, _P, _SZ, _SZ, _SZ, C.c_float, _I, C.c_uint64, C.c_uint32, _P, _P, _P]),
    "nnb_policy_logprobs": (_I, [_P, _P, _SZ, _SZ, _SZ, _P, _P, _P]),
    "nnb_policy_train_step": (_I, [_P, _P, _SZ, _SZ, _SZ, _P, _P]),
    "nnb_policy_sft_step": (_I, [_P, _P, _SZ, _SZ, _SZ, _SZ, _P, C.c_float, _P]),
    "nnb_policy_cached_activation": (_I, [_P, C.c_int, C.c_int, _P, _P, _P, _P]),
    "nnb_policy_logprobs_grouped": (_I, [_P, _P, _SZ, _SZ, _SZ, _SZ, _P, _P, _P]),
    "nnb_policy_train_step_grouped": (_I, [_P, _P, _SZ, _SZ, _SZ, _SZ, _P, _P]),
    "nnb_policy_grads": (_P, [_P]),
    "nnb_policy_zero_grad": (_I, [_P]),
    "nnb_policy_optimizer_step": (_I, [_P, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, _P]),
    "nnb_policy_release_workspaces": (_I, [_P]),
    "nnb_gae": (_I, [_P, _P, _P, _P, _P, _P, _SZ, _SZ, C.c_float, C.c_float, _P, _P]),
    "nnb_group_advantage": (_I, [_P, _P, _SZ, _P, _P, _SZ, C.c_float, _P]),
    "nnb_group_advantage_noalloc": (_I, [_P, _P, _SZ, _P, _P, _SZ, C.c_float, _P]),
    "nnb_masked_normalize": (_I, [_P, _P, _P, _SZ, C.c_float, _P]),
    "nnb_categorical_logp_entropy": (_I, [_P, _P, _P, _SZ, _SZ, _P, _P]),
    "nnb_categorical_backward": (_I, [_P, _P, _P, _P, _P, _SZ, _SZ, _P]),
    "nnb_token_objective": (_I, [_P, _P, _P, _P, _P, _P, _P, _SZ, C.c_float, C.c_float, C.c_float, C.c_float, _P, _P, _P]),
    "nnb_clipped_value": (_I, [_P, _P, _P, _P, _P, _SZ, C.c_float, C.c_float, C.c_float, _P, _P]),
    "nnb_value_regression": (_I, [_P, _P, _P, _P, _SZ, C.c_float, C.c_float, _P, _P]),
    "nnb_monte_carlo_return": (_I, [_P, _P, _P, _P, _SZ, _SZ, C.c_float, _P]),
    "nnb_clip_grad_norm": (_I, [_P, _P, _SZ, C.c_float, _P]),
    "nnb_scale_inplace": (_I, [_P, _P, _SZ, C.c_float]),
    "nnb_adamw_step": (_I, [_P, _P, _P, _P, _P, _SZ, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, _I]),
    "nnb_rollout_grouped": (_I, [_P, _P, _SZ, _SZ, _SZ, _SZ, C.c_float, _I, C.c_uint64, C.c_uint32, _P, _P, _P]),
    "nnb_rollout_sampled": (_I, [_P, _P, _SZ, _SZ, _SZ, _SZ, _P, C.c_uint32, _P, _P, _P, _P]),
    "nnb_rollout_set_step_timing": (_I, [_P, _SZ]),
    "nnb_rollout_step_times": (_I, [_P, _P, _P, _SZ, C.POINTER(_SZ)]),
    "nnb_rollout_host": (_I, [_P, _P, _SZ, _SZ, _SZ, C.c_float, _I, C.c_uint64, C.c_uint32, _P, _P]),
}


def exported_symbols() -> list[str]:
    return sorted(_SIGNATURES)


def lib() -> C.CDLL:
    """Load libnn-b200.so (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise NnbError(
                f"{path} is missing: build it with `python neuralnet.cpp_b200/build.py` "
                "(nvcc, sm_100a). This engine has no CPU fallback."
            )
        handle = C.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != 0:
        msg = lib().nnb_last_error()
        err = NnbError(f"nnb_status {status}: {msg.decode() if msg else '?'}")
        err.status = status
        raise err
