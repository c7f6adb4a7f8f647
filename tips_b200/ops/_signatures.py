"""ctypes prototypes of the kernel library (csrc/kernels/tips_kernels.h)."""
from __future__ import annotations

from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_uint64, c_void_p

P = c_void_p
I = c_int
L = c_int64
U = c_uint64
F = c_float
PP = POINTER(c_void_p)

_PROTOS = {
    "tipsk_last_error": (c_char_p, []),
    "tipsk_sgd_momentum_flat": (I, [P, P, I, P, I, P, L, F, F, F, F, I, F, I, P]),
    "tipsk_adam_flat": (I, [P, P, I, P, I, P, P, L, F, F, F, F, F, L, F, I, P]),
    "tipsk_adam_flat_devstep": (I, [P, P, I, P, I, P, P, L, F, F, F, F, F, L, P, F, I, P]),
    "tipsk_pack": (I, [PP, POINTER(L), POINTER(L), I, I, P, I, F, I, P]),
    "tipsk_unpack": (I, [P, I, PP, POINTER(L), POINTER(L), I, I, F, P]),
    "tipsk_scale_cast": (I, [P, I, P, I, L, F, P]),
    "tipsk_bn_partials": (I, [L, I]),
    "tipsk_bn_fwd_train": (I, [P, P, P, P, P, P, P, P, P, P, L, I, F, F, I, I, P]),
    "tipsk_bn_fwd_train_mask": (I, [P, P, P, P, P, P, P, P, P, P, P, P, L, I, F, F, I, I, P]),
    "tipsk_bn_bwd_bitmask": (I, [P, P, P, P, P, P, P, P, P, P, P, L, I, I, P]),
    "tipsk_bn_bwd_relu_recompute": (I, [P, P, P, P, P, P, P, P, P, P, L, I, I, P]),
    "tipsk_bn_fwd_train_stats": (I, [P, P, P, P, P, P, P, P, P, P, L, I, F, F, I, I, P]),
    "tipsk_bn_fwd_eval": (I, [P, P, P, P, P, P, P, L, I, F, I, I, P]),
    "tipsk_bn_bwd": (I, [P, P, P, P, P, P, P, P, P, P, P, L, I, I, I, P]),
    "tipsk_ln_fwd": (I, [P, P, P, P, P, P, L, I, F, I, P]),
    "tipsk_ln_fwd_residual": (I, [P, P, P, P, P, P, P, P, L, I, F, I, P]),
    "tipsk_ln_bwd": (I, [P, P, P, P, P, P, P, P, I, L, I, I, P]),
    "tipsk_ln_bwd_partials": (I, [L, I]),
    "tipsk_ln_reduce_partials": (I, [P, P, I, I, P, P, I, P]),
    "tipsk_bias_act_fwd": (I, [P, P, P, L, I, I, I, P]),
    "tipsk_bias_act_bwd": (I, [P, P, P, P, P, L, I, I, I, P]),
    "tipsk_sigmoid_bce": (I, [P, P, P, P, L, F, I, P]),
    "tipsk_embed_sum_fwd": (I, [P, P, P, P, P, L, I, I, L, I, P]),
    "tipsk_embed_sum_bwd": (I, [P, P, P, P, P, L, I, I, L, I, P]),
    "tipsk_dot_sigmoid_bce_fwd": (I, [P, P, P, P, P, P, P, L, I, L, F, I, P]),
    "tipsk_dot_sigmoid_bce_bwd": (I, [P, P, P, P, P, P, P, L, I, L, I, P]),
    "tipsk_softmax_xent": (I, [P, P, P, P, P, L, I, L, F, I, P]),
    "tipsk_comm_init": (I, [I, I, PP, P, U, U, I, I, U, I, I]),
    "tipsk_comm_shutdown": (I, []),
    "tipsk_comm_ready": (I, []),
    "tipsk_comm_staging_offset": (U, []),
    "tipsk_comm_launches": (U, []),
    "tipsk_comm_stream": (P, [I]),
    "tipsk_comm_uses_multimem": (I, []),
    "tipsk_comm_set_budget_ms": (I, [I]),
    "tipsk_comm_status": (I, [I, POINTER(c_int32), I]),
    "tipsk_comm_reset": (I, []),
    "tipsk_allreduce": (I, [PP, PP, L, U, I, I, F, F, I, P]),
    "tipsk_allgatherv": (I, [PP, PP, POINTER(U), I, P]),
    "tipsk_broadcast": (I, [PP, PP, U, I, I, P]),
    "tipsk_comm_wait_never": (I, [I, P]),
    "tipsk_comm_update_subtile": (I, []),
    "tipsk_comm_update_shard_vecs": (L, [U]),
    "tipsk_comm_attach_update": (I, [L, U, I, L, I, PP, PP, PP]),
    "tipsk_comm_detach_update": (I, [L]),
    "tipsk_comm_update_attached": (I, [L, U]),
    "tipsk_comm_set_update_hyper": (I, [L, POINTER(c_float), I, L]),
    "tipsk_comm_update_launches": (U, [L]),
    "tipsk_allreduce_update": (I, [L, F, I, P]),
    "tipsk_event_create": (P, []),
    "tipsk_event_recycle": (None, [P]),
    "tipsk_event_record": (I, [P, P]),
    "tipsk_stream_wait_event": (I, [P, P]),
    "tipsk_stream_synchronize": (I, [P]),
    "tipsk_executor_configure": (I, [I, P, U]),
    "tipsk_device_executor_ptr": (P, []),
    "tipsk_comm_fence": (I, [I, P]),
    "tipsk_table_init": (I, [P, L, I, I, I, I, L, U, F, P]),
    "tipsk_ps_place": (I, [I, L, I, POINTER(c_int32), POINTER(L)]),
    "tipsk_ps_acc_bytes": (U, [U, I]),
    "tipsk_ps_inbox_bytes": (U, [I, U, I]),
    "tipsk_ps_ctl_bytes": (U, []),
    "tipsk_ps_configure": (I, [PP, PP, PP, PP, PP, PP, PP, I, I, POINTER(c_int32), I, POINTER(U), POINTER(U), POINTER(L),
                               I, I, U, U, U, U]),
    "tipsk_ps_traffic": (I, [POINTER(U)]),
    "tipsk_ps_wire_follows_grads": (I, [I]),
    "tipsk_ps_phase_timing": (I, [I]),
    "tipsk_ps_phase_ms": (I, [POINTER(F)]),
    "tipsk_ps_pull_phase_ms": (I, [POINTER(F)]),
    "tipsk_ps_status": (I, [POINTER(c_int32), POINTER(U)]),
    "tipsk_ps_pull": (I, [PP, PP, L, L, L, I, I, I, P]),
    "tipsk_ps_push": (I, [PP, PP, L, L, L, I, F, I, F, F, I, P]),
    "tipsk_hash_pull": (I, [PP, PP, I, U, I, PP, PP, I, L, L, I, P, P]),
    "tipsk_hash_push": (I, [PP, PP, PP, I, U, I, PP, PP, I, L, L, I, F, I, F, F, P, P, P]),
    "tipsk_ps_push_async": (I, [PP, PP, L, L, L, I, F, I, F, F, P]),
    "tipsk_gemm_bf16": (I, [P, P, P, P, P, I, I, I, I, I, I, I, P]),
    "tipsk_copy4d": (I, [P, P, L, L, L, L, P, P, P]),
    "tipsk_gemm_bf16_nn": (I, [P, P, P, I, I, I, I, I, I, I, P]),
    "tipsk_gemm_supported": (I, [I, I, I, I, I]),
    "tipsk_gemm_status": (I, []),
    "tipsk_conv2d_supported": (I, [I, I, I, I, I, I]),
    "tipsk_conv2d_fwd": (I, [P, P, P, I, I, I, I, I, I, I, I, I, P, P, P]),
    "tipsk_conv2d_dgrad": (I, [P, P, P, I, I, I, I, I, I, I, I, I, I, P]),
    "tipsk_conv2d_dgrad_ohwi": (I, [P, P, P, I, I, I, I, I, I, I, I, I, I, P]),
    "tipsk_conv2d_wgrad": (I, [P, P, P, I, I, I, I, I, I, I, I, I, P]),
    "tipsk_conv_status": (I, []),
    "tipsk_stem_geometry": (I, [I, I, P, P, P, P]),
    "tipsk_stem_pad": (I, [P, P, I, I, I, P]),
    "tipsk_stem_pad_nchw_f32": (I, [P, P, I, I, I, P]),
    "tipsk_stem_conv_fwd": (I, [P, P, P, I, I, I, I, P, P, P]),
    "tipsk_stem_conv_wgrad": (I, [P, P, P, I, I, I, I, P]),
    "tipsk_global_avgpool_fwd": (I, [P, P, I, I, I, I, P]),
    "tipsk_global_avgpool_bwd": (I, [P, P, I, I, I, I, P]),
    "tipsk_maxpool3x3s2_fwd": (I, [P, P, P, I, I, I, I, I, P]),
    "tipsk_maxpool3x3s2_bwd": (I, [P, P, P, I, I, I, I, I, P]),
}


def declare(lib) -> None:
    for name, (res, args) in _PROTOS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.restype = res
        fn.argtypes = args
