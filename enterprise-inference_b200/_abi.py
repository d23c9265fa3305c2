"""ctypes binding of include/b200_decode.h.  Fails loudly when the CUDA extension is missing:
there is no CPU fallback on the product path."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("B200_LIB") or os.path.join(HERE, "lib", "libb200decode.so")   # B200_LIB: A/B builds


class B200Error(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"b200 error {code}: {text}")
        self.code = code


class ModelCfg(C.Structure):
    """struct b200_model_cfg"""
    _fields_ = [(n, C.c_int32) for n in ("hidden", "n_layers", "n_q_heads", "n_kv_heads", "head_dim",
                                         "intermediate", "vocab", "qkv_bias")] + \
               [("rms_eps", C.c_float)] + \
               [(n, C.c_int32) for n in ("block_size", "max_tokens", "max_blocks_per_seq", "tp_rank", "tp_world")]


class StackLayer(C.Structure):
    """struct b200_stack_layer"""
    _fields_ = [(n, C.c_int32) for n in ("mixer", "heads", "kv_heads", "dim", "vdim", "rot_dims", "rot_table", "vrot_table")] + \
               [("scale", C.c_float)] + [(n, C.c_int32) for n in ("mlp", "experts", "top", "groups", "keep", "ff")] + \
               [(n, C.c_int32) for n in ("kv_rank", "rot_dim", "mixer_flags")] + [("gate_cap", C.c_float)] + \
               [(n, C.c_int32) for n in ("act", "ungated", "sigmoid_scores", "weight_input", "shared_ff")] + \
               [(n, C.c_int32) for n in ("window", "q_rank", "kv_share", "conv_taps", "decay_rank", "gate_rank", "norm_groups")] + \
               [("act_limit", C.c_float), ("route_chosen", C.c_int32)]


class StackCfg(C.Structure):
    """struct b200_stack_cfg"""
    _fields_ = [(n, C.c_int32) for n in ("width", "vocab", "n_layers")] + [("embed_scale", C.c_float), ("norm_eps", C.c_float)] + \
               [(n, C.c_int32) for n in ("f32", "block_size", "max_tokens", "max_blocks_per_seq", "max_logit_rows")] + \
               [(n, C.c_int32) for n in ("form", "canon_taps", "depth_avg", "bigram_buckets", "bigram_mul_prev", "bigram_mul_cur")] + \
               [("logit_softcap", C.c_float), ("n_state_slots", C.c_int32), ("residual_alpha", C.c_float), ("streams", C.c_int32),
                ("residual_mult", C.c_float)]


MIXER_ATTENTION, MIXER_LATENT, MIXER_MLSTM, MIXER_DELTA, MIXER_SSD = 1, 2, 3, 4, 5
MLP_NONE, MLP_MOE, MLP_DENSE = 0, 1, 2
ACT_SILU, ACT_GELU_TANH, ACT_RELU2, ACT_RELU, ACT_SWIGLU_CLAMP, ACT_POLYNORM = 0, 1, 2, 3, 4, 5
ACTS = {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH, "relu2": ACT_RELU2, "relu": ACT_RELU, "swiglu_clamp": ACT_SWIGLU_CLAMP,
        "polynorm": ACT_POLYNORM}
FORM_SANDWICH, FORM_PARALLEL, FORM_POSTNORM, FORM_HYPER = 0, 1, 2, 3
MIXF_SINK, MIXF_GATE, MIXF_HEAD_NORM, MIXF_VALUE_IS_KEY, MIXF_SINK_ONE, MIXF_HEAD_GATE = 1, 2, 4, 8, 16, 32
MIXF_ROT_HALF, MIXF_NO_QK_NORM, MIXF_HEAD_DECAY = 64, 128, 256
MAX_STREAMS = 8
(SW_EMBED, SW_FINAL_NORM, SW_HEAD, SW_NORM_MIX_PRE, SW_NORM_MIX_POST, SW_NORM_MLP_PRE, SW_NORM_MLP_POST, SW_QKV, SW_Q_NORM,
 SW_K_NORM, SW_O, SW_ROUTER, SW_ROUTER_BIAS, SW_EXPERT_GATE_UP, SW_EXPERT_DOWN, SW_BIGRAM, SW_CANON, SW_DEPTH_AVG, SW_UK_T, SW_UV,
 SW_SINK, SW_GATES, SW_GATES_BIAS, SW_HEAD_NORM, SW_MLP_GATE_UP, SW_MLP_DOWN, SW_SHARED_UP, SW_SHARED_DOWN, SW_NORM_MIX_POST_BIAS,
 SW_NORM_MLP_POST_BIAS, SW_FINAL_NORM_BIAS, SW_Q_LATENT_NORM, SW_UQ, SW_CONV, SW_DECAY_UP, SW_DECAY_BIAS, SW_DECAY_LOG,
 SW_GATE_UP, SW_MLP_GATE_UP_INTERLEAVED, SW_NORM_MIX_PRE_BIAS, SW_NORM_MLP_PRE_BIAS, SW_SCALE_MIX, SW_SCALE_MLP, SW_HC_MIX, SW_HC_MLP,
 SW_CANON_MLP, SW_CONV_BIAS, SW_SKIP, SW_MLP_ACT) = range(49)
SW_F32 = {SW_FINAL_NORM, SW_NORM_MIX_PRE, SW_NORM_MIX_POST, SW_NORM_MLP_PRE, SW_NORM_MLP_POST, SW_Q_NORM, SW_K_NORM, SW_ROUTER_BIAS,
          SW_CANON, SW_DEPTH_AVG, SW_SINK, SW_GATES_BIAS, SW_HEAD_NORM, SW_NORM_MIX_POST_BIAS, SW_NORM_MLP_POST_BIAS,
          SW_FINAL_NORM_BIAS, SW_Q_LATENT_NORM, SW_CONV, SW_DECAY_BIAS, SW_DECAY_LOG, SW_NORM_MIX_PRE_BIAS, SW_NORM_MLP_PRE_BIAS,
          SW_SCALE_MIX, SW_SCALE_MLP, SW_HC_MIX, SW_HC_MLP, SW_CANON_MLP, SW_CONV_BIAS, SW_SKIP, SW_MLP_ACT}

W_EMBED, W_LN1, W_QKV, W_QKV_BIAS, W_O, W_LN2, W_GATE_UP, W_DOWN, W_FINAL_NORM, W_LM_HEAD, W_GATE_UP_INTERLEAVED = range(11)

_vp, _i32, _i64, _f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float

# name -> (restype, argtypes); every symbol declared in include/b200_decode.h
SIGNATURES = {
    "b200_last_error": (C.c_char_p, []),
    "b200_abi_version": (C.c_int, []),
    "b200_device_ok": (C.c_int, []),
    "b200_ctx_create": (C.c_int, [C.POINTER(ModelCfg), C.POINTER(_vp)]),
    "b200_ctx_destroy": (C.c_int, [_vp]),
    "b200_ctx_workspace_bytes": (_i64, [_vp]),
    "b200_set_weight": (C.c_int, [_vp, _i32, _i32, _vp, _i64, _i64]),
    "b200_set_kv_cache": (C.c_int, [_vp, _vp, _vp, _i64]),
    "b200_set_rope_cache": (C.c_int, [_vp, _vp, _i64]),
    "b200_nccl_unique_id": (C.c_int, [_vp]),
    "b200_nccl_init": (C.c_int, [_vp, _vp]),
    "b200_tp_ipc_export": (C.c_int, [_vp, _vp]),
    "b200_tp_ipc_import": (C.c_int, [_vp, _vp, _i32]),
    "b200_decode_step": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _i32, _i32, _vp, _i32, _vp, _vp, _vp]),
    "b200_decode_step_host": (C.c_int, [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "b200_set_launch_pdl": (C.c_int, [_i32]),
    "b200_ctx_set_graphs": (C.c_int, [_vp, _i32]),
    "b200_ctx_last_step_launches": (C.c_int, [_vp]),
    "b200_ctx_set_tap": (C.c_int, [_vp, _i32, _vp, _vp]),
    "b200_linear_workspace_bytes": (_i64, [_i32, _i32, _i32]),
    "b200_linear_bf16": (C.c_int, [_vp, _i64, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp, _i64, _vp]),
    "b200_linear_fused_bf16": (C.c_int, [_vp, _i64, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp,
                                         _i32, _i32, _i32, _vp, _i64, _vp]),
    "b200_embed_stream": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "b200_linear_residual_bf16": (C.c_int, [_vp, _i64, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _i64, _vp]),
    "b200_linear_normed_bf16": (C.c_int, [_vp, _vp, _vp, _f32, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp, _vp, _vp,
                                          _vp, _vp, _i32, _i32, _i32, _vp, _i64, _vp]),
    "b200_rmsnorm_stream": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _f32, _vp]),
    "b200_rmsnorm": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _i32, _f32, _vp]),
    "b200_embed": (C.c_int, [_vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "b200_rope_kv_append": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "b200_paged_attn_workspace_bytes": (_i64, [_i32, _i32, _i32, _i32]),
    "b200_paged_attn_decode": (C.c_int, [_vp, _i64, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _i64, _i32, _i32, _i32,
                                         _i32, _i32, _f32, _vp, _i64, _vp]),
    "b200_paged_attn_prefill": (C.c_int, [_vp, _i64, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _i64, _i32, _i32, _i32,
                                          _i32, _i32, _f32, _vp, _i64, _vp]),
    "b200_paged_attn_static_scratch_bytes": (_i64, []),
    "b200_paged_attn_decode_static": (C.c_int, [_vp, _i64, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _i64, _i32, _i32, _i32,
                                                _i32, _i32, _f32, _vp]),
    "b200_silu_mul": (C.c_int, [_vp, _vp, _i32, _i32, _vp]),
    "b200_argmax": (C.c_int, [_vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp]),
    "b200_sample": (C.c_int, [_vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_ctx_sample_last": (C.c_int, [_vp, _i32, _vp, _vp, _vp]),
    "b200_logit_adjust": (C.c_int, [_vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_ctx_adjust_last": (C.c_int, [_vp, _i32, _vp, _i32, _vp]),
    "b200_logprobs": (C.c_int, [_vp, _i64, _i32, _i32, _vp, _i32, _vp, _vp, _vp, _vp]),
    "b200_ctx_logprobs_last": (C.c_int, [_vp, _i32, _vp, _i32, _vp, _vp]),
    "b200_advance_decode_rows": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _i32, _i32, _vp]),
    "b200_allreduce_bf16": (C.c_int, [_vp, _vp, _i64, _vp]),
    "b200_tp_allreduce": (C.c_int, [_vp, _i32, _vp, _i32, _vp, _vp, _vp, _vp]),
    "b200_stack_create": (C.c_int, [C.POINTER(StackCfg), C.POINTER(StackLayer), C.POINTER(_vp)]),
    "b200_stack_set_weight": (C.c_int, [_vp, _i32, _i32, _vp, _i64, _i64]),
    "b200_stack_set_kv_cache": (C.c_int, [_vp, _i32, _vp, _vp, _i64]),
    "b200_stack_cache_dims": (C.c_int, [_vp, _i32, _vp, _vp]),
    "b200_stack_set_rot_table": (C.c_int, [_vp, _i32, _vp, _i64, _i32]),
    "b200_stack_set_stream_tap": (C.c_int, [_vp, _vp]),
    "b200_stack_state_bytes": (_i64, [_vp]),
    "b200_stack_set_state": (C.c_int, [_vp, _vp]),
    "b200_stack_set_step_slots": (C.c_int, [_vp, _vp, _i32]),
    "b200_ctx_logits_last_f32": (C.c_int, [_vp, _i32, _vp, _vp]),
    "b200_layernorm_stream": (C.c_int, [_i32, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _f32, _vp]),
    "b200_qk_norm_rotate_cache": (C.c_int, [_i32, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32,
                                            _i32, _i32, _f32, _i64, _vp]),
    "b200_qk_norm_rotate_cache_wide": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32,
                                                 _f32, _i64, _i32, _i32, _vp]),
    "b200_rotate_back_rows": (C.c_int, [_vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i64, _vp]),
    "b200_paged_attn_anydim_workspace_bytes": (_i64, [_i32]),
    "b200_paged_attn_anydim": (C.c_int, [_i32, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i64, _vp, _i32, _i32, _i32, _i32, _i32,
                                         _i32, _f32, _i32, _vp, _vp]),
    "b200_moe_route": (C.c_int, [_i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp]),
    "b200_moe_route_linear": (C.c_int, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "b200_moe_workspace_bytes": (_i64, [_i32, _i32, _i32, _i32, _i32]),
    "b200_moe_experts": (C.c_int, [_i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp]),
    "b200_linear_simt": (C.c_int, [_i32, _i32, _vp, _i64, _vp, _vp, _i64, _i32, _i32, _i32, _vp]),
    "b200_seq_bounds": (C.c_int, [_vp, _i32, _i32, _vp, _vp]),
    "b200_embed_bigram": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _f32, _vp, _vp, _vp, _vp, _i32, _vp, _i64, _i32, _i32, _i32, _vp]),
    "b200_parallel_close": (C.c_int, [_i32, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _i64, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32,
                                      _f32, _vp]),
    "b200_canon_conv": (C.c_int, [_i32, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i64, _vp]),
    "b200_latent_prep": (C.c_int, [_i32, _vp, _i64, _vp, _vp, _vp, _vp, _i32, _i64, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _f32, _vp]),
    "b200_head_linear": (C.c_int, [_i32, _i32, _vp, _i64, _i32, _vp, _vp, _i64, _i32, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200_paged_attn_anydim_ex": (C.c_int, [_i32, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _f32,
                                            _i32, _vp, _i32, _i32, _vp, _vp]),
    "b200_latent_attn_supported": (C.c_int, [_i32, _i32, _i32]),
    "b200_latent_attn": (C.c_int, [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _f32, _vp, _vp, _i32, _vp, _vp]),
    "b200_mlstm_gates": (C.c_int, [_i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _f32, _vp]),
    "b200_mlstm_state_floats": (_i64, [_i32, _i32, _i32]),
    "b200_mlstm_scan": (C.c_int, [_i32, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i32, _i32, _i32, _i32, _vp]),
    "b200_head_norm_gate": (C.c_int, [_i32, _vp, _vp, _vp, _i64, _vp, _i32, _i32, _i32, _f32, _vp]),
    "b200_ff_act": (C.c_int, [_i32, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "b200_moe_route_scores": (C.c_int, [_i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp]),
    "b200_delta_fused_rows": (_i32, [_i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200_postnorm_stream": (C.c_int, [_i32, _vp, _vp, _f32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _f32, _vp]),
    "b200_qk_headnorm_rotate_cache": (C.c_int, [_i32, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _vp, _vp, _vp, _i32, _i32, _i32, _i32,
                                                _i32, _i32, _f32, _vp]),
    "b200_paged_attn_window": (C.c_int, [_i32, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _f32,
                                         _i32, _vp, _i32, _i32, _vp, _i32, _vp]),
    "b200_latent_attn_window": (C.c_int, [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _f32, _vp, _vp, _i32, _vp]),
    "b200_paged_attn_mma_supported": (C.c_int, [_i32, _i32, _i32, _i32]),
    "b200_paged_attn_mma": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _vp, _vp, _i32, _i32,
                                      _vp, _vp]),
    "b200_latent_norms": (C.c_int, [_i32, _vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _f32, _vp]),
    "b200_head_linear_head_gate": (C.c_int, [_i32, _vp, _i64, _i32, _vp, _vp, _i64, _i32, _vp, _i64, _i32, _i32, _i32, _i32, _vp]),
    "b200_delta_prep": (C.c_int, [_i32, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i32, _i32,
                                  _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200_delta_tails": (C.c_int, [_i32, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _vp]),
    "b200_delta_scan": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200_moe_experts_form": (C.c_int, [_i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _vp]),
    "b200_hyper_step": (C.c_int, [_i32, _vp, _i64, _i32, _i32, _vp, _vp, _i32, _vp, _vp, _f32, _vp, _vp, _vp, _f32, _vp, _vp, _vp, _vp, _i32,
                                  _i32, _vp]),
    "b200_qkv_rotate_cache": (C.c_int, [_i32, _vp, _i64, _vp, _vp, _vp, _i32, _i32, _i64, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200_polynorm": (C.c_int, [_i32, _vp, _vp, _vp, _i32, _i32, _f32, _vp]),
    "b200_ff_act_limit": (C.c_int, [_i32, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _vp]),
    "b200_moe_route_chosen": (C.c_int, [_i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp]),
    "b200_moe_experts_limit": (C.c_int, [_i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _i32, _i32, _f32, _vp]),
    "b200_delta_prep_head": (C.c_int, [_i32, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32,
                                       _i32, _i32, _i32, _vp]),
    "b200_linear_scan": (C.c_int, [_i32, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _i64, _vp, _i32, _i32, _i32, _i32, _i32,
                                   _vp]),
    "b200_head_norm_gate_act": (C.c_int, [_i32, _vp, _vp, _vp, _i64, _vp, _i32, _i32, _i32, _f32, _i32, _vp]),
    "b200_ssd_prep": (C.c_int, [_i32, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32,
                                _i32, _i32, _i32, _vp]),
    "b200_ssd_gate_norm": (C.c_int, [_i32, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _vp]),
}

_lib = None


def lib() -> C.CDLL:
    """Load libb200decode.so (built in-tree by build.py).  No fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python enterprise-inference_b200/build.py` "
                              "(nvcc, sm_100a). There is no CPU fallback.")
        _lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype, fn.argtypes = res, args
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise B200Error(rc, lib().b200_last_error().decode(errors="replace"))


def ptr(t) -> int:
    """Device (or pinned host) address of a torch tensor, None -> NULL."""
    return None if t is None else t.data_ptr()
