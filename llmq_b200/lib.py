"""ctypes binding of libb200q.so — the only way Python reaches the CUDA code.

The library is built in-tree (``llmq_b200/libb200q.so``) by ``__graft_entry__.build()`` /
``make -C llmq_b200/csrc``.  There is NO fallback: if the shared object is missing, or no
sm_100 device is present when a compute entry point is used, the call raises.

PyTorch tensors are used purely as device buffers: every wrapper passes ``tensor.data_ptr()``
and sizes across the C ABI declared in ``include/b200q.h``.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200q.so")


class B200QError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"libb200q error {code}: {msg}")
        self.code = code


class ModelConfig(C.Structure):
    _fields_ = [
        ("hidden", C.c_int32),
        ("n_layers", C.c_int32),
        ("n_q_heads", C.c_int32),
        ("n_kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("intermediate", C.c_int32),
        ("vocab", C.c_int32),
        ("block_size", C.c_int32),
        ("max_tokens", C.c_int32),
        ("max_seqs", C.c_int32),
        ("max_pos", C.c_int32),
        ("tie_embeddings", C.c_int32),
        ("rms_eps", C.c_float),
        ("attn_scale", C.c_float),
        # architecture extras (all zero = Llama)
        ("arch", C.c_int32),
        ("sliding_window", C.c_int32),
        ("attn_softcap", C.c_float),
        ("final_softcap", C.c_float),
        ("embed_scale", C.c_float),
        # layered architectures
        ("dtype", C.c_int32),
        ("max_logit_rows", C.c_int32),
        ("state_slots", C.c_int32),
        # form of a layer (layered architectures)
        ("layer_form", C.c_int32),
        ("norm_groups", C.c_int32),
        ("residual_alpha", C.c_float),
        ("input_taps", C.c_int32),
        ("learned_pos", C.c_int32),
        ("token_shift", C.c_int32),
        ("logit_softcap", C.c_float),
        # sandwich form
        ("norm_kind", C.c_int32),
        ("residual_mult", C.c_float),
        ("side_dim", C.c_int32),
        ("logit_scale", C.c_float),
    ]


ARCH_LLAMA = 0
ARCH_GEMMA2 = 1
ARCH_RAMOPEL = 2
ARCH_NORIDRA = 3
ARCH_PALUZEN = 4
ARCH_KABAVIK = 5
FORM_PARALLEL = 0
FORM_POSTNORM = 1
FORM_PRENORM = 2
FORM_SANDWICH = 3
NORM_RMS = 0
NORM_DYT = 1
NORM_CAST = 2
NORM_NONE = 3
DTYPE_BF16 = 0
DTYPE_F32 = 1
MIXER_LATENT_ATTN = 1
MIXER_GENERAL_DELTA = 2
MIXER_GATED_DELTA = 3
MIXER_CHUNK_ATTN = 4
MIXER_SELECTIVE_SCAN = 5
MIXER_LIGHTNING = 6
MIXER_WINDOW_ATTN = 7
MIXER_DECAY_MIX = 8
FF_NONE = 0
FF_POLYNORM = 1
FF_MOE = 2
FF_MOE_SIGMOID = 3
FF_RELU2 = 4
FF_MOE_GROUPED = 5
FF_GEGLU = 6


class LayerDesc(C.Structure):
    _fields_ = [
        ("mixer", C.c_int32), ("heads", C.c_int32), ("dim", C.c_int32), ("rot_dim", C.c_int32),
        ("vdim", C.c_int32), ("q_rank", C.c_int32), ("kv_rank", C.c_int32), ("kv_from", C.c_int32),
        ("window", C.c_int32), ("rot_dims", C.c_int32), ("rot_base", C.c_double), ("attn_scale", C.c_float),
        ("decay_rank", C.c_int32), ("ff", C.c_int32), ("ff_dim", C.c_int32), ("n_experts", C.c_int32),
        ("top_k", C.c_int32), ("expert_limit", C.c_float), ("shared_dim", C.c_int32), ("shared_limit", C.c_float),
        ("kv_heads", C.c_int32), ("conv_taps", C.c_int32), ("softcap", C.c_float), ("chunk", C.c_int32),
        ("inner", C.c_int32), ("state_dim", C.c_int32), ("dt_rank", C.c_int32),
        ("inject", C.c_int32), ("mix_scale", C.c_float), ("n_identity", C.c_int32), ("n_groups", C.c_int32),
        ("keep_groups", C.c_int32), ("side_mixer", C.c_int32), ("side_heads", C.c_int32), ("side_dim", C.c_int32),
        ("side_vdim", C.c_int32), ("side_decay_rank", C.c_int32), ("side_scale", C.c_float),
        ("keep_first", C.c_int32), ("qk_norm", C.c_int32), ("proj_bias", C.c_int32), ("bare", C.c_int32),
        ("head_gate", C.c_int32), ("q_temp_coef", C.c_float), ("q_temp_every", C.c_int32),
        ("rot_factor", C.c_double), ("rot_original", C.c_double), ("rot_fast", C.c_double), ("rot_slow", C.c_double),
    ]


class Batch(C.Structure):
    _fields_ = [
        ("T", C.c_int32),
        ("n_dec", C.c_int32),
        ("n_tiles", C.c_int32),
        ("n_sample", C.c_int32),
        ("bt_stride", C.c_int32),
        ("token_ids", C.c_void_p),
        ("positions", C.c_void_p),
        ("slot_mapping", C.c_void_p),
        ("block_table", C.c_void_p),
        ("ctx_lens", C.c_void_p),
        ("tiles", C.c_void_p),
        ("sample_rows", C.c_void_p),
        ("out_ids", C.c_void_p),
        ("sample_params", C.c_void_p),
        ("sum_ctx_dec", C.c_int64),
        ("prefill_flops_per_layer", C.c_int64),
        ("prev_out_ids", C.c_void_p),
        ("n_rows", C.c_int32),
        ("seq_desc", C.c_void_p),
        ("row_seq", C.c_void_p),
        ("no_sampling", C.c_int32),
    ]


class EngineConfig(C.Structure):
    _fields_ = [
        ("max_num_seqs", C.c_int32),
        ("max_num_batched_tokens", C.c_int32),
        ("max_model_len", C.c_int32),
        ("eos_token_id", C.c_int32),
        ("policy", C.c_int32),
    ]


class EngineStats(C.Structure):
    _fields_ = [
        ("steps", C.c_int64),
        ("tokens_prefilled", C.c_int64),
        ("tokens_decoded", C.c_int64),
        ("preemptions", C.c_int64),
        ("running", C.c_int32),
        ("waiting", C.c_int32),
        ("free_blocks", C.c_int32),
        ("total_blocks", C.c_int32),
        ("last_step_tokens", C.c_int32),
        ("last_step_seqs", C.c_int32),
        ("h2d_bytes", C.c_int64),
        ("d2h_bytes", C.c_int64),
    ]


class Profile(C.Structure):
    _fields_ = [("ms", C.c_double * 4), ("work", C.c_double * 4), ("launches", C.c_int64 * 4)]


PROF_NAMES = ("gemm", "decode_attn", "prefill_attn", "elementwise")


FLAG_FINISHED_EOS = 1
FLAG_FINISHED_LENGTH = 2
FLAG_FINISHED_ABORT = 4

_vp, _i, _f, _i64, _ll = C.c_void_p, C.c_int, C.c_float, C.c_int64, C.c_longlong

# name -> (restype, argtypes); must list every symbol include/b200q.h declares
SIGNATURES = {
    "b200q_version": (_i, []),
    "b200q_last_error": (C.c_char_p, []),
    "b200q_device_check": (_i, []),
    "b200q_launch_count": (_i64, []),
    "b200q_embed": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "b200q_embed_ex": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _vp]),
    "b200q_rmsnorm": (_i, [_vp, _vp, _vp, _i, _i, _f, _vp]),
    "b200q_add_rmsnorm": (_i, [_vp, _vp, _vp, _i, _i, _f, _vp]),
    "b200q_rope_kvwrite": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "b200q_decode_attn": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _f, _vp]),
    "b200q_prefill_attn": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _f, _vp]),
    "b200q_gemm_bf16": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "b200q_gemm_swiglu_bf16": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "b200q_gemm_bf16_splitk": (_i, [_vp, _vp, _i, _i, _i, _vp, C.POINTER(_vp), C.POINTER(_i)]),
    "b200q_add_rmsnorm_splitk": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp]),
    "b200q_rope_kvwrite_splitk": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "b200q_swiglu": (_i, [_vp, _vp, _i, _i, _vp]),
    "b200q_gather_rows": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "b200q_argmax_bf16": (_i, [_vp, _vp, _i, _i, _vp]),
    "b200q_sample_bf16": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "b200q_embed_scaled": (_i, [_vp, _vp, _vp, _i, _i, _f, _vp]),
    "b200q_gemma_rmsnorm": (_i, [_vp, _vp, _vp, _i, _i, _f, _vp]),
    "b200q_gemma_norm_add_norm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _vp]),
    "b200q_decode_attn_ex": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _f, _f, _i, _vp]),
    "b200q_prefill_attn_ex": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _f, _f, _i, _vp]),
    "b200q_gemm_geglu_bf16": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "b200q_softcap_bf16": (_i, [_vp, _i64, _f, _vp]),
    # layered architectures
    "b200q_embed_f32": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp]),
    "b200q_centered_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp]),
    "b200q_linear": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "b200q_linear_batched": (_i, [_vp, _i, _ll, _vp, _ll, _vp, _i, _ll, _i, _i, _i, _i, _i, _i, _vp]),
    "b200q_linear_grouped": (_i, [_vp, _i, _vp, _vp, _ll, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp]),
    "b200q_gemm_grouped_bf16": (_i, [_vp, _ll, _ll, _i, _vp, _i, _vp, _ll, _i, _i, _i, _i, _vp, _vp, _i, _i, _vp]),
    "b200q_gemm_grouped_ok": (_i, [_vp, _ll, _i, _vp, _vp, _ll, _i, _i, _i, _i]),
    "b200q_latent_prep": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp]),
    "b200q_rope_pairs_q": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "b200q_latent_attn": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _i, _vp]),
    "b200q_delta_rule": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _ll, _vp, _i, _i, _i, _i, _f, _vp, _i, _vp, _i, _vp]),
    "b200q_polynorm": (_i, [_vp, _vp, _vp, _i, _i, _f, _i, _vp]),
    "b200q_clamped_glu": (_i, [_vp, _vp, _i64, _i, _f, _i, _vp]),
    "b200q_moe_route": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200q_moe_route_ex": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200q_embed_pos_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "b200q_group_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _f, _vp, _i, _f, _vp, _vp, _i, _i, _i, _vp]),
    "b200q_causal_conv": (_i, [_vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _vp, _ll, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp]),
    "b200q_gated_delta": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _ll, _vp, _i, _i, _i, _i, _i, _f, _vp, _i, _i,
                               _vp]),
    "b200q_chunk_attn_prep": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _f, _i, _vp]),
    "b200q_chunk_attn": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _vp, _vp, _i, _f, _vp, _i,
                              _vp]),
    "b200q_chunk_attn_seq": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _vp, _vp, _i, _f,
                                  _vp, _i, _vp]),
    "b200q_selective_scan": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp, _i, _vp, _vp, _vp, _ll, _vp, _i, _i, _i, _vp, _i, _i,
                                  _vp]),
    "b200q_scatter_scaled_rows": (_i, [_vp, _vp, _vp, _i, _vp, _i, _i, _i, _vp]),
    "b200q_silu_glu": (_i, [_vp, _vp, _i64, _i, _i, _vp]),
    "b200q_layer_sum": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _vp]),
    "b200q_argmax_f32": (_i, [_vp, _vp, _i, _i, _vp]),
    # pre-norm layers, token shift, mixers 6-8
    "b200q_rmsnorm_shift": (_i, [_vp, _vp, _vp, _vp, _vp, _ll, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _f, _i, _vp]),
    "b200q_store_carry": (_i, [_vp, _i, _vp, _ll, _vp, _i, _i, _i, _vp]),
    "b200q_shift_blend": (_i, [_vp, _vp, _i, _vp, _ll, _vp, _vp, _i, _vp, _i, _i, _i, _vp]),
    "b200q_residual_add_rmsnorm": (_i, [_vp, _vp, _f, _vp, _f, _vp, _vp, _i, _i, _f, _i, _vp]),
    "b200q_relu2": (_i, [_vp, _i64, _i, _vp]),
    "b200q_tanh_cast": (_i, [_vp, _vp, _i64, _i, _vp]),
    "b200q_act_to_f32": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _i, _vp]),
    "b200q_decay_from_logits": (_i, [_vp, _i, _vp, _i, _i, _i, _vp]),
    "b200q_decay_attn": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _ll, _vp, _i, _i, _i, _i, _vp, _vp]),
    "b200q_gated_rmsnorm": (_i, [_vp, _i, _i, _vp, _vp, _i, _i, _f, _vp, _i, _i, _vp]),
    "b200q_window_attn_prep": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _i, _vp]),
    "b200q_window_attn": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _i, _vp, _i, _vp]),
    "b200q_moe_route_grouped": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200q_residual_add": (_i, [_vp, _vp, _f, _vp, _f, _i, _i, _i, _vp]),
    "b200q_residual_add_routed": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _i, _i, _i, _vp]),
    "b200q_concat_cast": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "b200q_softcap_f32": (_i, [_vp, _i64, _f, _vp]),
    "b200q_f32_to_bf16": (_i, [_vp, _vp, _i64, _vp]),
    "b200q_copy_f32": (_i, [_vp, _vp, _i64, _vp]),
    # sandwich layers, options of window / latent attention
    "b200q_rot_frequencies": (_i, [_i, C.c_double, C.c_double, C.c_double, C.c_double, C.c_double, _vp, _vp]),
    "b200q_row_norm": (_i, [_vp, _vp, _i, _vp, _vp, _i, _i, _f, _i, _vp]),
    "b200q_sandwich_add": (_i, [_vp, _vp, _vp, _i, _vp, _f, _i, _vp, _vp, _i, _i, _f, _i, _vp]),
    "b200q_scale_f32": (_i, [_vp, _i64, _f, _vp]),
    "b200q_gelu_glu": (_i, [_vp, _vp, _i64, _i, _i, _vp]),
    "b200q_gelu_glu_ex": (_i, [_vp, _vp, _i64, _i, _i, _i, _vp]),
    "b200q_token_side_gate": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _vp, _i, _i, _i, _vp]),
    "b200q_window_attn_prep_ex": (_i, [_vp, _i, _i, _i, _i, _vp, _i, _i, _i, _i, _i, _vp, _vp, _f, _i, _vp, _f, _vp, _vp,
                                       _vp, _f, _f, _i, _vp, _vp, _i, _i, _vp]),
    "b200q_window_attn_ex": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _i, _vp,
                                  _i, _vp]),
    "b200q_latent_prep_ex": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp]),
    "b200q_rope_pairs_q_ex": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _f, _vp, _vp, _i, _i, _i, _vp]),
    "b200q_latent_attn_ex": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _i, _vp, _i, _vp]),
    "b200q_model_create_layered": (_i, [C.POINTER(ModelConfig), C.POINTER(LayerDesc), C.POINTER(_vp)]),
    "b200q_model_kv_block_bytes": (_i64, [_vp]),
    "b200q_model_state_slot_bytes": (_i64, [_vp]),
    "b200q_model_bind_state": (_i, [_vp, _vp, _i64]),
    "b200q_model_logits_f32_ptr": (_vp, [_vp]),
    "b200q_model_set_layer_tap": (_i, [_vp, _vp]),
    "b200q_model_workspace_bytes_of": (_i64, [_vp]),
    "b200q_engine_step_replay": (_i, [_vp, C.c_int32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200q_model_create": (_i, [C.POINTER(ModelConfig), C.POINTER(_vp)]),
    "b200q_model_destroy": (_i, [_vp]),
    "b200q_model_bind_weight": (_i, [_vp, C.c_char_p, _vp, _i64, _i64]),
    "b200q_model_bind_kv": (_i, [_vp, _vp, _i64]),
    "b200q_model_bind_rope": (_i, [_vp, _vp]),
    "b200q_model_workspace_bytes": (_i64, [C.POINTER(ModelConfig)]),
    "b200q_model_bind_workspace": (_i, [_vp, _vp, _i64]),
    "b200q_model_forward": (_i, [_vp, C.POINTER(Batch), _vp]),
    "b200q_model_logits_ptr": (_vp, [_vp]),
    "b200q_model_set_profiling": (_i, [_vp, _i]),
    "b200q_model_profile_collect": (_i, [_vp, C.POINTER(Profile), _i]),
    "b200q_engine_stream": (_vp, [_vp]),
    "b200q_engine_create": (_i, [_vp, C.POINTER(EngineConfig), C.POINTER(_vp)]),
    "b200q_engine_create_dryrun": (_i, [C.POINTER(EngineConfig), C.c_int32, C.c_int32, C.c_int32, C.POINTER(_vp)]),
    "b200q_engine_destroy": (_i, [_vp]),
    "b200q_engine_add_request": (_i, [_vp, _i64, _vp, C.c_int32, C.c_int32, C.c_int32]),
    "b200q_engine_add_request_sampled": (_i, [_vp, _i64, _vp, C.c_int32, C.c_int32, C.c_int32, C.c_float, C.c_uint64]),
    "b200q_engine_set_stop_ids": (_i, [_vp, _vp, C.c_int32]),
    "b200q_engine_abort": (_i, [_vp, _i64]),
    "b200q_engine_set_async": (_i, [_vp, C.c_int32]),
    "b200q_engine_has_work": (_i, [_vp]),
    "b200q_engine_step": (_i, [_vp, _vp, _vp, _vp, C.c_int32, C.POINTER(C.c_int32)]),
    "b200q_engine_get_stats": (_i, [_vp, C.POINTER(EngineStats)]),
}
# test / tuning hooks that are not part of the reference-facing header
EXTRA_SIGNATURES = {
    "b200q_gemm_set_tile_n": (_i, [_i]),
    "b200q_gemm_set_mode": (_i, [_i]),
    "b200q_gemm_resident_pairs": (_i, []),
    "b200q_gemm_set_debug": (_i, [_i]),
    "b200q_decode_attn_set_variant": (_i, [_i]),
    "b200q_gemm_set_splitk": (_i, [_i]),
    "b200q_stream_probe": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp]),
}

_lib: Optional[C.CDLL] = None


def load() -> C.CDLL:
    """Load libb200q.so (once).  Raises if it has not been built — there is no CPU path."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python -c 'import __graft_entry__ as g; "
            "g.build()'` or `make -C llmq_b200/csrc`. llmq_b200 has no CPU fallback."
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in {**SIGNATURES, **EXTRA_SIGNATURES}.items():
        fn = getattr(lib, name)  # AttributeError if the .so does not export it
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def ensure_built() -> None:
    """Build libb200q.so in-tree if it is missing or older than its sources (a fresh checkout holds no
    built files).  One builder at a time: concurrent callers wait on a lock file beside the sources."""
    import fcntl
    import subprocess

    csrc = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
    inc = os.path.join(os.path.dirname(csrc), os.pardir, "include", "b200q.h")
    srcs = [os.path.join(csrc, f) for f in os.listdir(csrc) if f.endswith((".cu", ".cuh")) or f == "Makefile"] + [inc]

    def fresh() -> bool:
        return os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= max(os.path.getmtime(f) for f in srcs)

    if fresh():
        return
    with open(os.path.join(csrc, ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not fresh():
            env = dict(os.environ)
            env["PATH"] = env.get("PATH", "") + os.pathsep + "/usr/local/cuda/bin"
            r = subprocess.run(["make", "-C", csrc, f"-j{min(os.cpu_count() or 4, 16)}"], env=env,
                               stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if r.returncode != 0:
                raise ImportError(f"building {LIB_PATH} failed:\n{r.stdout[-4000:]}")


def check(rc: int) -> None:
    if rc != 0:
        msg = load().b200q_last_error()
        raise B200QError(rc, msg.decode("utf-8", "replace") if msg else "?")


def require_device() -> None:
    check(load().b200q_device_check())


def launch_count() -> int:
    return int(load().b200q_launch_count())


def _p(t) -> int:
    """data_ptr of a CUDA tensor (contiguity is the caller's contract)."""
    if t is None:
        return 0
    assert t.is_cuda and t.is_contiguous(), "libb200q wants contiguous CUDA tensors"
    return t.data_ptr()


def _stream(stream=None) -> int:
    import torch

    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


# ---- thin op wrappers (used by tests/bench; the worker goes through Engine) ------------------
def embed(ids, table, out, stream=None):
    check(load().b200q_embed(_p(ids), _p(table), _p(out), ids.numel(), table.shape[1], _stream(stream)))


def embed_ex(ids, prev_out, table, out, scale=0.0, stream=None):
    """ids < 0 are read through prev_out[-1 - id] (the previous step's sampled ids)"""
    check(load().b200q_embed_ex(_p(ids), _p(prev_out), _p(table), _p(out), ids.numel(), table.shape[1], scale,
                                _stream(stream)))


def rmsnorm(x, w, y, eps, stream=None):
    check(load().b200q_rmsnorm(_p(x), _p(w), _p(y), x.shape[0], x.shape[1], eps, _stream(stream)))


def add_rmsnorm(x, residual, w, eps, stream=None):
    check(load().b200q_add_rmsnorm(_p(x), _p(residual), _p(w), x.shape[0], x.shape[1], eps, _stream(stream)))


def rope_kvwrite(qkv, cos_sin, positions, slot_mapping, kv_layer, n_q, n_kv, D, block_size, stream=None):
    check(load().b200q_rope_kvwrite(_p(qkv), _p(cos_sin), _p(positions), _p(slot_mapping), _p(kv_layer),
                                    qkv.shape[0], n_q, n_kv, D, block_size, _stream(stream)))


def decode_attn(qkv, out, kv_layer, block_table, ctx_lens, n_q, n_kv, D, block_size, scale, stream=None,
                softcap: float = 0.0, window: int = 0):
    if softcap or window:
        check(load().b200q_decode_attn_ex(_p(qkv), qkv.shape[1], _p(out), _p(kv_layer), _p(block_table),
                                          block_table.shape[1], _p(ctx_lens), ctx_lens.numel(), n_q, n_kv, D,
                                          block_size, scale, softcap, window, _stream(stream)))
        return
    check(load().b200q_decode_attn(_p(qkv), qkv.shape[1], _p(out), _p(kv_layer), _p(block_table),
                                   block_table.shape[1], _p(ctx_lens), ctx_lens.numel(), n_q, n_kv, D,
                                   block_size, scale, _stream(stream)))


def prefill_attn(qkv, out, kv_layer, block_table, tiles, n_q, n_kv, D, block_size, scale, stream=None,
                 softcap: float = 0.0, window: int = 0):
    if softcap or window:
        check(load().b200q_prefill_attn_ex(_p(qkv), qkv.shape[1], _p(out), _p(kv_layer), _p(block_table),
                                           block_table.shape[1], _p(tiles), tiles.shape[0], n_q, n_kv, D,
                                           block_size, scale, softcap, window, _stream(stream)))
        return
    check(load().b200q_prefill_attn(_p(qkv), qkv.shape[1], _p(out), _p(kv_layer), _p(block_table),
                                    block_table.shape[1], _p(tiles), tiles.shape[0], n_q, n_kv, D,
                                    block_size, scale, _stream(stream)))


def embed_scaled(ids, table, out, scale, stream=None):
    check(load().b200q_embed_scaled(_p(ids), _p(table), _p(out), ids.numel(), table.shape[1], scale, _stream(stream)))


def gemma_rmsnorm(x, w, y, eps, stream=None):
    check(load().b200q_gemma_rmsnorm(_p(x), _p(w), _p(y), x.shape[0], x.shape[1], eps, _stream(stream)))


def gemma_norm_add_norm(x, residual, w_post, w_next, eps, stream=None):
    """in place: residual <- bf16(residual + gemma_norm(x, w_post)); x <- gemma_norm(residual, w_next)"""
    check(load().b200q_gemma_norm_add_norm(_p(x), _p(residual), _p(w_post), _p(w_next), x.shape[0], x.shape[1],
                                           eps, _stream(stream)))


def gemm_geglu_bf16(a, w_interleaved, c, stream=None):
    M, K = a.shape
    N = w_interleaved.shape[0]
    assert w_interleaved.shape[1] == K and tuple(c.shape) == (M, N // 2)
    check(load().b200q_gemm_geglu_bf16(_p(a), _p(w_interleaved), _p(c), M, N, K, _stream(stream)))


def softcap_bf16(logits, cap, stream=None):
    check(load().b200q_softcap_bf16(_p(logits), logits.numel(), cap, _stream(stream)))


def gemm_bf16(a, w, c, stream=None):
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and tuple(c.shape) == (M, N)
    check(load().b200q_gemm_bf16(_p(a), _p(w), _p(c), M, N, K, _stream(stream)))


def gemm_bf16_splitk(a, w, stream=None):
    """decode-sized batches: split-K GEMM without its reduce pass.  Returns (partials_ptr, splits);
    splits == 1 means nothing was launched (the library would not split this shape)"""
    M, K = a.shape
    N = w.shape[0]
    part, splits = C.c_void_p(), C.c_int(1)
    check(load().b200q_gemm_bf16_splitk(_p(a), _p(w), M, N, K, _stream(stream), C.byref(part), C.byref(splits)))
    return part.value, splits.value


def add_rmsnorm_splitk(x, residual, w, partials_ptr, splits, eps, stream=None):
    check(load().b200q_add_rmsnorm_splitk(_p(x), _p(residual), _p(w), partials_ptr, splits, x.shape[0], x.shape[1], eps,
                                          _stream(stream)))


def rope_kvwrite_splitk(qkv, partials_ptr, splits, cos_sin, positions, slot_mapping, kv_layer, n_q, n_kv, D, block_size,
                        stream=None):
    check(load().b200q_rope_kvwrite_splitk(_p(qkv), partials_ptr, splits, _p(cos_sin), _p(positions), _p(slot_mapping),
                                           _p(kv_layer), qkv.shape[0], n_q, n_kv, D, block_size, _stream(stream)))


def gemm_swiglu_bf16(a, w_interleaved, c, stream=None):
    M, K = a.shape
    N = w_interleaved.shape[0]
    assert w_interleaved.shape[1] == K and tuple(c.shape) == (M, N // 2)
    check(load().b200q_gemm_swiglu_bf16(_p(a), _p(w_interleaved), _p(c), M, N, K, _stream(stream)))


def gemm_set_tile_n(bn: int):
    check(load().b200q_gemm_set_tile_n(bn))


def gemm_set_mode(mode: int):
    check(load().b200q_gemm_set_mode(mode))


def swiglu(gate_up, out, stream=None):
    check(load().b200q_swiglu(_p(gate_up), _p(out), gate_up.shape[0], out.shape[1], _stream(stream)))


def gather_rows(x, rows, out, stream=None):
    check(load().b200q_gather_rows(_p(x), _p(rows), _p(out), rows.numel(), x.shape[1], _stream(stream)))


def sample_bf16(logits, params, ids, stream=None):
    """params: int32 [B,4] = (temperature float bits, seed lo, seed hi, position)"""
    check(load().b200q_sample_bf16(_p(logits), _p(params), _p(ids), logits.shape[0], logits.shape[1], _stream(stream)))


def argmax_bf16(logits, ids, stream=None):
    check(load().b200q_argmax_bf16(_p(logits), _p(ids), logits.shape[0], logits.shape[1], _stream(stream)))
