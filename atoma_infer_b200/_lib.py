"""ctypes binding of libflashattention.so (include/atoma_flash.h + include/atoma_ops.h).

The library is the product; this module only loads it and declares signatures.  There is no
fallback: if the shared library is missing the import fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = Path(os.environ.get("ATOMA_FLASH_LIB", _PKG / "lib" / "libflashattention.so"))

MAX_RANK = 5
DEVICE_CPU = -1
F16, BF16, F32, U32, I64, U8, F64 = range(7)


class Tensor(C.Structure):
    """struct atoma_tensor"""

    _fields_ = [
        ("data", C.c_void_p),
        ("dtype", C.c_int32),
        ("device", C.c_int32),
        ("rank", C.c_int32),
        ("shape", C.c_int64 * MAX_RANK),
        ("stride", C.c_int64 * MAX_RANK),
    ]


class MhaArgs(C.Structure):
    """struct atoma_mha_args — the run_mha argument tuple (reference csrc/src/ffi.rs:4-66)."""

    _fields_ = [
        ("q_ptr", C.c_void_p), ("k_ptr", C.c_void_p), ("v_ptr", C.c_void_p), ("o_ptr", C.c_void_p),
        ("softmax_lse_ptr", C.c_void_p), ("alibi_slopes_ptr", C.c_void_p),
        ("cu_seqlens_q_ptr", C.c_void_p), ("cu_seqlens_k_ptr", C.c_void_p),
        ("is_seqlens_k_cumulative", C.c_bool),
        ("q_batch_stride", C.c_uint32), ("k_batch_stride", C.c_uint32),
        ("v_batch_stride", C.c_uint32), ("o_batch_stride", C.c_uint32),
        ("alibi_slopes_batch_stride", C.c_uint32),
        ("q_row_stride", C.c_uint32), ("k_row_stride", C.c_uint32),
        ("v_row_stride", C.c_uint32), ("o_row_stride", C.c_uint32),
        ("q_head_stride", C.c_uint32), ("k_head_stride", C.c_uint32),
        ("v_head_stride", C.c_uint32), ("o_head_stride", C.c_uint32),
        ("num_splits", C.c_uint32),
        ("b", C.c_uint32), ("h", C.c_uint32), ("h_k", C.c_uint32), ("d", C.c_uint32),
        ("d_rounded", C.c_uint32),
        ("softmax_scale", C.c_float), ("scale_softmax_log2", C.c_float),
        ("block_table", C.c_void_p), ("block_table_batch_stride", C.c_uint32),
        ("page_block_size", C.c_int),
        ("seqused_k", C.c_void_p),
        ("seqlen_q", C.c_uint32), ("seqlen_k", C.c_uint32),
        ("seqlen_q_rounded", C.c_uint32), ("seqlen_k_rounded", C.c_uint32),
        ("is_bf16", C.c_int), ("is_causal", C.c_int),
        ("window_size_left", C.c_int), ("window_size_right", C.c_int),
        ("softcap", C.c_float),
        ("unpadded_lse", C.c_bool), ("force_split_kernel", C.c_bool),
        ("softmax_lseaccum_ptr", C.c_void_p), ("oaccum_ptr", C.c_void_p),
    ]


class MhaPlan(C.Structure):
    """struct atoma_mha_plan"""

    _fields_ = [
        ("args", MhaArgs),
        ("out_rank", C.c_int32),
        ("out_shape", C.c_int64 * 4),
        ("lse_elems", C.c_int64),
        ("lseaccum_elems", C.c_int64),
        ("oaccum_elems", C.c_int64),
        ("seqlenq_ngroups_swapped", C.c_int32),
    ]


class Sequence(C.Structure):
    """struct atoma_sequence"""

    _fields_ = [("token_ids", C.POINTER(C.c_uint32)), ("length", C.c_int64), ("num_computed_tokens", C.c_int64),
                ("token_chunk_size", C.c_int64), ("block_table", C.POINTER(C.c_uint32)), ("num_blocks", C.c_int64),
                ("is_prompt", C.c_int32)]


class ModelInputLayout(C.Structure):
    """struct atoma_model_input_layout"""

    _fields_ = [(n, C.c_int64) for n in (
        "total_bytes", "input_tokens_off", "input_positions_off", "slot_mapping_off", "sequence_lengths_off",
        "context_lengths_off", "sequence_start_loc_off", "query_start_loc_off", "block_tables_off",
        "num_tokens", "num_slots", "num_sequences", "max_block_table_len",
        "num_prefills", "num_prefill_tokens", "num_decode_tokens",
        "max_query_len", "max_prefill_seq_len", "max_decode_seq_len")]


class AttentionConfig(C.Structure):
    _fields_ = [
        ("num_heads", C.c_int64), ("num_kv_heads", C.c_int64), ("head_dim", C.c_int64),
        ("softmax_scale", C.c_float), ("sliding_window", C.c_int64),
    ]


class AttentionMetadata(C.Structure):
    _fields_ = [
        ("slot_mapping", C.POINTER(Tensor)),
        ("num_prefill_tokens", C.c_int64), ("num_decoding_tokens", C.c_int64),
        ("has_prefill", C.c_int32),
        ("prefill_block_tables", C.POINTER(Tensor)),
        ("max_prefill_sequence_length", C.c_int64),
        ("query_start_locations", C.POINTER(Tensor)),
        ("sequence_start_locations", C.POINTER(Tensor)),
        ("max_prefill_sequence_length_k", C.c_int64),
        ("has_decode", C.c_int32),
        ("decode_block_tables", C.POINTER(Tensor)),
        ("decode_sequence_lengths", C.POINTER(Tensor)),
    ]


class LlamaLayer(C.Structure):
    """struct atoma_llama_layer (include/atoma_llama.h)"""

    _fields_ = [(n, C.c_void_p) for n in ("wqkv", "wo", "w_gate_up", "w_down", "rms_attn", "rms_mlp",
                                          "key_cache", "value_cache")]


class LlamaModel(C.Structure):
    """struct atoma_llama_model"""

    _fields_ = ([(n, C.c_int64) for n in ("hidden", "inter", "num_layers", "num_heads", "num_kv_heads", "head_dim",
                                           "vocab", "block_size", "block_stride", "rot_stride")] +
                [("rms_eps", C.c_float), ("softmax_scale", C.c_float), ("dtype", C.c_uint32),
                 ("embed", C.c_void_p), ("norm_f", C.c_void_p), ("lm_head", C.c_void_p),
                 ("cos", C.c_void_p), ("sin", C.c_void_p), ("layers", C.POINTER(LlamaLayer)),
                 ("tp_rank", C.c_int32), ("tp_world", C.c_int32), ("p2p_regions", C.POINTER(C.c_void_p)),
                 ("p2p_slot_bytes", C.c_int64), ("lm_head_rows", C.c_int64), ("lm_head_row0", C.c_int64)])


class DecodeBatch(C.Structure):
    """struct atoma_decode_batch"""

    _fields_ = [("num_tokens", C.c_int64), ("tokens", C.c_void_p), ("hidden_in", C.c_void_p),
                ("positions", C.c_void_p), ("slot_mapping", C.c_void_p), ("block_tables", C.c_void_p),
                ("sequence_lengths", C.c_void_p), ("max_blocks", C.c_int64), ("scratch", C.c_void_p),
                ("scratch_bytes", C.c_int64), ("hidden_out", C.c_void_p), ("logits", C.c_void_p),
                ("logits_f32", C.c_void_p), ("next_tokens", C.c_void_p), ("next_logits", C.c_void_p)]



class SigmoidAttnArgs(C.Structure):
    """struct atoma_sigmoid_attn_args (include/atoma_hybrid.h)"""

    _fields_ = ([(n, C.c_void_p) for n in ("q", "k_cache", "v_cache", "out", "positions", "token_seq", "query_start", "block_tables",
                                           "slopes", "head_bias", "talk")] +
                [(n, C.c_int64) for n in ("T", "B", "max_blocks", "H", "G", "dim", "vdim", "block_size")] +
                [("scale", C.c_float), ("softcap", C.c_float), ("dtype", C.c_uint32), ("max_query_len", C.c_int32),
                 ("max_seq_len", C.c_int32)])


class HybridLayer(C.Structure):
    """struct atoma_hybrid_layer"""

    _fields_ = ([("mixer", C.c_int32), ("has_mlp", C.c_int32)] +
                [(n, C.c_void_p) for n in ("norm1", "norm1b", "norm2", "norm2b")] +
                [(n, C.c_int64) for n in ("heads", "kv_heads", "dim", "vdim", "temp_every")] +
                [("scale", C.c_float), ("softcap", C.c_float), ("temp_coef", C.c_float)] +
                [(n, C.c_void_p) for n in ("w_qkv", "b_qkv", "q_norm", "k_norm", "talk", "head_bias", "slopes",
                                           "k_cache", "v_cache")] +
                [("state_width", C.c_int64)] +
                [(n, C.c_void_p) for n in ("w_zxg", "b_zxg", "state", "w_o")] +
                [("ff", C.c_int64), ("act", C.c_int32), ("w_gate_up", C.c_void_p), ("w_down", C.c_void_p)] +
                # pre-norm blocks: latent attention, gated residuals, mixture of experts, token side input
                [(n, C.c_int64) for n in ("q_rank", "kv_rank", "window")] +
                [(n, C.c_void_p) for n in ("w_down_in", "dq_norm", "dkv_norm", "sink", "w_uq", "w_uk", "w_uv", "latent_cache",
                                           "gate1_bias", "gate2_bias")] +
                [("ff_kind", C.c_int32), ("renormalize", C.c_int32)] +
                [(n, C.c_int64) for n in ("experts", "top", "expert_ff")] +
                [(n, C.c_float) for n in ("expert_limit", "shared_limit", "act_alpha", "act_up_shift")] +
                [(n, C.c_void_p) for n in ("w_router", "w_shared_gate", "w_expert_gate_up", "w_expert_down", "w_ff_in")] +
                [("side_part", C.c_int64)] +
                [(n, C.c_void_p) for n in ("side_gate", "side_proj", "side_norm")] +
                # blocks on residual lanes: softmax attention with a distance table, lane weights, biases, restricted routing
                [("keep_first", C.c_int64), ("dist_rows", C.c_int64), ("dist_bias", C.c_void_p),
                 ("values_are_keys", C.c_int32), ("out_gate", C.c_int32)] +
                [(n, C.c_void_p) for n in ("lanes_in1", "lanes_out1", "lanes_mix1", "lanes_in2", "lanes_out2", "lanes_mix2",
                                           "b_gate_up", "b_down", "router_correction")] +
                [(n, C.c_int64) for n in ("route_groups", "route_keep", "identity_experts")] +
                [("score_fn", C.c_int32), ("scale_input", C.c_int32)] +
                # parallel blocks: what precedes the layer, tap filters, the layer's state row, the stacked projection's columns,
                # gated linear attention, the pair of mixers (rotary sigmoid attention + gated delta rule), rotated latent keys
                [("add_embedding", C.c_int32), ("add_vec", C.c_void_p), ("taps", C.c_int64), ("tap_w1", C.c_void_p), ("tap_w2", C.c_void_p),
                 ("layer_state", C.c_void_p), ("layer_state_stride", C.c_int64), ("proj_cols", C.c_int64)] +
                [(n, C.c_int64) for n in ("q_off", "k_off", "v_off", "g_off", "a_off", "a_rank")] +
                [(n, C.c_void_p) for n in ("w_a2", "a2_bias", "head_norm")] + [("tau", C.c_float)] +
                [("qk_freq", C.c_void_p), ("v_freq", C.c_void_p), ("rot_pairs", C.c_int64), ("v_pairs", C.c_int64), ("rot_interleaved", C.c_int32)] +
                [(n, C.c_int64) for n in ("r_heads", "r_kv_heads", "r_dim", "r_vdim", "r_taps", "rq_off", "rk_off", "rv_off", "rg_off", "rb_off",
                                          "ra_off")] +
                [(n, C.c_void_p) for n in ("r_tap_w", "r_a_log", "r_dt_bias", "r_head_norm", "r_w_o", "out_norm_a", "out_norm_b")] +
                [("rot_dim", C.c_int64)])


class HybridModel(C.Structure):
    """struct atoma_hybrid_model"""

    _fields_ = ([(n, C.c_int64) for n in ("width", "vocab", "num_layers", "block_size")] +
                [("eps", C.c_float), ("logit_scale", C.c_float), ("norm_offset", C.c_float), ("dtype", C.c_uint32)] +
                [(n, C.c_void_p) for n in ("embed", "inv_freq", "final_norm", "head")] +
                [("layers", C.POINTER(HybridLayer))] +
                [("block_style", C.c_int32), ("norm_groups", C.c_int32), ("pos_table", C.c_void_p), ("max_positions", C.c_int64),
                 ("logit_softcap", C.c_float), ("side_table", C.c_void_p), ("side_dim", C.c_int64), ("side_table_width", C.c_int64),
                 ("lanes", C.c_int32), ("embed_scale", C.c_float)])


class GatedResidualArgs(C.Structure):
    """struct atoma_gated_residual_args"""

    _fields_ = [("y", C.c_void_p), ("ld_y", C.c_int64), ("row_scale", C.c_void_p), ("expert_out", C.c_void_p), ("pair_row", C.c_void_p),
                ("top", C.c_int64), ("gate", C.c_void_p), ("ld_gate", C.c_int64), ("gate_bias", C.c_void_p), ("x", C.c_void_p),
                ("w_next", C.c_void_p), ("h", C.c_void_p), ("x_cast", C.c_void_p), ("T", C.c_int64), ("width", C.c_int64),
                ("groups", C.c_int64), ("eps", C.c_float), ("weight_offset", C.c_float), ("dtype", C.c_uint32)]


class LanesUpdateArgs(C.Structure):
    """struct atoma_lanes_update_args"""

    _fields_ = ([(n, C.c_void_p) for n in ("y", "y_bias", "expert_out", "pair_row", "top_expert", "top_weight", "h_in")] +
                [("top", C.c_int64), ("experts", C.c_int64)] +
                [(n, C.c_void_p) for n in ("x", "w_mix", "w_out", "w_in_next", "w_next", "h", "lane_sum")] +
                [(n, C.c_int64) for n in ("T", "lanes", "width")] +
                [("eps", C.c_float), ("weight_offset", C.c_float), ("dtype", C.c_uint32)])


class SoftmaxAttnArgs(C.Structure):
    """struct atoma_softmax_attn_args"""

    _fields_ = ([(n, C.c_void_p) for n in ("q", "k_cache", "v_cache", "out", "gate")] + [("ld_gate", C.c_int64), ("dist_bias", C.c_void_p),
                                                                                          ("dist_rows", C.c_int64)] +
                [(n, C.c_void_p) for n in ("positions", "token_seq", "query_start", "block_tables")] +
                [(n, C.c_int64) for n in ("T", "B", "max_blocks", "H", "G", "dim", "vdim", "block_size", "window", "keep_first")] +
                [("scale", C.c_float), ("dtype", C.c_uint32), ("max_query_len", C.c_int32), ("max_seq_len", C.c_int32),
                 ("skip_min_q", C.c_int32), ("long_min_q", C.c_int32), ("long_seqs", C.c_int32), ("long_tokens", C.c_int64),
                 ("long_ctx_sum", C.c_int64)])


class ParallelResidualArgs(C.Structure):
    """struct atoma_parallel_residual_args"""

    _fields_ = ([(n, C.c_void_p) for n in ("y_a", "y_b", "y_ff", "norm_a", "norm_b")] + [("mix_scale", C.c_float)] +
                [(n, C.c_void_p) for n in ("x", "trace", "add_rows", "add_vec", "w_next", "h")] +
                [("T", C.c_int64), ("width", C.c_int64), ("eps", C.c_float), ("weight_offset", C.c_float), ("dtype", C.c_uint32)])


class TapFilterArgs(C.Structure):
    """struct atoma_tap_filter_args"""

    _fields_ = ([("in_", C.c_void_p), ("ld_in", C.c_int64)] + [(n, C.c_void_p) for n in ("w1", "w2", "out1", "out2")] +
                [("ld_out", C.c_int64), ("history", C.c_void_p), ("history_stride", C.c_int64)] +
                [(n, C.c_void_p) for n in ("state_slots", "token_seq", "query_start", "context_lens")] +
                [(n, C.c_int64) for n in ("T", "B", "channels", "taps")] +
                [("residual", C.c_int32), ("act", C.c_int32), ("dtype", C.c_uint32)])


class StateScanArgs(C.Structure):
    """struct atoma_state_scan_args"""

    _fields_ = ([("kind", C.c_int32)] + [(n, C.c_void_p) for n in ("q", "k", "v", "z", "b_pre", "a_pre")] +
                [(n, C.c_int64) for n in ("ld_q", "ld_k", "ld_v", "ld_z", "ld_b", "ld_a")] +
                [(n, C.c_void_p) for n in ("z_bias", "a_log", "dt_bias")] +
                [(n, C.c_float) for n in ("tau", "q_scale", "unit_eps")] +
                [("state", C.c_void_p), ("state_stride", C.c_int64)] +
                [(n, C.c_void_p) for n in ("state_slots", "query_start", "context_lens", "out")] +
                [(n, C.c_int64) for n in ("T", "B", "H", "G", "dim", "vdim")] + [("dtype", C.c_uint32)])


class QkvRopeArgs(C.Structure):
    """struct atoma_qkv_rope_args"""

    _fields_ = ([("proj", C.c_void_p)] + [(n, C.c_int64) for n in ("ld", "q_off", "k_off", "v_off")] +
                [(n, C.c_void_p) for n in ("q_weight", "k_weight", "qk_freq", "v_freq")] +
                [("rot_pairs", C.c_int64), ("v_pairs", C.c_int64), ("interleaved", C.c_int32)] +
                [(n, C.c_void_p) for n in ("positions", "slot_mapping", "q_out", "k_cache", "v_cache")] +
                [(n, C.c_int64) for n in ("T", "H", "G", "dim", "vdim")] + [("eps", C.c_float), ("dtype", C.c_uint32)])


class LatentAttnArgs(C.Structure):
    """struct atoma_latent_attn_args"""

    _fields_ = ([(n, C.c_void_p) for n in ("q_lat", "latent_cache", "out", "positions", "token_seq", "query_start", "block_tables", "sink")] +
                [(n, C.c_int64) for n in ("T", "B", "max_blocks", "H", "R", "block_size", "window")] +
                [("scale", C.c_float), ("dtype", C.c_uint32), ("max_query_len", C.c_int32), ("max_seq_len", C.c_int32),
                 ("skip_min_q", C.c_int32), ("out_cols", C.c_int64)])


class LatentExpandedArgs(C.Structure):
    """struct atoma_latent_expanded_args"""

    _fields_ = ([(n, C.c_void_p) for n in ("q", "latent_cache", "w_uk", "w_uv", "out", "query_start", "context_lens", "block_tables", "sink")] +
                [(n, C.c_int64) for n in ("T", "B", "max_blocks", "H", "dim", "R", "block_size", "window", "max_keys")] +
                [("scale", C.c_float), ("min_q", C.c_int32), ("max_query_len", C.c_int32), ("max_seq_len", C.c_int32)])


class MoeArgs(C.Structure):
    """struct atoma_moe_args"""

    _fields_ = ([(n, C.c_void_p) for n in ("h", "top_expert", "top_weight", "w_gate_up", "w_down", "workspace")] +
                [(n, C.c_int64) for n in ("workspace_bytes", "T", "width", "experts", "top", "ff")] +
                [(n, C.c_float) for n in ("limit", "alpha", "up_shift")] + [("scale_input", C.c_int32), ("dtype", C.c_uint32)])


class HybridBatch(C.Structure):
    """struct atoma_hybrid_batch"""

    _fields_ = ([(n, C.c_int64) for n in ("num_tokens", "num_seqs", "num_selected", "max_blocks")] +
                [("max_query_len", C.c_int32), ("max_seq_len", C.c_int32)] +
                [(n, C.c_void_p) for n in ("tokens", "positions", "slot_mapping", "token_seq", "query_start", "context_lens",
                                           "block_tables", "state_slots", "selected", "scratch")] +
                [("scratch_bytes", C.c_int64)] +
                [(n, C.c_void_p) for n in ("logits", "next_tokens", "residual_trace")] +
                [("long_seqs", C.c_int32), ("long_min_q", C.c_int32), ("long_tokens", C.c_int64), ("long_ctx_sum", C.c_int64)])


# Exact C parameter lists, in header order.
_RUN_MHA_ARGS = [
    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,  # q k v o lse alibi
    C.c_void_p, C.c_void_p,  # cu_seqlens_q, cu_seqlens_k
    C.c_bool,
    C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,  # batch strides + alibi
    C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,  # row strides
    C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,  # head strides
    C.c_uint32,  # num_splits
    C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,  # b h h_k d d_rounded
    C.c_float, C.c_float,
    C.c_void_p, C.c_uint32, C.c_int,  # block_table, stride, page
    C.c_void_p,  # seqused_k
    C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,  # seqlens
    C.c_int, C.c_int, C.c_int, C.c_int,  # is_bf16 is_causal wl wr
    C.c_float, C.c_bool, C.c_bool,
    C.c_void_p, C.c_void_p,
]

# symbol -> (restype, argtypes); every symbol include/*.h declares is listed here and checked by
# tests/test_abi.py against the headers.
SIGNATURES = {
    # atoma_flash.h, part 1 (reference ABI)
    "run_mha": (None, _RUN_MHA_ARGS),
    "copy_blocks_f16": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "copy_blocks_bf16": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "reshape_and_cache_flash": (None, [C.c_void_p] * 5 + [C.c_int64] * 7 + [C.c_uint32, C.c_void_p]),
    # part 2 (extensions)
    "run_mha_stream": (None, _RUN_MHA_ARGS + [C.c_void_p]),
    "atoma_rope_reshape_and_cache": (None, [C.c_void_p] * 9 + [C.c_int64] * 10 + [C.c_uint32, C.c_void_p]),
    "swap_blocks_batched": (None, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                   C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "atoma_gemm_bf16_tn": (None, [C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int64] * 6 + [C.c_void_p]),
    "atoma_p2p_region_bytes": (C.c_int64, [C.c_int64]),
    "atoma_p2p_alloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_int64]),
    "atoma_p2p_free": (C.c_int, [C.c_void_p]),
    "atoma_p2p_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "atoma_p2p_import": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "atoma_p2p_close": (C.c_int, [C.c_void_p]),
    "atoma_p2p_slot": (C.c_void_p, [C.c_void_p, C.c_int64, C.c_int]),
    "atoma_p2p_error": (C.c_int, [C.c_void_p, C.c_void_p]),
    "atoma_allreduce_sum_p2p": (None, [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int64, C.c_int, C.c_void_p,
                                       C.c_int64, C.c_uint32, C.c_void_p]),
    "atoma_debug_allreduce_algo": (None, [C.c_int]),
    "atoma_debug_decode_trace": (None, [C.c_void_p]),
    "atoma_debug_decode_merge": (None, [C.c_int]),
    "atoma_debug_step_trace": (None, [C.c_void_p, C.c_int]),
    "atoma_debug_step_trace_names": (C.c_int, [C.c_char_p, C.c_int]),
    "atoma_debug_gemm_trace": (None, [C.c_void_p]),
    "atoma_debug_gemm_stages": (None, [C.c_int]),
    "atoma_debug_gemm_algo": (None, [C.c_int]),
    "atoma_set_launch_mode": (None, [C.c_int]),
    "atoma_get_launch_mode": (C.c_int, []),
    "atoma_last_status": (C.c_int, []),
    "atoma_last_error": (C.c_char_p, []),
    "atoma_last_mha_path": (C.c_char_p, []),
    "atoma_last_decode_mode": (C.c_int, []),
    "atoma_launch_count": (C.c_int64, []),
    "atoma_reset_launch_count": (None, []),
    "atoma_version": (C.c_char_p, []),
    "atoma_source_hash": (C.c_char_p, []),
    "atoma_mha_call_flags": (None, [C.c_int]),
    # atoma_llama.h
    "atoma_gemm_tn": (None, [C.c_void_p] * 3 + [C.c_int64] * 6 + [C.c_uint32, C.c_void_p]),
    "atoma_qkv_rope_cache": (None, [C.c_void_p] * 3 + [C.c_int64] * 8 + [C.c_void_p] * 3 + [C.c_int64] +
                             [C.c_void_p] * 3 + [C.c_int64] * 2 + [C.c_uint32, C.c_void_p]),
    "atoma_gate_up_silu": (None, [C.c_void_p] * 3 + [C.c_int64] * 6 + [C.c_uint32, C.c_void_p]),
    "atoma_gate_up_act": (None, [C.c_void_p] * 3 + [C.c_int64] * 6 + [C.c_int32, C.c_uint32, C.c_void_p]),
    "atoma_gate_up_clamped": (None, [C.c_void_p] * 4 + [C.c_int64] * 6 + [C.c_float] * 3 + [C.c_uint32, C.c_void_p]),
    "atoma_add_rmsnorm": (None, [C.c_void_p] * 5 + [C.c_int64] * 6 + [C.c_float, C.c_uint32, C.c_void_p]),
    "atoma_embedding": (None, [C.c_void_p] * 3 + [C.c_int64] * 5 + [C.c_uint32, C.c_void_p]),
    "atoma_sample_greedy": (None, [C.c_void_p] + [C.c_int64] * 3 + [C.c_uint32] + [C.c_void_p] * 3 +
                            [C.c_int64, C.c_void_p]),
    "atoma_gemm_tn_push": (None, [C.c_void_p] * 2 + [C.c_int64] * 5 + [C.POINTER(C.c_void_p), C.c_int, C.c_int,
                                                                       C.c_int64, C.c_uint32, C.c_void_p]),
    "atoma_allreduce_recv_add_rmsnorm": (None, [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int64] + [C.c_void_p] * 4 +
                                         [C.c_int64] * 5 + [C.c_float, C.c_uint32, C.c_void_p]),
    "atoma_llama_decode_scratch_bytes": (C.c_int64, [C.POINTER(LlamaModel), C.c_int64]),
    "atoma_llama_decode_step": (None, [C.POINTER(LlamaModel), C.POINTER(DecodeBatch), C.c_void_p]),
    "atoma_debug_skinny_trace": (None, [C.c_void_p]),
    "atoma_debug_skinny_tuning": (None, [C.c_int] * 3),
    "atoma_debug_skinny_mode": (None, [C.c_int] * 2),
    "atoma_debug_skinny_budget": (None, [C.c_int]),
    "atoma_debug_step_prefetch": (None, [C.c_int] * 2),
    "atoma_debug_step_fusion": (None, [C.c_int]),
    "atoma_llama_abi_sizeof": (C.c_int64, [C.c_int]),
    "atoma_llama_step_status": (C.c_int, [C.c_void_p]),
    "atoma_mlp_gate_up_down": (None, [C.c_void_p] * 5 + [C.c_int64] * 8 + [C.c_uint32, C.c_void_p]),
    "atoma_sample_greedy_tp": (None, [C.c_void_p] + [C.c_int64] * 4 + [C.c_uint32, C.c_void_p, C.c_void_p,
                                                                        C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int64, C.c_void_p]),
    "atoma_gemm_tn_add_rmsnorm": (None, [C.c_void_p] * 3 + [C.c_int64] * 6 + [C.c_void_p] * 4 + [C.c_int64] * 3 +
                                  [C.c_float, C.c_uint32, C.c_void_p]),
    # atoma_hybrid.h
    "atoma_embed_sinusoid": (None, [C.c_void_p] * 5 + [C.c_int64] * 3 + [C.c_uint32, C.c_void_p]),
    "atoma_rmsnorm_rows": (None, [C.c_void_p] * 3 + [C.c_float, C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_uint32, C.c_void_p]),
    "atoma_postnorm_add_prenorm": (None, [C.c_void_p] * 5 + [C.c_int64, C.c_int64, C.c_float, C.c_float, C.c_uint32, C.c_void_p]),
    "atoma_qk_norm_cache": (None, [C.c_void_p] * 9 + [C.c_int64] * 5 + [C.c_float, C.c_float, C.c_int64, C.c_uint32, C.c_void_p]),
    "atoma_sigmoid_attention_paged": (None, [C.POINTER(SigmoidAttnArgs), C.c_void_p]),
    "atoma_mingru_scan": (None, [C.c_void_p] * 7 + [C.c_int64] * 3 + [C.c_int32, C.c_uint32, C.c_void_p]),
    "atoma_glu": (None, [C.c_void_p] * 2 + [C.c_int64] * 2 + [C.c_int32, C.c_uint32, C.c_void_p]),
    "atoma_linear": (None, [C.c_void_p] * 3 + [C.c_int64] * 3 + [C.c_uint32, C.c_void_p]),
    "atoma_scale_logits_greedy": (None, [C.c_void_p] * 3 + [C.c_int64] * 2 + [C.c_float, C.c_uint32, C.c_void_p]),
    "atoma_embed_learned": (None, [C.c_void_p] * 5 + [C.c_int64] * 4 + [C.c_uint32, C.c_void_p]),
    "atoma_group_rmsnorm_rows": (None, [C.c_void_p] * 3 + [C.c_float, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_uint32,
                                        C.c_void_p]),
    "atoma_gated_residual_norm": (None, [C.POINTER(GatedResidualArgs), C.c_void_p]),
    "atoma_side_gate": (None, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_int64,
                               C.c_int64, C.c_uint32, C.c_void_p]),
    "atoma_unitnorm_add_norm": (None, [C.c_void_p] * 5 + [C.c_int64] * 3 + [C.c_float, C.c_float, C.c_uint32, C.c_void_p]),
    "atoma_latent_norm_cache": (None, [C.c_void_p, C.c_int64] + [C.c_void_p] * 5 + [C.c_int64] * 3 + [C.c_float, C.c_uint32, C.c_void_p]),
    "atoma_head_project": (None, [C.c_void_p] * 3 + [C.c_int64] * 4 + [C.c_int32, C.c_uint32, C.c_void_p]),
    "atoma_latent_attention_paged": (None, [C.POINTER(LatentAttnArgs), C.c_void_p]),
    "atoma_latent_attention_expanded": (None, [C.POINTER(LatentExpandedArgs), C.c_void_p]),
    "atoma_moe_route": (None, [C.c_void_p] * 6 + [C.c_int64] * 4 + [C.c_int32, C.c_uint32, C.c_void_p]),
    "atoma_glu_clamped": (None, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_float, C.c_float, C.c_uint32,
                                 C.c_void_p]),
    "atoma_moe_workspace_bytes": (C.c_int64, [C.c_int64] * 5 + [C.c_uint32]),
    "atoma_moe_experts": (None, [C.POINTER(MoeArgs), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_void_p]),
    "atoma_finish_logits_greedy": (None, [C.c_void_p] * 3 + [C.c_int64] * 2 + [C.c_float, C.c_float, C.c_uint32, C.c_void_p]),
    "atoma_embed_scaled_lanes": (None, [C.c_void_p, C.c_void_p, C.c_float, C.c_void_p] + [C.c_int64] * 4 + [C.c_uint32, C.c_void_p]),
    "atoma_lanes_read_norm": (None, [C.c_void_p] * 4 + [C.c_float, C.c_void_p, C.c_void_p] + [C.c_int64] * 3 + [C.c_float, C.c_uint32, C.c_void_p]),
    "atoma_lanes_update_norm": (None, [C.POINTER(LanesUpdateArgs), C.c_void_p]),
    "atoma_qk_headnorm_cache": (None, [C.c_void_p] + [C.c_int64] * 4 + [C.c_void_p, C.c_void_p, C.c_float] + [C.c_void_p] * 4 + [C.c_int64] * 5 +
                                [C.c_float, C.c_uint32, C.c_void_p]),
    "atoma_softmax_attention_paged": (None, [C.POINTER(SoftmaxAttnArgs), C.c_void_p]),
    "atoma_moe_route_grouped": (None, [C.c_void_p] * 5 + [C.c_int64] * 6 + [C.c_int32, C.c_int32, C.c_uint32, C.c_void_p]),
    "atoma_glu_clamped_bias": (None, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_float, C.c_float,
                                      C.c_uint32, C.c_void_p]),
    "atoma_linear_glu_clamped": (None, [C.c_void_p] * 5 + [C.c_int64] * 3 + [C.c_float] * 3 + [C.c_uint32, C.c_void_p]),
    "atoma_parallel_residual_norm": (None, [C.POINTER(ParallelResidualArgs), C.c_void_p]),
    "atoma_tap_filter": (None, [C.POINTER(TapFilterArgs), C.c_void_p]),
    "atoma_state_scan": (None, [C.POINTER(StateScanArgs), C.c_void_p]),
    "atoma_headnorm_gate": (None, [C.c_void_p] * 3 + [C.c_int64, C.c_void_p] + [C.c_int64] * 3 + [C.c_float, C.c_uint32, C.c_void_p]),
    "atoma_qkv_headnorm_rope_cache": (None, [C.POINTER(QkvRopeArgs), C.c_void_p]),
    "atoma_rotate_heads": (None, [C.c_void_p] * 3 + [C.c_int64] * 4 + [C.c_int32, C.c_float, C.c_uint32, C.c_void_p]),
    "atoma_latent_norm_rope_cache": (None, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32] + [C.c_void_p] * 4 +
                                     [C.c_int64] * 4 + [C.c_float, C.c_uint32, C.c_void_p]),
    "atoma_latent_query_absorb_rope": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p] + [C.c_int64] * 5 +
                                       [C.c_uint32, C.c_void_p]),
    "atoma_latent_expand_values": (None, [C.c_void_p] * 3 + [C.c_int64] * 5 + [C.c_uint32, C.c_void_p]),
    "atoma_hybrid_abi_sizeof": (C.c_int64, [C.c_int]),
    "atoma_hybrid_scratch_bytes": (C.c_int64, [C.POINTER(HybridModel), C.c_int64, C.c_int64]),
    "atoma_hybrid_step": (None, [C.POINTER(HybridModel), C.POINTER(HybridBatch), C.c_void_p]),
    "atoma_debug_hybrid": (None, [C.c_int]),
    # atoma_ops.h
    "atoma_flash_attn_plan": (C.c_char_p, [C.POINTER(Tensor)] * 4 + [C.c_float, C.c_int64, C.c_int64, C.c_float,
                                                                    C.c_int, C.POINTER(MhaPlan)]),
    "atoma_flash_attn_varlen_plan": (C.c_char_p, [C.POINTER(Tensor)] * 8 + [C.c_int64, C.c_int64, C.c_float,
                                                                           C.c_int64, C.c_int64, C.c_float, C.c_int,
                                                                           C.POINTER(MhaPlan)]),
    "atoma_flash_attn_kv_cache_plan": (C.c_char_p, [C.POINTER(Tensor)] * 6 + [C.c_float, C.c_int64, C.c_int64,
                                                                             C.c_int, C.POINTER(MhaPlan)]),
    "atoma_mha_execute": (C.c_char_p, [C.POINTER(MhaPlan), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_int, C.c_void_p]),
    "atoma_compute_num_splits": (C.c_uint32, [C.c_int64] * 5 + [C.c_int]),
    "atoma_reshape_and_cache_flash": (C.c_char_p, [C.POINTER(Tensor)] * 5 + [C.c_void_p]),
    "atoma_copy_blocks": (C.c_char_p, [C.POINTER(Tensor), C.c_int64, C.POINTER(Tensor), C.c_int64,
                                       C.POINTER(Tensor), C.c_void_p, C.c_void_p]),
    "atoma_swap_blocks": (C.c_char_p, [C.POINTER(Tensor), C.POINTER(Tensor), C.POINTER(C.c_int64),
                                       C.POINTER(C.c_int64), C.c_int64, C.c_void_p]),
    "atoma_prepare_input": (C.c_char_p, [C.POINTER(Sequence), C.c_int64, C.c_int64, C.c_int64, C.c_int,
                                         C.POINTER(ModelInputLayout), C.c_void_p, C.c_int64]),
    "atoma_flash_attention_forward": (C.c_char_p, [C.POINTER(AttentionConfig)] + [C.POINTER(Tensor)] * 5 +
                                      [C.POINTER(AttentionMetadata), C.POINTER(Tensor), C.c_void_p]),
}


def source_hash() -> str:
    """What csrc/Makefile compiles into atoma_source_hash(): SHA-256 (16 hex digits) of the library's sources,
    csrc/ then include/, each in sorted order.  Equal to the loaded library's hash <=> the binary was built
    from this tree."""
    import hashlib
    src = _PKG / "csrc"
    files = sorted(str(p) for pat in ("*.cu", "*.cuh", "*.h", "*.cpp") for p in src.glob(pat))
    files += sorted(str(p) for p in (_PKG.parent / "include").glob("*.h"))
    h = hashlib.sha256()
    for f in files:
        h.update(Path(f).read_bytes())
    return h.hexdigest()[:16]


def load(path: os.PathLike | str | None = None) -> C.CDLL:
    p = Path(path) if path else LIB_PATH
    if not p.exists():
        raise ImportError(
            f"{p} not found: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            f"(or `make -C atoma_infer_b200/csrc`). There is no CPU or PyTorch fallback for this library."
        )
    lib = C.CDLL(str(p), mode=C.RTLD_LOCAL)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing
        fn.restype = res
        fn.argtypes = args
    return lib


def ensure_built(verbose: bool = True) -> None:
    """Builds lib/libflashattention.so from csrc/ when it is missing or was built from other sources (a fresh
    checkout holds no binaries).  Needs nvcc; everything is compiled for sm_100a."""
    import shutil
    import subprocess
    import sys
    if LIB_PATH.exists():
        try:
            have = C.CDLL(str(LIB_PATH), mode=C.RTLD_LOCAL)
            have.atoma_source_hash.restype = C.c_char_p
            if have.atoma_source_hash().decode() == source_hash():
                return
        except (OSError, AttributeError):
            pass
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = ["make", "-C", str(_PKG / "csrc"), "-j", str(min(16, os.cpu_count() or 4)), "shared", f"NVCC={nvcc}"]
    if verbose:
        print("building", LIB_PATH, file=sys.stderr, flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout[-8000:])
        raise ImportError(f"building {LIB_PATH} failed (exit code {r.returncode})")


_LIB: C.CDLL | None = None


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = load()
    return _LIB
