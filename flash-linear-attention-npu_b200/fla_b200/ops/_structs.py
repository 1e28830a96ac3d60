"""ctypes twins of the argument structs declared in include/fla_b200.h (field order must match)."""
import ctypes

from .._runtime import TensorDesc


class RecurrentGdnArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("q", "k", "v", "g", "beta", "state_in", "state_out", "out",
                                           "cu_seqlens", "state_indices", "num_accepted_tokens", "gk", "a_log",
                                           "dt_bias")] + [
        ("scale", ctypes.c_float), ("lower_bound", ctypes.c_float), ("tokens_per_seq", ctypes.c_int32),
        ("state_v_first", ctypes.c_int32), ("use_qk_l2norm", ctypes.c_int32), ("gate_mode", ctypes.c_int32),
        ("beta_mode", ctypes.c_int32)]


class CausalConv1dFwdArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("x", "weight", "bias", "residual", "initial_state", "y", "final_state",
                                           "cu_seqlens")] + [("activation_silu", ctypes.c_int32)]


class CausalConv1dBwdArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("x", "weight", "bias", "dy", "y_pre", "initial_state", "dht", "dx", "dw", "db",
                                           "dh0", "cu_seqlens")] + [("activation_silu", ctypes.c_int32)]


class CausalConv1dUpdateArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("x", "weight", "bias", "residual", "conv_state", "y", "cache_indices",
                                           "num_accepted_tokens")] + [
        ("activation_silu", ctypes.c_int32), ("pad_slot_id", ctypes.c_int32)]


class GdnChunkFwdArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("q", "k", "v", "g", "beta", "initial_state", "o", "final_state", "gam",
                                           "x_inv", "s_img", "vn_img", "p_img", "cu_seqlens",
                                           "chunk_offsets")] + [
        ("scale", ctypes.c_float), ("chunk_size", ctypes.c_int32), ("max_seqlen", ctypes.c_int32),
        ("total_chunks", ctypes.c_int32)]


class GdnChunkBwdArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("q", "k", "v", "beta", "gam", "x_inv", "s_img", "vn_img", "p_img", "d_o", "dht",
                                           "dq", "dk", "dv", "dg", "dbeta", "dh0", "cu_seqlens", "chunk_offsets")] + [
        ("scale", ctypes.c_float), ("chunk_size", ctypes.c_int32), ("max_seqlen", ctypes.c_int32),
        ("total_chunks", ctypes.c_int32)]


class KdaChunkFwdArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("q", "k", "v", "g", "beta", "a_log", "dt_bias", "initial_state", "o",
                                           "final_state", "gk", "cu_seqlens", "chunk_offsets", "saved", "aqk", "akk")] + [
        ("scale", ctypes.c_float), ("lower_bound", ctypes.c_float), ("gate_mode", ctypes.c_int32),
        ("chunk_size", ctypes.c_int32), ("max_seqlen", ctypes.c_int32), ("total_chunks", ctypes.c_int32)]


class KdaChunkBwdArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("q", "k", "v", "g", "beta", "initial_state", "d_o", "dht", "dq", "dk", "dv",
                                           "dg", "dbeta", "dh0", "cu_seqlens", "chunk_offsets", "saved")] + [
        ("scale", ctypes.c_float), ("chunk_size", ctypes.c_int32), ("max_seqlen", ctypes.c_int32),
        ("total_chunks", ctypes.c_int32)]


class KdaIntermediatesArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("q", "k", "v", "beta", "saved", "cu_seqlens", "chunk_offsets", "w", "u", "qg", "kg",
                                           "v_new", "h")] + [
        ("max_seqlen", ctypes.c_int32), ("total_chunks", ctypes.c_int32), ("state_v_first", ctypes.c_int32)]


class KdaMergeBlocksArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("q", "k", "beta", "gk", "aqk64", "akk64", "cu_seqlens", "chunk_offsets", "aqk", "akk",
                                           "gk_out")] + [("scale", ctypes.c_float), ("max_seqlen", ctypes.c_int32), ("gk_base2", ctypes.c_int32)]


class KdaMergeInterArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("k", "beta", "gk", "akk64", "w64", "u64", "qg64", "kg64", "cu_seqlens", "chunk_offsets",
                                           "w", "u", "qg", "kg")] + [("max_seqlen", ctypes.c_int32), ("gk_base2", ctypes.c_int32)]


class KdaGateArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("g", "a_log", "dt_bias", "gate", "d_gate", "d_g", "d_a_log", "d_dt_bias")] + [
        ("lower_bound", ctypes.c_float), ("gate_mode", ctypes.c_int32)]


class L2NormArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("x", "y", "rstd", "dy", "dx")] + [("eps", ctypes.c_float)]


class FastGeluArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("x", "y", "dy", "dx")]


class ChunkStageArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("q", "k", "v", "w", "u", "g", "beta", "A", "h", "initial_state", "out0", "out1",
                                           "out2", "out3", "cu_seqlens", "chunk_offsets")] + [
        ("scale", ctypes.c_float), ("chunk_size", ctypes.c_int32), ("max_seqlen", ctypes.c_int32),
        ("total_chunks", ctypes.c_int32), ("reverse", ctypes.c_int32), ("gate_mode", ctypes.c_int32),
        ("lower_bound", ctypes.c_float)]


class ChunkKdaBwdIntraArgs(ctypes.Structure):
    _fields_ = [(n, TensorDesc) for n in ("q", "k", "gk", "beta", "d_aqk", "d_akk", "dq", "dk", "db", "dg", "cu_seqlens",
                                           "chunk_offsets")] + [
        ("chunk_size", ctypes.c_int32), ("max_seqlen", ctypes.c_int32), ("total_chunks", ctypes.c_int32)]
