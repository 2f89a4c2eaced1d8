"""ctypes binding of libcallaghan_b200.so (the C ABI declared in include/callaghan_b200.h).

The library is the product; this module only loads it.  There is no fallback: if the shared library is missing,
import fails with instructions to build it, and if no CUDA device is present ``b200_create`` returns an error that
is raised as RuntimeError.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libcallaghan_b200.so"

OK, ERR_INVALID_ARG, ERR_SHAPE, ERR_OUT_OF_RANGE, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_NONFINITE, ERR_UNSUPPORTED, ERR_PEER = 0, 1, 2, 3, 4, 5, 6, 7, 8, 9
GEMM_AUTO, GEMM_FP32_SIMT, GEMM_TF32_TCGEN05 = 0, 1, 2
OPT_SGD, OPT_ADAM = 0, 1
ENGINES = ("gemm_simt", "gemm_tile", "gemm_persistent", "gemm_pair", "attn_fp32", "attn_mma_sync", "attn_tcgen05", "ce_fused")
ACT = {"None": 0, "Sigmoid": 1, "Tanh": 2, "Relu": 3, "Leakyrelu": 4, "Swish": 5}
COST = {"mse": 0, "ZeroWeightedMSE": 1, "binaryCrossEntropy": 2, "mae": 3, "categoricalCrossEntropy": 4, "huberLoss": 5}


class LMConfig(C.Structure):
    """b200_lm_config."""

    _fields_ = [(n, C.c_int32) for n in ("vocab_size", "input_feature_dim", "output_dim", "embedding_dim", "num_heads", "num_layers",
                                          "ffn_dim", "ffn_activation", "discrete", "loss_kind", "causal", "align_floats")]


GRAD_READY_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p)

_f = C.POINTER(C.c_float)
_i = C.POINTER(C.c_int32)
_b = C.POINTER(C.c_uint8)
_pp = C.POINTER(C.c_void_p)
_i32, _i64, _fl, _vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p

# name -> (restype, argtypes).  Every symbol declared in include/callaghan_b200.h appears here; a CPU-only test checks
# that the header, this table and the built library agree.
PROTOTYPES = {
    "b200_create": (_i32, [_i32, _pp]),
    "b200_destroy": (_i32, [_vp]),
    "b200_last_error": (C.c_char_p, [_vp]),
    "b200_set_stream": (_i32, [_vp, _vp]),
    "b200_set_gemm_mode": (_i32, [_vp, _i32]),
    "b200_synchronize": (_i32, [_vp]),
    "b200_kernel_launches": (_i64, [_vp]),
    "b200_has_tcgen05": (_i32, [_vp]),
    "b200_engine_launches": (_i32, [_vp, C.POINTER(_i64)]),
    "b200_set_gemm_kernel": (_i32, [_vp, _i32]),
    "b200_set_wait_budget_us": (_i32, [_vp, _i64]),
    "b200_probe_wait_timeout": (_i32, [_vp]),
    "b200_profile_gemm": (_i32, [_vp, _i32]),
    "b200_gemm_profile_csv": (_i64, [_vp, C.c_char_p, _i64]),
    "b200_gemm_profile": (_i32, [_vp, _i32, C.POINTER(_i64), C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "b200_MatrixMultiply": (_i32, [_vp, _f, _i32, _i32, _f, _i32, _i32, _f]),
    "b200_MatrixMultiplyTranspose": (_i32, [_vp, _f, _i32, _i32, _f, _i32, _i32, _f]),
    "b200_BatchDotProductAddBias": (_i32, [_vp, _f, _i32, _i32, _f, _i32, _i32, _i32, _i32, _f, _i32, _f]),
    "b200_ProjectOutputBatch": (_i32, [_vp, _f, _i32, _i32, _f, _f, _i32, _i32, _f]),
    "b200_MatrixAddInPlace": (_i32, [_vp, _f, _f, _i64]),
    "b200_VectorAccumulate": (_i32, [_vp, _f, _f, _i64]),
    "b200_ZeroMatrix": (_i32, [_vp, _f, _i64]),
    "b200_ZeroVector": (_i32, [_vp, _f, _i64]),
    "b200_ResidualLayerNormForward": (_i32, [_vp, _f, _f, _f, _f, _i32, _i32, _fl, _f, _f, _f, _f, _f]),
    "b200_LayerNormBackward": (_i32, [_vp, _f, _f, _f, _f, _f, _f, _i32, _i32, _fl, _f, _f, _f]),
    "b200_LayerNormBackward_noalloc": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _fl, _vp, _vp, _vp]),
    "b200_ScaledDotProductAttention": (_i32, [_vp, _f, _f, _f, _i32, _i32, _i32, _i32, _b, _i32, _f]),
    "b200_MultiHeadAttentionForward": (_i32, [_vp, _f, _f, _f, _i32, _i32, _i32, _i32, _fl, _b, _f]),
    "b200_MultiHeadAttentionBackward": (_i32, [_vp, _f, _f, _f, _f, _i32, _i32, _i32, _i32, _fl, _b, _i32, _f, _f, _f]),
    "b200_SegmentedAttentionForward": (_i32, [_vp, _f, _f, _f, _i32, _i32, _i32, _i32, _i32, _f]),
    "b200_SegmentedAttentionBackward": (_i32, [_vp, _f, _f, _f, _f, _i32, _i32, _i32, _i32, _fl, _i32, _f, _f, _f]),
    "b200_ApplyRotaryPositionEmbeddingInPlace": (_i32, [_vp, _f, _i32, _i32, _i32, _fl, _i32, _i32]),
    "b200_ApplyRotaryPositionEmbeddingHeadInPlace": (_i32, [_vp, _f, _i32, _i32, _i32, _i32, _fl, _i32]),
    "b200_ProjectQKV": (_i32, [_vp, _f, _i32, _i32, _f, _f, _f, _f, _f, _f, _i32, _f, _f, _f]),
    "b200_BackpropQKV": (_i32, [_vp, _f, _i32, _i32, _f, _f, _f, _i32, _f, _f, _f, _f, _f, _f, _f, _f, _f, _f]),
    "b200_ProjectKV": (_i32, [_vp, _f, _i32, _i32, _f, _f, _f, _f, _i32, _f, _f]),
    "b200_BackpropKV": (_i32, [_vp, _f, _i32, _i32, _f, _f, _i32, _f, _f, _f, _f, _f, _f, _f]),
    "b200_BackpropLinearProjection": (_i32, [_vp, _f, _f, _f, _i32, _i32, _i32, _f, _f, _f]),
    # sibling trainers' operators
    "b200_ContentAwareCrossAttentionForward": (_i32, [_vp, _f, _i32, _f, _f, _i32, _i32, _i32, _fl, _f, _f, _f, _f]),
    "b200_BackpropTimeDecayedAttention": (_i32, [_vp, _f, _i32, _f, _f, _i32, _f, _f, _i32, _i32, _f, _f, _f, _f]),
    "b200_ApplyContextTypeEmbedding": (_i32, [_vp, _f, _i32, _i32, _f, _i32, _i]),
    "b200_ComputeTimeDiffMatrix": (_i32, [_vp, _i32, _f, _i32, _f]),
    "b200_ComputeMemoryAttentionScores": (_i32, [_vp, _f, _i32, _i32, _i32, _f, _i32, _fl, _f]),
    "b200_ProjectGlobalFeatures": (_i32, [_vp, _f, _i32, _f, _f, _i32, _f]),
    "b200_MeanPoolRows": (_i32, [_vp, _f, _i32, _i32, _f]),
    "b200_ExpandMeanPoolGradient": (_i32, [_vp, _f, _i32, _i32, _i32, _i32, _i32, _f]),
    "b200_SoftmaxVector": (_i32, [_vp, _f, _i32, _f]),
    "b200_SigmoidInPlace": (_i32, [_vp, _f, _i64]),
    "b200_ZeroMatrixColumns": (_i32, [_vp, _f, _i32, _i32, _i32]),
    "b200_VectorUpdateClamped": (_i32, [_vp, _f, _f, _i64, _fl, _fl, _fl]),
    "b200_AccumulateGlobalProjectionGradients": (_i32, [_vp, _f, _i32, _f, _i32, _f, _f]),
    "b200_Matrix3DScaleInPlace": (_i32, [_vp, _f, _i64, _fl]),
    "b200_MatrixSquaredNorm3D": (_i32, [_vp, _f, _i64, _f]),
    "b200_Matrix3DAddInPlace": (_i32, [_vp, _f, _f, _i64]),
    "b200_Matrix3DUpdate": (_i32, [_vp, _f, _f, _i64, _fl]),
    "b200_BackpropOutputProjection": (_i32, [_vp, _f, _f, _f, _f, _f, _i32, _i32, _i32, _f]),
    "b200_BackpropInputProjection": (_i32, [_vp, _f, _i32, _i32, _f, _i32, _i32, _i32, _f, _f, _i32, _i32, _i32]),
    "b200_EmbedTokenIds": (_i32, [_vp, _i, _i32, _i32, _i32, _f, _i32, _i32, _f]),
    "b200_AccumulateTokenEmbeddingGrad": (_i32, [_vp, _f, _i32, _f, _i, _i32, _i32, _i32, _i32]),
    "b200_CrossEntropyLossAndGradient": (_i32, [_vp, _f, _i32, _i32, _i, _i32, _i32, _i32, _f, _f]),
    "b200_MSELossAndGradient": (_i32, [_vp, _f, _i32, _i32, _f, _i32, _i32, _i32, _f, _f]),
    "b200_MatrixSquaredNorm": (_i32, [_vp, _f, _i64, _f]),
    "b200_VectorSquaredNorm": (_i32, [_vp, _f, _i64, _f]),
    "b200_MatrixScaleInPlace": (_i32, [_vp, _f, _i64, _fl]),
    "b200_VectorScaleInPlace": (_i32, [_vp, _f, _i64, _fl]),
    "b200_MatrixUpdate": (_i32, [_vp, _f, _f, _i64, _fl]),
    "b200_VectorUpdate": (_i32, [_vp, _f, _f, _i64, _fl]),
    "b200_FFNForwardBatch": (_i32, [_vp, _f, _i32, _i32, _i, _i, _pp, _pp, _f]),
    "b200_FFNInputGradientBatch": (_i32, [_vp, _f, _f, _i32, _i32, _i, _i, _pp, _pp, _pp, _pp, _f]),
    "b200_lm_param_count": (_i64, [C.POINTER(LMConfig)]),
    "b200_lm_tensor_count": (_i32, [C.POINTER(LMConfig)]),
    "b200_lm_tensor_info": (_i32, [C.POINTER(LMConfig), _i32, C.POINTER(_i64), _i, _i]),
    "b200_lm_create": (_i32, [_vp, C.POINTER(LMConfig), _vp, _vp, _i32, _pp]),
    "b200_lm_destroy": (_i32, [_vp]),
    "b200_lm_upload_params": (_i32, [_vp, _f, _i64, _i64]),
    "b200_lm_download_params": (_i32, [_vp, _f, _i64, _i64]),
    "b200_lm_download_grads": (_i32, [_vp, _f, _i64, _i64]),
    "b200_lm_params_device": (_vp, [_vp]),
    "b200_lm_grads_device": (_vp, [_vp]),
    "b200_lm_set_optimizer": (_i32, [_vp, _i32, _fl, _fl, _fl]),
    "b200_lm_train_step_discrete": (_i32, [_vp, _i, _i, _i32, _fl, _i32, _fl, _i32, _f, _f, _i]),
    "b200_lm_train_step_continuous": (_i32, [_vp, _f, _f, _i, _i, _i32, _fl, _i32, _fl, _i32, _f, _f, _i]),
    "b200_lm_set_grad_ready_callback": (_i32, [_vp, GRAD_READY_FN, _vp]),
    "b200_lm_zero_grads": (_i32, [_vp]),
    "b200_lm_accumulate_discrete": (_i32, [_vp, _i, _i, _i32, _f, _i]),
    "b200_lm_accumulate_continuous": (_i32, [_vp, _f, _f, _i, _i, _i32, _f, _i]),
    "b200_lm_apply_step": (_i32, [_vp, _i32, _fl, _i32, _fl, _i32, _f]),
    "b200_lm_batch_create_discrete": (_i32, [_vp, _i, _i, _i32, _pp]),
    "b200_lm_batch_create_continuous": (_i32, [_vp, _f, _f, _i, _i, _i32, _pp]),
    "b200_lm_batch_destroy": (_i32, [_vp]),
    "b200_lm_accumulate_batch": (_i32, [_vp, _vp, _f, _i]),
    "b200_lm_train_step_batch": (_i32, [_vp, _vp, _fl, _i32, _fl, _i32, _f, _f, _i]),
    "b200_lm_validate_discrete": (_i32, [_vp, _i, _i, _i32, _f, _i]),
    "b200_lm_validate_continuous": (_i32, [_vp, _f, _f, _i, _i, _i32, _f, _i]),
    "b200_lm_download_optimizer_state": (_i32, [_vp, _i32, _f, _i64, _i64]),
    "b200_lm_upload_optimizer_state": (_i32, [_vp, _i32, _f, _i64, _i64]),
    "b200_lm_get_step_index": (_i32, [_vp, _i]),
    "b200_lm_set_step_index": (_i32, [_vp, _i32]),
    "b200_lm_gen_create": (_i32, [_vp, _i32, _pp]),
    "b200_lm_gen_destroy": (_i32, [_vp]),
    "b200_lm_gen_reset": (_i32, [_vp]),
    "b200_lm_gen_length": (_i32, [_vp, _i]),
    "b200_lm_gen_graph_nodes": (_i32, [_vp, _i]),
    "b200_lm_gen_single_kernel": (_i32, [_vp]),
    "b200_lm_gen_set_single_kernel": (_i32, [_vp, _i32]),
    "b200_lm_gen_step": (_i32, [_vp, _i32, _f]),
    "b200_lm_gen_greedy": (_i32, [_vp, _i, _i32, _i32, _i, _i]),
    "b200_lm_get_timings": (_i32, [_vp, _f]),
    "b200_dp_set_nccl_library": (_i32, [C.c_char_p]),
    "b200_dp_set_nccl_max_ctas": (_i32, [_i32]),
    "b200_dp_unique_id": (_i32, [_b]),
    "b200_dp_create_rank": (_i32, [_vp, _b, _i32, _i32, _pp]),
    "b200_dp_destroy": (_i32, [_vp]),
    "b200_dp_shard": (_i32, [_i32, _i32, _i32, _i, _i]),
    "b200_dp_set_deadline_ms": (_i32, [_vp, _i32]),
    "b200_dp_broadcast_params": (_i32, [_vp, _i32]),
    "b200_dp_train_step_discrete": (_i32, [_vp, _i, _i, _i32, _fl, _i32, _fl, _i32, _f, _f, _i]),
    "b200_dp_train_step_continuous": (_i32, [_vp, _f, _f, _i, _i, _i32, _fl, _i32, _fl, _i32, _f, _f, _i]),
    "b200_dp_batch_create_discrete": (_i32, [_vp, _i, _i, _i32, _pp]),
    "b200_dp_batch_create_continuous": (_i32, [_vp, _f, _f, _i, _i, _i32, _pp]),
    "b200_dp_train_step_batch": (_i32, [_vp, _vp, _fl, _i32, _fl, _i32, _f, _f, _i]),
    "b200_dp_get_timings": (_i32, [_vp, _f]),
    "b200_dp_group_create": (_i32, [_i, _i32, C.POINTER(LMConfig), _i32, _i32, _pp]),
    "b200_dp_group_destroy": (_i32, [_vp]),
    "b200_dp_group_last_error": (C.c_char_p, [_vp]),
    "b200_dp_group_size": (_i32, [_vp]),
    "b200_dp_group_trainer": (_vp, [_vp, _i32]),
    "b200_dp_group_set_optimizer": (_i32, [_vp, _i32, _fl, _fl, _fl]),
    "b200_dp_group_upload_params": (_i32, [_vp, _f, _i64, _i64]),
    "b200_dp_group_train_step_discrete": (_i32, [_vp, _i, _i, _i32, _fl, _i32, _fl, _i32, _f, _f, _i]),
    "b200_dp_group_train_step_continuous": (_i32, [_vp, _f, _f, _i, _i, _i32, _fl, _i32, _fl, _i32, _f, _f, _i]),
    "b200_mlp_create": (_i32, [_vp, _i32, _i, _i, _i32, _fl, _fl, _fl, _i32, _pp]),
    "b200_mlp_destroy": (_i32, [_vp]),
    "b200_mlp_upload_layer": (_i32, [_vp, _i32, _f, _f]),
    "b200_mlp_download_layer": (_i32, [_vp, _i32, _f, _f]),
    "b200_mlp_learn_batch": (_i32, [_vp, _f, _f, _i32, _fl, _f, _f, _f]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library (once) and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m callaghandev.build_b200` (needs nvcc). "
                          "There is no CPU fallback.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class B200Error(RuntimeError):
    pass


def check(lib, ctx, rc: int):
    """Map a status code to the Python counterpart of the exception type the reference throws."""
    if rc == OK:
        return
    msg = lib.b200_last_error(ctx).decode("utf-8", "replace") if ctx else "no context"
    if rc in (ERR_INVALID_ARG, ERR_SHAPE):
        raise ValueError(msg)            # ArgumentNullException / ArgumentException
    if rc == ERR_OUT_OF_RANGE:
        raise IndexError(msg)            # ArgumentOutOfRangeException
    if rc == ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise B200Error(f"status {rc}: {msg}")
