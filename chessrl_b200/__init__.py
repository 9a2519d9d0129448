"""chessrl_b200: B200-native forward pass of the ChessRL board transformer (hand-written sm_100a CUDA
behind a C ABI, see include/chessrl_b200.h)."""
from ._lib import (CrlError, LN_POST, LN_PRE, ACT_GELU, ACT_MISH, FFN_ACT_END, FFN_ACT_MID, BIAS_NONE, BIAS_CAUSAL,
                   BIAS_RELPOS, BIAS_SMOLGEN, POLICY_NONE, POLICY_DENSE4096, POLICY_GATHER1858, VALUE_NONE, VALUE_WDL,
                   VALUE_WDL_Q, DTYPE_F16, DTYPE_F8E4M3, DTYPE_I8, MASK_NONE, MASK_BITS, MASK_ADDITIVE, MASK_FROM_RECORDS,
                   FUSE_LN_AUTO, FUSE_LN_OFF, FUSE_LN_ON, FUSE_LN_OUT, PREC_QKV_F16, PREC_LN_F32, PREC_MISH_F32, PREC_ATTN_F32, PREC_FFN_F16,
                   PREC_ATTN_GEMM_F16)
from .engine import Engine, EngineConfig
from .modules import BoardTransformer, BT4, BT4Planes19, BT4Baseline, GPT, GPTConfig

__all__ = ["Engine", "EngineConfig", "BoardTransformer", "BT4", "BT4Planes19", "BT4Baseline", "GPT", "GPTConfig", "CrlError"]
