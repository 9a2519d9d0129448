"""ctypes binding of libchessrl_b200.so (the C ABI in include/chessrl_b200.h).

There is no CPU fallback: if the library is missing this module raises at import of the symbols, and
every compute entry point needs a B200.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# CHESSRL_B200_LIB names another build of the same library (e.g. one compiled with different tuning macros)
LIB_PATH = os.environ.get("CHESSRL_B200_LIB") or os.path.join(HERE, "libchessrl_b200.so")

# enums of include/chessrl_b200.h
LN_POST, LN_PRE = 0, 1
ACT_GELU, ACT_MISH = 1, 2
FFN_ACT_END, FFN_ACT_MID = 0, 1
BIAS_NONE, BIAS_CAUSAL, BIAS_RELPOS, BIAS_SMOLGEN = 0, 1, 2, 3
POLICY_NONE, POLICY_DENSE4096, POLICY_GATHER1858, POLICY_LM_HEAD = 0, 1, 2, 3
VALUE_NONE, VALUE_WDL, VALUE_WDL_Q = 0, 1, 2
DTYPE_F16, DTYPE_F8E4M3, DTYPE_I8 = 0, 1, 2
LAYOUT_NHWC_F32, LAYOUT_NHWC_F16, LAYOUT_NCHW_F16, LAYOUT_NCHW_F32, LAYOUT_PACKED104 = 0, 1, 2, 3, 4
PACKED104_BYTES = 840
MASK_NONE, MASK_BITS, MASK_ADDITIVE, MASK_FROM_RECORDS = 0, 1, 2, 3
OUT_F32, OUT_F16 = 0, 1
VOCAB_NATIVE, VOCAB_RL1929 = 0, 1
FUSE_LN_AUTO, FUSE_LN_ON, FUSE_LN_OUT, FUSE_LN_OFF = 0, 1, 2, 3
PREC_QKV_F16, PREC_LN_F32, PREC_MISH_F32, PREC_ATTN_F32, PREC_FFN_F16, PREC_ATTN_GEMM_F16 = 1, 2, 4, 8, 16, 32

EXPORTS = [
    "crl_create", "crl_destroy", "crl_set_weight", "crl_num_required_keys", "crl_required_key", "crl_finalize",
    "crl_calibrate", "crl_workspace_bytes", "crl_num_moves", "crl_forward", "crl_forward_host", "crl_last_status",
    "crl_last_launch_count", "crl_error_detail", "crl_strerror", "crl_linear", "crl_linear_ex", "crl_vocab_move",
    "crl_vocab_mirror_index", "crl_profile", "crl_profile_read", "crl_profile_entry", "crl_forward_static", "crl_perft", "crl_fen_to_planes19", "crl_legal_mask_1929",
    "crl_playout_positions", "crl_pack_planes104", "crl_legal_masks_packed104", "crl_game_records", "crl_successors",
]


class Config(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "planes", "d_model", "n_layers", "n_heads", "d_ff", "ln_mode", "act", "ffn_act_pos", "bias_mode",
        "policy_mode", "value_mode", "dtype", "smolgen_compress", "smolgen_hidden", "smolgen_gen", "chunk", "pos_embed",
        "lm_vocab", "fuse_layernorm", "precision")]


class IO(ctypes.Structure):
    _fields_ = [
        ("planes", ctypes.c_void_p), ("layout", ctypes.c_int32), ("batch", ctypes.c_int64),
        ("legal_mask", ctypes.c_void_p), ("mask_mode", ctypes.c_int32), ("mask_stride", ctypes.c_int64),
        ("policy_out", ctypes.c_void_p), ("policy_dtype", ctypes.c_int32), ("policy_softmax", ctypes.c_int32),
        ("policy_stride", ctypes.c_int64),
        ("wdl_out", ctypes.c_void_p), ("wdl_softmax", ctypes.c_int32),
        ("q_out", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("stream", ctypes.c_void_p),
        ("policy_vocab", ctypes.c_int32), ("black_rows", ctypes.c_void_p),
        ("move_out", ctypes.c_void_p), ("move_uniform", ctypes.c_void_p), ("move_temperature", ctypes.c_float),
    ]


class LinearArgs(ctypes.Structure):
    """Mirror of `crl_linear_args` (include/chessrl_b200.h)."""
    _fields_ = [
        ("kind", ctypes.c_int32), ("out_dtype", ctypes.c_int32),
        ("a", ctypes.c_void_p), ("lda", ctypes.c_int64),
        ("w", ctypes.c_void_p), ("ldw", ctypes.c_int64),
        ("c", ctypes.c_void_p), ("ldc", ctypes.c_int64),
        ("m", ctypes.c_int64), ("n", ctypes.c_int64), ("k", ctypes.c_int64),
        ("bias", ctypes.c_void_p),
        ("residual", ctypes.c_void_p), ("ldr", ctypes.c_int64), ("res_mod", ctypes.c_int32),
        ("alpha", ctypes.c_float), ("act", ctypes.c_int32), ("out_scale", ctypes.c_float),
        ("row_scale", ctypes.c_void_p), ("col_scale", ctypes.c_void_p),
        ("device_status", ctypes.c_void_p), ("stream", ctypes.c_void_p),
        ("ln_y", ctypes.c_void_p), ("ln_weight", ctypes.c_void_p), ("ln_bias", ctypes.c_void_p),
        ("ln_x", ctypes.c_void_p), ("ln_x8", ctypes.c_void_p), ("ln_out8_scale", ctypes.c_float),
        ("lno_weight", ctypes.c_void_p), ("lno_bias", ctypes.c_void_p), ("lno_x8", ctypes.c_void_p),
        ("lno_out8_scale", ctypes.c_float), ("lno_scratch", ctypes.c_void_p), ("lno_qscale", ctypes.c_void_p),
    ]


_lib = None


def load():
    """Load the shared library (once) and declare the signatures. Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m chessrl_b200.build` (needs nvcc). "
            "chessrl_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
    lib.crl_create.argtypes = [ctypes.POINTER(Config), ctypes.c_int, ctypes.POINTER(vp)]
    lib.crl_create.restype = ctypes.c_int
    lib.crl_destroy.argtypes = [vp]
    lib.crl_destroy.restype = None
    lib.crl_set_weight.argtypes = [vp, ctypes.c_char_p, vp, i64]
    lib.crl_set_weight.restype = ctypes.c_int
    lib.crl_num_required_keys.argtypes = [vp]
    lib.crl_num_required_keys.restype = ctypes.c_int
    lib.crl_required_key.argtypes = [vp, ctypes.c_int]
    lib.crl_required_key.restype = ctypes.c_char_p
    lib.crl_finalize.argtypes = [vp]
    lib.crl_finalize.restype = ctypes.c_int
    lib.crl_calibrate.argtypes = [vp, vp, i32, i64, vp, ctypes.c_size_t, vp]
    lib.crl_calibrate.restype = ctypes.c_int
    lib.crl_workspace_bytes.argtypes = [vp, i64]
    lib.crl_workspace_bytes.restype = ctypes.c_size_t
    lib.crl_num_moves.argtypes = [vp]
    lib.crl_num_moves.restype = ctypes.c_int
    lib.crl_forward.argtypes = [vp, ctypes.POINTER(IO)]
    lib.crl_forward.restype = ctypes.c_int
    lib.crl_forward_host.argtypes = [vp, ctypes.POINTER(IO)]
    lib.crl_forward_host.restype = ctypes.c_int
    lib.crl_forward_static.argtypes = [vp, ctypes.POINTER(IO)]
    lib.crl_forward_static.restype = ctypes.c_int
    lib.crl_last_status.argtypes = [vp, ctypes.POINTER(ctypes.c_int)]
    lib.crl_last_status.restype = ctypes.c_int
    lib.crl_last_launch_count.argtypes = [vp]
    lib.crl_last_launch_count.restype = i64
    lib.crl_profile.argtypes = [vp, ctypes.c_int]
    lib.crl_profile.restype = ctypes.c_int
    lib.crl_profile_read.argtypes = [vp, ctypes.c_int, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double),
                                     ctypes.POINTER(ctypes.c_double), ctypes.POINTER(i64)]
    lib.crl_profile_read.restype = ctypes.c_int
    lib.crl_profile_entry.argtypes = [vp, i64, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_double),
                                      ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double),
                                      ctypes.POINTER(ctypes.c_int * 4)]
    lib.crl_profile_entry.restype = ctypes.c_int
    lib.crl_error_detail.argtypes = [vp]
    lib.crl_error_detail.restype = ctypes.c_char_p
    lib.crl_strerror.argtypes = [ctypes.c_int]
    lib.crl_strerror.restype = ctypes.c_char_p
    lib.crl_linear.argtypes = [ctypes.c_int, vp, i64, vp, i64, vp, i64, ctypes.c_int, i64, i64, i64, vp, vp, i64,
                               ctypes.c_float, ctypes.c_int, vp, vp]
    lib.crl_linear.restype = ctypes.c_int
    lib.crl_linear_ex.argtypes = [ctypes.POINTER(LinearArgs)]
    lib.crl_linear_ex.restype = ctypes.c_int
    lib.crl_perft.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(ctypes.c_uint64)]
    lib.crl_perft.restype = ctypes.c_int
    lib.crl_fen_to_planes19.argtypes = [ctypes.c_char_p, vp]
    lib.crl_fen_to_planes19.restype = ctypes.c_int
    lib.crl_legal_mask_1929.argtypes = [ctypes.c_char_p, vp]
    lib.crl_legal_mask_1929.restype = ctypes.c_int
    lib.crl_playout_positions.argtypes = [ctypes.c_uint64, i64, i64, i32, i32, vp, vp, vp, vp, vp, vp]
    lib.crl_playout_positions.restype = ctypes.c_int
    lib.crl_pack_planes104.argtypes = [vp, i32, i64, vp]
    lib.crl_pack_planes104.restype = ctypes.c_int
    lib.crl_legal_masks_packed104.argtypes = [vp, vp, i64, vp, i64, vp]
    lib.crl_legal_masks_packed104.restype = ctypes.c_int
    lib.crl_game_records.argtypes = [ctypes.c_char_p, i32, i32, i32, vp, vp, vp, vp, vp]
    lib.crl_game_records.restype = ctypes.c_int
    lib.crl_successors.argtypes = [ctypes.c_char_p, i32, vp, vp, vp, vp]
    lib.crl_successors.restype = ctypes.c_int
    lib.crl_vocab_move.argtypes = [ctypes.c_int, ctypes.c_char_p]
    lib.crl_vocab_move.restype = ctypes.c_int
    lib.crl_vocab_mirror_index.argtypes = [ctypes.c_int]
    lib.crl_vocab_mirror_index.restype = ctypes.c_int
    _lib = lib
    return lib


class CrlError(RuntimeError):
    def __init__(self, code, detail=""):
        self.code = code
        msg = load().crl_strerror(code).decode()
        super().__init__(f"chessrl_b200 error {code} ({msg})" + (f": {detail}" if detail else ""))
