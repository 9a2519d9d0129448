/* chessrl_b200 - C ABI of the B200 board-transformer inference engine.
 *
 * The reference (maxlegrec1/ChessRL) has no FFI: its boundary is the PyTorch nn.Module protocol
 * (constructor, forward, state_dict). Each entry point below names the reference interface it stands
 * behind. All pointers are plain device or host addresses; nothing here depends on torch. Functions
 * return 0 on success or a negative crl_status; nothing is printed or thrown; kernels never trap:
 * device-side waits are bounded and report through crl_last_status.
 *
 * Threading: a handle is bound to one CUDA device and is not re-entrant; use one handle per GPU.
 */
#ifndef CHESSRL_B200_H_
#define CHESSRL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct crl_handle crl_handle;

enum crl_status {
  CRL_OK = 0,
  CRL_ERR_INVALID = -1,        /* null pointer, negative size, unknown enum value */
  CRL_ERR_SHAPE = -2,          /* shape / alignment the kernels cannot take */
  CRL_ERR_CUDA = -3,           /* a CUDA call failed (crl_error_detail has the text) */
  CRL_ERR_MISSING_WEIGHT = -4, /* finalize: a state_dict key the configuration needs was never set */
  CRL_ERR_NOT_FINALIZED = -5,
  CRL_ERR_DEVICE_TIMEOUT = -6, /* a bounded device-side wait ran out; see crl_last_status */
  CRL_ERR_WORKSPACE = -7,      /* workspace too small */
  CRL_ERR_UNSUPPORTED = -8
};

enum { CRL_LN_POST = 0, CRL_LN_PRE = 1 };
enum { CRL_ACT_GELU = 1, CRL_ACT_MISH = 2 };
enum { CRL_FFN_ACT_END = 0, CRL_FFN_ACT_MID = 1 };
enum { CRL_BIAS_NONE = 0, CRL_BIAS_CAUSAL = 1, CRL_BIAS_RELPOS = 2, CRL_BIAS_SMOLGEN = 3 };
enum { CRL_POLICY_NONE = 0, CRL_POLICY_DENSE4096 = 1, CRL_POLICY_GATHER1858 = 2, CRL_POLICY_LM_HEAD = 3 };
enum { CRL_VALUE_NONE = 0, CRL_VALUE_WDL = 1, CRL_VALUE_WDL_Q = 2 };
enum { CRL_DTYPE_F16 = 0, CRL_DTYPE_F8E4M3 = 1, CRL_DTYPE_I8 = 2 };
enum { CRL_LAYOUT_NHWC_F32 = 0, CRL_LAYOUT_NHWC_F16 = 1, CRL_LAYOUT_NCHW_F16 = 2, CRL_LAYOUT_NCHW_F32 = 3,
       CRL_LAYOUT_PACKED104 = 4 };
/* CRL_LAYOUT_PACKED104 (112-plane networks only): CRL_PACKED104_BYTES per position, the plane block of the lc0
 * training record as the reference reads it (LeelaData/show_value_head_ground_truth.py:58-88,191-203):
 *   bytes [0,832)  104 planes x 8 bytes; byte r of a plane = rank r as seen by the side to move (r 0 = its first
 *                  rank), bit (7 - f) of that byte = file f (the order numpy.unpackbits yields);
 *   byte 832..835  castling rights: ours O-O-O, ours O-O, theirs O-O-O, theirs O-O  -> planes 104..107;
 *   byte 836       non-zero = Black to move                                          -> plane 108;
 *   byte 837       half-move clock c, plane 109 = min(c/100, 1) (0 for networks without that plane);
 *   byte 838, 839  ignored (plane 110 is empty, plane 111 is all ones).
 * The library expands it on the device into the token rows of the embedding GEMM. */
#define CRL_PACKED104_BYTES 840
enum { CRL_MASK_NONE = 0, CRL_MASK_BITS = 1, CRL_MASK_ADDITIVE = 2, CRL_MASK_FROM_RECORDS = 3 };
/* CRL_MASK_FROM_RECORDS (input layout CRL_LAYOUT_PACKED104, 1858-move gather head): the library generates the
 * legal moves of every position on the device from its packed record and masks like CRL_MASK_BITS; legal_mask
 * is ignored. Stands for the python-chess loop of model_bis.py:373-380 / pgn_to_input_data_decoder.py:35-42. */
enum { CRL_OUT_F32 = 0, CRL_OUT_F16 = 1 };
enum { CRL_VOCAB_NATIVE = 0, CRL_VOCAB_RL1929 = 1 };

/* Network description. Stands for the reference constructors
 *   BT4(num_layers, d_model, d_ff, num_heads)      new_paradigm/value.py:122, value_q.py:122
 * (planes 19 / 112 are fixed per class there: value.py:132, value_q.py:132) and, with ln_mode PRE, bias_mode CAUSAL,
 * pos_embed and CRL_POLICY_LM_HEAD, the board-only path of GPT(GPTConfig) (model_bis.py:127-156, 358-370), whose
 * weights are passed under the BT4 key names (the Python module renames them); the remaining fields select
 * the variants of the target specification (Mish, activation position, pre-LN, smolgen, gather policy)
 * and the arithmetic type of the QKV / out-proj / FFN GEMMs. */
typedef struct crl_config {
  int32_t planes;
  int32_t d_model;
  int32_t n_layers;
  int32_t n_heads;
  int32_t d_ff;
  int32_t ln_mode;
  int32_t act;
  int32_t ffn_act_pos;
  int32_t bias_mode;
  int32_t policy_mode;
  int32_t value_mode;
  int32_t dtype;
  int32_t smolgen_compress; /* 32 */
  int32_t smolgen_hidden;   /* 256 */
  int32_t smolgen_gen;      /* 256 */
  int32_t chunk;            /* positions processed per pass over the layers; 0 = library default */
  int32_t pos_embed;        /* 1: add the `pe` table [>=64, d] to the embedded tokens (model_bis.py:363-366) */
  int32_t lm_vocab;         /* CRL_POLICY_LM_HEAD: rows of lm_head.weight (1929 in the reference's scripts) */
  int32_t fuse_layernorm;   /* where the per-block LayerNorms of post-LN networks run. CRL_FUSE_LN_AUTO (0): the library
                               chooses (CRL_FUSE_LN_OUT where it applies, separate row passes elsewhere); CRL_FUSE_LN_OUT:
                               large passes normalise inside the out-projection / ff2 GEMM kernels that produce the rows,
                               so x + sublayer(x) never crosses HBM (equal to the separate passes within f16 rounding;
                               measured 4-6 % faster on B200 for FP16 / FP8, which is where AUTO uses it; no gain for INT8); CRL_FUSE_LN_ON: inside the ff1 / QKV GEMM kernels
                               that consume the rows (same bits as the separate passes, no measured gain);
                               CRL_FUSE_LN_OFF: always separate row passes */
  int32_t precision;        /* bit mask of CRL_PREC_*; 0 = the fastest arithmetic of the chosen dtype */
} crl_config;

enum { CRL_FUSE_LN_AUTO = 0, CRL_FUSE_LN_ON = 1, CRL_FUSE_LN_OUT = 2, CRL_FUSE_LN_OFF = 3 };
/* Precision switches. The FP8 engine (model_fp8.py:43-140: per-tensor e4m3 linears, everything else in higher
 * precision) takes several shortcuts around its e4m3 GEMMs by default; each bit takes one of them back, so that its
 * cost in accuracy and speed can be measured on its own:
 *   QKV_F16        Q, K, V and the smolgen bias tile cross HBM as f16 (default: e4m3 with one scale each)
 *   LN_F32         LayerNorm with two-pass fp32 statistics and fp32 affine (default on large passes: one-pass
 *                  statistics, f16 affine); also keeps the LayerNorms out of the GEMM kernels
 *   MISH_F32       Mish of the ff1 epilogue in fp32 (default for e4m3 outputs: packed f16 pairs)
 *   ATTN_F32       attention scores accumulated and soft-maxed in fp32 (default: f16 accumulate, packed-f16
 *                  softmax); implies QKV_F16
 *   FFN_F16        ff1 / ff2 on f16 operands (a mixed engine: only the attention GEMMs stay e4m3)
 *   ATTN_GEMM_F16  QKV projection / out-projection on f16 operands (only the FFN GEMMs stay e4m3)
 * LN_F32 and ATTN_F32 also apply to the FP16 and INT8 engines. */
enum { CRL_PREC_QKV_F16 = 1, CRL_PREC_LN_F32 = 2, CRL_PREC_MISH_F32 = 4, CRL_PREC_ATTN_F32 = 8, CRL_PREC_FFN_F16 = 16,
       CRL_PREC_ATTN_GEMM_F16 = 32 };

/* One forward call. Stands for BT4.forward / get_batch_position_values (new_paradigm/value.py:155-212,
 * 275-317) and the server's bt4(X)['policy'] + mask + softmax (Leela/server.py:28-34,54-56).
 * Every pointer is a DEVICE pointer for crl_forward and a HOST pointer for crl_forward_host. */
typedef struct crl_io {
  const void* planes;      /* input planes in `layout`, `batch` positions */
  int32_t layout;
  int64_t batch;
  const void* legal_mask;  /* nullable. BITS: u8 [batch, mask_stride] bit m of a row = move m legal,
                              applied as logits + (1-bit)*(-999) (model_bis.py:383); ADDITIVE: f32
                              [batch, mask_stride] added to the logits (server.py:56) */
  int32_t mask_mode;
  int64_t mask_stride;     /* bytes per row (BITS) or floats per row (ADDITIVE) */
  void* policy_out;        /* nullable. [batch, policy_stride] logits (or probabilities) */
  int32_t policy_dtype;    /* CRL_OUT_F32 / CRL_OUT_F16 */
  int32_t policy_softmax;  /* 1: softmax over the (masked) logits */
  int64_t policy_stride;   /* elements per row, >= number of moves */
  float* wdl_out;          /* nullable. [batch, 3] */
  int32_t wdl_softmax;     /* 1: probabilities (value.py:271), 0: raw logits */
  float* q_out;            /* nullable. [batch] tanh value (value_q.py:430-464), value_mode WDL_Q only */
  void* workspace;         /* device scratch, >= crl_workspace_bytes(h, batch) (ignored by _host) */
  size_t workspace_bytes;
  void* stream;            /* cudaStream_t, may be null (default stream) */
  int32_t policy_vocab;    /* CRL_VOCAB_NATIVE: the head's own move list. CRL_VOCAB_RL1929 (gather head only): the
                              1858 Leela entries scattered into zero-filled rows of 1929 like map_leela_to_rl
                              (Leela/compare_policy.py:493-523); policy_stride >= 1929 */
  const uint8_t* black_rows; /* nullable, [batch]: 1 = Black to move, the row goes through the rank-mirror table;
                              0 / null = White, identity (the reference alternates rows: first_is_white) */
  int32_t* move_out;       /* nullable, [batch]: the move chosen from each policy row on the device, as an index
                              into that row (model_bis.py:385-394: temperature 0 -> arg-max, else a draw from
                              softmax(logits / T)). crl_forward needs policy_out as well (the rows it reads);
                              crl_forward_host may leave policy_out null and then copies only the indices back */
  const float* move_uniform; /* nullable, [batch] numbers in [0,1): the draw is the first index whose cumulative
                              probability exceeds move_uniform[b] (the caller owns the random stream, so a run
                              can be reproduced); null = arg-max (lowest index on ties) */
  float move_temperature;  /* T above; 0 = arg-max */
} crl_io;

/* Constructor: replaces BT4.__init__ (value.py:122-153). The device must be a B200 (sm_100). */
int crl_create(const crl_config* cfg, int device, crl_handle** out);
void crl_destroy(crl_handle* h);

/* load_state_dict: one call per state_dict entry, with the reference's key names
 * (layers.{i}.attention.query_proj.weight, ..., linear1.weight, ma_gating.a, value_head.dense1.weight;
 * listed by crl_required_key). `data` is f32, host or device memory, row-major, `numel` elements. */
int crl_set_weight(crl_handle* h, const char* key, const float* data, int64_t numel);
/* Number of keys the configuration needs, and the i-th key (null past the end). */
int crl_num_required_keys(const crl_handle* h);
const char* crl_required_key(const crl_handle* h, int i);
/* Repack once: f16 (and e4m3 / int8 + scales) device copies, fused QKV, folded positional tables. */
int crl_finalize(crl_handle* h);

/* FP8 only: per-tensor activation scales from a calibration batch (device pointer), the static
 * equivalent of the reference's delayed scaling recipe (pretrain_fp8.py:75-79: E4M3, margin 0). The same pass
 * measures the mean input of every FP8 GEMM and folds the mean effect of the weights' e4m3 rounding into the
 * GEMM's bias (the FP16 / calibration path keeps the original biases). */
int crl_calibrate(crl_handle* h, const void* planes, int32_t layout, int64_t batch, void* workspace,
                  size_t workspace_bytes, void* stream);

size_t crl_workspace_bytes(const crl_handle* h, int64_t batch);
int crl_num_moves(const crl_handle* h); /* 1929 (dense policy), 1858 (gather policy), lm_vocab (LM head), 0 (none) */

int crl_forward(crl_handle* h, const crl_io* io);
/* Same call with HOST buffers: copies the planes (and mask) to the device, runs, copies results back and
 * synchronises. Staging buffers and workspace are owned by the handle and grow on demand. */
int crl_forward_host(crl_handle* h, const crl_io* io);

/* crl_forward for callers that must not allocate device memory (no counterpart in the reference, which
 * leaves all memory management to PyTorch). Think of a search or serving thread that runs beside a
 * framework which has already reserved the GPU's memory for its own caching allocator, or of a
 * latency-critical loop in which the device-wide synchronisation hidden in cudaMalloc / cudaFree would
 * stall every other stream: such a caller passes device pointers for planes, mask and outputs as usual and
 * leaves io->workspace unset; the scratch comes from a CRL_STATIC_SCRATCH_BYTES array inside the
 * library's device image (each GPU that loads the library holds it until the process exits). The call
 * itself makes no cudaMalloc / cudaFree and uses no allocating library.
 *   - Limit: crl_workspace_bytes(h, io->batch) must not exceed CRL_STATIC_SCRATCH_BYTES (a few dozen
 *     positions of a 1024-wide network, a few hundred of a 256-wide one); larger batches are refused with
 *     CRL_ERR_WORKSPACE and crl_error_detail() says how many bytes were needed.
 *   - The first call on each device looks up the array's device address; make that first call outside
 *     any stream capture.
 *   - All calls (all handles on a device) share the one array, and it keeps what the last call left in
 *     it. The forward pass writes every scratch buffer before reading it, so nothing needs clearing, but
 *     two calls whose kernels overlap on the GPU (different streams, different handles) race on it:
 *     serialise them. */
#define CRL_STATIC_SCRATCH_BYTES (64u << 20)
int crl_forward_static(crl_handle* h, const crl_io* io);

/* Reads and clears the device status word (0 = fine; 101 / 102 / 103 = a bounded wait of the GEMM's producer /
 * MMA / epilogue role ran out, 104 = shared memory less aligned than the GEMM's layout needs, 113 = a bounded wait
 * of the attention kernel on its tile loads ran out). Synchronises the device. */
int crl_last_status(crl_handle* h, int* device_status_word);
/* Number of kernels the last crl_forward launched. */
int64_t crl_last_launch_count(const crl_handle* h);
/* Per-kernel timing for roofline reports (no reference counterpart; the reference has no profiler hooks,
 * only time.time() deltas in Leela/test_inference.py:16-33). While enabled, every launch of crl_forward is
 * bracketed by CUDA events on the launch stream. crl_profile(h, 1) also clears earlier records.
 * Categories: 0 tcgen05 GEMMs, 1 attention, 2 LayerNorm, 3 policy scores. crl_profile_read synchronises
 * and returns summed device time, algorithmic FLOPs and algorithmic bytes of that category. */
int crl_profile(crl_handle* h, int enable);
int crl_profile_read(crl_handle* h, int category, double* ms, double* flops, double* bytes, int64_t* launches);
/* The index-th recorded launch (in launch order): its category, device time, algorithmic FLOPs and bytes, and
 * for GEMMs {M, N, K, kind} in mnk_kind[4] (zeros otherwise). CRL_ERR_INVALID past the last record. */
int crl_profile_entry(crl_handle* h, int64_t index, int* category, double* ms, double* flops, double* bytes,
                      int* mnk_kind);
const char* crl_error_detail(const crl_handle* h);
const char* crl_strerror(int status);

/* Operator-level entry (tests, tuning): C = act(alpha * A W^T + bias) + residual on device buffers.
 * kind: CRL_DTYPE_* of A and W (f16, e4m3, int8); out_dtype: 0 f16, 1 f32, 2 e4m3. Stands for one
 * nn.Linear call (e.g. new_paradigm/value.py:65-67). */
int crl_linear(int kind, const void* a, int64_t lda, const void* w, int64_t ldw, void* c, int64_t ldc,
               int out_dtype, int64_t m, int64_t n, int64_t k, const float* bias, const void* residual,
               int64_t ldr, float alpha, int act, int* device_status, void* stream);

/* The same operator with every epilogue term the engine's quantised paths use (one nn.Linear under the
 * per-tensor FP8 recipe of model_fp8.py:43-45 / pretrain_fp8.py:75-79, or its W8A8 twin):
 *   C = out_scale * ( act( alpha * row_scale[m] * col_scale[n] * (A W^T)[m,n] + bias[n] ) + residual[m % res_mod, n] )
 * row_scale [M] and col_scale [N] f32 are nullable (per-token / per-output-channel de-quantisation); res_mod 0 means
 * residual[m, n]; out_scale applies to e4m3 outputs only (the next GEMM's input multiplier). */
typedef struct crl_linear_args {
  int32_t kind;            /* CRL_DTYPE_* of A and W */
  int32_t out_dtype;       /* 0 f16, 1 f32, 2 e4m3 */
  const void* a; int64_t lda;
  const void* w; int64_t ldw;
  void* c; int64_t ldc;
  int64_t m, n, k;
  const float* bias;
  const void* residual; int64_t ldr; int32_t res_mod;
  float alpha;
  int32_t act;             /* 0 none, 1 GELU, 2 Mish, 3 ReLU */
  float out_scale;
  const float* row_scale;
  const float* col_scale;
  int* device_status;      /* >= 4 ints of device memory, zero before the call */
  void* stream;
  /* Optional fused LayerNorm (all null / 0 = off): A is LayerNorm(ln_y) * ln_weight + ln_bias (eps 1e-5, the
   * nn.LayerNorm in front of a Linear: new_paradigm/value.py:58-75), computed inside the GEMM kernel. ln_y is
   * [m, k] f16 with row pitch k; ln_weight / ln_bias are [k] f16; the normalised rows are written to ln_x ([m, k]
   * f16, required for f16 operands) and ln_x8 ([m, k] e4m3 of the rows times ln_out8_scale, required for e4m3
   * operands), and `a` must point at the one the GEMM consumes. Needs m >= 256 x the SM count, k <= 1024,
   * n >= 256 and a 16-bit or 8-bit output; CRL_ERR_UNSUPPORTED otherwise. */
  const void* ln_y;
  const void* ln_weight;
  const void* ln_bias;
  void* ln_x;
  void* ln_x8;
  float ln_out8_scale;
  /* Optional LayerNorm of the OUTPUT rows (all null / 0 = off): c = LayerNorm(acc + bias + residual) * lno_weight +
   * lno_bias over the n columns (eps 1e-5: the post-LN block's norm1 / norm2 behind its out-projection / second FFN
   * linear, Leela/attn.py:478-486), computed inside the GEMM kernel; `residual` is required and may be `c` itself.
   * lno_weight / lno_bias are [n] f16; lno_x8 ([m, n] e4m3 of the rows times lno_out8_scale) is optional; lno_scratch
   * is device memory of 32 KiB * ceil(m / 256) the kernel exchanges row sums through. Needs an
   * f16 output, n a multiple of 256 up to 1024 and at least half the SM count of 256 x 256 tiles;
   * CRL_ERR_UNSUPPORTED otherwise. */
  const void* lno_weight;
  const void* lno_bias;
  void* lno_x8;
  float lno_out8_scale;
  void* lno_scratch;
  float* lno_qscale;       /* int8 operands only: lno_x8 receives the per-token int8 copy of the rows (W8A8 activations:
                              row maximum / 127 as the scale, written here, [m] f32); required with lno_x8 then */
} crl_linear_args;
int crl_linear_ex(const crl_linear_args* args);

/* ---- host-side input producers (no GPU needed) ------------------------------------------------------------
 * The reference builds its inputs with python-chess; these entry points are the library's own rules
 * implementation (validated by perft counts and against the test oracle). */

/* Number of leaf nodes of the legal-move tree of depth 1..8 below `fen` (null = start position). */
int crl_perft(const char* fen, int depth, uint64_t* nodes);
/* fen_to_tensor (utils/fen_encoder.py:5-38): FEN -> [8,8,19] f32, row 0 = rank 8. */
int crl_fen_to_planes19(const char* fen, float* out);
/* Legal-move bitset over the 1929 vocabulary (242 bytes, bit m = entry m legal; a knight promotion sets the
 * 4-character move), the index set of model_bis.py:373-380. */
int crl_legal_mask_1929(const char* fen, uint8_t* bits);
/* Seeded random playouts from the start position (plies ~ U{0..max_plies}, uniformly random legal moves, a
 * finished game restarts): positions first .. first+count-1 of the stream `seed`. Every output is optional:
 *   planes112_f16 [count,64,112]  the server input in token-major f16 (history of 8 boards in the mover's view,
 *                                 Leela/gen_TC.py:255-319 + pgn_to_input_data_decoder.py:61-72 + ustotheirs.py:4-23;
 *                                 plane 109 = halfmove/100 when rule50_plane is set, else empty)
 *   planes19_f32  [count,8,8,19]  utils/fen_encoder.py:5-38
 *   legal1858     [count,233]     bitset over the Leela entries from the mover's view (pgn_to_input_data_decoder.py:35-42)
 *   legal1929     [count,242]     bitset over the 1929 vocabulary (model_bis.py:373-380)
 *   black         [count]         1 = Black to move
 *   fens          [count,96]      zero-terminated FEN strings */
int crl_playout_positions(uint64_t seed, int64_t first, int64_t count, int32_t max_plies, int32_t rule50_plane,
                          uint16_t* planes112_f16, float* planes19_f32, uint8_t* legal1858, uint8_t* legal1929,
                          uint8_t* black, char* fens);

/* Packs `count` positions of 112 planes in token-major order ([count,64,112]; layout CRL_LAYOUT_NHWC_F16 or
 * CRL_LAYOUT_NHWC_F32, host memory) into CRL_LAYOUT_PACKED104 records. CRL_ERR_INVALID when a plane cannot be
 * represented: a piece plane holding something other than 0/1, an auxiliary plane that is not constant over
 * the board, a plane-109 value that is not min(c/100, 1) for an integer c, plane 110 not empty or plane 111
 * not all ones. */
int crl_pack_planes104(const void* planes, int32_t layout, int64_t count, uint8_t* packed);

/* The legal moves of `fen` (ordered by from-square, to-square, promotion piece) with the positions they lead to:
 * the loop of calculate_move_values (new_paradigm/value.py:319-345: push, fen, pop for every legal move). Optional
 * outputs: ucis [max_moves,8], fens [max_moves,96] (zero-terminated), planes19_out [max_moves,8,8,19] f32
 * (fen_to_tensor of every successor). *count = number of legal moves; CRL_ERR_SHAPE if it exceeds max_moves. */
int crl_successors(const char* fen, int32_t max_moves, char* ucis, char* fens, float* planes19_out, int32_t* count);

/* Replays a game from the start position and emits the positions after first_ply .. first_ply+count-1 moves as
 * packed records with their history of up to 8 boards - the input side of list_uci_to_input
 * (Leela/pgn_to_input_data_decoder.py:14-78). `moves`: space-separated SAN (what the reference parses: board.parse_san,
 * line 24) or UCI tokens; all of them are checked and played, so first_ply + count - 1 <= number of moves.
 * Optional outputs: packed [count,840], black [count] (1 = Black to move), legal1858 [count,233], fens [count,96].
 * A token that does not select exactly one legal move: CRL_ERR_INVALID and its index in *bad_move. */
int crl_game_records(const char* moves, int32_t first_ply, int32_t count, int32_t rule50_plane, uint8_t* packed,
                     uint8_t* black, uint8_t* legal1858, char* fens, int32_t* bad_move);

/* Legal-move bitsets on the device: `count` packed records (device memory, CRL_LAYOUT_PACKED104) -> bits
 * [count, stride] (device memory, stride >= 233; bit m of a row = entry m of the 1858-move list legal in the
 * mover's view, a knight promotion sets the plain from-to entry). Same rows as crl_playout_positions' legal1858. */
int crl_legal_masks_packed104(crl_handle* h, const void* packed, int64_t count, uint8_t* bits, int64_t stride, void* stream);

/* Move vocabulary (utils/vocab.py:9-438): writes the UCI string of entry `index` of the 1929-entry
 * list into buf (>= 16 bytes); entries < 1858 are the Leela list. Returns 0, or CRL_ERR_INVALID. */
int crl_vocab_move(int index, char* buf);
/* Index in the 1929 list of the rank-mirrored Leela move `leela_index` (compare_policy.py:465-483). */
int crl_vocab_mirror_index(int leela_index);

#ifdef __cplusplus
}
#endif
#endif /* CHESSRL_B200_H_ */
