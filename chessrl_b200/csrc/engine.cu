// C ABI of the engine: handle, weight repacking and the forward pass that strings the kernels
// together. See include/chessrl_b200.h for the contract of every entry point.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/chessrl_b200.h"
#include "attention.cuh"
#include "attention_tma.cuh"
#include "gemm_launch.cuh"
#include "policy.cuh"
#include "rows.cuh"
#include "vocab.h"
#include "movegen.cuh"

using namespace crl;

namespace {

constexpr float kFp8Max = 448.0f;

struct LayerW {
  __half *wqkv = nullptr, *pos = nullptr, *u = nullptr, *v = nullptr, *wo = nullptr, *wff1 = nullptr, *wff2 = nullptr;
  float *bqkv = nullptr, *bo = nullptr, *bff1 = nullptr, *bff2 = nullptr;
  float *ln1w = nullptr, *ln1b = nullptr, *ln2w = nullptr, *ln2b = nullptr;
  __half *ln1w16 = nullptr, *ln1b16 = nullptr, *ln2w16 = nullptr, *ln2b16 = nullptr;   // f16 copies for the GEMM-fused LayerNorm
  __half *sg_wc = nullptr, *sg_w1 = nullptr, *sg_w2 = nullptr;
  float *sg_b1 = nullptr, *sg_b2 = nullptr, *sg_ln1w = nullptr, *sg_ln1b = nullptr, *sg_ln2w = nullptr, *sg_ln2b = nullptr;
  // FP8: e4m3 weights, the multipliers they were quantised with, and the activation multipliers
  uint8_t *wqkv8 = nullptr, *wo8 = nullptr, *wff1_8 = nullptr, *wff2_8 = nullptr, *sg_wc8 = nullptr;
  float sw_qkv = 1, sw_o = 1, sw_ff1 = 1, sw_ff2 = 1, sw_c = 1;
  // INT8: per-output-channel symmetric weights and their scales
  int8_t *wqkv_q = nullptr, *wo_q = nullptr, *wff1_q = nullptr, *wff2_q = nullptr;
  float *cs_qkv = nullptr, *cs_o = nullptr, *cs_ff1 = nullptr, *cs_ff2 = nullptr;
  float sa_in = 1, sa_ctx = 1, sa_ffn = 1, sa_hid = 1, sa_bias = 1, sa_qkv = 1, sa_gen = 1;
  // FP8: biases corrected for the mean effect of the weights' e4m3 rounding (filled by crl_calibrate)
  float *bqkv8 = nullptr, *bo8 = nullptr, *bff1_8 = nullptr, *bff2_8 = nullptr;
};

struct ValueW {
  __half *w1 = nullptr, *w2 = nullptr;
  float *b1 = nullptr, *b2 = nullptr, *w3 = nullptr, *b3 = nullptr;
  int n_out = 3;
};

}  // namespace

struct crl_handle {
  crl_config cfg{};
  int device = 0;
  int num_sms = 148;
  int hd = 32;
  int ppad = 112;       // planes rounded up to 8 (16-byte rows for TMA)
  int qk_ld = 0;        // policy Q|K|promo projection width
  int chunk = 8192;
  bool finalized = false;
  bool calibrated = false;
  std::vector<std::string> required;
  std::map<std::string, std::vector<float>> raw;
  std::vector<void*> allocs;
  std::string detail;
  int* status_dev = nullptr;
  float* mean_dev = nullptr;          // [L][4][max(d, ff)] column sums of the four GEMM inputs over the calibration batch
  float* mean_part = nullptr;         // [64][max(d, ff)] scratch of the column-sum kernel
  long long mean_rows = 0;            // rows summed so far in this calibration call
  unsigned int* amax_dev = nullptr;   // [L*8] float bit patterns (7 taps per layer used)
  int64_t launches = 0;
  // optional per-kernel timing (crl_profile): event pairs around every launch, by category
  struct ProfRec { cudaEvent_t a, b; int cat; double flops, bytes; int m, n, k, kind; };
  std::vector<ProfRec> prof;
  size_t prof_used = 0;
  bool profiling = false;

  __half *w_embed = nullptr, *pe16 = nullptr, *sg_shared = nullptr, *w_pt = nullptr, *w_qk = nullptr, *w_ph = nullptr;
  uint8_t* sg_shared8 = nullptr;      // FP8 engine: e4m3 copy of the shared smolgen weight and its multiplier
  float sw_shared = 1.0f;
  float *b_embed = nullptr, *lnE_w = nullptr, *lnE_b = nullptr, *gate_ea = nullptr, *gate_b = nullptr;
  float *lnF_w = nullptr, *lnF_b = nullptr, *b_pt = nullptr, *b_qk = nullptr;
  short* gather_idx = nullptr;
  signed char* gather_promo = nullptr;
  short* mirror_idx = nullptr;
  std::vector<LayerW> layers;
  ValueW vh, vq;

  // crl_forward_host staging (device) and workspace, grown on demand
  short* plain_idx = nullptr;         // [4096] from*64+to -> entry of the 1858 list, -1 where none (device)
  void* st_black = nullptr; size_t st_black_b = 0;
  void* st_move = nullptr; size_t st_move_b = 0;     // [B] int32 moves, then [B] f32 uniforms
  void *st_planes = nullptr, *st_mask = nullptr, *st_policy = nullptr, *st_wdl = nullptr, *st_q = nullptr, *st_ws = nullptr;
  size_t st_planes_b = 0, st_mask_b = 0, st_policy_b = 0, st_wdl_b = 0, st_q_b = 0, st_ws_b = 0;
};

namespace {

int fail(crl_handle* h, int code, const std::string& msg) {
  if (h != nullptr) h->detail = msg;
  return code;
}
int cuda_fail(crl_handle* h, cudaError_t e, const char* what) {
  return fail(h, CRL_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}
#define CRL_CUDA(h, expr)                                          \
  do {                                                             \
    cudaError_t e__ = (expr);                                      \
    if (e__ != cudaSuccess) return cuda_fail((h), e__, #expr);     \
  } while (0)

// Makes the handle's device current for one entry point and puts the caller's device back on every return
// path: frameworks read the current device from the runtime, so an entry point must not leave it changed.
struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  cudaError_t err = cudaSuccess;
  explicit DeviceGuard(int device) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != device) err = cudaSetDevice(device);
    ok = err == cudaSuccess;
    if (prev == device) prev = -1;       // nothing to restore
  }
  ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
  DeviceGuard(const DeviceGuard&) = delete;
  DeviceGuard& operator=(const DeviceGuard&) = delete;
};
#define CRL_ON_DEVICE(h)                                            \
  DeviceGuard guard__((h)->device);                                 \
  if (!guard__.ok) return cuda_fail((h), guard__.err, "cudaSetDevice")

std::string lkey(int l, const char* tail) { return "layers." + std::to_string(l) + "." + tail; }

void build_required(crl_handle* h) {
  const crl_config& c = h->cfg;
  auto& r = h->required;
  r.clear();
  for (int l = 0; l < c.n_layers; ++l) {
    for (const char* t : {"attention.query_proj.weight", "attention.query_proj.bias", "attention.key_proj.weight",
                          "attention.key_proj.bias", "attention.value_proj.weight", "attention.value_proj.bias",
                          "attention.out_proj.weight", "attention.out_proj.bias", "norm1.weight", "norm1.bias",
                          "norm2.weight", "norm2.bias", "ff1.weight", "ff1.bias", "ff2.weight", "ff2.bias"})
      r.push_back(lkey(l, t));
    if (c.bias_mode == CRL_BIAS_RELPOS)
      for (const char* t : {"attention.pos_proj.weight", "attention.u_bias", "attention.v_bias"}) r.push_back(lkey(l, t));
    if (c.bias_mode == CRL_BIAS_SMOLGEN)
      for (const char* t : {"smolgen.compress.weight", "smolgen.dense1.weight", "smolgen.dense1.bias", "smolgen.ln1.weight",
                            "smolgen.ln1.bias", "smolgen.dense2.weight", "smolgen.dense2.bias", "smolgen.ln2.weight",
                            "smolgen.ln2.bias"})
        r.push_back(lkey(l, t));
  }
  for (const char* t : {"linear1.weight", "linear1.bias", "layernorm1.weight", "layernorm1.bias", "ma_gating.a", "ma_gating.b"})
    r.push_back(t);
  if (c.bias_mode == CRL_BIAS_SMOLGEN) r.push_back("smolgen_shared.weight");
  if (c.ln_mode == CRL_LN_PRE) { r.push_back("norm_f.weight"); r.push_back("norm_f.bias"); }
  if (c.policy_mode == CRL_POLICY_DENSE4096 || c.policy_mode == CRL_POLICY_GATHER1858)
    for (const char* t : {"policy_tokens_lin.weight", "policy_tokens_lin.bias", "queries_pol.weight", "queries_pol.bias",
                          "keys_pol.weight", "keys_pol.bias"})
      r.push_back(t);
  if (c.policy_mode == CRL_POLICY_LM_HEAD) r.push_back("lm_head.weight");
  if (c.pos_embed) r.push_back("pe");
  if (c.policy_mode == CRL_POLICY_DENSE4096) r.push_back("policy_head.weight");
  if (c.policy_mode == CRL_POLICY_GATHER1858) r.push_back("policy_promo.weight");
  if (c.value_mode != CRL_VALUE_NONE)
    for (const char* t : {"value_head.dense1.weight", "value_head.dense1.bias", "value_head.dense2.weight",
                          "value_head.dense2.bias", "value_head.dense3.weight", "value_head.dense3.bias"})
      r.push_back(t);
  if (c.value_mode == CRL_VALUE_WDL_Q)
    for (const char* t : {"value_head_q.dense1.weight", "value_head_q.dense1.bias", "value_head_q.dense2.weight",
                          "value_head_q.dense2.bias", "value_head_q.dense3.weight", "value_head_q.dense3.bias"})
      r.push_back(t);
}

template <typename T>
int dev_alloc(crl_handle* h, T** out, size_t count) {
  void* p = nullptr;
  CRL_CUDA(h, cudaMalloc(&p, std::max<size_t>(count * sizeof(T), 16)));
  h->allocs.push_back(p);
  *out = static_cast<T*>(p);
  return CRL_OK;
}

// [rows, cols] f32 (host) -> [rows, ld] f16 (device), zero padded
int upload_f16(crl_handle* h, __half** out, const float* src, size_t rows, size_t cols, size_t ld) {
  std::vector<__half> tmp(rows * ld, __float2half_rn(0.0f));
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) tmp[r * ld + c] = __float2half_rn(src[r * cols + c]);
  int rc = dev_alloc(h, out, rows * ld);
  if (rc != CRL_OK) return rc;
  CRL_CUDA(h, cudaMemcpy(*out, tmp.data(), tmp.size() * sizeof(__half), cudaMemcpyHostToDevice));
  return CRL_OK;
}
int upload_f32(crl_handle* h, float** out, const float* src, size_t n) {
  int rc = dev_alloc(h, out, n);
  if (rc != CRL_OK) return rc;
  CRL_CUDA(h, cudaMemcpy(*out, src, n * sizeof(float), cudaMemcpyHostToDevice));
  return CRL_OK;
}
// per-tensor e4m3 copy: multiplier = 448 / max|w|
int upload_e4m3(crl_handle* h, uint8_t** out, float* mult, const float* src, size_t n) {
  float amax = 0.0f;
  for (size_t i = 0; i < n; ++i) amax = std::max(amax, std::fabs(src[i]));
  const float m = amax > 0.0f ? kFp8Max / amax : 1.0f;
  std::vector<uint8_t> tmp(n);
  for (size_t i = 0; i < n; ++i)
    tmp[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(src[i] * m, __NV_SATFINITE, __NV_E4M3));
  int rc = dev_alloc(h, out, n);
  if (rc != CRL_OK) return rc;
  CRL_CUDA(h, cudaMemcpy(*out, tmp.data(), n, cudaMemcpyHostToDevice));
  *mult = m;
  return CRL_OK;
}

// per-output-channel symmetric int8: scale[n] = max|w[n,:]| / 127
int upload_i8_rows(crl_handle* h, int8_t** out, float** scales, const float* src, size_t rows, size_t cols) {
  std::vector<int8_t> q(rows * cols);
  std::vector<float> sc(rows);
  for (size_t r = 0; r < rows; ++r) {
    float amax = 0.0f;
    for (size_t c = 0; c < cols; ++c) amax = std::max(amax, std::fabs(src[r * cols + c]));
    const float s1 = amax > 0.0f ? amax / 127.0f : 1.0f;
    sc[r] = s1;
    for (size_t c = 0; c < cols; ++c) {
      const float v = std::nearbyint(src[r * cols + c] / s1);
      q[r * cols + c] = static_cast<int8_t>(std::max(-127.0f, std::min(127.0f, v)));
    }
  }
  int rc = dev_alloc(h, out, rows * cols);
  if (rc != CRL_OK) return rc;
  CRL_CUDA(h, cudaMemcpy(*out, q.data(), q.size(), cudaMemcpyHostToDevice));
  return upload_f32(h, scales, sc.data(), rows);
}

struct Expect { std::string key; size_t numel; };

const std::vector<float>* get(crl_handle* h, const std::string& k) {
  auto it = h->raw.find(k);
  return it == h->raw.end() ? nullptr : &it->second;
}

// ---- workspace -----------------------------------------------------------------------------------
struct Workspace {
  __half *xin, *x, *xn, *t1, *t2, *y;
  uint8_t *x8, *t2_8, *t1_8;
  float *xs, *t2s, *t1s;   // INT8: per-token scales of x8 / t2_8 / t1_8
  __half *sg_c, *sg_h1, *sg_h1n, *sg_h2, *sg_h2n, *sg_bias;
  uint8_t* sg_h2n8;   // FP8 engine: e4m3 copy of the normalised generator rows (A operand of the bias GEMM)
  __half *flat;     // [bc, 4096] policy scores (dense form)
  float* logits;    // [bc, 1929] f32 (dense form)
  __half *v2, *v2q;
  uint8_t* legal;      // [batch, 236] legal-move bitsets generated from the packed records
  unsigned long long* lno_stats;   // exchange buffer of the GEMM kernels that normalise their output rows
  size_t total;
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// bc: positions per pass over the layers; total: positions of the whole call (the legal-move bitsets are
// generated for all of them at once, before the first pass)
Workspace carve(const crl_handle* h, char* base, int64_t bc, int64_t total) {
  const crl_config& c = h->cfg;
  const size_t M = static_cast<size_t>(bc) * 64;
  const size_t d = c.d_model;
  const size_t wide = std::max<size_t>({3 * d, static_cast<size_t>(c.d_ff), static_cast<size_t>(h->qk_ld)});
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char* p = base != nullptr ? base + off : nullptr;
    off += align_up(std::max<size_t>(bytes, 16), 256);
    return p;
  };
  Workspace w{};
  w.xin = reinterpret_cast<__half*>(take(M * h->ppad * 2));
  w.x = reinterpret_cast<__half*>(take(M * d * 2));
  w.xn = reinterpret_cast<__half*>(take(M * d * 2));
  w.t1 = reinterpret_cast<__half*>(take(M * wide * 2));
  w.t2 = reinterpret_cast<__half*>(take(M * d * 2));
  w.y = reinterpret_cast<__half*>(take(M * d * 2));
  const bool f8 = c.dtype == CRL_DTYPE_F8E4M3 || c.dtype == CRL_DTYPE_I8;
  const bool rowsc = c.dtype == CRL_DTYPE_I8;
  w.xs = reinterpret_cast<float*>(take(rowsc ? M * 4 : 0));
  w.t2s = reinterpret_cast<float*>(take(rowsc ? M * 4 : 0));
  w.t1s = reinterpret_cast<float*>(take(rowsc ? M * 4 : 0));
  w.x8 = reinterpret_cast<uint8_t*>(take(f8 ? M * d : 0));
  w.t2_8 = reinterpret_cast<uint8_t*>(take(f8 ? M * d : 0));
  w.t1_8 = reinterpret_cast<uint8_t*>(take(f8 ? M * c.d_ff : 0));
  const bool sg = c.bias_mode == CRL_BIAS_SMOLGEN;
  const size_t hg = static_cast<size_t>(c.n_heads) * c.smolgen_gen;
  w.sg_c = reinterpret_cast<__half*>(take(sg ? M * c.smolgen_compress * 2 : 0));
  w.sg_h1 = reinterpret_cast<__half*>(take(sg ? bc * c.smolgen_hidden * 2 : 0));
  w.sg_h1n = reinterpret_cast<__half*>(take(sg ? bc * c.smolgen_hidden * 2 : 0));
  w.sg_h2 = reinterpret_cast<__half*>(take(sg ? bc * hg * 2 : 0));
  w.sg_h2n = reinterpret_cast<__half*>(take(sg ? bc * hg * 2 : 0));
  w.sg_h2n8 = reinterpret_cast<uint8_t*>(take(sg && c.dtype == CRL_DTYPE_F8E4M3 ? bc * hg : 0));
  w.sg_bias = reinterpret_cast<__half*>(take(sg ? static_cast<size_t>(bc) * c.n_heads * 4096 * 2 : 0));
  const bool dense = c.policy_mode == CRL_POLICY_DENSE4096;
  const bool lm = c.policy_mode == CRL_POLICY_LM_HEAD;
  w.flat = reinterpret_cast<__half*>(take(dense ? static_cast<size_t>(bc) * 4096 * 2 : 0));
  w.logits = reinterpret_cast<float*>(take((dense || lm) ? static_cast<size_t>(bc) * 2048 * 4 : 0));
  w.v2 = reinterpret_cast<__half*>(take(static_cast<size_t>(bc) * 128 * 2));
  w.v2q = reinterpret_cast<__half*>(take(static_cast<size_t>(bc) * 128 * 2));
  w.legal = reinterpret_cast<uint8_t*>(take(c.policy_mode == CRL_POLICY_GATHER1858 ? static_cast<size_t>(total) * 236 : 0));
  const bool lno = (c.fuse_layernorm == CRL_FUSE_LN_OUT || c.fuse_layernorm == CRL_FUSE_LN_AUTO) && c.ln_mode == CRL_LN_POST &&
                   d % 256 == 0;
  w.lno_stats = reinterpret_cast<unsigned long long*>(take(lno ? gemm_ln_out_scratch_bytes(static_cast<long long>(M)) : 0));
  w.total = off;
  return w;
}

// ---- launch helpers --------------------------------------------------------------------------------
enum ProfCat : int { kCatGemm = 0, kCatAttention = 1, kCatLayerNorm = 2, kCatOther = 3 };

// Brackets one launch with CUDA events on the launch stream while profiling is on.
struct ProfScope {
  crl_handle* h; cudaStream_t s; crl_handle::ProfRec* rec = nullptr;
  ProfScope(crl_handle* h_, cudaStream_t s_, int cat, double flops, double bytes) : h(h_), s(s_) {
    if (!h->profiling) return;
    if (h->prof_used == h->prof.size()) {
      crl_handle::ProfRec r{};
      if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return;
      h->prof.push_back(r);
    }
    rec = &h->prof[h->prof_used++];
    rec->cat = cat; rec->flops = flops; rec->bytes = bytes; rec->m = rec->n = rec->k = rec->kind = 0;
    cudaEventRecord(rec->a, s);
  }
  ~ProfScope() { if (rec != nullptr) cudaEventRecord(rec->b, s); }
};

struct Lin {
  int kind = kKindF16;
  const void* a = nullptr; long long lda = 0;
  const void* w = nullptr; long long ldw = 0;
  void* c = nullptr; long long ldc = 0; int out = kOutF16;
  long long m = 0; int n = 0, k = 0;
  const float* bias = nullptr;
  const __half* res = nullptr; long long ldr = 0; int res_mod = 0;
  float alpha = 1.0f; int act = kActNone; float out_scale = 1.0f;
  const float* row_scale = nullptr; const float* col_scale = nullptr;
  // fused LayerNorm: A = LN(ln_y) * w + b, normalised inside the GEMM kernel, written to ln_x (f16) / ln_x8 (e4m3)
  const __half* ln_y = nullptr; const __half* ln_w16 = nullptr; const __half* ln_b16 = nullptr;
  __half* ln_x = nullptr; uint8_t* ln_x8 = nullptr; float ln_out8_scale = 1.0f;
  int precise_act = 0;
  // output LayerNorm: C = LN(acc + bias + residual) * w + b over the whole row, inside the GEMM kernel, with an optional
  // e4m3 copy (lno_x8) scaled by lno_out8_scale; lno_stats is the kernel's exchange buffer
  const __half* lno_w16 = nullptr; const __half* lno_b16 = nullptr; uint8_t* lno_x8 = nullptr; float lno_out8_scale = 1.0f;
  float* lno_qscale = nullptr;      // int8 operands: per-token scales of the int8 copy in lno_x8
  unsigned long long* lno_stats = nullptr;
};

int linear(crl_handle* h, const Lin& l, cudaStream_t s) {
  GemmArgs g;
  g.kind = l.kind;
  g.A = l.a; g.lda = l.lda; g.W = l.w; g.ldw = l.ldw;
  g.p.M = static_cast<int>(l.m); g.p.N = l.n; g.p.K = l.k;
  g.p.C = l.c; g.p.ldc = l.ldc; g.p.out_dtype = l.out;
  g.p.bias = l.bias; g.p.residual = l.res; g.p.ldr = l.ldr; g.p.res_mod = l.res_mod;
  g.p.alpha = l.alpha; g.p.row_scale = l.row_scale; g.p.col_scale = l.col_scale;
  g.p.act = l.act; g.p.out_scale = l.out_scale; g.p.status = h->status_dev;
  g.p.ln_y = l.ln_y; g.p.ln_ldy = l.k; g.p.ln_w16 = l.ln_w16; g.p.ln_b16 = l.ln_b16; g.p.ln_x = l.ln_x; g.p.ln_x8 = l.ln_x8;
  g.p.ln_out8_scale = l.ln_out8_scale; g.p.precise_act = l.precise_act;
  g.p.lno_w16 = l.lno_w16; g.p.lno_b16 = l.lno_b16; g.p.lno_stats = l.lno_stats; g.p.lno_out8_scale = l.lno_out8_scale;
  g.p.lno_x8 = l.lno_x8; g.p.lno_qscale = l.lno_qscale;
  const size_t esz_in = l.kind == kKindF16 ? 2 : 1, esz_out = l.out == kOutF32 ? 4 : (l.out == kOutF16 ? 2 : 1);
  ProfScope ps(h, s, kCatGemm, 2.0 * l.m * l.n * l.k,
               static_cast<double>(l.m) * l.k * esz_in + static_cast<double>(l.n) * l.k * esz_in +
                   static_cast<double>(l.m) * l.n * esz_out + (l.res != nullptr && l.res_mod == 0 ? 2.0 * l.m * l.n : 0.0));
  if (ps.rec != nullptr) { ps.rec->m = static_cast<int>(l.m); ps.rec->n = l.n; ps.rec->k = l.k; ps.rec->kind = l.kind; }
  const int rc = gemm_launch(g, h->num_sms, s);
  if (rc != kOk) return fail(h, rc, "gemm launch failed (M=" + std::to_string(l.m) + " N=" + std::to_string(l.n) +
                                        " K=" + std::to_string(l.k) + ")");
  ++h->launches;
  return CRL_OK;
}

int layer_norm(crl_handle* h, const __half* x, long long rows, int d, const float* w, const float* b, __half* y,
               uint8_t* y8, float y8_scale, const float* gate_ea, const float* gate_b, cudaStream_t s,
               int8_t* yq = nullptr, float* yq_scale = nullptr) {
  LnParams p{};
  p.x = x; p.ldx = d; p.rows = rows; p.d = d; p.w = w; p.b = b;
  p.gate_ea = gate_ea; p.gate_b = gate_b;
  p.y = y; p.ldy = d; p.y8 = y8; p.ldy8 = d; p.out8_scale = y8_scale;
  p.yq = yq; p.yq_scale = yq_scale;
  const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
  ProfScope ps(h, s, kCatLayerNorm, 0.0, static_cast<double>(rows) * d * (2 + (y != nullptr ? 2 : 0) + (y8 != nullptr ? 1 : 0)));
  if (gate_ea == nullptr && rows >= 8192 && (h->cfg.precision & CRL_PREC_LN_F32) == 0) {
    const long long want = (rows + 7) / 8;
    const unsigned grid = static_cast<unsigned>(std::min<long long>(want, static_cast<long long>(h->num_sms) * 2));
    // narrow rows (the smolgen generator rows): a quarter of the registers, so four CTAs per SM keep as many bytes in flight
    const unsigned grid_narrow = static_cast<unsigned>(std::min<long long>(want, static_cast<long long>(h->num_sms) * 4));
    if (yq != nullptr) ln_rows_persistent_kernel<true><<<grid, 256, 0, s>>>(p);
    else if (d <= 256) ln_rows_persistent_kernel<false, 1><<<grid_narrow, 256, 0, s>>>(p);
    else ln_rows_persistent_kernel<false><<<grid, 256, 0, s>>>(p);
  } else {
    ln_rows_kernel<<<blocks, 256, 0, s>>>(p);
  }
  CRL_CUDA(h, cudaGetLastError());
  ++h->launches;
  return CRL_OK;
}

int quant_rows_i8(crl_handle* h, const __half* x, long long rows, int cols, uint8_t* q, float* scale, cudaStream_t s) {
  ProfScope ps(h, s, kCatLayerNorm, 0.0, static_cast<double>(rows) * cols * 3);
  if (cols > 4096 || cols % 8 != 0) return fail(h, CRL_ERR_SHAPE, "per-token int8 rows are at most 4096 wide");
  const long long want = (rows + 7) / 8;
  const unsigned grid = static_cast<unsigned>(std::min<long long>(want, static_cast<long long>(h->num_sms) * 8));
  int8_t* q8 = reinterpret_cast<int8_t*>(q);
  // the row sits in registers: the narrowest instantiation that holds it keeps the most warps resident
  if (cols <= 1024) quant_rows_i8_kernel<4><<<grid, 256, 0, s>>>(x, rows, cols, q8, scale);
  else if (cols <= 1536) quant_rows_i8_kernel<6><<<grid, 256, 0, s>>>(x, rows, cols, q8, scale);
  else if (cols <= 2048) quant_rows_i8_kernel<8><<<grid, 256, 0, s>>>(x, rows, cols, q8, scale);
  else quant_rows_i8_kernel<16><<<grid, 256, 0, s>>>(x, rows, cols, q8, scale);
  CRL_CUDA(h, cudaGetLastError());
  ++h->launches;
  return CRL_OK;
}

int tap_amax(crl_handle* h, const __half* x, long long rows, int cols, int slot, cudaStream_t s) {
  absmax_f16_kernel<<<h->num_sms * 4, 256, 0, s>>>(x, rows, cols, cols, h->amax_dev + slot);
  CRL_CUDA(h, cudaGetLastError());
  return CRL_OK;
}

// calibration: add the column sums of x [rows, cols] to slot (layer, which) of mean_dev
int tap_mean(crl_handle* h, const __half* x, long long rows, int cols, long long ld, int layer, int which, cudaStream_t s) {
  if (h->mean_dev == nullptr) return CRL_OK;
  const int wide = std::max(h->cfg.d_model, h->cfg.d_ff);
  const int segments = 64;
  colsum_f16_kernel<<<dim3((cols + 255) / 256, segments), 256, 0, s>>>(x, rows, cols, ld, h->mean_part, segments);
  colsum_finish_kernel<<<(cols + 255) / 256, 256, 0, s>>>(h->mean_part, cols, segments,
                                                          h->mean_dev + (static_cast<size_t>(layer) * 4 + which) * wide);
  CRL_CUDA(h, cudaGetLastError());
  return CRL_OK;
}

template <int NW, int BIAS, int OUT8>
int attention_tma_launch_t(crl_handle* h, const AttnTmaParams& t, const CUtensorMap& tq, const CUtensorMap& tb,
                           const CUtensorMap& to, cudaStream_t s) {
  static bool attr_set[64] = {};
  if (h->device >= 0 && h->device < 64 && !attr_set[h->device]) {
    CRL_CUDA(h, cudaFuncSetAttribute(attention_tma_kernel<NW, BIAS, OUT8>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnTmaSmem<NW>::BYTES));
    attr_set[h->device] = true;
  }
  const long long items = static_cast<long long>(t.B) * t.H;
  const long long want = (items + NW - 1) / NW;
  const unsigned grid = static_cast<unsigned>(want < h->num_sms ? want : h->num_sms);
  attention_tma_kernel<NW, BIAS, OUT8><<<grid, NW * 32, AttnTmaSmem<NW>::BYTES, s>>>(tq, tb, to, t);
  CRL_CUDA(h, cudaGetLastError());
  return CRL_OK;
}

int attention_tma_launch(crl_handle* h, const AttnTmaParams& t, const __half* qkv, const void* bias, void* out,
                         cudaStream_t s) {
  const uint64_t M = static_cast<uint64_t>(t.B) * 64;
  CUtensorMap tq, tb, to;
  std::memset(&tb, 0, sizeof(tb));
  int rc = make_tmap_2d(&tq, qkv, 2, 3ull * t.d, M, 3ull * t.d * 2, 64, 64);
  if (rc == kOk && t.has_bias == 1) rc = make_tmap_2d(&tb, bias, 2, 64, static_cast<uint64_t>(t.B) * t.H * 64, 128, 64, 128);
  if (rc == kOk && t.has_bias == 2) rc = make_tmap_2d(&tb, bias, 1, 64, static_cast<uint64_t>(t.B) * t.H * 64, 64, 64, 64);
  if (rc == kOk) rc = t.out_e4m3 ? make_tmap_2d(&to, out, 1, t.d, M, t.d, 64, 32) : make_tmap_2d(&to, out, 2, t.d, M, 2ull * t.d, 64, 64);
  if (rc != kOk) return fail(h, rc, "attention: tensor map encoding failed");
  if (t.has_bias == 1)
    return t.out_e4m3 ? attention_tma_launch_t<11, 1, 1>(h, t, tq, tb, to, s) : attention_tma_launch_t<11, 1, 0>(h, t, tq, tb, to, s);
  if (t.has_bias == 2)
    return t.out_e4m3 ? attention_tma_launch_t<14, 2, 1>(h, t, tq, tb, to, s) : attention_tma_launch_t<14, 2, 0>(h, t, tq, tb, to, s);
  return t.out_e4m3 ? attention_tma_launch_t<14, 0, 1>(h, t, tq, tb, to, s) : attention_tma_launch_t<14, 0, 0>(h, t, tq, tb, to, s);
}

template <int NW, int BIAS>
int attention_tma8_launch_t(crl_handle* h, const AttnTma8Params& t, const CUtensorMap& tq, const CUtensorMap& tb,
                            const CUtensorMap& to, cudaStream_t s) {
  static bool attr_set[64] = {};
  if (h->device >= 0 && h->device < 64 && !attr_set[h->device]) {
    CRL_CUDA(h, cudaFuncSetAttribute(attention_tma8_kernel<NW, BIAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnTma8Smem<NW>::BYTES));
    attr_set[h->device] = true;
  }
  const long long items = static_cast<long long>(t.B) * t.H;
  const long long want = (items + NW - 1) / NW;
  const unsigned grid = static_cast<unsigned>(want < h->num_sms ? want : h->num_sms);
  attention_tma8_kernel<NW, BIAS><<<grid, NW * 32, AttnTma8Smem<NW>::BYTES, s>>>(tq, tb, to, t);
  CRL_CUDA(h, cudaGetLastError());
  return CRL_OK;
}

// e4m3 Q/K/V rows [M, 3d], e4m3 bias tiles, e4m3 context
int attention_tma8_launch(crl_handle* h, const AttnTma8Params& t, const uint8_t* qkv8, const void* bias, void* out, cudaStream_t s) {
  const uint64_t M = static_cast<uint64_t>(t.B) * 64;
  CUtensorMap tq, tb, to;
  std::memset(&tb, 0, sizeof(tb));
  int rc = make_tmap_2d(&tq, qkv8, 1, 3ull * t.d, M, 3ull * t.d, 64, 32);
  if (rc == kOk && t.has_bias == 2) rc = make_tmap_2d(&tb, bias, 1, 64, static_cast<uint64_t>(t.B) * t.H * 64, 64, 64, 64);
  if (rc == kOk) rc = make_tmap_2d(&to, out, 1, t.d, M, t.d, 64, 32);
  if (rc != kOk) return fail(h, rc, "attention: tensor map encoding failed");
  return t.has_bias != 0 ? attention_tma8_launch_t<16, 1>(h, t, tq, tb, to, s) : attention_tma8_launch_t<16, 0>(h, t, tq, tb, to, s);
}

int act_of(const crl_config& c) { return c.act == CRL_ACT_MISH ? kActMish : kActGelu; }

int value_head(crl_handle* h, const ValueW& vw, const __half* x, __half* v1, __half* v2, int64_t bc, float* out,
               int tail_mode, cudaStream_t s) {
  const int d = h->cfg.d_model;
  Lin a; a.a = x; a.lda = d; a.w = vw.w1; a.ldw = d; a.c = v1; a.ldc = 128; a.m = bc * 64; a.n = 128; a.k = d;
  a.bias = vw.b1; a.act = kActGelu;
  int rc = linear(h, a, s);
  if (rc != CRL_OK) return rc;
  Lin b; b.a = v1; b.lda = 8192; b.w = vw.w2; b.ldw = 8192; b.c = v2; b.ldc = 128; b.m = bc; b.n = 128; b.k = 8192;
  b.bias = vw.b2; b.act = kActGelu;
  rc = linear(h, b, s);
  if (rc != CRL_OK) return rc;
  value_tail_kernel<<<static_cast<unsigned>((bc + 7) / 8), 256, 0, s>>>(v2, vw.w3, vw.b3, out, bc, vw.n_out, tail_mode);
  CRL_CUDA(h, cudaGetLastError());
  ++h->launches;
  return CRL_OK;
}

// One pass over `bc` positions starting at position b0 of the call's batch.
int forward_chunk(crl_handle* h, const crl_io* io, int64_t b0, int64_t bc, const Workspace& w, bool calib,
                  cudaStream_t s) {
  const crl_config& c = h->cfg;
  const int d = c.d_model, H = c.n_heads, ff = c.d_ff, P = c.planes;
  const long long M = bc * 64;
  const bool f8 = c.dtype == CRL_DTYPE_F8E4M3 && !calib;
  const bool i8 = c.dtype == CRL_DTYPE_I8;
  const int prec = c.precision;
  const bool attn_f32 = (prec & CRL_PREC_ATTN_F32) != 0;
  const bool f8_attn = f8 && (prec & CRL_PREC_ATTN_GEMM_F16) == 0;   // QKV / out-projection on e4m3 operands
  const bool f8_ffn = f8 && (prec & CRL_PREC_FFN_F16) == 0;          // ff1 / ff2 on e4m3 operands
  // FP8 engine on the TMA attention path: the QKV projection writes e4m3 and attention reads it
  const bool qkv8 = f8 && h->hd == 32 && (c.bias_mode == CRL_BIAS_NONE || c.bias_mode == CRL_BIAS_SMOLGEN) &&
                    (prec & (CRL_PREC_QKV_F16 | CRL_PREC_ATTN_F32 | CRL_PREC_ATTN_GEMM_F16)) == 0;
  const bool ctx8 = f8_attn;      // attention writes its context as e4m3 for an e4m3 out-projection
  int8_t* const xq = reinterpret_cast<int8_t*>(w.x8);
  const int act = act_of(c);
  // Optional (crl_config.fuse_layernorm): post-LN blocks on large passes run the LayerNorm in front of ff1 and the one
  // in front of the next block's QKV projection inside those GEMM kernels (their own warps normalise a row block
  // ahead of the MMAs) instead of as separate passes over the rows.
  const bool fuse_ln = !calib && !i8 && c.ln_mode == CRL_LN_POST && c.fuse_layernorm == CRL_FUSE_LN_ON &&
                       (prec & CRL_PREC_LN_F32) == 0 && gemm_can_fuse_ln(M, std::min(3 * d, ff), d, h->num_sms);
  // CRL_FUSE_LN_OUT: the out-projection and ff2 kernels normalise their own output rows (the warps holding a row's
  // slabs, in the CTAs working on the row block's column tiles, exchange the row sums), so the sum x + sublayer(x)
  // never crosses HBM and the two row passes per block go away. The result lands in w.x, over the residual it was
  // computed from.
  // (CRL_FUSE_LN_AUTO takes it from four tiles per CTA pair on: below that it measures neither faster nor slower.)
  const bool lno = !calib && c.ln_mode == CRL_LN_POST && (prec & CRL_PREC_LN_F32) == 0 && w.lno_stats != nullptr &&
                   c.ffn_act_pos == CRL_FFN_ACT_MID &&      // (no activation between the GEMM and the residual sum)
                   ((c.fuse_layernorm == CRL_FUSE_LN_OUT && gemm_can_fuse_ln_out(M, d, h->num_sms)) ||
                    (c.fuse_layernorm == CRL_FUSE_LN_AUTO && !i8 && gemm_can_fuse_ln_out(M / 4, d, h->num_sms)));
  // (The INT8 engine takes this route only when asked to: its per-token int8 copy needs a second exchange - the row
  // maximum - and a third pass over the slab, and the longer GEMMs cost what the saved row passes gave: 63.0 against
  // 63.5 ms per 4096 positions.)

  // ---- input planes -> token-major f16 rows ------------------------------------------------------
  {
    const size_t per_pos = static_cast<size_t>(64) * P;
    if (io->layout == CRL_LAYOUT_NHWC_F32 || io->layout == CRL_LAYOUT_NHWC_F16) {
      const long long n = M * (h->ppad / 8);
      const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
      if (io->layout == CRL_LAYOUT_NHWC_F32)
        tokens_from_nhwc_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(io->planes) + b0 * per_pos, w.xin, M, P, h->ppad);
      else
        tokens_from_nhwc_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<const __half*>(io->planes) + b0 * per_pos, w.xin, M, P, h->ppad);
    } else if (io->layout == CRL_LAYOUT_NCHW_F16 || io->layout == CRL_LAYOUT_NCHW_F32) {
      const size_t smem = static_cast<size_t>(P) * 66 * 2;
      if (io->layout == CRL_LAYOUT_NCHW_F16)
        tokens_from_nchw_kernel<__half><<<static_cast<unsigned>(bc), 256, smem, s>>>(static_cast<const __half*>(io->planes) + b0 * per_pos, w.xin, P, h->ppad);
      else
        tokens_from_nchw_kernel<float><<<static_cast<unsigned>(bc), 256, smem, s>>>(static_cast<const float*>(io->planes) + b0 * per_pos, w.xin, P, h->ppad);
    } else if (io->layout == CRL_LAYOUT_PACKED104) {
      tokens_from_packed104_kernel<<<static_cast<unsigned>(bc), 256, 0, s>>>(static_cast<const uint8_t*>(io->planes) + b0 * CRL_PACKED104_BYTES, w.xin, h->ppad);
    } else {
      return fail(h, CRL_ERR_INVALID, "unknown plane layout");
    }
    CRL_CUDA(h, cudaGetLastError());
    ++h->launches;
  }

  int rc;
  // ---- embedding: Linear -> GELU -> LayerNorm -> gating (utils/fen_encoder.py:61-67) ---------------
  {
    Lin e; e.a = w.xin; e.lda = h->ppad; e.w = h->w_embed; e.ldw = h->ppad; e.c = w.t2; e.ldc = d; e.m = M; e.n = d;
    e.k = h->ppad; e.bias = h->b_embed; e.act = kActGelu;
    if ((rc = linear(h, e, s)) != CRL_OK) return rc;
    const bool emit8 = f8 && c.ln_mode == CRL_LN_POST;
    if ((rc = layer_norm(h, w.t2, M, d, h->lnE_w, h->lnE_b, w.x, emit8 ? w.x8 : nullptr,
                         emit8 ? h->layers[0].sa_in : 1.0f, h->gate_ea, h->gate_b, s,
                         (i8 && c.ln_mode == CRL_LN_POST) ? xq : nullptr, w.xs)) != CRL_OK)
      return rc;
  }

  for (int l = 0; l < c.n_layers; ++l) {
    LayerW& L = h->layers[l];
    const __half* attn_in = w.x;
    const uint8_t* attn_in8 = w.x8;
    if (c.ln_mode == CRL_LN_PRE) {
      if ((rc = layer_norm(h, w.x, M, d, L.ln1w, L.ln1b, w.xn, f8 ? w.x8 : nullptr, L.sa_in, nullptr, nullptr, s, i8 ? xq : nullptr, w.xs)) != CRL_OK)
        return rc;
      attn_in = w.xn;
    }
    if (calib && (rc = tap_amax(h, attn_in, M, d, l * 8 + 0, s)) != CRL_OK) return rc;
    if (calib && (rc = tap_mean(h, attn_in, M, d, d, l, 0, s)) != CRL_OK) return rc;
    // QKV projection (attn.py:501-503 fused into one [3d, d] weight)
    {
      Lin q; q.m = M; q.n = 3 * d; q.k = d; q.c = w.t1; q.ldc = 3 * d; q.bias = L.bqkv;
      if (f8_attn) { q.kind = kKindF8; q.a = attn_in8; q.w = L.wqkv8; q.alpha = 1.0f / (L.sa_in * L.sw_qkv); q.bias = L.bqkv8; }
      else if (!i8) { q.a = attn_in; q.w = L.wqkv; }
      if (qkv8) { q.out = kOutE4M3; q.out_scale = L.sa_qkv; }   // Q, K, V cross HBM as e4m3 (one scale for the three)
      else if (i8) { q.kind = kKindI8; q.a = w.x8; q.w = L.wqkv_q; q.row_scale = w.xs; q.col_scale = L.cs_qkv; }
      q.lda = d; q.ldw = d;
      if (fuse_ln && l > 0) {      // norm2 of the previous block: w.y -> w.x (+ w.x8), inside this kernel
        const LayerW& P = h->layers[l - 1];
        q.ln_y = w.y; q.ln_w16 = P.ln2w16; q.ln_b16 = P.ln2b16; q.ln_x = w.x; q.ln_x8 = f8 ? w.x8 : nullptr; q.ln_out8_scale = L.sa_in;
        // (the e4m3 copy is written even when this GEMM reads the f16 rows: the smolgen compression reads it)
      }
      if ((rc = linear(h, q, s)) != CRL_OK) return rc;
      if (calib && (rc = tap_amax(h, w.t1, M, 3 * d, l * 8 + 5, s)) != CRL_OK) return rc;
    }
    if (c.bias_mode == CRL_BIAS_SMOLGEN) {
      const int cc = c.smolgen_compress, hid = c.smolgen_hidden, gen = c.smolgen_gen;
      Lin a; a.a = attn_in; a.lda = d; a.w = L.sg_wc; a.ldw = d; a.c = w.sg_c; a.ldc = cc; a.m = M; a.n = cc; a.k = d;
      // FP8 engine: this projection is a pure read of the token rows, so it takes the e4m3 copy (half the bytes)
      if (f8) { a.kind = kKindF8; a.a = attn_in8; a.w = L.sg_wc8; a.alpha = 1.0f / (L.sa_in * L.sw_c); }
      if ((rc = linear(h, a, s)) != CRL_OK) return rc;
      Lin b; b.a = w.sg_c; b.lda = 64 * cc; b.w = L.sg_w1; b.ldw = 64 * cc; b.c = w.sg_h1; b.ldc = hid; b.m = bc; b.n = hid;
      b.k = 64 * cc; b.bias = L.sg_b1; b.act = act;
      if ((rc = linear(h, b, s)) != CRL_OK) return rc;
      if ((rc = layer_norm(h, w.sg_h1, bc, hid, L.sg_ln1w, L.sg_ln1b, w.sg_h1n, nullptr, 1.0f, nullptr, nullptr, s)) != CRL_OK) return rc;
      Lin e; e.a = w.sg_h1n; e.lda = hid; e.w = L.sg_w2; e.ldw = hid; e.c = w.sg_h2; e.ldc = H * gen; e.m = bc; e.n = H * gen;
      e.k = hid; e.bias = L.sg_b2; e.act = act;
      if ((rc = linear(h, e, s)) != CRL_OK) return rc;
      // FP8 engine (default precision): the generator rows get an e4m3 copy and the 256 -> 4096 product runs on e4m3
      // operands (it is bound by operand traffic, and its rounding is two orders of magnitude below the block GEMMs')
      const bool bias8 = qkv8 && gen % 16 == 0;
      if ((rc = layer_norm(h, w.sg_h2, bc * H, gen, L.sg_ln2w, L.sg_ln2b, w.sg_h2n, bias8 ? w.sg_h2n8 : nullptr, bias8 ? L.sa_gen : 1.0f, nullptr, nullptr, s)) != CRL_OK) return rc;
      if (calib && (rc = tap_amax(h, w.sg_h2n, bc * H, gen, l * 8 + 6, s)) != CRL_OK) return rc;
      Lin f; f.a = w.sg_h2n; f.lda = gen; f.w = h->sg_shared; f.ldw = gen; f.c = w.sg_bias; f.ldc = 4096; f.m = bc * H; f.n = 4096;
      f.k = gen;
      if (bias8) { f.kind = kKindF8; f.a = w.sg_h2n8; f.w = h->sg_shared8; f.alpha = 1.0f / (L.sa_gen * h->sw_shared); }
      if (qkv8) { f.out = kOutE4M3; f.out_scale = L.sa_bias; }   // the bias tile crosses HBM as e4m3
      if ((rc = linear(h, f, s)) != CRL_OK) return rc;
      if (calib && (rc = tap_amax(h, w.sg_bias, bc * H, 4096, l * 8 + 4, s)) != CRL_OK) return rc;
    }
    // fused attention
    {
      AttnParams a{};
      a.qkv = w.t1; a.ld = 3 * d; a.d = d; a.H = H; a.B = static_cast<int>(bc);
      a.bias = w.sg_bias; a.pos = L.pos; a.u = L.u; a.v = L.v;
      a.scale = c.bias_mode == CRL_BIAS_RELPOS ? 1.0f / std::sqrt(static_cast<float>(d)) : 1.0f / std::sqrt(static_cast<float>(h->hd));
      a.ldo = d;
      if (ctx8) { a.out = nullptr; a.out8 = w.t2_8; a.out8_scale = L.sa_ctx; }
      else { a.out = w.t2; a.out8 = nullptr; a.out8_scale = 1.0f; }
      ProfScope ps(h, s, kCatAttention, 4.0 * M * 64 * d,
                   static_cast<double>(M) * d * (qkv8 ? 1 : 2) * 3 + static_cast<double>(M) * d * (ctx8 ? 1 : 2) +
                       (c.bias_mode == CRL_BIAS_SMOLGEN ? static_cast<double>(bc) * H * (qkv8 ? 4096 : 8192) : 0.0));
      if (qkv8) {
        AttnTma8Params t{};
        t.B = static_cast<int>(bc); t.H = H; t.scale = a.scale; t.d = d; t.status = h->status_dev;
        t.q_mult = 1.0f / (L.sa_qkv * L.sa_qkv);
        t.has_bias = c.bias_mode == CRL_BIAS_SMOLGEN ? 2 : 0;
        t.bias_mult = 1.0f / L.sa_bias;
        t.out_mult = L.sa_ctx / L.sa_qkv;
        if ((rc = attention_tma8_launch(h, t, reinterpret_cast<const uint8_t*>(w.t1), w.sg_bias, w.t2_8, s)) != CRL_OK) return rc;
      } else if (!attn_f32 && h->hd == 32 && (c.bias_mode == CRL_BIAS_NONE || c.bias_mode == CRL_BIAS_SMOLGEN)) {
        AttnTmaParams t{};
        t.B = static_cast<int>(bc); t.H = H; t.scale = a.scale; t.d = d; t.status = h->status_dev;
        t.has_bias = c.bias_mode == CRL_BIAS_SMOLGEN ? 1 : 0;      // f16 bias tile (the e4m3 tile goes with e4m3 Q/K/V)
        t.bias_mult = 1.0f;
        t.out_e4m3 = ctx8 ? 1 : 0; t.out_scale = ctx8 ? L.sa_ctx : 1.0f;
        if ((rc = attention_tma_launch(h, t, w.t1, w.sg_bias, ctx8 ? static_cast<void*>(w.t2_8) : static_cast<void*>(w.t2), s)) != CRL_OK)
          return rc;
      } else {
        CRL_CUDA(h, attention_launch(a, h->hd, c.bias_mode, s));
      }
      ++h->launches;
    }
    if (calib && (rc = tap_amax(h, w.t2, M, d, l * 8 + 1, s)) != CRL_OK) return rc;
    if (calib && (rc = tap_mean(h, w.t2, M, d, d, l, 1, s)) != CRL_OK) return rc;
    if (i8 && (rc = quant_rows_i8(h, w.t2, M, d, w.t2_8, w.t2s, s)) != CRL_OK) return rc;
    // out-proj + residual (+ LayerNorm for post-LN)
    {
      Lin o; o.m = M; o.n = d; o.k = d; o.bias = L.bo; o.res = w.x; o.ldr = d; o.lda = d; o.ldw = d;
      o.c = c.ln_mode == CRL_LN_POST ? w.y : w.x; o.ldc = d;
      if (f8_attn) { o.kind = kKindF8; o.a = w.t2_8; o.w = L.wo8; o.alpha = 1.0f / (L.sa_ctx * L.sw_o); o.bias = L.bo8; }
      else if (i8) { o.kind = kKindI8; o.a = w.t2_8; o.w = L.wo_q; o.row_scale = w.t2s; o.col_scale = L.cs_o; }
      else { o.a = w.t2; o.w = L.wo; }
      if (lno) {
        o.c = w.x; o.lno_w16 = L.ln1w16; o.lno_b16 = L.ln1b16; o.lno_x8 = (f8 || i8) ? w.x8 : nullptr; o.lno_out8_scale = L.sa_ffn;
        o.lno_qscale = i8 ? w.xs : nullptr; o.lno_stats = w.lno_stats;
      }
      if ((rc = linear(h, o, s)) != CRL_OK) return rc;
    }
    const __half* ffn_in;
    if (c.ln_mode == CRL_LN_POST) {
      if (!fuse_ln && !lno &&
          (rc = layer_norm(h, w.y, M, d, L.ln1w, L.ln1b, w.x, f8 ? w.x8 : nullptr, L.sa_ffn, nullptr, nullptr, s, i8 ? xq : nullptr, w.xs)) != CRL_OK) return rc;
      ffn_in = w.x;
    } else {
      if ((rc = layer_norm(h, w.x, M, d, L.ln2w, L.ln2b, w.xn, f8 ? w.x8 : nullptr, L.sa_ffn, nullptr, nullptr, s, i8 ? xq : nullptr, w.xs)) != CRL_OK) return rc;
      ffn_in = w.xn;
    }
    if (calib && (rc = tap_amax(h, ffn_in, M, d, l * 8 + 2, s)) != CRL_OK) return rc;
    if (calib && (rc = tap_mean(h, ffn_in, M, d, d, l, 2, s)) != CRL_OK) return rc;
    // FFN (value.py:65-67: act after ff2; specification: act between)
    {
      Lin a; a.m = M; a.n = ff; a.k = d; a.bias = L.bff1; a.lda = d; a.ldw = d; a.ldc = ff;
      a.act = c.ffn_act_pos == CRL_FFN_ACT_MID ? act : kActNone;
      a.precise_act = (prec & CRL_PREC_MISH_F32) != 0;
      if (f8_ffn) { a.kind = kKindF8; a.a = w.x8; a.w = L.wff1_8; a.alpha = 1.0f / (L.sa_ffn * L.sw_ff1); a.c = w.t1_8; a.out = kOutE4M3; a.out_scale = L.sa_hid; a.bias = L.bff1_8; }
      else if (i8) { a.kind = kKindI8; a.a = w.x8; a.w = L.wff1_q; a.row_scale = w.xs; a.col_scale = L.cs_ff1; a.c = w.t1; }
      else { a.a = ffn_in; a.w = L.wff1; a.c = w.t1; }
      if (fuse_ln) {               // norm1 of this block: w.y -> w.x (+ w.x8), inside this kernel
        a.ln_y = w.y; a.ln_w16 = L.ln1w16; a.ln_b16 = L.ln1b16; a.ln_x = w.x; a.ln_x8 = f8 ? w.x8 : nullptr; a.ln_out8_scale = L.sa_ffn;
      }
      if ((rc = linear(h, a, s)) != CRL_OK) return rc;
      if (i8 && (rc = quant_rows_i8(h, w.t1, M, ff, w.t1_8, w.t1s, s)) != CRL_OK) return rc;
      if (calib && (rc = tap_amax(h, w.t1, M, ff, l * 8 + 3, s)) != CRL_OK) return rc;
      if (calib && (rc = tap_mean(h, w.t1, M, ff, ff, l, 3, s)) != CRL_OK) return rc;
      Lin b; b.m = M; b.n = d; b.k = ff; b.bias = L.bff2; b.lda = ff; b.ldw = ff; b.res = w.x; b.ldr = d;
      b.act = c.ffn_act_pos == CRL_FFN_ACT_END ? act : kActNone;
      b.c = c.ln_mode == CRL_LN_POST ? w.y : w.x; b.ldc = d;
      if (f8_ffn) { b.kind = kKindF8; b.a = w.t1_8; b.w = L.wff2_8; b.alpha = 1.0f / (L.sa_hid * L.sw_ff2); b.bias = L.bff2_8; }
      else if (i8) { b.kind = kKindI8; b.a = w.t1_8; b.w = L.wff2_q; b.row_scale = w.t1s; b.col_scale = L.cs_ff2; }
      else { b.a = w.t1; b.w = L.wff2; }
      if (lno) {
        const bool emit8 = (f8 || i8) && l + 1 < c.n_layers;
        b.c = w.x; b.lno_w16 = L.ln2w16; b.lno_b16 = L.ln2b16; b.lno_x8 = emit8 ? w.x8 : nullptr;
        b.lno_out8_scale = (emit8 && f8) ? h->layers[l + 1].sa_in : 1.0f; b.lno_qscale = (emit8 && i8) ? w.xs : nullptr;
        b.lno_stats = w.lno_stats;
      }
      if ((rc = linear(h, b, s)) != CRL_OK) return rc;
    }
    if (c.ln_mode == CRL_LN_POST && !lno && !(fuse_ln && l + 1 < c.n_layers)) {
      const bool emit8 = f8 && l + 1 < c.n_layers;
      if ((rc = layer_norm(h, w.y, M, d, L.ln2w, L.ln2b, w.x, emit8 ? w.x8 : nullptr,
                           emit8 ? h->layers[l + 1].sa_in : 1.0f, nullptr, nullptr, s,
                           (i8 && l + 1 < c.n_layers) ? xq : nullptr, w.xs)) != CRL_OK)
        return rc;
    }
  }
  if (c.ln_mode == CRL_LN_PRE) {
    if ((rc = layer_norm(h, w.x, M, d, h->lnF_w, h->lnF_b, w.x, nullptr, 1.0f, nullptr, nullptr, s)) != CRL_OK) return rc;
  }
  if (calib) return CRL_OK;

  // ---- value heads (value.py:402-435, value_q.py:430-464) --------------------------------------------
  if (c.value_mode != CRL_VALUE_NONE && io->wdl_out != nullptr) {
    if ((rc = value_head(h, h->vh, w.x, w.t1, w.v2, bc, io->wdl_out + b0 * 3, io->wdl_softmax ? 1 : 0, s)) != CRL_OK) return rc;
  }
  if (c.value_mode == CRL_VALUE_WDL_Q && io->q_out != nullptr) {
    if ((rc = value_head(h, h->vq, w.x, w.t1, w.v2q, bc, io->q_out + b0, 2, s)) != CRL_OK) return rc;
  }

  // ---- last-token LM head of the decoder model (model_bis.py:369-370, 383-389) ----------------------------
  if (c.policy_mode == CRL_POLICY_LM_HEAD && io->policy_out != nullptr) {
    const int V = c.lm_vocab;
    Lin e; e.a = w.x + static_cast<size_t>(63) * d; e.lda = static_cast<long long>(64) * d; e.w = h->w_ph; e.ldw = d;
    e.c = w.logits; e.ldc = 2048; e.out = kOutF32; e.m = bc; e.n = V; e.k = d;
    if ((rc = linear(h, e, s)) != CRL_OK) return rc;
    const char* mask = static_cast<const char*>(io->legal_mask);
    const void* mask_row = nullptr;
    if (mask != nullptr && io->mask_mode == CRL_MASK_BITS) mask_row = mask + b0 * io->mask_stride;
    if (mask != nullptr && io->mask_mode == CRL_MASK_ADDITIVE) mask_row = mask + b0 * io->mask_stride * 4;
    MaskRowsParams m{};
    m.logits = w.logits; m.ld = 2048; m.n = V; m.mask = mask_row; m.mask_mode = mask_row != nullptr ? io->mask_mode : CRL_MASK_NONE;
    m.mask_ld = io->mask_stride; m.softmax = io->policy_softmax;
    m.out_f32 = io->policy_dtype == CRL_OUT_F32 ? static_cast<float*>(io->policy_out) + b0 * io->policy_stride : nullptr;
    m.out_f16 = io->policy_dtype == CRL_OUT_F16 ? static_cast<__half*>(io->policy_out) + b0 * io->policy_stride : nullptr;
    m.out_ld = io->policy_stride;
    mask_rows_kernel<<<static_cast<unsigned>(bc), 128, 0, s>>>(m);
    CRL_CUDA(h, cudaGetLastError());
    ++h->launches;
  }

  // ---- policy head (value.py:173-187) -----------------------------------------------------------------
  if ((c.policy_mode == CRL_POLICY_DENSE4096 || c.policy_mode == CRL_POLICY_GATHER1858) && io->policy_out != nullptr) {
    Lin a; a.a = w.x; a.lda = d; a.w = h->w_pt; a.ldw = d; a.c = w.t2; a.ldc = d; a.m = M; a.n = d; a.k = d;
    a.bias = h->b_pt; a.act = kActGelu; a.res = h->pe16; a.ldr = d; a.res_mod = 64;
    if ((rc = linear(h, a, s)) != CRL_OK) return rc;
    Lin b; b.a = w.t2; b.lda = d; b.w = h->w_qk; b.ldw = d; b.c = w.t1; b.ldc = h->qk_ld; b.m = M; b.n = h->qk_ld; b.k = d;
    b.bias = h->b_qk;
    if ((rc = linear(h, b, s)) != CRL_OK) return rc;
    const int n_moves = crl_num_moves(h);
    const char* mask = static_cast<const char*>(io->legal_mask);
    const void* mask_row = nullptr;
    if (mask != nullptr && io->mask_mode == CRL_MASK_BITS) mask_row = mask + b0 * io->mask_stride;
    if (mask != nullptr && io->mask_mode == CRL_MASK_ADDITIVE) mask_row = mask + b0 * io->mask_stride * 4;
    int mask_mode = mask_row != nullptr ? io->mask_mode : CRL_MASK_NONE;
    long long mask_ld = io->mask_stride;
    if (io->mask_mode == CRL_MASK_FROM_RECORDS) {   // generated for the whole call before the first pass
      mask_row = w.legal + b0 * 236; mask_mode = CRL_MASK_BITS; mask_ld = 236;
    }
    float* out32 = io->policy_dtype == CRL_OUT_F32 ? static_cast<float*>(io->policy_out) + b0 * io->policy_stride : nullptr;
    __half* out16 = io->policy_dtype == CRL_OUT_F16 ? static_cast<__half*>(io->policy_out) + b0 * io->policy_stride : nullptr;
    PolicyParams p{};
    p.qk = w.t1; p.ld = h->qk_ld; p.d = d; p.scale = 1.0f / std::sqrt(static_cast<float>(d));
    if (c.policy_mode == CRL_POLICY_DENSE4096) {
      p.flat = w.flat;
    } else {
      p.gather_idx = h->gather_idx; p.gather_promo = h->gather_promo; p.n_moves = n_moves;
      p.mask = mask_row; p.mask_mode = mask_mode; p.mask_ld = mask_ld; p.softmax = io->policy_softmax;
      p.out_f32 = out32; p.out_f16 = out16; p.out_ld = io->policy_stride;
      if (io->policy_vocab == CRL_VOCAB_RL1929) {
        p.mirror = h->mirror_idx; p.out_width = 1929;
        p.black_rows = io->black_rows != nullptr ? io->black_rows + b0 : nullptr;
      }
    }
    ProfScope ps(h, s, kCatOther, 2.0 * bc * 64 * 64 * d, static_cast<double>(M) * 2 * d * 2 + static_cast<double>(bc) * n_moves * 4);
    policy_scores_kernel<<<static_cast<unsigned>(bc), 128, 0, s>>>(p);
    CRL_CUDA(h, cudaGetLastError());
    ++h->launches;
    if (c.policy_mode == CRL_POLICY_DENSE4096) {
      Lin e; e.a = w.flat; e.lda = 4096; e.w = h->w_ph; e.ldw = 4096; e.c = w.logits; e.ldc = 2048; e.out = kOutF32;
      e.m = bc; e.n = 1929; e.k = 4096;
      if ((rc = linear(h, e, s)) != CRL_OK) return rc;
      MaskRowsParams m{};
      m.logits = w.logits; m.ld = 2048; m.n = 1929; m.mask = mask_row; m.mask_mode = mask_mode; m.mask_ld = mask_ld;
      m.softmax = io->policy_softmax; m.out_f32 = out32; m.out_f16 = out16; m.out_ld = io->policy_stride;
      mask_rows_kernel<<<static_cast<unsigned>(bc), 128, 0, s>>>(m);
      CRL_CUDA(h, cudaGetLastError());
      ++h->launches;
    }
  }
  return CRL_OK;
}

int check_io(crl_handle* h, const crl_io* io) {
  if (h == nullptr || io == nullptr) return CRL_ERR_INVALID;
  if (!h->finalized) return fail(h, CRL_ERR_NOT_FINALIZED, "crl_finalize has not run");
  if (io->batch < 0) return fail(h, CRL_ERR_INVALID, "negative batch");
  if (io->batch > 0 && io->planes == nullptr) return fail(h, CRL_ERR_INVALID, "planes is null");
  if (io->layout < 0 || io->layout > CRL_LAYOUT_PACKED104) return fail(h, CRL_ERR_INVALID, "unknown plane layout");
  if (io->layout == CRL_LAYOUT_PACKED104 && h->cfg.planes != 112) return fail(h, CRL_ERR_INVALID, "the packed layout holds 112 planes");
  if (io->layout == CRL_LAYOUT_PACKED104 && (reinterpret_cast<uintptr_t>(io->planes) & 3) != 0) return fail(h, CRL_ERR_INVALID, "packed planes must be 4-byte aligned");
  if (io->mask_mode < 0 || io->mask_mode > CRL_MASK_FROM_RECORDS) return fail(h, CRL_ERR_INVALID, "unknown mask mode");
  if (io->mask_mode == CRL_MASK_FROM_RECORDS && (io->layout != CRL_LAYOUT_PACKED104 || h->cfg.policy_mode != CRL_POLICY_GATHER1858))
    return fail(h, CRL_ERR_INVALID, "masks from records need the packed input layout and the 1858-move gather head");
  const int n_moves = crl_num_moves(h);
  if (io->policy_out != nullptr || io->move_out != nullptr) {
    if (n_moves == 0) return fail(h, CRL_ERR_INVALID, "policy_out given but the configuration has no policy head");
    if (io->policy_vocab != CRL_VOCAB_NATIVE && io->policy_vocab != CRL_VOCAB_RL1929) return fail(h, CRL_ERR_INVALID, "unknown policy_vocab");
    if (io->policy_vocab == CRL_VOCAB_RL1929 && h->cfg.policy_mode != CRL_POLICY_GATHER1858)
      return fail(h, CRL_ERR_INVALID, "policy_vocab RL1929 needs the 1858-move gather head");
    if (io->policy_out != nullptr && io->policy_stride < (io->policy_vocab == CRL_VOCAB_RL1929 ? 1929 : n_moves))
      return fail(h, CRL_ERR_SHAPE, "policy_stride smaller than the move count");
    if (io->policy_out != nullptr && io->policy_dtype != CRL_OUT_F32 && io->policy_dtype != CRL_OUT_F16)
      return fail(h, CRL_ERR_INVALID, "unknown policy dtype");
    if (io->legal_mask != nullptr && io->mask_mode == CRL_MASK_BITS && io->mask_stride * 8 < n_moves)
      return fail(h, CRL_ERR_SHAPE, "mask_stride too small for a bitset over the moves");
    if (io->legal_mask != nullptr && io->mask_mode == CRL_MASK_ADDITIVE && io->mask_stride < n_moves)
      return fail(h, CRL_ERR_SHAPE, "mask_stride smaller than the move count");
  }
  if (io->move_out != nullptr) {
    if (n_moves == 0) return fail(h, CRL_ERR_INVALID, "move_out given but the configuration has no policy head");
    if (io->move_temperature < 0.0f || !(io->move_temperature == io->move_temperature))
      return fail(h, CRL_ERR_INVALID, "move_temperature must be >= 0");
  }
  if (io->wdl_out != nullptr && h->cfg.value_mode == CRL_VALUE_NONE)
    return fail(h, CRL_ERR_INVALID, "wdl_out given but the configuration has no value head");
  if (io->q_out != nullptr && h->cfg.value_mode != CRL_VALUE_WDL_Q)
    return fail(h, CRL_ERR_INVALID, "q_out given but the configuration has no Q head");
  if (h->cfg.dtype == CRL_DTYPE_F8E4M3 && !h->calibrated)
    return fail(h, CRL_ERR_NOT_FINALIZED, "FP8 engine needs crl_calibrate before crl_forward");
  return CRL_OK;
}

int run_batch(crl_handle* h, const crl_io* io, bool calib) {
  CRL_ON_DEVICE(h);
  cudaStream_t s = static_cast<cudaStream_t>(io->stream);
  if (io->batch == 0) return CRL_OK;
  const int64_t chunk = std::min<int64_t>(h->chunk, io->batch);
  const size_t need = carve(h, nullptr, chunk, io->batch).total;
  if (io->workspace == nullptr || io->workspace_bytes < need)
    return fail(h, CRL_ERR_WORKSPACE, "workspace needs " + std::to_string(need) + " bytes");
  if ((reinterpret_cast<uintptr_t>(io->workspace) & 255) != 0) return fail(h, CRL_ERR_SHAPE, "workspace must be 256-byte aligned");
  const Workspace w = carve(h, static_cast<char*>(io->workspace), chunk, io->batch);
  if (io->mask_mode == CRL_MASK_FROM_RECORDS && io->policy_out != nullptr && !calib) {
    // one thread per position: all positions of the call in one launch keep the whole GPU busy
    MoveGenParams mg{};
    mg.recs = static_cast<const uint8_t*>(io->planes); mg.batch = io->batch;
    mg.plain_idx = h->plain_idx; mg.bits = w.legal; mg.stride = 236;
    legal_mask_packed104_kernel<<<static_cast<unsigned>((io->batch + 63) / 64), 64, 0, s>>>(mg);
    CRL_CUDA(h, cudaGetLastError());
    ++h->launches;
  }
  for (int64_t b0 = 0; b0 < io->batch; b0 += chunk) {
    const int64_t bc = std::min<int64_t>(chunk, io->batch - b0);
    const int rc = forward_chunk(h, io, b0, bc, w, calib, s);
    if (rc != CRL_OK) return rc;
  }
  if (io->move_out != nullptr && !calib) {
    SampleParams sp{};
    sp.r32 = io->policy_dtype == CRL_OUT_F32 ? static_cast<const float*>(io->policy_out) : nullptr;
    sp.r16 = io->policy_dtype == CRL_OUT_F16 ? static_cast<const __half*>(io->policy_out) : nullptr;
    sp.ld = io->policy_stride;
    sp.n = io->policy_vocab == CRL_VOCAB_RL1929 ? 1929 : crl_num_moves(h);
    sp.rows = io->batch;
    sp.is_prob = io->policy_softmax;
    sp.inv_t = io->move_temperature > 0.0f ? 1.0f / io->move_temperature : 0.0f;
    sp.u = io->move_uniform;
    sp.out = io->move_out;
    sample_rows_kernel<<<static_cast<unsigned>((io->batch + 7) / 8), 256, 0, s>>>(sp);
    CRL_CUDA(h, cudaGetLastError());
    ++h->launches;
  }
  return CRL_OK;
}

template <typename T>
int grow(crl_handle* h, T** p, size_t* have, size_t need) {
  if (*have >= need) return CRL_OK;
  if (*p != nullptr) CRL_CUDA(h, cudaFree(*p));
  *p = nullptr; *have = 0;
  void* q = nullptr;
  CRL_CUDA(h, cudaMalloc(&q, need));
  *p = static_cast<T*>(q);
  *have = need;
  return CRL_OK;
}

// FP8 bias correction. The e4m3 copy W' of a weight matrix differs from W by a fixed, known rounding error; for
// inputs x its effect on the output is (W' - W) x, whose mean over the data is (W' - W) mean(x). Subtracting that
// from the bias removes the coherent part of the weight-rounding error (on the benchmark network it is half of the
// rms logit error) at no cost per call. mean(x) comes from the calibration pass: column sums of the four GEMM
// inputs of every layer.
int correct_fp8_biases(crl_handle* h, long long rows, cudaStream_t s) {
  const crl_config& c = h->cfg;
  const int d = c.d_model, ff = c.d_ff, L = c.n_layers, wide = std::max(d, ff);
  const float inv_rows = 1.0f / static_cast<float>(rows);
  auto run = [&](const __half* W, const uint8_t* W8, float mult, const float* colsum, const float* bias, float* out, int n_out, int k_in) {
    bias_correct_kernel<<<(n_out + 7) / 8, 256, 0, s>>>(W, W8, 1.0f / mult, colsum, inv_rows, bias, out, n_out, k_in);
  };
  for (int l = 0; l < L; ++l) {
    LayerW& Lw = h->layers[l];
    const float* m = h->mean_dev + static_cast<size_t>(l) * 4 * wide;
    run(Lw.wqkv, Lw.wqkv8, Lw.sw_qkv, m, Lw.bqkv, Lw.bqkv8, 3 * d, d);
    run(Lw.wo, Lw.wo8, Lw.sw_o, m + wide, Lw.bo, Lw.bo8, d, d);
    run(Lw.wff1, Lw.wff1_8, Lw.sw_ff1, m + 2 * wide, Lw.bff1, Lw.bff1_8, ff, d);
    run(Lw.wff2, Lw.wff2_8, Lw.sw_ff2, m + 3 * wide, Lw.bff2, Lw.bff2_8, d, ff);
  }
  CRL_CUDA(h, cudaGetLastError());
  CRL_CUDA(h, cudaStreamSynchronize(s));
  return CRL_OK;
}

size_t plane_bytes(const crl_handle* h, int layout) {
  if (layout == CRL_LAYOUT_PACKED104) return CRL_PACKED104_BYTES;
  const size_t e = (layout == CRL_LAYOUT_NHWC_F32 || layout == CRL_LAYOUT_NCHW_F32) ? 4 : 2;
  return static_cast<size_t>(64) * h->cfg.planes * e;
}

}  // namespace

// =====================================================================================================
extern "C" {

const char* crl_strerror(int status) {
  switch (status) {
    case CRL_OK: return "ok";
    case CRL_ERR_INVALID: return "invalid argument";
    case CRL_ERR_SHAPE: return "unsupported shape or alignment";
    case CRL_ERR_CUDA: return "CUDA error";
    case CRL_ERR_MISSING_WEIGHT: return "missing weight";
    case CRL_ERR_NOT_FINALIZED: return "handle not finalized (or FP8 engine not calibrated)";
    case CRL_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    case CRL_ERR_WORKSPACE: return "workspace too small";
    case CRL_ERR_UNSUPPORTED: return "unsupported configuration";
    default: return "unknown status";
  }
}

const char* crl_error_detail(const crl_handle* h) { return h != nullptr ? h->detail.c_str() : ""; }

int crl_create(const crl_config* cfg, int device, crl_handle** out) {
  if (cfg == nullptr || out == nullptr) return CRL_ERR_INVALID;
  *out = nullptr;
  const crl_config& c = *cfg;
  if (c.planes <= 0 || c.d_model <= 0 || c.n_layers <= 0 || c.n_heads <= 0 || c.d_ff <= 0) return CRL_ERR_INVALID;
  if (c.d_model % c.n_heads != 0) return CRL_ERR_SHAPE;
  const int hd = c.d_model / c.n_heads;
  if (hd != 32 && hd != 64) return CRL_ERR_SHAPE;
  if (c.d_model % 64 != 0 || c.d_model > 1024 || c.d_ff % 16 != 0) return CRL_ERR_SHAPE;
  if (c.ln_mode < 0 || c.ln_mode > 1 || (c.act != CRL_ACT_GELU && c.act != CRL_ACT_MISH) || c.ffn_act_pos < 0 || c.ffn_act_pos > 1 ||
      c.bias_mode < 0 || c.bias_mode > 3 || c.policy_mode < 0 || c.policy_mode > 3 || c.value_mode < 0 || c.value_mode > 2)
    return CRL_ERR_INVALID;
  if (c.dtype != CRL_DTYPE_F16 && c.dtype != CRL_DTYPE_F8E4M3 && c.dtype != CRL_DTYPE_I8) return CRL_ERR_UNSUPPORTED;
  if (c.fuse_layernorm < 0 || c.fuse_layernorm > CRL_FUSE_LN_OFF || c.precision < 0 || c.precision > 63) return CRL_ERR_INVALID;
  if (c.dtype == CRL_DTYPE_I8 && (c.d_model % 16 != 0 || c.d_ff % 16 != 0)) return CRL_ERR_SHAPE;
  if (c.policy_mode == CRL_POLICY_LM_HEAD && (c.lm_vocab <= 0 || c.lm_vocab > 2048)) return CRL_ERR_SHAPE;
  if (c.bias_mode == CRL_BIAS_SMOLGEN &&
      (c.smolgen_compress <= 0 || c.smolgen_compress % 8 != 0 || c.smolgen_hidden % 8 != 0 || c.smolgen_hidden > 1024 ||
       c.smolgen_gen % 8 != 0 || c.smolgen_gen > 1024 || c.smolgen_hidden <= 0 || c.smolgen_gen <= 0))
    return CRL_ERR_SHAPE;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return CRL_ERR_CUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return CRL_ERR_CUDA;
  if (prop.major != 10) return CRL_ERR_UNSUPPORTED;   // the kernels are sm_100a only
  DeviceGuard guard(device);
  if (!guard.ok) return CRL_ERR_CUDA;
  crl_handle* h = new crl_handle();
  h->cfg = c;
  h->device = device;
  h->num_sms = prop.multiProcessorCount;
  h->hd = hd;
  h->ppad = (c.planes + 7) / 8 * 8;
  h->qk_ld = c.policy_mode == CRL_POLICY_GATHER1858 ? 2 * c.d_model + 8 : 2 * c.d_model;
  h->chunk = c.chunk > 0 ? c.chunk : 8192;   // larger passes amortise launch gaps and tile tails: 8192 measured 3 % faster than 2048
  build_required(h);
  void* p = nullptr;
  if (cudaMalloc(&p, 16) != cudaSuccess) { delete h; return CRL_ERR_CUDA; }
  h->status_dev = static_cast<int*>(p);
  cudaMemset(p, 0, 16);
  h->allocs.push_back(p);
  if (cudaMalloc(&p, sizeof(unsigned int) * 8 * c.n_layers) != cudaSuccess) { crl_destroy(h); return CRL_ERR_CUDA; }
  h->amax_dev = static_cast<unsigned int*>(p);
  h->allocs.push_back(p);
  *out = h;
  return CRL_OK;
}

void crl_destroy(crl_handle* h) {
  if (h == nullptr) return;
  DeviceGuard guard(h->device);
  for (void* p : h->allocs) cudaFree(p);
  for (auto& r : h->prof) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
  for (void* p : {h->st_move, h->st_black, h->st_planes, h->st_mask, h->st_policy, h->st_wdl, h->st_q, h->st_ws})
    if (p != nullptr) cudaFree(p);
  delete h;
}

int crl_num_required_keys(const crl_handle* h) { return h != nullptr ? static_cast<int>(h->required.size()) : 0; }
const char* crl_required_key(const crl_handle* h, int i) {
  if (h == nullptr || i < 0 || i >= static_cast<int>(h->required.size())) return nullptr;
  return h->required[i].c_str();
}

int crl_set_weight(crl_handle* h, const char* key, const float* data, int64_t numel) {
  if (h == nullptr || key == nullptr || data == nullptr || numel <= 0) return CRL_ERR_INVALID;
  if (std::find(h->required.begin(), h->required.end(), key) == h->required.end())
    return fail(h, CRL_ERR_INVALID, std::string("unexpected key ") + key);
  CRL_ON_DEVICE(h);
  std::vector<float>& v = h->raw[key];
  v.resize(static_cast<size_t>(numel));
  CRL_CUDA(h, cudaMemcpy(v.data(), data, static_cast<size_t>(numel) * sizeof(float), cudaMemcpyDefault));
  h->finalized = false;
  return CRL_OK;
}

int crl_num_moves(const crl_handle* h) {
  if (h == nullptr) return 0;
  if (h->cfg.policy_mode == CRL_POLICY_DENSE4096) return 1929;
  if (h->cfg.policy_mode == CRL_POLICY_GATHER1858) return 1858;
  if (h->cfg.policy_mode == CRL_POLICY_LM_HEAD) return h->cfg.lm_vocab;
  return 0;
}

int crl_finalize(crl_handle* h) {
  if (h == nullptr) return CRL_ERR_INVALID;
  CRL_ON_DEVICE(h);
  const crl_config& c = h->cfg;
  const size_t d = c.d_model, ff = c.d_ff, H = c.n_heads, P = c.planes;
  // --- every key present with the right size ---
  std::vector<Expect> ex;
  for (int l = 0; l < c.n_layers; ++l) {
    for (const char* t : {"attention.query_proj", "attention.key_proj", "attention.value_proj", "attention.out_proj"}) {
      ex.push_back({lkey(l, (std::string(t) + ".weight").c_str()), d * d});
      ex.push_back({lkey(l, (std::string(t) + ".bias").c_str()), d});
    }
    for (const char* t : {"norm1.weight", "norm1.bias", "norm2.weight", "norm2.bias", "ff2.bias"}) ex.push_back({lkey(l, t), d});
    ex.push_back({lkey(l, "ff1.weight"), ff * d}); ex.push_back({lkey(l, "ff1.bias"), ff}); ex.push_back({lkey(l, "ff2.weight"), d * ff});
    if (c.bias_mode == CRL_BIAS_RELPOS) {
      ex.push_back({lkey(l, "attention.pos_proj.weight"), d * d});
      ex.push_back({lkey(l, "attention.u_bias"), d}); ex.push_back({lkey(l, "attention.v_bias"), d});
    }
    if (c.bias_mode == CRL_BIAS_SMOLGEN) {
      const size_t cc = c.smolgen_compress, hid = c.smolgen_hidden, gen = c.smolgen_gen;
      ex.push_back({lkey(l, "smolgen.compress.weight"), cc * d});
      ex.push_back({lkey(l, "smolgen.dense1.weight"), hid * 64 * cc}); ex.push_back({lkey(l, "smolgen.dense1.bias"), hid});
      ex.push_back({lkey(l, "smolgen.ln1.weight"), hid}); ex.push_back({lkey(l, "smolgen.ln1.bias"), hid});
      ex.push_back({lkey(l, "smolgen.dense2.weight"), H * gen * hid}); ex.push_back({lkey(l, "smolgen.dense2.bias"), H * gen});
      ex.push_back({lkey(l, "smolgen.ln2.weight"), gen}); ex.push_back({lkey(l, "smolgen.ln2.bias"), gen});
    }
  }
  ex.push_back({"linear1.weight", d * P}); ex.push_back({"linear1.bias", d});
  ex.push_back({"layernorm1.weight", d}); ex.push_back({"layernorm1.bias", d});
  ex.push_back({"ma_gating.a", 64 * d}); ex.push_back({"ma_gating.b", 64 * d});
  if (c.bias_mode == CRL_BIAS_SMOLGEN) ex.push_back({"smolgen_shared.weight", static_cast<size_t>(4096) * c.smolgen_gen});
  if (c.ln_mode == CRL_LN_PRE) { ex.push_back({"norm_f.weight", d}); ex.push_back({"norm_f.bias", d}); }
  if (c.policy_mode == CRL_POLICY_LM_HEAD) ex.push_back({"lm_head.weight", static_cast<size_t>(c.lm_vocab) * d});
  if (c.policy_mode == CRL_POLICY_DENSE4096 || c.policy_mode == CRL_POLICY_GATHER1858)
    for (const char* t : {"policy_tokens_lin", "queries_pol", "keys_pol"}) {
      ex.push_back({std::string(t) + ".weight", d * d}); ex.push_back({std::string(t) + ".bias", d});
    }
  if (c.policy_mode == CRL_POLICY_DENSE4096) ex.push_back({"policy_head.weight", static_cast<size_t>(1929) * 4096});
  if (c.policy_mode == CRL_POLICY_GATHER1858) ex.push_back({"policy_promo.weight", 3 * d});
  auto value_keys = [&](const std::string& pre, size_t n_out) {
    ex.push_back({pre + ".dense1.weight", 128 * d}); ex.push_back({pre + ".dense1.bias", 128});
    ex.push_back({pre + ".dense2.weight", static_cast<size_t>(128) * 8192}); ex.push_back({pre + ".dense2.bias", 128});
    ex.push_back({pre + ".dense3.weight", n_out * 128}); ex.push_back({pre + ".dense3.bias", n_out});
  };
  if (c.value_mode != CRL_VALUE_NONE) value_keys("value_head", 3);
  if (c.value_mode == CRL_VALUE_WDL_Q) value_keys("value_head_q", 1);
  if (c.pos_embed) {
    const std::vector<float>* v = get(h, "pe");
    if (v == nullptr) return fail(h, CRL_ERR_MISSING_WEIGHT, "pe");
    if (v->size() < 64 * d || v->size() % d != 0) return fail(h, CRL_ERR_SHAPE, "pe: expected [>=64, d_model]");
  }
  for (const Expect& e : ex) {
    const std::vector<float>* v = get(h, e.key);
    if (v == nullptr) return fail(h, CRL_ERR_MISSING_WEIGHT, e.key);
    if (v->size() != e.numel)
      return fail(h, CRL_ERR_SHAPE, e.key + ": expected " + std::to_string(e.numel) + " elements, got " + std::to_string(v->size()));
  }
  // --- drop earlier device copies (a second finalize after new weights) ---
  for (size_t i = 2; i < h->allocs.size(); ++i) cudaFree(h->allocs[i]);
  h->allocs.resize(2);
  h->layers.assign(c.n_layers, LayerW());
  h->calibrated = false;

  int rc;
#define UP16(dst, key, rows, cols, ld) if ((rc = upload_f16(h, &(dst), get(h, key)->data(), rows, cols, ld)) != CRL_OK) return rc
#define UP32(dst, key, n) if ((rc = upload_f32(h, &(dst), get(h, key)->data(), n)) != CRL_OK) return rc
  // sinusoid table (value.py:77-88)
  std::vector<float> pe(64 * d);
  for (size_t pos = 0; pos < 64; ++pos)
    for (size_t i = 0; i < d; i += 2) {
      const float div = std::pow(10000.0f, static_cast<float>(i) / static_cast<float>(d));
      pe[pos * d + i] = std::sin(static_cast<float>(pos) / div);
      if (i + 1 < d) pe[pos * d + i + 1] = std::cos(static_cast<float>(pos) / div);
    }
  if ((rc = upload_f16(h, &h->pe16, pe.data(), 64, d, d)) != CRL_OK) return rc;

  UP16(h->w_embed, "linear1.weight", d, P, h->ppad);
  UP32(h->b_embed, "linear1.bias", d);
  UP32(h->lnE_w, "layernorm1.weight", d);
  UP32(h->lnE_b, "layernorm1.bias", d);
  {
    std::vector<float> ea(*get(h, "ma_gating.a"));
    for (float& x : ea) x = std::exp(x);
    if ((rc = upload_f32(h, &h->gate_ea, ea.data(), ea.size())) != CRL_OK) return rc;
    // positions added right after the gating (model_bis.py:363-366) fold into the gating offset
    std::vector<float> gb(*get(h, "ma_gating.b"));
    if (c.pos_embed) {
      const std::vector<float>& pev = *get(h, "pe");
      for (size_t i = 0; i < 64 * d; ++i) gb[i] += pev[i];
    }
    if ((rc = upload_f32(h, &h->gate_b, gb.data(), gb.size())) != CRL_OK) return rc;
  }
  for (int l = 0; l < c.n_layers; ++l) {
    LayerW& L = h->layers[l];
    std::vector<float> wqkv(3 * d * d), bqkv(3 * d);
    const char* names[3] = {"attention.query_proj", "attention.key_proj", "attention.value_proj"};
    for (int i = 0; i < 3; ++i) {
      const auto* wv = get(h, lkey(l, (std::string(names[i]) + ".weight").c_str()));
      const auto* bv = get(h, lkey(l, (std::string(names[i]) + ".bias").c_str()));
      std::copy(wv->begin(), wv->end(), wqkv.begin() + i * d * d);
      std::copy(bv->begin(), bv->end(), bqkv.begin() + i * d);
    }
    if ((rc = upload_f16(h, &L.wqkv, wqkv.data(), 3 * d, d, d)) != CRL_OK) return rc;
    if ((rc = upload_f32(h, &L.bqkv, bqkv.data(), 3 * d)) != CRL_OK) return rc;
    UP16(L.wo, lkey(l, "attention.out_proj.weight"), d, d, d);
    UP32(L.bo, lkey(l, "attention.out_proj.bias"), d);
    UP32(L.ln1w, lkey(l, "norm1.weight"), d); UP32(L.ln1b, lkey(l, "norm1.bias"), d);
    UP32(L.ln2w, lkey(l, "norm2.weight"), d); UP32(L.ln2b, lkey(l, "norm2.bias"), d);
    UP16(L.ln1w16, lkey(l, "norm1.weight"), 1, d, d); UP16(L.ln1b16, lkey(l, "norm1.bias"), 1, d, d);
    UP16(L.ln2w16, lkey(l, "norm2.weight"), 1, d, d); UP16(L.ln2b16, lkey(l, "norm2.bias"), 1, d, d);
    UP16(L.wff1, lkey(l, "ff1.weight"), ff, d, d); UP32(L.bff1, lkey(l, "ff1.bias"), ff);
    UP16(L.wff2, lkey(l, "ff2.weight"), d, ff, ff); UP32(L.bff2, lkey(l, "ff2.bias"), d);
    if (c.bias_mode == CRL_BIAS_RELPOS) {
      // P = pos_proj(sinusoid) is the same for every board (attn.py:505): fold it here, in fp32
      const auto& wp = *get(h, lkey(l, "attention.pos_proj.weight"));
      std::vector<float> pos(64 * d);
      for (size_t t = 0; t < 64; ++t)
        for (size_t o = 0; o < d; ++o) {
          float acc = 0.0f;
          for (size_t k = 0; k < d; ++k) acc += pe[t * d + k] * wp[o * d + k];
          pos[t * d + o] = acc;
        }
      if ((rc = upload_f16(h, &L.pos, pos.data(), 64, d, d)) != CRL_OK) return rc;
      UP16(L.u, lkey(l, "attention.u_bias"), 1, d, d);
      UP16(L.v, lkey(l, "attention.v_bias"), 1, d, d);
    }
    if (c.bias_mode == CRL_BIAS_SMOLGEN) {
      const size_t cc = c.smolgen_compress, hid = c.smolgen_hidden, gen = c.smolgen_gen;
      UP16(L.sg_wc, lkey(l, "smolgen.compress.weight"), cc, d, d);
      UP16(L.sg_w1, lkey(l, "smolgen.dense1.weight"), hid, 64 * cc, 64 * cc); UP32(L.sg_b1, lkey(l, "smolgen.dense1.bias"), hid);
      UP32(L.sg_ln1w, lkey(l, "smolgen.ln1.weight"), hid); UP32(L.sg_ln1b, lkey(l, "smolgen.ln1.bias"), hid);
      UP16(L.sg_w2, lkey(l, "smolgen.dense2.weight"), H * gen, hid, hid); UP32(L.sg_b2, lkey(l, "smolgen.dense2.bias"), H * gen);
      UP32(L.sg_ln2w, lkey(l, "smolgen.ln2.weight"), gen); UP32(L.sg_ln2b, lkey(l, "smolgen.ln2.bias"), gen);
    }
    if (c.dtype == CRL_DTYPE_I8) {
      if ((rc = upload_i8_rows(h, &L.wqkv_q, &L.cs_qkv, wqkv.data(), 3 * d, d)) != CRL_OK) return rc;
      if ((rc = upload_i8_rows(h, &L.wo_q, &L.cs_o, get(h, lkey(l, "attention.out_proj.weight"))->data(), d, d)) != CRL_OK) return rc;
      if ((rc = upload_i8_rows(h, &L.wff1_q, &L.cs_ff1, get(h, lkey(l, "ff1.weight"))->data(), ff, d)) != CRL_OK) return rc;
      if ((rc = upload_i8_rows(h, &L.wff2_q, &L.cs_ff2, get(h, lkey(l, "ff2.weight"))->data(), d, ff)) != CRL_OK) return rc;
    }
    if (c.dtype == CRL_DTYPE_F8E4M3) {
      if ((rc = upload_e4m3(h, &L.wqkv8, &L.sw_qkv, wqkv.data(), wqkv.size())) != CRL_OK) return rc;
      if ((rc = upload_f32(h, &L.bqkv8, bqkv.data(), 3 * d)) != CRL_OK) return rc;
      if ((rc = upload_f32(h, &L.bo8, get(h, lkey(l, "attention.out_proj.bias"))->data(), d)) != CRL_OK) return rc;
      if ((rc = upload_f32(h, &L.bff1_8, get(h, lkey(l, "ff1.bias"))->data(), ff)) != CRL_OK) return rc;
      if ((rc = upload_f32(h, &L.bff2_8, get(h, lkey(l, "ff2.bias"))->data(), d)) != CRL_OK) return rc;
      const auto& wo = *get(h, lkey(l, "attention.out_proj.weight"));
      const auto& w1 = *get(h, lkey(l, "ff1.weight"));
      const auto& w2 = *get(h, lkey(l, "ff2.weight"));
      if ((rc = upload_e4m3(h, &L.wo8, &L.sw_o, wo.data(), wo.size())) != CRL_OK) return rc;
      if ((rc = upload_e4m3(h, &L.wff1_8, &L.sw_ff1, w1.data(), w1.size())) != CRL_OK) return rc;
      if ((rc = upload_e4m3(h, &L.wff2_8, &L.sw_ff2, w2.data(), w2.size())) != CRL_OK) return rc;
      if (c.bias_mode == CRL_BIAS_SMOLGEN) {
        const auto& wc = *get(h, lkey(l, "smolgen.compress.weight"));
        if ((rc = upload_e4m3(h, &L.sg_wc8, &L.sw_c, wc.data(), wc.size())) != CRL_OK) return rc;
      }
    }
  }
  if (c.bias_mode == CRL_BIAS_SMOLGEN) UP16(h->sg_shared, "smolgen_shared.weight", 4096, c.smolgen_gen, c.smolgen_gen);
  if (c.bias_mode == CRL_BIAS_SMOLGEN && c.dtype == CRL_DTYPE_F8E4M3) {
    const auto& ws = *get(h, "smolgen_shared.weight");
    if ((rc = upload_e4m3(h, &h->sg_shared8, &h->sw_shared, ws.data(), ws.size())) != CRL_OK) return rc;
  }
  if (c.ln_mode == CRL_LN_PRE) { UP32(h->lnF_w, "norm_f.weight", d); UP32(h->lnF_b, "norm_f.bias", d); }
  if (c.policy_mode == CRL_POLICY_LM_HEAD) UP16(h->w_ph, "lm_head.weight", c.lm_vocab, d, d);
  if (c.policy_mode == CRL_POLICY_DENSE4096 || c.policy_mode == CRL_POLICY_GATHER1858) {
    UP16(h->w_pt, "policy_tokens_lin.weight", d, d, d); UP32(h->b_pt, "policy_tokens_lin.bias", d);
    const size_t rows = h->qk_ld;
    std::vector<float> wqk(rows * d, 0.0f), bqk(rows, 0.0f);
    std::copy(get(h, "queries_pol.weight")->begin(), get(h, "queries_pol.weight")->end(), wqk.begin());
    std::copy(get(h, "keys_pol.weight")->begin(), get(h, "keys_pol.weight")->end(), wqk.begin() + d * d);
    std::copy(get(h, "queries_pol.bias")->begin(), get(h, "queries_pol.bias")->end(), bqk.begin());
    std::copy(get(h, "keys_pol.bias")->begin(), get(h, "keys_pol.bias")->end(), bqk.begin() + d);
    if (c.policy_mode == CRL_POLICY_GATHER1858)
      std::copy(get(h, "policy_promo.weight")->begin(), get(h, "policy_promo.weight")->end(), wqk.begin() + 2 * d * d);
    if ((rc = upload_f16(h, &h->w_qk, wqk.data(), rows, d, d)) != CRL_OK) return rc;
    if ((rc = upload_f32(h, &h->b_qk, bqk.data(), rows)) != CRL_OK) return rc;
  }
  if (c.policy_mode == CRL_POLICY_DENSE4096) UP16(h->w_ph, "policy_head.weight", 1929, 4096, 4096);
  {
    const Vocab& v = Vocab::get();
    std::vector<short> plain(4096, -1);
    for (size_t i = 0; i < v.from_to.size(); ++i)
      if (v.promo[i] == 0) plain[v.from_to[i]] = static_cast<short>(i);
    if ((rc = dev_alloc(h, &h->plain_idx, plain.size())) != CRL_OK) return rc;
    CRL_CUDA(h, cudaMemcpy(h->plain_idx, plain.data(), plain.size() * sizeof(short), cudaMemcpyHostToDevice));
  }
  if (c.policy_mode == CRL_POLICY_GATHER1858) {
    const Vocab& v = Vocab::get();
    if ((rc = dev_alloc(h, &h->gather_idx, v.from_to.size())) != CRL_OK) return rc;
    if ((rc = dev_alloc(h, &h->gather_promo, v.promo.size())) != CRL_OK) return rc;
    CRL_CUDA(h, cudaMemcpy(h->gather_idx, v.from_to.data(), v.from_to.size() * sizeof(short), cudaMemcpyHostToDevice));
    CRL_CUDA(h, cudaMemcpy(h->gather_promo, v.promo.data(), v.promo.size(), cudaMemcpyHostToDevice));
    std::vector<short> mir(v.mirror.begin(), v.mirror.end());
    if ((rc = dev_alloc(h, &h->mirror_idx, mir.size())) != CRL_OK) return rc;
    CRL_CUDA(h, cudaMemcpy(h->mirror_idx, mir.data(), mir.size() * sizeof(short), cudaMemcpyHostToDevice));
  }
  auto value_up = [&](ValueW& vw, const std::string& pre, int n_out) -> int {
    vw.n_out = n_out;
    UP16(vw.w1, pre + ".dense1.weight", 128, d, d); UP32(vw.b1, pre + ".dense1.bias", 128);
    UP16(vw.w2, pre + ".dense2.weight", 128, 8192, 8192); UP32(vw.b2, pre + ".dense2.bias", 128);
    UP32(vw.w3, pre + ".dense3.weight", static_cast<size_t>(n_out) * 128); UP32(vw.b3, pre + ".dense3.bias", n_out);
    return CRL_OK;
  };
  if (c.value_mode != CRL_VALUE_NONE && (rc = value_up(h->vh, "value_head", 3)) != CRL_OK) return rc;
  if (c.value_mode == CRL_VALUE_WDL_Q && (rc = value_up(h->vq, "value_head_q", 1)) != CRL_OK) return rc;
#undef UP16
#undef UP32
  CRL_CUDA(h, cudaDeviceSynchronize());
  h->finalized = true;
  return CRL_OK;
}

size_t crl_workspace_bytes(const crl_handle* h, int64_t batch) {
  if (h == nullptr || batch <= 0) return 0;
  return carve(h, nullptr, std::min<int64_t>(h->chunk, batch), batch).total;
}

int crl_forward(crl_handle* h, const crl_io* io) {
  int rc = check_io(h, io);
  if (rc != CRL_OK) return rc;
  if (io->move_out != nullptr && io->policy_out == nullptr) return fail(h, CRL_ERR_INVALID, "move_out needs policy_out (the rows it reads)");
  h->launches = 0;
  return run_batch(h, io, false);
}

int crl_calibrate(crl_handle* h, const void* planes, int32_t layout, int64_t batch, void* workspace,
                  size_t workspace_bytes, void* stream) {
  if (h == nullptr || planes == nullptr || batch <= 0) return CRL_ERR_INVALID;
  if (!h->finalized) return fail(h, CRL_ERR_NOT_FINALIZED, "crl_finalize has not run");
  if (layout < 0 || layout > CRL_LAYOUT_PACKED104) return fail(h, CRL_ERR_INVALID, "unknown plane layout");
  if (layout == CRL_LAYOUT_PACKED104 && h->cfg.planes != 112) return fail(h, CRL_ERR_INVALID, "the packed layout holds 112 planes");
  if (layout == CRL_LAYOUT_PACKED104 && (reinterpret_cast<uintptr_t>(planes) & 3) != 0) return fail(h, CRL_ERR_INVALID, "packed planes must be 4-byte aligned");
  CRL_ON_DEVICE(h);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int L = h->cfg.n_layers;
  CRL_CUDA(h, cudaMemsetAsync(h->amax_dev, 0, sizeof(unsigned int) * 8 * L, s));
  const int wide = std::max(h->cfg.d_model, h->cfg.d_ff);
  const bool correct = h->cfg.dtype == CRL_DTYPE_F8E4M3;
  if (correct) {
    if (h->mean_dev == nullptr) {
      int rc0 = dev_alloc(h, &h->mean_dev, static_cast<size_t>(L) * 4 * wide);
      if (rc0 == CRL_OK) rc0 = dev_alloc(h, &h->mean_part, static_cast<size_t>(64) * wide);
      if (rc0 != CRL_OK) return rc0;
    }
    CRL_CUDA(h, cudaMemsetAsync(h->mean_dev, 0, sizeof(float) * L * 4 * wide, s));
  }
  crl_io io{};
  io.planes = planes; io.layout = layout; io.batch = batch; io.workspace = workspace; io.workspace_bytes = workspace_bytes;
  io.stream = stream;
  int rc = run_batch(h, &io, true);
  if (rc != CRL_OK) return rc;
  std::vector<float> amax(8 * L);
  CRL_CUDA(h, cudaMemcpyAsync(amax.data(), h->amax_dev, sizeof(float) * 8 * L, cudaMemcpyDeviceToHost, s));
  CRL_CUDA(h, cudaStreamSynchronize(s));
  auto mult = [](float a) { return a > 0.0f ? kFp8Max / a : 1.0f; };
  for (int l = 0; l < L; ++l) {
    h->layers[l].sa_in = mult(amax[l * 8 + 0]);
    h->layers[l].sa_ctx = mult(amax[l * 8 + 1]);
    h->layers[l].sa_ffn = mult(amax[l * 8 + 2]);
    h->layers[l].sa_hid = mult(amax[l * 8 + 3]);
    h->layers[l].sa_bias = mult(amax[l * 8 + 4]);
    h->layers[l].sa_qkv = mult(amax[l * 8 + 5]);
    h->layers[l].sa_gen = mult(amax[l * 8 + 6]);
  }
  if (correct && (rc = correct_fp8_biases(h, batch * 64, s)) != CRL_OK) return rc;
  h->calibrated = true;
  return CRL_OK;
}

int crl_legal_masks_packed104(crl_handle* h, const void* packed, int64_t count, uint8_t* bits, int64_t stride, void* stream) {
  if (h == nullptr) return CRL_ERR_INVALID;
  if (!h->finalized) return fail(h, CRL_ERR_NOT_FINALIZED, "crl_finalize has not run");
  if (count < 0 || stride < 233 || (count > 0 && (packed == nullptr || bits == nullptr))) return fail(h, CRL_ERR_INVALID, "bad arguments");
  if (count == 0) return CRL_OK;
  CRL_ON_DEVICE(h);
  MoveGenParams mg{};
  mg.recs = static_cast<const uint8_t*>(packed); mg.batch = count; mg.plain_idx = h->plain_idx; mg.bits = bits; mg.stride = stride;
  legal_mask_packed104_kernel<<<static_cast<unsigned>((count + 63) / 64), 64, 0, static_cast<cudaStream_t>(stream)>>>(mg);
  CRL_CUDA(h, cudaGetLastError());
  return CRL_OK;
}

int crl_forward_host(crl_handle* h, const crl_io* io) {
  int rc = check_io(h, io);
  if (rc != CRL_OK) return rc;
  h->launches = 0;
  if (io->batch == 0) return CRL_OK;
  CRL_ON_DEVICE(h);
  cudaStream_t s = static_cast<cudaStream_t>(io->stream);
  const size_t B = static_cast<size_t>(io->batch);
  const size_t pb = plane_bytes(h, io->layout) * B;
  const size_t esz = io->policy_dtype == CRL_OUT_F32 ? 4 : 2;
  const size_t mb = io->legal_mask == nullptr ? 0 : (io->mask_mode == CRL_MASK_BITS ? B * io->mask_stride : (io->mask_mode == CRL_MASK_ADDITIVE ? B * io->mask_stride * 4 : 0));
  // moves without policy rows: the rows live in the staging buffer only (f16, dense) and are not copied back
  const bool own_rows = io->policy_out == nullptr && io->move_out != nullptr;
  const size_t own_stride = io->policy_vocab == CRL_VOCAB_RL1929 ? 1929 : static_cast<size_t>(crl_num_moves(h));
  const size_t ob = io->policy_out != nullptr ? B * io->policy_stride * esz : (own_rows ? B * own_stride * 2 : 0);
  if ((rc = grow(h, &h->st_planes, &h->st_planes_b, pb)) != CRL_OK) return rc;
  if (mb > 0 && (rc = grow(h, &h->st_mask, &h->st_mask_b, mb)) != CRL_OK) return rc;
  if (ob > 0 && (rc = grow(h, &h->st_policy, &h->st_policy_b, ob)) != CRL_OK) return rc;
  if (io->wdl_out != nullptr && (rc = grow(h, &h->st_wdl, &h->st_wdl_b, B * 12)) != CRL_OK) return rc;
  if (io->q_out != nullptr && (rc = grow(h, &h->st_q, &h->st_q_b, B * 4)) != CRL_OK) return rc;
  if ((rc = grow(h, &h->st_ws, &h->st_ws_b, crl_workspace_bytes(h, io->batch))) != CRL_OK) return rc;
  CRL_CUDA(h, cudaMemcpyAsync(h->st_planes, io->planes, pb, cudaMemcpyHostToDevice, s));
  if (mb > 0) CRL_CUDA(h, cudaMemcpyAsync(h->st_mask, io->legal_mask, mb, cudaMemcpyHostToDevice, s));
  if (io->black_rows != nullptr && io->policy_vocab == CRL_VOCAB_RL1929) {
    if ((rc = grow(h, &h->st_black, &h->st_black_b, B)) != CRL_OK) return rc;
    CRL_CUDA(h, cudaMemcpyAsync(h->st_black, io->black_rows, B, cudaMemcpyHostToDevice, s));
  }
  if (io->move_out != nullptr) {
    if ((rc = grow(h, &h->st_move, &h->st_move_b, B * 8)) != CRL_OK) return rc;
    if (io->move_uniform != nullptr)
      CRL_CUDA(h, cudaMemcpyAsync(static_cast<char*>(h->st_move) + B * 4, io->move_uniform, B * 4, cudaMemcpyHostToDevice, s));
  }
  crl_io dev = *io;
  if (own_rows) { dev.policy_stride = static_cast<int64_t>(own_stride); dev.policy_dtype = CRL_OUT_F16; }
  dev.move_out = io->move_out != nullptr ? static_cast<int32_t*>(h->st_move) : nullptr;
  dev.move_uniform = (io->move_out != nullptr && io->move_uniform != nullptr)
                         ? reinterpret_cast<const float*>(static_cast<char*>(h->st_move) + B * 4) : nullptr;
  dev.black_rows = (io->black_rows != nullptr && io->policy_vocab == CRL_VOCAB_RL1929) ? static_cast<const uint8_t*>(h->st_black) : nullptr;
  dev.planes = h->st_planes;
  dev.legal_mask = mb > 0 ? h->st_mask : nullptr;
  dev.policy_out = ob > 0 ? h->st_policy : nullptr;
  dev.wdl_out = io->wdl_out != nullptr ? static_cast<float*>(h->st_wdl) : nullptr;
  dev.q_out = io->q_out != nullptr ? static_cast<float*>(h->st_q) : nullptr;
  dev.workspace = h->st_ws;
  dev.workspace_bytes = h->st_ws_b;
  if ((rc = run_batch(h, &dev, false)) != CRL_OK) return rc;
  if (ob > 0 && !own_rows) CRL_CUDA(h, cudaMemcpyAsync(io->policy_out, h->st_policy, ob, cudaMemcpyDeviceToHost, s));
  if (io->move_out != nullptr) CRL_CUDA(h, cudaMemcpyAsync(io->move_out, h->st_move, B * 4, cudaMemcpyDeviceToHost, s));
  if (io->wdl_out != nullptr) CRL_CUDA(h, cudaMemcpyAsync(io->wdl_out, h->st_wdl, B * 12, cudaMemcpyDeviceToHost, s));
  if (io->q_out != nullptr) CRL_CUDA(h, cudaMemcpyAsync(io->q_out, h->st_q, B * 4, cudaMemcpyDeviceToHost, s));
  CRL_CUDA(h, cudaStreamSynchronize(s));
  return CRL_OK;
}

// Scratch for crl_forward_static: lives in the library's device image, so no allocation call is ever
// needed for it. Every GPU that loads the library carries these bytes until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[CRL_STATIC_SCRATCH_BYTES];
// Device address of g_static_scratch per device (the name above is only a host-side stand-in for the
// symbol; kernels must be given the address cudaGetSymbolAddress reports for the current device).
static void* g_static_scratch_addr[64] = {};

int crl_forward_static(crl_handle* h, const crl_io* io) {
  int rc = check_io(h, io);
  if (rc != CRL_OK) return rc;
  if (h->device < 0 || h->device >= 64) return fail(h, CRL_ERR_UNSUPPORTED, "device index beyond the static scratch table");
  if (io->move_out != nullptr && io->policy_out == nullptr) return fail(h, CRL_ERR_INVALID, "move_out needs policy_out (the rows it reads)");
  const size_t need = crl_workspace_bytes(h, io->batch);
  if (need > static_cast<size_t>(CRL_STATIC_SCRATCH_BYTES))
    return fail(h, CRL_ERR_WORKSPACE, "batch " + std::to_string(io->batch) + " needs " + std::to_string(need) +
                                          " bytes of scratch; the static scratch of crl_forward_static holds " +
                                          std::to_string(static_cast<size_t>(CRL_STATIC_SCRATCH_BYTES)));
  CRL_ON_DEVICE(h);
  if (g_static_scratch_addr[h->device] == nullptr) {
    // one-time set-up per device, with that device current
    void* ptr = nullptr;
    CRL_CUDA(h, cudaGetSymbolAddress(&ptr, g_static_scratch));
    g_static_scratch_addr[h->device] = ptr;
  }
  crl_io with_scratch = *io;
  with_scratch.workspace = g_static_scratch_addr[h->device];
  with_scratch.workspace_bytes = static_cast<size_t>(CRL_STATIC_SCRATCH_BYTES);
  h->launches = 0;
  return run_batch(h, &with_scratch, false);
}

int crl_last_status(crl_handle* h, int* device_status_word) {
  if (h == nullptr || device_status_word == nullptr) return CRL_ERR_INVALID;
  CRL_ON_DEVICE(h);
  CRL_CUDA(h, cudaDeviceSynchronize());
  int st = 0;
  CRL_CUDA(h, cudaMemcpy(&st, h->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
  CRL_CUDA(h, cudaMemset(h->status_dev, 0, sizeof(int)));
  *device_status_word = st;
  return st == 0 ? CRL_OK : CRL_ERR_DEVICE_TIMEOUT;
}

int64_t crl_last_launch_count(const crl_handle* h) { return h != nullptr ? h->launches : 0; }

int crl_profile(crl_handle* h, int enable) {
  if (h == nullptr) return CRL_ERR_INVALID;
  h->profiling = enable != 0;
  h->prof_used = 0;
  return CRL_OK;
}

int crl_profile_entry(crl_handle* h, int64_t index, int* category, double* ms, double* flops, double* bytes, int* mnk_kind) {
  if (h == nullptr || category == nullptr || ms == nullptr || flops == nullptr || bytes == nullptr || mnk_kind == nullptr)
    return CRL_ERR_INVALID;
  if (index < 0 || static_cast<size_t>(index) >= h->prof_used) return CRL_ERR_INVALID;
  CRL_ON_DEVICE(h);
  const auto& r = h->prof[index];
  CRL_CUDA(h, cudaEventSynchronize(r.b));
  float t = 0.0f;
  CRL_CUDA(h, cudaEventElapsedTime(&t, r.a, r.b));
  *category = r.cat; *ms = t; *flops = r.flops; *bytes = r.bytes;
  mnk_kind[0] = r.m; mnk_kind[1] = r.n; mnk_kind[2] = r.k; mnk_kind[3] = r.kind;
  return CRL_OK;
}

int crl_profile_read(crl_handle* h, int category, double* ms, double* flops, double* bytes, int64_t* launches) {
  if (h == nullptr || ms == nullptr || flops == nullptr || bytes == nullptr || launches == nullptr) return CRL_ERR_INVALID;
  CRL_ON_DEVICE(h);
  CRL_CUDA(h, cudaDeviceSynchronize());
  *ms = 0.0; *flops = 0.0; *bytes = 0.0; *launches = 0;
  for (size_t i = 0; i < h->prof_used; ++i) {
    const auto& r = h->prof[i];
    if (r.cat != category) continue;
    float t = 0.0f;
    CRL_CUDA(h, cudaEventElapsedTime(&t, r.a, r.b));
    *ms += t; *flops += r.flops; *bytes += r.bytes; ++*launches;
  }
  return CRL_OK;
}

int crl_linear_ex(const crl_linear_args* x) {
  if (x == nullptr) return CRL_ERR_INVALID;
  if (x->kind < 0 || x->kind > 2 || x->out_dtype < 0 || x->out_dtype > 2 || x->act < 0 || x->act > 3) return CRL_ERR_INVALID;
  if (x->m <= 0 || x->n <= 0 || x->k <= 0 || x->m > INT32_MAX || x->n > INT32_MAX || x->k > INT32_MAX || x->res_mod < 0)
    return CRL_ERR_INVALID;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return CRL_ERR_CUDA;
  GemmArgs g;
  g.kind = x->kind; g.A = x->a; g.lda = x->lda; g.W = x->w; g.ldw = x->ldw;
  g.p.M = static_cast<int>(x->m); g.p.N = static_cast<int>(x->n); g.p.K = static_cast<int>(x->k);
  g.p.C = x->c; g.p.ldc = x->ldc; g.p.out_dtype = x->out_dtype; g.p.bias = x->bias;
  g.p.residual = static_cast<const __half*>(x->residual); g.p.ldr = x->ldr; g.p.res_mod = x->res_mod;
  g.p.alpha = x->alpha; g.p.row_scale = x->row_scale; g.p.col_scale = x->col_scale; g.p.act = x->act;
  g.p.out_scale = x->out_dtype == kOutE4M3 ? x->out_scale : 1.0f;
  g.p.status = x->device_status;
  if (x->ln_y != nullptr) {
    if (x->ln_weight == nullptr || x->ln_bias == nullptr) return CRL_ERR_INVALID;
    g.p.ln_y = static_cast<const __half*>(x->ln_y); g.p.ln_ldy = x->k;
    g.p.ln_w16 = static_cast<const __half*>(x->ln_weight); g.p.ln_b16 = static_cast<const __half*>(x->ln_bias);
    g.p.ln_x = static_cast<__half*>(x->ln_x); g.p.ln_x8 = static_cast<uint8_t*>(x->ln_x8); g.p.ln_out8_scale = x->ln_out8_scale;
    if (x->a != (x->kind == CRL_DTYPE_F16 ? x->ln_x : x->ln_x8) || x->lda != x->k) return CRL_ERR_INVALID;
  }
  if (x->lno_weight != nullptr || x->lno_bias != nullptr || x->lno_scratch != nullptr || x->lno_x8 != nullptr) {
    if (x->lno_weight == nullptr || x->lno_bias == nullptr || x->lno_scratch == nullptr || x->residual == nullptr) return CRL_ERR_INVALID;
    g.p.lno_w16 = static_cast<const __half*>(x->lno_weight); g.p.lno_b16 = static_cast<const __half*>(x->lno_bias);
    g.p.lno_stats = static_cast<unsigned long long*>(x->lno_scratch); g.p.lno_out8_scale = x->lno_out8_scale;
    g.p.lno_x8 = static_cast<uint8_t*>(x->lno_x8); g.p.lno_qscale = x->lno_qscale;
  }
  return gemm_launch(g, sms, static_cast<cudaStream_t>(x->stream));
}

int crl_linear(int kind, const void* a, int64_t lda, const void* w, int64_t ldw, void* c, int64_t ldc, int out_dtype,
               int64_t m, int64_t n, int64_t k, const float* bias, const void* residual, int64_t ldr, float alpha,
               int act, int* device_status, void* stream) {
  crl_linear_args x{};
  x.kind = kind; x.out_dtype = out_dtype; x.a = a; x.lda = lda; x.w = w; x.ldw = ldw; x.c = c; x.ldc = ldc;
  x.m = m; x.n = n; x.k = k; x.bias = bias; x.residual = residual; x.ldr = ldr; x.res_mod = 0; x.alpha = alpha;
  x.act = act; x.out_scale = 1.0f; x.row_scale = nullptr; x.col_scale = nullptr; x.device_status = device_status;
  x.stream = stream;
  return crl_linear_ex(&x);
}

int crl_vocab_move(int index, char* buf) {
  const Vocab& v = Vocab::get();
  if (buf == nullptr || index < 0 || index >= static_cast<int>(v.moves.size())) return CRL_ERR_INVALID;
  std::snprintf(buf, 16, "%s", v.moves[index].c_str());
  return CRL_OK;
}

int crl_vocab_mirror_index(int leela_index) {
  const Vocab& v = Vocab::get();
  if (leela_index < 0 || leela_index >= static_cast<int>(v.mirror.size())) return CRL_ERR_INVALID;
  return v.mirror[leela_index];
}

}  // extern "C"
