// Attention-policy head: per board S = Q K^T / sqrt(d) over the full model width (64 x 64 x d), then
// either (a) the flat [4096] score vector for the reference's dense 4096 -> 1929 layer
// (new_paradigm/value.py:176-187, flat index = query*64 + key), or (b) the specification's gather to
// the 1858 Leela moves (+ per-destination promotion logits), with the legal-move mask and an
// optional softmax fused in. One CTA (4 warps) per board; Q/K chunks of 64 columns are double-buffered
// through cp.async; the score tile lives in shared memory only.
//
// Mask conventions (integer-exact index sets):
//   bits     : u8 bitset per board, bit m set = move m legal -> logits + (1-bit)*(-999)
//              (model_bis.py:383, value.py:231)
//   additive : f32 vector added to the logits, -1000 / 0 (Leela/server.py:56)
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "attention.cuh"

namespace crl {

enum MaskMode : int { kMaskNone = 0, kMaskBits = 1, kMaskAdditive = 2 };

struct PolicyParams {
  const __half* qk;      // [B*64, ld]: Q at column 0, K at column d, promotion logits at column 2d..2d+2
  long long ld;
  int d;
  float scale;
  // mode (a)
  __half* flat;          // [B, 4096] or null
  // mode (b)
  const short* gather_idx;     // [n_moves] from*64+to
  const signed char* gather_promo;  // [n_moves] 0 none, 1..3 piece
  int n_moves;
  const void* mask; int mask_mode; long long mask_ld;   // bits: bytes per row; additive: floats per row
  int softmax;
  float* out_f32; __half* out_f16; long long out_ld;
  // optional scatter of the 1858 Leela entries into zero-filled rows of 1929 (Leela/compare_policy.py:
  // 493-523): rows flagged in black_rows go through the rank-mirror table, the others keep their index
  const short* mirror;          // [1858] or null
  const uint8_t* black_rows;    // [B] (already offset to this chunk) or null = every row is White
  int out_width;                // 1929 when scattering
};

__device__ __forceinline__ float block_reduce_128(float v, float* red, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, other) : v + other;
  }
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
  for (int w = 1; w < 4; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
  return r;
}

__global__ void __launch_bounds__(128) policy_scores_kernel(const PolicyParams p) {
  // two stages x (Q chunk 64x64 f16 + K chunk 64x64 f16) = 32 KB; the 64 x 65 f32 score tile
  // (16.25 KB) later overlays them
  __shared__ __align__(128) uint8_t stage[2][2][64 * 128];
  __shared__ float red[4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long board = blockIdx.x;
  const __half* src = p.qk + board * 64 * p.ld;
  const int nchunks = p.d / 64;

  auto issue = [&](int chunk, int st) {
    for (int i = threadIdx.x; i < 64 * 8; i += 128) {
      const int r = i >> 3, c = i & 7;
      const __half* g = src + (long long)r * p.ld + chunk * 64 + c * 8;
      cp_async16(smem_u32(&stage[st][0][0]) + tile_off<64>(r, c), g);
      cp_async16(smem_u32(&stage[st][1][0]) + tile_off<64>(r, c), g + p.d);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float s[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;

  issue(0, 0);
  for (int ch = 0; ch < nchunks; ++ch) {
    const int st = ch & 1;
    if (ch + 1 < nchunks) {
      issue(ch + 1, st ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const uint32_t sQ = smem_u32(&stage[st][0][0]), sK = smem_u32(&stage[st][1][0]);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(sQ + tile_off<64>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)), a0, a1, a2, a3);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(sK + tile_off<64>(np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8, ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
        mma16816(s[2 * np], a0, a1, a2, a3, b0, b1);
        mma16816(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();   // everyone is done with stage st before it is refilled
  }

  // the score tile reuses the staging buffers (every warp passed the loop's last barrier)
  float* sc = reinterpret_cast<float*>(&stage[0][0][0]);
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int n = 0; n < 8; ++n) {
    const int r0 = warp * 16 + g, c0 = n * 8 + 2 * t;
    sc[r0 * 65 + c0] = s[n][0] * p.scale;
    sc[r0 * 65 + c0 + 1] = s[n][1] * p.scale;
    sc[(r0 + 8) * 65 + c0] = s[n][2] * p.scale;
    sc[(r0 + 8) * 65 + c0 + 1] = s[n][3] * p.scale;
  }
  __syncthreads();

  if (p.flat != nullptr) {
    __half* dst = p.flat + board * 4096;
    for (int i = threadIdx.x; i < 2048; i += 128) {
      const int q = (2 * i) >> 6, k = (2 * i) & 63;
      *reinterpret_cast<__half2*>(dst + 2 * i) = __floats2half2_rn(sc[q * 65 + k], sc[q * 65 + k + 1]);
    }
    return;
  }

  // gather + promotion + mask (+ softmax)
  constexpr int PER = 16;                      // ceil(1929 / 128)
  float vals[PER];
  float vmax = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int m = threadIdx.x + j * 128;
    float v = -INFINITY;
    if (m < p.n_moves) {
      const int idx = p.gather_idx[m];
      v = sc[(idx >> 6) * 65 + (idx & 63)];
      const int pr = p.gather_promo[m];
      if (pr > 0) v += __half2float(src[(long long)(idx & 63) * p.ld + 2 * p.d + (pr - 1)]);
      if (p.mask_mode == kMaskBits) {
        const uint8_t byte = reinterpret_cast<const uint8_t*>(p.mask)[board * p.mask_ld + (m >> 3)];
        if (((byte >> (m & 7)) & 1) == 0) v += -999.0f;
      } else if (p.mask_mode == kMaskAdditive) {
        v += reinterpret_cast<const float*>(p.mask)[board * p.mask_ld + m];
      }
      vmax = fmaxf(vmax, v);
    }
    vals[j] = v;
  }
  if (p.softmax) {
    vmax = block_reduce_128(vmax, red, true);
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int m = threadIdx.x + j * 128;
      if (m < p.n_moves) { vals[j] = __expf(vals[j] - vmax); sum += vals[j]; }
    }
    sum = block_reduce_128(sum, red, false);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int j = 0; j < PER; ++j) vals[j] *= inv;
  }
  const bool scatter = p.mirror != nullptr;
  const bool black = scatter && p.black_rows != nullptr && p.black_rows[board] != 0;
  if (scatter) {
    for (int o = threadIdx.x; o < p.out_width; o += 128) {
      if (p.out_f32 != nullptr) p.out_f32[board * p.out_ld + o] = 0.0f;
      else p.out_f16[board * p.out_ld + o] = __float2half_rn(0.0f);
    }
    __syncthreads();   // zero fill lands before the scattered values of other threads
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int m = threadIdx.x + j * 128;
    if (m < p.n_moves) {
      const int o = black ? p.mirror[m] : m;
      if (p.out_f32 != nullptr) p.out_f32[board * p.out_ld + o] = vals[j];
      else p.out_f16[board * p.out_ld + o] = __float2half_rn(vals[j]);
    }
  }
}

// Mask (+ softmax) over rows of f32 logits that a GEMM produced (dense 4096 -> 1929 policy form).
struct MaskRowsParams {
  const float* logits; long long ld; int n;
  const void* mask; int mask_mode; long long mask_ld;
  int softmax;
  float* out_f32; __half* out_f16; long long out_ld;
};

__global__ void __launch_bounds__(128) mask_rows_kernel(const MaskRowsParams p) {
  __shared__ float red[4];
  const long long row = blockIdx.x;
  constexpr int PER = 16;
  float vals[PER];
  float vmax = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int m = threadIdx.x + j * 128;
    float v = -INFINITY;
    if (m < p.n) {
      v = p.logits[row * p.ld + m];
      if (p.mask_mode == kMaskBits) {
        const uint8_t byte = reinterpret_cast<const uint8_t*>(p.mask)[row * p.mask_ld + (m >> 3)];
        if (((byte >> (m & 7)) & 1) == 0) v += -999.0f;
      } else if (p.mask_mode == kMaskAdditive) {
        v += reinterpret_cast<const float*>(p.mask)[row * p.mask_ld + m];
      }
      vmax = fmaxf(vmax, v);
    }
    vals[j] = v;
  }
  if (p.softmax) {
    vmax = block_reduce_128(vmax, red, true);
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int m = threadIdx.x + j * 128;
      if (m < p.n) { vals[j] = __expf(vals[j] - vmax); sum += vals[j]; }
    }
    sum = block_reduce_128(sum, red, false);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int j = 0; j < PER; ++j) vals[j] *= inv;
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int m = threadIdx.x + j * 128;
    if (m < p.n) {
      if (p.out_f32 != nullptr) p.out_f32[row * p.out_ld + m] = vals[j];
      else p.out_f16[row * p.out_ld + m] = __float2half_rn(vals[j]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Move choice per policy row (model_bis.py:385-394), one warp per row: arg-max (lowest index on ties) or the
// inverse-CDF draw for a caller-supplied uniform number: weights e_i = exp((x_i - max) / T) for logit rows,
// (p_i / max p)^(1/T) for probability rows; the first index whose running sum exceeds u * total wins. Sums
// run in double so that the order of additions does not move a boundary.
// ---------------------------------------------------------------------------------------------
struct SampleParams {
  const float* r32; const __half* r16; long long ld;
  int n; long long rows;
  int is_prob; float inv_t;
  const float* u;          // null: arg-max
  int32_t* out;
};

__global__ void __launch_bounds__(256) sample_rows_kernel(const SampleParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + warp;
  if (row >= p.rows) return;
  auto val = [&](int i) -> float {
    return p.r32 != nullptr ? p.r32[row * p.ld + i] : __half2float(p.r16[row * p.ld + i]);
  };
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lane; i < p.n; i += 32) {
    const float x = val(i);
    if (x > best || bi == 0x7fffffff) { best = x; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
  }
  if (p.u == nullptr || p.inv_t == 0.0f) {
    if (lane == 0) p.out[row] = bi;
    return;
  }
  auto weight = [&](int i) -> float {
    const float x = val(i);
    if (p.is_prob) return x > 0.0f ? powf(x / best, p.inv_t) : 0.0f;
    return expf((x - best) * p.inv_t);
  };
  double part = 0.0;
  for (int i = lane; i < p.n; i += 32) part += static_cast<double>(weight(i));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  const double thr = static_cast<double>(p.u[row]) * part;
  double running = 0.0;
  int pick = -1;
  for (int base = 0; base < p.n && pick < 0; base += 32) {
    const int i = base + lane;
    double c = i < p.n ? static_cast<double>(weight(i)) : 0.0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double up = __shfl_up_sync(0xffffffffu, c, o);
      if (lane >= o) c += up;
    }
    c += running;
    const unsigned hit = __ballot_sync(0xffffffffu, i < p.n && c > thr);
    if (hit != 0u) pick = base + (__ffs(hit) - 1);
    running = __shfl_sync(0xffffffffu, c, 31);
  }
  if (lane == 0) p.out[row] = pick >= 0 ? pick : bi;   // u * total rounded up to the total itself: the mode
}

}  // namespace crl
