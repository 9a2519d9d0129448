// Memory-bound row kernels around the GEMMs: input-plane conversion, LayerNorm (+ the embedding's
// gating, + an optional e4m3 copy for the next FP8 GEMM), the value-head tail, and absolute-maximum
// reduction used for FP8 calibration. All are vectorised to 16-byte accesses along the row.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "ptx.cuh"

namespace crl {

enum PlaneLayout : int {
  kLayoutNHWC_F32 = 0,   // [B, 8, 8, P] f32 - the nn.Module signature (value_q.py:156-159)
  kLayoutNHWC_F16 = 1,   // [B, 8, 8, P] f16
  kLayoutNCHW_F16 = 2,   // [B, P, 8, 8] f16 - what the Leela server feeds (Leela/server.py:54)
  kLayoutNCHW_F32 = 3,   // [B, P, 8, 8] f32
};

// token-major rows [B*64, ldo] f16 with zero padding in columns [P, ldo)
template <typename TIn>
__global__ void tokens_from_nhwc_kernel(const TIn* __restrict__ in, __half* __restrict__ out, long long rows,
                                        int P, int ldo) {
  const int chunks = ldo / 8;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * chunks) return;
  const long long r = i / chunks;
  const int c0 = static_cast<int>(i % chunks) * 8;
  __align__(16) __half h[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = c0 + j;
    float v = 0.0f;
    if (c < P) v = static_cast<float>(in[r * P + c]);
    h[j] = __float2half_rn(v);
  }
  *reinterpret_cast<uint4*>(out + r * ldo + c0) = *reinterpret_cast<const uint4*>(h);
}

// one block per board: [P][64] -> [64][ldo] through shared memory
template <typename TIn>
__global__ void tokens_from_nchw_kernel(const TIn* __restrict__ in, __half* __restrict__ out, int P, int ldo) {
  extern __shared__ __half tile[];   // [P][66]
  const long long b = blockIdx.x;
  const TIn* src = in + b * P * 64;
  for (int i = threadIdx.x; i < P * 64; i += blockDim.x)
    tile[(i >> 6) * 66 + (i & 63)] = __float2half_rn(static_cast<float>(src[i]));
  __syncthreads();
  __half* dst = out + b * 64 * ldo;
  for (int i = threadIdx.x; i < 64 * ldo; i += blockDim.x) {
    const int tok = i / ldo, c = i % ldo;
    dst[i] = c < P ? tile[c * 66 + tok] : __float2half_rn(0.0f);
  }
}

// One block per position: a 840-byte packed record (104 bit planes + 8 auxiliary bytes; byte r of a plane =
// rank r, bit 7-f = file f) -> [64][ldo] f16 token rows, columns [112, ldo) zero. The record is staged in
// shared memory; each thread then builds 16-byte pieces (8 planes of one token) from it.
__global__ void __launch_bounds__(256) tokens_from_packed104_kernel(const uint8_t* __restrict__ in,
                                                                    __half* __restrict__ out, int ldo) {
  __shared__ __align__(16) uint8_t rec[848];
  const long long b = blockIdx.x;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(in + b * 840);   // 840 = 4 * 210: word-aligned
  for (int i = threadIdx.x; i < 210; i += blockDim.x) reinterpret_cast<uint32_t*>(rec)[i] = src[i];
  __syncthreads();
  const int chunks = ldo / 8;
  const __half one = __float2half_rn(1.0f), zero = __float2half_rn(0.0f);
  __half* dst = out + b * 64 * ldo;
  for (int i = threadIdx.x; i < 64 * chunks; i += blockDim.x) {
    const int tok = i / chunks, c0 = (i % chunks) * 8;
    const int byte = tok >> 3, bit = 7 - (tok & 7);
    __align__(16) __half h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int p = c0 + j;
      __half v = zero;
      if (p < 104) v = ((rec[p * 8 + byte] >> bit) & 1) ? one : zero;
      else if (p < 109) v = rec[832 + (p - 104)] ? one : zero;
      else if (p == 109) v = __float2half_rn(fminf(static_cast<float>(rec[837]) / 100.0f, 1.0f));
      else if (p == 111) v = one;
      h[j] = v;
    }
    *reinterpret_cast<uint4*>(dst + tok * ldo + c0) = *reinterpret_cast<const uint4*>(h);
  }
}

// ---------------------------------------------------------------------------------------------
// LayerNorm over rows of up to 1024 f16 elements (eps 1e-5, affine), one warp per row.
//   y = LN(x) * w + b ; optional gating y = y * ea[token] + gb[token] (token = row % 64; ea = exp(a),
//   utils/fen_encoder.py:41-49); writes f16 and/or e4m3 (y * out8_scale).
// ---------------------------------------------------------------------------------------------
struct LnParams {
  const __half* x; long long ldx;
  long long rows; int d;
  const float* w; const float* b;
  const float* gate_ea; const float* gate_b;   // [64, d] or null
  __half* y; long long ldy;                    // nullable
  uint8_t* y8; long long ldy8; float out8_scale;  // nullable
  int8_t* yq; float* yq_scale;                 // nullable: per-row symmetric int8 (row scale = max|y| / 127)
};

__global__ void __launch_bounds__(256) ln_rows_kernel(const LnParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + warp;
  if (row >= p.rows) return;
  constexpr int NV = 4;                 // up to 4 x (32 lanes x 8 elements) = 1024 columns
  float v[NV][8];
  const __half* xr = p.x + row * p.ldx;
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < p.d) {
      const uint4 u = *reinterpret_cast<const uint4*>(xr + c);
      const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        v[i][2 * j] = f.x; v[i][2 * j + 1] = f.y;
        sum += f.x + f.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float mean = sum / p.d;
  float var = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < p.d) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float dlt = v[i][j] - mean; var += dlt * dlt; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
  const float rstd = rsqrtf(var / p.d + 1e-5f);
  const int tok = static_cast<int>(row & 63);
  float qinv = 0.0f;
  if (p.yq != nullptr) {
    // dynamic per-token int8: one extra pass over the registers for the row maximum of |y|
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < p.d) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float yy = (v[i][j] - mean) * rstd * __ldg(p.w + c + j) + __ldg(p.b + c + j);
          if (p.gate_ea != nullptr) yy = yy * __ldg(p.gate_ea + (long long)tok * p.d + c + j) + __ldg(p.gate_b + (long long)tok * p.d + c + j);
          amax = fmaxf(amax, fabsf(yy));
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = amax > 0.0f ? amax / 127.0f : 1.0f;
    qinv = 1.0f / sc;
    if (lane == 0) p.yq_scale[row] = sc;
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < p.d) {
      float y[8];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const float4 w4 = __ldg(reinterpret_cast<const float4*>(p.w + c) + q);
        const float4 b4 = __ldg(reinterpret_cast<const float4*>(p.b + c) + q);
        y[q * 4 + 0] = (v[i][q * 4 + 0] - mean) * rstd * w4.x + b4.x;
        y[q * 4 + 1] = (v[i][q * 4 + 1] - mean) * rstd * w4.y + b4.y;
        y[q * 4 + 2] = (v[i][q * 4 + 2] - mean) * rstd * w4.z + b4.z;
        y[q * 4 + 3] = (v[i][q * 4 + 3] - mean) * rstd * w4.w + b4.w;
      }
      if (p.gate_ea != nullptr) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const float4 e4 = __ldg(reinterpret_cast<const float4*>(p.gate_ea + (long long)tok * p.d + c) + q);
          const float4 g4 = __ldg(reinterpret_cast<const float4*>(p.gate_b + (long long)tok * p.d + c) + q);
          y[q * 4 + 0] = y[q * 4 + 0] * e4.x + g4.x;
          y[q * 4 + 1] = y[q * 4 + 1] * e4.y + g4.y;
          y[q * 4 + 2] = y[q * 4 + 2] * e4.z + g4.z;
          y[q * 4 + 3] = y[q * 4 + 3] * e4.w + g4.w;
        }
      }
      if (p.y != nullptr) {
        uint4 pk;
        __half2 h0 = __floats2half2_rn(y[0], y[1]), h1 = __floats2half2_rn(y[2], y[3]);
        __half2 h2 = __floats2half2_rn(y[4], y[5]), h3 = __floats2half2_rn(y[6], y[7]);
        pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
        pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
        *reinterpret_cast<uint4*>(p.y + row * p.ldy + c) = pk;
      }
      if (p.y8 != nullptr) {
        const float s = p.out8_scale;
        uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(y[0] * s, y[1] * s), __NV_SATFINITE, __NV_E4M3) |
                      (uint32_t(__nv_cvt_float2_to_fp8x2(make_float2(y[2] * s, y[3] * s), __NV_SATFINITE, __NV_E4M3)) << 16);
        uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(y[4] * s, y[5] * s), __NV_SATFINITE, __NV_E4M3) |
                      (uint32_t(__nv_cvt_float2_to_fp8x2(make_float2(y[6] * s, y[7] * s), __NV_SATFINITE, __NV_E4M3)) << 16);
        *reinterpret_cast<uint2*>(p.y8 + row * p.ldy8 + c) = make_uint2(lo, hi);
      }
      if (p.yq != nullptr) {
        __align__(8) signed char q8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) q8[j] = static_cast<signed char>(max(-127, min(127, __float2int_rn(y[j] * qinv))));
        *reinterpret_cast<uint2*>(p.yq + row * p.d + c) = *reinterpret_cast<const uint2*>(q8);
      }
    }
  }
}

// The per-layer LayerNorms (no gating): persistent warps walk rows grid-stride with the affine
// parameters of their own columns held in registers as f16 pairs. The plain kernel above re-reads weight and
// bias through L1 for every row (four times the bytes of the row itself), which made L1 throughput, not HBM,
// its limit; here a row costs one 16-byte load and at most two stores per lane and vector.
// NV: 16-byte vectors per lane, rows of up to 256 NV columns (1 for the 256-wide smolgen generator rows, 4 for d_model)
template <bool Q8, int NV = 4>      // Q8: also emit per-token int8 rows (the W8A8 engine)
__global__ void __launch_bounds__(256, 2) ln_rows_persistent_kernel(const LnParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long stride = (long long)gridDim.x * 8;
  long long row = (long long)blockIdx.x * 8 + warp;
  if (row >= p.rows) return;
  uint32_t wh[NV][4], bh[NV][4];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * 32 + lane) * 8;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool ok = c < p.d;
      const __half2 w2 = __floats2half2_rn(ok ? p.w[c + 2 * j] : 0.0f, ok ? p.w[c + 2 * j + 1] : 0.0f);
      const __half2 b2 = __floats2half2_rn(ok ? p.b[c + 2 * j] : 0.0f, ok ? p.b[c + 2 * j + 1] : 0.0f);
      wh[i][j] = *reinterpret_cast<const uint32_t*>(&w2);
      bh[i][j] = *reinterpret_cast<const uint32_t*>(&b2);
    }
  }
  uint4 raw[NV], nxt[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * 32 + lane) * 8;
    raw[i] = c < p.d ? *reinterpret_cast<const uint4*>(p.x + row * p.ldx + c) : make_uint4(0u, 0u, 0u, 0u);
  }
  const __half2 s8 = __floats2half2_rn(p.out8_scale, p.out8_scale);
  uint32_t yrow[Q8 ? NV : 1][4];      // the normalised row as f16 pairs (int8 output only)
  for (; row < p.rows; row += stride) {
    const long long nrow = row + stride;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 8;
      nxt[i] = (nrow < p.rows && c < p.d) ? *reinterpret_cast<const uint4*>(p.x + nrow * p.ldx + c) : make_uint4(0u, 0u, 0u, 0u);
    }
    float sum = 0.0f, sq = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        sum += f.x + f.y;
        sq = fmaf(f.x, f.x, fmaf(f.y, f.y, sq));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sum += __shfl_xor_sync(0xffffffffu, sum, o);
      sq += __shfl_xor_sync(0xffffffffu, sq, o);
    }
    const float mean = sum / p.d;
    const float rstd = rsqrtf(fmaxf(sq / p.d - mean * mean, 0.0f) + 1e-5f);
    const float shift = -mean * rstd;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < p.d) {
        const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
        uint32_t o16[4];
        __half2 y2[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h[j]);
          const __half2 xn = __floats2half2_rn(fmaf(f.x, rstd, shift), fmaf(f.y, rstd, shift));
          y2[j] = __hfma2(xn, *reinterpret_cast<const __half2*>(&wh[i][j]), *reinterpret_cast<const __half2*>(&bh[i][j]));
          o16[j] = *reinterpret_cast<const uint32_t*>(&y2[j]);
        }
        if (p.y != nullptr) *reinterpret_cast<uint4*>(p.y + row * p.ldy + c) = make_uint4(o16[0], o16[1], o16[2], o16[3]);
        if (p.y8 != nullptr) {
          uint32_t w8[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const __half2 a = __hmul2(y2[2 * j], s8), b = __hmul2(y2[2 * j + 1], s8);
            w8[j] = uint32_t(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<const __half2_raw*>(&a), __NV_SATFINITE, __NV_E4M3)) |
                    (uint32_t(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<const __half2_raw*>(&b), __NV_SATFINITE, __NV_E4M3)) << 16);
          }
          *reinterpret_cast<uint2*>(p.y8 + row * p.ldy8 + c) = make_uint2(w8[0], w8[1]);
        }
        if constexpr (Q8) {
#pragma unroll
          for (int j = 0; j < 4; ++j) yrow[i][j] = o16[j];       // kept for the per-token int8 pass below
        }
      }
    }
    if constexpr (Q8) {
      // dynamic per-token int8 (W8A8): row maximum of |y| over the normalised values still in registers
      __half2 m2 = __float2half2_rn(0.0f);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        if ((i * 32 + lane) * 8 < p.d) {
#pragma unroll
          for (int j = 0; j < 4; ++j) m2 = __hmax2(m2, __habs2(*reinterpret_cast<const __half2*>(&yrow[i][j])));
        }
      }
      float amax = fmaxf(__low2float(m2), __high2float(m2));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float sc = amax > 0.0f ? amax / 127.0f : 1.0f;
      const float qinv = 1.0f / sc;
      if (lane == 0) p.yq_scale[row] = sc;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 8;
        if (c < p.d) {
          __align__(8) signed char q8[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&yrow[i][j]));
            q8[2 * j] = static_cast<signed char>(max(-127, min(127, __float2int_rn(f.x * qinv))));
            q8[2 * j + 1] = static_cast<signed char>(max(-127, min(127, __float2int_rn(f.y * qinv))));
          }
          *reinterpret_cast<uint2*>(p.yq + row * p.d + c) = *reinterpret_cast<const uint2*>(q8);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) raw[i] = nxt[i];
  }
}

// ---------------------------------------------------------------------------------------------
// Value-head tail (new_paradigm/value.py:427-435 last layer + the softmax of value.py:271):
// in [B,128] f16 -> Linear(128 -> n_out) -> mode 0 raw / 1 softmax / 2 tanh -> out [B, n_out] f32.
// One warp per board.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) value_tail_kernel(const __half* __restrict__ in, const float* __restrict__ w,
                                                         const float* __restrict__ b, float* __restrict__ out,
                                                         long long B, int n_out, int mode) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + warp;
  if (row >= B) return;
  const uint2 u = *reinterpret_cast<const uint2*>(in + row * 128 + lane * 4);
  const __half2* h = reinterpret_cast<const __half2*>(&u);
  const float2 x01 = __half22float2(h[0]), x23 = __half22float2(h[1]);
  float acc[3] = {0.0f, 0.0f, 0.0f};
  for (int o = 0; o < n_out && o < 3; ++o) {
    const float4 w4 = __ldg(reinterpret_cast<const float4*>(w + o * 128 + lane * 4));
    float s = x01.x * w4.x + x01.y * w4.y + x23.x * w4.z + x23.y * w4.w;
#pragma unroll
    for (int k = 16; k > 0; k >>= 1) s += __shfl_xor_sync(0xffffffffu, s, k);
    acc[o] = s + b[o];
  }
  if (lane == 0) {
    if (mode == 1) {
      float m = acc[0];
      for (int o = 1; o < n_out; ++o) m = fmaxf(m, acc[o]);
      float e[3], sum = 0.0f;
      for (int o = 0; o < n_out; ++o) { e[o] = __expf(acc[o] - m); sum += e[o]; }
      for (int o = 0; o < n_out; ++o) out[row * n_out + o] = e[o] / sum;
    } else if (mode == 2) {
      for (int o = 0; o < n_out; ++o) out[row * n_out + o] = tanhf(acc[o]);
    } else {
      for (int o = 0; o < n_out; ++o) out[row * n_out + o] = acc[o];
    }
  }
}

// max |x| over an f16 buffer (grid-stride), result combined with atomicMax on the float's bit pattern
__global__ void absmax_f16_kernel(const __half* __restrict__ x, long long rows, int cols, long long ld,
                                  unsigned int* __restrict__ out_bits) {
  float m = 0.0f;
  const long long total = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols;
    const int c = static_cast<int>(i % cols);
    m = fmaxf(m, fabsf(__half2float(x[r * ld + c])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(out_bits, __float_as_uint(m));
}

// Column sums of an f16 matrix in a fixed order (calibration only): block (x = column group of 256, y = row
// segment) adds its rows top to bottom into part[y][col]; colsum_finish_kernel adds the segments in order.
__global__ void __launch_bounds__(256) colsum_f16_kernel(const __half* __restrict__ x, long long rows, int cols, long long ld,
                                                         float* __restrict__ part, int segments) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= cols) return;
  const long long per = (rows + segments - 1) / segments;
  const long long r0 = per * blockIdx.y, r1 = r0 + per < rows ? r0 + per : rows;
  float acc = 0.0f;
  for (long long r = r0; r < r1; ++r) acc += __half2float(x[r * ld + c]);
  part[static_cast<long long>(blockIdx.y) * cols + c] = acc;
}
__global__ void colsum_finish_kernel(const float* __restrict__ part, int cols, int segments, float* __restrict__ acc) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float t = 0.0f;
  for (int s = 0; s < segments; ++s) t += part[static_cast<long long>(s) * cols + c];
  acc[c] += t;        // accumulates over the passes of one calibration call (one launch at a time per stream)
}

// FP8 bias correction (calibration only): out[n] = bias[n] + sum_k (W[n,k] - W8[n,k] / mult) * colsum[k] / rows, one
// warp per output row. W is the f16 copy of the weights, W8 their e4m3 copy (value * mult rounded).
__global__ void __launch_bounds__(256) bias_correct_kernel(const __half* __restrict__ W, const uint8_t* __restrict__ W8, float inv_mult,
                                                           const float* __restrict__ colsum, float inv_rows,
                                                           const float* __restrict__ bias, float* __restrict__ out, int n_out, int k_in) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  if (n >= n_out) return;
  float acc = 0.0f;
  for (int k = lane; k < k_in; k += 32) {
    const size_t i = static_cast<size_t>(n) * k_in + k;
    const __half_raw hr = __nv_cvt_fp8_to_halfraw(W8[i], __NV_E4M3);
    const float w8 = __half2float(*reinterpret_cast<const __half*>(&hr)) * inv_mult;
    acc = fmaf(__half2float(W[i]) - w8, colsum[k] * inv_rows, acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[n] = bias[n] + acc;
}

// f16 rows -> per-row symmetric int8 + scale (dynamic per-token activation quantisation); one warp per row, the row
// read once and held in registers (cols a multiple of 8, at most 4096).
template <int NV>       // NV x 256 columns at most
__global__ void __launch_bounds__(256) quant_rows_i8_kernel(const __half* __restrict__ x, long long rows, int cols,
                                                            int8_t* __restrict__ q, float* __restrict__ scale) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long stride = (long long)gridDim.x * 8;
  for (long long row = (long long)blockIdx.x * 8 + warp; row < rows; row += stride) {
    const __half* xr = x + row * cols;
    uint4 raw[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 8;
      raw[i] = c < cols ? *reinterpret_cast<const uint4*>(xr + c) : make_uint4(0u, 0u, 0u, 0u);
    }
    __half2 m2 = __float2half2_rn(0.0f);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) m2 = __hmax2(m2, __habs2(h[j]));
    }
    float amax = fmaxf(__low2float(m2), __high2float(m2));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = amax > 0.0f ? amax / 127.0f : 1.0f;
    const float inv = 1.0f / sc;
    if (lane == 0) scale[row] = sc;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < cols) {
        const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
        __align__(8) signed char q8[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h[j]);
          q8[2 * j] = static_cast<signed char>(max(-127, min(127, __float2int_rn(f.x * inv))));
          q8[2 * j + 1] = static_cast<signed char>(max(-127, min(127, __float2int_rn(f.y * inv))));
        }
        *reinterpret_cast<uint2*>(q + row * cols + c) = *reinterpret_cast<const uint2*>(q8);
      }
    }
  }
}

// f16 -> e4m3 with a per-tensor scale (used where the producer kernel cannot emit e4m3 itself)
__global__ void quant_e4m3_kernel(const __half* __restrict__ x, uint8_t* __restrict__ y, long long n8, float scale) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 u = reinterpret_cast<const uint4*>(x)[i];
  const __half2* h = reinterpret_cast<const __half2*>(&u);
  uint32_t w[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float2 a = __half22float2(h[2 * j]), b = __half22float2(h[2 * j + 1]);
    w[j] = __nv_cvt_float2_to_fp8x2(make_float2(a.x * scale, a.y * scale), __NV_SATFINITE, __NV_E4M3) |
           (uint32_t(__nv_cvt_float2_to_fp8x2(make_float2(b.x * scale, b.y * scale), __NV_SATFINITE, __NV_E4M3)) << 16);
  }
  reinterpret_cast<uint2*>(y)[i] = make_uint2(w[0], w[1]);
}

}  // namespace crl
