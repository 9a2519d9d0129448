// Fused per-board attention: for one board and one head, scores = Q K^T * scale (+ bias), row softmax
// and P V without the 64x64 score tile ever leaving the SM (registers; shared memory only for the
// relative-position term). One warp owns one (board, head): Q, K, V tiles (64 x head_dim f16) are
// staged with cp.async into swizzled shared memory, ldmatrix feeds mma.sync m16n8k16, the softmax is
// done on the accumulator fragments with quad shuffles.
//
// Bias modes
//   none / causal : softmax(Q K^T / sqrt(hd))                       (model_bis.py:71 is the causal one)
//   smolgen       : + bias[board, head, 64, 64] (f16, produced by the smolgen GEMM chain)
//   relpos        : ((Q+u) K^T + relshift((Q+v) P^T)) * scale       (new_paradigm/attn.py:507-533),
//                   P = pos_proj(sinusoid table) folded at weight-load time, relshift done as the
//                   index remap out[i][j] = padded_flat[(i+1)*64 + j]
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "ptx.cuh"

namespace crl {

enum AttnBias : int { kBiasNone = 0, kBiasCausal = 1, kBiasRelpos = 2, kBiasSmolgen = 3 };

struct AttnParams {
  const __half* qkv;     // [B*64, ld]: Q at column 0, K at d, V at 2d; head h at h*HD inside each
  long long ld;
  int d, H, B;
  const __half* bias;    // smolgen: [B*H, 4096]
  const __half* pos;     // relpos: [64, d]
  const __half* u;       // relpos: [d]
  const __half* v;       // relpos: [d]
  float scale;
  __half* out;           // [B*64, ldo] f16 (null when out8 is used)
  uint8_t* out8;         // e4m3 output scaled by out8_scale
  long long ldo;
  float out8_scale;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// f16-accumulating variant: c holds two packed f16 pairs (row g, row g+8)
__device__ __forceinline__ void mma16816_h(uint32_t (&c)[2], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f16.f16.f16.f16 {%0,%1}, {%2,%3,%4,%5}, {%6,%7}, {%0,%1};"
               : "+r"(c[0]), "+r"(c[1])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// packed-f16 arithmetic on raw 32-bit registers
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b), *reinterpret_cast<__half2*>(&c));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
  __half2 r = __hsub2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t hmax2_u32(uint32_t a, uint32_t b) {
  __half2 r = __hmax2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t hexp2_u32(uint32_t a) {     // 2^x on both halves, one special-function op
  uint32_t r;
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(r) : "r"(a));
  return r;
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t hadd2_u32(uint32_t a, uint32_t b) {
  __half2 r = __hadd2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

// Byte offset of 16-byte chunk c of row r in a [64][HD] f16 tile, XOR-swizzled so that the eight rows
// an ldmatrix phase touches fall into distinct banks.
template <int HD>
__device__ __forceinline__ uint32_t tile_off(int r, int c) {
  if constexpr (HD == 32) return r * 64 + ((c ^ ((r >> 1) & 3)) << 4);
  else return r * 128 + ((c ^ (r & 7)) << 4);
}

template <int HD, int HPC, int MODE>
struct AttnSmem {
  static constexpr int TILE = 64 * HD * 2;
  static constexpr int NT = (MODE == kBiasRelpos) ? 4 : 3;     // Q K V (+P)
  static constexpr int PS = (MODE == kBiasRelpos) ? 64 * 65 * 4 : 0;
  static constexpr int PER_HEAD = NT * TILE + PS;
  static constexpr int BYTES = HPC * PER_HEAD + 128;
};

template <int HD, int HPC, int MODE>
__global__ void __launch_bounds__(HPC * 32) attention_kernel(const AttnParams p) {
  using SM = AttnSmem<HD, HPC, MODE>;
  constexpr int CH = HD / 8;        // 16-byte chunks per row
  constexpr int KS = HD / 16;       // k-steps of Q K^T
  extern __shared__ uint8_t smem_attn_raw[];
  const uint32_t raw = smem_u32(smem_attn_raw);
  const uint32_t base = (raw + 127u) & ~127u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = p.H / HPC;
  const int board = blockIdx.x / groups;
  const int h = (blockIdx.x % groups) * HPC + warp;
  const uint32_t sQ = base + warp * SM::PER_HEAD;
  const uint32_t sK = sQ + SM::TILE, sV = sK + SM::TILE;
  const uint32_t sP = sV + SM::TILE;                                   // relpos only
  float* ps = reinterpret_cast<float*>(smem_attn_raw + (base - raw) + warp * SM::PER_HEAD + 4 * SM::TILE);

  // ---- stage this head's tiles ------------------------------------------------------------------
  {
    const __half* src = p.qkv + (long long)board * 64 * p.ld + h * HD;
    for (int i = lane; i < 64 * CH; i += 32) {
      const int r = i / CH, c = i % CH;
      const __half* g = src + (long long)r * p.ld + c * 8;
      cp_async16(sQ + tile_off<HD>(r, c), g);
      cp_async16(sK + tile_off<HD>(r, c), g + p.d);
      cp_async16(sV + tile_off<HD>(r, c), g + 2 * p.d);
      if constexpr (MODE == kBiasRelpos)
        cp_async16(sP + tile_off<HD>(r, c), p.pos + (long long)r * p.d + h * HD + c * 8);
    }
    cp_async_wait_all();
    __syncwarp();
  }

  const int g = lane >> 2, t = lane & 3;

  // ---- relpos: positional scores for the whole head into the padded-flat buffer --------------------
  if constexpr (MODE == kBiasRelpos) {
    for (int r = lane; r < 64; r += 32) ps[r * 65] = 0.0f;
    for (int slab = 0; slab < 4; ++slab) {
      float s[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t a0, a1, a2, a3;
        ldsm_x4(sQ + tile_off<HD>(slab * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)), a0, a1, a2, a3);
        const uint32_t v0 = *reinterpret_cast<const uint32_t*>(p.v + h * HD + ks * 16 + 2 * t);
        const uint32_t v1 = *reinterpret_cast<const uint32_t*>(p.v + h * HD + ks * 16 + 8 + 2 * t);
        a0 = hadd2_u32(a0, v0); a1 = hadd2_u32(a1, v0); a2 = hadd2_u32(a2, v1); a3 = hadd2_u32(a3, v1);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4(sP + tile_off<HD>(np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8, ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
          mma16816(s[2 * np], a0, a1, a2, a3, b0, b1);
          mma16816(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
        }
      }
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const int r0 = slab * 16 + g, c0 = n * 8 + 2 * t;
        ps[r0 * 65 + 1 + c0] = s[n][0];
        ps[r0 * 65 + 2 + c0] = s[n][1];
        ps[(r0 + 8) * 65 + 1 + c0] = s[n][2];
        ps[(r0 + 8) * 65 + 2 + c0] = s[n][3];
      }
    }
    __syncwarp();
  }

  // ---- main loop over the four 16-row slabs of queries ---------------------------------------------
  for (int slab = 0; slab < 4; ++slab) {
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(sQ + tile_off<HD>(slab * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)), a0, a1, a2, a3);
      if constexpr (MODE == kBiasRelpos) {
        const uint32_t u0 = *reinterpret_cast<const uint32_t*>(p.u + h * HD + ks * 16 + 2 * t);
        const uint32_t u1 = *reinterpret_cast<const uint32_t*>(p.u + h * HD + ks * 16 + 8 + 2 * t);
        a0 = hadd2_u32(a0, u0); a1 = hadd2_u32(a1, u0); a2 = hadd2_u32(a2, u1); a3 = hadd2_u32(a3, u1);
      }
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(sK + tile_off<HD>(np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8, ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
        mma16816(s[2 * np], a0, a1, a2, a3, b0, b1);
        mma16816(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    const int r0 = slab * 16 + g;
    // scale, bias
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const int c0 = n * 8 + 2 * t;
      if constexpr (MODE == kBiasRelpos) {
        s[n][0] = (s[n][0] + ps[(r0 + 1) * 64 + c0]) * p.scale;
        s[n][1] = (s[n][1] + ps[(r0 + 1) * 64 + c0 + 1]) * p.scale;
        s[n][2] = (s[n][2] + ps[(r0 + 9) * 64 + c0]) * p.scale;
        s[n][3] = (s[n][3] + ps[(r0 + 9) * 64 + c0 + 1]) * p.scale;
      } else if constexpr (MODE == kBiasSmolgen) {
        const __half* bp = p.bias + ((long long)board * p.H + h) * 4096;
        const float2 b0 = __half22float2(*reinterpret_cast<const __half2*>(bp + r0 * 64 + c0));
        const float2 b1 = __half22float2(*reinterpret_cast<const __half2*>(bp + (r0 + 8) * 64 + c0));
        s[n][0] = s[n][0] * p.scale + b0.x;
        s[n][1] = s[n][1] * p.scale + b0.y;
        s[n][2] = s[n][2] * p.scale + b1.x;
        s[n][3] = s[n][3] * p.scale + b1.y;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) s[n][j] *= p.scale;
        if constexpr (MODE == kBiasCausal) {
          if (c0 > r0) s[n][0] = -INFINITY;
          if (c0 + 1 > r0) s[n][1] = -INFINITY;
          if (c0 > r0 + 8) s[n][2] = -INFINITY;
          if (c0 + 1 > r0 + 8) s[n][3] = -INFINITY;
        }
      }
    }
    // row softmax (rows r0 and r0+8; a row lives in the 4 lanes of a quad)
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      m0 = fmaxf(m0, fmaxf(s[n][0], s[n][1]));
      m1 = fmaxf(m1, fmaxf(s[n][2], s[n][3]));
    }
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1));
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
    float l0 = 0.0f, l1 = 0.0f;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      s[n][0] = __expf(s[n][0] - m0); s[n][1] = __expf(s[n][1] - m0);
      s[n][2] = __expf(s[n][2] - m1); s[n][3] = __expf(s[n][3] - m1);
      l0 += s[n][0] + s[n][1];
      l1 += s[n][2] + s[n][3];
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;

    // O = P V
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t a0 = pack_h2(s[2 * kk][0], s[2 * kk][1]);
      const uint32_t a1 = pack_h2(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack_h2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const uint32_t a3 = pack_h2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(sV + tile_off<HD>(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dp * 2 + ((lane >> 4) & 1)), b0, b1, b2, b3);
        mma16816(o[2 * dp], a0, a1, a2, a3, b0, b1);
        mma16816(o[2 * dp + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    const long long row0 = (long long)board * 64 + r0;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      const int col = h * HD + n * 8 + 2 * t;
      if (p.out8 != nullptr) {
        const float sc = p.out8_scale;
        const uint16_t w0 = __nv_cvt_float2_to_fp8x2(make_float2(o[n][0] * inv0 * sc, o[n][1] * inv0 * sc), __NV_SATFINITE, __NV_E4M3);
        const uint16_t w1 = __nv_cvt_float2_to_fp8x2(make_float2(o[n][2] * inv1 * sc, o[n][3] * inv1 * sc), __NV_SATFINITE, __NV_E4M3);
        *reinterpret_cast<uint16_t*>(p.out8 + row0 * p.ldo + col) = w0;
        *reinterpret_cast<uint16_t*>(p.out8 + (row0 + 8) * p.ldo + col) = w1;
      } else {
        *reinterpret_cast<__half2*>(p.out + row0 * p.ldo + col) = __floats2half2_rn(o[n][0] * inv0, o[n][1] * inv0);
        *reinterpret_cast<__half2*>(p.out + (row0 + 8) * p.ldo + col) = __floats2half2_rn(o[n][2] * inv1, o[n][3] * inv1);
      }
    }
  }
}

template <int HD, int HPC, int MODE>
inline cudaError_t attention_launch_t(const AttnParams& p, cudaStream_t stream) {
  using SM = AttnSmem<HD, HPC, MODE>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attention_kernel<HD, HPC, MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SM::BYTES);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  const long long blocks = (long long)p.B * (p.H / HPC);
  attention_kernel<HD, HPC, MODE><<<static_cast<unsigned>(blocks), HPC * 32, SM::BYTES, stream>>>(p);
  return cudaGetLastError();
}

template <int HD, int MODE>
inline cudaError_t attention_launch_m(const AttnParams& p, cudaStream_t stream) {
  constexpr int kMax = (MODE == kBiasRelpos) ? 4 : 8;
  if (kMax >= 8 && p.H % 8 == 0) return attention_launch_t<HD, kMax >= 8 ? 8 : 4, MODE>(p, stream);
  if (p.H % 4 == 0) return attention_launch_t<HD, 4, MODE>(p, stream);
  if (p.H % 2 == 0) return attention_launch_t<HD, 2, MODE>(p, stream);
  return attention_launch_t<HD, 1, MODE>(p, stream);
}

// head_dim must be 32 or 64; returns cudaErrorInvalidValue otherwise.
inline cudaError_t attention_launch(const AttnParams& p, int head_dim, int mode, cudaStream_t stream) {
#define CRL_ATTN_CASE(HD_)                                                              \
  switch (mode) {                                                                       \
    case kBiasNone: return attention_launch_m<HD_, kBiasNone>(p, stream);               \
    case kBiasCausal: return attention_launch_m<HD_, kBiasCausal>(p, stream);           \
    case kBiasRelpos: return attention_launch_m<HD_, kBiasRelpos>(p, stream);           \
    case kBiasSmolgen: return attention_launch_m<HD_, kBiasSmolgen>(p, stream);         \
    default: return cudaErrorInvalidValue;                                              \
  }
  if (head_dim == 32) { CRL_ATTN_CASE(32) }
  if (head_dim == 64) { CRL_ATTN_CASE(64) }
#undef CRL_ATTN_CASE
  return cudaErrorInvalidValue;
}

}  // namespace crl
