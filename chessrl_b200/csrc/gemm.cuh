// C[M,N] = epilogue(A[M,K] * W[N,K]^T): the one GEMM behind every nn.Linear of the board transformer
// (QKV, out-proj, FFN, embedding, smolgen, policy and value projections). Both operands are K-major,
// which is exactly nn.Linear's [out,in] weight layout, so no transposes are ever materialised.
//
// sm_100a design: persistent CTAs (one per SM) walk a static tile list. Inside a CTA
//   warp 0      : TMA producer  - cp.async.bulk.tensor loads of 128 x 128-byte A and BN x 128-byte W
//                 boxes (128-byte swizzle) into a ring of shared-memory stages
//   warp 1      : MMA issuer    - one thread issues tcgen05.mma (128 x BN x 32-byte-K) with fp32
//                 (int32 for int8) accumulators in tensor memory; two accumulator buffers so the
//                 next tile's main loop overlaps this tile's epilogue
//   warps 2..5  : epilogue      - tcgen05.ld of the accumulator (each warp owns the 32 TMEM lanes
//                 its rank allows), then scale / bias / activation / residual, convert, store
// All waits are bounded (see ptx.cuh); a wait that runs out records a status code and unwinds.
#pragma once
#include <cuda_runtime.h>
#include "ptx.cuh"

namespace crl {

enum OutType : int { kOutF16 = 0, kOutF32 = 1, kOutE4M3 = 2 };

struct GemmParams {
  int M, N, K;
  void* C;                 // [M, ldc] in out_dtype
  long long ldc;           // elements
  int out_dtype;
  const float* bias;       // [N] or null
  const __half* residual;  // [M, ldr] f16 or null; added after the activation
  long long ldr;
  int res_mod;             // > 0: residual row = row % res_mod (a table broadcast over boards)
  float alpha;             // multiplies the accumulator (per-tensor dequantisation scale)
  const float* row_scale;  // [M] or null (per-token int8 scales)
  const float* col_scale;  // [N] or null (per-output-channel int8 scales)
  int act;                 // Act
  float out_scale;         // multiplies the result before an e4m3 store
  int* status;             // device status word
};

template <int BN, int KIND>
struct GemmCfg {
  static constexpr int BM = 128;
  static constexpr int ESZ = (KIND == kKindF16) ? 2 : 1;
  static constexpr int BK = 128 / ESZ;   // elements per stage along K: one 128-byte swizzle row
  static constexpr int UK = 32 / ESZ;    // elements per tcgen05.mma along K
  static constexpr uint32_t A_BYTES = BM * 128;
  static constexpr uint32_t B_BYTES = BN * 128;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int ACC_COLS = 2 * BN;  // two accumulator buffers; 128, 256 or 512 columns
  static constexpr size_t SMEM_BYTES = size_t(STAGES) * STAGE_BYTES + 1024 /*alignment slack*/ + 256;
};

template <int OUT>
__device__ __forceinline__ void store_chunk32(void* C, long long off, const float (&v)[32]) {
  if constexpr (OUT == kOutF16) {
    __half* dst = reinterpret_cast<__half*>(C) + off;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 pk;
      __half2 h0 = __floats2half2_rn(v[q * 8 + 0], v[q * 8 + 1]);
      __half2 h1 = __floats2half2_rn(v[q * 8 + 2], v[q * 8 + 3]);
      __half2 h2 = __floats2half2_rn(v[q * 8 + 4], v[q * 8 + 5]);
      __half2 h3 = __floats2half2_rn(v[q * 8 + 6], v[q * 8 + 7]);
      pk.x = *reinterpret_cast<uint32_t*>(&h0);
      pk.y = *reinterpret_cast<uint32_t*>(&h1);
      pk.z = *reinterpret_cast<uint32_t*>(&h2);
      pk.w = *reinterpret_cast<uint32_t*>(&h3);
      reinterpret_cast<uint4*>(dst)[q] = pk;
    }
  } else if constexpr (OUT == kOutF32) {
    float* dst = reinterpret_cast<float*>(C) + off;
#pragma unroll
    for (int q = 0; q < 8; ++q)
      reinterpret_cast<float4*>(dst)[q] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
  } else {
    uint8_t* dst = reinterpret_cast<uint8_t*>(C) + off;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float* s = &v[q * 16 + j * 4];
        uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(s[0], s[1]), __NV_SATFINITE, __NV_E4M3);
        uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(s[2], s[3]), __NV_SATFINITE, __NV_E4M3);
        w[j] = lo | (hi << 16);
      }
      reinterpret_cast<uint4*>(dst)[q] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

__device__ __forceinline__ void store_one(void* C, int out_dtype, long long off, float v) {
  if (out_dtype == kOutF16) reinterpret_cast<__half*>(C)[off] = __float2half_rn(v);
  else if (out_dtype == kOutF32) reinterpret_cast<float*>(C)[off] = v;
  else reinterpret_cast<uint8_t*>(C)[off] =
      static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

template <int BN, int KIND>
__global__ void __launch_bounds__(192, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const GemmParams p) {
  using Cfg = GemmCfg<BN, KIND>;
  constexpr int BM = Cfg::BM, BK = Cfg::BK, STAGES = Cfg::STAGES;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;          // swizzled tiles need 1024-byte alignment
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t bar0 = base + STAGES * Cfg::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot =
      reinterpret_cast<uint32_t*>(smem + STAGES * Cfg::STAGE_BYTES + 8 * (2 * STAGES + 4));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);   // one arrival per epilogue warp
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::ACC_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m0 = (t / tiles_n) * BM;
        const int n0 = (t % tiles_n) * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u)) {
            atomicCAS(p.status, 0, kDevTimeoutProducer);
            ok = false;
            break;
          }
          const uint32_t a_dst = base + s * Cfg::STAGE_BYTES;
          const uint32_t b_dst = a_dst + Cfg::A_BYTES;
          mbar_expect_tx(full_bar(s), Cfg::STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, kb * BK, m0, full_bar(s));
          tma_load_2d(b_dst, &tmB, kb * BK, n0, full_bar(s));
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc =
          umma_idesc(BM, BN, KIND == kKindI8 ? 1 : 0, KIND == kKindI8 ? 2 : 1);
      int s = 0;
      uint32_t ph = 0;
      int local = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
        const int as = local & 1;
        const uint32_t aph = (local >> 1) & 1u;
        if (!mbar_wait(tempty_bar(as), aph ^ 1u)) {
          atomicCAS(p.status, 0, kDevTimeoutMma);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full_bar(s), ph)) {
            atomicCAS(p.status, 0, kDevTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_src = base + s * Cfg::STAGE_BYTES;
          const uint64_t da = umma_desc_k_sw128(a_src);
          const uint64_t db = umma_desc_k_sw128(a_src + Cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // 32 bytes further along K inside the swizzle row: +2 in the 16-byte address field
            umma<KIND>(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(empty_bar(s));          // frees the stage once these MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (ok) tc_commit(tfull_bar(as));   // accumulator complete
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;           // TMEM lanes [32*quarter, 32*quarter+32)
    int local = 0;
    const bool vec_c = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    const bool vec_r = p.residual == nullptr ||
                       ((p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0));
    const bool vec_b = p.bias == nullptr || ((reinterpret_cast<uintptr_t>(p.bias) & 15) == 0);
    const bool vec_cs = p.col_scale == nullptr || ((reinterpret_cast<uintptr_t>(p.col_scale) & 15) == 0);
    const bool vec_ok = vec_c && vec_r && vec_b && vec_cs;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++local) {
      const int as = local & 1;
      const uint32_t aph = (local >> 1) & 1u;
      const int m0 = (t / tiles_n) * BM;
      const int n0 = (t % tiles_n) * BN;
      if (!mbar_wait(tfull_bar(as), aph)) {
        if (lane == 0) atomicCAS(p.status, 0, kDevTimeoutEpilogue);
        break;
      }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const int rrow = p.res_mod > 0 ? row % p.res_mod : row;
      const float rs = (p.row_scale != nullptr && row_ok) ? p.row_scale[row] : 1.0f;
      const float a_scale = p.alpha * rs;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int c0 = n0 + c * 32;
        if (c0 >= p.N) break;               // warp-uniform
        uint32_t acc[32];
        tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(as * BN + c * 32), acc);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if constexpr (KIND == kKindI8) v[j] = static_cast<float>(static_cast<int>(acc[j])) * a_scale;
          else v[j] = __uint_as_float(acc[j]) * a_scale;
        }
        if (c0 + 32 <= p.N && vec_ok) {
          if (p.col_scale != nullptr) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.col_scale + c0) + q);
              v[q * 4] *= s4.x; v[q * 4 + 1] *= s4.y; v[q * 4 + 2] *= s4.z; v[q * 4 + 3] *= s4.w;
            }
          }
          if (p.bias != nullptr) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 b4 = __ldg(reinterpret_cast<const float4*>(p.bias + c0) + q);
              v[q * 4] += b4.x; v[q * 4 + 1] += b4.y; v[q * 4 + 2] += b4.z; v[q * 4 + 3] += b4.w;
            }
          }
          if (p.act != kActNone) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], p.act);
          }
          if (row_ok) {
            if (p.residual != nullptr) {
              const uint4* r4 = reinterpret_cast<const uint4*>(p.residual + (long long)rrow * p.ldr + c0);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 u = r4[q];
                const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 f = __half22float2(h[j]);
                  v[q * 8 + 2 * j] += f.x;
                  v[q * 8 + 2 * j + 1] += f.y;
                }
              }
            }
            const long long off = (long long)row * p.ldc + c0;
            if (p.out_dtype == kOutF16) store_chunk32<kOutF16>(p.C, off, v);
            else if (p.out_dtype == kOutF32) store_chunk32<kOutF32>(p.C, off, v);
            else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] *= p.out_scale;
              store_chunk32<kOutE4M3>(p.C, off, v);
            }
          }
        } else if (row_ok) {
          // ragged edge (N not a multiple of 32, or unaligned pitches): scalar, predicated;
          // fully unrolled so that v[] stays in registers
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = c0 + j;
            if (col < p.N) {
              float x = v[j];
              if (p.col_scale != nullptr) x *= p.col_scale[col];
              if (p.bias != nullptr) x += p.bias[col];
              x = apply_act(x, p.act);
              if (p.residual != nullptr) x += __half2float(p.residual[(long long)rrow * p.ldr + col]);
              if (p.out_dtype == kOutE4M3) x *= p.out_scale;
              store_one(p.C, p.out_dtype, (long long)row * p.ldc + col, x);
            }
          }
        }
      }
      // hand the accumulator buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(as));
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::ACC_COLS);
  }
}

}  // namespace crl
