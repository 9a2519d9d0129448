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
//   warps 2..17 : epilogue      - tcgen05.ld of the accumulator (a warp may read the 32 TMEM lanes
//                 its rank modulo 4 selects; four warps share a lane quarter and split the columns),
//                 then scale / bias / activation / residual, convert, store through a swizzled staging
//                 buffer and TMA stores. CTA pairs: one 32 x 64 slab per warp and tile (both TMEM loads in
//                 flight together, accumulator released before the arithmetic, one store; the residual
//                 slab arrives by TMA a tile ahead). Single CTAs: 32 x 32 chunks in a loop.
// All waits are bounded (see ptx.cuh); a wait that runs out records a status code and unwinds.
#pragma once
#include <cuda_runtime.h>
#include <type_traits>
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
  int use_tma_store;       // host built a tensor map for C (f16 / e4m3 output, 16-byte aligned pitch)
  int use_tma_res;         // host built a tensor map for the residual (res_mod == 0, 16-byte aligned pitch)
  // LNA kernels: A is LayerNorm(y) of these rows, produced inside the GEMM kernel by its own warps, a row block
  // ahead of the MMAs (see ln_rows_of_block). x (f16) and x8 (e4m3 * out8_scale) are written to global memory; the
  // tensor map of A points at whichever of the two the MMA kind consumes.
  const __half* ln_y;      // [M, K] f16, row pitch ln_ldy
  long long ln_ldy;
  const __half* ln_w16;    // [K] f16 LayerNorm weight
  const __half* ln_b16;    // [K] f16 LayerNorm bias
  __half* ln_x;            // [M, K] f16 out (nullable), pitch K
  uint8_t* ln_x8;          // [M, K] e4m3 out (nullable), pitch K
  float ln_out8_scale;
  int precise_act;         // 1: Mish into an e4m3 output in fp32 instead of on packed f16 pairs
  // LNO kernels: the output rows are LayerNorm(acc + bias + residual) over all N columns (N <= 1024, a multiple of
  // 256). The warps that hold the 128-column slabs of a row - in the CTAs working on the row block's column tiles -
  // exchange per-row sums through `lno_stats`, one 8-byte record (sum, sum of squares) per row and slab, preset to
  // all-ones bits before the launch. The f16 result goes to C (which may be the residual buffer itself), an e4m3
  // copy * lno_out8_scale to lno_x8.
  const __half* lno_w16;   // [N] f16 LayerNorm weight
  const __half* lno_b16;   // [N] f16 LayerNorm bias
  unsigned long long* lno_stats;   // [2][tiles_m][8 slabs][256 rows]: sums; row maxima (int8 copy)
  uint8_t* lno_x8;         // [M, N] e4m3 copy (nullable); int8 operands: the per-token int8 copy
  float* lno_qscale;       // int8 operands: [M] per-token scales of the int8 copy (row maximum / 127), with lno_x8
  float lno_out8_scale;
};

#ifndef CRL_PAIR_O8_STAGES
#define CRL_PAIR_O8_STAGES 5     // ring stages of the CTA-pair kernels with an e4m3 output (2 KB slabs leave room for 6)
#endif
constexpr int kGemmThreads = 576;   // TMA warp + MMA warp + 16 epilogue warps

constexpr int kEpiWarps = 16;
constexpr int kLnWarps = 6;          // LNA kernels: LayerNorm warps after the epilogue warps

// PAIR = 1: two CTAs of a cluster work on one 256 x BN tile with cta_group::2 MMAs. Each CTA stages
// its own 128 rows of A and its own BN/2 rows of W, so a pair moves a third less data from L2 into
// shared memory per FLOP than two independent CTAs; the leader CTA (cluster rank 0) issues the MMAs
// for both, each CTA drains the 128 accumulator rows that land in its own tensor memory.
// Pairs run the slab epilogue (one 32-row x 64-column slab per epilogue warp and tile, one TMA store each):
//   O8  = 1: the output is e4m3 (2 KB slabs), 0: f16 (4 KB slabs);
//   RES = 1 (f16 output only): the residual slab arrives by TMA in the warp's own slab buffer, requested a
//         tile ahead, and the result overwrites it in place before the store.
//   LNO = 1 (with RES): the slab is normalised over the whole output row before it is stored (see the epilogue).
template <int BN, int KIND, int PAIR = 0, int RES = 0, int O8 = 0, int LNA = 0, int LNO = 0>
struct GemmCfg {
  static_assert(!LNA || PAIR, "the fused LayerNorm exists for CTA pairs only");
  static_assert(!LNO || (PAIR && RES && !O8 && !LNA), "the output LayerNorm extends the residual kernel of CTA pairs");
  static constexpr int THREADS = kGemmThreads + (LNA ? 32 * kLnWarps : 0);
  static_assert(!(RES && O8), "the residual variant writes f16");
  static_assert(!PAIR || BN == 256, "pairs work on 256 x 256 tiles");
  static constexpr int BM = 128;           // rows per CTA
  static constexpr int TM = PAIR ? 256 : 128;  // rows per tile
  static constexpr int ESZ = (KIND == kKindF16) ? 2 : 1;
  static constexpr int BK = 128 / ESZ;   // elements per stage along K: one 128-byte swizzle row
  static constexpr int UK = 32 / ESZ;    // elements per tcgen05.mma along K
  static constexpr uint32_t A_BYTES = BM * 128;
  static constexpr uint32_t B_BYTES = (PAIR ? BN / 2 : BN) * 128;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  // single CTAs stage the tile's bias [2][BN] and per-column scales [2][BN] in shared memory; pairs read them
  // straight from global memory (L1-resident), which needs no barrier among the epilogue warps
  static constexpr uint32_t TAB_BYTES = PAIR ? 0 : 4 * BN * 4;
  // per epilogue warp: pairs one slab (32 rows x 64 columns of the output type), single CTAs one 32 x 32 chunk
  // (LNO: a 32 x 128 slab as two sub-slabs of 64 columns)
  static constexpr uint32_t SLOT_BYTES = PAIR ? (O8 ? 2048 : (LNO ? 8192 : 4096)) : 2048;
  // pairs: f16 slabs leave room for five 32 KB stages (four with the int8 scale table)
  // pairs: five 32 KB stages; the f16-output kernels with a fused LayerNorm give one up for its parameter table
  // (LNO kernels keep three: their 8 KB slabs take the room of two)
  static constexpr int STAGES = PAIR ? (LNO ? 3 : ((LNA && !O8) ? 4 : ((O8 && KIND != kKindI8) ? CRL_PAIR_O8_STAGES : 5)))
                                     : ((BN == 256) ? 3 : (BN == 128 ? 5 : 6));
  static constexpr uint32_t LN_PRM_BYTES = LNA ? 4096 : 0;    // LayerNorm weight [1024] and bias [1024] as f16
  static constexpr int ACC_COLS = 2 * BN;  // two accumulator buffers; 128, 256 or 512 columns
  // after the stages: the tables, the per-warp slabs (1024-byte aligned: TMA swizzles by absolute address
  // bits), then the mbarriers (ring, accumulators, one per epilogue warp for its residual slab) + TMEM slot
  static constexpr uint32_t EPI_OFF = STAGES * STAGE_BYTES;
  static constexpr uint32_t LN_PRM_OFF = EPI_OFF + TAB_BYTES + kEpiWarps * SLOT_BYTES;
  static constexpr uint32_t BAR_OFF = LN_PRM_OFF + LN_PRM_BYTES;
  // barrier region: [0,128) ring (2 x STAGES <= 12) and accumulator (4) mbarriers, [128,144) the TMEM address slot,
  // [144, 144 + 16 x 16) the epilogue warps' mbarriers (residual slabs), then the LayerNorm progress words
  static_assert(2 * STAGES + 4 <= 16, "the ring and accumulator barriers share 128 bytes");
  static constexpr uint32_t TMEM_SLOT_OFF = BAR_OFF + 128;
  static constexpr uint32_t RBAR_OFF = BAR_OFF + 144;
  static constexpr uint32_t LN_COUNTER_OFF = RBAR_OFF + kEpiWarps * 16;     // (room for two mbarriers per warp; one is used)
  static constexpr uint32_t USED_BYTES = LN_COUNTER_OFF + 48;   // [0] epilogue warps' arrivals, [4 + w] blocks done by LayerNorm warp w
  static constexpr size_t SMEM_BYTES = size_t(USED_BYTES) + ((PAIR && (!O8 || STAGES > 5)) ? 496 : 896) /*alignment slack*/;
  static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA can opt into");
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

__device__ __forceinline__ uint32_t pack_f16x2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void store_one(void* C, int out_dtype, long long off, float v) {
  if (out_dtype == kOutF16) reinterpret_cast<__half*>(C)[off] = __float2half_rn(v);
  else if (out_dtype == kOutF32) reinterpret_cast<float*>(C)[off] = v;
  else reinterpret_cast<uint8_t*>(C)[off] =
      static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ uint4 ln_load_row_piece(const __half* src) {
  uint4 u;      // streamed once: no L1 allocation
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(src));
  return u;
}

// LayerNorm (eps 1e-5, affine) of rows [row0, row0 + nrows) of p.ln_y, shared among `nw` warps: warp `wi` takes rows
// wi, wi + nw, ... with the next row's loads in flight while one is normalised. Same arithmetic as ln_rows_persistent_kernel (fp32 statistics, f16 affine), so a network gives
// the same bits whichever kernel normalises a row. K <= 1024, K % 8 == 0.
// One bulk L2 prefetch of a whole row of ln_y (a hint; issued by one lane).
__device__ __forceinline__ void ln_prefetch_row(const GemmParams& p, long long row) {
  if (row < p.M)
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.ln_y + row * p.ln_ldy), "r"(uint32_t(p.K) * 2u) : "memory");
}

// `next_first` / `next_nw`: the warp's first row and row stride in the block it will normalise after this one (-1:
// none). While row k is normalised, row k + 1 is on its way into registers and row k + 3 - of this block or the next -
// is requested into L2: close enough ahead to still be there, far enough to hide the HBM round trip.
__device__ __forceinline__ void ln_rows_of_block(const GemmParams& p, uint32_t prm_smem, long long row0, int nrows, int wi,
                                                 int nw, int lane, long long next_first = -1, int next_nw = 1) {
  constexpr int NV = 4;
  constexpr int kAhead = 3;
  const int d = p.K;
  long long row = row0 + wi;                            // the warp's rows wi, wi + nw, ...
  const long long end = (row0 + nrows < p.M) ? row0 + nrows : p.M;
  // first value of the sequence wi, wi + nw, ... beyond the block: rows past it continue in the next block
  const long long seq_end = row + ((end - row + nw - 1) / nw) * nw;
  auto prefetch_ahead = [&](long long r) {
    if (lane == 0) {
      if (r < end) ln_prefetch_row(p, r);
      else if (next_first >= 0) ln_prefetch_row(p, next_first + ((r - seq_end) / nw) * next_nw);
    }
  };
  if (row >= end) {
    if (next_first >= 0 && lane < kAhead) ln_prefetch_row(p, next_first + (long long)lane * next_nw);
    return;
  }
  uint4 raw[NV], nxt[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * 32 + lane) * 8;
    raw[i] = c < d ? ln_load_row_piece(p.ln_y + row * p.ln_ldy + c) : make_uint4(0u, 0u, 0u, 0u);
  }
  const __half2 s8 = __floats2half2_rn(p.ln_out8_scale, p.ln_out8_scale);
  for (; row < end; row += nw) {
    const long long nrow = row + nw;
    prefetch_ahead(row + (long long)kAhead * nw);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 8;
      nxt[i] = (nrow < end && c < d) ? ln_load_row_piece(p.ln_y + nrow * p.ln_ldy + c) : make_uint4(0u, 0u, 0u, 0u);
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
    const float mean = sum / d;
    const float rstd = rsqrtf(fmaxf(sq / d - mean * mean, 0.0f) + 1e-5f);
    const float shift = -mean * rstd;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < d) {
        const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
        uint4 w4, b4;      // this lane's 8 weight and 8 bias columns from the table in shared memory
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w4.x), "=r"(w4.y), "=r"(w4.z), "=r"(w4.w) : "r"(prm_smem + 2u * c));
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(b4.x), "=r"(b4.y), "=r"(b4.z), "=r"(b4.w) : "r"(prm_smem + 2048u + 2u * c));
        const __half2* wh = reinterpret_cast<const __half2*>(&w4);
        const __half2* bh = reinterpret_cast<const __half2*>(&b4);
        uint32_t o16[4];
        __half2 y2[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h[j]);
          const __half2 xn = __floats2half2_rn(fmaf(f.x, rstd, shift), fmaf(f.y, rstd, shift));
          y2[j] = __hfma2(xn, wh[j], bh[j]);
          o16[j] = *reinterpret_cast<const uint32_t*>(&y2[j]);
        }
        if (p.ln_x != nullptr) *reinterpret_cast<uint4*>(p.ln_x + row * p.K + c) = make_uint4(o16[0], o16[1], o16[2], o16[3]);
        if (p.ln_x8 != nullptr) {
          uint32_t w8[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const __half2 a = __hmul2(y2[2 * j], s8), b = __hmul2(y2[2 * j + 1], s8);
            w8[j] = uint32_t(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<const __half2_raw*>(&a), __NV_SATFINITE, __NV_E4M3)) |
                    (uint32_t(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<const __half2_raw*>(&b), __NV_SATFINITE, __NV_E4M3)) << 16);
          }
          *reinterpret_cast<uint2*>(p.ln_x8 + row * p.K + c) = make_uint2(w8[0], w8[1]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) raw[i] = nxt[i];
  }
}

// A warp's rows of a row block are written: make them visible to the TMA loads that will read them (generic-proxy
// stores, async-proxy loads of the same global memory), then publish the warp's progress.
//   add != 0: add 1 to the word (the epilogue warps' shared arrival count for the worker's first block)
//   add == 0: store `value` (a LayerNorm warp's own count of finished blocks)
__device__ __forceinline__ void ln_publish(uint32_t word_smem, int lane, int add, uint32_t value) {
  __threadfence();                                          // every lane's rows are in L2 ...
  asm volatile("fence.proxy.async.global;" ::: "memory");   // ... and ordered before async-proxy reads of them
  __syncwarp();
  if (lane == 0) {
    if (add) asm volatile("red.release.gpu.shared::cta.add.u32 [%0], 1;" ::"r"(word_smem) : "memory");
    else asm volatile("st.release.gpu.shared::cta.u32 [%0], %1;" ::"r"(word_smem), "r"(value) : "memory");
  }
}
// Bounded wait of the TMA producer until the epilogue warps have all counted in (first block) and every LayerNorm
// warp has finished `blocks` row blocks. Each warp publishes only its own progress, so a warp that runs ahead
// cannot stand in for one that is behind.
__device__ __forceinline__ bool ln_wait_blocks(uint32_t words_smem, uint32_t blocks) {
  unsigned long long t0 = 0;
  for (int i = 0;; ++i) {
    uint32_t v, lo = 0xffffffffu;
    asm volatile("ld.acquire.gpu.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(words_smem) : "memory");
    bool ok = v >= uint32_t(kEpiWarps);
#pragma unroll
    for (int w = 0; w < kLnWarps; ++w) {
      asm volatile("ld.acquire.gpu.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(words_smem + 16u + 4u * w) : "memory");
      lo = v < lo ? v : lo;
    }
    if (ok && lo >= blocks) {
      asm volatile("fence.proxy.async.global;" ::: "memory");
      return true;
    }
    if (i == 64) t0 = global_timer_ns();
    if (i > 64) {
      __nanosleep(100);
      if (global_timer_ns() - t0 > 2000000000ull) return false;
    }
  }
}

// EPI != 0 (CTA pairs; N a multiple of 64, 16-byte aligned tables; a residual only by TMA; int8 operands with per-token
// and per-channel scales, the others with neither): the epilogue's switches are fixed at compile time - 1: bias, no
// activation; 2: no bias, no activation; 3: bias and Mish (on packed f16 pairs where the output is e4m3) - which
// takes their tests and the untaken paths out of the hot instantiations. Same arithmetic as EPI = 0.
template <int BN, int KIND, int PAIR, int RES, int O8, int LNA, int LNO = 0, int EPI = 0>
__global__ void __launch_bounds__(kGemmThreads + (LNA ? 32 * kLnWarps : 0), 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmR,
               const __grid_constant__ CUtensorMap tmX8, const GemmParams p) {
  using Cfg = GemmCfg<BN, KIND, PAIR, RES, O8, LNA, LNO>;
  constexpr int BM = Cfg::BM, TM = Cfg::TM, BK = Cfg::BK, STAGES = Cfg::STAGES;
  // cluster rank (0 = leader) and the persistent worker this CTA belongs to
  const int rank = PAIR ? static_cast<int>(cluster_ctarank()) : 0;
  const int worker = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
  const int num_workers = PAIR ? (gridDim.x >> 1) : gridDim.x;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;          // swizzled tiles need 1024-byte alignment
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t bar0 = base + Cfg::BAR_OFF;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot =
      reinterpret_cast<uint32_t*>(smem + Cfg::TMEM_SLOT_OFF);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (base + Cfg::USED_BYTES > raw + Cfg::SMEM_BYTES) {   // dynamic smem less aligned than planned for
    if (threadIdx.x == 0) atomicCAS(p.status, 0, kDevBadSmemAlign);
    return;
  }

  const int tiles_m = (p.M + TM - 1) / TM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;
  // The i-th tile of this worker. Plain kernels deal the tiles out round-robin (n fastest); LNA kernels give a
  // worker whole row blocks (all column tiles of row block worker, worker + W, ...), because the worker's own
  // warps normalise the rows of a block before its first tile loads them.
  auto tile_of = [&](int i, int& mi, int& ni) -> bool {
    if constexpr (LNA) {
      mi = worker + (i / tiles_n) * num_workers;
      ni = (i % tiles_n + worker) % tiles_n;      // staggered: the workers do not all want the same W tile at once
      return mi < tiles_m;
    } else {
      const int t = worker + i * num_workers;
      mi = t / tiles_n;
      ni = t % tiles_n;
      return t < num_tiles;
    }
  };
  const uint32_t ln_counter = base + Cfg::LN_COUNTER_OFF;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int w = 0; w < 2 * kEpiWarps; ++w) mbar_init(base + Cfg::RBAR_OFF + 8u * w, 1);
    for (int w = 0; w < 12; ++w) asm volatile("st.shared::cta.u32 [%0], %1;" ::"r"(ln_counter + 4u * w), "r"(0u) : "memory");
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      // one arrival per epilogue warp (of both CTAs) that drains the buffer: all 16, or the 8 of a set (LNO)
      mbar_init(tempty_bar(a), (LNO ? kEpiWarps / 2 : kEpiWarps) * (PAIR ? 2 : 1));
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc<PAIR>(smem_u32(tmem_slot), Cfg::ACC_COLS);
    tmem_relinquish<PAIR>();
  }
  if constexpr (LNA) {
    // LayerNorm weight and bias (f16) into shared memory: every row needs them, and from global memory they would
    // put a second round trip behind each row's own loads
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
      const bool in = i % 128 * 8 < p.K;
      const __half* src = (i < 128 ? p.ln_w16 : p.ln_b16) + i % 128 * 8;
      const uint4 u = in ? __ldg(reinterpret_cast<const uint4*>(src)) : make_uint4(0u, 0u, 0u, 0u);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + Cfg::LN_PRM_OFF + 16u * i), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w) : "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync();      // the peer's barriers and tensor memory are ready too
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int mi = 0, ni = 0;
      for (int i = 0; ok && tile_of(i, mi, ni); ++i) {
        const int m0 = mi * TM + rank * BM;                  // this CTA's rows of A
        const int n0 = ni * BN + rank * (PAIR ? BN / 2 : 0);  // this CTA's rows of W
        if constexpr (LNA) {
          // the first tile of a row block waits until this CTA's 128 rows of it are normalised
          if (i % tiles_n == 0 && !ln_wait_blocks(ln_counter, uint32_t(i / tiles_n + 1))) {
            atomicCAS(p.status, 0, kDevTimeoutProducer);
            ok = false;
            break;
          }
        }
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u)) {
            atomicCAS(p.status, 0, kDevTimeoutProducer);
            ok = false;
            break;
          }
          const uint32_t a_dst = base + s * Cfg::STAGE_BYTES;
          const uint32_t b_dst = a_dst + Cfg::A_BYTES;
          if constexpr (PAIR) {
            // both CTAs' bytes are counted on the leader's barrier, which the MMA thread waits on
            const uint32_t lead_full = mapa_u32(full_bar(s), 0);
            if (rank == 0) mbar_expect_tx(full_bar(s), 2 * Cfg::STAGE_BYTES);
            tma_load_2d_pair(a_dst, &tmA, kb * BK, m0, lead_full);
            tma_load_2d_pair(b_dst, &tmB, kb * BK, n0, lead_full);
          } else {
            mbar_expect_tx(full_bar(s), Cfg::STAGE_BYTES);
            tma_load_2d(a_dst, &tmA, kb * BK, m0, full_bar(s));
            tma_load_2d(b_dst, &tmB, kb * BK, n0, full_bar(s));
          }
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc =
          umma_idesc(TM, BN, KIND == kKindI8 ? 1 : 0, KIND == kKindI8 ? 2 : 1);
      int s = 0;
      uint32_t ph = 0;
      int local = 0;
      bool ok = true;
      int mi = 0, ni = 0;
      for (; ok && tile_of(local, mi, ni); ++local) {
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
            umma<KIND, PAIR>(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit<PAIR>(empty_bar(s));    // frees the stage (in both CTAs) once these MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (ok) tc_commit<PAIR>(tfull_bar(as));   // accumulator complete
      }
    }
    __syncwarp();
  } else if (LNA != 0 && warp >= 2 + kEpiWarps) {
    // ------------------------------------------------------------------ LayerNorm warps (LNA kernels)
    // This CTA's 128 rows of every row block of the worker, block after block, normalised into x / x8 ahead of
    // the TMA producer (which waits for a block's rows before it loads the block's first tile). The worker's
    // first block is shared with the epilogue warps, which have nothing to drain yet; the rows of the block
    // after the one in work are requested into L2 while it is normalised.
    const int lw = warp - 2 - kEpiWarps;
    const uint32_t prm = base + Cfg::LN_PRM_OFF;
    if (worker < tiles_m && lane < 3)      // the warp's first rows, before anything else
      ln_prefetch_row(p, (long long)worker * TM + rank * BM + kEpiWarps + lw + (long long)lane * (kEpiWarps + kLnWarps));
    for (int j = 0;; ++j) {
      const int mi = worker + j * num_workers;
      if (mi >= tiles_m) break;
      const long long row0 = (long long)mi * TM + rank * BM;
      const long long next_first = (mi + num_workers < tiles_m) ? row0 + (long long)num_workers * TM + lw : -1;
      if (j == 0) ln_rows_of_block(p, prm, row0, BM, kEpiWarps + lw, kEpiWarps + kLnWarps, lane, next_first, kLnWarps);
      else ln_rows_of_block(p, prm, row0, BM, lw, kLnWarps, lane, next_first, kLnWarps);
      ln_publish(ln_counter + 16u + 4u * lw, lane, 0, uint32_t(j + 1));
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int ew = warp - 2;                // 0..15
    const int quarter = warp & 3;           // TMEM lanes [32*quarter, 32*quarter+32)
    const int part = ew >> 2;
    const int et = threadIdx.x - 64;        // 0..511 among the epilogue threads
    float* bias_s = reinterpret_cast<float*>(smem + Cfg::EPI_OFF);                  // [2][BN]
    float* cs_s = bias_s + 2 * BN;                                                  // [2][BN] per-column scales (int8)
    if constexpr (LNO) {
      // Slab epilogue with the LayerNorm of the output row. The 16 epilogue warps form two sets of 8 that take the
      // worker's tiles in turn (set s drains accumulator buffer s), so that a warp has two tile times for its chain of
      // dependent waits: accumulator -> y = acc + bias + residual as f16 into the warp's 32 x 128 slab (over the
      // residual TMA put there) -> the row's sum and sum of squares over these 128 columns into the statistics
      // record of (row, slab) -> the 2 tiles_n records of the row, written by the warps that hold the row's other
      // slabs in this CTA and in the CTAs working on the row block's other column tiles -> normalise in place ->
      // TMA store (f16) and plain stores (e4m3 copy) -> residual slab of the set's next tile.
      // (The shared-memory loads and stores below are volatile asm without a memory clobber: they keep their order among
      // themselves and with every barrier, fence and TMA operation - all volatile asm too - while the read-only
      // parameter loads around them stay free to be scheduled early.)
      // EPI != 0 fixes the switches at compile time (f16 / e4m3 operands): 1 = bias and an e4m3 copy, 2 = bias, no copy
      constexpr bool kSpecL = EPI != 0 && KIND != kKindI8;
      const bool l_bias = kSpecL ? true : (p.bias != nullptr);
      const bool l_copy = kSpecL ? (EPI == 1) : (p.lno_x8 != nullptr);
      const int set = ew >> 3;
      const int half = (ew >> 2) & 1;          // columns [128 half, +128) of the CTA's 256
      const uint32_t slab = base + Cfg::EPI_OFF + Cfg::TAB_BYTES + ew * Cfg::SLOT_BYTES;     // two 32 x 64 sub-slabs
      const uint32_t rbar = base + Cfg::RBAR_OFF + 8u * ew;
      const int slabs = 2 * tiles_n;
      bool res_pending = false;
      uint32_t pending_ph = 0;
      auto res_issue = [&](int i) {
        int rm, rn;
        tile_of(i, rm, rn);
        pending_ph = (i >> 1) & 1u;
        if (lane == 0) {
          mbar_expect_tx(rbar, 8192u);
          tma_load_2d(slab, &tmR, rn * BN + half * 128, rm * TM + rank * BM + quarter * 32, rbar);
          tma_load_2d(slab + 4096u, &tmR, rn * BN + half * 128 + 64, rm * TM + rank * BM + quarter * 32, rbar);
        }
        res_pending = true;
      };
      auto exists = [&](int i) {
        int rm, rn;
        return tile_of(i, rm, rn);
      };
      if (exists(set)) res_issue(set);
      const __half2 s8 = __floats2half2_rn(p.lno_out8_scale, p.lno_out8_scale);
      const float inv_n = 1.0f / static_cast<float>(p.N);
      const float a_scale = p.alpha;
      // Bounded wait for the `slabs` records of this lane's row; returns their sums (low and high word as floats), or
      // the maximum of the low words.
      auto poll_records = [&](const unsigned long long* recs, float& lo, float& hi, auto take_max) -> bool {
        unsigned long long t0 = 0;
        for (int it = 0;; ++it) {
          bool ok = true;
          unsigned long long r[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            r[j] = 0ull;
            if (j < slabs) asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(r[j]) : "l"(recs + (long long)j * TM) : "memory");
          }
          lo = 0.0f; hi = 0.0f;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            ok = ok && r[j] != ~0ull;
            const float a = __uint_as_float(static_cast<uint32_t>(r[j]));
            if constexpr (decltype(take_max)::value) {
              lo = fmaxf(lo, a);
            } else {
              lo += a;
              hi += __uint_as_float(static_cast<uint32_t>(r[j] >> 32));
            }
          }
          if (__all_sync(0xffffffffu, ok)) return true;
          if (it == 8) t0 = global_timer_ns();
          if (it > 8) {
            __nanosleep(64);
            const bool late = global_timer_ns() - t0 > 2000000000ull;
            if (__any_sync(0xffffffffu, late)) return false;
          }
        }
      };
      bool alive = true;
      int mi = 0, ni = 0;
      for (int local = set; tile_of(local, mi, ni); local += 2) {
        const uint32_t ph = (local >> 1) & 1u;      // the set's k-th tile: accumulator buffer and slab phase k & 1
        if (!mbar_wait(tfull_bar(set), ph)) {
          alive = false;
          break;
        }
        tc_fence_after();
        if (!mbar_wait(rbar, ph)) {      // the residual slab has landed
          alive = false;
          break;
        }
        res_pending = false;
        {
          // the residual slab of the set's next tile can only land once this tile's stores have read the buffer:
          // have it waiting in L2 by then
          int rm, rn;
          if (lane == 0 && tile_of(local + 2, rm, rn)) {
            tma_prefetch_l2_2d(&tmR, rn * BN + half * 128, rm * TM + rank * BM + quarter * 32);
            tma_prefetch_l2_2d(&tmR, rn * BN + half * 128 + 64, rm * TM + rank * BM + quarter * 32);
          }
        }
        const int c0 = ni * BN + half * 128;
        const int row0 = mi * TM + rank * BM + quarter * 32;
        const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(set * BN + half * 128);
        float row_scale = a_scale;
        if constexpr (KIND == kKindI8) {
          if (p.row_scale != nullptr && row0 + lane < p.M) row_scale *= p.row_scale[row0 + lane];
        }
        uint32_t acc[32];
        // (four independent partial sums each: one running sum would chain 128 dependent additions)
        float ps[4] = {0.0f, 0.0f, 0.0f, 0.0f}, pq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        auto chunk_off = [&](int k) {      // k-th 16-byte chunk (8 columns) of this lane's 128-column row
          const int q = k & 7;
          return slab + 4096u * (k >> 3) + lane * 128 + ((q ^ (lane & 7)) << 4);
        };
        uint4 rnext;      // the residual's next chunk, requested one chunk ahead of its use
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(rnext.x), "=r"(rnext.y), "=r"(rnext.z), "=r"(rnext.w) : "r"(chunk_off(0)));
#pragma unroll 1
        for (int g = 0; g < 4; ++g) {
          tmem_ld_32x32(taddr + 32u * g, acc);
          tmem_ld_wait();
          if (g == 3) {
            // the last columns sit in registers: the accumulator buffer goes back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if (rank != 0) mbar_arrive_cluster(mapa_u32(tempty_bar(set), 0));   // the leader's barrier
              else mbar_arrive(tempty_bar(set));
            }
          }
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int k = g * 4 + c;
            const uint4 u = rnext;
            if (k + 1 < 16)
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(rnext.x), "=r"(rnext.y), "=r"(rnext.z), "=r"(rnext.w) : "r"(chunk_off(k + 1)));
            float v[8];
            if constexpr (KIND == kKindI8) {
              // int32 accumulators, alpha x the row's scale x the column scales
              float sc[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) sc[j] = row_scale;
              if (p.col_scale != nullptr) {
                const float4 s0 = __ldg(reinterpret_cast<const float4*>(p.col_scale + c0 + k * 8));
                const float4 s1 = __ldg(reinterpret_cast<const float4*>(p.col_scale + c0 + k * 8 + 4));
                sc[0] *= s0.x; sc[1] *= s0.y; sc[2] *= s0.z; sc[3] *= s0.w;
                sc[4] *= s1.x; sc[5] *= s1.y; sc[6] *= s1.z; sc[7] *= s1.w;
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = static_cast<float>(static_cast<int>(acc[c * 8 + j])) * sc[j];
              if (l_bias) {
                const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.bias + c0 + k * 8));
                const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.bias + c0 + k * 8 + 4));
                v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
                v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
              }
            } else if (l_bias) {
              const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.bias + c0 + k * 8));
              const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.bias + c0 + k * 8 + 4));
              const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = fmaf(__uint_as_float(acc[c * 8 + j]), row_scale, bb[j]);
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(acc[c * 8 + j]) * row_scale;
            }
            const __half2* h = reinterpret_cast<const __half2*>(&u);
            uint32_t ws[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __half22float2(h[j]);
              const float y0 = v[2 * j] + f.x, y1 = v[2 * j + 1] + f.y;
              ws[j] = pack_f16x2(y0, y1);
              // row statistics from the fp32 sums (the stored f16 values differ from them by their rounding only)
              ps[j] += y0 + y1;
              pq[j] = fmaf(y0, y0, fmaf(y1, y1, pq[j]));
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(chunk_off(k)), "r"(ws[0]), "r"(ws[1]), "r"(ws[2]), "r"(ws[3]));
          }
        }
        const float lsum = (ps[0] + ps[1]) + (ps[2] + ps[3]), lsq = (pq[0] + pq[1]) + (pq[2] + pq[3]);
        const unsigned long long* recs = p.lno_stats + (long long)mi * 8 * TM + rank * BM + quarter * 32 + lane;
        {
          const unsigned long long pk = (static_cast<unsigned long long>(__float_as_uint(lsq)) << 32) | __float_as_uint(lsum);
          asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(recs + (long long)(ni * 2 + half) * TM), "l"(pk) : "memory");
        }
        // the row's records (each is valid as soon as it is not the preset all-ones pattern: a record is one 8-byte
        // store), added in a fixed order: a row's result does not depend on who computes it
        float S = 0.0f, Q = 0.0f;
        if (!poll_records(recs, S, Q, std::false_type{})) {
          alive = false;
          break;
        }
        const float mean = S * inv_n;
        const float rstd = rsqrtf(fmaxf(Q * inv_n - mean * mean, 0.0f) + 1e-5f);
        const float shift = -mean * rstd;
        const bool row_ok = row0 + lane < p.M;
        uint32_t w8[32];      // the e4m3 (int8) copy of this lane's 128 columns
        __half2 m2 = __float2half2_rn(0.0f);      // int8: largest |x'| of this lane's 128 columns
        uint4 ynext;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(ynext.x), "=r"(ynext.y), "=r"(ynext.z), "=r"(ynext.w) : "r"(chunk_off(0)));
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          const uint4 u = ynext;
          if (k + 1 < 16)
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(ynext.x), "=r"(ynext.y), "=r"(ynext.z), "=r"(ynext.w) : "r"(chunk_off(k + 1)));
          const uint4 w4 = __ldg(reinterpret_cast<const uint4*>(p.lno_w16 + c0 + k * 8));
          const uint4 b4 = __ldg(reinterpret_cast<const uint4*>(p.lno_b16 + c0 + k * 8));
          const __half2* h = reinterpret_cast<const __half2*>(&u);
          const __half2* wh = reinterpret_cast<const __half2*>(&w4);
          const __half2* bh = reinterpret_cast<const __half2*>(&b4);
          __half2 y2[4];
          uint32_t o16[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            const __half2 xn = __floats2half2_rn(fmaf(f.x, rstd, shift), fmaf(f.y, rstd, shift));
            y2[j] = __hfma2(xn, wh[j], bh[j]);
            o16[j] = *reinterpret_cast<const uint32_t*>(&y2[j]);
          }
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(chunk_off(k)), "r"(o16[0]), "r"(o16[1]), "r"(o16[2]), "r"(o16[3]));
          if constexpr (KIND == kKindI8) {
#pragma unroll
            for (int j = 0; j < 4; ++j) m2 = __hmax2(m2, __habs2(y2[j]));
          } else if (l_copy) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const __half2 a = __hmul2(y2[2 * j], s8), b = __hmul2(y2[2 * j + 1], s8);
              w8[k * 2 + j] = uint32_t(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<const __half2_raw*>(&a), __NV_SATFINITE, __NV_E4M3)) |
                              (uint32_t(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<const __half2_raw*>(&b), __NV_SATFINITE, __NV_E4M3)) << 16);
            }
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tmC, slab, c0, row0);      // rows beyond the matrix are clipped by the TMA unit
          tma_store_2d(&tmC, slab + 4096u, c0 + 64, row0);
          bulk_commit();
        }
        if constexpr (KIND == kKindI8) {
          if (p.lno_qscale != nullptr) {
            // per-token int8 copy: the largest |x'| of the whole row, exchanged like the sums (second half of the
            // record buffer), then the slab's values quantised with the row's scale
            const unsigned long long* arecs = recs + (long long)tiles_m * 8 * TM;
            const unsigned long long pk = __float_as_uint(fmaxf(__low2float(m2), __high2float(m2)));
            asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(arecs + (long long)(ni * 2 + half) * TM), "l"(pk) : "memory");
            float amax = 0.0f, unused = 0.0f;
            if (!poll_records(arecs, amax, unused, std::true_type{})) {
              alive = false;
              break;
            }
            const float qs = amax > 0.0f ? amax / 127.0f : 1.0f;
            const float qinv = 1.0f / qs;
            if (ni == 0 && half == 0 && row_ok) p.lno_qscale[row0 + lane] = qs;
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              uint4 u;
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "r"(chunk_off(k)));
              const __half2* h = reinterpret_cast<const __half2*>(&u);
              uint32_t b8[8];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                b8[2 * j] = static_cast<uint32_t>(max(-127, min(127, __float2int_rn(f.x * qinv)))) & 0xffu;
                b8[2 * j + 1] = static_cast<uint32_t>(max(-127, min(127, __float2int_rn(f.y * qinv)))) & 0xffu;
              }
              w8[k * 2] = b8[0] | (b8[1] << 8) | (b8[2] << 16) | (b8[3] << 24);
              w8[k * 2 + 1] = b8[4] | (b8[5] << 8) | (b8[6] << 16) | (b8[7] << 24);
            }
          }
        }
        if (l_copy) {
          // the e4m3 copy leaves the same way: once the stores above have read the slab, its first 4 KB take the 32
          // rows of 128 bytes (the same 128-byte swizzle), and one more TMA store follows
          if (lane == 0) bulk_wait_read0();
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t off = slab + lane * 128 + ((q ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(off), "r"(w8[q * 4]), "r"(w8[q * 4 + 1]), "r"(w8[q * 4 + 2]), "r"(w8[q * 4 + 3]));
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmX8, slab, c0, row0);
            bulk_commit();
          }
        }
        if (exists(local + 2)) {
          if (lane == 0) bulk_wait_read0();          // the stores have read the slab: the next residual slab may land
          res_issue(local + 2);
        }
      }
      if (!alive) {
        if (lane == 0) atomicCAS(p.status, 0, kDevTimeoutEpilogue);
        if (res_pending) mbar_wait(rbar, pending_ph);      // no copy into this CTA's memory stays in flight
      }
      if (lane == 0) bulk_wait_all();   // this warp's TMA stores have left shared memory and landed
      __syncwarp();
    } else if constexpr (PAIR) {
      // Slab epilogue. Per tile this warp owns rows [32*quarter, +32) x columns [64*part, +64) of the CTA's
      // accumulator half, drained in two TMEM loads of 32 columns; the accumulator buffer goes back to the MMA warp
      // as soon as the second load has landed in registers, before the arithmetic on it, and the finished slab
      // leaves through one TMA store (64- or 128-byte rows). The slab buffer is
      // free again long before the next tile needs it, so no store is ever waited for inside a tile.
      const uint32_t slot = base + Cfg::EPI_OFF + Cfg::TAB_BYTES + ew * Cfg::SLOT_BYTES;
      const uint32_t rbar = base + Cfg::RBAR_OFF + 8u * ew;
      uint32_t rph = 0;
      bool res_pending = false;
      // RES: the residual slab (32 rows x 64 f16, 128-byte swizzle) is fetched into the slab buffer itself, a tile
      // ahead: right after this tile's store has read the buffer.
      auto res_issue = [&](int i) {
        int rm, rn;
        tile_of(i, rm, rn);
        if (lane == 0) {
          mbar_expect_tx(rbar, 4096u);
          tma_load_2d(slot, &tmR, rn * BN + part * 64, rm * TM + rank * BM + quarter * 32, rbar);
        }
        res_pending = true;
      };
      // the residual slab of this worker's i-th tile is wanted if that tile exists and this warp's columns lie in it
      auto res_wanted = [&](int i) {
        int rm, rn;
        return tile_of(i, rm, rn) && rn * BN + part * 64 < p.N;
      };
      const bool tma_res = (EPI != 0) ? (RES != 0) : (RES != 0 && p.use_tma_res != 0 && p.residual != nullptr);
      if (RES != 0 && tma_res && res_wanted(0)) res_issue(0);
      constexpr bool kSpec = EPI != 0;
      static_assert(!kSpec || !LNA, "specialised epilogues: not for the kernels with a LayerNorm in front");
      const bool has_bias = kSpec ? (EPI != 2) : (p.bias != nullptr);
      const int act = kSpec ? (EPI == 3 ? kActMish : kActNone) : p.act;
      const bool mish8 = kSpec ? (EPI == 3 && O8 != 0) : (O8 != 0 && p.act == kActMish && p.residual == nullptr && p.precise_act == 0);
      if constexpr (LNA) {
        // the worker's first row block: nothing to drain yet, so the epilogue warps normalise rows too
        if (worker < tiles_m) {
          const long long row0 = (long long)worker * TM + rank * BM;
          if (lane < 3) ln_prefetch_row(p, row0 + ew + (long long)lane * (kEpiWarps + kLnWarps));
          ln_rows_of_block(p, base + Cfg::LN_PRM_OFF, row0, BM, ew, kEpiWarps + kLnWarps, lane);
        }
        ln_publish(ln_counter, lane, 1, 0u);
      }
      bool alive = true;
      int local = 0;
      int mi = 0, ni = 0;
      for (; tile_of(local, mi, ni); ++local) {
        const int as = local & 1;
        const uint32_t aph = (local >> 1) & 1u;
        const int m0 = mi * TM + rank * BM;   // first row of this CTA's accumulator half
        const int n0 = ni * BN;
        // (no barrier among the epilogue warps anywhere in this loop: a warp that is late - a residual slab or a
        // LayerNorm row still on its way - must not keep the others from draining the next accumulator)
        if (!mbar_wait(tfull_bar(as), aph)) {
          if (lane == 0) atomicCAS(p.status, 0, kDevTimeoutEpilogue);
          alive = false;
          break;
        }
        tc_fence_after();
        const int c0 = n0 + part * 64;
        const bool active = c0 < p.N;       // warp-uniform
        if (!active) {
          // nothing to drain: hand the accumulator buffer back, keep the residual pipeline moving
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (rank != 0) mbar_arrive_cluster(mapa_u32(tempty_bar(as), 0));   // the leader's barrier
            else mbar_arrive(tempty_bar(as));
          }
          if (RES != 0 && tma_res && res_wanted(local + 1)) {
            if (lane == 0) bulk_wait_read0();
            res_issue(local + 1);
          }
          continue;
        }
        const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(as * BN + part * 64);
        const int row = m0 + quarter * 32 + lane;
        const bool row_ok = row < p.M;
        const int rrow = p.res_mod > 0 ? row % p.res_mod : row;
        // (specialised epilogues: int8 operands come with per-token and per-channel scales, the others with neither)
        const float rs = kSpec ? ((KIND == kKindI8 && row_ok) ? p.row_scale[row] : 1.0f)
                               : ((p.row_scale != nullptr && row_ok) ? p.row_scale[row] : 1.0f);
        // e4m3 output without an activation or residual: out = (alpha acc + bias) s = (alpha s) acc + (bias s), one
        // multiply-add per element instead of three operations
        const bool fold = kSpec ? (O8 != 0 && EPI != 3) : (O8 != 0 && p.act == kActNone && p.residual == nullptr);
        const float os = fold ? 1.0f : p.out_scale;
        const float bs = fold ? p.out_scale : 1.0f;
        const float a_scale = p.alpha * rs * bs;
        // the slab buffer: the residual slab has landed in it (RES), or the previous tile's store has read it
        if (RES != 0 && tma_res) {
          if (!mbar_wait(rbar, rph)) {
            if (lane == 0) atomicCAS(p.status, 0, kDevTimeoutEpilogue);
            alive = false;
            break;
          }
          rph ^= 1u;
          res_pending = false;
        } else {
          if (lane == 0) bulk_wait_read0();
          __syncwarp();
        }
        const bool direct_res = kSpec ? false : (p.residual != nullptr && !(RES != 0 && tma_res) && row_ok);
        // bias and per-column scales: 16 floats per piece, the same addresses for every lane (one L1 transaction each)
        const bool tab_vec = kSpec ? true
                                   : (c0 + 64 <= p.N && (p.bias == nullptr || (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) &&
                                      (p.col_scale == nullptr || (reinterpret_cast<uintptr_t>(p.col_scale) & 15) == 0));
        const bool res_vec = (p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0);
        // two TMEM loads of 32 columns, each waited for before anything else touches its registers (a tcgen05.ld
        // fills them asynchronously); each half is then worked on as two pieces of 16 columns
        uint32_t acc[32];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if ((i & 1) == 0) {
            tmem_ld_32x32(taddr + 16u * i, acc);
            tmem_ld_wait();
            if (i == 2) {
              // the last columns sit in registers: the accumulator buffer goes back to the MMA warp
              tc_fence_before();
              __syncwarp();
              if (lane == 0) {
                if (rank != 0) mbar_arrive_cluster(mapa_u32(tempty_bar(as), 0));   // the leader's barrier
                else mbar_arrive(tempty_bar(as));
              }
            }
          }
          float v[16];
          float sc[16];      // per-element multiplier of the raw accumulator: alpha, row scale (and column scale)
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if constexpr (KIND == kKindI8) v[j] = static_cast<float>(static_cast<int>(acc[(i & 1) * 16 + j]));
            else v[j] = __uint_as_float(acc[(i & 1) * 16 + j]);
            sc[j] = a_scale;
          }
          if constexpr (KIND == kKindI8) {
            if (kSpec || p.col_scale != nullptr) {
              if (tab_vec) {
                const float4* c4p = reinterpret_cast<const float4*>(p.col_scale + c0 + i * 16);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const float4 c4 = __ldg(c4p + q);
                  sc[q * 4] *= c4.x; sc[q * 4 + 1] *= c4.y; sc[q * 4 + 2] *= c4.z; sc[q * 4 + 3] *= c4.w;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) sc[j] *= (c0 + i * 16 + j < p.N) ? __ldg(p.col_scale + c0 + i * 16 + j) : 0.0f;
              }
            }
          }
          // v = raw * sc + bias * bs: one multiply-add per element when bs is 1 (no folded output scale)
          float bv[16];
          if (has_bias) {
            if (tab_vec) {
              const float4* b4p = reinterpret_cast<const float4*>(p.bias + c0 + i * 16);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float4 b4 = __ldg(b4p + q);
                bv[q * 4] = b4.x; bv[q * 4 + 1] = b4.y; bv[q * 4 + 2] = b4.z; bv[q * 4 + 3] = b4.w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) bv[j] = (c0 + i * 16 + j < p.N) ? __ldg(p.bias + c0 + i * 16 + j) : 0.0f;
            }
            if (fold) {
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = fmaf(v[j], sc[j], bv[j] * bs);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = fmaf(v[j], sc[j], bv[j]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] *= sc[j];
          }
          // activation: the switch sits outside the element loop so that the independent evaluations interleave;
          // Mish into an e4m3 output runs on packed f16 pairs at the conversion below
          if (mish8) {
          } else if (act == kActMish) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = act_mish(v[j]);
          } else if (act == kActGelu) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = act_gelu(v[j]);
          } else if (act == kActRelu) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = fmaxf(v[j], 0.0f);
          }
          if constexpr (O8) {
            // ---- e4m3 slab: 64-byte rows, 64-byte swizzle (16-byte chunk q of row r at q ^ ((r >> 1) & 3))
            if (direct_res) {      // rare (no hot GEMM adds a residual into an e4m3 output): scalar loads
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c0 + i * 16 + j < p.N) v[j] += __half2float(p.residual[(long long)rrow * p.ldr + c0 + i * 16 + j]);
            }
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float* e = &v[j * 4];
              if (mish8) {
                const __half2 s2 = __float2half2_rn(p.out_scale);
                const uint32_t y0 = mish_f16x2(pack_f16x2(e[0], e[1])), y1 = mish_f16x2(pack_f16x2(e[2], e[3]));
                const __half2 z0 = __hmul2(*reinterpret_cast<const __half2*>(&y0), s2);
                const __half2 z1 = __hmul2(*reinterpret_cast<const __half2*>(&y1), s2);
                w[j] = uint32_t(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<const __half2_raw*>(&z0), __NV_SATFINITE, __NV_E4M3)) |
                       (uint32_t(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<const __half2_raw*>(&z1), __NV_SATFINITE, __NV_E4M3)) << 16);
              } else if (fold) {
                w[j] = uint32_t(__nv_cvt_float2_to_fp8x2(make_float2(e[0], e[1]), __NV_SATFINITE, __NV_E4M3)) |
                       (uint32_t(__nv_cvt_float2_to_fp8x2(make_float2(e[2], e[3]), __NV_SATFINITE, __NV_E4M3)) << 16);
              } else {
                w[j] = uint32_t(__nv_cvt_float2_to_fp8x2(make_float2(e[0] * os, e[1] * os), __NV_SATFINITE, __NV_E4M3)) |
                       (uint32_t(__nv_cvt_float2_to_fp8x2(make_float2(e[2] * os, e[3] * os), __NV_SATFINITE, __NV_E4M3)) << 16);
              }
            }
            const uint32_t off8 = slot + lane * 64 + ((i ^ ((lane >> 1) & 3)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(off8), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
          } else {
            // ---- f16 slab: 128-byte rows, 128-byte swizzle (16-byte chunk q of row r at q ^ (r & 7))
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              const int q = i * 2 + h2;
              const uint32_t off = slot + lane * 128 + ((q ^ (lane & 7)) << 4);
              if (RES != 0 && tma_res) {
                uint4 u;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "r"(off));
                const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 f = __half22float2(h[j]);
                  v[h2 * 8 + 2 * j] += f.x;
                  v[h2 * 8 + 2 * j + 1] += f.y;
                }
              } else if (direct_res) {
                // residual without a tensor map (a broadcast table, an unaligned pitch): this row's 16 bytes
                if (c0 + q * 8 + 8 <= p.N && res_vec) {
                  const uint4 u = *reinterpret_cast<const uint4*>(p.residual + (long long)rrow * p.ldr + c0 + q * 8);
                  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(h[j]);
                    v[h2 * 8 + 2 * j] += f.x;
                    v[h2 * 8 + 2 * j + 1] += f.y;
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    if (c0 + q * 8 + j < p.N) v[h2 * 8 + j] += __half2float(p.residual[(long long)rrow * p.ldr + c0 + q * 8 + j]);
                }
              }
              const uint32_t w0 = pack_f16x2(v[h2 * 8 + 0], v[h2 * 8 + 1]), w1 = pack_f16x2(v[h2 * 8 + 2], v[h2 * 8 + 3]);
              const uint32_t w2 = pack_f16x2(v[h2 * 8 + 4], v[h2 * 8 + 5]), w3 = pack_f16x2(v[h2 * 8 + 6], v[h2 * 8 + 7]);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(off), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
            }
          }
        }
        fence_proxy_async_smem();   // every writing lane, before the barrier (the documented order)
        __syncwarp();
        if (lane == 0) {
          // rows and columns beyond the matrix are clipped by the TMA unit
          tma_store_2d(&tmC, slot, c0, m0 + quarter * 32);
          bulk_commit();
        }
        if (RES != 0 && tma_res) {
          if (res_wanted(local + 1)) {
            if (lane == 0) bulk_wait_read0();   // the store above has read the buffer: the next residual slab may land
            res_issue(local + 1);
          }
        }
      }
      if (RES != 0 && res_pending) mbar_wait(rbar, rph);   // only after a timeout: no copy into this CTA's memory stays in flight
      if (lane == 0) bulk_wait_all();   // this warp's TMA stores have left shared memory and landed
      __syncwarp();
    } else {
      const int chunk_part = part;   // this warp takes the 32-column chunks part, part+4, ...
      (void)chunk_part;
      const uint32_t stage_u = base + Cfg::EPI_OFF + Cfg::TAB_BYTES + ew * 2048;       // 32 rows x 64 B
      // 16-byte chunk q of staged row r; XOR swizzle keeps both access patterns bank-conflict free
      auto stage_off = [&](int r, int q) { return stage_u + r * 64 + ((q ^ ((r >> 1) & 3)) << 4); };

      const bool al_c = (reinterpret_cast<uintptr_t>(p.C) & 15) == 0 && p.ldc % 8 == 0;
      const bool al_r = p.residual == nullptr ||
                        ((p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0));
      const bool al_b = p.bias == nullptr || ((reinterpret_cast<uintptr_t>(p.bias) & 15) == 0);
      const bool al_cs = p.col_scale == nullptr || ((reinterpret_cast<uintptr_t>(p.col_scale) & 15) == 0);
      const bool vec_ok = al_c && al_r && al_b && al_cs;
      // staged path: f16 / e4m3 outputs on aligned buffers (the shapes of the network's hot GEMMs)
      const bool staged_ok = p.use_tma_store != 0 && al_r && p.out_dtype != kOutF32;
      bool alive = true;
      int local = 0;
      for (int t = worker; t < num_tiles; t += num_workers, ++local) {
        const int as = local & 1;
        const uint32_t aph = (local >> 1) & 1u;
        const int m0 = (t / tiles_n) * TM + rank * BM;   // first row of this CTA's accumulator half
        const int n0 = (t % tiles_n) * BN;
        // this tile's bias slice goes to shared memory while the MMAs are still running
        if (p.bias != nullptr) {
          for (int e = et; e < BN; e += kEpiWarps * 32) bias_s[as * BN + e] = (n0 + e < p.N) ? __ldg(p.bias + n0 + e) : 0.0f;
        }
        if (p.col_scale != nullptr) {
          for (int e = et; e < BN; e += kEpiWarps * 32) cs_s[as * BN + e] = (n0 + e < p.N) ? __ldg(p.col_scale + n0 + e) : 0.0f;
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");   // epilogue warps only; also orders reuse of bias_s
        if (alive && !mbar_wait(tfull_bar(as), aph)) {
          if (lane == 0) atomicCAS(p.status, 0, kDevTimeoutEpilogue);
          alive = false;           // keep iterating so that the named barrier above stays balanced
        }
        if (!alive) continue;
        tc_fence_after();
        const int row = m0 + quarter * 32 + lane;
        const bool row_ok = row < p.M;
        const int rrow = p.res_mod > 0 ? row % p.res_mod : row;
        const float rs = (p.row_scale != nullptr && row_ok) ? p.row_scale[row] : 1.0f;
        const float a_scale = p.alpha * rs;
  #pragma unroll 1
        for (int c = part; c < BN / 32; c += 4) {
          const int c0 = n0 + c * 32;
          if (c0 >= p.N) break;               // warp-uniform
          const bool staged = staged_ok && c0 + 32 <= p.N;
          // residual rows in the coalesced mapping (lane -> row (lane>>2)+8i, 16-byte chunk lane&3),
          // requested before the accumulator is touched so that the latency overlaps
          uint4 rres[4];
          if (staged && p.residual != nullptr) {
  #pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int gr = m0 + quarter * 32 + (lane >> 2) + 8 * i;
              if (gr < p.M) {
                const int rr = p.res_mod > 0 ? gr % p.res_mod : gr;
                rres[i] = *reinterpret_cast<const uint4*>(p.residual + (long long)rr * p.ldr + c0 + (lane & 3) * 8);
              } else {
                rres[i] = make_uint4(0u, 0u, 0u, 0u);
              }
            }
          }
          uint32_t acc[32];
          tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(as * BN + c * 32), acc);
          tmem_ld_wait();
          float v[32];
  #pragma unroll
          for (int j = 0; j < 32; ++j) {
            if constexpr (KIND == kKindI8) v[j] = static_cast<float>(static_cast<int>(acc[j])) * a_scale;
            else v[j] = __uint_as_float(acc[j]) * a_scale;
          }
          if (staged) {
            if (p.col_scale != nullptr) {
              const float4* c4p = reinterpret_cast<const float4*>(cs_s + as * BN + c * 32);
  #pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 c4 = c4p[q];
                v[q * 4] *= c4.x; v[q * 4 + 1] *= c4.y; v[q * 4 + 2] *= c4.z; v[q * 4 + 3] *= c4.w;
              }
            }
            if (p.bias != nullptr) {
              const float4* b4p = reinterpret_cast<const float4*>(bias_s + as * BN + c * 32);
  #pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 b4 = b4p[q];
                v[q * 4] += b4.x; v[q * 4 + 1] += b4.y; v[q * 4 + 2] += b4.z; v[q * 4 + 3] += b4.w;
              }
            }
            // activation: the switch sits outside the element loop so that the 32 independent
            // evaluations interleave
            // Mish into an e4m3 output runs on packed f16 pairs at the conversion below
            const bool mish8 = p.act == kActMish && p.out_dtype == kOutE4M3 && p.residual == nullptr && p.precise_act == 0;
            if (mish8) {
            } else if (p.act == kActMish) {
  #pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = act_mish(v[j]);
            } else if (p.act == kActGelu) {
  #pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = act_gelu(v[j]);
            } else if (p.act == kActRelu) {
  #pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
            }
            if (p.out_dtype == kOutE4M3 && !mish8) {
  #pragma unroll
              for (int j = 0; j < 32; ++j) v[j] *= p.out_scale;
            }
            if (p.residual != nullptr) {
              // transpose the coalesced residual rows through the staging tile into row-per-thread order
              if (lane == 0) bulk_wait_read0();   // the previous chunk's TMA store has read the tile
              __syncwarp();
  #pragma unroll
              for (int i = 0; i < 4; ++i)
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage_off((lane >> 2) + 8 * i, lane & 3)),
                             "r"(rres[i].x), "r"(rres[i].y), "r"(rres[i].z), "r"(rres[i].w) : "memory");
              __syncwarp();
  #pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 u;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "r"(stage_off(lane, q)));
                const __half2* h = reinterpret_cast<const __half2*>(&u);
  #pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 f = __half22float2(h[j]);
                  v[q * 8 + 2 * j] += f.x;
                  v[q * 8 + 2 * j + 1] += f.y;
                }
              }
              __syncwarp();
            } else {
              if (lane == 0) bulk_wait_read0();
              __syncwarp();
            }
            // row-per-thread results -> swizzled staging tile (the layout a TMA box with the 64-byte,
            // for e4m3 32-byte, swizzle expects) -> one TMA store per warp and chunk; rows and columns
            // beyond the matrix are clipped by the TMA unit
            if (p.out_dtype == kOutF16) {
  #pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint32_t w0 = pack_f16x2(v[q * 8 + 0], v[q * 8 + 1]), w1 = pack_f16x2(v[q * 8 + 2], v[q * 8 + 3]);
                const uint32_t w2 = pack_f16x2(v[q * 8 + 4], v[q * 8 + 5]), w3 = pack_f16x2(v[q * 8 + 6], v[q * 8 + 7]);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage_off(lane, q)), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
              }
            } else if (mish8) {
              const __half2 s2 = __float2half2_rn(p.out_scale);
  #pragma unroll
              for (int q = 0; q < 2; ++q) {
                uint32_t w[4];
  #pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float* e = &v[q * 16 + j * 4];
                  const uint32_t y0 = mish_f16x2(pack_f16x2(e[0], e[1])), y1 = mish_f16x2(pack_f16x2(e[2], e[3]));
                  const __half2 z0 = __hmul2(*reinterpret_cast<const __half2*>(&y0), s2);
                  const __half2 z1 = __hmul2(*reinterpret_cast<const __half2*>(&y1), s2);
                  w[j] = uint32_t(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<const __half2_raw*>(&z0), __NV_SATFINITE, __NV_E4M3)) |
                         (uint32_t(__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<const __half2_raw*>(&z1), __NV_SATFINITE, __NV_E4M3)) << 16);
                }
                const uint32_t off8 = stage_u + lane * 32 + ((q ^ ((lane >> 2) & 1)) << 4);   // 32-byte swizzle
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(off8), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
              }
            } else {
  #pragma unroll
              for (int q = 0; q < 2; ++q) {
                uint32_t w[4];
  #pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float* e = &v[q * 16 + j * 4];
                  w[j] = uint32_t(__nv_cvt_float2_to_fp8x2(make_float2(e[0], e[1]), __NV_SATFINITE, __NV_E4M3)) |
                         (uint32_t(__nv_cvt_float2_to_fp8x2(make_float2(e[2], e[3]), __NV_SATFINITE, __NV_E4M3)) << 16);
                }
                const uint32_t off8 = stage_u + lane * 32 + ((q ^ ((lane >> 2) & 1)) << 4);   // 32-byte swizzle
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(off8), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
              }
            }
            fence_proxy_async_smem();   // every writing lane, before the barrier (the documented order)
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmC, stage_u, c0, m0 + quarter * 32);
              bulk_commit();
            }
          } else if (c0 + 32 <= p.N && vec_ok) {
            // direct path (f32 output, per-column scales): each thread stores its own row segment
            if (p.col_scale != nullptr) {
  #pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.col_scale + c0) + q);
                v[q * 4] *= s4.x; v[q * 4 + 1] *= s4.y; v[q * 4 + 2] *= s4.z; v[q * 4 + 3] *= s4.w;
              }
            }
            if (p.bias != nullptr) {
              const float4* b4p = reinterpret_cast<const float4*>(bias_s + as * BN + c * 32);
  #pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 b4 = b4p[q];
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
                if (p.bias != nullptr) x += bias_s[as * BN + c * 32 + j];
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
        if (lane == 0) {
          mbar_arrive(tempty_bar(as));
        }
      }
      if (lane == 0) bulk_wait_all();   // this warp's TMA stores have left shared memory and landed
      __syncwarp();
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync();      // neither CTA leaves while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<PAIR>(tmem_base, Cfg::ACC_COLS);
  }
}

}  // namespace crl
