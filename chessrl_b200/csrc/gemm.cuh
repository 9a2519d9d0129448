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
//                 its rank modulo 4 selects; four warps share a lane quarter and split the columns;
//                 the epilogue is latency-bound, so it wants many warps in flight),
//                 then scale / bias / activation / residual, convert, store through a swizzled staging tile
//                 and one TMA store per 32 x 32 chunk; in the RES variant the residual chunk arrives by TMA,
//                 requested a chunk ahead
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
  int use_tma_store;       // host built a tensor map for C (f16 / e4m3 output, 16-byte aligned pitch)
  int use_tma_res;         // host built a tensor map for the residual (res_mod == 0, 16-byte aligned pitch)
};

constexpr int kGemmThreads = 576;   // TMA warp + MMA warp + 16 epilogue warps

// Optional cycle probes of the epilogue (compile with -DCRL_EPI_PROBE; the status buffer must then hold 64
// ints): lane 0 of every epilogue warp adds its clock64 deltas per phase to status[8..19].
#ifdef CRL_EPI_PROBE
#define EPI_PROBE_DECL long long pr_t = 0, pr_acc[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}
#define EPI_PROBE_START() pr_t = clock64()
#define EPI_PROBE(i) do { const long long n_ = clock64(); pr_acc[i] += n_ - pr_t; pr_t = n_; } while (0)
#define EPI_PROBE_COUNT(i) pr_acc[i] += 1
#define EPI_PROBE_FLUSH() do { if (lane == 0) for (int i_ = 0; i_ < 12; ++i_) atomicAdd(p.status + 8 + i_, static_cast<int>(pr_acc[i_] >> (i_ == 0 || i_ == 8 ? 0 : 4))); } while (0)
#else
#define EPI_PROBE_DECL
#define EPI_PROBE_START()
#define EPI_PROBE(i)
#define EPI_PROBE_COUNT(i)
#define EPI_PROBE_FLUSH()
#endif
constexpr int kEpiWarps = 16;

// PAIR = 1: two CTAs of a cluster work on one 256 x BN tile with cta_group::2 MMAs. Each CTA stages
// its own 128 rows of A and its own BN/2 rows of W, so a pair moves a third less data from L2 into
// shared memory per FLOP than two independent CTAs; the leader CTA (cluster rank 0) issues the MMAs
// for both, each CTA drains the 128 accumulator rows that land in its own tensor memory.
// RES = 1 (pairs only): residual rows arrive by TMA into a per-warp tile; that variant trades one ring stage for
// the tiles, the others keep five stages and carry none of its code.
template <int BN, int KIND, int PAIR = 0, int RES = 0>
struct GemmCfg {
  static constexpr int BM = 128;           // rows per CTA
  static constexpr int TM = PAIR ? 256 : 128;  // rows per tile
  static constexpr int ESZ = (KIND == kKindF16) ? 2 : 1;
  static constexpr int BK = 128 / ESZ;   // elements per stage along K: one 128-byte swizzle row
  static constexpr int UK = 32 / ESZ;    // elements per tcgen05.mma along K
  static constexpr uint32_t A_BYTES = BM * 128;
  static constexpr uint32_t B_BYTES = (PAIR ? BN / 2 : BN) * 128;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  // the residual variant fits five stages only without the per-column scale table (int8 keeps it and four stages)
  static constexpr int STAGES = PAIR ? ((RES && KIND == kKindI8) ? 4 : 5) : ((BN == 256) ? 3 : (BN == 128 ? 5 : 6));
  static constexpr uint32_t TAB_BYTES = ((RES && KIND != kKindI8) ? 2 : 4) * BN * 4;   // bias [2][BN] (+ column scales [2][BN])
  static constexpr int ACC_COLS = 2 * BN;  // two accumulator buffers; 128, 256 or 512 columns
  // after the stages: the bias and column-scale tables [2][2][BN] f32, one 32-row x 64-byte staging tile per epilogue
  // warp (512-byte aligned: the TMA store swizzles by absolute address bits), one tile of the same shape per
  // warp for residual rows arriving by TMA, then the mbarriers (ring, accumulators, one per epilogue warp for
  // its residual tile) + TMEM slot
  static constexpr uint32_t EPI_OFF = STAGES * STAGE_BYTES;
  static constexpr uint32_t RES_OFF = EPI_OFF + TAB_BYTES + kEpiWarps * 2048;
  static constexpr uint32_t BAR_OFF = RES_OFF + (RES ? kEpiWarps * 2048 : 0);
  static constexpr uint32_t USED_BYTES = BAR_OFF + 128 + kEpiWarps * 8;
  static constexpr size_t SMEM_BYTES = size_t(USED_BYTES) + (RES ? 768 : 896) /*alignment slack*/;
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

template <int BN, int KIND, int PAIR, int RES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmR, const GemmParams p) {
  using Cfg = GemmCfg<BN, KIND, PAIR, RES>;
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
      reinterpret_cast<uint32_t*>(smem + Cfg::BAR_OFF + 8 * (2 * STAGES + 4));

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

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int w = 0; w < kEpiWarps; ++w) mbar_init(bar0 + 128u + 8u * w, 1);
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), kEpiWarps * (PAIR ? 2 : 1));   // one arrival per epilogue warp (of both CTAs)
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc<PAIR>(smem_u32(tmem_slot), Cfg::ACC_COLS);
    tmem_relinquish<PAIR>();
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
      for (int t = worker; t < num_tiles && ok; t += num_workers) {
        const int m0 = (t / tiles_n) * TM + rank * BM;                  // this CTA's rows of A
        const int n0 = (t % tiles_n) * BN + rank * (PAIR ? BN / 2 : 0);  // this CTA's rows of W
        for (int kb = 0; kb < kblocks; ++kb) {
#ifdef CRL_EPI_PROBE
          const long long pw0 = clock64();
#endif
          if (!mbar_wait(empty_bar(s), ph ^ 1u)) {
            atomicCAS(p.status, 0, kDevTimeoutProducer);
            ok = false;
            break;
          }
#ifdef CRL_EPI_PROBE
          atomicAdd(p.status + 26 + rank, static_cast<int>((clock64() - pw0) >> 4));
#endif
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
#ifdef CRL_EPI_PROBE
      long long mt = clock64(), m_acc[4] = {0, 0, 0, 0};
#define MMA_PROBE(i) do { const long long n_ = clock64(); m_acc[i] += n_ - mt; mt = n_; } while (0)
#else
#define MMA_PROBE(i)
#endif
      for (int t = worker; t < num_tiles && ok; t += num_workers, ++local) {
        const int as = local & 1;
        const uint32_t aph = (local >> 1) & 1u;
        MMA_PROBE(3);
        if (!mbar_wait(tempty_bar(as), aph ^ 1u)) {
          atomicCAS(p.status, 0, kDevTimeoutMma);
          break;
        }
        MMA_PROBE(0);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full_bar(s), ph)) {
            atomicCAS(p.status, 0, kDevTimeoutMma);
            ok = false;
            break;
          }
          MMA_PROBE(1);
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
          MMA_PROBE(2);
        }
        if (ok) tc_commit<PAIR>(tfull_bar(as));   // accumulator complete
      }
#ifdef CRL_EPI_PROBE
      for (int i = 0; i < 4; ++i) atomicAdd(p.status + 20 + i, static_cast<int>(m_acc[i] >> 4));
      atomicAdd(p.status + 24, local);
#endif
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int ew = warp - 2;                // 0..15
    const int quarter = warp & 3;           // TMEM lanes [32*quarter, 32*quarter+32)
    const int part = ew >> 2;               // this warp takes the 32-column chunks part, part+4, ...
    const int et = threadIdx.x - 64;        // 0..511 among the epilogue threads
    float* bias_s = reinterpret_cast<float*>(smem + Cfg::EPI_OFF);                  // [2][BN]
    float* cs_s = bias_s + 2 * BN;                                                  // [2][BN] per-column scales
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
    // Residual rows by TMA: a warp's 32 x 32 f16 tile of the residual lands in its own shared-memory tile (the
    // store box's shape and swizzle), requested one chunk ahead - the next chunk's as soon as this one's has been
    // read, the next tile's first chunk before the wait for that tile's accumulator - so the HBM latency of the
    // residual never sits between the accumulator and the store.
    const bool tma_res = RES != 0 && p.use_tma_res != 0 && staged_ok && p.residual != nullptr && p.res_mod == 0 && p.N % 32 == 0;
    const uint32_t res_u = base + Cfg::RES_OFF + ew * 2048;
    const uint32_t rbar = bar0 + 128u + 8u * ew;
    uint32_t rph = 0;
    bool res_pending = false;
    auto res_issue = [&](int tile, int c) {
      if (lane == 0) {
        mbar_expect_tx(rbar, 2048u);
        tma_load_2d(res_u, &tmR, (tile % tiles_n) * BN + c * 32, (tile / tiles_n) * TM + rank * BM + quarter * 32, rbar);
      }
      res_pending = true;
    };
    if (RES != 0 && tma_res && part < BN / 32 && worker < num_tiles && (worker % tiles_n) * BN + part * 32 < p.N) res_issue(worker, part);
    bool alive = true;
    int local = 0;
    EPI_PROBE_DECL;
    for (int t = worker; t < num_tiles; t += num_workers, ++local) {
      EPI_PROBE_START();
      EPI_PROBE_COUNT(8);
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
      EPI_PROBE(9);
      if (alive && !mbar_wait(tfull_bar(as), aph)) {
        if (lane == 0) atomicCAS(p.status, 0, kDevTimeoutEpilogue);
        alive = false;           // keep iterating so that the named barrier above stays balanced
      }
      if (!alive) continue;
      tc_fence_after();
      EPI_PROBE(7);
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
        if (staged && p.residual != nullptr && !tma_res) {
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
        EPI_PROBE_COUNT(0);
        EPI_PROBE(1);
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
          const bool mish8 = p.act == kActMish && p.out_dtype == kOutE4M3 && p.residual == nullptr;
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
          EPI_PROBE(2);
          if (RES != 0 && tma_res) {
            if (!mbar_wait(rbar, rph)) {
              if (lane == 0) atomicCAS(p.status, 0, kDevTimeoutEpilogue);
              alive = false;
              break;
            }
            rph ^= 1u;
            res_pending = false;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u;
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
                           : "r"(res_u + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)));
              const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                v[q * 8 + 2 * j] += f.x;
                v[q * 8 + 2 * j + 1] += f.y;
              }
            }
            __syncwarp();   // every lane has read its row: the tile may be refilled
            {
              // this warp's next chunk: further along this tile, else the first chunk of its next tile
              int nt = t, nc = c + 4;
              if (nc >= BN / 32 || n0 + nc * 32 >= p.N) { nt = t + num_workers; nc = part; }
              if (nt < num_tiles && nc < BN / 32 && (nt % tiles_n) * BN + nc * 32 < p.N) res_issue(nt, nc);
            }
            if (lane == 0) bulk_wait_read0();   // the previous chunk's TMA store has read the staging tile
            __syncwarp();
          } else if (p.residual != nullptr) {
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
          EPI_PROBE(3);
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
          EPI_PROBE(4);
          fence_proxy_async_smem();   // every writing lane, before the barrier (the documented order)
          __syncwarp();
          EPI_PROBE(5);
          if (lane == 0) {
            tma_store_2d(&tmC, stage_u, c0, m0 + quarter * 32);
            bulk_commit();
          }
          EPI_PROBE(6);
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
        if (PAIR && rank != 0) mbar_arrive_cluster(mapa_u32(tempty_bar(as), 0));   // the leader's barrier
        else mbar_arrive(tempty_bar(as));
      }
      EPI_PROBE(10);
    }
    EPI_PROBE_FLUSH();
    if (RES != 0 && res_pending) mbar_wait(rbar, rph);   // only after a timeout: no copy into this CTA's memory stays in flight
    if (lane == 0) bulk_wait_all();   // this warp's TMA stores have left shared memory and landed
    __syncwarp();
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
