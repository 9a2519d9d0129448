// Host side of the tcgen05 GEMM: tensor-map encoding (driver entry point fetched at run time, so the
// library links against the CUDA runtime only) and tile-shape selection.
#pragma once
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include "gemm.cuh"

namespace crl {

enum HostErr : int {
  kOk = 0,
  kErrInvalid = -1,      // bad argument (null pointer, negative size, unknown enum)
  kErrShape = -2,        // shape or alignment the kernels cannot take
  kErrCuda = -3,         // a CUDA runtime / driver call failed
  kErrMissingWeight = -4,
  kErrNotFinalized = -5,
  kErrDeviceTimeout = -6,  // a bounded device-side wait ran out (status word holds the code)
  kErrWorkspace = -7,
  kErrUnsupported = -8,
};

inline PFN_cuTensorMapEncodeTiled_v12000 tmap_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

// 2-D row-major tensor [outer, inner] with a row pitch in bytes; box = 128 bytes x box_outer rows,
// 128-byte swizzle, out-of-range elements read as zero.
// box_bytes is the box's inner extent and selects the swizzle: 128 (operand tiles), 64 or 32 (the
// epilogue's staging tiles).
inline int make_tmap_2d(CUtensorMap* out, const void* ptr, int esz, uint64_t inner, uint64_t outer,
                        uint64_t pitch_bytes, uint32_t box_outer, uint32_t box_bytes = 128) {
  auto enc = tmap_encoder();
  if (enc == nullptr) return kErrCuda;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (pitch_bytes & 15) != 0) return kErrShape;
  cuuint64_t gdim[2] = {inner, outer};
  cuuint64_t gstride[1] = {pitch_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes / esz), box_outer};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : (box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
  CUresult r = enc(out, esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                   const_cast<void*>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kOk : kErrCuda;
}

struct GemmArgs {
  int kind = kKindF16;          // MmaKind: element type of A and W
  const void* A = nullptr;      // [M, lda]
  long long lda = 0;            // elements
  const void* W = nullptr;      // [N, ldw]
  long long ldw = 0;
  GemmParams p{};
};

// box shape of the epilogue's stores (and of the residual slab): pairs 64 columns x 32 rows, single CTAs 32 x 32
inline bool out_map_ok(const GemmParams& p) {
  if (p.out_dtype == kOutF32) return false;
  const int oesz = p.out_dtype == kOutF16 ? 2 : 1;
  // a slab that sticks out of the matrix is clipped by the TMA unit in whole 16-byte pieces: the row length in
  // bytes has to be a multiple of 16 for the clipping to be exact
  return (reinterpret_cast<uintptr_t>(p.C) & 15) == 0 && (static_cast<uint64_t>(p.ldc) * oesz) % 16 == 0 &&
         (static_cast<uint64_t>(p.N) * oesz) % 16 == 0;
}

// The fused-LayerNorm GEMM gives every CTA pair whole blocks of 256 rows; it pays when each pair has several.
inline bool gemm_can_fuse_ln(long long M, int N, int K, int num_sms) {
  return N >= 256 && K <= 1024 && K % 8 == 0 && (M + 255) / 256 >= 2ll * (num_sms / 2);
}

// The GEMM that also normalises its output rows (LNO kernels): the CTAs holding the column tiles of a row block
// exchange row sums, so every CTA pair has to be resident at once and busy: N a multiple of 256 up to 1024, at least
// one tile per pair.
inline bool gemm_can_fuse_ln_out(long long M, int N, int num_sms) {
  return N % 256 == 0 && N <= 1024 && ((M + 255) / 256) * (N / 256) >= num_sms / 2;
}
// bytes of the exchange buffer: one 8-byte record per row (rounded up to whole 256-row blocks) and 128-column slab for
// the sums, and as many again for the row maxima of the int8 copy
inline size_t gemm_ln_out_scratch_bytes(long long M) { return static_cast<size_t>((M + 255) / 256) * 2 * 8 * 256 * 8; }

template <int BN, int KIND, int PAIR = 0, int RES = 0, int O8 = 0, int LNA = 0, int LNO = 0, int EPI = 0>
inline int gemm_launch_t(const GemmArgs& a, int num_sms, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, KIND, PAIR, RES, O8, LNA, LNO>;
  static bool attr_set[64] = {};  // per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_tn_kernel<BN, KIND, PAIR, RES, O8, LNA, LNO, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(Cfg::SMEM_BYTES)) != cudaSuccess)
      return kErrCuda;
    attr_set[dev] = true;
  }
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, a.A, Cfg::ESZ, a.p.K, a.p.M, a.lda * Cfg::ESZ, Cfg::BM);
  if (rc != kOk) return rc;
  rc = make_tmap_2d(&tmB, a.W, Cfg::ESZ, a.p.K, a.p.N, a.ldw * Cfg::ESZ, PAIR ? BN / 2 : BN);
  if (rc != kOk) return rc;
  // output tensor map for the epilogue's TMA stores
  CUtensorMap tmC;
  GemmParams prm = a.p;
  prm.use_tma_store = 0;
  std::memset(&tmC, 0, sizeof(tmC));
  constexpr int kBoxCols = PAIR ? 64 : 32;
  if (prm.out_dtype != kOutF32) {
    const int oesz = prm.out_dtype == kOutF16 ? 2 : 1;
    if (make_tmap_2d(&tmC, prm.C, oesz, prm.N, prm.M, static_cast<uint64_t>(prm.ldc) * oesz, 32, kBoxCols * oesz) == kOk)
      prm.use_tma_store = 1;
  }
  if (PAIR && !prm.use_tma_store) return kErrShape;   // the slab epilogue has no other way out
  if (PAIR && (O8 != 0) != (prm.out_dtype == kOutE4M3)) return kErrInvalid;
  // the residual slab arrives through the same box shape when the buffer allows a tensor map
  CUtensorMap tmR;
  std::memset(&tmR, 0, sizeof(tmR));
  prm.use_tma_res = 0;
  if (RES != 0 && prm.residual != nullptr && prm.res_mod == 0 &&
      make_tmap_2d(&tmR, prm.residual, 2, prm.N, prm.M, static_cast<uint64_t>(prm.ldr) * 2, 32, 128) == kOk)
    prm.use_tma_res = 1;
  const int tiles = ((a.p.M + Cfg::TM - 1) / Cfg::TM) * ((a.p.N + BN - 1) / BN);
  // LNO: the e4m3 copy of the normalised rows leaves through a tensor map of its own (32 rows x 128 columns)
  CUtensorMap tmX8;
  std::memset(&tmX8, 0, sizeof(tmX8));
  if constexpr (LNO != 0) {
    if (!prm.use_tma_res || prm.lno_stats == nullptr || prm.lno_w16 == nullptr || prm.lno_b16 == nullptr) return kErrInvalid;
    if (prm.lno_x8 != nullptr &&
        make_tmap_2d(&tmX8, prm.lno_x8, 1, prm.N, prm.M, static_cast<uint64_t>(prm.N), 32, 128) != kOk)
      return kErrShape;
  }
  if constexpr (PAIR) {
    // one 2-CTA cluster per pair of SMs (LNA: a pair owns whole row blocks, so no more pairs than row blocks)
    const int units = LNA ? (a.p.M + Cfg::TM - 1) / Cfg::TM : tiles;
    int pairs = units < num_sms / 2 ? units : num_sms / 2;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
    cfg.blockDim = dim3(Cfg::THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if constexpr (LNO != 0) {
      // CTAs of this kernel wait for one another: launch no more pairs than the device holds at once
      static int resident[64] = {};
      if (dev < 0 || dev >= 64) return kErrInvalid;
      if (resident[dev] == 0) {
        int n = 0;
        cfg.gridDim = dim3(static_cast<unsigned>(2 * (num_sms / 2)));
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tn_kernel<BN, KIND, PAIR, RES, O8, LNA, LNO, EPI>, &cfg) != cudaSuccess || n <= 0)
          return kErrCuda;
        resident[dev] = n;
        if (std::getenv("CRL_DEBUG") != nullptr) std::fprintf(stderr, "chessrl_b200: %d CTA pairs resident at once on device %d\n", n, dev);
      }
      if (pairs > resident[dev]) pairs = resident[dev];
      cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
      // every record of the exchange buffer starts as the "not written yet" pattern
      const size_t recs = gemm_ln_out_scratch_bytes(a.p.M) / sizeof(unsigned long long);
      if (cudaMemsetAsync(prm.lno_stats, 0xFF, recs * sizeof(unsigned long long), stream) != cudaSuccess) return kErrCuda;
    }
    return cudaLaunchKernelEx(&cfg, gemm_tn_kernel<BN, KIND, PAIR, RES, O8, LNA, LNO, EPI>, tmA, tmB, tmC, tmR, tmX8, prm) == cudaSuccess ? kOk : kErrCuda;
  } else {
    const int grid = tiles < num_sms ? tiles : num_sms;
    gemm_tn_kernel<BN, KIND, 0, 0, 0, 0><<<grid, kGemmThreads, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, tmC, tmR, tmX8, prm);
    return cudaGetLastError() == cudaSuccess ? kOk : kErrCuda;
  }
}

template <int KIND>
inline int gemm_launch_k(const GemmArgs& a, int num_sms, cudaStream_t stream) {
  const int tiles_m = (a.p.M + 127) / 128;
  int bn = 256;
  if (a.p.N <= 64) bn = 64;
  else if (a.p.N <= 128) bn = 128;
  else if (tiles_m * ((a.p.N + 255) / 256) < num_sms) bn = 128;  // small batch: more, smaller tiles
  if (a.p.ln_y != nullptr) {
    // A = LayerNorm(ln_y), normalised inside the kernel (f16 / e4m3 operands, no TMA-fetched residual)
    if (KIND == kKindI8 || !gemm_can_fuse_ln(a.p.M, a.p.N, a.p.K, num_sms) || !out_map_ok(a.p) || a.p.col_scale != nullptr ||
        a.p.ln_w16 == nullptr || a.p.ln_b16 == nullptr || (KIND == kKindF8 ? a.p.ln_x8 == nullptr : a.p.ln_x == nullptr) ||
        a.p.ln_ldy % 8 != 0 || (reinterpret_cast<uintptr_t>(a.p.ln_y) & 15) != 0)
      return kErrUnsupported;
    if constexpr (KIND != kKindI8) {
      return a.p.out_dtype == kOutE4M3 ? gemm_launch_t<256, KIND, 1, 0, 1, 1>(a, num_sms, stream)
                                       : gemm_launch_t<256, KIND, 1, 0, 0, 1>(a, num_sms, stream);
    }
  }
  if (a.p.lno_stats != nullptr) {
    // output rows normalised inside the kernel: the residual kernel of CTA pairs. int8 operands may carry per-token
    // and per-channel scales and ask for a per-token int8 copy (lno_x8 with lno_qscale); f16 / e4m3 operands for an
    // e4m3 copy (lno_x8 alone)
    const bool res_tma = a.p.residual != nullptr && a.p.res_mod == 0 && a.p.ldr % 8 == 0 &&
                         (reinterpret_cast<uintptr_t>(a.p.residual) & 15) == 0;
    const bool scales_ok = KIND == kKindI8 ? ((reinterpret_cast<uintptr_t>(a.p.col_scale) & 15) == 0 &&
                                              (a.p.lno_qscale == nullptr || a.p.lno_x8 != nullptr))
                                           : (a.p.col_scale == nullptr && a.p.row_scale == nullptr && a.p.lno_qscale == nullptr);
    if (!gemm_can_fuse_ln_out(a.p.M, a.p.N, num_sms) || a.p.out_dtype != kOutF16 || !out_map_ok(a.p) || !res_tma || !scales_ok ||
        (KIND == kKindI8 && a.p.lno_x8 != nullptr && a.p.lno_qscale == nullptr) ||
        a.p.ln_y != nullptr || a.p.lno_w16 == nullptr || a.p.act != kActNone ||
        a.p.lno_b16 == nullptr || (reinterpret_cast<uintptr_t>(a.p.lno_w16) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.p.lno_x8) & 15) != 0 ||
        (reinterpret_cast<uintptr_t>(a.p.bias) & 15) != 0 ||
        (reinterpret_cast<uintptr_t>(a.p.lno_b16) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.p.lno_stats) & 7) != 0)
      return kErrUnsupported;
    static const bool generic_only = std::getenv("CRL_GEMM_GENERIC") != nullptr;
    if constexpr (KIND != kKindI8) {
      // the two forms the engines launch get their switches fixed at compile time
      if (generic_only) return gemm_launch_t<256, KIND, 1, 1, 0, 0, 1>(a, num_sms, stream);
      if (a.p.bias != nullptr && a.p.lno_x8 != nullptr) return gemm_launch_t<256, KIND, 1, 1, 0, 0, 1, 1>(a, num_sms, stream);
      if (a.p.bias != nullptr && a.p.lno_x8 == nullptr) return gemm_launch_t<256, KIND, 1, 1, 0, 0, 1, 2>(a, num_sms, stream);
    }
    return gemm_launch_t<256, KIND, 1, 1, 0, 0, 1>(a, num_sms, stream);
  }
  // large problems with a 16-bit or 8-bit output a tensor map can describe: CTA pairs on 256 x 256 tiles
  if (a.p.N >= 256 && ((a.p.M + 255) / 256) * ((a.p.N + 255) / 256) >= num_sms / 2 && out_map_ok(a.p) &&
      (a.p.col_scale == nullptr || KIND == kKindI8)) {
    // a residual that a tensor map can describe is fetched by TMA (out-projection, ff2)
    const bool res_tma = a.p.residual != nullptr && a.p.res_mod == 0 && a.p.ldr % 8 == 0 &&
                         (reinterpret_cast<uintptr_t>(a.p.residual) & 15) == 0;
    // The shapes the engines launch get epilogues with their switches fixed at compile time (EPI): bias or not,
    // no activation or Mish; int8 operands with both scale vectors, the others with neither.
    const bool scales = KIND == kKindI8 ? (a.p.row_scale != nullptr && a.p.col_scale != nullptr &&
                                           (reinterpret_cast<uintptr_t>(a.p.col_scale) & 15) == 0)
                                        : (a.p.row_scale == nullptr && a.p.col_scale == nullptr);
    const bool plain = scales && a.p.N % 64 == 0 && (reinterpret_cast<uintptr_t>(a.p.bias) & 15) == 0 &&
                       (a.p.residual == nullptr || res_tma);
    // (CRL_GEMM_GENERIC in the environment keeps every launch on the run-time switches: the reference the
    // specialised instantiations are tested against)
    static const bool generic_only = std::getenv("CRL_GEMM_GENERIC") != nullptr;
    int epi = 0;
    if (generic_only) epi = 0;
    else if (plain && a.p.act == kActNone) epi = a.p.bias != nullptr ? 1 : 2;
    else if (plain && a.p.act == kActMish && a.p.bias != nullptr && a.p.residual == nullptr &&
             (a.p.out_dtype != kOutE4M3 || a.p.precise_act == 0))
      epi = 3;
    if (a.p.out_dtype == kOutE4M3) {
      if (a.p.residual != nullptr) epi = 0;      // (no hot GEMM adds a residual into an e4m3 output)
      if constexpr (KIND != kKindI8) {
        if (epi == 1) return gemm_launch_t<256, KIND, 1, 0, 1, 0, 0, 1>(a, num_sms, stream);
        if (epi == 2) return gemm_launch_t<256, KIND, 1, 0, 1, 0, 0, 2>(a, num_sms, stream);
        if (epi == 3) return gemm_launch_t<256, KIND, 1, 0, 1, 0, 0, 3>(a, num_sms, stream);
      }
      return gemm_launch_t<256, KIND, 1, 0, 1>(a, num_sms, stream);
    }
    if (res_tma) {
      if (epi == 1) return gemm_launch_t<256, KIND, 1, 1, 0, 0, 0, 1>(a, num_sms, stream);
      return gemm_launch_t<256, KIND, 1, 1, 0>(a, num_sms, stream);
    }
    if (a.p.residual == nullptr) {
      if (epi == 1) return gemm_launch_t<256, KIND, 1, 0, 0, 0, 0, 1>(a, num_sms, stream);
      if (epi == 3) return gemm_launch_t<256, KIND, 1, 0, 0, 0, 0, 3>(a, num_sms, stream);
    }
    return gemm_launch_t<256, KIND, 1, 0, 0>(a, num_sms, stream);
  }
  if (bn == 64) return gemm_launch_t<64, KIND>(a, num_sms, stream);
  if (bn == 128) return gemm_launch_t<128, KIND>(a, num_sms, stream);
  return gemm_launch_t<256, KIND>(a, num_sms, stream);
}

inline int gemm_launch(const GemmArgs& a, int num_sms, cudaStream_t stream) {
  if (a.A == nullptr || a.W == nullptr || a.p.C == nullptr || a.p.status == nullptr) return kErrInvalid;
  if (a.p.M <= 0 || a.p.N <= 0 || a.p.K <= 0) return kErrInvalid;
  switch (a.kind) {
    case kKindF16: return gemm_launch_k<kKindF16>(a, num_sms, stream);
    case kKindF8: return gemm_launch_k<kKindF8>(a, num_sms, stream);
    case kKindI8: return gemm_launch_k<kKindI8>(a, num_sms, stream);
    default: return kErrInvalid;
  }
}

}  // namespace crl
