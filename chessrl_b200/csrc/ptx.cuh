// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM
// allocation, MMA, commit, load) and the descriptors tcgen05.mma consumes.
//
// Every wait in this file is bounded: a wait that runs out returns false, the caller records a
// status code and leaves its loop, so a protocol bug ends the kernel instead of hanging the GPU.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace crl {

// ---------------------------------------------------------------------------------------------
// status codes written by kernels into the handle's device status word (0 = fine)
// ---------------------------------------------------------------------------------------------
enum DeviceStatus : int {
  kDevOk = 0,
  kDevTimeoutProducer = 101,   // TMA producer never saw a free stage
  kDevTimeoutMma = 102,        // MMA issuer never saw a filled stage / free accumulator
  kDevTimeoutEpilogue = 103,   // epilogue never saw a finished accumulator
  kDevBadSmemAlign = 104,      // dynamic shared memory base less aligned than the layout allows for
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  // The last operand is the suspend-time hint: the thread may sleep inside the instruction until the phase
  // completes (it is woken then) or the hint runs out, instead of returning at once and spinning through issue
  // slots the working warps of the SM need.
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(0x989680u)
      : "memory");
  return ok;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: every try may sleep inside the instruction; the wall-clock bound (two seconds on the GPU's
// nanosecond timer) is what ends a wait that can never succeed, however long or short the hardware lets a
// single try sleep. Returns false when it gives up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (;;) {
    // the clock is looked at once per 256 tries only: the loop around a failed try stays three instructions
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > 2000000000ull) return false;
  }
}

// ---------------------------------------------------------------------------------------------
// 2-CTA clusters
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// cluster-window address of this CTA's shared-memory address `addr` in the CTA of rank `rank`
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on an mbarrier of another CTA of the cluster. Relaxed: the barrier only hands a tensor-memory
// buffer back (ordered by tcgen05.fence::before_thread_sync), no generic-memory data travels with it; a
// cluster-scope release here was measured at ~2000 cycles per arrival.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// ---------------------------------------------------------------------------------------------
// TMA: 2-D tiled load global -> shared (this CTA only), completion on an mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// Same load into this CTA's shared memory, but the bytes are counted on an mbarrier given by its
// cluster-window address (the leader CTA's barrier when a CTA pair feeds one cta_group::2 MMA).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tm, int x, int y,
                                                 uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(cluster_bar)
      : "memory");
}

// 2-D tiled store shared -> global (bulk async-group completion). Elements outside the tensor are
// not written. Generic-proxy writes to the source tile need fence_proxy_async_smem() + a barrier first.
// Hint: bring the box at (x, y) into L2 (no shared-memory destination, nothing to wait for).
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* tm, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                   reinterpret_cast<uint64_t>(tm)),
               "r"(x), "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all earlier bulk groups of this thread have finished READING their shared-memory source
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... have completed entirely
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// tcgen05: tensor memory + MMA
// ---------------------------------------------------------------------------------------------
// PAIR = 1 variants act on both CTAs of a 2-CTA cluster (cta_group::2): the same warp of each CTA
// executes them with the same operands.
template <int PAIR = 0>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  if constexpr (PAIR)
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
template <int PAIR = 0>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (PAIR) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  else asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <int PAIR = 0>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// The mbarrier gets one arrival once every MMA issued so far by this thread has finished.
// PAIR = 1: issued by the leader CTA; the barrier at the same shared-memory offset in both CTAs of the pair
// gets its arrival from one commit (CTA mask 0b11). This is the commit's own multicast form - a signal, not a
// data copy; two separate commits to the two cluster-window addresses measured 2-5 % slower per GEMM.
template <int PAIR = 0>
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  if constexpr (PAIR) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"(static_cast<uint16_t>(3))
                 : "memory");
  } else {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  }
}

// Shared-memory matrix descriptor for a K-major tile stored with the 128-byte swizzle (the layout
// a TMA box of 128 bytes x rows with CU_TENSOR_MAP_SWIZZLE_128B produces): rows are 128 bytes
// apart, groups of 8 rows are 1024 bytes apart (the "stride byte offset").
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);        // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                           // leading byte offset (unused)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                   // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                           // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                           // layout type: 128-byte swizzle
  return d;
}

// Instruction descriptor: D fp32 (or s32), A and B K-major, M x N tile.
//   fmt_ab: kind::f16 -> 0 = f16, 1 = bf16; kind::f8f6f4 -> 0 = e4m3; kind::i8 -> 1 = signed
//   c_fmt : 1 = f32, 2 = s32
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, int fmt_ab, int c_fmt) {
  return (static_cast<uint32_t>(c_fmt) << 4) | (static_cast<uint32_t>(fmt_ab) << 7) |
         (static_cast<uint32_t>(fmt_ab) << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

enum MmaKind : int { kKindF16 = 0, kKindF8 = 1, kKindI8 = 2 };

#define CRL_UMMA_ASM(GROUP, KINDSTR)                                                              \
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"                                   \
               "tcgen05.mma.cta_group::" GROUP ".kind::" KINDSTR " [%0], %1, %2, %3, p;\n\t}\n" ::"r"( \
                   tmem_d),                                                                       \
               "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)                              \
               : "memory")

// D[tmem] (+)= A[smem] * B[smem]^T. PAIR = 1: one instruction drives the tensor cores of both CTAs
// (M = 256: rows 0..127 accumulate in the leader's tensor memory, 128..255 in the peer's).
template <int KIND, int PAIR = 0>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                     uint32_t idesc, uint32_t accumulate) {
  if constexpr (KIND == kKindF16) {
    if constexpr (PAIR) CRL_UMMA_ASM("2", "f16"); else CRL_UMMA_ASM("1", "f16");
  } else if constexpr (KIND == kKindF8) {
    if constexpr (PAIR) CRL_UMMA_ASM("2", "f8f6f4"); else CRL_UMMA_ASM("1", "f8f6f4");
  } else {
    if constexpr (PAIR) CRL_UMMA_ASM("2", "i8"); else CRL_UMMA_ASM("1", "i8");
  }
}
#undef CRL_UMMA_ASM

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives row (lane base + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// activations shared by the GEMM epilogue and the row kernels
// ---------------------------------------------------------------------------------------------
enum Act : int { kActNone = 0, kActGelu = 1, kActMish = 2, kActRelu = 3 };

// Mish on two packed f16 values, for outputs that are rounded to e4m3 anyway: one MUFU op (ex2.approx.f16x2)
// per pair instead of four, the reciprocal by two Newton steps from an exponent-flip seed. With u = e^x:
// mish(x) = x * n / (n + 2), n = u (u + 2); x is clamped to 5 inside the exponential so that n stays below the
// f16 range (the gate is 1 - 9e-5 there). Relative error <= 4.2e-3 over [-12, 12] (e4m3 steps are 6e-2).
__device__ __forceinline__ uint32_t mish_f16x2(uint32_t xu) {
  const __half2 x = *reinterpret_cast<const __half2*>(&xu);
  const __half2 two = __float2half2_rn(2.0f);
  const __half2 l = __hmul2(__hmin2(x, __float2half2_rn(5.0f)), __float2half2_rn(1.4426950408889634f));
  uint32_t tu;
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(tu) : "r"(*reinterpret_cast<const uint32_t*>(&l)));
  const __half2 t = *reinterpret_cast<const __half2*>(&tu);
  const __half2 n = __hmul2(t, __hadd2(t, two));
  const __half2 d = __hadd2(n, two);
  const __half2 nd = __hneg2(d);
  const uint32_t ru = 0x77fc77fcu - *reinterpret_cast<const uint32_t*>(&d);   // ~1/d within 12 %, both halves at once
  __half2 r = *reinterpret_cast<const __half2*>(&ru);
  r = __hmul2(r, __hfma2(nd, r, two));
  r = __hmul2(r, __hfma2(nd, r, two));
  const __half2 y = __hmul2(x, __hmul2(n, r));
  return *reinterpret_cast<const uint32_t*>(&y);
}

__device__ __forceinline__ float act_gelu(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
}
__device__ __forceinline__ float act_mish(float x) {
  // x * tanh(softplus(x)) with tanh(log(1+e)) = ((1+e)^2 - 1) / ((1+e)^2 + 1) = n / (n + 2),
  // n = e * (e + 2), e = exp(x): one ex2 and one rcp on the special-function unit, no branches.
  // The exponent is clamped at 15, where n / (n + 2) already rounds to 1 in fp32.
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(fminf(x, 15.0f) * 1.4426950408889634f));
  const float n = fmaf(e, e, 2.0f * e);
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(n + 2.0f));
  return x * n * r;
}
__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case kActGelu: return act_gelu(x);
    case kActMish: return act_mish(x);
    case kActRelu: return fmaxf(x, 0.0f);
    default: return x;
  }
}

}  // namespace crl
