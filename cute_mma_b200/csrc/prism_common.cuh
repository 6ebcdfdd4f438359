// Shared device-side building blocks for the Prism sm_100a kernels:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (UMMA + TMEM) wrappers,
// shared-memory matrix descriptors and the 128-byte swizzle address map.
//
// Every wait in this file is bounded: a wait that does not complete within
// PRISM_WAIT_LIMIT_CYCLES gives up and returns false; the caller records an
// error code in global memory and runs on to its normal teardown, so a
// mis-programmed pipeline shows up as a status code instead of a hung GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/prism_b200.h"

// Suspend-time hint (ns) of mbarrier.try_wait: a waiting warp sleeps in hardware instead of
// polling, which leaves issue slots and power to the warps that work (measured: forward -3.6 %).
#ifndef PRISM_TRYWAIT_HINT
#define PRISM_TRYWAIT_HINT 20000
#endif
#ifndef PRISM_WAIT_LIMIT_CYCLES
#define PRISM_WAIT_LIMIT_CYCLES (2000000000ll)  // about one second of SM clocks
#endif

namespace prism {

// status codes (PRISM_OK, PRISM_ERR_*) come from the public header
enum : int { DT_F16 = 0, DT_BF16 = 1 };
enum : int { GATE_NONE = 0, GATE_SILU = 1, GATE_SIGMOID = 2 };   // plain, A*silu(S), A*2*sigmoid(S)

// ----------------------------------------------------------------------------
// small helpers
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "elect.sync _|P1, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// Byte offset of 16-byte chunk `chunk16` (0..7) of row `row` inside a tile whose
// rows are 128 bytes wide, stored with the 128-byte swizzle (what TMA
// SWIZZLE_128B writes and what a SWIZZLE_128B UMMA descriptor reads).
// The tile base must be 1024-byte aligned.
__device__ __host__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t chunk16) {
  return row * 128u + ((chunk16 ^ (row & 7u)) << 4);
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
#ifdef PRISM_TRYWAIT_HINT
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2, %3;\n\t"
#else
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
#endif
      "selp.b32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(ok)
#ifdef PRISM_TRYWAIT_HINT
      : "r"(smem_u32(bar)), "r"(parity), "r"((uint32_t)PRISM_TRYWAIT_HINT)
#else
      : "r"(smem_u32(bar)), "r"(parity)
#endif
      : "memory");
  return ok != 0;
}
// Bounded wait for the phase with the given parity to complete.
// Returns false if the limit ran out (the barrier state is then unknown).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (clock64() - t0 > PRISM_WAIT_LIMIT_CYCLES) return false;
  }
}

// Position in a ring of n buffers plus the mbarrier phase parity of the current pass.
// Advancing is an increment and a compare: the single-thread producer / MMA-issuer roles are
// latency-bound, and a runtime division per stage would cost more than the work they hand out.
struct Ring {
  uint32_t idx, phase, n;
  __device__ __forceinline__ explicit Ring(uint32_t n_) : idx(0), phase(0), n(n_) {}
  __device__ __forceinline__ void next() {
    if (++idx == n) { idx = 0; phase ^= 1u; }
  }
};

// Make generic-proxy writes to shared memory visible to the async proxy
// (TMA stores, tcgen05.mma operand reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ----------------------------------------------------------------------------
// TMA
// ----------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load: c0 = innermost (contiguous) coordinate, c1 = row coordinate.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0),
        "r"(c1)
      : "memory");
}
// The same with an L2 eviction-priority hint (a policy made by l2_policy_*): read-once streams
// are loaded evict-first so that they do not push reused data out of L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
        "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int c0,
                                             int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------
// tcgen05: TMEM allocation, MMA, commit, loads
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// TMEM -> registers: each thread of the warp reads its own lane (row), N consecutive
// 32-bit columns starting at taddr (lane field must be the warp's lane-quarter base).
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------
// Single-CTA tcgen05 (cta_group::1): M = 128 rows of the A operand, accumulator in this CTA's TMEM.
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc_cta(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_cta() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_cta(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_cta_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive (count 1) on this CTA's barrier once all MMAs issued so far by this thread are complete.
__device__ __forceinline__ void umma_commit_cta(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ----------------------------------------------------------------------------
// CTA pairs (cluster of 2, tcgen05 cta_group::2): one MMA instruction spans two SMs, each
// holding its own 128 rows of the A operand and half of the B operand's N extent.
// No load here uses cluster multicast; only tcgen05.commit does.
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t cta_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
#ifdef PRISM_TRYWAIT_HINT
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2, %3;\n\t"
#else
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
#endif
      "selp.b32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(ok)
#ifdef PRISM_TRYWAIT_HINT
      : "r"(smem_u32(bar)), "r"(parity), "r"((uint32_t)PRISM_TRYWAIT_HINT)
#else
      : "r"(smem_u32(bar)), "r"(parity)
#endif
      : "memory");
  return ok != 0;
}
// Bounded wait with cluster-scope acquire (the barrier is arrived on by the peer CTA as well).
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait_cluster(bar, parity)) return true;
    }
    if (clock64() - t0 > PRISM_WAIT_LIMIT_CYCLES) return false;
  }
}
// TMA load into this CTA's shared memory whose completion is signalled on a barrier that may
// live in the peer CTA (bar_cluster_addr is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Same with each descriptor given as (low word, high word).  The start address (>> 4) sits in bits
// [0,14) of the low word, so an issuer steps through a tile with one 32-bit add per operand; the
// single issuing thread is latency-bound, every instruction saved per MMA shows in the MMA rate.
__device__ __forceinline__ void umma_f16_pair_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                 uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A from TMEM, B descriptor as (low word, high word).
__device__ __forceinline__ void umma_f16_pair_ts_lh(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                                    uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], db, %4, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive (count 1) on the barrier at this shared-memory offset in every CTA of `cta_mask`
// once all MMAs issued so far by this thread are complete.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// registers -> TMEM: an mma.sync A-operand fragment (16 rows x 16 K elements of 16-bit data, four
// registers) lands as [lane = row][column = k/2]; taddr's lane field is the first of the 16 rows.
__device__ __forceinline__ void tmem_st_frag16x16(uint32_t taddr, const uint32_t (&r)[4]) {
  asm volatile("tcgen05.st.sync.aligned.16x128b.x2.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3])
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------
// UMMA descriptors (sm_100 format: version field = 1, 128-byte swizzle = 2)
// ----------------------------------------------------------------------------
// Operand whose contraction (K) dimension is contiguous in shared memory:
// rows = M/N index, 64 16-bit elements (128 B) per row, 8-row swizzle atoms of
// 1024 B; `sbo_bytes` = distance between consecutive 8-row atoms.
// Advancing 16 elements along K inside the atom = +32 bytes on the start address.
__device__ __forceinline__ uint64_t desc_kmajor_sw128(uint32_t saddr, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);        // start address  [0,14)
  d |= static_cast<uint64_t>(1) << 16;                         // LBO (unused with swizzle)
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;  // SBO           [32,46)
  d |= static_cast<uint64_t>(1) << 46;                         // descriptor version
  d |= static_cast<uint64_t>(2) << 61;                         // SWIZZLE_128B
  return d;
}
// Operand whose M/N dimension is contiguous in shared memory ("MN-major"):
// each shared-memory row holds 64 consecutive M/N elements of ONE K index;
// 8 K-rows form a 1024 B swizzle atom. `sbo_bytes` = distance between
// consecutive groups of 8 K-rows, `lbo_bytes` = distance between consecutive
// groups of 64 M/N elements.
__device__ __forceinline__ uint64_t desc_mnmajor_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                       uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// Instruction descriptor for kind::f16 with fp32 accumulation.
// dt: DT_F16 / DT_BF16 for both operands; a_mn / b_mn: 1 if that operand is MN-major.
__device__ __host__ __forceinline__ uint32_t make_idesc(int dt, int m, int n, int a_mn, int b_mn) {
  uint32_t d = 0;
  d |= 1u << 4;                        // D format: F32
  d |= static_cast<uint32_t>(dt) << 7;   // A format
  d |= static_cast<uint32_t>(dt) << 10;  // B format
  d |= static_cast<uint32_t>(a_mn) << 15;
  d |= static_cast<uint32_t>(b_mn) << 16;
  d |= static_cast<uint32_t>(n >> 3) << 17;
  d |= static_cast<uint32_t>(m >> 4) << 24;
  return d;
}

// ----------------------------------------------------------------------------
// 16-bit element helpers (two elements packed in one 32-bit word)
// ----------------------------------------------------------------------------
template <int DT>
struct Elem;
template <>
struct Elem<DT_F16> {
  __device__ __forceinline__ static float2 unpack(uint32_t w) {
    __half2 h = *reinterpret_cast<__half2*>(&w);
    return __half22float2(h);
  }
  __device__ __forceinline__ static uint32_t pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <>
struct Elem<DT_BF16> {
  __device__ __forceinline__ static float2 unpack(uint32_t w) {
    float2 f;
    f.x = __uint_as_float(w << 16);
    f.y = __uint_as_float(w & 0xFFFF0000u);
    return f;
  }
  __device__ __forceinline__ static uint32_t pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// sigmoid(x) = 0.5 * tanh(0.5 x) + 0.5 : one MUFU op, no division.
__device__ __forceinline__ float sigmoid_fast(float x) {
  return fmaf(tanh_approx(0.5f * x), 0.5f, 0.5f);
}

// ----------------------------------------------------------------------------
// Packed two-element arithmetic in the data's own 16-bit type (one instruction per pair).
// ----------------------------------------------------------------------------
#ifndef PRISM_FWD_CVT_HW
#define PRISM_FWD_CVT_HW 1   // gated forward: S converted by the one-instruction cvt (measured 2 % faster; plain mode: slower)
#endif
#ifndef PRISM_DB_CVT_HW
#define PRISM_DB_CVT_HW 1   // dB gate warps: S converted by the one-instruction cvt (their ALU pipe is the busier one)
#endif
// Precision of the gate arithmetic, per data type.  1: fp32 per element (tanh.approx.f32, packed
// fp32 FMAs), one rounding when H / dS is converted to 16 bits: the result sits at the error floor
// that 16-bit tensor-core operands allow, like the reference's bf16 kernels, which evaluate the gate
// in fp32 (cute_prism_coop_pc.cu:323-330).  0: arithmetic on f16x2 / bf16x2 pairs, four roundings
// per element: half the instructions, twice the error.  Measured on bf16 at K = 4096: mean
// relative error of C 0.0097 (fp32 gate) against 0.0197 (packed), forward 10 % slower.
// fp16 keeps the packed form by default: its roundings are 8 times finer, and the reference's fp16
// kernels use tanh.approx.f16x2 too (cute_prism_util.hpp:55-77).
#ifndef PRISM_GATE_F32_BF16
#define PRISM_GATE_F32_BF16 1
#endif
#ifndef PRISM_GATE_F32_F16
#define PRISM_GATE_F32_F16 0
#endif
template <int DT>
__device__ __forceinline__ constexpr bool gate_in_f32() {
  return DT == DT_BF16 ? (PRISM_GATE_F32_BF16 != 0) : (PRISM_GATE_F32_F16 != 0);
}

// Two fp32 operations per instruction (sm_100 packed fp32 arithmetic).
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t"
      ".reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t"
      "}\n"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t"
      ".reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t"
      "}\n"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

template <int DT>
struct Pk;
template <>
struct Pk<DT_F16> {
  static constexpr uint32_t kHalf = 0x38003800u;  // (0.5, 0.5)
  static constexpr uint32_t kOne = 0x3C003C00u, kNegOne = 0xBC00BC00u, kOneLo = 0x00003C00u;
  __device__ __forceinline__ static uint32_t cvt(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
  }
  __device__ __forceinline__ static uint32_t cvt_hw(float lo, float hi) { return cvt(lo, hi); }
  __device__ __forceinline__ static uint32_t mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  __device__ __forceinline__ static uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
  }
  __device__ __forceinline__ static uint32_t tanh(uint32_t a) {
    uint32_t d;
    asm("tanh.approx.f16x2 %0, %1;" : "=r"(d) : "r"(a));
    return d;
  }
};
template <>
struct Pk<DT_BF16> {
  static constexpr uint32_t kHalf = 0x3F003F00u;
  static constexpr uint32_t kOne = 0x3F803F80u, kNegOne = 0xBF80BF80u, kOneLo = 0x00003F80u;
  // fp32 pair -> bf16x2 with integer ops: add half an ulp to the bit patterns and keep the upper
  // halves (round to nearest, ties away from zero).  The cvt.rn.bf16x2.f32 instruction runs on the
  // 16-lane/clk special-function pipe (measured: as expensive as a tanh), these ALU ops do not.
  // A NaN keeps its upper half with the quiet bit set (the plain add would carry out of a NaN whose
  // upper mantissa bits are all ones and turn it into a zero); infinities pass through unchanged.
  __device__ __forceinline__ static uint32_t round_bits(uint32_t u) {
    return ((u << 1) > 0xFF000000u) ? (u | 0x00400000u) : (u + 0x8000u);
  }
  __device__ __forceinline__ static uint32_t cvt(float lo, float hi) {
    return __byte_perm(round_bits(__float_as_uint(lo)), round_bits(__float_as_uint(hi)), 0x7632);
  }
  // The single-instruction conversion (special-function pipe): for code whose ALU pipe is the busier one.
  __device__ __forceinline__ static uint32_t cvt_hw(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
  }
  __device__ __forceinline__ static uint32_t mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  __device__ __forceinline__ static uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
  }
  __device__ __forceinline__ static uint32_t tanh(uint32_t a) {
    uint32_t d;
    asm("tanh.approx.bf16x2 %0, %1;" : "=r"(d) : "r"(a));
    return d;
  }
};

// silu(s) for a pair, from fp32 s: with hs = s/2, silu(s) = hs + hs*tanh(hs).
// HW: convert S with the one-instruction cvt (special-function pipe) instead of three ALU ops
template <int DT, bool HW = false>
__device__ __forceinline__ uint32_t silu_pair(float s0, float s1) {
  const uint32_t hs = Pk<DT>::mul(HW ? Pk<DT>::cvt_hw(s0, s1) : Pk<DT>::cvt(s0, s1), Pk<DT>::kHalf);
  return Pk<DT>::fma(hs, Pk<DT>::tanh(hs), hs);
}

// ----------------------------------------------------------------------------
// Warp-level matrix fragments (ldmatrix / stmatrix / mma.sync m16n8k16).
// ldmatrix / stmatrix move 16-bit tiles between shared memory and the register layout that
// tcgen05.ld.16x256b delivers for fp32 TMEM data, so the gate math is elementwise on registers.
// mma.sync itself is only used for the small dR products of the dA+dR kernel: it shares the tensor
// cores with tcgen05.mma and only gets the gaps that tcgen05.mma leaves.
// ----------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t saddr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t saddr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
__device__ __forceinline__ void stmatrix_x4(uint32_t saddr, const uint32_t (&r)[4]) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(saddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3])
               : "memory");
}
template <int DT>
__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                             uint32_t b1) {
  if (DT == DT_BF16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
        "{%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
        "{%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}


// ----------------------------------------------------------------------------
// Hash dropout of the gated modes (training): element (m, k) of group g is kept iff
//   u = top24(splitmix64(splitmix64(seed_g + 0xdeadbeef) ^ splitmix64(m*K + k))) / 2^24  >=  p
// and kept elements are scaled by 1 / (1 - p): the same counter-based mask as the reference's kernels
// (cute_prism_dtype.hpp:28-40, applied to H in the forward and dB kernels, cute_prism_coop_pc.cu:250-301,
// and to dH in the dA+dR kernel), so that forward and backward regenerate it from the per-group seeds.
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}
struct DropCtx {
  uint64_t h1;       // splitmix64(seed_g + 0xdeadbeef)
  long long base;    // m*K + k of this thread's first element: row r0 + lane/4 of the warp, column 2 (lane%4) of the chunk
  long long row8;    // 8 * K: the thread's second row
  float p, inv_keep;
  // multiplier of the element `rsel` rows of 8 down and `col` columns to the right
  __device__ __forceinline__ float mul(int rsel, int col) const {
    const uint64_t h = splitmix64(h1 ^ splitmix64((uint64_t)(base + rsel * row8 + col)));
    const float u = (float)((h >> 40) & 0xFFFFFFull) * (1.0f / 16777216.0f);
    return u >= p ? inv_keep : 0.f;
  }
};
__device__ __forceinline__ uint64_t drop_group_hash(const long long* seeds, int g) {
  return splitmix64((uint64_t)__ldg(seeds + g) + 0xdeadbeefull);
}

// H for one pair of elements from fp32 S and packed 16-bit A: A*silu(S), A*2*sigmoid(S), or S in
// plain mode.  With hs = s/2 and t = tanh(hs): silu(s) = hs + hs t and 2 sigmoid(s) = 1 + t: one
// special-function operation per element, no division.
// DROP: the pair is multiplied by (m0, m1), the dropout multipliers (0 or 1 / (1 - p)).
template <int DT, int GATE, bool HW = false, bool DROP = false>
__device__ __forceinline__ uint32_t gate_pair(uint32_t a2, float s0, float s1, float m0 = 1.f, float m1 = 1.f) {
  if (GATE == GATE_NONE) return Pk<DT>::cvt(s0, s1);
  if (gate_in_f32<DT>()) {
    const float2 hs = mul2(make_float2(s0, s1), make_float2(0.5f, 0.5f));
    const float2 t = make_float2(tanh_approx(hs.x), tanh_approx(hs.y));
    const float2 a = Elem<DT>::unpack(a2);
    float2 h = (GATE == GATE_SILU) ? mul2(a, fma2(hs, t, hs)) : fma2(a, t, a);
    if (DROP) h = mul2(h, make_float2(m0, m1));
    return Pk<DT>::cvt_hw(h.x, h.y);
  }
  uint32_t h;
  if (GATE == GATE_SILU) {
    h = Pk<DT>::mul(a2, silu_pair<DT, HW>(s0, s1));
  } else {
    const uint32_t hs = Pk<DT>::mul(HW ? Pk<DT>::cvt_hw(s0, s1) : Pk<DT>::cvt(s0, s1), Pk<DT>::kHalf);
    h = Pk<DT>::fma(a2, Pk<DT>::tanh(hs), a2);
  }
  if (DROP) h = Pk<DT>::mul(h, Pk<DT>::cvt_hw(m0, m1));
  return h;
}

// TMEM -> registers in the mma.sync accumulator layout: 16 lanes x 16 columns; thread t gets
// r[0..1] = (lane t/4, cols 2(t%4)+{0,1}), r[2..3] = (lane t/4+8, same cols), r[4..7] = cols + 8.
__device__ __forceinline__ void tmem_ld_16x256b_x2(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}

// Internal bias of the gated modes: S[:, k] += factor * ib[k] before the gate.  `ib` points at the bias of
// the warp's 64-column chunk (16-bit, row g of the [G, K] bias, 4-byte aligned), `kvalid` is the number
// of columns of the chunk that lie inside K.  s[pc] holds piece pc (16 columns) in the accumulator
// fragment layout: values 0-3 in columns 2(lane%4) + {0,1}, values 4-7 eight columns further on.
template <int DT>
__device__ __forceinline__ void add_internal_bias(uint32_t (&s)[4][8], const uint16_t* ib, int kvalid, int lane,
                                                  float factor) {
#pragma unroll
  for (int pc = 0; pc < 4; ++pc) {
    const int c = pc * 16 + 2 * (lane & 3);
    float2 lo = make_float2(0.f, 0.f), hi = make_float2(0.f, 0.f);
    if (c < kvalid) lo = Elem<DT>::unpack(__ldg(reinterpret_cast<const uint32_t*>(ib + c)));
    if (c + 8 < kvalid) hi = Elem<DT>::unpack(__ldg(reinterpret_cast<const uint32_t*>(ib + c + 8)));
    s[pc][0] = __float_as_uint(fmaf(lo.x, factor, __uint_as_float(s[pc][0])));
    s[pc][1] = __float_as_uint(fmaf(lo.y, factor, __uint_as_float(s[pc][1])));
    s[pc][2] = __float_as_uint(fmaf(lo.x, factor, __uint_as_float(s[pc][2])));
    s[pc][3] = __float_as_uint(fmaf(lo.y, factor, __uint_as_float(s[pc][3])));
    s[pc][4] = __float_as_uint(fmaf(hi.x, factor, __uint_as_float(s[pc][4])));
    s[pc][5] = __float_as_uint(fmaf(hi.y, factor, __uint_as_float(s[pc][5])));
    s[pc][6] = __float_as_uint(fmaf(hi.x, factor, __uint_as_float(s[pc][6])));
    s[pc][7] = __float_as_uint(fmaf(hi.y, factor, __uint_as_float(s[pc][7])));
  }
}

// Gate step when the rotation runs on tcgen05: one warp turns its 16 rows x 64 columns of
// S = A . blockdiag(R_g)^T (fp32 in TMEM at s_tmem, lane field = the warp's first row) into H
// (16-bit) and writes H to TMEM at h_tmem as the A operand of the dense MMA (8 columns per 16 K
// elements).  The TMEM load delivers the mma.sync accumulator layout and ldmatrix of the A tile the
// matching A-fragment layout, so the gate is elementwise on registers.  h_tmem may alias the first
// 32 of the S columns: every S value is in registers before the first H column is written.
// Nothing here touches the legacy tensor path: mma.sync shares the tensor cores with tcgen05.mma
// and is starved while a burst of tcgen05.mma runs (measured: 13x slower), which would serialise
// the gate warps with the dense product.
// ib / kvalid: internal bias of the chunk (see add_internal_bias), or null.
// DROP / drop: hash dropout of H (see DropCtx).
template <int DT, int GATE, bool DROP = false>
__device__ __forceinline__ void gate_rows16_tmem(uint32_t s_tmem, uint32_t tile, uint32_t r0, int lane,
                                                 uint32_t h_tmem, const uint16_t* ib = nullptr, int kvalid = 64,
                                                 const DropCtx* drop = nullptr) {
  const uint32_t mat = lane >> 3, l8 = lane & 7;
  const uint32_t a_row = r0 + l8 + (mat & 1) * 8;
  uint32_t s[4][8], af[4][4], h[4][4];
#pragma unroll
  for (int pc = 0; pc < 4; ++pc) tmem_ld_16x256b_x2(s_tmem + pc * 16, s[pc]);
  if (GATE != GATE_NONE) {
#pragma unroll
    for (int pc = 0; pc < 4; ++pc) ldmatrix_x4(tile + sw128_offset(a_row, pc * 2 + (mat >> 1)), af[pc]);
  } else {
#pragma unroll
    for (int pc = 0; pc < 4; ++pc) af[pc][0] = af[pc][1] = af[pc][2] = af[pc][3] = 0u;
  }
  tmem_ld_wait();
  if (GATE != GATE_NONE && ib != nullptr) add_internal_bias<DT>(s, ib, kvalid, lane, 1.0f);
#pragma unroll
  for (int pc = 0; pc < 4; ++pc) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // pair e: row r (e even) or r + 8 (e odd), columns pc*16 + 2(lane%4) + {0,1}, eight further on for e >= 2
      float m0 = 1.f, m1 = 1.f;
      if (DROP && GATE != GATE_NONE) {
        m0 = drop->mul(e & 1, pc * 16 + (e >> 1) * 8);
        m1 = drop->mul(e & 1, pc * 16 + (e >> 1) * 8 + 1);
      }
      h[pc][e] = gate_pair<DT, GATE, (PRISM_FWD_CVT_HW != 0) && GATE != GATE_NONE, DROP>(
          af[pc][e], __uint_as_float(s[pc][2 * e]), __uint_as_float(s[pc][2 * e + 1]), m0, m1);
    }
  }
#pragma unroll
  for (int pc = 0; pc < 4; ++pc) tmem_st_frag16x16(h_tmem + pc * 8, h[pc]);
}

// The same gate step with H going to shared memory: the warp's 16 rows x 64 columns of the A tile
// are overwritten in place with H (stmatrix), for kernels whose dense product needs H as a
// shared-memory operand.  Piece pc (16 columns) of S sits at TMEM column s_col(pc) of s_tmem:
// with S laid out in rotation blocks of `blk_stride` columns (>= E), the piece of block b, part np
// starts at b * blk_stride + np * 16.
// s_free (a shared::cluster barrier address, or 0) is arrived on as soon as this warp holds its S
// values in registers: a single S buffer can then be refilled while the gate math still runs.
template <int DT, int GATE, int E, bool DROP = false>
__device__ __forceinline__ void gate_rows16_tmem_smem(uint32_t s_tmem, uint32_t blk_stride, uint32_t tile, uint32_t r0,
                                                      int lane, uint32_t s_free, const uint16_t* ib = nullptr,
                                                      int kvalid = 64, const DropCtx* drop = nullptr,
                                                      uint32_t h_tile = 0, uint32_t h_r0 = 0) {
  constexpr int KS = E / 16;
  const uint32_t mat = lane >> 3, l8 = lane & 7;
  const uint32_t a_row = r0 + l8 + (mat & 1) * 8;
  // H goes back over the A rows, or (h_tile != 0) to rows h_r0 ... of a tile of its own
  const uint32_t h_row = (h_tile != 0) ? h_r0 + l8 + (mat & 1) * 8 : a_row;
  if (h_tile == 0) h_tile = tile;
  uint32_t s[4][8], af[4][4], h[4][4];
#pragma unroll
  for (int pc = 0; pc < 4; ++pc) tmem_ld_16x256b_x2(s_tmem + (pc / KS) * blk_stride + (pc % KS) * 16, s[pc]);
  if (GATE != GATE_NONE) {
#pragma unroll
    for (int pc = 0; pc < 4; ++pc) ldmatrix_x4(tile + sw128_offset(a_row, pc * 2 + (mat >> 1)), af[pc]);
  } else {
#pragma unroll
    for (int pc = 0; pc < 4; ++pc) af[pc][0] = af[pc][1] = af[pc][2] = af[pc][3] = 0u;
  }
  tmem_ld_wait();
  if (s_free != 0) {
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(s_free);
  }
  if (GATE != GATE_NONE && ib != nullptr) add_internal_bias<DT>(s, ib, kvalid, lane, 1.0f);
#pragma unroll
  for (int pc = 0; pc < 4; ++pc) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float m0 = 1.f, m1 = 1.f;
      if (DROP && GATE != GATE_NONE) {
        m0 = drop->mul(e & 1, pc * 16 + (e >> 1) * 8);
        m1 = drop->mul(e & 1, pc * 16 + (e >> 1) * 8 + 1);
      }
      h[pc][e] = gate_pair<DT, GATE, (PRISM_DB_CVT_HW != 0) && GATE != GATE_NONE, DROP>(
          af[pc][e], __uint_as_float(s[pc][2 * e]), __uint_as_float(s[pc][2 * e + 1]), m0, m1);
    }
  }
#pragma unroll
  for (int pc = 0; pc < 4; ++pc) stmatrix_x4(h_tile + sw128_offset(h_row, pc * 2 + (mat >> 1)), h[pc]);
}

}  // namespace prism
