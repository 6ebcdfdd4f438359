// Kernel of the Prism backward for input and rotation gradients, for sm_100a (included by the per-dtype
// translation units prism_bwd_dadr_f16.cu / prism_bwd_dadr_bf16.cu, which instantiate it, and by the launcher):
//   dH_g = dC_g . B_g                                   (dense)
//   S_g  = A . blockdiag(R_g)^T                         (recomputed)
//   gated:  dS = dH * A * silu'(S),  dA += dH * silu(S) + blockdiag(dS) . R_g
//   plain:  dS = dH,                 dA += blockdiag(dS) . R_g
//   dR_g[block b] = dS_b^T . A_b
// summed over groups g for dA and over tokens for dR.
//
// Replaces the reference's bwd_dadr_kernel + dR_reduce_kernel + prism_backward_dA_dR_launch
// (cute_prism_backward_dadr.cu:735-995) and its binding (torch_ext/prism_bwd_dadr_torch.cu:42-210).
// The reference adds dR partials with fp32 atomicAdd (cute_prism_backward_dadr.cu:675-682); here
// every CTA owns one exclusive partial buffer that it updates in a fixed order, and a second
// kernel adds the buffers in a fixed order, so dR is bit-stable from run to run.
//
// CTAs work in pairs (cluster of 2, tcgen05 cta_group::2) on [256 tokens x 128 features]: each CTA
// owns 128 of the tokens and loads half of the B_g features, which cuts the L2 traffic per flop.
// One CTA works on its [128 tokens x 128 features] tile of dA and walks over all groups.  All three
// products of the dA path run on tcgen05 (mma.sync shares the tensor cores with tcgen05.mma and is
// starved while tcgen05.mma bursts run, which would put the gate warps behind the dense product):
//   warp 0       TMA producer: A tiles once per tile; per group the R_g tiles and the dC / B_g stages
//   warps 1, 22, 23  MMA issuers (leader CTA), one product each, per group
//                  rotation  S_g = A . blockdiag(R_g)^T: M256 N=E K=16 per rotation block (gated mode)
//                  dense     dH_g = dC_g . B_g: M256 N128 K16 (dC K-major, B_g MN-major), two TMEM buffers
//                  dS . R    dA += blockdiag(dS_g) . R_g: M256 N=E K=16 per block (dS K-major from shared
//                            memory, R_g MN-major), accumulated over the groups in TMEM
//   warps 4-19   gate warps, 16 tokens x 64 features each: S and dH fragments straight from TMEM
//                (tcgen05.ld.16x256b delivers the mma.sync accumulator layout), A fragments by ldmatrix
//                (same layout), gate math on registers, dS -> stmatrix to shared memory; the gate
//                term dH * silu(S) of dA stays in fp32 registers for the whole tile
//   warps 2,3,20,21  dR warps: ldmatrix.trans of the dS and A tiles, mma.sync over the 128 tokens
//                (off the critical path), fixed-order accumulation into this CTA's fp32 partial buffer.
// TMEM: dH 2 x 128 columns, S 128, dA 128.
#pragma once
#include "prism_host.cuh"
#include "prism_kernels.cuh"

namespace prism {

#ifndef PRISM_K2_CVT_HW
#define PRISM_K2_CVT_HW 1
#endif
namespace dadr {
constexpr int kThreads = 768;
constexpr int kWarpTma = 0, kWarpMma = 1, kWarpRot = 22, kWarpDsr = 23;
constexpr int kGateWarp0 = 4;      // multiple of 4: (warp & 3) is the TMEM lane quarter
constexpr int kNumGateWarps = 16;
constexpr int kNumDrWarps = 4;     // warps 2, 3, 20, 21
constexpr int kDhCol0 = 0, kSCol0 = 256, kDaCol0 = 384;   // TMEM columns: dH ring (2 x 128), S, dA
constexpr int kTile = 128 * 128;   // bytes of a [128 x 64] 16-bit tile
constexpr int kMaxStages = 6;
constexpr int kMaxRBufs = 4;
// one pipeline stage = kOut outputs of the group: kOut/64 dC tiles [128 tokens x 64] and this CTA's
// half of the B_g features, a [kOut outputs x 64 features] tile.  64-output stages (24 KB) are
// released after four MMAs, which keeps the TMA queue fuller than 128-output stages do.
template <int E> struct Stage {
  static constexpr int kOut = 64;
  static constexpr int kDcTiles = kOut / 64;
  static constexpr int kBTile = kOut * 128;
  static constexpr int kBytes = kDcTiles * kTile + kBTile;
};
}  // namespace dadr

struct DadrParams {
  int M, N, K, gs, E, G;
  int n_mtiles, runs;
  int n_ft;            // 128-feature columns of dA
  int n_main;          // main CTA pairs: n_ft * runs, pair = run * n_ft + column
  int n_extra, steal;  // extra CTA pairs; token tiles each main pair leaves to them (0: none)
  int slots;           // dR partial slabs per extra CTA (one per main pair it helps)
  int ns, rb;          // stages of the dC/B ring, number of R buffers
  int rr_tile_bytes;   // bytes reserved per rotation R tile [E/2 x 64] (multiple of 1024)
  int rd_tile_bytes;   // bytes reserved per dS.R R tile [E x 64] (multiple of 1024)
  float scale;
  void* dA;
  long long ldda;
  float* partial;      // [2*runs][G*E][K] fp32: one buffer per CTA of every main pair
  float* partial_x;    // [2*n_extra][slots][G*E][128] fp32: slabs of the extra pairs' CTAs
  int* err;
};

// Arguments of the internal-bias and dropout instances only.  A kernel parameter of its own: with these
// fields inside DadrParams the instance without either (the benchmarked one) compiled to more spills.
struct DadrExtra {
  const long long* drop_seeds;   // per-group dropout seeds (DROP kernels)
  float drop_p, drop_inv_keep;
  const void* ib;      // internal bias [G, K] (gated modes, IB kernels) or null
  float* partial_ib;   // [2*runs][G][K] fp32: column sums of dS of the main CTAs
  float* partial_ib_x; // [2*n_extra][slots][G][128] fp32: ... of the extra pairs' CTAs
};

struct DadrBarriers {
  uint64_t a_full;                         // local: this CTA's A tiles landed
  uint64_t a_peer;                         // leader's copy is used: the peer's A tiles landed (forwarded by the peer)
  uint64_t a_empty;                        // local: gate and dR warps are done with the A tiles
  uint64_t r_full[dadr::kMaxRBufs];        // leader's copy is used: both CTAs' R tiles of the group landed
  uint64_t r_empty[dadr::kMaxRBufs];       // local, multicast commit: dS.R of the group has read them
  uint64_t st_full[dadr::kMaxStages];      // leader's copy is used
  uint64_t st_empty[dadr::kMaxStages];     // local, multicast commit
  uint64_t dh_full[2];                     // local, multicast commit: dH of the group is in its TMEM buffer
  uint64_t s_full;                         // local, multicast commit: S of the group is in TMEM
  uint64_t s_free;                         // leader's copy is used: the gate warps hold S in registers
  uint64_t gate_done[2];                   // leader's copy is used: gate warps read dH, wrote dS (both CTAs)
  uint64_t ds_full[2];                     // local: the gate warps wrote dS (for the dR warps)
  uint64_t ds_empty[2];                    // local: dR warps + the commit after dS.R
  uint64_t da_full;                        // local, multicast commit: dA of the tile is complete in TMEM
  uint64_t ib_full[2];                     // local (IB): every gate warp wrote its column sums of dS
  uint32_t tmem_base;
};

__device__ __forceinline__ void dr_accumulate(float* addr, float x, float y, bool first) {
  if (first) {
    *reinterpret_cast<float2*>(addr) = make_float2(x, y);
  } else {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(x), "f"(y) : "memory");
  }
}

// One pair of elements of the gated backward.  The R tiles of the gated mode hold R/2, so the
// rotation delivers hs = S/2 directly.  With t = tanh(hs):
//   silu(S)  = g = hs + hs t
//   silu'(S) = (1 + x) / 2,  x = g + t (1 - g)
// Returns 2 dS = dh a (1 + x) (the factor 2 is undone by the halved R in dS.R and by the scale of
// the dR reduction) and adds the gate term dh silu(S) of dA to acc0 / acc1.
// sigmoid gate (gate value 2 sigmoid(S) = 1 + t, derivative (1 - t^2) / 2): 2 dS = dh a (1 - t^2).
template <int DT, int GATE>
__device__ __forceinline__ uint32_t gate_bwd_pair(uint32_t a2, uint32_t hs, float dh0, float dh1, float& acc0,
                                                  float& acc1) {
  const uint32_t t = Pk<DT>::tanh(hs);
  if (GATE == GATE_SIGMOID) {
    const uint32_t g1 = Pk<DT>::fma(t, Pk<DT>::kOne, Pk<DT>::kOne);
    const uint32_t q1 = Pk<DT>::mul(Pk<DT>::cvt(dh0, dh1), a2);
    const float2 gf1 = Elem<DT>::unpack(g1);
    acc0 = fmaf(dh0, gf1.x, acc0);
    acc1 = fmaf(dh1, gf1.y, acc1);
    return Pk<DT>::fma(Pk<DT>::mul(q1, t), Pk<DT>::mul(t, Pk<DT>::kNegOne), q1);
  }
  const uint32_t g = Pk<DT>::fma(hs, t, hs);
  const uint32_t w = Pk<DT>::fma(g, Pk<DT>::kNegOne, Pk<DT>::kOne);
  const uint32_t x = Pk<DT>::fma(t, w, g);
  const uint32_t q = Pk<DT>::mul(Pk<DT>::cvt(dh0, dh1), a2);
  const float2 gf = Elem<DT>::unpack(g);
  acc0 = fmaf(dh0, gf.x, acc0);
  acc1 = fmaf(dh1, gf.y, acc1);
  return Pk<DT>::fma(q, x, q);
}

// The same in fp32 (hs0, hs1 = S/2 as delivered by the rotation): one rounding, when 2 dS is
// converted to 16 bits for the dS . R and dR products.
template <int DT, int GATE>
__device__ __forceinline__ uint32_t gate_bwd_pair_f32(uint32_t a2, float hs0, float hs1, float dh0, float dh1, float& acc0,
                                                      float& acc1) {
  const float2 hs = make_float2(hs0, hs1), dh = make_float2(dh0, dh1), one = make_float2(1.f, 1.f);
  const float2 t = make_float2(tanh_approx(hs0), tanh_approx(hs1));
  if (GATE == GATE_SIGMOID) {
    const float2 q1 = mul2(dh, Elem<DT>::unpack(a2));
    const float2 acc1s = fma2(dh, make_float2(1.f + t.x, 1.f + t.y), make_float2(acc0, acc1));
    acc0 = acc1s.x;
    acc1 = acc1s.y;
    const float2 qt = mul2(q1, t);
    const float2 ds1 = fma2(qt, make_float2(-t.x, -t.y), q1);
    return Pk<DT>::cvt_hw(ds1.x, ds1.y);
  }
  const float2 g = fma2(hs, t, hs);
  const float2 w = fma2(g, make_float2(-1.f, -1.f), one);
  const float2 x = fma2(t, w, g);
  const float2 q = mul2(dh, Elem<DT>::unpack(a2));
  const float2 acc = fma2(dh, g, make_float2(acc0, acc1));
  acc0 = acc.x;
  acc1 = acc.y;
  const float2 ds = fma2(q, x, q);
  return Pk<DT>::cvt_hw(ds.x, ds.y);
}

// Work of a CTA pair: a list of tiles [256 tokens x 128 features].  A main pair (column fx, run)
// walks the token-tile pairs run, run + runs, ... of its column and leaves the last `steal` of them
// to the extra pairs, which exist when the main pairs do not fill the GPU: extra pair e helps the
// main pairs [e n_main / n_extra, (e+1) n_main / n_extra), token tile by token tile.  Every CTA
// adds its dR contributions to memory of its own (a [G*E x K] buffer per main CTA, a [G*E x 128]
// slab per helped main pair in an extra CTA), first tile stored, later tiles added in order.
struct DadrUnit {
  int f0;         // first feature of the tile
  int mp;         // token-tile pair
  bool first;     // first tile that touches this dR slab: store, do not add
  float* part;    // dR slab of this CTA for the tile's column (row 0, feature f0)
  long long ld;   // its row pitch
};
__device__ __forceinline__ int dadr_tiles_of_run(const DadrParams& p, int run) {
  return ((p.n_mtiles + 1) / 2 - run + p.runs - 1) / p.runs;
}
__device__ __forceinline__ int dadr_num_units(const DadrParams& p, int pidx) {
  if (pidx < p.n_main) return dadr_tiles_of_run(p, pidx / p.n_ft) - p.steal;
  const int e = pidx - p.n_main;
  return ((e + 1) * p.n_main / p.n_extra - e * p.n_main / p.n_extra) * p.steal;
}
__device__ __forceinline__ DadrUnit dadr_unit(const DadrParams& p, int pidx, int rank, int k) {
  DadrUnit u;
  const long long GE = (long long)p.G * p.E;
  if (pidx < p.n_main) {
    const int fx = pidx % p.n_ft, run = pidx / p.n_ft;
    u.f0 = fx * 128;
    u.mp = run + k * p.runs;
    u.first = (k == 0);
    u.part = p.partial + (long long)(run * 2 + rank) * GE * p.K + u.f0;
    u.ld = p.K;
  } else {
    const int e = pidx - p.n_main;
    const int m_lo = e * p.n_main / p.n_extra;
    const int cnt = (e + 1) * p.n_main / p.n_extra - m_lo;
    const int j = k / cnt, mi = k - j * cnt;      // token tile by token tile over the helped pairs
    const int m = m_lo + mi;
    const int fx = m % p.n_ft, run = m / p.n_ft;
    u.f0 = fx * 128;
    u.mp = run + (dadr_tiles_of_run(p, run) - p.steal + j) * p.runs;
    u.first = (j == 0);
    u.part = p.partial_x + ((long long)(e * 2 + rank) * p.slots + mi) * GE * 128;
    u.ld = 128;
  }
  return u;
}
// d(internal bias) slab of this CTA for unit k's column (group 0, feature f0); row pitch as the dR slab's
__device__ __forceinline__ float* dadr_unit_ib(const DadrParams& p, const DadrExtra& x, int pidx, int rank, int k) {
  if (pidx < p.n_main) {
    const int fx = pidx % p.n_ft, run = pidx / p.n_ft;
    return x.partial_ib + (long long)(run * 2 + rank) * p.G * p.K + fx * 128;
  }
  const int e = pidx - p.n_main;
  const int m_lo = e * p.n_main / p.n_extra;
  const int cnt = (e + 1) * p.n_main / p.n_extra - m_lo;
  const int mi = k % cnt;
  return x.partial_ib_x + ((long long)(e * 2 + rank) * p.slots + mi) * p.G * 128;
}

// IB: the internal-bias variant (gated modes): S += bias before the gate, and the column sums of dS over
// the tokens (the bias gradient) leave through a second set of per-CTA fp32 buffers: every gate warp
// sums its 16 token rows with shuffles, the 8 warps of a 64-feature chunk meet in shared memory, are
// added in a fixed order, and one thread per column stores (first tile) or adds (later tiles).
// DROP: hash dropout (see DropCtx): dH is multiplied by the forward's mask before it is used.
template <int DT, int GATE, int E, bool IB, bool DROP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(dadr::kThreads, 1)
prism_bwd_dadr_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmRr,
                      const __grid_constant__ CUtensorMap tmRd, const __grid_constant__ CUtensorMap tmdC,
                      const __grid_constant__ CUtensorMap tmB, const DadrParams p, const DadrExtra ex) {
  using namespace dadr;
  using St = Stage<E>;
  constexpr int KS = E / 16;       // 16-wide steps per rotation block
  constexpr int NB = 64 / E;       // rotation blocks per 64-column tile
  constexpr int NBLK = 128 / E;    // rotation blocks of the tile's 128 features
  constexpr bool kGated = (GATE != GATE_NONE);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  // R buffer of a group: two rotation tiles [E/2 x 64] (this CTA's half of the rows), then two dS.R
  // tiles [E x 64] (shifted by E/2 columns in the peer, see the producer)
  const int r_buf_bytes = 2 * p.rr_tile_bytes + 2 * p.rd_tile_bytes;
  uint8_t* smemA = smem;                        // 2 tiles [128 x 64]
  uint8_t* smemDS = smemA + 2 * kTile;          // 2 buffers x 2 tiles [128 x 64]
  uint8_t* smemR = smemDS + 4 * kTile;          // rb buffers
  uint8_t* smemSt = smemR + p.rb * r_buf_bytes; // ns stages: dC tiles + B tile
  float* smemIb = reinterpret_cast<float*>(smemSt + p.ns * St::kBytes);   // IB: [2][16 gate warps][64] column sums
  DadrBarriers* bars = reinterpret_cast<DadrBarriers*>(smemSt + p.ns * St::kBytes + (IB ? 8192 : 0));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0 = leader (issues the MMAs), 1 = peer
  const int pidx = blockIdx.x >> 1;          // CTA pair: main pairs first, then the extra pairs
  const int G = p.G;
  const int nstg = (p.gs + St::kOut - 1) / St::kOut;  // stages per group
  const bool is_gate = warp >= kGateWarp0 && warp < kGateWarp0 + kNumGateWarps;
  const bool is_dr = warp == 2 || warp == 3 || warp == 20 || warp == 21;
  const int n_units = dadr_num_units(p, pidx);                  // tiles of this CTA pair
  const int total = n_units * G;                                // groups it walks

  if (threadIdx.x == 0) {
    mbar_init(&bars->a_full, 1);
    mbar_init(&bars->a_peer, 1);
    mbar_init(&bars->a_empty, kNumGateWarps + kNumDrWarps);
    for (int i = 0; i < kMaxRBufs; ++i) { mbar_init(&bars->r_full[i], 2); mbar_init(&bars->r_empty[i], 1); }
    for (int i = 0; i < kMaxStages; ++i) { mbar_init(&bars->st_full[i], 2); mbar_init(&bars->st_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->dh_full[i], 1);
      mbar_init(&bars->gate_done[i], 2 * kNumGateWarps);
      mbar_init(&bars->ds_full[i], kNumGateWarps);
      mbar_init(&bars->ds_empty[i], kNumDrWarps + 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->s_free, 2 * kNumGateWarps);
    mbar_init(&bars->da_full, 1);
    mbar_init(&bars->ib_full[0], kNumGateWarps);
    mbar_init(&bars->ib_full[1], kNumGateWarps);
    fence_mbar_init();
  }
  if (warp == kWarpMma) {
    tmem_alloc_pair(&bars->tmem_base, 512);
    tmem_relinquish_pair();
  }
  if (warp == kWarpTma && lane == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmRr);
    prefetch_tmap(&tmRd);
    prefetch_tmap(&tmdC);
    prefetch_tmap(&tmB);
  }
  // the peer's barriers must be initialised before anything arrives on them remotely
  tc_fence_before_sync();
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == kWarpTma) {
    // ------------------------------------------------------------------ TMA producer
    // The completion of the R and stage loads is counted on the leader's barriers: its MMAs read both
    // CTAs' tiles.  The A tiles complete on the local barrier (gate and dR warps read them too).
    if (lane == 0) {
      bool ok = true;
      uint32_t tile_iter = 0;
      Ring rr(p.rb), rst(p.ns);
      for (int k = 0; k < n_units && ok; ++k, ++tile_iter) {
        const DadrUnit u = dadr_unit(p, pidx, (int)rank, k);
        const int f0 = u.f0;
        const int m0 = (u.mp * 2 + (int)rank) * 128;
        if (!mbar_wait(&bars->a_empty, (tile_iter & 1) ^ 1)) { ok = false; break; }
        mbar_arrive_expect_tx(&bars->a_full, 2 * kTile);
        tma_load_2d(smemA, &tmA, &bars->a_full, f0, m0);
        tma_load_2d(smemA + kTile, &tmA, &bars->a_full, f0 + 64, m0);
        for (int g = 0; g < G && ok; ++g, rr.next()) {
          if (!mbar_wait(&bars->r_empty[rr.idx], rr.phase ^ 1)) { ok = false; break; }
          uint8_t* dstR = smemR + rr.idx * r_buf_bytes;
          const uint32_t rfull = mapa_shared(smem_u32(&bars->r_full[rr.idx]), 0);
          mbar_arrive_expect_tx_cluster(rfull, (kGated ? 2 * (E / 2) * 128 : 0) + 2 * E * 128);
          if (kGated) {
            // rotation: an MMA spanning the pair takes the first E/2 rows of R_g from the leader, the rest from the peer
            tma_load_2d_pair(dstR, &tmRr, rfull, f0, g * E + (int)rank * (E / 2));
            tma_load_2d_pair(dstR + p.rr_tile_bytes, &tmRr, rfull, f0 + 64, g * E + (int)rank * (E / 2));
          }
          // dS . R: R_g is the MN-major operand there and the pair splits its N (the block's columns):
          // the peer loads its tiles E/2 columns further right, so that its half of every block sits
          // where the leader's half sits
          uint8_t* dstD = dstR + 2 * p.rr_tile_bytes;
          tma_load_2d_pair(dstD, &tmRd, rfull, f0 + (int)rank * (E / 2), g * E);
          tma_load_2d_pair(dstD + p.rd_tile_bytes, &tmRd, rfull, f0 + 64 + (int)rank * (E / 2), g * E);
          for (int s = 0; s < nstg; ++s, rst.next()) {
            const int st = rst.idx;
            if (!mbar_wait(&bars->st_empty[st], rst.phase ^ 1)) { ok = false; break; }
            uint8_t* dst = smemSt + st * St::kBytes;
            const int n0 = g * p.gs + s * St::kOut;
            const bool two = St::kDcTiles == 2 && p.gs - s * St::kOut > 64;   // the slice has more than 64 outputs
            const uint32_t stfull = mapa_shared(smem_u32(&bars->st_full[st]), 0);
            mbar_arrive_expect_tx_cluster(stfull, (two ? 2 : 1) * kTile + St::kBTile);
            tma_load_2d_pair(dst, &tmdC, stfull, n0, m0);
            if (two) tma_load_2d_pair(dst + kTile, &tmdC, stfull, n0 + 64, m0);
            tma_load_2d_pair(dst + St::kDcTiles * kTile, &tmB, stfull, f0 + (int)rank * 64, n0);
          }
        }
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA issuer
    // Three threads of the leader CTA issue tcgen05.mma, one per product (this one: the dense product).
    // Issuing costs a thread 60-80 clocks per MMA whatever its size, a barrier test ~65 and a commit
    // ~90, so one thread cannot feed the tensor pipe with the 32 MMAs of a group; the products are
    // ordered among themselves by barriers only.
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_h = make_idesc(DT, 256, 128, 0, 1);   // dH: M = 256 tokens; dC K-major, B_g MN-major
      // descriptors of stage 0; a stage further on adds its size >> 4 to the low words
      const uint64_t dst0 = desc_kmajor_sw128(smem_u32(smemSt), 1024);
      const uint64_t dsb0 = desc_mnmajor_sw128(smem_u32(smemSt) + St::kDcTiles * kTile, St::kBTile, 1024);
      const uint32_t k_hi = (uint32_t)(dst0 >> 32), b_hi = (uint32_t)(dsb0 >> 32);
      bool ok = true;
      Ring rst(p.ns);
      for (int n = 0; n < total && ok; ++n) {
        if (n >= 2) {   // the gate warps have read dH of group n - 2 out of this buffer
          const uint32_t gd = (uint32_t)(n - 2);
          if (!mbar_wait_cluster(&bars->gate_done[gd & 1], (gd >> 1) & 1)) { ok = false; break; }
        }
        const uint32_t d_tmem = tmem_base + kDhCol0 + ((uint32_t)n & 1) * 128;
        for (int s = 0; s < nstg; ++s, rst.next()) {
          const int st = rst.idx;
          if (!mbar_wait_cluster(&bars->st_full[st], rst.phase)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_lo = (uint32_t)dst0 + st * (St::kBytes >> 4);
          const uint32_t b_lo = (uint32_t)dsb0 + st * (St::kBytes >> 4);
          constexpr int kSteps = St::kOut / 16;
          const int ksteps = min(kSteps, (p.gs - s * St::kOut) / 16);
          if (ksteps == kSteps) {
            // K16 step ks: dC tile ks/4 (+kTile), 32 bytes per step inside it; B_g rows 16 ks (+2048 bytes)
            umma_f16_pair_lh(d_tmem, a_lo, k_hi, b_lo, b_hi, idesc_h, s > 0 ? 1u : 0u);
#pragma unroll
            for (int ks = 1; ks < kSteps; ++ks)
              umma_f16_pair_lh(d_tmem, a_lo + (((ks >> 2) * kTile + (ks & 3) * 32) >> 4), k_hi,
                               b_lo + ((ks * 2048) >> 4), b_hi, idesc_h, 1u);
          } else {
            for (int ks = 0; ks < ksteps; ++ks)
              umma_f16_pair_lh(d_tmem, a_lo + (((ks >> 2) * kTile + (ks & 3) * 32) >> 4), k_hi,
                               b_lo + ((ks * 2048) >> 4), b_hi, idesc_h, (s > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit_pair(&bars->st_empty[st], 0x3);
        }
        if (!ok) break;
        umma_commit_pair(&bars->dh_full[n & 1], 0x3);
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    } else if (lane == 0 && rank == 1 && kGated) {
      // the peer tells the leader's MMA issuer when its A tiles have landed
      bool ok = true;
      uint32_t ph = 0;
      const uint32_t a_peer = mapa_shared(smem_u32(&bars->a_peer), 0);
      for (int u = 0; u < n_units && ok; ++u, ph ^= 1u) {
        if (!mbar_wait(&bars->a_full, ph)) { ok = false; break; }
        mbar_arrive_cluster(a_peer);
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp == kWarpRot) {
    // ------------------------------------------------------------------ MMA issuer: rotation S_g = A . blockdiag(R_g)^T
    if (lane == 0 && rank == 0 && kGated) {
      const uint32_t idesc_s = make_idesc(DT, 256, E, 0, 0);     // S block: A K-major, R_g K-major
      const uint64_t dA0 = desc_kmajor_sw128(smem_u32(smemA), 1024);
      const uint64_t dRr0 = desc_kmajor_sw128(smem_u32(smemR), 1024);
      const uint32_t k_hi = (uint32_t)(dA0 >> 32);
      const uint32_t r_step = (uint32_t)r_buf_bytes >> 4;
      const uint32_t rr_tile = (uint32_t)p.rr_tile_bytes >> 4;
      bool ok = true;
      Ring rr(p.rb);
      uint32_t a_phase = 0;
      int gi = 0;   // index of group n inside its tile
      for (int n = 0; n < total && ok; ++n, rr.next(), gi = (gi + 1 == G) ? 0 : gi + 1) {
        if (gi == 0) {   // a new tile: its A tiles must have landed in both CTAs
          if (!mbar_wait(&bars->a_full, a_phase)) { ok = false; break; }
          if (!mbar_wait_cluster(&bars->a_peer, a_phase)) { ok = false; break; }
          a_phase ^= 1u;
        }
        if (n >= 1) {    // the gate warps hold S of group n - 1 in registers
          if (!mbar_wait_cluster(&bars->s_free, (uint32_t)(n - 1) & 1)) { ok = false; break; }
        }
        if (!mbar_wait_cluster(&bars->r_full[rr.idx], rr.phase)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t r_lo = (uint32_t)dRr0 + rr.idx * r_step;
#pragma unroll
        for (int b = 0; b < NBLK; ++b) {
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
            const int fo = b * E + ks * 16;   // features fo .. fo+16 of the 128: tile and 32-byte step inside it
            const uint32_t ta = (uint32_t)((fo >> 6) * (kTile >> 4) + ((fo & 63) >> 4) * 2);
            const uint32_t tr = (uint32_t)(fo >> 6) * rr_tile + (uint32_t)(((fo & 63) >> 4) * 2);
            umma_f16_pair_lh(tmem_base + kSCol0 + b * E, (uint32_t)dA0 + ta, k_hi, r_lo + tr, k_hi, idesc_s,
                             ks > 0 ? 1u : 0u);
          }
        }
        umma_commit_pair(&bars->s_full, 0x3);
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp == kWarpDsr) {
    // ------------------------------------------------------------------ MMA issuer: dA += blockdiag(dS_g) . R_g
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_a = make_idesc(DT, 256, E, 0, 1);     // dA block: dS K-major, R_g MN-major
      const uint64_t dS0 = desc_kmajor_sw128(smem_u32(smemDS), 1024);
      const uint64_t dRd0 = desc_mnmajor_sw128(smem_u32(smemR) + 2 * p.rr_tile_bytes, (uint32_t)p.rd_tile_bytes, 1024);
      const uint32_t k_hi = (uint32_t)(dS0 >> 32), rd_hi = (uint32_t)(dRd0 >> 32);
      const uint32_t r_step = (uint32_t)r_buf_bytes >> 4;
      const uint32_t rd_tile = (uint32_t)p.rd_tile_bytes >> 4;
      bool ok = true;
      Ring rr(p.rb);
      int gi = 0;
      for (int n = 0; n < total && ok; ++n, rr.next()) {
        // the gate warps of both CTAs have written dS of group n
        if (!mbar_wait_cluster(&bars->gate_done[n & 1], ((uint32_t)n >> 1) & 1)) { ok = false; break; }
        if (!kGated) {   // (in the gated mode the rotation has waited for these R tiles already)
          if (!mbar_wait_cluster(&bars->r_full[rr.idx], rr.phase)) { ok = false; break; }
        }
        tc_fence_after_sync();
        const uint32_t s_lo = (uint32_t)dS0 + ((uint32_t)n & 1) * ((2 * kTile) >> 4);
        const uint32_t r_lo = (uint32_t)dRd0 + rr.idx * r_step;
#pragma unroll
        for (int b = 0; b < NBLK; ++b) {
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
            // dS (K-major): features b*E + ks*16 ..; R_g (MN-major): rows ks*16 .. (2048 bytes per 16 rows),
            // columns of block b
            const int fo = b * E + ks * 16;
            const uint32_t ta = (uint32_t)((fo >> 6) * (kTile >> 4) + ((fo & 63) >> 4) * 2);
            const int co = b * E;
            const uint32_t tr = (uint32_t)(co >> 6) * rd_tile + (uint32_t)(((co & 63) * 2) >> 4) + (uint32_t)(ks * 128);
            umma_f16_pair_lh(tmem_base + kDaCol0 + b * E, s_lo + ta, k_hi, r_lo + tr, rd_hi, idesc_a,
                             (gi > 0 || ks > 0) ? 1u : 0u);
          }
        }
        umma_commit_pair(&bars->ds_empty[n & 1], 0x3);
        umma_commit_pair(&bars->r_empty[rr.idx], 0x3);
        if (++gi == G) {
          gi = 0;
          umma_commit_pair(&bars->da_full, 0x3);   // the tile's dA is complete
        }
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (is_gate) {
    // ------------------------------------------------------------------ gate warps
    const int gw = warp - kGateWarp0;
    const int q = gw & 3, half = (gw >> 2) & 1, ch = gw >> 3;   // lane quarter, 16-row half, 64-column tile
    const uint32_t r0 = q * 32 + half * 16;                    // first of this warp's 16 token rows
    const uint32_t lane_base = r0 << 16;                       // TMEM lane window [r0, r0+16)
    const uint32_t mat = lane >> 3, l8 = lane & 7;
    const uint32_t a_row = r0 + l8 + (mat & 1) * 8;            // A fragments, dS stores
    const uint32_t tileA = smem_u32(smemA + ch * kTile);
    const uint32_t s_free_addr = mapa_shared(smem_u32(&bars->s_free), 0);
    const uint32_t gate_done_addr = mapa_shared(smem_u32(&bars->gate_done[0]), 0);
    // internal bias: this warp's 64 columns of row 0 of the [G, K] bias, and how many of them lie inside K
    const uint16_t* ib_row = nullptr;
    int ib_valid = 0;
    float dacc[8][4];   // gate term of dA, 16 rows x 64 columns of this warp, whole tile
#pragma unroll
    for (int i = 0; i < 8; ++i) { dacc[i][0] = dacc[i][1] = dacc[i][2] = dacc[i][3] = 0.f; }
    bool ok = true;
    uint32_t tile_iter = 0, gg = 0;
    for (int k = 0; k < n_units && ok; ++k, ++tile_iter) {
      const DadrUnit u = dadr_unit(p, pidx, (int)rank, k);
      const int f0 = u.f0;
      const int mt = u.mp * 2 + (int)rank;
      float* part_ib = nullptr;
      if (IB) {
        part_ib = dadr_unit_ib(p, ex, pidx, (int)rank, k);
        ib_row = reinterpret_cast<const uint16_t*>(ex.ib) + f0 + ch * 64;
        ib_valid = p.K - (f0 + ch * 64);
      }
      if (!mbar_wait(&bars->a_full, tile_iter & 1)) { ok = false; break; }
      for (int g = 0; g < G && ok; ++g, ++gg) {
        const uint32_t hb = gg & 1, ph = (gg >> 1) & 1;
        if (kGated) {
          if (!mbar_wait(&bars->s_full, gg & 1)) { ok = false; break; }
        }
        if (!mbar_wait(&bars->dh_full[hb], ph)) { ok = false; break; }
        if (!mbar_wait(&bars->ds_empty[hb], ph ^ 1)) { ok = false; break; }
        tc_fence_after_sync();
        DropCtx dctx;
        if (DROP && kGated) {
          dctx.h1 = drop_group_hash(ex.drop_seeds, g);
          dctx.base = (long long)(mt * 128 + (int)r0 + (lane >> 2)) * p.K + f0 + ch * 64 + 2 * (lane & 3);
          dctx.row8 = 8ll * p.K;
          dctx.p = ex.drop_p;
          dctx.inv_keep = ex.drop_inv_keep;
        }
        const uint32_t tileDS = smem_u32(smemDS + hb * 2 * kTile + ch * kTile);
        const uint32_t tdh = tmem_base + lane_base + kDhCol0 + hb * 128 + ch * 64;
        const uint32_t ts = tmem_base + lane_base + kSCol0 + ch * 64;
        // two 16-column pieces per pass: all loads, then the gate math, then the stores
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          uint32_t sv[2][8], dh[2][8], af[2][4], dsf[2][4];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int pc = pass * 2 + i;
            if (kGated) {
              tmem_ld_16x256b_x2(ts + pc * 16, sv[i]);
              ldmatrix_x4(tileA + sw128_offset(a_row, pc * 2 + (mat >> 1)), af[i]);
            }
            tmem_ld_16x256b_x2(tdh + pc * 16, dh[i]);
          }
          tmem_ld_wait();
          if (IB && kGated) {
            // the rotation delivered S/2 (halved R): add half the bias
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const int c = (pass * 2 + i) * 16 + 2 * (lane & 3);
              const uint16_t* ibp = ib_row + (long long)g * p.K;
              float2 lo = make_float2(0.f, 0.f), hi = make_float2(0.f, 0.f);
              if (c < ib_valid) lo = Elem<DT>::unpack(__ldg(reinterpret_cast<const uint32_t*>(ibp + c)));
              if (c + 8 < ib_valid) hi = Elem<DT>::unpack(__ldg(reinterpret_cast<const uint32_t*>(ibp + c + 8)));
              sv[i][0] = __float_as_uint(fmaf(lo.x, 0.5f, __uint_as_float(sv[i][0])));
              sv[i][1] = __float_as_uint(fmaf(lo.y, 0.5f, __uint_as_float(sv[i][1])));
              sv[i][2] = __float_as_uint(fmaf(lo.x, 0.5f, __uint_as_float(sv[i][2])));
              sv[i][3] = __float_as_uint(fmaf(lo.y, 0.5f, __uint_as_float(sv[i][3])));
              sv[i][4] = __float_as_uint(fmaf(hi.x, 0.5f, __uint_as_float(sv[i][4])));
              sv[i][5] = __float_as_uint(fmaf(hi.y, 0.5f, __uint_as_float(sv[i][5])));
              sv[i][6] = __float_as_uint(fmaf(hi.x, 0.5f, __uint_as_float(sv[i][6])));
              sv[i][7] = __float_as_uint(fmaf(hi.y, 0.5f, __uint_as_float(sv[i][7])));
            }
          }
          if (kGated && pass == 1) {
            // this warp holds all its S values: the S buffer may be refilled for the next group
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(s_free_addr);
          }
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int pc = pass * 2 + i;
            float* d0 = dacc[pc * 2];
            float* d1 = dacc[pc * 2 + 1];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              // pair e of the fragment: (row, cols) as in the accumulator layout; e >> 1 selects columns + 8
              float x0 = __uint_as_float(dh[i][2 * e]), x1 = __uint_as_float(dh[i][2 * e + 1]);
              if (DROP && kGated) {
                x0 *= dctx.mul(e & 1, pc * 16 + (e >> 1) * 8);
                x1 *= dctx.mul(e & 1, pc * 16 + (e >> 1) * 8 + 1);
              }
              if (kGated) {
                float* d = (e >> 1) ? d1 : d0;
                const float h0 = __uint_as_float(sv[i][2 * e]), h1 = __uint_as_float(sv[i][2 * e + 1]);
                if (gate_in_f32<DT>()) {
                  dsf[i][e] = gate_bwd_pair_f32<DT, GATE>(af[i][e], h0, h1, x0, x1, d[(e & 1) * 2], d[(e & 1) * 2 + 1]);
                } else {
#if PRISM_K2_CVT_HW
                  const uint32_t hs = Pk<DT>::cvt_hw(h0, h1);
#else
                  const uint32_t hs = Pk<DT>::cvt(h0, h1);
#endif
                  dsf[i][e] = gate_bwd_pair<DT, GATE>(af[i][e], hs, x0, x1, d[(e & 1) * 2], d[(e & 1) * 2 + 1]);
                }
              } else {
                dsf[i][e] = Pk<DT>::cvt(x0, x1);
              }
            }
          }
#pragma unroll
          for (int i = 0; i < 2; ++i)
            stmatrix_x4(tileDS + sw128_offset(a_row, (pass * 2 + i) * 2 + (mat >> 1)), dsf[i]);
          if (IB && kGated) {
            // column sums of (2 dS) over this warp's 16 token rows: rows r and r+8 of the thread, then the
            // 8 lane groups; lanes 0-3 end up with columns 2 lane + {0,1} (+8) of each piece
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const float2 p0 = Elem<DT>::unpack(dsf[i][0]), p1 = Elem<DT>::unpack(dsf[i][1]);
              const float2 p2 = Elem<DT>::unpack(dsf[i][2]), p3 = Elem<DT>::unpack(dsf[i][3]);
              float c0 = p0.x + p1.x, c1 = p0.y + p1.y, c2 = p2.x + p3.x, c3 = p2.y + p3.y;
#pragma unroll
              for (int sh = 4; sh <= 16; sh <<= 1) {
                c0 += __shfl_xor_sync(0xffffffffu, c0, sh);
                c1 += __shfl_xor_sync(0xffffffffu, c1, sh);
                c2 += __shfl_xor_sync(0xffffffffu, c2, sh);
                c3 += __shfl_xor_sync(0xffffffffu, c3, sh);
              }
              if (lane < 4) {
                float* dst = smemIb + ((gg & 1) * kNumGateWarps + gw) * 64 + (pass * 2 + i) * 16 + 2 * lane;
                dst[0] = c0; dst[1] = c1; dst[8] = c2; dst[9] = c3;
              }
            }
          }
        }
        if (IB && kGated) {
          // the 8 warps of this 64-feature chunk (one per 16-token row group) are added in a fixed order
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->ib_full[gg & 1]);
          if (!mbar_wait(&bars->ib_full[gg & 1], (gg >> 1) & 1)) { ok = false; break; }
          if (lane < 8) {
            const int rid = gw & 7, col = rid * 8 + lane;
            const float* src = smemIb + ((gg & 1) * kNumGateWarps + ch * 8) * 64 + col;
            float tsum = 0.f;
#pragma unroll
            for (int r = 0; r < 8; ++r) tsum += src[r * 64];
            if (f0 + ch * 64 + col < p.K) {
              float* dst = part_ib + (long long)g * u.ld + ch * 64 + col;
              if (u.first) *dst = tsum;
              else asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst), "f"(tsum) : "memory");
            }
          }
        }
        fence_proxy_async_smem();   // dS is read by the dS . R MMAs through the async proxy
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->ds_full[hb]);                     // this CTA's dR warps
          mbar_arrive_cluster(gate_done_addr + hb * 8);        // the MMA issuer: dS written, dH and S consumed
        }
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->a_empty);   // this warp no longer reads the A tile
      // tile epilogue: dA = scale * (dS . R sums from TMEM + gate term), written straight from the fragments
      if (!mbar_wait(&bars->da_full, tile_iter & 1)) { ok = false; break; }
      tc_fence_after_sync();
      const long long grow = (long long)mt * 128 + r0 + (lane >> 2);
      uint16_t* out = reinterpret_cast<uint16_t*>(p.dA);
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) {
        uint32_t v[8];
        tmem_ld_16x256b_x2(tmem_base + lane_base + kDaCol0 + ch * 64 + pc * 16, v);
        tmem_ld_wait();
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {   // columns 0-7 / 8-15 of the piece
          const int nt = pc * 2 + hh;
          const int col = f0 + ch * 64 + nt * 8 + (lane & 3) * 2;
          if (col < p.K) {
            if (grow < p.M)
              *reinterpret_cast<uint32_t*>(out + grow * p.ldda + col) =
                  Elem<DT>::pack((dacc[nt][0] + __uint_as_float(v[hh * 4 + 0])) * p.scale,
                                 (dacc[nt][1] + __uint_as_float(v[hh * 4 + 1])) * p.scale);
            if (grow + 8 < p.M)
              *reinterpret_cast<uint32_t*>(out + (grow + 8) * p.ldda + col) =
                  Elem<DT>::pack((dacc[nt][2] + __uint_as_float(v[hh * 4 + 2])) * p.scale,
                                 (dacc[nt][3] + __uint_as_float(v[hh * 4 + 3])) * p.scale);
          }
          dacc[nt][0] = dacc[nt][1] = dacc[nt][2] = dacc[nt][3] = 0.f;
        }
      }
      tc_fence_before_sync();   // the TMEM reads are done before the next tile's first dS . R overwrites dA
    }
    if (!ok && lane == 0) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
  } else if (is_dr) {
    // ------------------------------------------------------------------ dR warps
    const int w = (warp < kGateWarp0) ? (warp - 2) : (warp - kGateWarp0 - kNumGateWarps + 2);
    constexpr int spb = KS * KS;                 // 16x16 sub-tiles per rotation block
    constexpr int n_sub = (128 / E) * spb;       // sub-tiles of this CTA's 128 features
    const int mat = lane >> 3, l8 = lane & 7;
    bool ok = true;
    uint32_t tile_iter = 0, gg = 0;
    for (int k = 0; k < n_units && ok; ++k, ++tile_iter) {
      const DadrUnit tu = dadr_unit(p, pidx, (int)rank, k);
      const int f0 = tu.f0;
      const bool first = tu.first;
      if (!mbar_wait(&bars->a_full, tile_iter & 1)) { ok = false; break; }
      for (int g = 0; g < G && ok; ++g, ++gg) {
        const int buf = gg & 1;
        if (!mbar_wait(&bars->ds_full[buf], (gg >> 1) & 1)) { ok = false; break; }
        for (int u = w; u < n_sub; u += kNumDrWarps) {
          const int block = u / spb, rem = u - block * spb;
          const int is = rem / KS, js = rem - is * KS;
          const int chunk = block / NB, b = block - chunk * NB;
          const uint32_t ds_tile = smem_u32(smemDS + buf * 2 * kTile + chunk * kTile);
          const uint32_t a_tile = smem_u32(smemA + chunk * kTile);
          const uint32_t ci = (b * E + is * 16) / 8;   // 16-byte chunk of the dS columns (i)
          const uint32_t cj = (b * E + js * 16) / 8;   // 16-byte chunk of the A columns (j)
          // Four token steps at a time: all eight fragment loads first, then the MMAs on two independent
          // accumulator pairs, so that a warp does not sit through one shared-memory and one tensor-pipe
          // latency per step (the legacy tensor path only gets the gaps that tcgen05.mma leaves).
          float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
          float e0[4] = {0.f, 0.f, 0.f, 0.f}, e1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int k4 = 0; k4 < 8; k4 += 4) {
            uint32_t af[4][4], bf[4][4];
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const int ks = k4 + kk;
              // A operand (i x tok) = dS^T: matrices (i-lo,tok-lo) (i-hi,tok-lo) (i-lo,tok-hi) (i-hi,tok-hi)
              const uint32_t tok_a = ks * 16 + l8 + ((mat & 2) ? 8 : 0);
              ldmatrix_x4_trans(ds_tile + sw128_offset(tok_a, ci + (mat & 1)), af[kk]);
              // B operand (tok x j) = A: matrices (tok-lo,j-lo) (tok-hi,j-lo) (tok-lo,j-hi) (tok-hi,j-hi)
              const uint32_t tok_b = ks * 16 + l8 + ((mat & 1) ? 8 : 0);
              ldmatrix_x4_trans(a_tile + sw128_offset(tok_b, cj + (mat >> 1)), bf[kk]);
            }
#pragma unroll
            for (int kk = 0; kk < 4; kk += 2) {
              mma_m16n8k16<DT>(d0, af[kk], bf[kk][0], bf[kk][1]);
              mma_m16n8k16<DT>(d1, af[kk], bf[kk][2], bf[kk][3]);
              mma_m16n8k16<DT>(e0, af[kk + 1], bf[kk + 1][0], bf[kk + 1][1]);
              mma_m16n8k16<DT>(e1, af[kk + 1], bf[kk + 1][2], bf[kk + 1][3]);
            }
          }
#pragma unroll
          for (int x = 0; x < 4; ++x) { d0[x] += e0[x]; d1[x] += e1[x]; }
          // Accumulate into this CTA's partial buffer.  Every address has exactly one writer thread,
          // which stores on its first token tile and afterwards issues fire-and-forget fp32 reductions
          // in token-tile order: same-address operations of one thread stay ordered, so the sum is
          // formed in a fixed order (bit-stable) without waiting for a read-modify-write round trip.
          const int rr0 = g * E + is * 16 + (lane >> 2);
          const int lc = chunk * 64 + b * E + js * 16 + (lane & 3) * 2;   // column inside the tile's 128
          const int col = f0 + lc;
          if (col < p.K) {
            dr_accumulate(tu.part + (long long)rr0 * tu.ld + lc, d0[0], d0[1], first);
            dr_accumulate(tu.part + (long long)(rr0 + 8) * tu.ld + lc, d0[2], d0[3], first);
          }
          if (col + 8 < p.K) {
            dr_accumulate(tu.part + (long long)rr0 * tu.ld + lc + 8, d1[0], d1[1], first);
            dr_accumulate(tu.part + (long long)(rr0 + 8) * tu.ld + lc + 8, d1[2], d1[3], first);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->ds_empty[buf]);
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->a_empty);
    }
    if (!ok && lane == 0) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
  }

  // neither CTA may leave (or free TMEM) while its peer can still reach its barriers or shared memory
  tc_fence_before_sync();
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
  if (warp == kWarpMma) tmem_dealloc_pair(tmem_base, 512);
}

using DadrKernel = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, DadrParams, DadrExtra);
// kernel instance for (gate, E, internal-bias variant), one function per data type and translation unit
DadrKernel dadr_kernel_f16(int gate, int E, bool ib, bool drop);
DadrKernel dadr_kernel_bf16(int gate, int E, bool ib, bool drop);

#define PRISM_DADR_PICK_IB(DT_, G_, E_, DROP_) \
  (ib ? (DadrKernel)prism_bwd_dadr_kernel<DT_, G_, E_, true, DROP_> : (DadrKernel)prism_bwd_dadr_kernel<DT_, G_, E_, false, DROP_>)
#define PRISM_DADR_PICK_G(DT_, E_, DROP_)                                                        \
  (gate == GATE_SILU ? PRISM_DADR_PICK_IB(DT_, GATE_SILU, E_, DROP_)                              \
   : gate == GATE_SIGMOID ? PRISM_DADR_PICK_IB(DT_, GATE_SIGMOID, E_, DROP_)                      \
                          : (DadrKernel)prism_bwd_dadr_kernel<DT_, GATE_NONE, E_, false, false>)
// dropout kernels exist for E = 16 (reconn_sz 8 and 16) only
#define PRISM_DADR_DEFINE_PICKER(NAME_, DT_)                                  \
  DadrKernel NAME_(int gate, int E, bool ib, bool drop) {                     \
    if (drop) return PRISM_DADR_PICK_G(DT_, 16, true);                        \
    if (E == 16) return PRISM_DADR_PICK_G(DT_, 16, false);                    \
    if (E == 32) return PRISM_DADR_PICK_G(DT_, 32, false);                    \
    return PRISM_DADR_PICK_G(DT_, 64, false);                                 \
  }

}  // namespace prism
