// Prism backward, input and rotation gradients, for sm_100a:
//   dH_g = dC_g . B_g                                   (dense, tcgen05, fp32 in TMEM)
//   S_g  = A . blockdiag(R_g)^T                         (recomputed, mma.sync)
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
// One CTA works on its [128 tokens x 128 features] tile of dA and walks over all groups:
//   warp 0       TMA producer: A tiles once per tile; per group the R_g tiles and, per 64 outputs,
//                two dC tiles [128 x 64] and this CTA's B_g tile [128 x 64]
//   warp 1       dense issuer (leader CTA): dH_g = dC_g . B_g as tcgen05.mma M256 N128 K16 (dC K-major, B_g
//                MN-major) into a ring of four 128-column TMEM buffers
//   warps 4-19   gate warps, 16 tokens x 64 features each: dH fragments straight from TMEM
//                (tcgen05.ld.16x256b delivers the mma.sync accumulator layout), A and R fragments by
//                ldmatrix, S by mma.sync; dS on registers -> stmatrix to shared memory for the dR
//                warps and, as the A operand of a second mma.sync, dA += dS . R_g; dA lives in
//                fp32 accumulator fragments for the whole tile
//   warps 2,3,20,21  dR warps: ldmatrix.trans of the dS and A tiles, mma.sync over the 128 tokens,
//                read-modify-write of this CTA's fp32 partial buffer.
#include "prism_host.cuh"
#include "prism_kernels.cuh"

#ifndef PRISM_DBG
#define PRISM_DBG 0   // debugging aid: bit 0 skips the gate warps' work, bit 1 the dR warps' work
#endif

namespace prism {

namespace dadr {
constexpr int kThreads = 704;
constexpr int kWarpTma = 0, kWarpMma = 1;
constexpr int kGateWarp0 = 4;      // multiple of 4: (warp & 3) is the TMEM lane quarter
constexpr int kNumGateWarps = 16;
constexpr int kNumDrWarps = 4;     // warps 2, 3, 20, 21
constexpr int kDhBufs = 4;         // TMEM ring of dH buffers, 128 columns each
constexpr int kTile = 128 * 128;   // bytes of a [128 x 64] 16-bit tile
#ifndef PRISM_DADR_STAGE_OUT
#define PRISM_DADR_STAGE_OUT 128
#endif
// one stage = kStageOut outputs of the group: kStageOut/64 dC tiles [128 tokens x 64] and this CTA's
// half of the B_g features, a [kStageOut outputs x 64 features] tile
constexpr int kStageOut = PRISM_DADR_STAGE_OUT;
constexpr int kDcTiles = kStageOut / 64;
constexpr int kBTile = kStageOut * 128;
constexpr int kStageBytes = kDcTiles * kTile + kBTile;
constexpr int kMaxStages = 6;
constexpr int kMaxRBufs = 4;
}  // namespace dadr

struct DadrParams {
  int M, N, K, gs, E, G;
  int n_mtiles, runs;
  int ns, rb;          // stages of the dC/B ring, number of R buffers
  int r_tile_bytes;    // bytes reserved per [E x 64] R tile (multiple of 1024)
  float scale;
  void* dA;
  long long ldda;
  float* partial;      // [2*runs][G*E][K] fp32: one buffer per CTA of every pair
  int* err;
};

struct DadrBarriers {
  uint64_t a_full, a_empty;
  uint64_t r_full[dadr::kMaxRBufs], r_empty[dadr::kMaxRBufs];
  uint64_t st_full[dadr::kMaxStages], st_empty[dadr::kMaxStages];
  uint64_t dh_full[dadr::kDhBufs], dh_empty[dadr::kDhBufs];
  uint64_t ds_full[2], ds_empty[2];
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
// the dR reduction) and p = dh silu(S), the gate term of dA, both packed 16-bit.
template <int DT>
__device__ __forceinline__ uint32_t gate_bwd_pair(uint32_t a2, uint32_t hs, float dh0, float dh1, uint32_t& p) {
  const uint32_t t = Pk<DT>::tanh(hs);
  const uint32_t g = Pk<DT>::fma(hs, t, hs);
  const uint32_t w = Pk<DT>::fma(g, Pk<DT>::kNegOne, Pk<DT>::kOne);
  const uint32_t x = Pk<DT>::fma(t, w, g);
  const uint32_t d = Pk<DT>::cvt(dh0, dh1);
  p = Pk<DT>::mul(d, g);
  const uint32_t q = Pk<DT>::mul(d, a2);
  return Pk<DT>::fma(q, x, q);
}

template <int DT, int GATE, int E>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(dadr::kThreads, 1)
prism_bwd_dadr_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmR,
                      const __grid_constant__ CUtensorMap tmdC, const __grid_constant__ CUtensorMap tmB,
                      const DadrParams p) {
  using namespace dadr;
  constexpr int KS = E / 16;       // 16-wide steps per rotation block
  constexpr int NB = 64 / E;       // rotation blocks per 64-column tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  const int r_buf_bytes = 2 * p.r_tile_bytes;
  uint8_t* smemA = smem;                        // 2 tiles [128 x 64]
  uint8_t* smemDS = smemA + 2 * kTile;          // 2 buffers x 2 tiles [128 x 64]
  uint8_t* smemR = smemDS + 4 * kTile;          // rb buffers x 2 tiles [E x 64]
  uint8_t* smemSt = smemR + p.rb * r_buf_bytes; // ns stages: dC tile + 2 B tiles
  DadrBarriers* bars = reinterpret_cast<DadrBarriers*>(smemSt + p.ns * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0 = leader (issues the MMAs), 1 = peer
  const int f0 = (blockIdx.x >> 1) * 128;    // the pair's 128 features
  const int run = blockIdx.y;                // the pair walks token-tile pairs run, run + runs, ...
  const int n_mpairs = (p.n_mtiles + 1) / 2;
  const int G = p.G;
  const int nstg = (p.gs + kStageOut - 1) / kStageOut;  // stages per group
  const bool is_gate = warp >= kGateWarp0 && warp < kGateWarp0 + kNumGateWarps;
  const bool is_dr = warp == 2 || warp == 3 || warp >= kGateWarp0 + kNumGateWarps;

  if (threadIdx.x == 0) {
    mbar_init(&bars->a_full, 1);
    mbar_init(&bars->a_empty, kNumGateWarps + kNumDrWarps);
    for (int i = 0; i < kMaxRBufs; ++i) { mbar_init(&bars->r_full[i], 1); mbar_init(&bars->r_empty[i], kNumGateWarps); }
    // st_full and dh_empty are used in the leader's copy only and count both CTAs
    for (int i = 0; i < kMaxStages; ++i) { mbar_init(&bars->st_full[i], 2); mbar_init(&bars->st_empty[i], 1); }
    for (int i = 0; i < kDhBufs; ++i) { mbar_init(&bars->dh_full[i], 1); mbar_init(&bars->dh_empty[i], 2 * kNumGateWarps); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars->ds_full[i], kNumGateWarps); mbar_init(&bars->ds_empty[i], kNumDrWarps); }
    fence_mbar_init();
  }
  if (warp == kWarpMma) {
    tmem_alloc_pair(&bars->tmem_base, 512);
    tmem_relinquish_pair();
  }
  if (warp == kWarpTma && lane == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmR);
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
    if (lane == 0) {
      bool ok = true;
      uint32_t tile_iter = 0;
      Ring rr(p.rb), rst(p.ns);
      for (int mp = run; mp < n_mpairs && ok; mp += p.runs, ++tile_iter) {
        const int m0 = (mp * 2 + (int)rank) * 128;
        if (!mbar_wait(&bars->a_empty, (tile_iter & 1) ^ 1)) { ok = false; break; }
        mbar_arrive_expect_tx(&bars->a_full, 2 * kTile);
        tma_load_2d(smemA, &tmA, &bars->a_full, f0, m0);
        tma_load_2d(smemA + kTile, &tmA, &bars->a_full, f0 + 64, m0);
        for (int g = 0; g < G && ok; ++g, rr.next()) {
          const int rb = rr.idx;
          if (!mbar_wait(&bars->r_empty[rb], rr.phase ^ 1)) { ok = false; break; }
          uint8_t* dstR = smemR + rb * r_buf_bytes;
          mbar_arrive_expect_tx(&bars->r_full[rb], 2 * E * 128);
          tma_load_2d(dstR, &tmR, &bars->r_full[rb], f0, g * E);
          tma_load_2d(dstR + p.r_tile_bytes, &tmR, &bars->r_full[rb], f0 + 64, g * E);
          for (int s = 0; s < nstg; ++s, rst.next()) {
            const int st = rst.idx;
            if (!mbar_wait(&bars->st_empty[st], rst.phase ^ 1)) { ok = false; break; }
            uint8_t* dst = smemSt + st * kStageBytes;
            const int n0 = g * p.gs + s * kStageOut;
            const bool two = kDcTiles == 2 && p.gs - s * kStageOut > 64;   // the slice has more than 64 outputs
            // completion is counted on the leader's barrier: its MMAs read both CTAs' tiles
            const uint32_t stfull = mapa_shared(smem_u32(&bars->st_full[st]), 0);
            mbar_arrive_expect_tx_cluster(stfull, (two ? 2 : 1) * kTile + kBTile);
            tma_load_2d_pair(dst, &tmdC, stfull, n0, m0);
            if (two) tma_load_2d_pair(dst + kTile, &tmdC, stfull, n0 + 64, m0);
            tma_load_2d_pair(dst + kDcTiles * kTile, &tmB, stfull, f0 + (int)rank * 64, n0);
          }
        }
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ dense issuer: dH = dC . B
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_h = make_idesc(DT, 256, 128, 0, 1);   // M = 256 tokens; dC K-major, B_g MN-major
      // descriptors of stage 0; a stage further on adds kStageBytes >> 4 to the low words
      const uint64_t da0 = desc_kmajor_sw128(smem_u32(smemSt), 1024);
      const uint64_t db0 = desc_mnmajor_sw128(smem_u32(smemSt) + kDcTiles * kTile, kBTile, 1024);
      const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
      bool ok = true;
      uint32_t gg = 0;
      Ring rst(p.ns);
      for (int mp = run; mp < n_mpairs && ok; mp += p.runs) {
        for (int g = 0; g < G && ok; ++g, ++gg) {
          const uint32_t hb = gg & (kDhBufs - 1);
          const uint32_t d_tmem = tmem_base + hb * 128;
          if (!mbar_wait_cluster(&bars->dh_empty[hb], ((gg / kDhBufs) & 1) ^ 1)) { ok = false; break; }
          for (int s = 0; s < nstg; ++s, rst.next()) {
            const int st = rst.idx;
            if (!mbar_wait_cluster(&bars->st_full[st], rst.phase)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t a_lo = (uint32_t)da0 + st * (kStageBytes >> 4);
            const uint32_t b_lo = (uint32_t)db0 + st * (kStageBytes >> 4);
            constexpr int kSteps = kStageOut / 16;
            const int ksteps = min(kSteps, (p.gs - s * kStageOut) / 16);
            if (ksteps == kSteps) {
              // K16 step ks: dC tile ks/4 (+kTile), 32 bytes per step inside it; B_g rows 16 ks (+2048 bytes)
              umma_f16_pair_lh(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc_h, s > 0 ? 1u : 0u);
#pragma unroll
              for (int ks = 1; ks < kSteps; ++ks)
                umma_f16_pair_lh(d_tmem, a_lo + (((ks >> 2) * kTile + (ks & 3) * 32) >> 4), a_hi,
                                 b_lo + ((ks * 2048) >> 4), b_hi, idesc_h, 1u);
            } else {
              for (int ks = 0; ks < ksteps; ++ks)
                umma_f16_pair_lh(d_tmem, a_lo + (((ks >> 2) * kTile + (ks & 3) * 32) >> 4), a_hi,
                                 b_lo + ((ks * 2048) >> 4), b_hi, idesc_h, (s > 0 || ks > 0) ? 1u : 0u);
            }
            umma_commit_pair(&bars->st_empty[st], 0x3);
          }
          if (!ok) break;
          umma_commit_pair(&bars->dh_full[hb], 0x3);
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
    const uint32_t a_row = r0 + l8 + (mat & 1) * 8;            // A-operand fragments (also dS stores)
    const uint32_t rn_row = l8 + (mat >> 1) * 8;               // R as B operand of S = A . R^T (rows = i)
    const uint32_t rt_row = l8 + (mat & 1) * 8;                // R as B operand of dS . R (rows = i, transposed load)
    const uint32_t tileA = smem_u32(smemA + ch * kTile);
    // B-operand fragment of a 16x16 identity (the k = n diagonal of one 8-column half): adds the gate
    // term p to the accumulators through the tensor pipe instead of unpack + FMA instructions
    const uint32_t idf = ((lane >> 3) == (lane & 3)) ? (((lane >> 2) & 1) ? (Pk<DT>::kOneLo << 16) : Pk<DT>::kOneLo) : 0u;
    float dacc[8][4];   // dA accumulator fragments: 16 rows x 64 columns of this warp, whole tile
#pragma unroll
    for (int i = 0; i < 8; ++i) { dacc[i][0] = dacc[i][1] = dacc[i][2] = dacc[i][3] = 0.f; }
    bool ok = true;
    uint32_t tile_iter = 0, gg = 0;
    Ring rr(p.rb);
    for (int mp = run; mp < n_mpairs && ok; mp += p.runs, ++tile_iter) {
      const int mt = mp * 2 + (int)rank;
      if (!mbar_wait(&bars->a_full, tile_iter & 1)) { ok = false; break; }
      for (int g = 0; g < G && ok; ++g, ++gg, rr.next()) {
        const uint32_t hb = gg & (kDhBufs - 1), db = gg & 1;
        if (!mbar_wait(&bars->r_full[rr.idx], rr.phase)) { ok = false; break; }
        if (!mbar_wait(&bars->dh_full[hb], (gg / kDhBufs) & 1)) { ok = false; break; }
        if (!mbar_wait(&bars->ds_empty[db], ((gg >> 1) & 1) ^ 1)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tileDS = smem_u32(smemDS + db * 2 * kTile + ch * kTile);
        const uint32_t rtile = smem_u32(smemR + rr.idx * r_buf_bytes + ch * p.r_tile_bytes);
        const uint32_t tdh = tmem_base + lane_base + hb * 128 + ch * 64;
#pragma unroll
        for (int b = 0; b < ((PRISM_DBG & 1) ? 0 : NB); ++b) {
          uint32_t af[KS][4], dsf[KS][4], pf[KS][4];
          if (GATE == GATE_SILU) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
              ldmatrix_x4(tileA + sw128_offset(a_row, b * (E / 8) + ks * 2 + (mat >> 1)), af[ks]);
          }
#pragma unroll
          for (int np = 0; np < KS; ++np) {
            uint32_t dh[8];
            tmem_ld_16x256b_x2(tdh + b * E + np * 16, dh);
            uint32_t sp[4] = {0u, 0u, 0u, 0u};   // packed S/2 of this thread's four pairs (the R tile holds R/2)
            if (GATE == GATE_SILU) {
              if (DT == DT_F16) {
                uint32_t c0[2] = {0u, 0u}, c1[2] = {0u, 0u};   // fp16 accumulation: packed result
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                  uint32_t rf[4];
                  ldmatrix_x4(rtile + sw128_offset(np * 16 + rn_row, b * (E / 8) + ks * 2 + (mat & 1)), rf);
                  mma_m16n8k16_f16acc(c0, af[ks], rf[0], rf[1]);
                  mma_m16n8k16_f16acc(c1, af[ks], rf[2], rf[3]);
                }
                sp[0] = c0[0]; sp[1] = c0[1]; sp[2] = c1[0]; sp[3] = c1[1];
              } else {
                float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                  uint32_t rf[4];
                  ldmatrix_x4(rtile + sw128_offset(np * 16 + rn_row, b * (E / 8) + ks * 2 + (mat & 1)), rf);
                  mma_m16n8k16<DT>(c0, af[ks], rf[0], rf[1]);
                  mma_m16n8k16<DT>(c1, af[ks], rf[2], rf[3]);
                }
                sp[0] = Pk<DT>::cvt(c0[0], c0[1]); sp[1] = Pk<DT>::cvt(c0[2], c0[3]);
                sp[2] = Pk<DT>::cvt(c1[0], c1[1]); sp[3] = Pk<DT>::cvt(c1[2], c1[3]);
              }
            }
            tmem_ld_wait();
            if (GATE == GATE_SILU) {
              dsf[np][0] = gate_bwd_pair<DT>(af[np][0], sp[0], __uint_as_float(dh[0]), __uint_as_float(dh[1]), pf[np][0]);
              dsf[np][1] = gate_bwd_pair<DT>(af[np][1], sp[1], __uint_as_float(dh[2]), __uint_as_float(dh[3]), pf[np][1]);
              dsf[np][2] = gate_bwd_pair<DT>(af[np][2], sp[2], __uint_as_float(dh[4]), __uint_as_float(dh[5]), pf[np][2]);
              dsf[np][3] = gate_bwd_pair<DT>(af[np][3], sp[3], __uint_as_float(dh[6]), __uint_as_float(dh[7]), pf[np][3]);
            } else {
              dsf[np][0] = Pk<DT>::cvt(__uint_as_float(dh[0]), __uint_as_float(dh[1]));
              dsf[np][1] = Pk<DT>::cvt(__uint_as_float(dh[2]), __uint_as_float(dh[3]));
              dsf[np][2] = Pk<DT>::cvt(__uint_as_float(dh[4]), __uint_as_float(dh[5]));
              dsf[np][3] = Pk<DT>::cvt(__uint_as_float(dh[6]), __uint_as_float(dh[7]));
            }
            stmatrix_x4(tileDS + sw128_offset(a_row, b * (E / 8) + np * 2 + (mat >> 1)), dsf[np]);
          }
          // dA[:, block b] += p + dS[:, block b] . R_g[block b]   (contraction over the block's i)
#pragma unroll
          for (int jp = 0; jp < KS; ++jp) {
            if (GATE == GATE_SILU) {
              mma_m16n8k16<DT>(dacc[(b * KS + jp) * 2], pf[jp], idf, 0u);
              mma_m16n8k16<DT>(dacc[(b * KS + jp) * 2 + 1], pf[jp], 0u, idf);
            }
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
              uint32_t rt[4];
              ldmatrix_x4_trans(rtile + sw128_offset(ks * 16 + rt_row, b * (E / 8) + jp * 2 + (mat >> 1)), rt);
              mma_m16n8k16<DT>(dacc[(b * KS + jp) * 2], dsf[ks], rt[0], rt[1]);
              mma_m16n8k16<DT>(dacc[(b * KS + jp) * 2 + 1], dsf[ks], rt[2], rt[3]);
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->ds_full[db]);
          mbar_arrive_cluster(mapa_shared(smem_u32(&bars->dh_empty[hb]), 0));
          mbar_arrive(&bars->r_empty[rr.idx]);
        }
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->a_empty);   // this warp no longer reads the A tile
      // tile epilogue: dA = scale * accumulators, written straight from the fragments
      const long long grow = (long long)mt * 128 + r0 + (lane >> 2);
      uint16_t* out = reinterpret_cast<uint16_t*>(p.dA);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int col = f0 + ch * 64 + nt * 8 + (lane & 3) * 2;
        if (col < p.K) {
          if (grow < p.M)
            *reinterpret_cast<uint32_t*>(out + grow * p.ldda + col) = Elem<DT>::pack(dacc[nt][0] * p.scale, dacc[nt][1] * p.scale);
          if (grow + 8 < p.M)
            *reinterpret_cast<uint32_t*>(out + (grow + 8) * p.ldda + col) = Elem<DT>::pack(dacc[nt][2] * p.scale, dacc[nt][3] * p.scale);
        }
        dacc[nt][0] = dacc[nt][1] = dacc[nt][2] = dacc[nt][3] = 0.f;
      }
    }
    if (!ok && lane == 0) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
  } else if (is_dr) {
    // ------------------------------------------------------------------ dR warps
    const int w = (warp < kGateWarp0) ? (warp - 2) : (warp - kGateWarp0 - kNumGateWarps + 2);
    constexpr int spb = KS * KS;                 // 16x16 sub-tiles per rotation block
    constexpr int n_sub = (128 / E) * spb;       // sub-tiles of this CTA's 128 features
    const int mat = lane >> 3, l8 = lane & 7;
    const long long GE = (long long)G * E;
    float* part = p.partial + (long long)(run * 2 + (int)rank) * GE * p.K;
    bool ok = true;
    uint32_t tile_iter = 0, gg = 0;
    for (int mp = run; mp < n_mpairs && ok; mp += p.runs, ++tile_iter) {
      if (!mbar_wait(&bars->a_full, tile_iter & 1)) { ok = false; break; }
      for (int g = 0; g < G && ok; ++g, ++gg) {
        const int buf = gg & 1;
        if (!mbar_wait(&bars->ds_full[buf], (gg >> 1) & 1)) { ok = false; break; }
        for (int u = w; u < ((PRISM_DBG & 2) ? 0 : n_sub); u += kNumDrWarps) {
          const int block = u / spb, rem = u - block * spb;
          const int is = rem / KS, js = rem - is * KS;
          const int chunk = block / NB, b = block - chunk * NB;
          const uint32_t ds_tile = smem_u32(smemDS + buf * 2 * kTile + chunk * kTile);
          const uint32_t a_tile = smem_u32(smemA + chunk * kTile);
          const uint32_t ci = (b * E + is * 16) / 8;   // 16-byte chunk of the dS columns (i)
          const uint32_t cj = (b * E + js * 16) / 8;   // 16-byte chunk of the A columns (j)
          float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            // A operand (i x tok) = dS^T: matrices (i-lo,tok-lo) (i-hi,tok-lo) (i-lo,tok-hi) (i-hi,tok-hi)
            const uint32_t tok_a = ks * 16 + l8 + ((mat & 2) ? 8 : 0);
            uint32_t af[4];
            ldmatrix_x4_trans(ds_tile + sw128_offset(tok_a, ci + (mat & 1)), af);
            // B operand (tok x j) = A: matrices (tok-lo,j-lo) (tok-hi,j-lo) (tok-lo,j-hi) (tok-hi,j-hi)
            const uint32_t tok_b = ks * 16 + l8 + ((mat & 1) ? 8 : 0);
            uint32_t bf[4];
            ldmatrix_x4_trans(a_tile + sw128_offset(tok_b, cj + (mat >> 1)), bf);
            mma_m16n8k16<DT>(d0, af, bf[0], bf[1]);
            mma_m16n8k16<DT>(d1, af, bf[2], bf[3]);
          }
          // Accumulate into this CTA's partial buffer.  Every address has exactly one writer thread,
          // which stores on its first token tile and afterwards issues fire-and-forget fp32 reductions
          // in token-tile order: same-address operations of one thread stay ordered, so the sum is
          // formed in a fixed order (bit-stable) without waiting for a read-modify-write round trip.
          const int rr0 = g * E + is * 16 + (lane >> 2);
          const int col = f0 + chunk * 64 + b * E + js * 16 + (lane & 3) * 2;
          if (col < p.K) {
            dr_accumulate(part + (long long)rr0 * p.K + col, d0[0], d0[1], tile_iter == 0);
            dr_accumulate(part + (long long)(rr0 + 8) * p.K + col, d0[2], d0[3], tile_iter == 0);
          }
          if (col + 8 < p.K) {
            dr_accumulate(part + (long long)rr0 * p.K + col + 8, d1[0], d1[1], tile_iter == 0);
            dr_accumulate(part + (long long)(rr0 + 8) * p.K + col + 8, d1[2], d1[3], tile_iter == 0);
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

// dR[g*rs + i, k] = cast( scale * sum_run partial[run][g*E + i'][k] ), runs in increasing order.
// For rs = 8 two neighbouring blocks share one 16-row group of the partial buffer:
// the block in the upper 8 columns of each 16-column pair sits in rows 8..15.
template <int DT>
__global__ void dr_reduce_kernel(const float* __restrict__ partial, uint16_t* __restrict__ dR, int G,
                                 int rs, int E, int K, long long lddr, int runs, float scale) {
  const long long pair = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)G * rs * K / 2;
  if (pair >= total) return;
  const long long idx = pair * 2;
  const int k = (int)(idx % K);
  const int row = (int)(idx / K);
  const int g = row / rs, i = row - g * rs;
  int ip = i;
  if (rs == 8) ip = i + (((k & 15) >= 8) ? 8 : 0);
  const long long GE = (long long)G * E;
  float2 acc = make_float2(0.f, 0.f);
  for (int r = 0; r < runs; ++r) {
    const float2 v = *reinterpret_cast<const float2*>(partial + ((long long)r * GE + (long long)g * E + ip) * K + k);
    acc.x += v.x;
    acc.y += v.y;
  }
  *reinterpret_cast<uint32_t*>(dR + (long long)row * lddr + k) = Elem<DT>::pack(acc.x * scale, acc.y * scale);
}

// Number of CTA pairs that share one 128-feature column of dA (each pair walks every runs-th
// 256-token tile).  Picks the count that minimises (waves of pairs over the SM pairs) x (tiles per
// pair); ties go to the smaller count, which needs less workspace.
int dadr_default_runs(int M, int K, int num_sms) {
  const int n_ft = (K + 127) / 128;
  const int n_mp = (M + 255) / 256;
  const int slots = num_sms / 2 > 0 ? num_sms / 2 : 1;
  int best = 1;
  long long best_cost = -1;
  for (int r = 1; r <= n_mp && r <= 32; ++r) {
    const long long waves = ((long long)n_ft * r + slots - 1) / slots;
    const long long cost = waves * ((n_mp + r - 1) / r);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = r; }
  }
  return best;
}

int launch_bwd_dadr(const DadrArgs& a) {
  DadrParams p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.gs = a.gs; p.E = a.E; p.G = a.N / a.gs;
  p.n_mtiles = (a.M + 127) / 128;
  p.runs = a.runs < 1 ? 1 : a.runs;
  if (p.runs > (p.n_mtiles + 1) / 2) p.runs = (p.n_mtiles + 1) / 2;
  p.r_tile_bytes = ((a.E * 128) + 1023) / 1024 * 1024;
  p.scale = a.scale;
  p.dA = a.dA; p.ldda = a.ldda; p.partial = a.partial; p.err = a.err;
  p.rb = (a.E <= 16) ? 4 : (a.E == 32 ? 3 : 2);
  const int fixed = 6 * dadr::kTile + p.rb * 2 * p.r_tile_bytes + (int)sizeof(DadrBarriers) + 1024 + 256;
  int ns = (227 * 1024 - fixed) / dadr::kStageBytes;
  if (ns > dadr::kMaxStages) ns = dadr::kMaxStages;
  if (ns < 2) return fail(PRISM_ERR_UNSUPPORTED, "bwd_dadr does not fit shared memory (E=%d)", a.E);
  p.ns = ns;
  const int smem_bytes = 6 * dadr::kTile +
 p.rb * 2 * p.r_tile_bytes + ns * dadr::kStageBytes +
                         (int)sizeof(DadrBarriers) + 1024;

  CUtensorMap tmA, tmR, tmdC, tmB;
  int rc;
  if ((rc = make_tmap_2d(&tmA, a.dtype, a.A, a.M, a.K, a.lda, 128, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmR, a.dtype, a.R_eff, (uint64_t)p.G * a.E, a.K, a.ldr, a.E, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmdC, a.dtype, a.dC, a.M, a.N, a.lddc, 128, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmB, a.dtype, a.B, a.N, a.K, a.ldb, dadr::kStageOut, 64, true))) return rc;

  using KernT = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, DadrParams);
  KernT kern = nullptr;
#define PRISM_PICK(E_)                                                                               \
  kern = (a.dtype == DT_BF16)                                                                        \
             ? (a.gate == GATE_SILU ? (KernT)prism_bwd_dadr_kernel<DT_BF16, GATE_SILU, E_> : (KernT)prism_bwd_dadr_kernel<DT_BF16, GATE_NONE, E_>) \
             : (a.gate == GATE_SILU ? (KernT)prism_bwd_dadr_kernel<DT_F16, GATE_SILU, E_> : (KernT)prism_bwd_dadr_kernel<DT_F16, GATE_NONE, E_>)
  if (a.E == 16) { PRISM_PICK(16); } else if (a.E == 32) { PRISM_PICK(32); } else { PRISM_PICK(64); }
#undef PRISM_PICK
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return fail(PRISM_ERR_CUDA, "bwd_dadr: cannot set %d B of shared memory: %s", smem_bytes, cudaGetErrorString(e));
  dim3 grid(2 * ((a.K + 127) / 128), p.runs, 1);   // x: the two CTAs of a pair
  kern<<<grid, dadr::kThreads, smem_bytes, a.stream>>>(tmA, tmR, tmdC, tmB, p);
  if ((rc = check_launch("prism_bwd_dadr"))) return rc;

  // gated mode: the kernel formed 2 dS against the halved R tiles, so the dR partials are doubled
  const float r_scale = (a.gate == GATE_SILU) ? 0.5f * a.scale : a.scale;
  const long long pairs = (long long)p.G * a.rs * a.K / 2;
  const int threads = 256;
  const long long blocks = (pairs + threads - 1) / threads;
  if (a.dtype == DT_BF16)
    dr_reduce_kernel<DT_BF16><<<(unsigned)blocks, threads, 0, a.stream>>>(a.partial, reinterpret_cast<uint16_t*>(a.dR), p.G, a.rs, a.E, a.K, a.lddr, 2 * p.runs, r_scale);
  else
    dr_reduce_kernel<DT_F16><<<(unsigned)blocks, threads, 0, a.stream>>>(a.partial, reinterpret_cast<uint16_t*>(a.dR), p.G, a.rs, a.E, a.K, a.lddr, 2 * p.runs, r_scale);
  return check_launch("prism_bwd_dadr reduce");
}

}  // namespace prism
