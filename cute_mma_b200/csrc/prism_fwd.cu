// Prism forward for sm_100a:  C[:, group g] = H_g @ B_g^T  with
//   H_g = A . blockdiag(R_g)^T                 (plain / "ar" mode)
//   H_g = A * silu(A . blockdiag(R_g)^T)       (silu_gate mode)
// in one kernel; H never leaves the SM.
//
// Replaces the reference's prism_tn / prism_device forward kernel
// (cute_prism_coop_pc.cu:567-804) and its binding (torch_ext/prism_fwd_torch.cu:23-196).
//
// CTAs work in pairs (cluster of 2, tcgen05 cta_group::2) on (256-row, BN-column) output tiles: each CTA
// owns 128 of the rows and loads half of the B tile, which halves the L2 traffic per flop.  Per CTA a
// persistent loop over the pair's tiles.  One ring of shared-memory stages, one stage per 64-wide K
// chunk: the A tile [128 x 64], this CTA's half of the R_g tile [E/2 x 64] and of the B_g tile [BN/2 x 64].
//   warps 0, 2  TMA producers (A + R, B); 128-byte swizzle, zero fill outside the tensors
//   warp 1      MMA issuer (leader CTA only), per chunk
//                 rotation  S = A_blk . R_blk^T per rotation block: tcgen05.mma M256 N=E K=16, fp32 into
//                           one of four 64-column TMEM slots
//                 dense     C += H . B^T: 4 x tcgen05.mma M256 N=BN K=16 with H read from TMEM, two chunks
//                           behind the rotation
//   warps 4-19  gate warps, two groups of eight that take alternate chunks, 16 rows per warp: S from
//               TMEM (tcgen05.ld delivers the accumulator-fragment layout), A by ldmatrix (same layout),
//               H = A*silu(S) (or H = S) on registers, H back to TMEM over the first half of the S slot
//   warps 20-23 epilogue: tcgen05.ld C, + bias, cast, swizzled staging tile, TMA store.
// Both products run on tcgen05: mma.sync shares the tensor cores with tcgen05.mma and is starved
// while tcgen05.mma bursts run, so a rotation on mma.sync serialises the gate warps with the dense
// product.  The issuing thread runs alone on its instruction stream (a barrier test costs it ~65
// clocks, a tcgen05.commit ~90): descriptors advance by 32-bit adds, and there is one wait and one
// commit per product and chunk.
#include "prism_host.cuh"
#include "prism_kernels.cuh"

namespace prism {

namespace fwd {
constexpr int kThreads = 768;
constexpr int kWarpTma = 0, kWarpMma = 1, kWarpTmaB = 2, kWarpRot = 3;
constexpr int kGateWarp0 = 4;         // multiple of 4: (warp & 3) is the TMEM lane quarter a warp may touch
constexpr int kGateGroups = 2;        // groups take alternate chunks ...
constexpr int kWarpsPerGroup = 8;     // ... with 16 rows per warp
constexpr int kNumGateWarps = kGateGroups * kWarpsPerGroup;
constexpr int kEpiWarp0 = kGateWarp0 + kNumGateWarps;   // 20
constexpr int kNumEpiWarps = 4;
constexpr int kSlots = 4;             // TMEM slots of 64 columns: S (fp32), then H over its first 32 columns
constexpr int kSlotCol0 = 256;        // accumulator: TMEM columns [0, 256); slots: [256, 512)
constexpr int kMaxStages = 8;
constexpr int kATileBytes = 128 * 128;   // [128 rows x 64 elems] 16-bit
constexpr int kEpiStageBytes = 32 * 128; // per epilogue warp: [32 rows x 64 elems]
}  // namespace fwd

struct FwdParams {
  int M, N, K;
  int gs, E;            // group size, effective rotation block (16/32/64)
  int BN;               // N tile, divides gs
  int n_mtiles, n_ntiles, ntiles_per_group, n_tiles;
  int PM;               // m-tiles per rasterisation panel
  int n_kchunks;
  int ns;               // stages of the shared-memory ring
  int r_tile_bytes;     // bytes reserved for this CTA's half of the R tile (multiple of 1024)
  int stage_bytes;
  int tma_store;        // 1: epilogue goes through TMA stores (BN multiple of 64)
  const void* bias;     // [N] or null
  const void* ib;       // internal bias [G, K] or null
  const long long* drop_seeds;   // per-group dropout seeds (DROP kernels)
  float drop_p, drop_inv_keep;
  void* C;
  long long ldc;
  int* err;
};

struct FwdBarriers {
  uint64_t loads_full[fwd::kMaxStages];   // leader's copy is used: A, R, B of the stage landed in both CTAs
  uint64_t done[fwd::kMaxStages];         // local, multicast commit: the dense product has read the stage
  uint64_t s_full[fwd::kSlots];           // local, multicast commit: S of the chunk is in the slot
  uint64_t h_full[fwd::kSlots];           // leader's copy is used: the gate warps of both CTAs wrote H
  uint64_t acc_full;                      // local, multicast commit
  uint64_t acc_empty;                     // leader's copy is used
  uint32_t tmem_base;
};

__device__ __forceinline__ void tile_coords(const FwdParams& p, int t, int& mt, int& nt) {
  const int per_panel = p.PM * p.n_ntiles;
  const int panel = t / per_panel;
  const int rem = t - panel * per_panel;
  const int m0 = panel * p.PM;
  const int pm = min(p.PM, p.n_mtiles - m0);  // last panel may be short
  nt = rem / pm;
  mt = m0 + (rem - nt * pm);
}

// EXTRA: 0 the plain gate warps; 1 internal bias (a null bias is allowed); 2 hash dropout (+ optional bias)
template <int DT, int GATE, int E, int EXTRA>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(fwd::kThreads, 1)
prism_fwd_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmR,
                 const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
                 const FwdParams p) {
  using namespace fwd;
  constexpr int KS = E / 16;   // K16 steps per rotation block
  constexpr int NB = 64 / E;   // rotation blocks per chunk
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  // stage: [A tile | this CTA's half of the R tile | this CTA's half of the B tile]
  const int b_off = kATileBytes + p.r_tile_bytes;
  const int b_bytes = p.BN * 64;   // BN/2 rows of 128 bytes
  uint8_t* smemSt = smem;
  uint8_t* smemEpi = smemSt + p.ns * p.stage_bytes;
  FwdBarriers* bars = reinterpret_cast<FwdBarriers*>(smemEpi + kNumEpiWarps * kEpiStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs), 1 = peer
  const int cid = blockIdx.x >> 1;                  // cluster index
  const int n_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(&bars->loads_full[i], 4);   // two producers in each CTA, one arrive.expect_tx each
      mbar_init(&bars->done[i], 1);
    }
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->h_full[i], 2 * kWarpsPerGroup);
    }
    mbar_init(&bars->acc_full, 1);
    mbar_init(&bars->acc_empty, 2 * kNumEpiWarps);
    fence_mbar_init();
  }
  if (warp == kWarpMma) {
    tmem_alloc_pair(&bars->tmem_base, 512);
    tmem_relinquish_pair();
  }
  if (warp == kWarpTma && lane == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmR);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmC);
  }
  // the peer's barriers must be initialised before anything arrives on them remotely
  tc_fence_before_sync();
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const int nk = p.n_kchunks;
  const int my_tiles = (p.n_tiles - cid + n_clusters - 1) / n_clusters;
  const uint32_t total = (uint32_t)my_tiles * nk;   // chunks this CTA pair processes

  if (warp == kWarpTma) {
    // ------------------------------------------------------------------ TMA producer: A tile and half of the R tile
    if (lane == 0) {
      Ring rs(p.ns);
      int ta = cid, ca = 0, mta, nta;
      tile_coords(p, ta, mta, nta);
      int ga = nta / p.ntiles_per_group;
      bool ok = true;
      for (uint32_t j = 0; j < total; ++j, rs.next()) {
        if (!mbar_wait(&bars->done[rs.idx], rs.phase ^ 1)) { ok = false; break; }
        uint8_t* dst = smemSt + rs.idx * p.stage_bytes;
        // completion is counted on the leader's barrier: its MMAs read both CTAs' tiles
        const uint32_t full = mapa_shared(smem_u32(&bars->loads_full[rs.idx]), 0);
        mbar_arrive_expect_tx_cluster(full, kATileBytes + (E / 2) * 128);
        tma_load_2d_pair(dst, &tmA, full, ca * 64, mta * 256 + (int)rank * 128);
        tma_load_2d_pair(dst + kATileBytes, &tmR, full, ca * 64, ga * E + (int)rank * (E / 2));
        if (++ca == nk) {
          ca = 0;
          ta += n_clusters;
          if (ta < p.n_tiles) { tile_coords(p, ta, mta, nta); ga = nta / p.ntiles_per_group; }
        }
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp == kWarpTmaB) {
    // ------------------------------------------------------------------ TMA producer: this CTA's half of the B tiles
    if (lane == 0) {
      Ring rs(p.ns);
      int tb = cid, cb = 0, mtb, ntb;
      tile_coords(p, tb, mtb, ntb);
      bool ok = true;
      for (uint32_t j = 0; j < total; ++j, rs.next()) {
        if (!mbar_wait(&bars->done[rs.idx], rs.phase ^ 1)) { ok = false; break; }
        const uint32_t full = mapa_shared(smem_u32(&bars->loads_full[rs.idx]), 0);
        mbar_arrive_expect_tx_cluster(full, b_bytes);
        tma_load_2d_pair(smemSt + rs.idx * p.stage_bytes + b_off, &tmB, full, cb * 64,
                         ntb * p.BN + (int)rank * (p.BN / 2));
        if (++cb == nk) {
          cb = 0;
          tb += n_clusters;
          if (tb < p.n_tiles) tile_coords(p, tb, mtb, ntb);
        }
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp == kWarpRot) {
    // ------------------------------------------------------------------ MMA issuer 1: rotation S = A . blockdiag(R_g)^T
    // Two threads issue tcgen05.mma, one per product: while one of them tests barriers or commits, the
    // MMAs of the other keep the tensor pipe busy.  Their MMAs are ordered by barriers only.
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_r = make_idesc(DT, 256, E, 0, 0);      // S block: M = 256 rows, N = E
      // descriptors of stage 0; a stage further on adds stage_bytes >> 4 to the low words
      const uint64_t da0 = desc_kmajor_sw128(smem_u32(smemSt), 1024);
      const uint64_t dr0 = desc_kmajor_sw128(smem_u32(smemSt) + kATileBytes, 1024);
      const uint32_t d_hi = (uint32_t)(da0 >> 32);
      const uint32_t st_step = (uint32_t)p.stage_bytes >> 4;
      const uint32_t slot0 = tmem_base + kSlotCol0;
      Ring rl(p.ns), rf(p.ns);   // stage of chunk i / of chunk i - kSlots
      bool ok = true;
      for (uint32_t i = 0; i < total; ++i, rl.next()) {
        const uint32_t slot = i & (kSlots - 1);
        if (i >= (uint32_t)kSlots) {
          // the slot still holds H of chunk i - 4 until that chunk's dense product has completed
          // (the ring has at least kSlots stages, so this barrier cannot run a phase ahead)
          if (!mbar_wait_cluster(&bars->done[rf.idx], rf.phase)) { ok = false; break; }
          rf.next();
        }
        if (!mbar_wait_cluster(&bars->loads_full[rl.idx], rl.phase)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t a_lo = (uint32_t)da0 + rl.idx * st_step;
        const uint32_t r_lo = (uint32_t)dr0 + rl.idx * st_step;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
            const int kk = b * KS + ks;   // K16 step inside the 64-wide chunk: +32 bytes on both operands
            umma_f16_pair_lh(slot0 + slot * 64 + b * E, a_lo + kk * 2, d_hi, r_lo + kk * 2, d_hi, idesc_r,
                             ks > 0 ? 1u : 0u);
          }
        }
        umma_commit_pair(&bars->s_full[slot], 0x3);
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA issuer 2: dense product C += H . B^T
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_c = make_idesc(DT, 256, p.BN, 0, 0);   // C tile:  M = 256 rows, N = BN
      const uint64_t db0 = desc_kmajor_sw128(smem_u32(smemSt) + b_off, 1024);
      const uint32_t d_hi = (uint32_t)(db0 >> 32);
      const uint32_t st_step = (uint32_t)p.stage_bytes >> 4;
      const uint32_t slot0 = tmem_base + kSlotCol0;
      Ring rd(p.ns);
      int cm = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (uint32_t jd = 0; jd < total; ++jd, rd.next()) {
        const uint32_t slot = jd & (kSlots - 1);
        // H complete implies that the stage's loads (B included) landed: the rotation waited for them
        if (!mbar_wait_cluster(&bars->h_full[slot], (jd / kSlots) & 1)) { ok = false; break; }
        if (cm == 0) {
          if (!mbar_wait_cluster(&bars->acc_empty, acc_phase ^ 1)) { ok = false; break; }
        }
        tc_fence_after_sync();
        const uint32_t h_tmem = slot0 + slot * 64;
        const uint32_t b_lo = (uint32_t)db0 + rd.idx * st_step;
        umma_f16_pair_ts_lh(tmem_base, h_tmem, b_lo, d_hi, idesc_c, cm > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 1; ks < 4; ++ks)
          umma_f16_pair_ts_lh(tmem_base, h_tmem + ks * 8, b_lo + ks * 2, d_hi, idesc_c, 1u);
        umma_commit_pair(&bars->done[rd.idx], 0x3);   // both CTAs may refill the stage; the slot is free
        if (++cm == nk) {
          cm = 0;
          umma_commit_pair(&bars->acc_full, 0x3);
          acc_phase ^= 1u;
        }
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp >= kGateWarp0 && warp < kEpiWarp0) {
    // ------------------------------------------------------------------ gate warps
    const uint32_t gw = warp - kGateWarp0;
    const uint32_t group = gw / kWarpsPerGroup;               // which chunks (j mod kGateGroups)
    const uint32_t r0 = (gw & 3) * 32 + ((gw >> 2) & 1) * 16; // this warp's 16 rows, inside its TMEM lane quarter
    Ring rs(p.ns);
    for (uint32_t i = 0; i < group; ++i) rs.next();
    bool ok = true;
    // internal bias / dropout: tile, group and K chunk of chunk j, followed without a division per chunk
    const uint16_t* ibase = reinterpret_cast<const uint16_t*>(p.ib);
    constexpr bool DROP = (EXTRA == 2);
    constexpr bool track = (EXTRA != 0);
    int tg = cid, kc = (int)group, gcur = 0, mtcur = 0;
    if (track && total > 0) {
      while (kc >= nk) { kc -= nk; tg += n_clusters; }
      int nt0;
      tile_coords(p, tg, mtcur, nt0);
      gcur = nt0 / p.ntiles_per_group;
    }
    for (uint32_t j = group; j < total; j += kGateGroups, rs.next(), rs.next()) {
      const uint32_t slot = j & (kSlots - 1);
      if (!mbar_wait(&bars->s_full[slot], (j / kSlots) & 1)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t s_tmem = tmem_base + (r0 << 16) + kSlotCol0 + slot * 64;
      if (track) {
        const uint16_t* ib = ibase != nullptr ? ibase + (long long)gcur * p.K + kc * 64 : nullptr;
        DropCtx dc;
        if (DROP) {
          dc.h1 = drop_group_hash(p.drop_seeds, gcur);
          dc.base = (long long)((mtcur * 2 + (int)rank) * 128 + (int)r0 + (lane >> 2)) * p.K + kc * 64 + 2 * (lane & 3);
          dc.row8 = 8ll * p.K;
          dc.p = p.drop_p;
          dc.inv_keep = p.drop_inv_keep;
        }
        gate_rows16_tmem<DT, GATE, DROP>(s_tmem, smem_u32(smemSt + rs.idx * p.stage_bytes), r0, lane, s_tmem, ib,
                                         p.K - kc * 64, &dc);
        kc += kGateGroups;
        if (kc >= nk) {
          while (kc >= nk) { kc -= nk; tg += n_clusters; }
          if (tg < p.n_tiles) { int nt1; tile_coords(p, tg, mtcur, nt1); gcur = nt1 / p.ntiles_per_group; }
        }
      } else {
        gate_rows16_tmem<DT, GATE>(s_tmem, smem_u32(smemSt + rs.idx * p.stage_bytes), r0, lane, s_tmem);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&bars->h_full[slot]), 0));   // H is in TMEM
    }
    if (!ok && lane == 0) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
  } else if (warp >= kEpiWarp0) {
    // ------------------------------------------------------------------ epilogue warps
    const int q = warp & 3;
    const uint32_t row = q * 32 + lane;
    const uint32_t lane_base = uint32_t(q * 32) << 16;
    uint8_t* stage = smemEpi + (warp - kEpiWarp0) * kEpiStageBytes;
    const uint16_t* bias = reinterpret_cast<const uint16_t*>(p.bias);
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = cid; t < p.n_tiles && ok; t += n_clusters, acc_phase ^= 1u) {
      int mp, nt;
      tile_coords(p, t, mp, nt);
      const int mt = mp * 2 + (int)rank;   // this CTA's 128-row block
      if (!mbar_wait(&bars->acc_full, acc_phase)) { ok = false; break; }
      const uint32_t tacc = tmem_base + lane_base;
      tc_fence_after_sync();
      const long long grow = (long long)mt * 128 + row;
      const int n0 = nt * p.BN;
      if (p.tma_store) {
        // 64 columns at a time: TMEM -> registers -> swizzled staging tile -> TMA store
        for (int c0 = 0; c0 < p.BN; c0 += 64) {
          if (lane == 0) tma_store_wait_read<0>();   // the staging tile is free again
          __syncwarp();
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t v[32];
            tmem_ld_x32(tacc + c0 + hh * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t ow[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float x0 = __uint_as_float(v[j * 8 + e * 2]);
                float x1 = __uint_as_float(v[j * 8 + e * 2 + 1]);
                if (bias != nullptr) {
                  const uint32_t bw = *reinterpret_cast<const uint32_t*>(bias + n0 + c0 + hh * 32 + j * 8 + e * 2);
                  const float2 b2 = Elem<DT>::unpack(bw);
                  x0 += b2.x;
                  x1 += b2.y;
                }
                ow[e] = Elem<DT>::pack(x0, x1);
              }
              *reinterpret_cast<uint4*>(stage + sw128_offset(lane, hh * 4 + j)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && mt * 128 + q * 32 < p.M) {
            tma_store_2d(&tmC, stage, n0 + c0, mt * 128 + q * 32);
            tma_store_commit();
          }
        }
      } else {
        uint16_t* crow = reinterpret_cast<uint16_t*>(p.C) + grow * p.ldc + n0;
        for (int c0 = 0; c0 < p.BN; c0 += 16) {   // BN is a multiple of 16
          uint32_t v[16];
          tmem_ld_x16(tacc + c0, v);
          tmem_ld_wait();
          if (grow < p.M) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              uint32_t ow[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float x0 = __uint_as_float(v[j * 8 + e * 2]);
                float x1 = __uint_as_float(v[j * 8 + e * 2 + 1]);
                if (bias != nullptr) {
                  const uint32_t bw = *reinterpret_cast<const uint32_t*>(bias + n0 + c0 + j * 8 + e * 2);
                  const float2 b2 = Elem<DT>::unpack(bw);
                  x0 += b2.x;
                  x1 += b2.y;
                }
                ow[e] = Elem<DT>::pack(x0, x1);
              }
              *reinterpret_cast<uint4*>(crow + c0 + j * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&bars->acc_empty), 0));
    }
    if (lane == 0) tma_store_wait_all<0>();   // outstanding stores read shared memory
    if (!ok && lane == 0) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
  }

  // ------------------------------------------------------------------ teardown
  // neither CTA may leave (or free TMEM) while its peer can still reach its barriers or shared memory
  tc_fence_before_sync();
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
  if (warp == kWarpMma) tmem_dealloc_pair(tmem_base, 512);
}

// ----------------------------------------------------------------------------
// host launcher
// ----------------------------------------------------------------------------
int launch_fwd(const FwdArgs& a) {
  FwdParams p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.gs = a.gs; p.E = a.E; p.BN = a.BN;
  p.n_mtiles = (a.M + 255) / 256;   // row blocks of a CTA pair
  p.n_ntiles = a.N / a.BN;
  p.ntiles_per_group = a.gs / a.BN;
  p.n_tiles = p.n_mtiles * p.n_ntiles;
  p.PM = a.PM > 0 ? a.PM : 8;
  if (p.PM > p.n_mtiles) p.PM = p.n_mtiles;
  p.n_kchunks = (a.K + 63) / 64;
  p.r_tile_bytes = ((a.E / 2 * 128) + 1023) / 1024 * 1024;   // this CTA's E/2 rows of the R tile
  p.tma_store = (a.BN % 64 == 0) ? 1 : 0;
  p.bias = a.bias; p.ib = a.ib; p.C = a.C; p.ldc = a.ldc; p.err = a.err;
  const bool drop = a.drop_seeds != nullptr && a.drop_p > 0.f && a.gate != GATE_NONE;
  p.drop_seeds = a.drop_seeds; p.drop_p = a.drop_p; p.drop_inv_keep = drop ? 1.f / (1.f - a.drop_p) : 1.f;
  if (drop && a.E != 16) return fail(PRISM_ERR_UNSUPPORTED, "forward: dropout needs reconn_sz 8 or 16");

  const int budget = 227 * 1024 - 1024 - (int)sizeof(FwdBarriers) - 256 - fwd::kNumEpiWarps * fwd::kEpiStageBytes;
  p.stage_bytes = fwd::kATileBytes + p.r_tile_bytes + a.BN * 64;   // A tile, halves of the R and B tiles
  int ns = a.sa > 0 ? a.sa : fwd::kMaxStages;
  if (ns > fwd::kMaxStages) ns = fwd::kMaxStages;
  while (ns > fwd::kSlots && ns * p.stage_bytes > budget) --ns;
  if (ns < fwd::kSlots || ns * p.stage_bytes > budget)   // a stage per TMEM slot at least (see the rotation issuer)
    return fail(PRISM_ERR_UNSUPPORTED, "forward tile does not fit shared memory (BN=%d E=%d)", a.BN, a.E);
  p.ns = ns;
  const int smem_bytes = ns * p.stage_bytes + fwd::kNumEpiWarps * fwd::kEpiStageBytes +
                         (int)sizeof(FwdBarriers) + 1024;

  CUtensorMap tmA, tmR, tmB, tmC;
  int rc;
  if ((rc = make_tmap_2d(&tmA, a.dtype, a.A, a.M, a.K, a.lda, 128, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmR, a.dtype, a.R_eff, (uint64_t)(a.N / a.gs) * a.E, a.K, a.ldr, a.E / 2, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmB, a.dtype, a.B, a.N, a.K, a.ldb, a.BN / 2, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmC, a.dtype, a.C, a.M, a.N, a.ldc, 32, 64, true))) return rc;

  int n_clusters = a.num_sms / 2;
  if (n_clusters > p.n_tiles) n_clusters = p.n_tiles;
  const int grid = 2 * n_clusters;

  using KernT = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, FwdParams);
  KernT kern = nullptr;
#define PRISM_PICK_G(DT_, E_, X_)                                                                       \
  (a.gate == GATE_SILU ? (KernT)prism_fwd_kernel<DT_, GATE_SILU, E_, X_>                                 \
                       : a.gate == GATE_SIGMOID ? (KernT)prism_fwd_kernel<DT_, GATE_SIGMOID, E_, X_> : (KernT)prism_fwd_kernel<DT_, GATE_NONE, E_, 0>)
#define PRISM_PICK(E_, X_) kern = (a.dtype == DT_BF16) ? PRISM_PICK_G(DT_BF16, E_, X_) : PRISM_PICK_G(DT_F16, E_, X_)
  const bool ib = a.ib != nullptr && a.gate != GATE_NONE;
  if (drop) { PRISM_PICK(16, 2); }
  else if (ib) { if (a.E == 16) { PRISM_PICK(16, 1); } else if (a.E == 32) { PRISM_PICK(32, 1); } else { PRISM_PICK(64, 1); } }
  else if (a.E == 16) { PRISM_PICK(16, 0); } else if (a.E == 32) { PRISM_PICK(32, 0); } else { PRISM_PICK(64, 0); }
#undef PRISM_PICK_G
#undef PRISM_PICK
  if ((rc = set_max_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes, "forward"))) return rc;
  kern<<<grid, fwd::kThreads, smem_bytes, a.stream>>>(tmA, tmR, tmB, tmC, p);
  return check_launch("prism_fwd");
}

}  // namespace prism
