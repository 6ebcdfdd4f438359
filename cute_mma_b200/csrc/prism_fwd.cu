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
// persistent loop over the pair's tiles; per 64-wide K chunk
//   warps 0, 2  TMA producers: A tile [128 x 64] + R_g tile [E x 64] into the "AR" ring (warp 0), this
//               CTA's half of the B_g tile [BN/2 x 64] into the "B" ring (warp 2); 128-byte swizzle,
//               zero fill outside the tensors
//   warps 4-19  gate warps, two groups of eight that take alternate chunks, 16 rows per warp: A and R fragments by ldmatrix, block rotation
//               S = A_blk . R_blk^T by mma.sync (fp32), H = A*silu(S) (or H = S) on registers,
//               H written to TMEM (tcgen05.st) as the A operand of the dense MMA: H never goes
//               through shared memory, which is the scarce resource of this kernel
//   warp 1      dense issuer (leader CTA only): C += H . B^T as 4 x tcgen05.mma M256 N=BN K=16 spanning
//               both CTAs (A = H from TMEM, B = B_g from shared memory), fp32 accumulator in TMEM
//   warps 20-23 epilogue: tcgen05.ld C, + bias, cast, swizzled staging tile, TMA store.
// Every role keeps its ring positions as counters; the single-thread roles do no division.
#include "prism_host.cuh"
#include "prism_kernels.cuh"

#ifndef PRISM_DBG
#define PRISM_DBG 0   // debugging aid: bit 0 skips the gate math, bit 1 the output stores, bit 2 the rotation MMAs
#endif

namespace prism {

namespace fwd {
constexpr int kThreads = 768;
constexpr int kWarpTma = 0, kWarpMma = 1, kWarpTmaB = 2;
constexpr int kGateWarp0 = 4;         // multiple of 4: (warp & 3) is the TMEM lane quarter a warp may touch
constexpr int kGateGroups = 2;        // groups take alternate chunks ...
constexpr int kWarpsPerGroup = 8;     // ... with 16 rows per warp
constexpr int kNumGateWarps = kGateGroups * kWarpsPerGroup;
constexpr int kEpiWarp0 = kGateWarp0 + kNumGateWarps;   // 20
constexpr int kHBufs = 4;             // TMEM ring of H chunks (power of two), 32 columns each
constexpr int kHCol0 = 256;           // accumulator: TMEM columns [0, 256); H ring: [256, 384)
constexpr int kNumEpiWarps = 4;
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
  int sa, sb;           // stages of the AR ring / B ring
  int r_tile_bytes;     // bytes reserved for the R tile of one AR stage (multiple of 1024)
  int tma_store;        // 1: epilogue goes through TMA stores (BN multiple of 64)
  const void* bias;     // [N] or null
  void* C;
  long long ldc;
  int* err;
};

struct FwdBarriers {
  uint64_t ar_full[fwd::kMaxStages];
  uint64_t a_empty[fwd::kMaxStages];
  uint64_t b_full[fwd::kHBufs];
  uint64_t b_empty[fwd::kHBufs];
  uint64_t h_full[fwd::kHBufs];
  uint64_t h_empty[fwd::kHBufs];
  uint64_t acc_full;
  uint64_t acc_empty;
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

template <int DT, int GATE, int E>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(fwd::kThreads, 1)
prism_fwd_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmR,
                 const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
                 const FwdParams p) {
  using namespace fwd;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  const int ar_stage_bytes = kATileBytes + p.r_tile_bytes;
  const int b_stage_bytes = p.BN * 64;   // this CTA's half of the B tile: BN/2 rows of 128 bytes
  uint8_t* smemAR = smem;
  uint8_t* smemB = smemAR + p.sa * ar_stage_bytes;
  uint8_t* smemEpi = smemB + p.sb * b_stage_bytes;
  FwdBarriers* bars = reinterpret_cast<FwdBarriers*>(smemEpi + kNumEpiWarps * kEpiStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs), 1 = peer
  const int cid = blockIdx.x >> 1;                  // cluster index
  const int n_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(&bars->ar_full[i], 1);                    // local: this CTA's A and R tiles landed
      mbar_init(&bars->a_empty[i], kWarpsPerGroup);       // local: the gate warps have read the tiles
    }
    for (int i = 0; i < kHBufs; ++i) {
      mbar_init(&bars->b_full[i], 2);                     // leader's copy is used: both CTAs' B halves
      mbar_init(&bars->b_empty[i], 1);                    // local, arrived by the multicast commit
      mbar_init(&bars->h_full[i], 2 * kWarpsPerGroup);    // leader's copy is used: gate warps of both CTAs
      mbar_init(&bars->h_empty[i], 1);                    // local, arrived by the multicast commit
    }
    mbar_init(&bars->acc_full, 1);                        // local, arrived by the multicast commit
    mbar_init(&bars->acc_empty, 2 * kNumEpiWarps);        // leader's copy is used
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
    // ------------------------------------------------------------------ TMA producer: A and R tiles
    if (lane == 0) {
      Ring ra(p.sa);
      int ta = cid, ca = 0, mta, nta;
      tile_coords(p, ta, mta, nta);
      int ga = nta / p.ntiles_per_group;
      bool ok = true;
      for (uint32_t j = 0; j < total; ++j) {
        if (!mbar_wait(&bars->a_empty[ra.idx], ra.phase ^ 1)) { ok = false; break; }
        uint8_t* dstA = smemAR + ra.idx * ar_stage_bytes;
        mbar_arrive_expect_tx(&bars->ar_full[ra.idx], kATileBytes + p.E * 128);
        tma_load_2d(dstA, &tmA, &bars->ar_full[ra.idx], ca * 64, mta * 256 + (int)rank * 128);
        tma_load_2d(dstA + kATileBytes, &tmR, &bars->ar_full[ra.idx], ca * 64, ga * p.E);
        ra.next();
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
      int tb = cid, cb = 0, mtb, ntb;
      tile_coords(p, tb, mtb, ntb);
      bool ok = true;
      for (uint32_t j = 0; j < total; ++j) {
        const uint32_t hb = j & (kHBufs - 1), hphase = (j / kHBufs) & 1;   // B stage = H buffer index
        if (!mbar_wait(&bars->b_empty[hb], hphase ^ 1)) { ok = false; break; }
        // completion is counted on the leader's barrier
        const uint32_t bfull = mapa_shared(smem_u32(&bars->b_full[hb]), 0);
        mbar_arrive_expect_tx_cluster(bfull, b_stage_bytes);
        tma_load_2d_pair(smemB + hb * b_stage_bytes, &tmB, bfull, cb * 64, ntb * p.BN + (int)rank * (p.BN / 2));
        if (++cb == nk) {
          cb = 0;
          tb += n_clusters;
          if (tb < p.n_tiles) tile_coords(p, tb, mtb, ntb);
        }
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ dense issuer
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_c = make_idesc(DT, 256, p.BN, 0, 0);   // M = 256: 128 rows in each CTA
      int cm = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (uint32_t j = 0; j < total; ++j) {
        const uint32_t hb = j & (kHBufs - 1), hphase = (j / kHBufs) & 1;
        if (!mbar_wait_cluster(&bars->h_full[hb], hphase)) { ok = false; break; }
        if (!mbar_wait_cluster(&bars->b_full[hb], hphase)) { ok = false; break; }
        if (cm == 0) {
          if (!mbar_wait_cluster(&bars->acc_empty, acc_phase ^ 1)) { ok = false; break; }
        }
        tc_fence_after_sync();
        const uint32_t h_tmem = tmem_base + kHCol0 + hb * 32;
        const uint32_t b_addr = smem_u32(smemB + hb * b_stage_bytes);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          umma_f16_pair_ts(tmem_base, h_tmem + ks * 8, desc_kmajor_sw128(b_addr + ks * 32, 1024), idesc_c,
                           (cm > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit_pair(&bars->h_empty[hb], 0x3);   // both CTAs' gate warps may refill the H buffer
        umma_commit_pair(&bars->b_empty[hb], 0x3);   // both CTAs' B stages are free
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
    Ring ra(p.sa);
    for (uint32_t i = 0; i < group; ++i) ra.next();
    bool ok = true;
    for (uint32_t j = group; j < total; j += kGateGroups, ra.next(), ra.next()) {
      const uint32_t hb = j & (kHBufs - 1), hphase = (j / kHBufs) & 1;
      if (!mbar_wait(&bars->ar_full[ra.idx], ra.phase)) { ok = false; break; }
      if (!mbar_wait(&bars->h_empty[hb], hphase ^ 1)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t tile = smem_u32(smemAR + ra.idx * ar_stage_bytes);
      rotate_gate_rows16<DT, GATE, E>(tile, tile + kATileBytes, r0, lane, tmem_base + (r0 << 16) + kHCol0 + hb * 32);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars->a_empty[ra.idx]);                                   // A and R tiles are free again
        mbar_arrive_cluster(mapa_shared(smem_u32(&bars->h_full[hb]), 0));      // H chunk is in TMEM
      }
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
          if (lane == 0 && !(PRISM_DBG & 2) && mt * 128 + q * 32 < p.M) {
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
          if (grow < p.M && !(PRISM_DBG & 2)) {
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
  p.r_tile_bytes = ((a.E * 128) + 1023) / 1024 * 1024;
  p.tma_store = (a.BN % 64 == 0) ? 1 : 0;
  p.bias = a.bias; p.C = a.C; p.ldc = a.ldc; p.err = a.err;

  const int budget = 227 * 1024 - 1024 - (int)sizeof(FwdBarriers) - 256 - fwd::kNumEpiWarps * fwd::kEpiStageBytes;
  const int ar_bytes = fwd::kATileBytes + p.r_tile_bytes;
  const int b_bytes = a.BN * 64;   // per CTA: half of the B tile
  // the AR ring feeds rotation + gate, which run ahead of the dense product: give it the deeper pipeline
  // the B ring has one stage per H buffer (they share barriers); the AR ring takes what is left
  const int sb = fwd::kHBufs;
  int sa = a.sa > 0 ? a.sa : fwd::kMaxStages;
  if (sa > fwd::kMaxStages) sa = fwd::kMaxStages;
  while (sa > 2 && sa * ar_bytes + sb * b_bytes > budget) --sa;
  if (sa * ar_bytes + sb * b_bytes > budget)
    return fail(PRISM_ERR_UNSUPPORTED, "forward tile does not fit shared memory (BN=%d E=%d)", a.BN, a.E);
  p.sa = sa; p.sb = sb;
  const int smem_bytes = sa * ar_bytes + sb * b_bytes + fwd::kNumEpiWarps * fwd::kEpiStageBytes +
                         (int)sizeof(FwdBarriers) + 1024;

  CUtensorMap tmA, tmR, tmB, tmC;
  int rc;
  if ((rc = make_tmap_2d(&tmA, a.dtype, a.A, a.M, a.K, a.lda, 128, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmR, a.dtype, a.R_eff, (uint64_t)(a.N / a.gs) * a.E, a.K, a.ldr, a.E, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmB, a.dtype, a.B, a.N, a.K, a.ldb, a.BN / 2, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmC, a.dtype, a.C, a.M, a.N, a.ldc, 32, 64, true))) return rc;

  int n_clusters = a.num_sms / 2;
  if (n_clusters > p.n_tiles) n_clusters = p.n_tiles;
  const int grid = 2 * n_clusters;

  using KernT = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, FwdParams);
  KernT kern = nullptr;
#define PRISM_PICK(E_)                                                                               \
  kern = (a.dtype == DT_BF16)                                                                        \
             ? (a.gate == GATE_SILU ? (KernT)prism_fwd_kernel<DT_BF16, GATE_SILU, E_> : (KernT)prism_fwd_kernel<DT_BF16, GATE_NONE, E_>) \
             : (a.gate == GATE_SILU ? (KernT)prism_fwd_kernel<DT_F16, GATE_SILU, E_> : (KernT)prism_fwd_kernel<DT_F16, GATE_NONE, E_>)
  if (a.E == 16) { PRISM_PICK(16); } else if (a.E == 32) { PRISM_PICK(32); } else { PRISM_PICK(64); }
#undef PRISM_PICK
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return fail(PRISM_ERR_CUDA, "forward: cannot set %d B of shared memory: %s", smem_bytes, cudaGetErrorString(e));
  kern<<<grid, fwd::kThreads, smem_bytes, a.stream>>>(tmA, tmR, tmB, tmC, p);
  return check_launch("prism_fwd");
}

}  // namespace prism
