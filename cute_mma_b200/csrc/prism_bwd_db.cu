// Prism backward, weight gradient, for sm_100a:
//   dB_g [gs, K] = scale * dC_g^T [gs, M] . H_g [M, K],   H_g = A * silu(A . blockdiag(R_g)^T)
// (H_g = A . blockdiag(R_g)^T in plain mode), with H recomputed on chip.
//
// Replaces the reference's dB_pc_kernel / prism_backward_dB_launch
// (cute_prism_backward_db.cu:450-582) and its binding (torch_ext/prism_bwd_db_torch.cu:42-162).
//
// CTAs work in pairs (cluster of 2, tcgen05 cta_group::2).  A pair owns one accumulator tile
// D[f, n] (256 features x BN outputs of one group; each CTA holds its 128 features in its own TMEM
// and loads half of the dC columns) and a contiguous range of 128-token blocks.  The contraction runs over tokens, so both
// tensor-core operands are "MN-major": H tiles [128 tokens x 64 features] and dC tiles
// [128 tokens x 64 outputs] are used exactly as TMA / the gate warps lay them out, no transposes.
//   TMA warp   : R_g tiles once; per token block two A tiles and ceil(BN/64) dC tiles
//   gate warps : two groups taking alternate token blocks, 16 token rows per warp; block rotation S = A_blk . R_blk^T by mma.sync on ldmatrix
//                fragments, H = A*silu(S) on registers, stmatrix of H over the A tiles in place
//   MMA issuer : D += H^T . dC as 8 x tcgen05.mma M128 N=BN K=16 per token block
//   epilogue   : D -> dB (transposed store), or fp32 partials when the token range is split;
//                a second kernel then adds the partials in a fixed order (deterministic).
#include "prism_host.cuh"
#include "prism_kernels.cuh"

namespace prism {

namespace db {
constexpr int kThreads = 704;     // warp 0 TMA, 1 dense issuer, 2-17 gate, 18-21 epilogue
constexpr int kWarpTma = 0, kWarpMma = 1;
constexpr int kGateWarp0 = 2;
constexpr int kGateGroups = 2;    // groups take alternate token blocks ...
constexpr int kWarpsPerGroup = 8; // ... with 16 token rows per warp
constexpr int kNumGateWarps = kGateGroups * kWarpsPerGroup;
constexpr int kEpiWarp0 = kGateWarp0 + kNumGateWarps;   // (warp & 3) of warps 18..21 covers 2,3,0,1
constexpr int kMaxStages = 4;
constexpr int kTile = 128 * 128;  // bytes of a [128 x 64] 16-bit tile
}  // namespace db

struct DbParams {
  int M, N, K, gs, E, BN;
  int ntiles_per_group;
  int blocks_per_split, n_tokblocks;
  int dc_tiles;       // ceil(BN / 64)
  int r_tile_bytes;   // bytes reserved per R tile (multiple of 1024)
  int sa, sd;         // stages of the A ring / dC ring
  int splits;
  float scale;
  void* dB;
  long long lddb;
  float* partial;     // [splits][N][K] when splits > 1
  int* err;
};

struct DbBarriers {
  uint64_t r_full;
  uint64_t a_full[db::kMaxStages];
  uint64_t h_full[db::kMaxStages];
  uint64_t a_empty[db::kMaxStages];
  uint64_t dc_full[db::kMaxStages];
  uint64_t dc_empty[db::kMaxStages];
  uint64_t acc_full;
  uint32_t tmem_base;
};

template <int DT, int GATE, int E>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(db::kThreads, 1)
prism_bwd_db_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmR,
                    const __grid_constant__ CUtensorMap tmdC, const DbParams p) {
  using namespace db;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  const int a_stage_bytes = 2 * kTile;
  const int dc_stage_bytes = p.dc_tiles * kTile;
  uint8_t* smemR = smem;
  uint8_t* smemA = smemR + 2 * p.r_tile_bytes;
  uint8_t* smemD = smemA + p.sa * a_stage_bytes;
  DbBarriers* bars = reinterpret_cast<DbBarriers*>(smemD + p.sd * dc_stage_bytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0 = leader (issues the MMAs), 1 = peer
  const int f0 = blockIdx.x * 128;           // first of this CTA's 128 features (column of A / dB)
  const int nt = blockIdx.y;
  const int n0 = nt * p.BN;                  // first output (row of dB)
  const int g = nt / p.ntiles_per_group;
  const int split = blockIdx.z;
  const int tb0 = split * p.blocks_per_split;
  const int nb = min(p.blocks_per_split, p.n_tokblocks - tb0);  // token blocks of this CTA (>= 1)

  if (threadIdx.x == 0) {
    mbar_init(&bars->r_full, 1);
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(&bars->a_full[i], 1);                  // local: this CTA's A tiles landed
      mbar_init(&bars->h_full[i], 2 * kWarpsPerGroup); // leader's copy is used: gate warps of both CTAs
      mbar_init(&bars->a_empty[i], 1);                 // local, arrived by the multicast commit
      mbar_init(&bars->dc_full[i], 2);                 // leader's copy is used: both CTAs' dC halves
      mbar_init(&bars->dc_empty[i], 1);
    }
    mbar_init(&bars->acc_full, 1);
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
      mbar_arrive_expect_tx(&bars->r_full, 2 * p.E * 128);
      tma_load_2d(smemR, &tmR, &bars->r_full, f0, g * p.E);
      tma_load_2d(smemR + p.r_tile_bytes, &tmR, &bars->r_full, f0 + 64, g * p.E);
      Ring ra(p.sa), rd(p.sd);
      for (int j = 0; j < nb && ok; ++j, ra.next(), rd.next()) {
        const int tok0 = (tb0 + j) * 128;
        const int sa = ra.idx, sd = rd.idx;
        if (!mbar_wait(&bars->a_empty[sa], ra.phase ^ 1)) { ok = false; break; }
        uint8_t* dstA = smemA + sa * a_stage_bytes;
        mbar_arrive_expect_tx(&bars->a_full[sa], 2 * kTile);
        tma_load_2d(dstA, &tmA, &bars->a_full[sa], f0, tok0);
        tma_load_2d(dstA + kTile, &tmA, &bars->a_full[sa], f0 + 64, tok0);
        if (!mbar_wait(&bars->dc_empty[sd], rd.phase ^ 1)) { ok = false; break; }
        uint8_t* dstD = smemD + sd * dc_stage_bytes;
        // this CTA's half of the dC columns; completion is counted on the leader's barrier
        const uint32_t dcfull = mapa_shared(smem_u32(&bars->dc_full[sd]), 0);
        mbar_arrive_expect_tx_cluster(dcfull, dc_stage_bytes);
        for (int t = 0; t < p.dc_tiles; ++t)
          tma_load_2d_pair(dstD + t * kTile, &tmdC, dcfull, n0 + (int)rank * (p.BN / 2) + 64 * t, tok0);
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ dense issuer
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_d = make_idesc(DT, 256, p.BN, 1, 1);   // M = 256: 128 features in each CTA
      bool ok = true;
      Ring ra(p.sa), rd(p.sd);
      for (int j = 0; j < nb && ok; ++j, ra.next(), rd.next()) {
        if (!mbar_wait_cluster(&bars->h_full[ra.idx], ra.phase)) { ok = false; break; }
        if (!mbar_wait_cluster(&bars->dc_full[rd.idx], rd.phase)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t h_addr = smem_u32(smemA + ra.idx * a_stage_bytes);
        const uint32_t d_addr = smem_u32(smemD + rd.idx * dc_stage_bytes);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          umma_f16_pair(tmem_base, desc_mnmajor_sw128(h_addr + ks * 2048, kTile, 1024),
                        desc_mnmajor_sw128(d_addr + ks * 2048, kTile, 1024), idesc_d,
                        (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit_pair(&bars->a_empty[ra.idx], 0x3);
        umma_commit_pair(&bars->dc_empty[rd.idx], 0x3);
        if (j == nb - 1) umma_commit_pair(&bars->acc_full, 0x3);
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp >= kGateWarp0 && warp < kEpiWarp0) {
    // ------------------------------------------------------------------ gate warps
    const int gw = warp - kGateWarp0;
    const int group = gw / kWarpsPerGroup;            // which token blocks (j mod kGateGroups)
    const uint32_t r0 = (gw % kWarpsPerGroup) * 16;   // this warp's 16 token rows of the block
    bool ok = mbar_wait(&bars->r_full, 0);
    const uint32_t r_addr = smem_u32(smemR);
    Ring ra(p.sa);
    for (int i = 0; i < group; ++i) ra.next();
    for (int j = group; j < nb && ok; j += kGateGroups, ra.next(), ra.next()) {
      if (!mbar_wait(&bars->a_full[ra.idx], ra.phase)) { ok = false; break; }
      const uint32_t tile = smem_u32(smemA + ra.idx * a_stage_bytes);
      rotate_gate_rows16<DT, GATE, E>(tile, r_addr, r0, lane);
      rotate_gate_rows16<DT, GATE, E>(tile + kTile, r_addr + p.r_tile_bytes, r0, lane);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&bars->h_full[ra.idx]), 0));
    }
    if (!ok && lane == 0) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
  } else if (warp >= kEpiWarp0) {
    // ------------------------------------------------------------------ epilogue warps
    const int q = warp & 3;
    const int f = f0 + q * 32 + lane;  // feature = accumulator row
    bool ok = mbar_wait(&bars->acc_full, 0);
    if (ok) {
      tc_fence_after_sync();
      for (int c0 = 0; c0 < p.BN; c0 += 16) {
        uint32_t v[16];
        tmem_ld_x16(tmem_base + (uint32_t(q * 32) << 16) + c0, v);
        tmem_ld_wait();
        if (f < p.K) {
          if (p.splits > 1) {
            float* dst = p.partial + ((long long)split * p.N + n0 + c0) * p.K + f;
#pragma unroll
            for (int j = 0; j < 16; ++j) dst[(long long)j * p.K] = __uint_as_float(v[j]) * p.scale;
          } else {
            uint16_t* dst = reinterpret_cast<uint16_t*>(p.dB) + (long long)(n0 + c0) * p.lddb + f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const uint32_t w = Elem<DT>::pack(__uint_as_float(v[j]) * p.scale, 0.f);
              dst[(long long)j * p.lddb] = static_cast<uint16_t>(w & 0xFFFFu);
            }
          }
        }
      }
    } else if (lane == 0) {
      atomicExch(p.err, PRISM_ERR_DEVICE_WAIT);
    }
  }

  // neither CTA may leave (or free TMEM) while its peer can still reach its barriers or shared memory
  tc_fence_before_sync();
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
  if (warp == kWarpMma) tmem_dealloc_pair(tmem_base, 512);
}

// dB[n, k] = cast( sum_s partial[s][n][k] ), s in increasing order.
template <int DT>
__global__ void db_reduce_kernel(const float* __restrict__ partial, uint16_t* __restrict__ dB, int N,
                                 int K, long long lddb, int splits) {
  const long long pair = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // two elements per thread
  const long long total = (long long)N * K / 2;
  if (pair >= total) return;
  const long long idx = pair * 2;
  const int n = (int)(idx / K), k = (int)(idx % K);
  float2 acc = make_float2(0.f, 0.f);
  for (int s = 0; s < splits; ++s) {
    const float2 v = *reinterpret_cast<const float2*>(partial + ((long long)s * N + n) * K + k);
    acc.x += v.x;
    acc.y += v.y;
  }
  *reinterpret_cast<uint32_t*>(dB + (long long)n * lddb + k) = Elem<DT>::pack(acc.x, acc.y);
}

int db_default_splits(int M, int N, int K, int BN, int num_sms) {
  const int base = 2 * ((K + 255) / 256) * (N / BN);
  const int tokblocks = (M + 127) / 128;
  if (base >= 2 * num_sms) return 1;
  int s = (2 * num_sms + base - 1) / base;
  if (s > tokblocks) s = tokblocks;
  if (s > 16) s = 16;
  return s < 1 ? 1 : s;
}

int launch_bwd_db(const DbArgs& a) {
  DbParams p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.gs = a.gs; p.E = a.E; p.BN = a.BN;
  p.ntiles_per_group = a.gs / a.BN;
  p.n_tokblocks = (a.M + 127) / 128;
  p.splits = a.splits;
  p.blocks_per_split = (p.n_tokblocks + a.splits - 1) / a.splits;
  // drop splits that would own no token block
  p.splits = (p.n_tokblocks + p.blocks_per_split - 1) / p.blocks_per_split;
  p.dc_tiles = (a.BN / 2 + 63) / 64;   // per CTA: half of the tile's dC columns
  p.r_tile_bytes = ((a.E * 128) + 1023) / 1024 * 1024;
  p.scale = a.scale;
  p.dB = a.dB; p.lddb = a.lddb; p.partial = a.partial; p.err = a.err;
  if (p.splits > 1 && a.partial == nullptr)
    return fail(PRISM_ERR_WORKSPACE, "bwd_db: split accumulation needs a partial-sum workspace");

  const int budget = 227 * 1024 - 1024 - (int)sizeof(DbBarriers) - 256 - 2 * p.r_tile_bytes;
  const int a_bytes = 2 * db::kTile, d_bytes = p.dc_tiles * db::kTile;
  int sa = 2, sd = 2;
  if (sa * a_bytes + sd * d_bytes > budget)
    return fail(PRISM_ERR_UNSUPPORTED, "bwd_db tile does not fit shared memory (BN=%d E=%d)", a.BN, a.E);
  bool grew = true;
  while (grew) {
    grew = false;
    if (sd < db::kMaxStages && sa * a_bytes + (sd + 1) * d_bytes <= budget) { ++sd; grew = true; }
    if (sa < db::kMaxStages && (sa + 1) * a_bytes + sd * d_bytes <= budget) { ++sa; grew = true; }
  }
  p.sa = sa; p.sd = sd;
  const int smem_bytes = 2 * p.r_tile_bytes + sa * a_bytes + sd * d_bytes + (int)sizeof(DbBarriers) + 1024;

  CUtensorMap tmA, tmR, tmdC;
  int rc;
  if ((rc = make_tmap_2d(&tmA, a.dtype, a.A, a.M, a.K, a.lda, 128, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmR, a.dtype, a.R_eff, (uint64_t)(a.N / a.gs) * a.E, a.K, a.ldr, a.E, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmdC, a.dtype, a.dC, a.M, a.N, a.lddc, 128, 64, true))) return rc;

  using KernT = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, DbParams);
  KernT kern = nullptr;
#define PRISM_PICK(E_)                                                                               \
  kern = (a.dtype == DT_BF16)                                                                        \
             ? (a.gate == GATE_SILU ? (KernT)prism_bwd_db_kernel<DT_BF16, GATE_SILU, E_> : (KernT)prism_bwd_db_kernel<DT_BF16, GATE_NONE, E_>) \
             : (a.gate == GATE_SILU ? (KernT)prism_bwd_db_kernel<DT_F16, GATE_SILU, E_> : (KernT)prism_bwd_db_kernel<DT_F16, GATE_NONE, E_>)
  if (a.E == 16) { PRISM_PICK(16); } else if (a.E == 32) { PRISM_PICK(32); } else { PRISM_PICK(64); }
#undef PRISM_PICK
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return fail(PRISM_ERR_CUDA, "bwd_db: cannot set %d B of shared memory: %s", smem_bytes, cudaGetErrorString(e));
  dim3 grid(2 * ((a.K + 255) / 256), a.N / a.BN, p.splits);   // x: CTA pairs of 2 x 128 features
  kern<<<grid, db::kThreads, smem_bytes, a.stream>>>(tmA, tmR, tmdC, p);
  if ((rc = check_launch("prism_bwd_db"))) return rc;
  if (p.splits > 1) {
    const long long pairs = (long long)a.N * a.K / 2;
    const int threads = 256;
    const long long blocks = (pairs + threads - 1) / threads;
    if (a.dtype == DT_BF16)
      db_reduce_kernel<DT_BF16><<<(unsigned)blocks, threads, 0, a.stream>>>(a.partial, reinterpret_cast<uint16_t*>(a.dB), a.N, a.K, a.lddb, p.splits);
    else
      db_reduce_kernel<DT_F16><<<(unsigned)blocks, threads, 0, a.stream>>>(a.partial, reinterpret_cast<uint16_t*>(a.dB), a.N, a.K, a.lddb, p.splits);
    if ((rc = check_launch("prism_bwd_db reduce"))) return rc;
  }
  return PRISM_OK;
}

}  // namespace prism
