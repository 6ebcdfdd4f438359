// Prism backward, weight gradient, for sm_100a:
//   dB_g [gs, K] = scale * dC_g^T [gs, M] . H_g [M, K],   H_g = A * silu(A . blockdiag(R_g)^T)
// (H_g = A . blockdiag(R_g)^T in plain mode), with H recomputed on chip.
//
// Replaces the reference's dB_pc_kernel / prism_backward_dB_launch
// (cute_prism_backward_db.cu:450-582) and its binding (torch_ext/prism_bwd_db_torch.cu:42-162).
//
// CTAs work in pairs (cluster of 2, tcgen05 cta_group::2).  A pair owns one accumulator tile
// D[f, n] (256 features x BN outputs of one group; each CTA holds its 128 features in its own TMEM
// and loads half of the dC columns) and a contiguous range of 128-token blocks.  The contraction of
// the dense product runs over tokens, so both its operands are "MN-major": H tiles [128 tokens x 64
// features] and dC tiles [128 tokens x 64 outputs] are used as the gate warps / TMA lay them out.
//   warp 0      TMA: R_g tiles once; per token block two A tiles and ceil(BN/128) dC tiles
//   warps 1, 2  MMA issuers (leader), one per product.  Rotation S = A_blk . R_blk^T per rotation block
//               as tcgen05.mma M256 N=2E K=16.  The two CTAs hold different features, hence different R blocks; an
//               MMA spanning both takes its N rows half from each CTA, so it multiplies every row by
//               both R blocks: a CTA's own product lands in columns [rank*E, rank*E+E) of the block's
//               2E columns of S, the other half is ignored.
//   warps 4-19  gate warps, 16 token rows x 64 features each: S from TMEM, A by ldmatrix, H = A*silu(S)
//               on registers, stmatrix of H over the A tile in place
//               Dense product D += H^T . dC as 8 x tcgen05.mma M256 N=BN K=16 per token block.
//   warps 20-23 epilogue: D -> dB (transposed store), or fp32 partials when the token range is split;
//               a second kernel then adds the partials in a fixed order (deterministic).
// Both products run on tcgen05: mma.sync would share the tensor cores with tcgen05.mma and starve
// behind it.
#include "prism_host.cuh"
#include "prism_kernels.cuh"

namespace prism {

namespace db {
constexpr int kThreads = 768;
constexpr int kWarpTma = 0, kWarpMma = 1, kWarpRot = 2;
constexpr int kGateWarp0 = 4;      // multiple of 4: (warp & 3) is the TMEM lane quarter a warp may touch
constexpr int kNumGateWarps = 16;  // 8 row groups x 2 feature tiles
constexpr int kEpiWarp0 = kGateWarp0 + kNumGateWarps;   // 20
constexpr int kMaxStages = 4;
constexpr int kTile = 128 * 128;   // bytes of a [128 x 64] 16-bit tile
constexpr int kSCol0 = 256;        // accumulator: TMEM columns [0, 256); S: [256, 512)
}  // namespace db

struct DbParams {
  int M, N, K, gs, E, BN;
  int ntiles_per_group;
  int blocks_per_split, n_tokblocks;
  int dc_tiles;       // ceil(BN / 128): 64-column dC tiles per CTA
  int r_tile_bytes;   // bytes reserved per R tile (multiple of 1024)
  int ns;             // stages: two A tiles + this CTA's dC tiles
  int stage_bytes;
  int splits;
  int out_f32;        // 1: dB is fp32
  float scale;
  const void* ib;     // internal bias [G, K] or null
  const long long* drop_seeds;   // per-group dropout seeds (DROP kernels)
  float drop_p, drop_inv_keep;
  void* dB;
  long long lddb;
  float* partial;     // [splits][part_rows][K] when splits > 1
  int nt0;            // first n-tile of this launch (blockIdx.y counts from it)
  int part_rows;      // output rows covered by the partial buffer, starting at row nt0 * BN
  int* err;
};

struct DbBarriers {
  uint64_t r_full;                     // local: this CTA's R tiles landed (once)
  uint64_t a_full[db::kMaxStages];     // leader's copy is used: both CTAs' A tiles landed
  uint64_t hd_full[db::kMaxStages];    // leader's copy is used: gate warps of both CTAs wrote H, dC halves landed
  uint64_t stage_free[db::kMaxStages]; // local, multicast commit: the dense product has read the stage
  uint64_t s_full;                     // local, multicast commit: S of the token block is in TMEM
  uint64_t s_free;                     // leader's copy is used: the gate warps of both CTAs hold S in registers
  uint64_t acc_full;
  uint32_t tmem_base;
};

template <int DT, int GATE, int E, bool DROP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(db::kThreads, 1)
prism_bwd_db_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmR,
                    const __grid_constant__ CUtensorMap tmdC, const DbParams p) {
  using namespace db;
  constexpr int KS = E / 16;    // K16 steps per rotation block
  constexpr int NBLK = 128 / E; // rotation blocks of this CTA's 128 features
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* smemR = smem;                           // two R tiles [E x 64]
  uint8_t* smemSt = smemR + 2 * p.r_tile_bytes;    // stages: [A tile f0.. | A tile f0+64.. | dC tiles]
  DbBarriers* bars = reinterpret_cast<DbBarriers*>(smemSt + p.ns * p.stage_bytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0 = leader (issues the MMAs), 1 = peer
  const int f0 = blockIdx.x * 128;           // first of this CTA's 128 features (column of A / dB)
  const int nt = blockIdx.y + p.nt0;
  const int n0 = nt * p.BN;                  // first output (row of dB)
  const int g = nt / p.ntiles_per_group;
  const int split = blockIdx.z;
  const int tb0 = split * p.blocks_per_split;
  const int nb = min(p.blocks_per_split, p.n_tokblocks - tb0);  // token blocks of this CTA (>= 1)

  if (threadIdx.x == 0) {
    mbar_init(&bars->r_full, 1);
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(&bars->a_full[i], 2);                        // one arrive.expect_tx per CTA
      mbar_init(&bars->hd_full[i], 2 * kNumGateWarps + 2);   // gate warps of both CTAs + one arrive.expect_tx per CTA
      mbar_init(&bars->stage_free[i], 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->s_free, 2 * kNumGateWarps);
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
      mbar_arrive_expect_tx(&bars->r_full, 2 * E * 128);
      tma_load_2d(smemR, &tmR, &bars->r_full, f0, g * E);
      tma_load_2d(smemR + p.r_tile_bytes, &tmR, &bars->r_full, f0 + 64, g * E);
      // the rotation issuer (leader) reads the peer's R tiles too: it learns of them through the peer's
      // first A tiles, which are issued after this wait
      if (!mbar_wait(&bars->r_full, 0)) ok = false;
      Ring rs(p.ns);
      for (int j = 0; j < nb && ok; ++j, rs.next()) {
        const int tok0 = (tb0 + j) * 128;
        if (!mbar_wait(&bars->stage_free[rs.idx], rs.phase ^ 1)) { ok = false; break; }
        uint8_t* dst = smemSt + rs.idx * p.stage_bytes;
        // completion is counted on the leader's barriers: its MMAs read both CTAs' tiles
        const uint32_t afull = mapa_shared(smem_u32(&bars->a_full[rs.idx]), 0);
        mbar_arrive_expect_tx_cluster(afull, 2 * kTile);
        tma_load_2d_pair(dst, &tmA, afull, f0, tok0);
        tma_load_2d_pair(dst + kTile, &tmA, afull, f0 + 64, tok0);
        const uint32_t hdfull = mapa_shared(smem_u32(&bars->hd_full[rs.idx]), 0);
        mbar_arrive_expect_tx_cluster(hdfull, p.dc_tiles * kTile);
        for (int t = 0; t < p.dc_tiles; ++t)   // this CTA's half of the dC columns
          tma_load_2d_pair(dst + (2 + t) * kTile, &tmdC, hdfull, n0 + (int)rank * (p.BN / 2) + 64 * t, tok0);
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp == kWarpRot) {
    // ------------------------------------------------------------------ MMA issuer 1: rotation
    // S is single-buffered (TMEM: 256 columns of accumulator, 256 of S).  The gate warps copy their S
    // values to registers first thing and release the buffer, so the rotation of block j + 1 runs
    // while they still work on block j.  Rotation and dense product have an issuing thread each:
    // issuing costs a thread 60-80 clocks per MMA, a barrier test ~65, a commit ~90.
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_r = make_idesc(DT, 256, 2 * E, 0, 0);   // rows: both CTAs' tokens; N: E rows of R from each CTA
      const uint64_t da0 = desc_kmajor_sw128(smem_u32(smemSt), 1024);
      const uint64_t dr0 = desc_kmajor_sw128(smem_u32(smemR), 1024);
      const uint32_t k_hi = (uint32_t)(da0 >> 32);
      const uint32_t st_step = (uint32_t)p.stage_bytes >> 4;
      const uint32_t r_step = (uint32_t)p.r_tile_bytes >> 4;
      const uint32_t s0 = tmem_base + kSCol0;
      bool ok = true;
      Ring rr(p.ns);
      for (int j = 0; j < nb && ok; ++j, rr.next()) {
        if (j > 0) {   // the gate warps hold S of block j - 1 in registers
          if (!mbar_wait_cluster(&bars->s_free, (uint32_t)(j - 1) & 1)) { ok = false; break; }
        }
        if (!mbar_wait_cluster(&bars->a_full[rr.idx], rr.phase)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t a_lo = (uint32_t)da0 + rr.idx * st_step;
#pragma unroll
        for (int b = 0; b < NBLK; ++b) {
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
            // features b*E + ks*16 .. +16 of the CTA's 128: tile (64 features) and 32-byte step inside it
            const int fo = b * E + ks * 16;
            const uint32_t ta = (uint32_t)((fo >> 6) * (kTile >> 4) + ((fo & 63) >> 4) * 2);
            const uint32_t tr = (uint32_t)(fo >> 6) * r_step + (uint32_t)(((fo & 63) >> 4) * 2);
            umma_f16_pair_lh(s0 + b * 2 * E, a_lo + ta, k_hi, (uint32_t)dr0 + tr, k_hi, idesc_r, ks > 0 ? 1u : 0u);
          }
        }
        umma_commit_pair(&bars->s_full, 0x3);
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA issuer 2: dense product
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_d = make_idesc(DT, 256, p.BN, 1, 1);    // M = 256: 128 features in each CTA
      const uint64_t dh0 = desc_mnmajor_sw128(smem_u32(smemSt), kTile, 1024);
      const uint64_t dd0 = desc_mnmajor_sw128(smem_u32(smemSt) + 2 * kTile, kTile, 1024);
      const uint32_t h_hi = (uint32_t)(dh0 >> 32), d_hi = (uint32_t)(dd0 >> 32);
      const uint32_t st_step = (uint32_t)p.stage_bytes >> 4;
      bool ok = true;
      Ring rd(p.ns);
      for (int j = 0; j < nb && ok; ++j, rd.next()) {
        // gate warps done with block j: H written; the dC halves landed
        if (!mbar_wait_cluster(&bars->hd_full[rd.idx], rd.phase)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t h_lo = (uint32_t)dh0 + rd.idx * st_step;
        const uint32_t d_lo = (uint32_t)dd0 + rd.idx * st_step;
        umma_f16_pair_lh(tmem_base, h_lo, h_hi, d_lo, d_hi, idesc_d, j > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 1; ks < 8; ++ks)   // 16 tokens = 2048 bytes further on in both tiles
          umma_f16_pair_lh(tmem_base, h_lo + ks * 128, h_hi, d_lo + ks * 128, d_hi, idesc_d, 1u);
        umma_commit_pair(&bars->stage_free[rd.idx], 0x3);
        if (j == nb - 1) umma_commit_pair(&bars->acc_full, 0x3);
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp >= kGateWarp0 && warp < kEpiWarp0) {
    // ------------------------------------------------------------------ gate warps
    const uint32_t gw = warp - kGateWarp0;
    const uint32_t r0 = (gw & 3) * 32 + ((gw >> 2) & 1) * 16;   // 16 token rows inside the warp's TMEM lane quarter
    const uint32_t ft = gw >> 3;                                // which 64-feature tile
    // S of rotation block b sits in columns [2E b, 2E b + 2E); this CTA's product in the rank-th half
    const uint32_t s_tmem = tmem_base + (r0 << 16) + kSCol0 + ft * (64 / E) * 2 * E + rank * E;
    const uint32_t s_free_addr = mapa_shared(smem_u32(&bars->s_free), 0);
    // internal bias of this warp's 64 features (columns of A), the same for every token block
    const int kcol = f0 + (int)ft * 64;
    const int kvalid = p.K - kcol;
    const uint16_t* ib = (p.ib != nullptr && kvalid > 0)
                             ? reinterpret_cast<const uint16_t*>(p.ib) + (long long)g * p.K + kcol : nullptr;
    const uint64_t drop_h1 = DROP ? drop_group_hash(p.drop_seeds, g) : 0ull;
    bool ok = true;
    Ring rs(p.ns);
    for (int j = 0; j < nb && ok; ++j, rs.next()) {
      if (!mbar_wait(&bars->s_full, j & 1)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t tile = smem_u32(smemSt + rs.idx * p.stage_bytes + ft * kTile);
      DropCtx dc;
      if (DROP) {
        dc.h1 = drop_h1;
        dc.base = (long long)((tb0 + j) * 128 + (int)r0 + (lane >> 2)) * p.K + kcol + 2 * (lane & 3);
        dc.row8 = 8ll * p.K;
        dc.p = p.drop_p;
        dc.inv_keep = p.drop_inv_keep;
      }
      gate_rows16_tmem_smem<DT, GATE, E, DROP>(s_tmem, 2 * E, tile, r0, lane, s_free_addr, ib, kvalid, &dc);
      fence_proxy_async_smem();   // H was written by the generic proxy, the MMA reads it through the async proxy
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&bars->hd_full[rs.idx]), 0));
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
            float* dst = p.partial + ((long long)split * p.part_rows + (n0 - p.nt0 * p.BN) + c0) * p.K + f;
#pragma unroll
            for (int j = 0; j < 16; ++j) dst[(long long)j * p.K] = __uint_as_float(v[j]) * p.scale;
          } else if (p.out_f32) {
            float* dst = reinterpret_cast<float*>(p.dB) + (long long)(n0 + c0) * p.lddb + f;
#pragma unroll
            for (int j = 0; j < 16; ++j) dst[(long long)j * p.lddb] = __uint_as_float(v[j]) * p.scale;
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
template <int DT, bool F32OUT>
__global__ void db_reduce_kernel(const float* __restrict__ partial, void* __restrict__ dB_out, int N,
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
  if (F32OUT)
    *reinterpret_cast<float2*>(reinterpret_cast<float*>(dB_out) + (long long)n * lddb + k) = acc;
  else
    *reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(dB_out) + (long long)n * lddb + k) = Elem<DT>::pack(acc.x, acc.y);
}

static int db_default_splits(int M, int N, int K, int BN, int num_sms) {
  const int base = 2 * ((K + 255) / 256) * (N / BN);
  const int tokblocks = (M + 127) / 128;
  if (base >= 2 * num_sms) return 1;
  int s = (2 * num_sms + base - 1) / base;
  if (s > tokblocks) s = tokblocks;
  if (s > 16) s = 16;
  return s < 1 ? 1 : s;
}

// Launch plan.  cfg = {BN, splits} or null: splits > 0 splits the token range of every tile, splits < 0
// never splits.  Default: tiles that fill the GPU at least once are not split; when their count
// leaves a last wave that is mostly empty, the last n-tile rows go to a second launch whose token
// range is split so that it fills the GPU too (its partial sums cover those rows only).
void db_plan(int M, int N, int K, int BN, int num_sms, const int* cfg, DbPlan* pl) {
  pl->splits = 1; pl->tail_rows = 0; pl->tail_splits = 1;
  const int user = cfg ? cfg[1] : 0;
  if (user > 0) { pl->splits = user; return; }
  if (user < 0 || BN <= 0) return;
  pl->splits = db_default_splits(M, N, K, BN, num_sms);
  if (pl->splits != 1) return;
  const int x_pairs = (K + 255) / 256, rows = N / BN, slots = num_sms / 2 > 0 ? num_sms / 2 : 1;
  const int tiles = x_pairs * rows, tokblocks = (M + 127) / 128;
  if (tiles <= slots) return;
  const int tail = tiles % slots;
  if (tail == 0 || 2 * tail > slots) return;          // the last wave is full enough
  const int yb = (tail + x_pairs - 1) / x_pairs;       // n-tile rows that hold the tail
  int sb = slots / (yb * x_pairs);
  if (sb > 16) sb = 16;
  if (sb > tokblocks) sb = tokblocks;
  if (sb < 2 || yb >= rows) return;
  pl->tail_rows = yb;
  pl->tail_splits = sb;
}

int launch_bwd_db(const DbArgs& a) {
  DbParams p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.gs = a.gs; p.E = a.E; p.BN = a.BN;
  p.ntiles_per_group = a.gs / a.BN;
  p.n_tokblocks = (a.M + 127) / 128;
  p.dc_tiles = (a.BN / 2 + 63) / 64;   // per CTA: half of the tile's dC columns
  p.r_tile_bytes = ((a.E * 128) + 1023) / 1024 * 1024;
  p.scale = a.scale; p.out_f32 = a.out_f32; p.ib = a.ib;
  const bool drop = a.drop_seeds != nullptr && a.drop_p > 0.f && a.gate != GATE_NONE;
  p.drop_seeds = a.drop_seeds; p.drop_p = a.drop_p; p.drop_inv_keep = drop ? 1.f / (1.f - a.drop_p) : 1.f;
  if (drop && a.E != 16) return fail(PRISM_ERR_UNSUPPORTED, "bwd_db: dropout needs reconn_sz 8 or 16");
  p.dB = a.dB; p.lddb = a.lddb; p.partial = a.partial; p.err = a.err;
  if ((a.plan.splits > 1 || a.plan.tail_rows > 0) && a.partial == nullptr)
    return fail(PRISM_ERR_WORKSPACE, "bwd_db: split accumulation needs a partial-sum workspace");

  const int budget = 227 * 1024 - 1024 - (int)sizeof(DbBarriers) - 256 - 2 * p.r_tile_bytes;
  p.stage_bytes = (2 + p.dc_tiles) * db::kTile;
  int ns = db::kMaxStages;
  while (ns > 2 && ns * p.stage_bytes > budget) --ns;
  if (ns * p.stage_bytes > budget)
    return fail(PRISM_ERR_UNSUPPORTED, "bwd_db tile does not fit shared memory (BN=%d E=%d)", a.BN, a.E);
  p.ns = ns;
  const int smem_bytes = 2 * p.r_tile_bytes + ns * p.stage_bytes + (int)sizeof(DbBarriers) + 1024;

  CUtensorMap tmA, tmR, tmdC;
  int rc;
  if ((rc = make_tmap_2d(&tmA, a.dtype, a.A, a.M, a.K, a.lda, 128, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmR, a.dtype, a.R_eff, (uint64_t)(a.N / a.gs) * a.E, a.K, a.ldr, a.E, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmdC, a.dtype, a.dC, a.M, a.N, a.lddc, 128, 64, true))) return rc;

  using KernT = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, DbParams);
  KernT kern = nullptr;
#define PRISM_PICK_G(DT_, E_, DROP_)                                                                    \
  (a.gate == GATE_SILU ? (KernT)prism_bwd_db_kernel<DT_, GATE_SILU, E_, DROP_>                           \
                       : a.gate == GATE_SIGMOID ? (KernT)prism_bwd_db_kernel<DT_, GATE_SIGMOID, E_, DROP_> : (KernT)prism_bwd_db_kernel<DT_, GATE_NONE, E_, false>)
#define PRISM_PICK(E_) kern = (a.dtype == DT_BF16) ? PRISM_PICK_G(DT_BF16, E_, false) : PRISM_PICK_G(DT_F16, E_, false)
  if (drop) { kern = (a.dtype == DT_BF16) ? PRISM_PICK_G(DT_BF16, 16, true) : PRISM_PICK_G(DT_F16, 16, true); }
  else if (a.E == 16) { PRISM_PICK(16); } else if (a.E == 32) { PRISM_PICK(32); } else { PRISM_PICK(64); }
#undef PRISM_PICK_G
#undef PRISM_PICK
  if ((rc = set_max_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes, "bwd_db"))) return rc;
  const int rows = a.N / a.BN;
  // one launch over the n-tile rows [nt0, nt0 + nrows) with the token range of every tile split `splits` ways
  auto launch = [&](int nt0, int nrows, int splits) -> int {
    DbParams q = p;
    q.nt0 = nt0;
    q.part_rows = nrows * a.BN;
    q.blocks_per_split = (p.n_tokblocks + splits - 1) / splits;
    q.splits = (p.n_tokblocks + q.blocks_per_split - 1) / q.blocks_per_split;   // drop splits that would own no token block
    dim3 grid(2 * ((a.K + 255) / 256), nrows, q.splits);   // x: CTA pairs of 2 x 128 features
    kern<<<grid, db::kThreads, smem_bytes, a.stream>>>(tmA, tmR, tmdC, q);
    int rcl;
    if ((rcl = check_launch("prism_bwd_db"))) return rcl;
    if (q.splits > 1) {
      const long long pairs = (long long)q.part_rows * a.K / 2;
      const int threads = 256;
      const long long blocks = (pairs + threads - 1) / threads;
      void* out = reinterpret_cast<uint8_t*>(a.dB) + (long long)nt0 * a.BN * a.lddb * (a.out_f32 ? 4 : 2);
#define PRISM_DB_REDUCE(DT_, F32_) \
  db_reduce_kernel<DT_, F32_><<<(unsigned)blocks, threads, 0, a.stream>>>(a.partial, out, q.part_rows, a.K, a.lddb, q.splits)
      if (a.dtype == DT_BF16) { if (a.out_f32) PRISM_DB_REDUCE(DT_BF16, true); else PRISM_DB_REDUCE(DT_BF16, false); }
      else { if (a.out_f32) PRISM_DB_REDUCE(DT_F16, true); else PRISM_DB_REDUCE(DT_F16, false); }
#undef PRISM_DB_REDUCE
      if ((rcl = check_launch("prism_bwd_db reduce"))) return rcl;
    }
    return PRISM_OK;
  };
  if ((rc = launch(0, rows - a.plan.tail_rows, a.plan.splits))) return rc;
  if (a.plan.tail_rows > 0) {
    if ((rc = launch(rows - a.plan.tail_rows, a.plan.tail_rows, a.plan.tail_splits))) return rc;
  }
  return PRISM_OK;
}

}  // namespace prism
