// Prism forward for few tokens (M <= 128), for sm_100a: the decode-sized calls, which are bound by
// streaming B from HBM, not by the tensor cores.
//
//   C[:, group g] = H_g @ B_g^T,  H_g = A * silu(A . blockdiag(R_g)^T)   (or H_g = A . blockdiag(R_g)^T)
//
// The reference has no such path: its forward kernel tiles 128 tokens x 128 outputs without
// predication (cute_prism_coop_pc.cu:670-673), so a one-token call costs a full tile per group.
// Here the problem is turned around: the 128 rows of a B tile are the M dimension of the MMA and the
// tokens its N dimension (16 ... 128), so one tcgen05.mma per 16 K elements consumes 4 KB of B
// whatever the token count, and every SM streams an equal share of B exactly once:
//   * work unit = (group g, 64-wide K chunk): the group's gs x 64 slice of B (gs/128 tiles), the
//     token chunk A[:, 64] and the R_g chunk.  The G * ceil(K/64) units, group-major, are cut into
//     one contiguous range per CTA (one CTA per SM), so a group's K range is shared by a few CTAs.
//   * per unit: rotation S = A_chunk . R_g^T on tcgen05 (tokens as M, N = E per rotation block) into
//     TMEM, gate warps turn S into H in place over the A tile in shared memory, then
//     D_j[128 outputs, tokens] += B_tile_j . H^T for the gs/128 row tiles j.
//   * at the end of a group's share the CTA writes its fp32 partial [tokens, gs] to the workspace;
//     a second small kernel (launched with programmatic stream serialisation, so that its launch
//     latency hides behind this kernel) adds a group's partials in CTA order (a fixed order: the
//     result is bit-stable), adds the bias, casts and writes C.
// B is loaded with the evict-first L2 hint (it is read once), so the partial sums stay in L2.
//   warp 0       TMA producer            warps 1, 2   MMA issuers: dense product, rotation (an issuing
//                                                     thread spends 60-80 clocks per MMA, one could not keep up)
//   warps 4-11   gate warps, 16 tokens each         warps 12-19  epilogue (partial sums to the workspace)
#include "prism_host.cuh"
#include "prism_kernels.cuh"

namespace prism {

namespace fsm {
constexpr int kThreads = 640;
constexpr int kWarpTma = 0, kWarpMma = 1, kWarpRot = 2;
constexpr int kGateWarp0 = 4;       // multiple of 4: (warp & 3) is the TMEM lane quarter a warp may touch
constexpr int kNumGateWarps = 8;    // 16 token rows each
constexpr int kEpiWarp0 = 12;       // multiple of 4
constexpr int kNumEpiWarps = 8;    // two per TMEM lane quarter: each takes half of the token columns
constexpr int kMaxStages = 6;
constexpr int kTile = 128 * 128;    // bytes of a [128 x 64] 16-bit tile
constexpr int kSCol0 = 256;         // TMEM: accumulators in [0, 256), two S slots of 64 columns from 256
constexpr int kMaxRowTiles = 4;
}  // namespace fsm

struct FwdSmallParams {
  int M, N, K, gs, E, G;
  int Mp;              // tokens rounded up to 16: rows of the A box, N of the dense MMA
  int nrt;             // 128-row tiles of B per group (gs / 128)
  int nk;              // 64-wide K chunks
  int units, ncta;     // G * nk work units over ncta CTAs
  int pmax;            // partial slots per group
  int ns, stage_bytes, a_off, r_off, b_off;
  const void* bias;
  const void* ib;      // internal bias [G, K] or null
  const long long* drop_seeds;   // per-group dropout seeds (DROP kernels)
  float drop_p, drop_inv_keep;
  void* C;
  long long ldc;
  float* partial;      // [G][pmax][Mp][gs] fp32
  int* err;
};

struct FwdSmallBarriers {
  uint64_t full[fsm::kMaxStages];    // TMA: the unit's tiles landed
  uint64_t empty[fsm::kMaxStages];   // commit: the dense product has read the stage
  uint64_t h_full[fsm::kMaxStages];  // gate warps wrote H over the A tile
  uint64_t s_full[2];                // commit: S of the unit is in its TMEM slot
  uint64_t s_free[2];                // gate warps hold S in registers
  uint64_t acc_full;                 // commit: the accumulators hold a group's share
  uint64_t acc_empty;                // epilogue warps have read them
  uint32_t tmem_base;
};

// CTA that owns work unit x when `units` units are cut into `ncta` contiguous ranges [c*units/ncta, (c+1)*units/ncta)
__device__ __host__ __forceinline__ int fsm_owner(long long x, int units, int ncta) {
  return (int)(((x + 1) * ncta + units - 1) / units) - 1;
}

template <int DT, int GATE, int E, bool DROP>
__global__ void __launch_bounds__(fsm::kThreads, 1)
prism_fwd_small_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmR,
                       const __grid_constant__ CUtensorMap tmB, const FwdSmallParams p) {
  using namespace fsm;
  constexpr int KS = E / 16;   // K16 steps per rotation block
  constexpr int NB = 64 / E;   // rotation blocks per chunk
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // stage: [A tile (Mp rows) | R tile (E rows) | gs/128 B tiles]; the rotation MMA reads 128 rows from the
  // A tile's start whatever the token count: what lies behind the Mp loaded rows (R, B) only feeds S rows
  // that nobody reads
  uint8_t* smemSt = smem;
  FwdSmallBarriers* bars = reinterpret_cast<FwdSmallBarriers*>(smemSt + p.ns * p.stage_bytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const int u0 = (int)((long long)cta * p.units / p.ncta);
  const int u1 = (int)((long long)(cta + 1) * p.units / p.ncta);
  const int n_gate = p.Mp / 16;   // gate warps with token rows

  if (threadIdx.x == 0) {
    // the reduction kernel (launched with programmatic stream serialisation) may be scheduled from now on:
    // its blocks sit in their dependency wait until this grid has finished, so its launch latency is hidden
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1);
      mbar_init(&bars->h_full[i], n_gate);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->s_free[i], n_gate);
    }
    mbar_init(&bars->acc_full, 1);
    mbar_init(&bars->acc_empty, kNumEpiWarps);
    fence_mbar_init();
    // the first loads leave before the rest of the CTA is set up (this thread is the TMA producer)
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmR);
  }
  if (warp == kWarpMma) {
    tmem_alloc_cta(&bars->tmem_base, 512);
    tmem_relinquish_cta();
  }
  // the producer fills the ring's first pass before the CTA-wide synchronisation: nothing else has
  // touched these stages yet, so their "empty" barriers need no wait
  const uint64_t pol = l2_policy_evict_first();
  const uint32_t stage_tx = (uint32_t)(p.nrt * kTile + p.Mp * 128 + E * 128);
  int pre = 0;
  if (threadIdx.x == 0) {
    int g = u0 / p.nk, kc = u0 - g * p.nk;
    for (int u = u0; u < u1 && pre < p.ns; ++u, ++pre) {
      uint8_t* dst = smemSt + pre * p.stage_bytes;
      mbar_arrive_expect_tx(&bars->full[pre], stage_tx);
      for (int j = 0; j < p.nrt; ++j)
        tma_load_2d_hint(dst + p.b_off + j * kTile, &tmB, &bars->full[pre], kc * 64, g * p.gs + j * 128, pol);
      tma_load_2d(dst + p.a_off, &tmA, &bars->full[pre], kc * 64, 0);
      tma_load_2d(dst + p.r_off, &tmR, &bars->full[pre], kc * 64, g * E);
      if (++kc == p.nk) { kc = 0; ++g; }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == kWarpTma) {
    // ------------------------------------------------------------------ TMA producer (units after the first pass)
    if (lane == 0) {
      const uint32_t bytes = stage_tx;
      Ring rs(p.ns);
      bool ok = true;
      const int us = u0 + pre;
      int g = us / p.nk, kc = us - g * p.nk;
      if (pre == p.ns) rs.phase = 1;   // the ring has been filled once: idx 0 again, second pass
      else rs.idx = (uint32_t)pre;
      for (int u = us; u < u1; ++u, rs.next()) {
        if (!mbar_wait(&bars->empty[rs.idx], rs.phase ^ 1)) { ok = false; break; }
        uint8_t* dst = smemSt + rs.idx * p.stage_bytes;
        mbar_arrive_expect_tx(&bars->full[rs.idx], bytes);
        for (int j = 0; j < p.nrt; ++j)
          tma_load_2d_hint(dst + p.b_off + j * kTile, &tmB, &bars->full[rs.idx], kc * 64, g * p.gs + j * 128, pol);
        tma_load_2d(dst + p.a_off, &tmA, &bars->full[rs.idx], kc * 64, 0);
        tma_load_2d(dst + p.r_off, &tmR, &bars->full[rs.idx], kc * 64, g * E);
        if (++kc == p.nk) { kc = 0; ++g; }
      }
      if (!ok) atomicExch(p.err, PRISM_ERR_DEVICE_WAIT);
    }
  } else if (warp == kWarpRot) {
    // ------------------------------------------------------------------ MMA issuer 1: rotation S = A_chunk . R_g^T
    if (lane == 0) {
      const uint32_t idesc_r = make_idesc(DT, 128, E, 0, 0);        // S block: M = 128 token rows, N = E
      const uint64_t d0 = desc_kmajor_sw128(smem_u32(smemSt), 1024);
      const uint32_t d_hi = (uint32_t)(d0 >> 32);
      const uint32_t st_step = (uint32_t)p.stage_bytes >> 4;
      const uint32_t a_off = (uint32_t)p.a_off >> 4, r_off = (uint32_t)p.r_off >> 4;
      Ring rl(p.ns);
      bool ok = true;
      const int n = u1 - u0;
      for (int i = 0; i < n; ++i, rl.next()) {
        const uint32_t slot = (uint32_t)i & 1u;
        if (i >= 2) {   // the gate warps hold S of unit i - 2 in registers
          if (!mbar_wait(&bars->s_free[slot], (((uint32_t)i >> 1) - 1) & 1)) { ok = false; break; }
        }
        if (!mbar_wait(&bars->full[rl.idx], rl.phase)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t base = (uint32_t)d0 + rl.idx * st_step;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
            const int kk = b * KS + ks;   // K16 step inside the chunk: +32 bytes on both operands
            umma_f16_cta_lh(tmem_base + kSCol0 + slot * 64 + b * E, base + a_off + kk * 2, d_hi,
                            base + r_off + kk * 2, d_hi, idesc_r, ks > 0 ? 1u : 0u);
          }
        }
        umma_commit_cta(&bars->s_full[slot]);
      }
      if (!ok) atomicExch(p.err, PRISM_ERR_DEVICE_WAIT);
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA issuer 2: dense product D_j += B_j . H^T
    if (lane == 0) {
      const uint32_t idesc_d = make_idesc(DT, 128, p.Mp, 0, 0);     // D tile: M = 128 outputs, N = tokens
      const uint64_t d0 = desc_kmajor_sw128(smem_u32(smemSt), 1024);
      const uint32_t d_hi = (uint32_t)(d0 >> 32);
      const uint32_t st_step = (uint32_t)p.stage_bytes >> 4;
      const uint32_t a_off = (uint32_t)p.a_off >> 4, b_off = (uint32_t)p.b_off >> 4;
      Ring rd(p.ns);
      uint32_t acc_phase = 0;
      bool ok = true;
      const int n = u1 - u0;
      int kc = u0 - (u0 / p.nk) * p.nk;
      bool seg_first = true;   // first unit of this CTA's share of a group
      for (int i = 0; i < n; ++i, rd.next()) {
        const bool seg_last = (i == n - 1) || (kc == p.nk - 1);
        if (!mbar_wait(&bars->h_full[rd.idx], rd.phase)) { ok = false; break; }   // H written (so the tiles landed too)
        if (seg_first) {
          if (!mbar_wait(&bars->acc_empty, acc_phase ^ 1)) { ok = false; break; }
        }
        tc_fence_after_sync();
        const uint32_t base = (uint32_t)d0 + rd.idx * st_step;
        for (int j = 0; j < p.nrt; ++j) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16_cta_lh(tmem_base + j * p.Mp, base + b_off + j * (kTile >> 4) + ks * 2, d_hi, base + a_off + ks * 2, d_hi,
                            idesc_d, (seg_first && ks == 0) ? 0u : 1u);
        }
        umma_commit_cta(&bars->empty[rd.idx]);
        if (seg_last) {
          umma_commit_cta(&bars->acc_full);
          acc_phase ^= 1u;
        }
        seg_first = seg_last;
        if (++kc == p.nk) kc = 0;
      }
      if (!ok) atomicExch(p.err, PRISM_ERR_DEVICE_WAIT);
    }
  } else if (warp >= kGateWarp0 && warp < kGateWarp0 + kNumGateWarps) {
    // ------------------------------------------------------------------ gate warps
    const uint32_t gw = warp - kGateWarp0;
    const uint32_t r0 = (gw & 3) * 32 + ((gw >> 2) & 1) * 16;   // this warp's 16 token rows inside its lane quarter
    if ((int)r0 < p.Mp) {
      Ring rs(p.ns);
      bool ok = true;
      const int n = u1 - u0;
      const uint16_t* ibase = reinterpret_cast<const uint16_t*>(p.ib);
      int g = u0 / p.nk, kc = u0 - g * p.nk;
      for (int i = 0; i < n; ++i, rs.next()) {
        const uint32_t slot = (uint32_t)i & 1u;
        if (!mbar_wait(&bars->s_full[slot], ((uint32_t)i >> 1) & 1)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tile = smem_u32(smemSt + rs.idx * p.stage_bytes + p.a_off);
        const uint16_t* ib = ibase != nullptr ? ibase + (long long)g * p.K + kc * 64 : nullptr;
        DropCtx dc;
        if (DROP) {
          dc.h1 = drop_group_hash(p.drop_seeds, g);
          dc.base = (long long)((int)r0 + (lane >> 2)) * p.K + kc * 64 + 2 * (lane & 3);
          dc.row8 = 8ll * p.K;
          dc.p = p.drop_p;
          dc.inv_keep = p.drop_inv_keep;
        }
        gate_rows16_tmem_smem<DT, GATE, E, DROP>(tmem_base + (r0 << 16) + kSCol0 + slot * 64, E, tile, r0, lane,
                                                 smem_u32(&bars->s_free[slot]), ib, p.K - kc * 64, &dc);
        if (++kc == p.nk) { kc = 0; ++g; }
        fence_proxy_async_smem();   // H was written by the generic proxy, the MMA reads it through the async proxy
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->h_full[rs.idx]);
      }
      if (!ok && lane == 0) atomicExch(p.err, PRISM_ERR_DEVICE_WAIT);
    }
  } else if (warp >= kEpiWarp0) {
    // ------------------------------------------------------------------ epilogue warps
    const int q = warp & 3;
    uint32_t acc_phase = 0;
    bool ok = true;
    int g = u0 / p.nk;
    int u = u0;
    while (u < u1 && ok) {
      const int seg_end = min(u1, (g + 1) * p.nk);
      const int piece = cta - fsm_owner((long long)g * p.nk, p.units, p.ncta);
      if (!mbar_wait(&bars->acc_full, acc_phase)) { ok = false; break; }
      acc_phase ^= 1u;
      tc_fence_after_sync();
      float* part = p.partial + ((long long)(g * p.pmax + piece) * p.Mp) * p.gs;
      // 16-token column chunks, alternating between the quarter's two warps
      const int hsel = (warp - kEpiWarp0) >> 2;
      for (int j = 0; j < p.nrt; ++j) {
        for (int c0 = hsel * 16; c0 < p.Mp; c0 += 32) {
          uint32_t v[16];
          tmem_ld_x16(tmem_base + (uint32_t(q * 32) << 16) + j * p.Mp + c0, v);
          tmem_ld_wait();
          // row = output j*128 + q*32 + lane, columns = tokens c0 .. c0+15: one coalesced row segment per token
#pragma unroll
          for (int t = 0; t < 16; ++t)
            part[(long long)(c0 + t) * p.gs + j * 128 + q * 32 + lane] = __uint_as_float(v[t]);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty);
      u = seg_end;
      ++g;
    }
    if (!ok && lane == 0) atomicExch(p.err, PRISM_ERR_DEVICE_WAIT);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kWarpMma) tmem_dealloc_cta(tmem_base, 512);
}

// C[tok, n] = cast( sum of the partials of n's group in CTA order + bias[n] ).  Launched with
// programmatic stream serialisation: it may become resident while the main kernel still runs and
// waits here until that kernel's memory operations are complete and visible.
template <int DT>
__global__ void prism_fwd_small_reduce_kernel(const float* __restrict__ partial, const uint16_t* __restrict__ bias,
                                              uint16_t* __restrict__ C, int M, int N, int gs, int Mp, int nk, int units,
                                              int ncta, int pmax, long long ldc) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int half_n = N >> 1;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)M * half_n) return;
  const int tok = (int)(idx / half_n);
  const int n = (int)(idx - (long long)tok * half_n) * 2;
  const int g = n / gs, nl = n - g * gs;
  const int pieces = fsm_owner((long long)(g + 1) * nk - 1, units, ncta) - fsm_owner((long long)g * nk, units, ncta) + 1;
  const float* gp = partial + ((long long)g * pmax * Mp + tok) * gs + nl;
  float2 acc = make_float2(0.f, 0.f);
  for (int pc = 0; pc < pieces; ++pc) {
    const float2 x = __ldcg(reinterpret_cast<const float2*>(gp + (long long)pc * Mp * gs));
    acc.x += x.x;
    acc.y += x.y;
  }
  if (bias != nullptr) {
    const float2 b2 = Elem<DT>::unpack(*reinterpret_cast<const uint32_t*>(bias + n));
    acc.x += b2.x;
    acc.y += b2.y;
  }
  *reinterpret_cast<uint32_t*>(C + (long long)tok * ldc + n) = Elem<DT>::pack(acc.x, acc.y);
}

// ----------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------
static void fwd_small_partition(int G, int nk, int num_sms, int* units, int* ncta, int* pmax) {
  *units = G * nk;
  *ncta = num_sms < *units ? num_sms : *units;
  int pm = 1;
  for (int g = 0; g < G; ++g) {
    const int c_first = fsm_owner((long long)g * nk, *units, *ncta);
    const int c_last = fsm_owner((long long)(g + 1) * nk - 1, *units, *ncta);
    if (c_last - c_first + 1 > pm) pm = c_last - c_first + 1;
  }
  *pmax = pm;
}

// Token count up to which the streaming kernel is the default: measured at K = 4096, N = 14336, gs = 256
// it wins up to 48 tokens (31.7-37.9 us against 40-41 us), ties at 64 and loses above (its fp32
// partial sums, written and read back, grow with the token count).
bool fwd_small_preferred(int M) { return M <= 48; }

bool fwd_small_supported(int M, int N, int K, int gs, int E) {
  if (M < 1 || M > 128 || E < 16 || E > 64) return false;
  if (gs % 128 != 0 || gs / 128 > fsm::kMaxRowTiles) return false;
  const int Mp = (M + 15) / 16 * 16;
  return (gs / 128) * Mp <= fsm::kSCol0;   // the accumulators fit below the S slots in TMEM
}

// bytes of scratch after the status header and the rotation copy: the partial sums
size_t fwd_small_scratch_bytes(int M, int N, int K, int gs, int num_sms) {
  const int G = N / gs, nk = (K + 63) / 64, Mp = (M + 15) / 16 * 16;
  int units, ncta, pmax;
  fwd_small_partition(G, nk, num_sms, &units, &ncta, &pmax);
  return ((size_t)G * pmax * Mp * gs * 4 + 255) & ~size_t(255);
}

int launch_fwd_small(const FwdArgs& a, void* scratch) {
  FwdSmallParams p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.gs = a.gs; p.E = a.E; p.G = a.N / a.gs;
  p.Mp = (a.M + 15) / 16 * 16;
  p.nrt = a.gs / 128;
  p.nk = (a.K + 63) / 64;
  fwd_small_partition(p.G, p.nk, a.num_sms, &p.units, &p.ncta, &p.pmax);
  p.bias = a.bias; p.ib = a.ib; p.C = a.C; p.ldc = a.ldc; p.err = a.err;
  const bool drop = a.drop_seeds != nullptr && a.drop_p > 0.f && a.gate != GATE_NONE;
  p.drop_seeds = a.drop_seeds; p.drop_p = a.drop_p; p.drop_inv_keep = drop ? 1.f / (1.f - a.drop_p) : 1.f;
  if (drop && a.E != 16) return fail(PRISM_ERR_UNSUPPORTED, "forward: dropout needs reconn_sz 8 or 16");
  p.partial = reinterpret_cast<float*>(scratch);
  // stage: A tile (Mp rows), R tile, B tiles, each on a 1024-byte boundary (128-byte swizzle atoms)
  p.a_off = 0;
  p.r_off = ((p.Mp * 128 + 1023) / 1024) * 1024;
  p.b_off = p.r_off + ((a.E * 128 + 1023) / 1024) * 1024;
  p.stage_bytes = p.b_off + p.nrt * fsm::kTile;   // >= 16 KB behind a_off in every stage
  const int budget = 227 * 1024 - 1024 - (int)sizeof(FwdSmallBarriers) - 256;
  int ns = budget / p.stage_bytes;
  if (ns > fsm::kMaxStages) ns = fsm::kMaxStages;
  if (ns < 2) return fail(PRISM_ERR_UNSUPPORTED, "small-M forward does not fit shared memory (gs=%d E=%d)", a.gs, a.E);
  p.ns = ns;
  const int smem_bytes = ns * p.stage_bytes + (int)sizeof(FwdSmallBarriers) + 1024;

  CUtensorMap tmA, tmR, tmB;
  int rc;
  if ((rc = make_tmap_2d(&tmA, a.dtype, a.A, a.M, a.K, a.lda, p.Mp, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmR, a.dtype, a.R_eff, (uint64_t)p.G * a.E, a.K, a.ldr, a.E, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmB, a.dtype, a.B, a.N, a.K, a.ldb, 128, 64, true))) return rc;

  using KernT = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, FwdSmallParams);
  KernT kern = nullptr;
#define PRISM_PICK_G(DT_, E_, DROP_)                                                                    \
  (a.gate == GATE_SILU ? (KernT)prism_fwd_small_kernel<DT_, GATE_SILU, E_, DROP_>                        \
                       : a.gate == GATE_SIGMOID ? (KernT)prism_fwd_small_kernel<DT_, GATE_SIGMOID, E_, DROP_> : (KernT)prism_fwd_small_kernel<DT_, GATE_NONE, E_, false>)
#define PRISM_PICK(E_) kern = (a.dtype == DT_BF16) ? PRISM_PICK_G(DT_BF16, E_, false) : PRISM_PICK_G(DT_F16, E_, false)
  if (drop) { kern = (a.dtype == DT_BF16) ? PRISM_PICK_G(DT_BF16, 16, true) : PRISM_PICK_G(DT_F16, 16, true); }
  else if (a.E == 16) { PRISM_PICK(16); } else if (a.E == 32) { PRISM_PICK(32); } else { PRISM_PICK(64); }
#undef PRISM_PICK_G
#undef PRISM_PICK
  if ((rc = set_max_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes, "small-M forward"))) return rc;
  kern<<<p.ncta, fsm::kThreads, smem_bytes, a.stream>>>(tmA, tmR, tmB, p);
  if ((rc = check_launch("prism_fwd_small"))) return rc;

  // second level: add the partial sums (programmatic stream serialisation hides its launch latency)
  const long long pairs = (long long)a.M * (a.N / 2);
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3((unsigned)((pairs + 255) / 256));
  lc.blockDim = dim3(256);
  lc.dynamicSmemBytes = 0;
  lc.stream = a.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  const float* part = p.partial;
  const uint16_t* bias = reinterpret_cast<const uint16_t*>(a.bias);
  uint16_t* out = reinterpret_cast<uint16_t*>(a.C);
  cudaError_t e;
  if (a.dtype == DT_BF16)
    e = cudaLaunchKernelEx(&lc, prism_fwd_small_reduce_kernel<DT_BF16>, part, bias, out, a.M, a.N, a.gs, p.Mp, p.nk, p.units,
                           p.ncta, p.pmax, a.ldc);
  else
    e = cudaLaunchKernelEx(&lc, prism_fwd_small_reduce_kernel<DT_F16>, part, bias, out, a.M, a.N, a.gs, p.Mp, p.nk, p.units,
                           p.ncta, p.pmax, a.ldc);
  if (e != cudaSuccess) return fail(PRISM_ERR_CUDA, "small-M forward reduce: launch failed: %s", cudaGetErrorString(e));
  return check_launch("prism_fwd_small reduce");
}

}  // namespace prism
