// Prism backward, input and rotation gradients, for sm_100a:
//   dH_g = dC_g . B_g                                   (dense, tcgen05)
//   S_g  = A . blockdiag(R_g)^T                         (recomputed, tcgen05 M128 N=E K=16)
//   gated:  dS = dH * A * silu'(S),  dA += dH * silu(S) + blockdiag(dS) . R_g
//   plain:  dS = dH,                 dA += blockdiag(dS) . R_g
//   dR_g[block b] = dS_b^T . A_b                        (mma.sync on ldmatrix.trans fragments)
// summed over groups g for dA and over tokens for dR.
//
// Replaces the reference's bwd_dadr_kernel + dR_reduce_kernel + prism_backward_dA_dR_launch
// (cute_prism_backward_dadr.cu:735-995) and its binding (torch_ext/prism_bwd_dadr_torch.cu:42-210).
// The reference adds dR partials with fp32 atomicAdd (cute_prism_backward_dadr.cu:675-682); here
// every CTA owns one exclusive partial buffer that it updates in a fixed order, and a second
// kernel adds the buffers in a fixed order, so dR is bit-stable from run to run.
//
// One CTA works on a [128 tokens x 128 features] tile of dA and walks over all groups:
//   TMA warp   : A tiles once per tile; per group the R_g tiles and, per 64 outputs, a dC tile
//                [128 x 64] and two B_g tiles [64 x 64]
//   MMA warp   : S_g, dH_g (two TMEM buffers), and one group later dA += dS . R_g (TMEM)
//   gate warps : read S, dH (TMEM) and A (smem); keep sum_g dH*silu(S) in registers; write dS
//                (16-bit, swizzled) to shared memory; at the end of the tile add the TMEM part
//                and store dA
//   dR warps   : ldmatrix.trans of dS and A tiles, mma.sync m16n8k16 over the 128 tokens, then
//                read-modify-write of this CTA's fp32 partial buffer.
#include "prism_host.cuh"
#include "prism_kernels.cuh"

namespace prism {

namespace dadr {
constexpr int kThreads = 448;     // warp 0 TMA, warp 1 MMA, warps 2-9 gate, warps 10-13 dR
constexpr int kGateWarp0 = 2;
constexpr int kNumGateWarps = 8;
constexpr int kDrWarp0 = 10;
constexpr int kNumDrWarps = 4;
constexpr int kDhCol0 = 0;        // two dH buffers of 128 columns
constexpr int kSCol0 = 256;       // S buffer, 128 columns
constexpr int kDaCol0 = 384;      // dA accumulator, 128 columns
constexpr int kTile = 128 * 128;  // bytes of a [128 x 64] 16-bit tile
constexpr int kBTile = 64 * 128;  // bytes of a [64 x 64] 16-bit tile
constexpr int kStageBytes = kTile + 2 * kBTile;
constexpr int kMaxStages = 4;
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
  float* partial;      // [runs][G*E][K] fp32
  int* err;
};

struct DadrBarriers {
  uint64_t a_full, a_empty;
  uint64_t r_full[dadr::kMaxRBufs], r_empty[dadr::kMaxRBufs];
  uint64_t st_full[dadr::kMaxStages], st_empty[dadr::kMaxStages];
  uint64_t s_full, s_empty;
  uint64_t dh_full[2], dh_empty[2];
  uint64_t ds_full[2], ds_empty[2];
  uint64_t da_full, da_empty;
  uint32_t tmem_base;
};

template <int DT, int GATE>
__global__ void __launch_bounds__(dadr::kThreads, 1)
prism_bwd_dadr_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmR,
                      const __grid_constant__ CUtensorMap tmdC, const __grid_constant__ CUtensorMap tmB,
                      const DadrParams p) {
  using namespace dadr;
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
  const int f0 = blockIdx.x * 128;
  const int run = blockIdx.y;
  const int G = p.G;
  const int nstg = (p.gs + 63) / 64;  // 64-output slices per group

  if (threadIdx.x == 0) {
    mbar_init(&bars->a_full, 1);
    mbar_init(&bars->a_empty, 1 + kNumDrWarps);
    for (int i = 0; i < kMaxRBufs; ++i) { mbar_init(&bars->r_full[i], 1); mbar_init(&bars->r_empty[i], 1); }
    for (int i = 0; i < kMaxStages; ++i) { mbar_init(&bars->st_full[i], 1); mbar_init(&bars->st_empty[i], 1); }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->s_empty, kNumGateWarps);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->dh_full[i], 1);
      mbar_init(&bars->dh_empty[i], kNumGateWarps);
      mbar_init(&bars->ds_full[i], kNumGateWarps);
      mbar_init(&bars->ds_empty[i], 1 + kNumDrWarps);
    }
    mbar_init(&bars->da_full, 1);
    mbar_init(&bars->da_empty, kNumGateWarps);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmR);
    prefetch_tmap(&tmdC);
    prefetch_tmap(&tmB);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      uint32_t tile_iter = 0;
      Ring rr(p.rb), rst(p.ns);
      for (int mt = run; mt < p.n_mtiles && ok; mt += p.runs, ++tile_iter) {
        const int m0 = mt * 128;
        if (!mbar_wait(&bars->a_empty, (tile_iter & 1) ^ 1)) { ok = false; break; }
        mbar_arrive_expect_tx(&bars->a_full, 2 * kTile);
        tma_load_2d(smemA, &tmA, &bars->a_full, f0, m0);
        tma_load_2d(smemA + kTile, &tmA, &bars->a_full, f0 + 64, m0);
        for (int g = 0; g < G && ok; ++g, rr.next()) {
          const int rb = rr.idx;
          if (!mbar_wait(&bars->r_empty[rb], rr.phase ^ 1)) { ok = false; break; }
          uint8_t* dstR = smemR + rb * r_buf_bytes;
          mbar_arrive_expect_tx(&bars->r_full[rb], 2 * p.E * 128);
          tma_load_2d(dstR, &tmR, &bars->r_full[rb], f0, g * p.E);
          tma_load_2d(dstR + p.r_tile_bytes, &tmR, &bars->r_full[rb], f0 + 64, g * p.E);
          for (int s = 0; s < nstg; ++s, rst.next()) {
            const int st = rst.idx;
            if (!mbar_wait(&bars->st_empty[st], rst.phase ^ 1)) { ok = false; break; }
            uint8_t* dst = smemSt + st * kStageBytes;
            const int n0 = g * p.gs + s * 64;
            mbar_arrive_expect_tx(&bars->st_full[st], kStageBytes);
            tma_load_2d(dst, &tmdC, &bars->st_full[st], n0, m0);
            tma_load_2d(dst + kTile, &tmB, &bars->st_full[st], f0, n0);
            tma_load_2d(dst + kTile + kBTile, &tmB, &bars->st_full[st], f0 + 64, n0);
          }
        }
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(DT, 128, p.E, 0, 0);    // S  = A . R^T      (both K-major)
      const uint32_t idesc_h = make_idesc(DT, 128, 128, 0, 1);    // dH = dC . B       (B MN-major)
      const uint32_t idesc_r = make_idesc(DT, 128, p.E, 0, 1);    // dA += dS . R      (R MN-major)
      const int blocks_per_chunk = 64 / p.E;
      const int ksteps_per_block = p.E / 16;
      const uint32_t a_addr = smem_u32(smemA);
      bool ok = true;
      uint32_t tile_iter = 0, gg = 0;
      Ring rr(p.rb), rr_dsr(p.rb), rst(p.ns);

      // dA += dS(x) . R(x) for the group with global index x (called once per group, in order)
      auto issue_dsr = [&](uint32_t x, bool first_of_tile, bool last_of_tile, uint32_t titer) -> bool {
        const int buf = x & 1;
        const int rbx = rr_dsr.idx;
        rr_dsr.next();
        if (!mbar_wait(&bars->ds_full[buf], (x >> 1) & 1)) return false;
        if (first_of_tile) {
          if (!mbar_wait(&bars->da_empty, (titer & 1) ^ 1)) return false;
        }
        tc_fence_after_sync();
        const uint32_t ds_addr = smem_u32(smemDS + buf * 2 * kTile);
        const uint32_t r_addr = smem_u32(smemR + rbx * r_buf_bytes);
        for (int i = 0; i < 2; ++i) {
          for (int b = 0; b < blocks_per_chunk; ++b) {
            for (int ks = 0; ks < ksteps_per_block; ++ks) {
              umma_f16(tmem_base + kDaCol0 + i * 64 + b * p.E,
                       desc_kmajor_sw128(ds_addr + i * kTile + (b * p.E + ks * 16) * 2, 1024),
                       desc_mnmajor_sw128(r_addr + i * p.r_tile_bytes + b * p.E * 2 + ks * 2048,
                                          p.r_tile_bytes, 1024),
                       idesc_r, (!first_of_tile || ks > 0) ? 1u : 0u);
            }
          }
        }
        umma_commit(&bars->ds_empty[buf]);
        umma_commit(&bars->r_empty[rbx]);
        if (last_of_tile) {
          umma_commit(&bars->a_empty);
          umma_commit(&bars->da_full);
        }
        return true;
      };

      for (int mt = run; mt < p.n_mtiles && ok; mt += p.runs, ++tile_iter) {
        if (!mbar_wait(&bars->a_full, tile_iter & 1)) { ok = false; break; }
        for (int g = 0; g < G && ok; ++g, ++gg, rr.next()) {
          const int rb = rr.idx;
          const int hb = gg & 1;
          if (!mbar_wait(&bars->r_full[rb], rr.phase)) { ok = false; break; }
          if (GATE == GATE_SILU) {
            if (!mbar_wait(&bars->s_empty, (gg & 1) ^ 1)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t r_addr = smem_u32(smemR + rb * r_buf_bytes);
            for (int i = 0; i < 2; ++i) {
              for (int b = 0; b < blocks_per_chunk; ++b) {
                for (int ks = 0; ks < ksteps_per_block; ++ks) {
                  const uint32_t koff = (b * p.E + ks * 16) * 2;
                  umma_f16(tmem_base + kSCol0 + i * 64 + b * p.E,
                           desc_kmajor_sw128(a_addr + i * kTile + koff, 1024),
                           desc_kmajor_sw128(r_addr + i * p.r_tile_bytes + koff, 1024), idesc_s,
                           ks > 0 ? 1u : 0u);
                }
              }
            }
            umma_commit(&bars->s_full);
          }
          if (!mbar_wait(&bars->dh_empty[hb], ((gg >> 1) & 1) ^ 1)) { ok = false; break; }
          for (int s = 0; s < nstg; ++s, rst.next()) {
            const int st = rst.idx;
            if (!mbar_wait(&bars->st_full[st], rst.phase)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t dc_addr = smem_u32(smemSt + st * kStageBytes);
            const uint32_t b_addr = dc_addr + kTile;
            const int ksteps = min(4, (p.gs - s * 64) / 16);
            for (int ks = 0; ks < ksteps; ++ks) {
              umma_f16(tmem_base + kDhCol0 + hb * 128, desc_kmajor_sw128(dc_addr + ks * 32, 1024),
                       desc_mnmajor_sw128(b_addr + ks * 2048, kBTile, 1024), idesc_h,
                       (s > 0 || ks > 0) ? 1u : 0u);
            }
            umma_commit(&bars->st_empty[st]);
          }
          if (!ok) break;
          umma_commit(&bars->dh_full[hb]);
          if (g > 0) {
            if (!issue_dsr(gg - 1, g == 1, false, tile_iter)) { ok = false; break; }
          }
        }
        if (!ok) break;
        if (!issue_dsr(gg - 1, G == 1, true, tile_iter)) { ok = false; break; }
      }
      if (!ok) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
    }
  } else if (warp < kDrWarp0) {
    // ------------------------------------------------------------------ gate warps (+ dA epilogue)
    const int gw = warp - kGateWarp0;
    const int q = warp & 3;
    const int chunk = gw >> 2;
    const uint32_t row = q * 32 + lane;
    const uint32_t lane_base = uint32_t(q * 32) << 16;
    const uint8_t* tileA = smemA + chunk * kTile;
    float pacc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) pacc[i] = 0.f;
    bool ok = true;
    uint32_t tile_iter = 0, gg = 0;
    for (int mt = run; mt < p.n_mtiles && ok; mt += p.runs, ++tile_iter) {
      for (int g = 0; g < G && ok; ++g, ++gg) {
        const int hb = gg & 1;
        if (GATE == GATE_SILU) {
          if (!mbar_wait(&bars->s_full, gg & 1)) { ok = false; break; }
        }
        if (!mbar_wait(&bars->dh_full[hb], (gg >> 1) & 1)) { ok = false; break; }
        if (!mbar_wait(&bars->ds_empty[hb], ((gg >> 1) & 1) ^ 1)) { ok = false; break; }
        tc_fence_after_sync();
        uint8_t* tileDS = smemDS + hb * 2 * kTile + chunk * kTile;
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) {
          uint32_t dh[16], s[16];
          tmem_ld_x16(tmem_base + lane_base + kDhCol0 + hb * 128 + chunk * 64 + c0, dh);
          uint4 av[2];
          if (GATE == GATE_SILU) {
            tmem_ld_x16(tmem_base + lane_base + kSCol0 + chunk * 64 + c0, s);
            av[0] = *reinterpret_cast<const uint4*>(tileA + sw128_offset(row, c0 / 8));
            av[1] = *reinterpret_cast<const uint4*>(tileA + sw128_offset(row, c0 / 8 + 1));
          }
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            uint32_t aw[4] = {0, 0, 0, 0};
            if (GATE == GATE_SILU) { aw[0] = av[j].x; aw[1] = av[j].y; aw[2] = av[j].z; aw[3] = av[j].w; }
            uint32_t ow[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int c = j * 8 + e * 2;
              float d0 = __uint_as_float(dh[c]), d1 = __uint_as_float(dh[c + 1]);
              float ds0, ds1;
              if (GATE == GATE_SILU) {
                const float s0 = __uint_as_float(s[c]), s1 = __uint_as_float(s[c + 1]);
                const float2 a2 = Elem<DT>::unpack(aw[e]);
                const float sg0 = sigmoid_fast(s0), sg1 = sigmoid_fast(s1);
                const float t0 = s0 * sg0, t1 = s1 * sg1;            // silu(S)
                const float gp0 = fmaf(t0, 1.f - sg0, sg0);          // silu'(S) = sg + silu*(1-sg)
                const float gp1 = fmaf(t1, 1.f - sg1, sg1);
                pacc[c0 + c] = fmaf(d0, t0, pacc[c0 + c]);
                pacc[c0 + c + 1] = fmaf(d1, t1, pacc[c0 + c + 1]);
                ds0 = d0 * a2.x * gp0;
                ds1 = d1 * a2.y * gp1;
              } else {
                ds0 = d0;
                ds1 = d1;
              }
              ow[e] = Elem<DT>::pack(ds0, ds1);
            }
            *reinterpret_cast<uint4*>(tileDS + sw128_offset(row, c0 / 8 + j)) =
                make_uint4(ow[0], ow[1], ow[2], ow[3]);
          }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->ds_full[hb]);
          mbar_arrive(&bars->dh_empty[hb]);
          if (GATE == GATE_SILU) mbar_arrive(&bars->s_empty);
        }
      }
      if (!ok) break;
      // tile epilogue: dA = scale * (register part + tensor-core part)
      if (!mbar_wait(&bars->da_full, tile_iter & 1)) { ok = false; break; }
      tc_fence_after_sync();
      const long long grow = (long long)mt * 128 + row;
      uint16_t* drow = reinterpret_cast<uint16_t*>(p.dA) + grow * p.ldda + f0 + chunk * 64;
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 16) {
        uint32_t v[16];
        tmem_ld_x16(tmem_base + lane_base + kDaCol0 + chunk * 64 + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint32_t ow[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = j * 8 + e * 2;
            const float x0 = (__uint_as_float(v[c]) + pacc[c0 + c]) * p.scale;
            const float x1 = (__uint_as_float(v[c + 1]) + pacc[c0 + c + 1]) * p.scale;
            ow[e] = Elem<DT>::pack(x0, x1);
            pacc[c0 + c] = 0.f;
            pacc[c0 + c + 1] = 0.f;
          }
          if (grow < p.M && f0 + chunk * 64 + c0 + j * 8 < p.K)
            *reinterpret_cast<uint4*>(drow + c0 + j * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->da_empty);
    }
    if (!ok && lane == 0) { atomicExch(p.err, PRISM_ERR_DEVICE_WAIT); }
  } else {
    // ------------------------------------------------------------------ dR warps
    const int w = warp - kDrWarp0;
    const int sub_e = p.E / 16;                  // 16x16 sub-tiles per block edge
    const int spb = sub_e * sub_e;               // sub-tiles per block
    const int n_sub = (128 / p.E) * spb;         // sub-tiles of this CTA's 128 features
    const int bpc = 64 / p.E;
    const int mat = lane >> 3, l8 = lane & 7;
    const long long GE = (long long)G * p.E;
    float* part = p.partial + (long long)run * GE * p.K;
    bool ok = true;
    uint32_t tile_iter = 0, gg = 0;
    for (int mt = run; mt < p.n_mtiles && ok; mt += p.runs, ++tile_iter) {
      if (!mbar_wait(&bars->a_full, tile_iter & 1)) { ok = false; break; }
      for (int g = 0; g < G && ok; ++g, ++gg) {
        const int buf = gg & 1;
        if (!mbar_wait(&bars->ds_full[buf], (gg >> 1) & 1)) { ok = false; break; }
        for (int u = w; u < n_sub; u += kNumDrWarps) {
          const int block = u / spb, rem = u - block * spb;
          const int is = rem / sub_e, js = rem - is * sub_e;
          const int chunk = block / bpc, b = block - chunk * bpc;
          const uint32_t ds_tile = smem_u32(smemDS + buf * 2 * kTile + chunk * kTile);
          const uint32_t a_tile = smem_u32(smemA + chunk * kTile);
          const uint32_t ci = (b * p.E + is * 16) / 8;   // 16-byte chunk of the dS columns (i)
          const uint32_t cj = (b * p.E + js * 16) / 8;   // 16-byte chunk of the A columns (j)
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
          // accumulate into this CTA's partial buffer (fixed order: m-tiles ascending)
          const int r0 = g * p.E + is * 16 + (lane >> 2);
          const int col = f0 + chunk * 64 + b * p.E + js * 16 + (lane & 3) * 2;
          if (col < p.K) {
            float2* p00 = reinterpret_cast<float2*>(part + (long long)r0 * p.K + col);
            float2* p10 = reinterpret_cast<float2*>(part + (long long)(r0 + 8) * p.K + col);
            float2 v00 = make_float2(d0[0], d0[1]), v10 = make_float2(d0[2], d0[3]);
            if (tile_iter > 0) {
              const float2 o00 = *p00, o10 = *p10;
              v00.x += o00.x; v00.y += o00.y; v10.x += o10.x; v10.y += o10.y;
            }
            *p00 = v00; *p10 = v10;
          }
          if (col + 8 < p.K) {
            float2* p01 = reinterpret_cast<float2*>(part + (long long)r0 * p.K + col + 8);
            float2* p11 = reinterpret_cast<float2*>(part + (long long)(r0 + 8) * p.K + col + 8);
            float2 v01 = make_float2(d1[0], d1[1]), v11 = make_float2(d1[2], d1[3]);
            if (tile_iter > 0) {
              const float2 o01 = *p01, o11 = *p11;
              v01.x += o01.x; v01.y += o01.y; v11.x += o11.x; v11.y += o11.y;
            }
            *p01 = v01; *p11 = v11;
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

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// dR[g*rs + i, k] = cast( scale * sum_run partial[run][g*E + i'][k] ), runs in increasing order.
// For rs = 8 two neighbouring blocks share one 16-row group of the partial buffer:
// the block in the upper 8 columns of each 16-column pair sits in rows 8..15.
template <int DT>
__global__ void dr_reduce_kernel(const float* __restrict__ partial, uint16_t* __restrict__ dR, int G,
                                 int rs, int E, int K, long long lddr, int runs, int runs_alloc_rows,
                                 float scale) {
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
  (void)runs_alloc_rows;
  float2 acc = make_float2(0.f, 0.f);
  for (int r = 0; r < runs; ++r) {
    const float2 v = *reinterpret_cast<const float2*>(partial + ((long long)r * GE + (long long)g * E + ip) * K + k);
    acc.x += v.x;
    acc.y += v.y;
  }
  *reinterpret_cast<uint32_t*>(dR + (long long)row * lddr + k) = Elem<DT>::pack(acc.x * scale, acc.y * scale);
}

int dadr_default_runs(int M, int K, int num_sms) {
  const int n_ft = (K + 127) / 128;
  const int n_mt = (M + 127) / 128;
  // about two CTAs' worth of work per SM, but never more runs than token tiles
  int runs = (2 * num_sms + n_ft - 1) / n_ft;
  if (n_ft >= num_sms) runs = 1;
  if (runs > n_mt) runs = n_mt;
  if (runs > 64) runs = 64;
  return runs < 1 ? 1 : runs;
}

int launch_bwd_dadr(const DadrArgs& a) {
  DadrParams p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.gs = a.gs; p.E = a.E; p.G = a.N / a.gs;
  p.n_mtiles = (a.M + 127) / 128;
  p.runs = a.runs < 1 ? 1 : a.runs;
  if (p.runs > p.n_mtiles) p.runs = p.n_mtiles;
  p.r_tile_bytes = ((a.E * 128) + 1023) / 1024 * 1024;
  p.scale = a.scale;
  p.dA = a.dA; p.ldda = a.ldda; p.partial = a.partial; p.err = a.err;
  p.rb = (a.E <= 16) ? 4 : (a.E == 32 ? 3 : 2);
  const int fixed = 6 * dadr::kTile + p.rb * 2 * p.r_tile_bytes + (int)sizeof(DadrBarriers) + 1024 + 256;
  int ns = (227 * 1024 - fixed) / dadr::kStageBytes;
  if (ns > dadr::kMaxStages) ns = dadr::kMaxStages;
  if (ns < 2) return fail(PRISM_ERR_UNSUPPORTED, "bwd_dadr does not fit shared memory (E=%d)", a.E);
  p.ns = ns;
  const int smem_bytes = 6 * dadr::kTile + p.rb * 2 * p.r_tile_bytes + ns * dadr::kStageBytes +
                         (int)sizeof(DadrBarriers) + 1024;

  CUtensorMap tmA, tmR, tmdC, tmB;
  int rc;
  if ((rc = make_tmap_2d(&tmA, a.dtype, a.A, a.M, a.K, a.lda, 128, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmR, a.dtype, a.R_eff, (uint64_t)p.G * a.E, a.K, a.ldr, a.E, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmdC, a.dtype, a.dC, a.M, a.N, a.lddc, 128, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmB, a.dtype, a.B, a.N, a.K, a.ldb, 64, 64, true))) return rc;

  auto kern = (a.dtype == DT_BF16)
                  ? (a.gate == GATE_SILU ? prism_bwd_dadr_kernel<DT_BF16, GATE_SILU> : prism_bwd_dadr_kernel<DT_BF16, GATE_NONE>)
                  : (a.gate == GATE_SILU ? prism_bwd_dadr_kernel<DT_F16, GATE_SILU> : prism_bwd_dadr_kernel<DT_F16, GATE_NONE>);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return fail(PRISM_ERR_CUDA, "bwd_dadr: cannot set %d B of shared memory: %s", smem_bytes, cudaGetErrorString(e));
  dim3 grid((a.K + 127) / 128, p.runs, 1);
  kern<<<grid, dadr::kThreads, smem_bytes, a.stream>>>(tmA, tmR, tmdC, tmB, p);
  if ((rc = check_launch("prism_bwd_dadr"))) return rc;

  const long long pairs = (long long)p.G * a.rs * a.K / 2;
  const int threads = 256;
  const long long blocks = (pairs + threads - 1) / threads;
  if (a.dtype == DT_BF16)
    dr_reduce_kernel<DT_BF16><<<(unsigned)blocks, threads, 0, a.stream>>>(a.partial, reinterpret_cast<uint16_t*>(a.dR), p.G, a.rs, a.E, a.K, a.lddr, p.runs, 0, a.scale);
  else
    dr_reduce_kernel<DT_F16><<<(unsigned)blocks, threads, 0, a.stream>>>(a.partial, reinterpret_cast<uint16_t*>(a.dR), p.G, a.rs, a.E, a.K, a.lddr, p.runs, 0, a.scale);
  return check_launch("prism_bwd_dadr reduce");
}

}  // namespace prism
