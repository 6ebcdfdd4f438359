// Prism backward, input and rotation gradients: second-level reductions, launch plan and launcher of
// prism_bwd_dadr_kernel (prism_bwd_dadr_kernel.cuh; its instances live in prism_bwd_dadr_f16.cu and
// prism_bwd_dadr_bf16.cu).
#include "prism_bwd_dadr_kernel.cuh"

namespace prism {

// dR[g*rs + i, k] = cast( scale * sum of the CTAs' partial sums ), in a fixed order: the main CTAs'
// buffers in increasing order, then, for every run, the slabs of the extra pair that helped the
// main pair (run, column of k).  For rs = 8 two neighbouring blocks share one 16-row group of the
// partial buffers: the block in the upper 8 columns of each 16-column pair sits in rows 8..15.
template <int DT, bool F32OUT>
__global__ void dr_reduce_kernel(const float* __restrict__ partial, const float* __restrict__ partial_x,
                                 void* __restrict__ dR_out, int G, int rs, int E, int K, long long lddr, int runs,
                                 int n_ft, int n_main, int n_extra, int steal, int slots, float scale) {
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
  const long long prow = (long long)g * E + ip;
  float2 acc = make_float2(0.f, 0.f);
  for (int r = 0; r < 2 * runs; ++r) {
    const float2 v = *reinterpret_cast<const float2*>(partial + ((long long)r * GE + prow) * K + k);
    acc.x += v.x;
    acc.y += v.y;
  }
  if (steal > 0) {
    const int fx = k >> 7, kk = k & 127;
    for (int run = 0; run < runs; ++run) {
      const int m = run * n_ft + fx;
      const int e = ((m + 1) * n_extra - 1) / n_main;   // the extra pair that helps main pair m
      const int mi = m - e * n_main / n_extra;
      for (int rank = 0; rank < 2; ++rank) {
        const float2 v = *reinterpret_cast<const float2*>(
            partial_x + (((long long)(e * 2 + rank) * slots + mi) * GE + prow) * 128 + kk);
        acc.x += v.x;
        acc.y += v.y;
      }
    }
  }
  if (F32OUT)   // the fp32 sums leave as they are (mixed-precision optimisers)
    *reinterpret_cast<float2*>(reinterpret_cast<float*>(dR_out) + (long long)row * lddr + k) = make_float2(acc.x * scale, acc.y * scale);
  else
    *reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(dR_out) + (long long)row * lddr + k) = Elem<DT>::pack(acc.x * scale, acc.y * scale);
}

// d_ib[g, k] = cast( scale * sum of the CTAs' column sums of dS ), in the same fixed order as dR.
template <int DT>
__global__ void dib_reduce_kernel(const float* __restrict__ partial, const float* __restrict__ partial_x,
                                  uint16_t* __restrict__ d_ib, int G, int K, long long ldib, int runs, int n_ft,
                                  int n_main, int n_extra, int steal, int slots, float scale) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)G * K) return;
  const int k = (int)(idx % K), g = (int)(idx / K);
  float acc = 0.f;
  for (int r = 0; r < 2 * runs; ++r) acc += partial[((long long)r * G + g) * K + k];
  if (steal > 0) {
    const int fx = k >> 7, kk = k & 127;
    for (int run = 0; run < runs; ++run) {
      const int m = run * n_ft + fx;
      const int e = ((m + 1) * n_extra - 1) / n_main;
      const int mi = m - e * n_main / n_extra;
      for (int rank = 0; rank < 2; ++rank)
        acc += partial_x[(((long long)(e * 2 + rank) * slots + mi) * G + g) * 128 + kk];
    }
  }
  d_ib[(long long)g * ldib + k] = (uint16_t)(Elem<DT>::pack(acc * scale, 0.f) & 0xffffu);
}

// Grid of the dA+dR kernel.  runs: the number of main CTA pairs that share one feature column (each
// walks every runs-th 256-token tile).  When the main pairs leave SM pairs idle and have enough
// tiles each, the idle pairs become extra pairs and every main pair leaves its last `steal` tiles
// to them (see DadrUnit): measured faster than many short runs, with a quarter of the workspace.
// cfg (or null): {runs, steal, n_extra}; 0 = default; steal < 0 = no extra pairs.
void dadr_plan_grid(int M, int K, int num_sms, const int* cfg, DadrGrid* gr) {
  const int n_ft = (K + 127) / 128;
  const int n_mp = (M + 255) / 256;
  const int slots_sm = num_sms / 2 > 0 ? num_sms / 2 : 1;
  int runs = (cfg && cfg[0] > 0) ? cfg[0] : 0;
  if (runs <= 0) {
    runs = 1;
    if (n_ft <= slots_sm) {
      // one wave: the count that leaves the fewest tiles per pair (ties: fewer pairs, less workspace);
      // the SM pairs that stay idle become extra pairs below
      int best_tiles = n_mp;
      for (int r = 2; r <= n_mp && n_ft * r <= slots_sm; ++r) {
        const int tiles = (n_mp + r - 1) / r;
        if (tiles < best_tiles) { best_tiles = tiles; runs = r; }
      }
    } else {
      // more columns than SM pairs: minimise (waves of pairs) x (tiles per pair)
      long long best_cost = -1;
      for (int r = 1; r <= n_mp && r <= 32; ++r) {
        const long long waves = ((long long)n_ft * r + slots_sm - 1) / slots_sm;
        const long long cost = waves * ((n_mp + r - 1) / r);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; runs = r; }
      }
    }
  }
  if (runs > n_mp) runs = n_mp;
  if (runs < 1) runs = 1;
  gr->runs = runs;
  gr->n_ft = n_ft;
  gr->n_main = n_ft * runs;
  gr->n_extra = 0; gr->steal = 0; gr->slots = 0;
  const int t_min = n_mp / runs, t_max = (n_mp + runs - 1) / runs;   // tiles of the shortest / longest run
  int steal = cfg ? cfg[1] : 0;
  int n_extra = (cfg && cfg[2] > 0) ? cfg[2] : (slots_sm - gr->n_main);
  if (steal < 0 || n_extra < 1) return;
  if (n_extra > gr->n_main) n_extra = gr->n_main;
  const int cnt_max = (gr->n_main + n_extra - 1) / n_extra;          // main pairs per extra pair
  if (steal == 0) {
    steal = (t_max * n_extra + (gr->n_main + n_extra) / 2) / (gr->n_main + n_extra);
    while (steal > 0 && cnt_max * steal > t_max - steal) --steal;   // an extra pair must not become the longest
  }
  if (steal > t_min - 1) steal = t_min - 1;                           // every main pair keeps a tile
  if (steal < 1) return;
  gr->n_extra = n_extra; gr->steal = steal; gr->slots = cnt_max;
}

template <int E>
static int dadr_plan(DadrParams& p, int& smem_bytes, bool ib) {
  using St = dadr::Stage<E>;
  p.rr_tile_bytes = ((E / 2 * 128) + 1023) / 1024 * 1024;
  p.rd_tile_bytes = ((E * 128) + 1023) / 1024 * 1024;
  p.rb = (E <= 16) ? 4 : 2;
  const int fixed = 6 * dadr::kTile + p.rb * 2 * (p.rr_tile_bytes + p.rd_tile_bytes) + (int)sizeof(DadrBarriers) + 1024 +
                    (ib ? 8192 : 0);
  int ns = (227 * 1024 - 256 - fixed) / St::kBytes;
  if (ns > dadr::kMaxStages) ns = dadr::kMaxStages;
  if (ns < 2) return fail(PRISM_ERR_UNSUPPORTED, "bwd_dadr does not fit shared memory (E=%d)", E);
  p.ns = ns;
  smem_bytes = fixed + ns * St::kBytes;
  return PRISM_OK;
}

int launch_bwd_dadr(const DadrArgs& a) {
  DadrParams p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.gs = a.gs; p.E = a.E; p.G = a.N / a.gs;
  p.n_mtiles = (a.M + 127) / 128;
  p.runs = a.grid.runs;
  p.n_ft = a.grid.n_ft; p.n_main = a.grid.n_main;
  p.n_extra = a.grid.n_extra; p.steal = a.grid.steal; p.slots = a.grid.slots;
  p.partial_x = a.partial_x;
  p.scale = a.scale;
  p.dA = a.dA; p.ldda = a.ldda; p.partial = a.partial; p.err = a.err;
  int smem_bytes = 0;
  const bool ib = a.ib != nullptr && a.gate != GATE_NONE;
  DadrExtra x;
  x.ib = ib ? a.ib : nullptr; x.partial_ib = a.partial_ib; x.partial_ib_x = a.partial_ib_x;
  int rc = (a.E == 16) ? dadr_plan<16>(p, smem_bytes, ib) : (a.E == 32) ? dadr_plan<32>(p, smem_bytes, ib) : dadr_plan<64>(p, smem_bytes, ib);
  if (rc) return rc;
  const int stage_out = 64;

  CUtensorMap tmA, tmRr, tmRd, tmdC, tmB;
  if ((rc = make_tmap_2d(&tmA, a.dtype, a.A, a.M, a.K, a.lda, 128, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmRr, a.dtype, a.R_eff, (uint64_t)p.G * a.E, a.K, a.ldr, a.E / 2, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmRd, a.dtype, a.R_eff, (uint64_t)p.G * a.E, a.K, a.ldr, a.E, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmdC, a.dtype, a.dC, a.M, a.N, a.lddc, 128, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmB, a.dtype, a.B, a.N, a.K, a.ldb, stage_out, 64, true))) return rc;

  const bool drop = a.drop_seeds != nullptr && a.drop_p > 0.f && a.gate != GATE_NONE;
  if (drop && a.E != 16) return fail(PRISM_ERR_UNSUPPORTED, "bwd_dadr: dropout needs reconn_sz 8 or 16");
  x.drop_seeds = a.drop_seeds; x.drop_p = a.drop_p; x.drop_inv_keep = drop ? 1.f / (1.f - a.drop_p) : 1.f;
  DadrKernel kern = (a.dtype == DT_BF16) ? dadr_kernel_bf16(a.gate, a.E, ib, drop) : dadr_kernel_f16(a.gate, a.E, ib, drop);
  if ((rc = set_max_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes, "bwd_dadr"))) return rc;
  dim3 grid(2 * (p.n_main + p.n_extra), 1, 1);   // the two CTAs of a pair are neighbours
  kern<<<grid, dadr::kThreads, smem_bytes, a.stream>>>(tmA, tmRr, tmRd, tmdC, tmB, p, x);
  if ((rc = check_launch("prism_bwd_dadr"))) return rc;

  // gated mode: the kernel formed 2 dS against the halved R tiles, so the dR partials are doubled
  const float r_scale = (a.gate != GATE_NONE) ? 0.5f * a.scale : a.scale;
  const long long pairs = (long long)p.G * a.rs * a.K / 2;
  const int threads = 256;
  const long long blocks = (pairs + threads - 1) / threads;
#define PRISM_DR_REDUCE(DT_, F32_)                                                                          \
  dr_reduce_kernel<DT_, F32_><<<(unsigned)blocks, threads, 0, a.stream>>>(a.partial, a.partial_x, a.dR, p.G, a.rs, a.E, \
      a.K, a.lddr, p.runs, p.n_ft, p.n_main, p.n_extra, p.steal, p.slots, r_scale)
  if (a.dtype == DT_BF16) { if (a.dr_f32) PRISM_DR_REDUCE(DT_BF16, true); else PRISM_DR_REDUCE(DT_BF16, false); }
  else { if (a.dr_f32) PRISM_DR_REDUCE(DT_F16, true); else PRISM_DR_REDUCE(DT_F16, false); }
#undef PRISM_DR_REDUCE
  if ((rc = check_launch("prism_bwd_dadr reduce"))) return rc;
  if (ib) {
    const long long n = (long long)p.G * a.K;
    const long long nblocks = (n + threads - 1) / threads;
    if (a.dtype == DT_BF16)
      dib_reduce_kernel<DT_BF16><<<(unsigned)nblocks, threads, 0, a.stream>>>(a.partial_ib, a.partial_ib_x, reinterpret_cast<uint16_t*>(a.d_ib), p.G, a.K, a.K, p.runs, p.n_ft, p.n_main, p.n_extra, p.steal, p.slots, r_scale);
    else
      dib_reduce_kernel<DT_F16><<<(unsigned)nblocks, threads, 0, a.stream>>>(a.partial_ib, a.partial_ib_x, reinterpret_cast<uint16_t*>(a.d_ib), p.G, a.K, a.K, p.runs, p.n_ft, p.n_main, p.n_extra, p.steal, p.slots, r_scale);
    return check_launch("prism_bwd_dadr internal-bias reduce");
  }
  return PRISM_OK;
}

}  // namespace prism
