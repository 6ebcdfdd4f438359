// Host-side launch interfaces of the three Prism kernels (internal to the library;
// the exported C ABI is declared in include/prism_b200.h).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace prism {

struct FwdArgs {
  const void* A;      // [M, K]
  const void* B;      // [N, K]
  const void* R_eff;  // [(N/gs)*E, K]  rotation blocks padded to E x E
  const void* bias;   // [N] or null
  const void* ib;     // internal bias [N/gs, K] (gated modes) or null
  const long long* drop_seeds;  // [N/gs] per-group dropout seeds, or null (no dropout)
  float drop_p;       // dropout probability (with drop_seeds)
  void* C;            // [M, N]
  int M, N, K, gs, E;
  int dtype, gate;
  long long lda, ldb, ldr, ldc;
  int BN, PM, sa, sb;  // tile configuration (0 = default)
  int num_sms;
  int* err;           // device status word
  cudaStream_t stream;
};
int launch_fwd(const FwdArgs& a);

// Few-token forward (M <= 128, group_size a multiple of 128): B tiles as the M dimension of the MMA,
// every SM streams an equal share of B once (prism_fwd_small.cu).  `scratch`: fwd_small_scratch_bytes
// bytes after the workspace's status header and rotation copy.
bool fwd_small_supported(int M, int N, int K, int gs, int E);
bool fwd_small_preferred(int M);   // token counts for which it is the default choice
size_t fwd_small_scratch_bytes(int M, int N, int K, int gs, int num_sms);
int launch_fwd_small(const FwdArgs& a, void* scratch);

// R [(G*8), K] -> R_eff [(G*16), K]: two neighbouring 8x8 blocks become one 16x16
// block-diagonal block, so that every rotation is a 16-wide tensor-core product.
int launch_expand_r8(const void* R, void* R_eff, int G, int K, long long ldr, int dtype, cudaStream_t stream);
// R_eff [(G*E), K] = factor * R (widened as above when rs = 8)
int launch_prep_r(const void* R, void* R_eff, int G, int rs, int E, int K, long long ldr, float factor, int dtype,
                  cudaStream_t stream);

// launch plan of the dB kernel (see db_plan in prism_bwd_db.cu)
struct DbPlan {
  int splits;       // token-range splits of every tile of the main launch
  int tail_rows;    // n-tile rows handled by a second launch (0: none) ...
  int tail_splits;  // ... with this many token-range splits
};
struct DbArgs {
  const void* dC;     // [M, N]
  const void* A;      // [M, K]
  const void* R_eff;  // [(N/gs)*E, K]
  const void* ib;     // internal bias [N/gs, K] (gated modes) or null
  const long long* drop_seeds;  // [N/gs] per-group dropout seeds, or null
  float drop_p;
  void* dB;           // [N, K], 16-bit like the inputs or fp32 (out_f32)
  int M, N, K, gs, E;
  int dtype, gate;
  int out_f32;        // 1: dB is written as fp32
  float scale;        // dB = scale * dC^T H
  long long lddc, lda, ldr, lddb;
  int BN;
  DbPlan plan;        // token-range splits of the main launch and of the tail rows
  float* partial;     // fp32 scratch of the split launch: [splits][rows it covers][K]
  int num_sms;
  int* err;
  cudaStream_t stream;
};
int launch_bwd_db(const DbArgs& a);
void db_plan(int M, int N, int K, int BN, int num_sms, const int* cfg, DbPlan* plan);

// grid of the dA+dR kernel (see dadr_plan_grid in prism_bwd_dadr.cu); cfg = {runs, steal, n_extra} or null
struct DadrGrid {
  int runs;      // main CTA pairs per 128-feature column
  int n_ft;      // 128-feature columns
  int n_main;    // n_ft * runs
  int n_extra;   // extra CTA pairs that take over the main pairs' last tiles (0: none)
  int steal;     // tiles every main pair leaves to them
  int slots;     // dR slabs per extra CTA
};
struct DadrArgs {
  const void* dC;     // [M, N]
  const void* A;      // [M, K]
  const void* B;      // [N, K]
  const void* R_eff;  // [(N/gs)*E, K]
  void* dA;           // [M, K]
  void* dR;           // [(N/gs)*rs, K], 16-bit like the inputs or fp32 (dr_f32)
  const void* ib;     // internal bias [N/gs, K] (gated modes) or null
  const long long* drop_seeds;  // [N/gs] per-group dropout seeds, or null
  float drop_p;
  void* d_ib;         // its gradient [N/gs, K] (same dtype as the inputs), when ib is given
  float* partial_ib;  // fp32 column sums of dS per main CTA: [2*runs][N/gs][K]
  float* partial_ib_x;  // ... and per slab of the extra pairs' CTAs: [2*n_extra][slots][N/gs][128]
  int M, N, K, gs, rs, E;
  int dtype, gate;
  int dr_f32;         // 1: dR is written as fp32
  float scale;
  long long lddc, lda, ldb, ldr, ldda, lddr;
  DadrGrid grid;      // CTA pairs and their tiles
  float* partial;     // [2*runs][(N/gs)*E][K] fp32: dR buffers of the main pairs' CTAs
  float* partial_x;   // [2*n_extra][slots][(N/gs)*E][128] fp32: dR slabs of the extra pairs' CTAs
  int num_sms;
  int* err;
  cudaStream_t stream;
};
int launch_bwd_dadr(const DadrArgs& a);
void dadr_plan_grid(int M, int K, int num_sms, const int* cfg, DadrGrid* grid);

}  // namespace prism
