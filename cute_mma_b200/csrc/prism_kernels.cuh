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

// R [(G*8), K] -> R_eff [(G*16), K]: two neighbouring 8x8 blocks become one 16x16
// block-diagonal block, so that every rotation is a 16-wide tensor-core product.
int launch_expand_r8(const void* R, void* R_eff, int G, int K, long long ldr, int dtype, cudaStream_t stream);
// R_eff [(G*E), K] = factor * R (widened as above when rs = 8)
int launch_prep_r(const void* R, void* R_eff, int G, int rs, int E, int K, long long ldr, float factor, int dtype,
                  cudaStream_t stream);

struct DbArgs {
  const void* dC;     // [M, N]
  const void* A;      // [M, K]
  const void* R_eff;  // [(N/gs)*E, K]
  void* dB;           // [N, K]
  int M, N, K, gs, E;
  int dtype, gate;
  float scale;        // dB = scale * dC^T H
  long long lddc, lda, ldr, lddb;
  int BN, splits;
  float* partial;     // [splits][N][K] fp32 scratch when splits > 1
  int num_sms;
  int* err;
  cudaStream_t stream;
};
int launch_bwd_db(const DbArgs& a);
int db_default_splits(int M, int N, int K, int BN, int num_sms);

struct DadrArgs {
  const void* dC;     // [M, N]
  const void* A;      // [M, K]
  const void* B;      // [N, K]
  const void* R_eff;  // [(N/gs)*E, K]
  void* dA;           // [M, K]
  void* dR;           // [(N/gs)*rs, K]
  int M, N, K, gs, rs, E;
  int dtype, gate;
  float scale;
  long long lddc, lda, ldb, ldr, ldda, lddr;
  int runs;           // CTA pairs per 128-feature column; each CTA owns one fp32 partial dR buffer
  int fpass;          // feature passes (see dadr_plan_grid)
  float* partial;     // [runs][(N/gs)*E][K]
  int num_sms;
  int* err;
  cudaStream_t stream;
};
int launch_bwd_dadr(const DadrArgs& a);
// grid of the dA+dR kernel: CTA pairs per feature column and feature passes; cfg = {runs, fpass} or null
void dadr_plan_grid(int M, int N, int K, int num_sms, const int* cfg, int* runs_out, int* fpass_out);

}  // namespace prism
