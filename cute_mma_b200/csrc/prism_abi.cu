// extern "C" entry points of libprism_b200.so: argument checks, workspace carving,
// small helper kernels, dispatch to the kernel launchers.
#include "../../include/prism_b200.h"
#include "prism_host.cuh"
#include "prism_kernels.cuh"

namespace prism {

// R_eff[(G*E), K] = factor * R with, for reconn_sz = 8 (E = 16), two neighbouring 8x8 blocks widened
// to one block-diagonal 16x16 block.  One thread per output element.
template <int DT>
__global__ void prep_r_kernel(const uint16_t* __restrict__ R, uint16_t* __restrict__ Re, int G, int rs, int E,
                              int K, long long ldr, float factor) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)G * E * K;
  if (idx >= total) return;
  const int k = (int)(idx % K);
  const int row = (int)(idx / K);
  const int g = row / E, i = row - g * E;
  uint16_t v = 0;
  if (rs == 8) {
    const bool upper_cols = (k & 15) >= 8;
    if (i < 8 && !upper_cols) v = R[(long long)(g * 8 + i) * ldr + k];
    if (i >= 8 && upper_cols) v = R[(long long)(g * 8 + i - 8) * ldr + k];
  } else {
    v = R[(long long)(g * rs + i) * ldr + k];
  }
  if (factor != 1.0f) v = (uint16_t)(Elem<DT>::pack(Elem<DT>::unpack((uint32_t)v).x * factor, 0.f) & 0xffffu);
  Re[idx] = v;
}

int launch_prep_r(const void* R, void* R_eff, int G, int rs, int E, int K, long long ldr, float factor, int dtype,
                  cudaStream_t stream) {
  const long long total = (long long)G * E * K;
  const int threads = 256;
  const long long blocks = (total + threads - 1) / threads;
  if (dtype == DT_BF16)
    prep_r_kernel<DT_BF16><<<(unsigned)blocks, threads, 0, stream>>>(
        reinterpret_cast<const uint16_t*>(R), reinterpret_cast<uint16_t*>(R_eff), G, rs, E, K, ldr, factor);
  else
    prep_r_kernel<DT_F16><<<(unsigned)blocks, threads, 0, stream>>>(
        reinterpret_cast<const uint16_t*>(R), reinterpret_cast<uint16_t*>(R_eff), G, rs, E, K, ldr, factor);
  return check_launch("prep_r");
}

int launch_expand_r8(const void* R, void* R_eff, int G, int K, long long ldr, int dtype, cudaStream_t stream) {
  return launch_prep_r(R, R_eff, G, 8, 16, K, ldr, 1.0f, dtype, stream);
}

static int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

// effective rotation block: 8 -> 16 (two blocks fused), 16/32/64 native
static int effective_block(int rs) {
  if (rs == 8) return 16;
  if (rs == 16 || rs == 32 || rs == 64) return rs;
  return 0;
}

static int default_bn(int gs) {
  const int cands[] = {256, 128, 64, 32, 16};
  for (int c : cands)
    if (gs % c == 0) return c;
  if (gs <= 256 && gs % 16 == 0) return gs;
  return 0;
}

static int check_common(const char* fn, int M, int N, int K, int gs, int rs, int dtype, int gate) {
  if (M < 0 || N <= 0 || K <= 0) return fail(PRISM_ERR_BAD_ARG, "%s: bad shape M=%d N=%d K=%d", fn, M, N, K);
  if (gs <= 0 || rs <= 0) return fail(PRISM_ERR_BAD_ARG, "%s: group_size and reconn_sz must be positive", fn);
  if (rs % 8 != 0) return fail(PRISM_ERR_BAD_ARG, "%s: reconn_sz must be a multiple of 8, got %d", fn, rs);
  if (gs % 8 != 0) return fail(PRISM_ERR_BAD_ARG, "%s: group_size must be a multiple of 8, got %d", fn, gs);
  if (N % gs != 0) return fail(PRISM_ERR_BAD_ARG, "%s: N (%d) must be divisible by group_size (%d)", fn, N, gs);
  if (K % rs != 0) return fail(PRISM_ERR_BAD_ARG, "%s: K (%d) must be divisible by reconn_sz (%d)", fn, K, rs);
  if (dtype != DT_F16 && dtype != DT_BF16) return fail(PRISM_ERR_BAD_ARG, "%s: dtype must be 0 (fp16) or 1 (bf16)", fn);
  if (gate != GATE_NONE && gate != GATE_SILU) return fail(PRISM_ERR_BAD_ARG, "%s: gate must be 0 (none) or 1 (silu)", fn);
  if (effective_block(rs) == 0)
    return fail(PRISM_ERR_UNSUPPORTED, "%s: reconn_sz %d is not supported (supported: 8, 16, 32, 64)", fn, rs);
  if (default_bn(gs) == 0)
    return fail(PRISM_ERR_UNSUPPORTED, "%s: group_size %d is not supported (must be a multiple of 16)", fn, gs);
  return PRISM_OK;
}

static int check_ptr(const char* fn, const char* name, const void* p, long long ld, int min_ld) {
  if (p == nullptr) return fail(PRISM_ERR_BAD_ARG, "%s: %s is null", fn, name);
  if (reinterpret_cast<uintptr_t>(p) % 16 != 0) return fail(PRISM_ERR_BAD_ARG, "%s: %s must be 16-byte aligned", fn, name);
  if (ld < min_ld || ld % 8 != 0)
    return fail(PRISM_ERR_BAD_ARG, "%s: leading dimension of %s (%lld) must be >= %d and a multiple of 8", fn, name, ld, min_ld);
  return PRISM_OK;
}

}  // namespace prism

using namespace prism;

extern "C" int prism_abi_version(void) { return 1; }

extern "C" long long prism_launch_count(void) { return launch_counter(); }

extern "C" const char* prism_last_error_string(void) { return last_error_buf(); }

extern "C" size_t prism_workspace_bytes(int kind, int M, int N, int K, int gs, int rs, int dtype,
                                        const int* cfg) {
  (void)dtype; (void)cfg; (void)M;
  size_t bytes = PRISM_WORKSPACE_HEADER_BYTES;
  if (gs <= 0 || rs <= 0 || N <= 0 || K <= 0) return bytes;
  const size_t G = (size_t)(N / gs);
  // copy of R the kernels read: widened for rs = 8 (all kinds), halved for the gated dA+dR kernel
  if (rs == 8) bytes += align256(G * 16 * (size_t)K * 2);
  else if (kind == PRISM_KIND_BWD_DADR) bytes += align256(G * (size_t)effective_block(rs) * K * 2);
  if (kind == PRISM_KIND_FWD) return bytes;
  if (kind == PRISM_KIND_BWD_DB) {
    const int bn = (cfg && cfg[0] > 0) ? cfg[0] : default_bn(gs);
    if (bn <= 0) return bytes;
    DbPlan pl;
    db_plan(M, N, K, bn, num_sms(), cfg, &pl);
    if (pl.splits > 1) bytes += align256((size_t)pl.splits * N * K * 4);
    else if (pl.tail_rows > 0) bytes += align256((size_t)pl.tail_splits * pl.tail_rows * bn * K * 4);
    return bytes;
  }
  if (kind == PRISM_KIND_BWD_DADR) {
    const int E = effective_block(rs);
    if (E == 0) return bytes;
    DadrGrid gr;
    dadr_plan_grid(M, K, num_sms(), cfg, &gr);
    bytes += align256((size_t)2 * gr.runs * G * E * (size_t)K * 4);                 // one buffer per CTA of every main pair
    bytes += align256((size_t)2 * gr.n_extra * gr.slots * G * E * (size_t)128 * 4); // slabs of the extra pairs' CTAs
    return bytes;
  }
  return bytes;
}

extern "C" int prism_status(void* workspace, void* stream) {
  if (workspace == nullptr) return fail(PRISM_ERR_BAD_ARG, "prism_status: workspace is null");
  int code = 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(&code, workspace, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail(PRISM_ERR_CUDA, "prism_status: %s", cudaGetErrorString(e));
  if (code != 0) {
    cudaMemsetAsync(workspace, 0, sizeof(int), s);
    return fail(code, "a device-side wait ran out in an earlier prism kernel (status %d)", code);
  }
  return PRISM_OK;
}

extern "C" int prism_fwd(const void* A, const void* B, const void* R, const void* bias, void* C,
                         int M, int N, int K, int gs, int rs, int dtype, int gate,
                         long long lda, long long ldb, long long ldr, long long ldc,
                         const int* cfg, void* workspace, size_t workspace_bytes, void* stream) {
  const char* fn = "prism_fwd";
  int rc;
  if ((rc = check_common(fn, M, N, K, gs, rs, dtype, gate))) return rc;
  if (K % 8 != 0) return fail(PRISM_ERR_BAD_ARG, "%s: K must be a multiple of 8", fn);
  if (M == 0) return PRISM_OK;
  if ((rc = check_ptr(fn, "A", A, lda, K))) return rc;
  if ((rc = check_ptr(fn, "B", B, ldb, K))) return rc;
  if ((rc = check_ptr(fn, "R", R, ldr, K))) return rc;
  if ((rc = check_ptr(fn, "C", C, ldc, N))) return rc;
  if (bias != nullptr && reinterpret_cast<uintptr_t>(bias) % 4 != 0)
    return fail(PRISM_ERR_BAD_ARG, "%s: bias must be 4-byte aligned", fn);
  const size_t need = prism_workspace_bytes(PRISM_KIND_FWD, M, N, K, gs, rs, dtype, cfg);
  if (workspace == nullptr || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return fail(PRISM_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned and >= %zu bytes (got %zu)", fn, need, workspace_bytes);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);

  FwdArgs a;
  a.A = A; a.B = B; a.bias = bias; a.C = C;
  a.M = M; a.N = N; a.K = K; a.gs = gs; a.E = effective_block(rs);
  a.dtype = dtype; a.gate = gate;
  a.lda = lda; a.ldb = ldb; a.ldc = ldc;
  a.R_eff = R; a.ldr = ldr;
  if (rs == 8) {
    void* re = reinterpret_cast<uint8_t*>(workspace) + PRISM_WORKSPACE_HEADER_BYTES;
    if ((rc = launch_expand_r8(R, re, N / gs, K, ldr, dtype, s))) return rc;
    a.R_eff = re; a.ldr = K;
  }
  a.BN = (cfg && cfg[0] > 0) ? cfg[0] : default_bn(gs);
  a.PM = (cfg && cfg[1] > 0) ? cfg[1] : 16;
  a.sa = (cfg && cfg[2] > 0) ? cfg[2] : 0;
  a.sb = (cfg && cfg[3] > 0) ? cfg[3] : 0;
  if (a.BN % 16 != 0 || a.BN > 256 || gs % a.BN != 0)
    return fail(PRISM_ERR_BAD_ARG, "%s: tile BN=%d must be a multiple of 16, <= 256 and divide group_size=%d", fn, a.BN, gs);
  a.num_sms = num_sms();
  a.err = reinterpret_cast<int*>(workspace);
  a.stream = s;
  return launch_fwd(a);
}

extern "C" int prism_bwd_db(const void* dC, const void* A, const void* R, void* dB,
                            int M, int N, int K, int gs, int rs, int dtype, int gate, float dc_scale,
                            long long lddc, long long lda, long long ldr, long long lddb,
                            const int* cfg, void* workspace, size_t workspace_bytes, void* stream) {
  const char* fn = "prism_bwd_db";
  int rc;
  if ((rc = check_common(fn, M, N, K, gs, rs, dtype, gate))) return rc;
  if (K % 8 != 0) return fail(PRISM_ERR_BAD_ARG, "%s: K must be a multiple of 8", fn);
  if ((rc = check_ptr(fn, "dB", dB, lddb, K))) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (M == 0) {  // no tokens: the gradient is zero
    cudaError_t e = cudaMemset2DAsync(dB, lddb * 2, 0, (size_t)K * 2, N, s);
    return e == cudaSuccess ? PRISM_OK : fail(PRISM_ERR_CUDA, "%s: %s", fn, cudaGetErrorString(e));
  }
  if ((rc = check_ptr(fn, "dC", dC, lddc, N))) return rc;
  if ((rc = check_ptr(fn, "A", A, lda, K))) return rc;
  if ((rc = check_ptr(fn, "R", R, ldr, K))) return rc;
  const size_t need = prism_workspace_bytes(PRISM_KIND_BWD_DB, M, N, K, gs, rs, dtype, cfg);
  if (workspace == nullptr || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return fail(PRISM_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned and >= %zu bytes (got %zu)", fn, need, workspace_bytes);

  DbArgs a;
  a.dC = dC; a.A = A; a.dB = dB;
  a.M = M; a.N = N; a.K = K; a.gs = gs; a.E = effective_block(rs);
  a.dtype = dtype; a.gate = gate; a.scale = dc_scale;
  a.lddc = lddc; a.lda = lda; a.lddb = lddb;
  a.R_eff = R; a.ldr = ldr;
  uint8_t* wp = reinterpret_cast<uint8_t*>(workspace) + PRISM_WORKSPACE_HEADER_BYTES;
  if (rs == 8) {
    if ((rc = launch_expand_r8(R, wp, N / gs, K, ldr, dtype, s))) return rc;
    a.R_eff = wp; a.ldr = K;
    wp += align256((size_t)(N / gs) * 16 * K * 2);
  }
  a.BN = (cfg && cfg[0] > 0) ? cfg[0] : default_bn(gs);
  if (a.BN % 16 != 0 || a.BN > 256 || gs % a.BN != 0)
    return fail(PRISM_ERR_BAD_ARG, "%s: tile BN=%d must be a multiple of 16, <= 256 and divide group_size=%d", fn, a.BN, gs);
  a.num_sms = num_sms();
  db_plan(M, N, K, a.BN, a.num_sms, cfg, &a.plan);
  a.partial = (a.plan.splits > 1 || a.plan.tail_rows > 0) ? reinterpret_cast<float*>(wp) : nullptr;
  a.err = reinterpret_cast<int*>(workspace);
  a.stream = s;
  return launch_bwd_db(a);
}

extern "C" int prism_bwd_dadr(const void* dC, const void* A, const void* B, const void* R, void* dA,
                              void* dR, int M, int N, int K, int gs, int rs, int dtype, int gate,
                              float dc_scale, long long lddc, long long lda, long long ldb,
                              long long ldr, long long ldda, long long lddr, const int* cfg,
                              void* workspace, size_t workspace_bytes, void* stream) {
  const char* fn = "prism_bwd_dadr";
  int rc;
  if ((rc = check_common(fn, M, N, K, gs, rs, dtype, gate))) return rc;
  if (K % 8 != 0) return fail(PRISM_ERR_BAD_ARG, "%s: K must be a multiple of 8", fn);
  if ((rc = check_ptr(fn, "dR", dR, lddr, K))) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (M == 0) {  // no tokens: dA is empty and dR is zero
    cudaError_t e = cudaMemset2DAsync(dR, lddr * 2, 0, (size_t)K * 2, (size_t)(N / gs) * rs, s);
    return e == cudaSuccess ? PRISM_OK : fail(PRISM_ERR_CUDA, "%s: %s", fn, cudaGetErrorString(e));
  }
  if ((rc = check_ptr(fn, "dC", dC, lddc, N))) return rc;
  if ((rc = check_ptr(fn, "A", A, lda, K))) return rc;
  if ((rc = check_ptr(fn, "B", B, ldb, K))) return rc;
  if ((rc = check_ptr(fn, "R", R, ldr, K))) return rc;
  if ((rc = check_ptr(fn, "dA", dA, ldda, K))) return rc;
  const size_t need = prism_workspace_bytes(PRISM_KIND_BWD_DADR, M, N, K, gs, rs, dtype, cfg);
  if (workspace == nullptr || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return fail(PRISM_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned and >= %zu bytes (got %zu)", fn, need, workspace_bytes);

  DadrArgs a;
  a.dC = dC; a.A = A; a.B = B; a.dA = dA; a.dR = dR;
  a.M = M; a.N = N; a.K = K; a.gs = gs; a.rs = rs; a.E = effective_block(rs);
  a.dtype = dtype; a.gate = gate; a.scale = dc_scale;
  a.lddc = lddc; a.lda = lda; a.ldb = ldb; a.ldda = ldda; a.lddr = lddr;
  a.R_eff = R; a.ldr = ldr;
  uint8_t* wp = reinterpret_cast<uint8_t*>(workspace) + PRISM_WORKSPACE_HEADER_BYTES;
  // The kernel reads a copy of R: widened to 16x16 blocks for rs = 8, and halved in the gated mode
  // (its gate math works on S/2, see gate_bwd_pair).  The plain mode with rs >= 16 reads R itself.
  if (rs == 8 || gate == GATE_SILU) {
    if ((rc = launch_prep_r(R, wp, N / gs, rs, a.E, K, ldr, gate == GATE_SILU ? 0.5f : 1.0f, dtype, s))) return rc;
    a.R_eff = wp; a.ldr = K;
  }
  wp += align256((size_t)(N / gs) * a.E * K * 2);
  a.num_sms = num_sms();
  dadr_plan_grid(M, K, a.num_sms, cfg, &a.grid);
  a.partial = reinterpret_cast<float*>(wp);
  wp += align256((size_t)2 * a.grid.runs * (N / gs) * a.E * (size_t)K * 4);
  a.partial_x = reinterpret_cast<float*>(wp);
  a.err = reinterpret_cast<int*>(workspace);
  a.stream = s;
  return launch_bwd_dadr(a);
}
