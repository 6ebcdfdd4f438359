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

// dbias[n] = sum over token rows of dC[m, n], in a fixed order: a block owns 256 columns and a
// contiguous range of rows; its 8 warps take rows w, w + 8, ... (16-byte loads, 8 columns per lane)
// and are added in warp order, then the row ranges are added in range order by the second kernel.
template <int DT>
__global__ void dbias_partial_kernel(const uint16_t* __restrict__ dC, float* __restrict__ partial, int M, int N,
                                     long long lddc, int rows_per_split) {
  __shared__ float red[8][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col0 = blockIdx.x * 256 + lane * 8;
  const int r_lo = blockIdx.y * rows_per_split;
  const int r_hi = min(M, r_lo + rows_per_split);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col0 < N) {
    for (int r = r_lo + warp; r < r_hi; r += 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(dC + (long long)r * lddc + col0);
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = Elem<DT>::unpack(w4[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[warp][lane * 8 + e] = acc[e];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < N) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][threadIdx.x];
    partial[(long long)blockIdx.y * N + c] = t;
  }
}

template <int DT, bool F32OUT>
__global__ void dbias_final_kernel(const float* __restrict__ partial, void* __restrict__ out, int N, int splits) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float t = 0.f;
  for (int s = 0; s < splits; ++s) t += partial[(long long)s * N + c];
  if (F32OUT) reinterpret_cast<float*>(out)[c] = t;
  else reinterpret_cast<uint16_t*>(out)[c] = (uint16_t)(Elem<DT>::pack(t, 0.f) & 0xffffu);
}

// Weight folding of the "rw" mode: Bp[n, b*rs + j] = sum_i B[n, b*rs + i] * R[g*rs + i, b*rs + j] with
// g = n / gs, so that C = A . Bp^T equals the plain-mode layer (A . blockdiag(R_g)^T) . B_g^T.  One thread
// per (row n, rotation block b): rs contiguous inputs, rs contiguous outputs, fp32 accumulation.
template <int DT, int RS>
__global__ void fold_weight_kernel(const uint16_t* __restrict__ B, const uint16_t* __restrict__ R, uint16_t* __restrict__ Bp,
                                   int N, int K, int gs, long long ldb, long long ldr, long long ldbp) {
  const int nb = K / RS;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)N * nb) return;
  const int n = (int)(idx / nb), b = (int)(idx - (long long)n * nb);
  const int g = n / gs;
  float x[RS], acc[RS];
  const uint32_t* bp = reinterpret_cast<const uint32_t*>(B + (long long)n * ldb + b * RS);
#pragma unroll
  for (int i = 0; i < RS / 2; ++i) {
    const float2 v = Elem<DT>::unpack(bp[i]);
    x[2 * i] = v.x;
    x[2 * i + 1] = v.y;
  }
#pragma unroll
  for (int j = 0; j < RS; ++j) acc[j] = 0.f;
  for (int i = 0; i < RS; ++i) {
    const uint32_t* rp = reinterpret_cast<const uint32_t*>(R + (long long)(g * RS + i) * ldr + b * RS);
    float xi = x[0];
#pragma unroll
    for (int t = 1; t < RS; ++t) xi = (t == i) ? x[t] : xi;
#pragma unroll
    for (int j = 0; j < RS / 2; ++j) {
      const float2 r2 = Elem<DT>::unpack(rp[j]);
      acc[2 * j] = fmaf(xi, r2.x, acc[2 * j]);
      acc[2 * j + 1] = fmaf(xi, r2.y, acc[2 * j + 1]);
    }
  }
  uint32_t* op = reinterpret_cast<uint32_t*>(Bp + (long long)n * ldbp + b * RS);
#pragma unroll
  for (int j = 0; j < RS / 2; ++j) op[j] = Elem<DT>::pack(acc[2 * j], acc[2 * j + 1]);
}

static int num_sms();
static int dbias_splits(int M, int N, int sms) {
  const int strips = (N + 255) / 256;
  int s = (4 * sms + strips - 1) / strips;
  if (s > 64) s = 64;
  if (s > (M + 63) / 64) s = (M + 63) / 64;   // at least 64 rows per block
  return s < 1 ? 1 : s;
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
  if (gate != GATE_NONE && gate != GATE_SILU && gate != GATE_SIGMOID)
    return fail(PRISM_ERR_BAD_ARG, "%s: gate must be 0 (none), 1 (silu) or 2 (sigmoid)", fn);
  if (effective_block(rs) == 0)
    return fail(PRISM_ERR_UNSUPPORTED, "%s: reconn_sz %d is not supported (supported: 8, 16, 32, 64)", fn, rs);
  if (default_bn(gs) == 0)
    return fail(PRISM_ERR_UNSUPPORTED, "%s: group_size %d is not supported (must be a multiple of 16)", fn, gs);
  return PRISM_OK;
}

// dtype of a gradient output: the inputs' 16-bit type or fp32; returns 1 for fp32, 0 for 16 bit, -1 if invalid
static int grad_is_f32(int grad_dtype, int dtype) {
  if (grad_dtype == PRISM_DTYPE_F32) return 1;
  if (grad_dtype == PRISM_DTYPE_SAME || grad_dtype == dtype) return 0;
  return -1;
}

// internal bias [N/gs, K], 16-bit, contiguous rows of K: gated modes only
static int check_ib(const char* fn, const void* ib, int gate) {
  if (ib == nullptr) return PRISM_OK;
  if (gate == GATE_NONE) return fail(PRISM_ERR_BAD_ARG, "%s: internal_bias requires a gated mode", fn);
  if (reinterpret_cast<uintptr_t>(ib) % 4 != 0) return fail(PRISM_ERR_BAD_ARG, "%s: internal_bias must be 4-byte aligned", fn);
  return PRISM_OK;
}

// dropout: per-group seeds [N/gs] (int64) with a probability in (0, 1), gated modes only; null seeds = none
static int check_dropout(const char* fn, const void* seeds, float p, int gate) {
  if (seeds == nullptr) return PRISM_OK;
  if (gate == GATE_NONE) return fail(PRISM_ERR_BAD_ARG, "%s: dropout requires a gated mode", fn);
  if (!(p >= 0.f && p < 1.f)) return fail(PRISM_ERR_BAD_ARG, "%s: dropout_p must be in [0, 1), got %g", fn, (double)p);
  if (reinterpret_cast<uintptr_t>(seeds) % 8 != 0) return fail(PRISM_ERR_BAD_ARG, "%s: dropout_seeds must be 8-byte aligned", fn);
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

extern "C" int prism_abi_version(void) { return 4; }

extern "C" long long prism_launch_count(void) { return launch_counter().load(std::memory_order_relaxed); }

extern "C" const char* prism_last_error_string(void) { return last_error_buf(); }

extern "C" size_t prism_workspace_bytes(int kind, int M, int N, int K, int gs, int rs, int dtype,
                                        const int* cfg) {
  (void)dtype; (void)cfg; (void)M;
  size_t bytes = PRISM_WORKSPACE_HEADER_BYTES;
  if (kind == PRISM_KIND_DBIAS) {
    if (N <= 0 || M <= 0) return bytes;
    return bytes + align256((size_t)dbias_splits(M, N, num_sms()) * N * 4);
  }
  if (gs <= 0 || rs <= 0 || N <= 0 || K <= 0) return bytes;
  const size_t G = (size_t)(N / gs);
  // copy of R the kernels read: widened for rs = 8 (all kinds), halved for the gated dA+dR kernel
  if (rs == 8) bytes += align256(G * 16 * (size_t)K * 2);
  else if (kind == PRISM_KIND_BWD_DADR || kind == PRISM_KIND_BWD_DADR_IB) bytes += align256(G * (size_t)effective_block(rs) * K * 2);
  if (kind == PRISM_KIND_FWD) {
    // few tokens: the streaming forward keeps its arrival counters and fp32 partial sums here
    // (cfg[3] = 1 asks for the general kernel, which needs none)
    const int path = cfg ? cfg[3] : 0;
    if (path != 1 && fwd_small_supported(M, N, K, gs, effective_block(rs)) && (path == 2 || fwd_small_preferred(M)))
      bytes += fwd_small_scratch_bytes(M, N, K, gs, num_sms());
    return bytes;
  }
  if (kind == PRISM_KIND_BWD_DB) {
    const int bn = (cfg && cfg[0] > 0) ? cfg[0] : default_bn(gs);
    if (bn <= 0) return bytes;
    DbPlan pl;
    db_plan(M, N, K, bn, num_sms(), cfg, &pl);
    if (pl.splits > 1) bytes += align256((size_t)pl.splits * N * K * 4);
    else if (pl.tail_rows > 0) bytes += align256((size_t)pl.tail_splits * pl.tail_rows * bn * K * 4);
    return bytes;
  }
  if (kind == PRISM_KIND_BWD_DADR || kind == PRISM_KIND_BWD_DADR_IB) {
    const int E = effective_block(rs);
    if (E == 0) return bytes;
    DadrGrid gr;
    dadr_plan_grid(M, K, num_sms(), cfg, &gr);
    bytes += align256((size_t)2 * gr.runs * G * E * (size_t)K * 4);                 // one buffer per CTA of every main pair
    bytes += align256((size_t)2 * gr.n_extra * gr.slots * G * E * (size_t)128 * 4); // slabs of the extra pairs' CTAs
    if (kind == PRISM_KIND_BWD_DADR_IB) {   // the same for the column sums of dS (gradient of the internal bias)
      bytes += align256((size_t)2 * gr.runs * G * (size_t)K * 4);
      bytes += align256((size_t)2 * gr.n_extra * gr.slots * G * (size_t)128 * 4);
    }
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

extern "C" int prism_fwd_dropout(const void* A, const void* B, const void* R, const void* bias, const void* internal_bias,
                                 void* C, int M, int N, int K, int gs, int rs, int dtype, int gate,
                                 long long lda, long long ldb, long long ldr, long long ldc,
                                 const long long* dropout_seeds, float dropout_p,
                                 const int* cfg, void* workspace, size_t workspace_bytes, void* stream);

extern "C" int prism_fwd(const void* A, const void* B, const void* R, const void* bias, const void* internal_bias, void* C,
                         int M, int N, int K, int gs, int rs, int dtype, int gate,
                         long long lda, long long ldb, long long ldr, long long ldc,
                         const int* cfg, void* workspace, size_t workspace_bytes, void* stream) {
  return prism_fwd_dropout(A, B, R, bias, internal_bias, C, M, N, K, gs, rs, dtype, gate, lda, ldb, ldr, ldc, nullptr, 0.f, cfg,
                           workspace, workspace_bytes, stream);
}

extern "C" int prism_fwd_dropout(const void* A, const void* B, const void* R, const void* bias, const void* internal_bias,
                                 void* C, int M, int N, int K, int gs, int rs, int dtype, int gate,
                                 long long lda, long long ldb, long long ldr, long long ldc,
                                 const long long* dropout_seeds, float dropout_p,
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
  if ((rc = check_ib(fn, internal_bias, gate))) return rc;
  if ((rc = check_dropout(fn, dropout_seeds, dropout_p, gate))) return rc;
  const size_t need = prism_workspace_bytes(PRISM_KIND_FWD, M, N, K, gs, rs, dtype, cfg);
  if (workspace == nullptr || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return fail(PRISM_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned and >= %zu bytes (got %zu)", fn, need, workspace_bytes);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);

  FwdArgs a;
  a.A = A; a.B = B; a.bias = bias; a.ib = internal_bias; a.C = C;
  a.drop_seeds = dropout_seeds; a.drop_p = dropout_p;
  a.M = M; a.N = N; a.K = K; a.gs = gs; a.E = effective_block(rs);
  a.dtype = dtype; a.gate = gate;
  a.lda = lda; a.ldb = ldb; a.ldc = ldc;
  a.R_eff = R; a.ldr = ldr;
  uint8_t* wp = reinterpret_cast<uint8_t*>(workspace) + PRISM_WORKSPACE_HEADER_BYTES;
  if (rs == 8) {
    if ((rc = launch_expand_r8(R, wp, N / gs, K, ldr, dtype, s))) return rc;
    a.R_eff = wp; a.ldr = K;
    wp += align256((size_t)(N / gs) * 16 * K * 2);
  }
  a.num_sms = num_sms();
  a.err = reinterpret_cast<int*>(workspace);
  a.stream = s;
  // few tokens (M <= 128): the streaming kernel, unless cfg[3] = 1 asks for the general one
  const int path = cfg ? cfg[3] : 0;
  if (path == 2 && !fwd_small_supported(M, N, K, gs, a.E))
    return fail(PRISM_ERR_UNSUPPORTED, "%s: the few-token kernel needs M <= 128 and group_size a multiple of 128 (M=%d, group_size=%d)", fn, M, gs);
  if (path != 1 && fwd_small_supported(M, N, K, gs, a.E) && (path == 2 || fwd_small_preferred(M)))
    return launch_fwd_small(a, wp);
  a.BN = (cfg && cfg[0] > 0) ? cfg[0] : default_bn(gs);
  a.PM = (cfg && cfg[1] > 0) ? cfg[1] : 16;
  a.sa = (cfg && cfg[2] > 0) ? cfg[2] : 0;
  a.sb = 0;
  if (a.BN % 16 != 0 || a.BN > 256 || gs % a.BN != 0)
    return fail(PRISM_ERR_BAD_ARG, "%s: tile BN=%d must be a multiple of 16, <= 256 and divide group_size=%d", fn, a.BN, gs);
  return launch_fwd(a);
}

extern "C" int prism_bwd_db(const void* dC, const void* A, const void* R, const void* internal_bias, void* dB,
                            int M, int N, int K, int gs, int rs, int dtype, int gate, int db_dtype, float dc_scale,
                            long long lddc, long long lda, long long ldr, long long lddb,
                            const long long* dropout_seeds, float dropout_p,
                            const int* cfg, void* workspace, size_t workspace_bytes, void* stream) {
  const char* fn = "prism_bwd_db";
  int rc;
  if ((rc = check_common(fn, M, N, K, gs, rs, dtype, gate))) return rc;
  const int db_f32 = grad_is_f32(db_dtype, dtype);
  if (db_f32 < 0) return fail(PRISM_ERR_BAD_ARG, "%s: db_dtype must be the input dtype, PRISM_DTYPE_SAME or PRISM_DTYPE_F32", fn);
  if (K % 8 != 0) return fail(PRISM_ERR_BAD_ARG, "%s: K must be a multiple of 8", fn);
  if ((rc = check_ptr(fn, "dB", dB, lddb, K))) return rc;
  if ((rc = check_ib(fn, internal_bias, gate))) return rc;
  if ((rc = check_dropout(fn, dropout_seeds, dropout_p, gate))) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (M == 0) {  // no tokens: the gradient is zero
    const size_t es = db_f32 ? 4 : 2;
    cudaError_t e = cudaMemset2DAsync(dB, lddb * es, 0, (size_t)K * es, N, s);
    return e == cudaSuccess ? PRISM_OK : fail(PRISM_ERR_CUDA, "%s: %s", fn, cudaGetErrorString(e));
  }
  if ((rc = check_ptr(fn, "dC", dC, lddc, N))) return rc;
  if ((rc = check_ptr(fn, "A", A, lda, K))) return rc;
  if ((rc = check_ptr(fn, "R", R, ldr, K))) return rc;
  const size_t need = prism_workspace_bytes(PRISM_KIND_BWD_DB, M, N, K, gs, rs, dtype, cfg);
  if (workspace == nullptr || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return fail(PRISM_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned and >= %zu bytes (got %zu)", fn, need, workspace_bytes);

  DbArgs a;
  a.dC = dC; a.A = A; a.dB = dB; a.ib = internal_bias; a.drop_seeds = dropout_seeds; a.drop_p = dropout_p;
  a.M = M; a.N = N; a.K = K; a.gs = gs; a.E = effective_block(rs);
  a.dtype = dtype; a.gate = gate; a.scale = dc_scale; a.out_f32 = db_f32;
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

extern "C" int prism_bwd_dadr(const void* dC, const void* A, const void* B, const void* R, const void* internal_bias,
                              void* dA, void* dR, void* d_internal_bias, int M, int N, int K, int gs, int rs, int dtype, int gate,
                              int dr_dtype, float dc_scale, long long lddc, long long lda, long long ldb,
                              long long ldr, long long ldda, long long lddr,
                              const long long* dropout_seeds, float dropout_p, const int* cfg,
                              void* workspace, size_t workspace_bytes, void* stream) {
  const char* fn = "prism_bwd_dadr";
  int rc;
  if ((rc = check_common(fn, M, N, K, gs, rs, dtype, gate))) return rc;
  const int dr_f32 = grad_is_f32(dr_dtype, dtype);
  if (dr_f32 < 0) return fail(PRISM_ERR_BAD_ARG, "%s: dr_dtype must be the input dtype, PRISM_DTYPE_SAME or PRISM_DTYPE_F32", fn);
  if (K % 8 != 0) return fail(PRISM_ERR_BAD_ARG, "%s: K must be a multiple of 8", fn);
  if ((rc = check_ptr(fn, "dR", dR, lddr, K))) return rc;
  if ((rc = check_ib(fn, internal_bias, gate))) return rc;
  if ((rc = check_dropout(fn, dropout_seeds, dropout_p, gate))) return rc;
  const bool with_ib = internal_bias != nullptr;
  if (with_ib && d_internal_bias == nullptr) return fail(PRISM_ERR_BAD_ARG, "%s: d_internal_bias is null", fn);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (M == 0) {  // no tokens: dA is empty and dR is zero
    const size_t es = dr_f32 ? 4 : 2;
    if (with_ib) (void)cudaMemsetAsync(d_internal_bias, 0, (size_t)(N / gs) * K * 2, s);
    cudaError_t e = cudaMemset2DAsync(dR, lddr * es, 0, (size_t)K * es, (size_t)(N / gs) * rs, s);
    return e == cudaSuccess ? PRISM_OK : fail(PRISM_ERR_CUDA, "%s: %s", fn, cudaGetErrorString(e));
  }
  if ((rc = check_ptr(fn, "dC", dC, lddc, N))) return rc;
  if ((rc = check_ptr(fn, "A", A, lda, K))) return rc;
  if ((rc = check_ptr(fn, "B", B, ldb, K))) return rc;
  if ((rc = check_ptr(fn, "R", R, ldr, K))) return rc;
  if ((rc = check_ptr(fn, "dA", dA, ldda, K))) return rc;
  const size_t need = prism_workspace_bytes(with_ib ? PRISM_KIND_BWD_DADR_IB : PRISM_KIND_BWD_DADR, M, N, K, gs, rs, dtype, cfg);
  if (workspace == nullptr || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return fail(PRISM_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned and >= %zu bytes (got %zu)", fn, need, workspace_bytes);

  DadrArgs a;
  a.dC = dC; a.A = A; a.B = B; a.dA = dA; a.dR = dR; a.ib = internal_bias; a.d_ib = d_internal_bias;
  a.drop_seeds = dropout_seeds; a.drop_p = dropout_p;
  a.M = M; a.N = N; a.K = K; a.gs = gs; a.rs = rs; a.E = effective_block(rs);
  a.dtype = dtype; a.gate = gate; a.scale = dc_scale; a.dr_f32 = dr_f32;
  a.lddc = lddc; a.lda = lda; a.ldb = ldb; a.ldda = ldda; a.lddr = lddr;
  a.R_eff = R; a.ldr = ldr;
  uint8_t* wp = reinterpret_cast<uint8_t*>(workspace) + PRISM_WORKSPACE_HEADER_BYTES;
  // The kernel reads a copy of R: widened to 16x16 blocks for rs = 8, and halved in the gated mode
  // (its gate math works on S/2, see gate_bwd_pair).  The plain mode with rs >= 16 reads R itself.
  if (rs == 8 || gate != GATE_NONE) {
    if ((rc = launch_prep_r(R, wp, N / gs, rs, a.E, K, ldr, gate != GATE_NONE ? 0.5f : 1.0f, dtype, s))) return rc;
    a.R_eff = wp; a.ldr = K;
  }
  wp += align256((size_t)(N / gs) * a.E * K * 2);
  a.num_sms = num_sms();
  dadr_plan_grid(M, K, a.num_sms, cfg, &a.grid);
  a.partial = reinterpret_cast<float*>(wp);
  wp += align256((size_t)2 * a.grid.runs * (N / gs) * a.E * (size_t)K * 4);
  a.partial_x = reinterpret_cast<float*>(wp);
  wp += align256((size_t)2 * a.grid.n_extra * a.grid.slots * (N / gs) * a.E * (size_t)128 * 4);
  a.partial_ib = reinterpret_cast<float*>(wp);
  wp += align256((size_t)2 * a.grid.runs * (N / gs) * (size_t)K * 4);
  a.partial_ib_x = reinterpret_cast<float*>(wp);
  a.err = reinterpret_cast<int*>(workspace);
  a.stream = s;
  return launch_bwd_dadr(a);
}

extern "C" int prism_dbias(const void* dC, void* dbias, int M, int N, int dtype, int dbias_dtype, long long lddc,
                           void* workspace, size_t workspace_bytes, void* stream) {
  const char* fn = "prism_dbias";
  int rc;
  if (M < 0 || N <= 0) return fail(PRISM_ERR_BAD_ARG, "%s: bad shape M=%d N=%d", fn, M, N);
  if (N % 8 != 0) return fail(PRISM_ERR_BAD_ARG, "%s: N must be a multiple of 8", fn);
  if (dtype != DT_F16 && dtype != DT_BF16) return fail(PRISM_ERR_BAD_ARG, "%s: dtype must be 0 (fp16) or 1 (bf16)", fn);
  const int out_f32 = grad_is_f32(dbias_dtype, dtype);
  if (out_f32 < 0) return fail(PRISM_ERR_BAD_ARG, "%s: dbias_dtype must be the input dtype, PRISM_DTYPE_SAME or PRISM_DTYPE_F32", fn);
  if (dbias == nullptr) return fail(PRISM_ERR_BAD_ARG, "%s: dbias is null", fn);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (M == 0) {
    cudaError_t e = cudaMemsetAsync(dbias, 0, (size_t)N * (out_f32 ? 4 : 2), s);
    return e == cudaSuccess ? PRISM_OK : fail(PRISM_ERR_CUDA, "%s: %s", fn, cudaGetErrorString(e));
  }
  if ((rc = check_ptr(fn, "dC", dC, lddc, N))) return rc;
  const size_t need = prism_workspace_bytes(PRISM_KIND_DBIAS, M, N, 0, 0, 0, dtype, nullptr);
  if (workspace == nullptr || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return fail(PRISM_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned and >= %zu bytes (got %zu)", fn, need, workspace_bytes);
  float* partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + PRISM_WORKSPACE_HEADER_BYTES);
  const int splits = dbias_splits(M, N, num_sms());
  const int rows_per_split = (M + splits - 1) / splits;
  const int used = (M + rows_per_split - 1) / rows_per_split;
  dim3 grid((N + 255) / 256, used);
  const uint16_t* src = reinterpret_cast<const uint16_t*>(dC);
  if (dtype == DT_BF16) dbias_partial_kernel<DT_BF16><<<grid, 256, 0, s>>>(src, partial, M, N, lddc, rows_per_split);
  else dbias_partial_kernel<DT_F16><<<grid, 256, 0, s>>>(src, partial, M, N, lddc, rows_per_split);
  if ((rc = check_launch("prism_dbias"))) return rc;
  const int blocks = (N + 255) / 256;
  if (dtype == DT_BF16) {
    if (out_f32) dbias_final_kernel<DT_BF16, true><<<blocks, 256, 0, s>>>(partial, dbias, N, used);
    else dbias_final_kernel<DT_BF16, false><<<blocks, 256, 0, s>>>(partial, dbias, N, used);
  } else {
    if (out_f32) dbias_final_kernel<DT_F16, true><<<blocks, 256, 0, s>>>(partial, dbias, N, used);
    else dbias_final_kernel<DT_F16, false><<<blocks, 256, 0, s>>>(partial, dbias, N, used);
  }
  return check_launch("prism_dbias reduce");
}

extern "C" int prism_fold_weight(const void* B, const void* R, void* Bp, int N, int K, int gs, int rs, int dtype,
                                 long long ldb, long long ldr, long long ldbp, void* stream) {
  const char* fn = "prism_fold_weight";
  int rc;
  if ((rc = check_common(fn, 0, N, K, gs, rs, dtype, GATE_NONE))) return rc;
  if ((rc = check_ptr(fn, "B", B, ldb, K))) return rc;
  if ((rc = check_ptr(fn, "R", R, ldr, K))) return rc;
  if ((rc = check_ptr(fn, "Bp", Bp, ldbp, K))) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long total = (long long)N * (K / rs);
  const int threads = 128;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  const uint16_t* b = reinterpret_cast<const uint16_t*>(B);
  const uint16_t* r = reinterpret_cast<const uint16_t*>(R);
  uint16_t* o = reinterpret_cast<uint16_t*>(Bp);
#define PRISM_FOLD(DT_, RS_) fold_weight_kernel<DT_, RS_><<<blocks, threads, 0, s>>>(b, r, o, N, K, gs, ldb, ldr, ldbp)
#define PRISM_FOLD_DT(RS_) do { if (dtype == DT_BF16) PRISM_FOLD(DT_BF16, RS_); else PRISM_FOLD(DT_F16, RS_); } while (0)
  if (rs == 8) PRISM_FOLD_DT(8); else if (rs == 16) PRISM_FOLD_DT(16); else if (rs == 32) PRISM_FOLD_DT(32); else PRISM_FOLD_DT(64);
#undef PRISM_FOLD_DT
#undef PRISM_FOLD
  return check_launch("prism_fold_weight");
}
