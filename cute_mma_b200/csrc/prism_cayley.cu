// Batched Cayley transform of the rotation blocks, for sm_100a (any CUDA GPU would do: plain fp32 code).
//
// Plain-mode PrismLinear stores a matrix M per (group, rotation block) and uses
//   S = M - M^T,   R = (I - S)^-1 (I + S)                       (orthogonal for skew-symmetric S)
// The reference builds R with torch.linalg.solve on the (G, nb, rs, rs) batch
// (src/cute_prism/_module.py:534-577), which has no fp16 / bf16 kernels, launches a chain of small
// library kernels per layer and cannot be captured in a CUDA graph.  Here one thread owns one rs x rs
// block (rs = 8 or 16): Gauss-Jordan elimination of I - S in fp32 without pivoting (x^T (I - S) x =
// |x|^2 > 0, so every leading minor is positive), then R = P (I + S) with P = (I - S)^-1.
// Backward (R -> M): with G = dL/dR,  dL/dS = P^T G (R + I)^T  and  dL/dM = dL/dS - (dL/dS)^T.
// Layout as everywhere in the library: element (i, j) of block b of group g is X[g*rs + i, b*rs + j].
#include "prism_host.cuh"

namespace prism {

enum : int { CT_F16 = 0, CT_BF16 = 1, CT_F32 = 2 };

template <int CT> struct CIo;
template <> struct CIo<CT_F32> {
  using T = float;
  __device__ static float ld(const float* p) { return *p; }
  __device__ static void st(float* p, float v) { *p = v; }
};
template <> struct CIo<CT_F16> {
  using T = __half;
  __device__ static float ld(const __half* p) { return __half2float(*p); }
  __device__ static void st(__half* p, float v) { *p = __float2half_rn(v); }
};
template <> struct CIo<CT_BF16> {
  using T = __nv_bfloat16;
  __device__ static float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// 8 x 8 blocks are handled entirely in registers (every loop unrolled); for 16 x 16 the outermost loop of
// each step stays a loop (arrays in local memory): the unrolled form takes minutes to compile and these
// launches last microseconds either way.
#define PRISM_CAYLEY_OUTER(RS_, VAR_, ...)                                          \
  if constexpr ((RS_) <= 8) {                                                       \
    _Pragma("unroll") for (int VAR_ = 0; VAR_ < (RS_); ++VAR_) { __VA_ARGS__ }      \
  } else {                                                                          \
    _Pragma("unroll 1") for (int VAR_ = 0; VAR_ < (RS_); ++VAR_) { __VA_ARGS__ }    \
  }

template <int RS>
__device__ __forceinline__ void cayley_eliminate(float (&a)[RS][RS], float (&P)[RS][RS], int c) {
  const float inv = 1.f / a[c][c];
#pragma unroll
  for (int j = 0; j < RS; ++j) { a[c][j] *= inv; P[c][j] *= inv; }
#pragma unroll
  for (int r = 0; r < RS; ++r) {
    if (r == c) continue;
    const float f = a[r][c];
#pragma unroll
    for (int j = 0; j < RS; ++j) { a[r][j] -= f * a[c][j]; P[r][j] -= f * P[c][j]; }
  }
}

// P = (I - S)^-1 for S = M - M^T, by Gauss-Jordan on [I - S | I]
template <int RS>
__device__ __forceinline__ void cayley_inverse(const float (&S)[RS][RS], float (&P)[RS][RS]) {
  float a[RS][RS];
#pragma unroll
  for (int i = 0; i < RS; ++i)
#pragma unroll
    for (int j = 0; j < RS; ++j) {
      a[i][j] = (i == j ? 1.f : 0.f) - S[i][j];
      P[i][j] = (i == j ? 1.f : 0.f);
    }
  PRISM_CAYLEY_OUTER(RS, c, cayley_eliminate<RS>(a, P, c);)
}

// out[i][:] = sum_k X[i][k] * Y[k][:] (TRANS_X: X[k][i]; TRANS_Y: Y[:][k]) + (ADD_X ? X[i][:] : 0) + (ADD_I ? e_i : 0)
template <int RS, bool TRANS_X, bool TRANS_Y, bool ADD_X, bool ADD_I>
__device__ __forceinline__ void cayley_matmul_row(const float (&X)[RS][RS], const float (&Y)[RS][RS], float (&out)[RS][RS],
                                                  int i) {
#pragma unroll
  for (int j = 0; j < RS; ++j) {
    float acc = (ADD_X ? X[i][j] : 0.f) + ((ADD_I && i == j) ? 1.f : 0.f);
#pragma unroll
    for (int k = 0; k < RS; ++k) acc = fmaf(TRANS_X ? X[k][i] : X[i][k], TRANS_Y ? Y[j][k] : Y[k][j], acc);
    out[i][j] = acc;
  }
}

template <int CT, int RS>
__global__ void cayley_fwd_kernel(const typename CIo<CT>::T* __restrict__ M, typename CIo<CT>::T* __restrict__ R, int G,
                                  int nb, long long ldm, long long ldr) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)G * nb) return;
  const int g = (int)(idx / nb), b = (int)(idx - (long long)g * nb);
  const typename CIo<CT>::T* m = M + (long long)g * RS * ldm + (long long)b * RS;
  float Mv[RS][RS], S[RS][RS], P[RS][RS];
#pragma unroll
  for (int i = 0; i < RS; ++i)
#pragma unroll
    for (int j = 0; j < RS; ++j) Mv[i][j] = CIo<CT>::ld(m + i * ldm + j);
#pragma unroll
  for (int i = 0; i < RS; ++i)
#pragma unroll
    for (int j = 0; j < RS; ++j) S[i][j] = Mv[i][j] - Mv[j][i];
  cayley_inverse<RS>(S, P);
  typename CIo<CT>::T* r = R + (long long)g * RS * ldr + (long long)b * RS;
  PRISM_CAYLEY_OUTER(RS, i, cayley_matmul_row<RS, false, false, true, false>(P, S, Mv, i);)   // P (I + S) = P + P S
#pragma unroll
  for (int i = 0; i < RS; ++i)
#pragma unroll
    for (int j = 0; j < RS; ++j) CIo<CT>::st(r + i * ldr + j, Mv[i][j]);
}

template <int CT, int RS>
__global__ void cayley_bwd_kernel(const typename CIo<CT>::T* __restrict__ M, const typename CIo<CT>::T* __restrict__ dR,
                                  typename CIo<CT>::T* __restrict__ dM, int G, int nb, long long ldm, long long lddr,
                                  long long lddm) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)G * nb) return;
  const int g = (int)(idx / nb), b = (int)(idx - (long long)g * nb);
  const typename CIo<CT>::T* m = M + (long long)g * RS * ldm + (long long)b * RS;
  const typename CIo<CT>::T* gr = dR + (long long)g * RS * lddr + (long long)b * RS;
  float S[RS][RS], P[RS][RS], X[RS][RS], Y[RS][RS];
#pragma unroll
  for (int i = 0; i < RS; ++i)
#pragma unroll
    for (int j = 0; j < RS; ++j) X[i][j] = CIo<CT>::ld(m + i * ldm + j);
#pragma unroll
  for (int i = 0; i < RS; ++i)
#pragma unroll
    for (int j = 0; j < RS; ++j) S[i][j] = X[i][j] - X[j][i];
  cayley_inverse<RS>(S, P);
  // Y = R + I = P (I + S) + I
  PRISM_CAYLEY_OUTER(RS, i, cayley_matmul_row<RS, false, false, true, true>(P, S, Y, i);)
  // S <- G (the incoming gradient), X = G Y^T, then T = P^T X (kept in S)
#pragma unroll
  for (int i = 0; i < RS; ++i)
#pragma unroll
    for (int j = 0; j < RS; ++j) S[i][j] = CIo<CT>::ld(gr + i * lddr + j);
  PRISM_CAYLEY_OUTER(RS, i, cayley_matmul_row<RS, false, true, false, false>(S, Y, X, i);)
  PRISM_CAYLEY_OUTER(RS, i, cayley_matmul_row<RS, true, false, false, false>(P, X, S, i);)
  typename CIo<CT>::T* o = dM + (long long)g * RS * lddm + (long long)b * RS;
#pragma unroll
  for (int i = 0; i < RS; ++i)
#pragma unroll
    for (int j = 0; j < RS; ++j) CIo<CT>::st(o + i * lddm + j, S[i][j] - S[j][i]);
}

}  // namespace prism

using namespace prism;

static int cayley_check(const char* fn, int G, int K, int rs, int ctype) {
  if (G <= 0 || K <= 0) return fail(PRISM_ERR_BAD_ARG, "%s: bad shape G=%d K=%d", fn, G, K);
  if (rs != 8 && rs != 16) return fail(PRISM_ERR_UNSUPPORTED, "%s: reconn_sz %d is not supported (8 or 16)", fn, rs);
  if (K % rs != 0) return fail(PRISM_ERR_BAD_ARG, "%s: K (%d) must be divisible by reconn_sz (%d)", fn, K, rs);
  if (ctype != CT_F16 && ctype != CT_BF16 && ctype != CT_F32) return fail(PRISM_ERR_BAD_ARG, "%s: dtype must be 0 (fp16), 1 (bf16) or 2 (fp32)", fn);
  return PRISM_OK;
}

#define PRISM_CAYLEY_DISPATCH(CALL)                                                        \
  do {                                                                                     \
    if (rs == 8) {                                                                         \
      if (dtype == CT_F32) { CALL(CT_F32, 8); } else if (dtype == CT_BF16) { CALL(CT_BF16, 8); } else { CALL(CT_F16, 8); } \
    } else {                                                                               \
      if (dtype == CT_F32) { CALL(CT_F32, 16); } else if (dtype == CT_BF16) { CALL(CT_BF16, 16); } else { CALL(CT_F16, 16); } \
    }                                                                                      \
  } while (0)

extern "C" int prism_cayley(const void* M, void* R, int n_groups, int K, int reconn_sz, int dtype, long long ldm,
                            long long ldr, void* stream) {
  const char* fn = "prism_cayley";
  const int rs = reconn_sz;
  int rc;
  if ((rc = cayley_check(fn, n_groups, K, rs, dtype))) return rc;
  if (M == nullptr || R == nullptr) return fail(PRISM_ERR_BAD_ARG, "%s: null pointer", fn);
  if (ldm < K || ldr < K) return fail(PRISM_ERR_BAD_ARG, "%s: leading dimensions must be >= K", fn);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int nb = K / rs;
  const long long total = (long long)n_groups * nb;
  const int threads = 64;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
#define PRISM_CALL(CT_, RS_)                                                                                 \
  cayley_fwd_kernel<CT_, RS_><<<blocks, threads, 0, s>>>(reinterpret_cast<const CIo<CT_>::T*>(M),            \
                                                         reinterpret_cast<CIo<CT_>::T*>(R), n_groups, nb, ldm, ldr)
  PRISM_CAYLEY_DISPATCH(PRISM_CALL);
#undef PRISM_CALL
  return check_launch("prism_cayley");
}

extern "C" int prism_cayley_bwd(const void* M, const void* dR, void* dM, int n_groups, int K, int reconn_sz, int dtype,
                                long long ldm, long long lddr, long long lddm, void* stream) {
  const char* fn = "prism_cayley_bwd";
  const int rs = reconn_sz;
  int rc;
  if ((rc = cayley_check(fn, n_groups, K, rs, dtype))) return rc;
  if (M == nullptr || dR == nullptr || dM == nullptr) return fail(PRISM_ERR_BAD_ARG, "%s: null pointer", fn);
  if (ldm < K || lddr < K || lddm < K) return fail(PRISM_ERR_BAD_ARG, "%s: leading dimensions must be >= K", fn);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int nb = K / rs;
  const long long total = (long long)n_groups * nb;
  const int threads = 64;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
#define PRISM_CALL(CT_, RS_)                                                                                  \
  cayley_bwd_kernel<CT_, RS_><<<blocks, threads, 0, s>>>(reinterpret_cast<const CIo<CT_>::T*>(M),             \
                                                         reinterpret_cast<const CIo<CT_>::T*>(dR),            \
                                                         reinterpret_cast<CIo<CT_>::T*>(dM), n_groups, nb, ldm, lddr, lddm)
  PRISM_CAYLEY_DISPATCH(PRISM_CALL);
#undef PRISM_CALL
  return check_launch("prism_cayley_bwd");
}
