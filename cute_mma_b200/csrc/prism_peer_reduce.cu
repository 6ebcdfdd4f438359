// Sum of the parameter gradients (dR, dB, bias gradient) over the GPUs of one box, over peer memory.
//
// The reference has no collective of its own: its training script leaves the sum to
// DistributedDataParallel's NCCL all-reduce (integration/train.py:130-145, 299-300).  Here every rank's
// reduction kernels leave their fp32 sums in a buffer that all ranks of the box can address (symmetric
// memory: the same allocation on every GPU, mapped into every process), and this kernel is the exchange:
//   * rank r owns slice r of the flat gradient buffer.  It loads that slice from every rank's buffer with
//     plain loads over NVLink (its own included), adds the ranks in rank order -- a fixed order, so the sum
//     is bit-identical on every run and on every rank -- scales, casts, and stores the result into every
//     rank's result buffer with plain stores (reduce-scatter and all-gather in one pass: each element
//     crosses NVLink once as fp32 on the way in and once in the output type on the way out).
//   * there is no waiting inside the kernel: the caller orders it between two barriers over the ranks
//     (after every rank's gradients are in its buffer; before anybody reads a result or rewrites a buffer).
// No TMA, no multicast, no library kernel touches a peer's memory: 16-byte ld.global / st.global only.
#include "prism_host.cuh"

namespace prism {

constexpr int kMaxPeers = 16;

struct PeerReduceParams {
  const float* in[kMaxPeers];    // every rank's fp32 gradient buffer (this rank's mapping of it)
  void* out[kMaxPeers];          // every rank's result buffer
  long long lo, hi;              // this rank's slice [lo, hi) of the flat buffer, multiples of 4
  int world;
  float scale;
};

template <int OUT>
__device__ __forceinline__ void peer_store(const PeerReduceParams& p, long long e, float4 acc) {
  acc.x *= p.scale; acc.y *= p.scale; acc.z *= p.scale; acc.w *= p.scale;
  if constexpr (OUT == 2) {
    for (int r = 0; r < p.world; ++r) *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out[r]) + e) = acc;
  } else {
    uint2 w;
    w.x = Elem<OUT>::pack(acc.x, acc.y);
    w.y = Elem<OUT>::pack(acc.z, acc.w);
    for (int r = 0; r < p.world; ++r) *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.out[r]) + e) = w;
  }
}

// A load over NVLink takes a few microseconds: every thread keeps 16 16-byte loads in flight, kUnroll per rank
// and all ranks at once (a small grid must still cover the link's bandwidth-delay product).
// WORLD: 2, 4, 8 (all loads issued before the first add), or 0: any count, rank after rank.
template <int OUT, int WORLD>   // OUT: DT_F16, DT_BF16, or 2: fp32
__global__ void __launch_bounds__(512) prism_peer_reduce_kernel(const PeerReduceParams p) {
  constexpr int kUnroll = WORLD > 0 ? 16 / WORLD : 8;
  const long long n4 = (p.hi - p.lo) >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < n4; i0 += stride * kUnroll) {
    float4 acc[kUnroll];
    if constexpr (WORLD > 0) {
      float4 v[WORLD][kUnroll];
#pragma unroll
      for (int r = 0; r < WORLD; ++r)
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const long long i = i0 + u * stride;
          v[r][u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (i < n4) v[r][u] = __ldcg(reinterpret_cast<const float4*>(p.in[r] + p.lo + i * 4));
        }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        acc[u] = v[0][u];
#pragma unroll
        for (int r = 1; r < WORLD; ++r) {   // ranks in rank order: the sum is the same on every rank
          acc[u].x += v[r][u].x; acc[u].y += v[r][u].y; acc[u].z += v[r][u].z; acc[u].w += v[r][u].w;
        }
      }
    } else {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long i = i0 + u * stride;
        acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) acc[u] = __ldcg(reinterpret_cast<const float4*>(p.in[0] + p.lo + i * 4));
      }
      for (int r = 1; r < p.world; ++r) {
        float4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const long long i = i0 + u * stride;
          v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (i < n4) v[u] = __ldcg(reinterpret_cast<const float4*>(p.in[r] + p.lo + i * 4));
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long i = i0 + u * stride;
      if (i < n4) peer_store<OUT>(p, p.lo + i * 4, acc[u]);
    }
  }
}

template <int OUT>
static void peer_reduce_launch(const PeerReduceParams& p, int ctas, cudaStream_t s) {
  if (p.world == 2) prism_peer_reduce_kernel<OUT, 2><<<ctas, 512, 0, s>>>(p);
  else if (p.world == 4) prism_peer_reduce_kernel<OUT, 4><<<ctas, 512, 0, s>>>(p);
  else if (p.world == 8) prism_peer_reduce_kernel<OUT, 8><<<ctas, 512, 0, s>>>(p);
  else prism_peer_reduce_kernel<OUT, 0><<<ctas, 512, 0, s>>>(p);
}

}  // namespace prism

using namespace prism;

extern "C" int prism_peer_reduce(const void* const* in_ptrs, void* const* out_ptrs, int world, int rank, long long n,
                                 int out_dtype, float scale, int ctas, void* stream) {
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    return fail(PRISM_ERR_BAD_ARG, "prism_peer_reduce: world=%d rank=%d (at most %d ranks)", world, rank, kMaxPeers);
  if (n < 0 || (n & 3) != 0) return fail(PRISM_ERR_BAD_ARG, "prism_peer_reduce: n=%lld must be a multiple of 4", n);
  if (out_dtype != PRISM_DTYPE_F16 && out_dtype != PRISM_DTYPE_BF16 && out_dtype != PRISM_DTYPE_F32)
    return fail(PRISM_ERR_BAD_ARG, "prism_peer_reduce: out_dtype=%d", out_dtype);
  PeerReduceParams p;
  for (int r = 0; r < world; ++r) {
    if (in_ptrs[r] == nullptr || out_ptrs[r] == nullptr) return fail(PRISM_ERR_BAD_ARG, "prism_peer_reduce: null buffer of rank %d", r);
    if ((reinterpret_cast<uintptr_t>(in_ptrs[r]) | reinterpret_cast<uintptr_t>(out_ptrs[r])) & 15)
      return fail(PRISM_ERR_BAD_ARG, "prism_peer_reduce: buffers must be 16-byte aligned");
    p.in[r] = reinterpret_cast<const float*>(in_ptrs[r]);
    p.out[r] = out_ptrs[r];
  }
  const long long n4 = n >> 2;
  p.lo = (n4 * rank / world) << 2;
  p.hi = (n4 * (rank + 1) / world) << 2;
  p.world = world;
  p.scale = scale;
  if (p.hi == p.lo) return PRISM_OK;
  if (ctas < 1) ctas = 16;
  const long long want = ((p.hi - p.lo) / 4 + 512 * 8 - 1) / (512 * 8);
  if (ctas > want) ctas = (int)want;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (out_dtype == PRISM_DTYPE_F32) peer_reduce_launch<2>(p, ctas, s);
  else if (out_dtype == PRISM_DTYPE_BF16) peer_reduce_launch<DT_BF16>(p, ctas, s);
  else peer_reduce_launch<DT_F16>(p, ctas, s);
  return check_launch("prism_peer_reduce");
}
