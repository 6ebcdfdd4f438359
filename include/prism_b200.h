/* prism_b200 -- C ABI of the B200 (sm_100a) Prism linear-layer kernels.
 *
 * One shared library (libprism_b200.so) replaces the three per-variant torch
 * extensions of the reference:
 *   prism_fwd       <-> forward(A, B, R, group_size, reconn_sz, ...)          torch_ext/prism_fwd_bind.cpp:14-26
 *                       (prism_forward, torch_ext/prism_fwd_torch.cu:23-196)
 *   prism_bwd_dadr  <-> backward_dA_dR(dC, A, B, R, group_size, reconn_sz, ..) torch_ext/prism_bwd_dadr_bind.cpp:15-28
 *                       (prism_backward_dA_dR, torch_ext/prism_bwd_dadr_torch.cu:42-210)
 *   prism_bwd_db    <-> backward_dB(dC, A, R, group_size, reconn_sz, ...)      torch_ext/prism_bwd_db_bind.cpp:14-26
 *                       (prism_backward_dB, torch_ext/prism_bwd_db_torch.cu:42-162)
 *
 * Conventions
 *   - all matrices are row-major 16-bit (dtype 0 = fp16, 1 = bf16), device pointers,
 *     16-byte aligned, leading dimensions in elements and multiples of 8;
 *     A [M,K], B [N,K], R [(N/group_size)*reconn_sz, K], C/dC [M,N];
 *   - group_size must be a multiple of 16 (the reference accepts multiples of 8,
 *     src/cute_prism/_validate.py:26-30; the tensor-core tiles here are 16 wide) and reconn_sz one
 *     of 8, 16, 32, 64;
 *   - gate 0 = plain "ar" mode (C_g = (A.blockdiag(R_g)^T) B_g^T), 1 = silu_gate
 *     (C_g = (A * silu(A.blockdiag(R_g)^T)) B_g^T), 2 = sigmoid_gate
 *     (C_g = (A * 2 sigmoid(A.blockdiag(R_g)^T)) B_g^T; the reference has it in its cuBLAS
 *     and PyTorch backends only, src/cute_prism/_pytorch_backend.py:157-163);
 *   - the library never allocates or frees device memory: outputs and the workspace
 *     belong to the caller.  The workspace must be 256-byte aligned, at least
 *     prism_workspace_bytes(...) long, and its first 256 bytes (the status header)
 *     must be zero when it is first used; the kernels write every output element;
 *   - every call is asynchronous on `stream` (a cudaStream_t) and returns 0 on
 *     success or a PRISM_ERR_* code; prism_last_error_string() describes the last
 *     failure of the calling thread.  Errors detected on the device (a bounded wait
 *     that ran out) are recorded in the workspace header and read with prism_status();
 *   - `cfg` optionally overrides the tile configuration (null = built-in default);
 *     its meaning per kernel is given below.
 */
#ifndef PRISM_B200_H
#define PRISM_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PRISM_OK 0
#define PRISM_ERR_BAD_ARG 1
#define PRISM_ERR_UNSUPPORTED 2
#define PRISM_ERR_WORKSPACE 3
#define PRISM_ERR_CUDA 4
#define PRISM_ERR_DEVICE_WAIT 5
#define PRISM_ERR_NO_DRIVER 6

#define PRISM_KIND_FWD 0
#define PRISM_KIND_BWD_DADR 1
#define PRISM_KIND_BWD_DB 2
#define PRISM_KIND_DBIAS 3
#define PRISM_KIND_BWD_DADR_IB 4   /* prism_bwd_dadr with an internal bias (more scratch) */

/* element types: the 16-bit input types, and fp32 for gradient outputs that should leave unrounded */
#define PRISM_DTYPE_F16 0
#define PRISM_DTYPE_BF16 1
#define PRISM_DTYPE_F32 2
#define PRISM_DTYPE_SAME (-1)   /* a gradient output in the inputs' 16-bit type */

#define PRISM_WORKSPACE_HEADER_BYTES 256
/* size of the library's built-in scratch array used by prism_fwd_noalloc: 8 MiB + the status header */
#define PRISM_NOALLOC_SCRATCH_BYTES (8 * 1024 * 1024 + 256)

/* Forward.  bias: [N] in the same dtype, or NULL.  internal_bias: [N/group_size, K] in the same dtype
 * (contiguous rows), or NULL: added to A.blockdiag(R_g)^T before the gate (gated modes only; reference:
 * src/cute_prism/_pytorch_backend.py:154-156, cute_prism_coop_pc.cu:250-301).  cfg (4 ints, 0 = default): {BN, PM, stages, path}:
 * N tile (divides group_size, <= 256), row tiles per rasterisation panel, shared-memory stages, and the
 * kernel: 0 = by shape, 1 = the general tiled kernel, 2 = the few-token streaming kernel (M <= 128 and
 * group_size a multiple of 128; picked by default up to 48 tokens).  The streaming kernel cuts B into
 * equal shares for all SMs, keeps fp32 partial sums of the shares in the workspace and adds them in a
 * fixed order, so its result is bit-stable; ask prism_workspace_bytes with the same cfg. */
int prism_fwd(const void* A, const void* B, const void* R, const void* bias, const void* internal_bias, void* C,
              int M, int N, int K, int group_size, int reconn_sz, int dtype, int gate,
              long long lda, long long ldb, long long ldr, long long ldc,
              const int* cfg, void* workspace, size_t workspace_bytes, void* stream);

/* Forward with hash dropout of the gated activation (training): element (m, k) of group g of
 * H = A * gate(S) is kept iff top24(splitmix64(splitmix64(seed_g + 0xdeadbeef) ^ splitmix64(m*K + k))) / 2^24
 * >= dropout_p, and kept elements are scaled by 1 / (1 - dropout_p): the counter-based mask of the
 * reference's kernels (cute_prism_dtype.hpp:28-40).  dropout_seeds: [N/group_size] int64 on the device,
 * chosen by the caller (the reference draws them in [1, 2^62), src/cute_prism/__init__.py:242-250) and
 * passed again to the two backward calls, which regenerate the mask.  Gated modes, reconn_sz 8 or 16.
 * dropout_seeds = NULL: no dropout (prism_fwd is this call without dropout). */
int prism_fwd_dropout(const void* A, const void* B, const void* R, const void* bias, const void* internal_bias,
                      void* C, int M, int N, int K, int group_size, int reconn_sz, int dtype, int gate,
                      long long lda, long long ldb, long long ldr, long long ldc,
                      const long long* dropout_seeds, float dropout_p,
                      const int* cfg, void* workspace, size_t workspace_bytes, void* stream);

/* Forward for callers that cannot allocate device memory and therefore cannot supply a workspace.
 * (No counterpart in the reference: its bindings allocate outputs and scratch themselves.)
 * Same arguments and results as prism_fwd, except that the scratch is a fixed array of
 * PRISM_NOALLOC_SCRATCH_BYTES inside the library (resident on every GPU that loads the library
 * until the process exits).  The call fails with PRISM_ERR_WORKSPACE when the shape needs more:
 * 256 bytes, plus (N/group_size)*16*K*2 bytes when reconn_sz = 8.  It calls no cudaMalloc / cudaFree
 * and no allocating library routine.  All calls on a GPU share the array: calls ordered on one
 * stream are independent (each rewrites what it reads and clears the status word first), calls
 * that can overlap on the GPU race and give undefined results.  The first call on each GPU looks
 * up the array's device address; make that call outside any stream capture.
 * device_status: NULL, or where the 4-byte device status word of this call is copied
 * (stream-ordered; device or pinned host memory). */
int prism_fwd_noalloc(const void* A, const void* B, const void* R, const void* bias, void* C,
                      int M, int N, int K, int group_size, int reconn_sz, int dtype, int gate,
                      long long lda, long long ldb, long long ldr, long long ldc,
                      const int* cfg, int* device_status, void* stream);

/* Input and rotation gradients: dA [M,K] and dR [(N/group_size)*reconn_sz, K], both scaled by
 * dc_scale.  dr_dtype: PRISM_DTYPE_SAME (dR in the inputs' type) or PRISM_DTYPE_F32 (the fp32 sums of
 * the second-level reduction leave unrounded, lddr in fp32 elements; the reference offers the same
 * through dR_dtype, src/cute_prism/__init__.py:288-289,368).  cfg (3 ints, 0 = default): {runs, steal, n_extra} -- runs: the number of main CTA
 * pairs that share one 128-feature column of dA (each walks every runs-th 256-token tile); when
 * the main pairs leave SMs idle, n_extra extra pairs take over the last `steal` tiles of every
 * main pair (steal < 0: never).  Each CTA accumulates dR into fp32 memory of its own
 * in the workspace in a fixed order and a second kernel adds the buffers in a fixed order: dR is
 * bit-identical from run to run.  The workspace also holds the kernel's copy of R (widened for
 * reconn_sz = 8, halved in the gated mode).  internal_bias (or NULL): as in prism_fwd; then
 * d_internal_bias [N/group_size, K] (input dtype) receives dc_scale * sum over tokens of dS, summed in a
 * fixed order like dR, and the workspace is sized with PRISM_KIND_BWD_DADR_IB.  dropout_seeds /
 * dropout_p: the forward's (prism_fwd_dropout), or NULL / 0: dH is multiplied by the same mask. */
int prism_bwd_dadr(const void* dC, const void* A, const void* B, const void* R, const void* internal_bias,
                   void* dA, void* dR, void* d_internal_bias, int M, int N, int K, int group_size, int reconn_sz, int dtype, int gate,
                   int dr_dtype, float dc_scale, long long lddc, long long lda, long long ldb, long long ldr,
                   long long ldda, long long lddr, const long long* dropout_seeds, float dropout_p,
                   const int* cfg, void* workspace, size_t workspace_bytes, void* stream);

/* Weight gradient dB [N,K] = dc_scale * dC^T . H (H recomputed from A and R; B is not needed).
 * db_dtype: PRISM_DTYPE_SAME or PRISM_DTYPE_F32 (dB written as fp32, lddb in fp32 elements;
 * reference: dB_dtype, src/cute_prism/__init__.py:288-289,375).
 * cfg (2 ints, 0 = default): {BN, splits} -- splits > 1 divides the token range of every tile over
 * several CTA pairs whose fp32 partial sums (in the workspace) are added in a fixed order, so the
 * result is deterministic; splits < 0 never splits.  By default only the n-tile rows of a mostly
 * empty last wave are split (in a second launch). */
int prism_bwd_db(const void* dC, const void* A, const void* R, const void* internal_bias, void* dB,
                 int M, int N, int K, int group_size, int reconn_sz, int dtype, int gate,
                 int db_dtype, float dc_scale, long long lddc, long long lda, long long ldr, long long lddb,
                 const long long* dropout_seeds, float dropout_p,
                 const int* cfg, void* workspace, size_t workspace_bytes, void* stream);

/* Output-bias gradient dbias [N] = sum over the M token rows of dC [M,N] (not scaled: the bias is
 * added after the point where the reference's constant backward rescale applies).  The reference adds
 * the bias as a separate torch op (src/cute_prism/_module.py:736-737), whose autograd is this column
 * sum.  Two launches, partial sums over row ranges added in a fixed order: bit-stable.
 * dbias_dtype: PRISM_DTYPE_SAME or PRISM_DTYPE_F32.  Workspace: prism_workspace_bytes(PRISM_KIND_DBIAS, M, N, ...). */
int prism_dbias(const void* dC, void* dbias, int M, int N, int dtype, int dbias_dtype, long long lddc,
                void* workspace, size_t workspace_bytes, void* stream);

/* Weight folding of the reference's "rw" mode (inference with the rotation folded into the weight,
 * src/cute_prism/_pytorch_backend.py:115-124): Bp [N,K] with
 * Bp[n, b*rs + j] = sum_i B[n, b*rs + i] * R[(n/group_size)*rs + i, b*rs + j], so that A . Bp^T equals the
 * plain-mode forward.  No workspace.  The dense product that follows is an ordinary GEMM. */
int prism_fold_weight(const void* B, const void* R, void* Bp, int N, int K, int group_size, int reconn_sz,
                      int dtype, long long ldb, long long ldr, long long ldbp, void* stream);

/* Rotation blocks of the plain (fine-tuning) mode from the stored parameter: for every reconn_sz x
 * reconn_sz block, S = M - M^T and R = (I - S)^-1 (I + S), computed in fp32 by one thread per block
 * (reconn_sz 8 or 16).  Replaces the torch.linalg.solve chain of the reference's
 * PrismLinear._build_R (src/cute_prism/_module.py:534-577), works for fp16 / bf16 / fp32 parameters
 * (dtype 0 / 1 / 2) and can be captured in a CUDA graph.  M, R: [n_groups*reconn_sz, K].
 * prism_cayley_bwd: dM from dR (dL/dS = P^T dR (R + I)^T with P = (I - S)^-1, dM = dL/dS - (dL/dS)^T). */
int prism_cayley(const void* M, void* R, int n_groups, int K, int reconn_sz, int dtype, long long ldm,
                 long long ldr, void* stream);
int prism_cayley_bwd(const void* M, const void* dR, void* dM, int n_groups, int K, int reconn_sz, int dtype,
                     long long ldm, long long lddr, long long lddm, void* stream);

/* Sum of gradient buffers over the GPUs of one box, over peer memory: the exchange step of token-sharded
 * training (the reference leaves it to DistributedDataParallel's all-reduce, integration/train.py:130-145,
 * 299-300).  in_ptrs / out_ptrs: HOST arrays of `world` device pointers -- every rank's fp32 buffer of n
 * elements and every rank's result buffer (out_dtype: PRISM_DTYPE_F16 / BF16 / F32), as this process maps
 * them (symmetric memory, CUDA IPC).  Rank `rank` sums its n / world slice over the ranks in rank order
 * (bit-identical on every rank and run), multiplies by `scale`, and stores the result into every rank's
 * result buffer.  The kernel does not wait for anybody: call it between two barriers over the ranks
 * (all inputs written; nobody reads a result or rewrites an input before all ranks are done).
 * n: a multiple of 4; buffers 16-byte aligned; ctas: grid size (0 = 16). */
int prism_peer_reduce(const void* const* in_ptrs, void* const* out_ptrs, int world, int rank, long long n,
                      int out_dtype, float scale, int ctas, void* stream);

/* Bytes of workspace the given call needs (kind = PRISM_KIND_*), header included. */
size_t prism_workspace_bytes(int kind, int M, int N, int K, int group_size, int reconn_sz,
                             int dtype, const int* cfg);

/* Synchronises `stream`, returns the device status word of the workspace header
 * (0 = no device-side error since the header was last zero) and clears it. */
int prism_status(void* workspace, void* stream);

const char* prism_last_error_string(void);

/* Number of CUDA kernels the library has launched so far in this process. */
long long prism_launch_count(void);

/* Library / ABI version, for the loader's sanity check. */
int prism_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* PRISM_B200_H */
