// All-gather fused with the GEMM that consumes the gathered operand.
//
// One launch holds two kinds of CTAs:
//   * copy CTAs (blockIdx < n_copy): pull remote shards of the operand over NVLink with plain
//     peer loads, write them into this GPU's own buffer and publish a per-row-group flag;
//     after the flagged tasks they keep pulling "trailing" tasks (the rest of a parameter
//     group, which later kernels of the layer need) without flags;
//   * GEMM CTAs: the persistent tcgen05 GEMM of gemm_core.cuh; its TMA producer waits for the
//     flag of the rows a tile needs, and tiles are ordered so that rows this rank already owns
//     come first and remote rows follow in the order the copy CTAs fetch them.
// The operand therefore crosses NVLink once, lands where every later kernel reads it, and the
// transfer overlaps the tensor-core work tile by tile.  Both weight-gathered (FSDP: B operand)
// and activation-gathered (sequence parallel: A operand) forms are provided.
#include "comm.cuh"
#include "gemm_2sm.cuh"
#include "gemm_core.cuh"
#include "tensormap.cuh"

namespace ob {
namespace gemm {

constexpr int AG_THREADS = 512;  // copy CTAs use all of them; GEMM CTAs only the first 192 (512 keeps 128 registers per thread for the epilogue)

template <int B_MN, int SWIGLU>
__global__ void __launch_bounds__(AG_THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmB2, const Params p,
               const comm::CopyTask* __restrict__ tasks, int n_tasks, comm::PeerPtrs src, __nv_bfloat16* dst,
               int* flags, int epoch, int n_copy) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x < n_copy) {
    comm::run_copy_tasks<16>(tasks, n_tasks, blockIdx.x, n_copy, src, dst, flags, epoch);
    return;
  }
  if (threadIdx.x >= NUM_THREADS) return;  // spare warps of a GEMM CTA
  gemm_cta<0, B_MN, SWIGLU>(&tmA, &tmB, &tmB2, p, blockIdx.x - n_copy, gridDim.x - n_copy, smem_raw);
}

// Push form of the same launch: copy CTAs store this rank's slice into every peer's operand buffer.
template <int B_MN, int SWIGLU>
__global__ void __launch_bounds__(AG_THREADS, 1)
ag_push_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmB2, const Params p,
                    const comm::CopyTask* __restrict__ tasks, int n_tasks, const __nv_bfloat16* __restrict__ src,
                    long long slice_base, comm::PeerPtrs dst, comm::PeerPtrs flag_ptrs, int epoch, int n_copy) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x < n_copy) {
    comm::run_push_tasks<8>(tasks, n_tasks, blockIdx.x, n_copy, src, slice_base, dst, flag_ptrs, epoch);
    return;
  }
  if (threadIdx.x >= NUM_THREADS) return;
  gemm_cta<0, B_MN, SWIGLU>(&tmA, &tmB, &tmB2, p, blockIdx.x - n_copy, gridDim.x - n_copy, smem_raw);
}

template <int B_MN, int SWIGLU>
static int launch_ag_push(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const Params& p,
                          const void* tasks, int n_tasks, const void* src, long long slice_base,
                          const void* const* dst_ptrs, const void* const* flag_ptrs, int world, int epoch, int n_copy,
                          cudaStream_t stream) {
  auto kern = ag_push_gemm_kernel<B_MN, SWIGLU>;
  static bool configured = false;
  if (!configured) {
    OB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (n_tasks == 0) n_copy = 0;
  if (n_copy > sms / 2) n_copy = sms / 2;
  const int bn = SWIGLU ? BN / 2 : BN;
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + bn - 1) / bn);
  int gemm_ctas = sms - n_copy;
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  comm::PeerPtrs dst{}, fl{};
  for (int i = 0; i < world; ++i) {
    dst.p[i] = const_cast<void*>(dst_ptrs[i]);
    fl.p[i] = const_cast<void*>(flag_ptrs[i]);
  }
  kern<<<n_copy + gemm_ctas, AG_THREADS, SMEM_BYTES, stream>>>(ta, tb, tb2, p, (const comm::CopyTask*)tasks, n_tasks,
                                                               (const __nv_bfloat16*)src, slice_base, dst, fl, epoch,
                                                               n_copy);
  return (int)cudaGetLastError();
}

template <int B_MN, int SWIGLU>
static int launch_ag(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const Params& p,
                     const void* tasks, int n_tasks, const void* const* src_ptrs, int world, void* dst, int* flags,
                     int epoch, int n_copy, cudaStream_t stream) {
  auto kern = ag_gemm_kernel<B_MN, SWIGLU>;
  static bool configured = false;
  if (!configured) {
    OB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (n_tasks == 0) n_copy = 0;
  if (n_copy > sms / 2) n_copy = sms / 2;
  const int bn = SWIGLU ? BN / 2 : BN;
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + bn - 1) / bn);
  int gemm_ctas = sms - n_copy;
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  comm::PeerPtrs src{};
  for (int i = 0; i < world; ++i) src.p[i] = const_cast<void*>(src_ptrs[i]);
  kern<<<n_copy + gemm_ctas, AG_THREADS, SMEM_BYTES, stream>>>(ta, tb, tb2, p, (const comm::CopyTask*)tasks, n_tasks,
                                                               src, (__nv_bfloat16*)dst, flags, epoch, n_copy);
  return (int)cudaGetLastError();
}

}  // namespace gemm

namespace gemm2 {

// Weight-gathered form on the two-SM GEMM: the grid is made of CTA pairs (clusters of two); the first n_copy / 2
// pairs pull remote rows of B with plain peer loads and raise the row-group flags, the other pairs run the paired
// GEMM whose producers wait for the flags of the 128 B rows each of them stages.
constexpr int AG2_THREADS = 512;

__global__ void __launch_bounds__(AG2_THREADS, 1)
ag_gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const gemm::Params p,
                const comm::CopyTask* __restrict__ tasks, int n_tasks, comm::PeerPtrs src, __nv_bfloat16* dst, int* flags,
                int epoch, int n_copy) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x < n_copy) {
    comm::run_copy_tasks<16>(tasks, n_tasks, blockIdx.x, n_copy, src, dst, flags, epoch);
    return;
  }
  if (threadIdx.x >= NUM_THREADS) return;  // spare warps of a GEMM CTA
  gemm2_cta<0, 0, 0>(&tmA, &tmB, &tmB, p, ((int)blockIdx.x - n_copy) >> 1, ((int)gridDim.x - n_copy) >> 1, smem_raw);
}

}  // namespace gemm2
}  // namespace ob

using namespace ob;
using namespace ob::gemm;

// Two-SM form of ob_gemm_ag_bf16 for a gathered B operand (FSDP: the fused QKV weight).  Same arguments; n_copy is
// rounded up to an even number of copy CTAs.
extern "C" int ob_gemm2_ag_bf16(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc,
                                int M, int N, int K, const void* bias, const void* tasks, int n_tasks,
                                const void* const* src_ptrs, int world, void* dst, int* flags, int flag_rows,
                                int epoch, int first_tile_shift, int n_copy, int* status, cudaStream_t stream) {
  if (world > comm::MAX_RANKS) return -1;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, A, M, K, lda, 128, gemm2::BK, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tb, B, N, K, ldb, 128, gemm2::BK, 2);
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.alpha = 1.0f; p.bias = bias; p.status = status;
  p.a_flag_rows = 1;
  p.b_flags = flags; p.flag_rows = flag_rows > 0 ? flag_rows : 1; p.flag_value = epoch; p.tile_order = 1;
  p.first_tile_shift = first_tile_shift;
  auto kern = gemm2::ag_gemm2_kernel;
  static int max_pairs = 0;
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(gemm2::AG2_THREADS); cfg.dynamicSmemBytes = gemm2::SMEM_BYTES; cfg.stream = stream;
  cfg.attrs = attr; cfg.numAttrs = 1;
  if (max_pairs == 0) {
    OB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm2::SMEM_BYTES));
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cfg.gridDim = dim3(sms & ~1);
    int n = 0;
    OB_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
    if (n <= 0) return -4;
    max_pairs = n < sms / 2 ? n : sms / 2;
  }
  if (n_tasks == 0) n_copy = 0;
  n_copy = (n_copy + 1) & ~1;
  if (n_copy / 2 > max_pairs / 2) n_copy = (max_pairs / 2) * 2;
  const int tiles = ((M + gemm2::TM - 1) / gemm2::TM) * ((N + gemm2::TN - 1) / gemm2::TN);
  int pairs = max_pairs - n_copy / 2;
  if (pairs > tiles) pairs = tiles;
  if (pairs < 1) return -5;
  comm::PeerPtrs src{};
  for (int i = 0; i < world; ++i) src.p[i] = const_cast<void*>(src_ptrs[i]);
  cfg.gridDim = dim3(n_copy + 2 * pairs);
  return (int)cudaLaunchKernelEx(&cfg, kern, ta, tb, p, (const comm::CopyTask*)tasks, n_tasks, src, (__nv_bfloat16*)dst,
                                 flags, epoch, n_copy);
}

// C[M,N] = A[M,K] B[N,K]^T where B (gather_a = 0) or A (gather_a = 1) is being gathered by this
// same launch.  `dst` is the local buffer that holds the gathered operand (and possibly more:
// task offsets are relative to it), `src_ptrs` the peers' copies of it.  flags[i] >= epoch means
// rows [i*flag_rows, (i+1)*flag_rows) of the gathered operand are in place; the caller pre-sets
// the flags of locally owned rows.
extern "C" int ob_gemm_ag_bf16(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc,
                               int M, int N, int K, const void* bias, const void* tasks, int n_tasks,
                               const void* const* src_ptrs, int world, void* dst, int* flags, int flag_rows,
                               int epoch, int gather_a, int first_tile_shift, int n_copy, int* status,
                               cudaStream_t stream) {
  if (world > comm::MAX_RANKS) return -1;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tb, B, N, K, ldb, BN, BK, 2);
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.alpha = 1.0f; p.bias = bias; p.status = status;
  p.flag_rows = 1; p.a_flag_rows = 1;
  if (gather_a) { p.a_flags = flags; p.a_flag_rows = flag_rows; p.a_flag_value = epoch; p.tile_order = 2; }
  else { p.b_flags = flags; p.flag_rows = flag_rows; p.flag_value = epoch; p.tile_order = 1; }
  p.first_tile_shift = first_tile_shift;
  return launch_ag<0, 0>(ta, tb, tb, p, tasks, n_tasks, src_ptrs, world, dst, flags, epoch, n_copy, stream);
}

// Sequence-parallel forms: the activation A[M,K] is the gathered operand (flags per `flag_rows`
// rows of A, m-major tile order rotated by first_tile_shift m-tiles).
//   b_mn = 0: B is [N,K] row-major (column-parallel forward);  b_mn = 1: B is [K,N] row-major
//   (row-parallel backward, dx = dy_full W).
//   B2 != nullptr: dual-B SwiGLU, H = silu(A B^T) * (A B2^T) with optional G / U outputs (b_mn = 0 only).
extern "C" int ob_gemm_ag_act_bf16(const void* A, long long lda, const void* B, const void* B2, long long ldb, int b_mn,
                                   void* C, void* G, void* U, long long ldc, int M, int N, int K, const void* bias,
                                   const void* tasks, int n_tasks, const void* const* src_ptrs, int world, void* dst,
                                   int* flags, int flag_rows, int epoch, int first_tile_shift, int n_copy,
                                   int* status, cudaStream_t stream) {
  if (world > comm::MAX_RANKS) return -1;
  if (B2 != nullptr && b_mn) return -2;
  CUtensorMap ta, tb, tb2;
  int rc = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2);
  if (rc) return rc;
  if (B2 != nullptr) {
    rc = make_tmap_2d(&tb, B, N, K, ldb, BN / 2, BK, 2);
    if (rc) return rc;
    rc = make_tmap_2d(&tb2, B2, N, K, ldb, BN / 2, BK, 2);
  } else if (b_mn) {
    rc = make_tmap_2d(&tb, B, K, N, ldb, BK, 64, 2);
    tb2 = tb;
  } else {
    rc = make_tmap_2d(&tb, B, N, K, ldb, BN, BK, 2);
    tb2 = tb;
  }
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.alpha = 1.0f; p.bias = bias; p.status = status;
  p.G = G; p.U = U;
  p.flag_rows = 1;
  p.a_flags = flags; p.a_flag_rows = flag_rows > 0 ? flag_rows : 1; p.a_flag_value = epoch; p.tile_order = 2;
  p.first_tile_shift = first_tile_shift;
  if (B2 != nullptr)
    return launch_ag<0, 1>(ta, tb, tb2, p, tasks, n_tasks, src_ptrs, world, dst, flags, epoch, n_copy, stream);
  if (b_mn) return launch_ag<1, 0>(ta, tb, tb2, p, tasks, n_tasks, src_ptrs, world, dst, flags, epoch, n_copy, stream);
  return launch_ag<0, 0>(ta, tb, tb2, p, tasks, n_tasks, src_ptrs, world, dst, flags, epoch, n_copy, stream);
}

// Push form of ob_gemm_ag_act_bf16.  A is this rank's gathered-operand buffer [M,K] in symmetric memory (its own
// rows already copied and flagged by the caller); `x_local` is this rank's slice, whose chunks the copy CTAs
// store into dst_ptrs[peer] + task.offset and publish through flag_ptrs[peer][task.flag] = epoch.  The GEMM CTAs
// wait on this rank's own flag array `flags` (the one the peers write).
extern "C" int ob_gemm_ag_push_bf16(const void* A, long long lda, const void* x_local, long long slice_base,
                                    const void* B, const void* B2, long long ldb, int b_mn, void* C, void* G, void* U,
                                    long long ldc, int M, int N, int K, const void* bias, const void* tasks,
                                    int n_tasks, const void* const* dst_ptrs, const void* const* flag_ptrs, int world,
                                    int* flags, int flag_rows, int epoch, int first_tile_shift, int n_copy,
                                    int* status, cudaStream_t stream) {
  if (world > comm::MAX_RANKS) return -1;
  if (B2 != nullptr && b_mn) return -2;
  CUtensorMap ta, tb, tb2;
  int rc = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2);
  if (rc) return rc;
  if (B2 != nullptr) {
    rc = make_tmap_2d(&tb, B, N, K, ldb, BN / 2, BK, 2);
    if (rc) return rc;
    rc = make_tmap_2d(&tb2, B2, N, K, ldb, BN / 2, BK, 2);
  } else if (b_mn) {
    rc = make_tmap_2d(&tb, B, K, N, ldb, BK, 64, 2);
    tb2 = tb;
  } else {
    rc = make_tmap_2d(&tb, B, N, K, ldb, BN, BK, 2);
    tb2 = tb;
  }
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.alpha = 1.0f; p.bias = bias; p.status = status;
  p.G = G; p.U = U;
  p.flag_rows = 1;
  p.a_flags = flags; p.a_flag_rows = flag_rows > 0 ? flag_rows : 1; p.a_flag_value = epoch; p.tile_order = 2;
  p.first_tile_shift = first_tile_shift;
  if (B2 != nullptr)
    return launch_ag_push<0, 1>(ta, tb, tb2, p, tasks, n_tasks, x_local, slice_base, dst_ptrs, flag_ptrs, world, epoch,
                                n_copy, stream);
  if (b_mn)
    return launch_ag_push<1, 0>(ta, tb, tb2, p, tasks, n_tasks, x_local, slice_base, dst_ptrs, flag_ptrs, world, epoch,
                                n_copy, stream);
  return launch_ag_push<0, 0>(ta, tb, tb2, p, tasks, n_tasks, x_local, slice_base, dst_ptrs, flag_ptrs, world, epoch,
                              n_copy, stream);
}
