// Launchers for the persistent tcgen05 GEMM (see gemm_core.cuh).
#include "gemm_core.cuh"
#include "tensormap.cuh"

namespace ob {
namespace gemm {

template <int A_MN, int B_MN, int SWIGLU>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmB2, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  gemm_cta<A_MN, B_MN, SWIGLU>(&tmA, &tmB, &tmB2, p, blockIdx.x, gridDim.x, smem_raw);
}

template <int A_MN, int B_MN, int SWIGLU>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const Params& p, int sms,
                  cudaStream_t stream) {
  auto kern = gemm_kernel<A_MN, B_MN, SWIGLU>;
  static bool configured = false;
  if (!configured) {
    OB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  const int tiles_m = (p.M + BM - 1) / BM;
  const int bn = SWIGLU ? BN / 2 : BN;
  const int tiles_n = (p.N + bn - 1) / bn;
  int grid = tiles_m * tiles_n;
  if (grid > sms) grid = sms;
  kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, tb2, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace gemm
}  // namespace ob

using namespace ob;
using namespace ob::gemm;

static int g_sm_count = 0;
static int sm_count() {
  if (!g_sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_sm_count;
}

// C[M,N] = epilogue(A * B^T).  a_mn / b_mn select the storage of the operands:
//   a_mn = 0: A is [M,K] row-major (lda >= K);  a_mn = 1: A is [K,M] row-major (lda >= M)
//   b_mn = 0: B is [N,K] row-major (ldb >= K);  b_mn = 1: B is [K,N] row-major (ldb >= N)
// Returns 0 on success, a negative code for unsupported arguments, or a CUDA error code.
extern "C" int ob_gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* C,
                            long long ldc, int M, int N, int K, int out_fp32, int accumulate, const void* bias,
                            int act, float alpha, const int* b_flags, int flag_rows, int flag_value,
                            const int* a_flags, int a_flag_rows, int a_flag_value, int tile_order,
                            int first_tile_shift, int max_ctas, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap ta, tb;
  int rc;
  if (a_mn) rc = make_tmap_2d(&ta, A, K, M, lda, BK, 64, 2);
  else      rc = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2);
  if (rc) return rc;
  if (b_mn) rc = make_tmap_2d(&tb, B, K, N, ldb, BK, 64, 2);
  else      rc = make_tmap_2d(&tb, B, N, K, ldb, BN, BK, 2);
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.bias = bias; p.act = act; p.alpha = alpha; p.G = nullptr; p.U = nullptr;
  p.b_flags = b_flags; p.flag_rows = flag_rows > 0 ? flag_rows : 1; p.flag_value = flag_value;
  p.a_flags = a_flags; p.a_flag_rows = a_flag_rows > 0 ? a_flag_rows : 1; p.a_flag_value = a_flag_value;
  p.status = status; p.tile_order = tile_order; p.first_tile_shift = first_tile_shift;
  int sms = sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  if (!a_mn && !b_mn) return launch<0, 0, 0>(ta, tb, tb, p, sms, stream);
  if (!a_mn && b_mn) return launch<0, 1, 0>(ta, tb, tb, p, sms, stream);
  if (a_mn && !b_mn) return launch<1, 0, 0>(ta, tb, tb, p, sms, stream);
  return launch<1, 1, 0>(ta, tb, tb, p, sms, stream);
}

// H[M,N] = silu(X W1^T) * (X W2^T); optionally also writes G = X W1^T and U = X W2^T.
// X is [M,K], W1 and W2 are [N,K], all row-major bf16.
extern "C" int ob_gemm_swiglu_bf16(const void* X, long long ldx, const void* W1, const void* W2, long long ldw, void* H,
                                   void* G, void* U, long long ldh, int M, int N, int K, int* status,
                                   cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap ta, tb1, tb2;
  int rc = make_tmap_2d(&ta, X, M, K, ldx, BM, BK, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tb1, W1, N, K, ldw, BN / 2, BK, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tb2, W2, N, K, ldw, BN / 2, BK, 2);
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = H; p.ldc = ldh; p.G = G; p.U = U; p.alpha = 1.0f; p.status = status;
  p.flag_rows = 1; p.a_flag_rows = 1;
  return launch<0, 0, 1>(ta, tb1, tb2, p, sm_count(), stream);
}

// GEMM whose epilogue is the send half of a reduce-scatter.  Each rank computes its partial
// product P = A * B^T for all M rows; row r belongs to rank r / rows_per_rank and is stored from
// the accumulator straight into that rank's staging buffer dst_ptrs[owner] at
// [me][r % rows_per_rank][0..N) (staging layout [world][rows_per_rank][ldc], bf16).  Tiles run
// m-major starting at `first_tile_shift` m-tiles so that ranks send to different owners at the
// same time and their own rows come last.  After a barrier the owner sums its `world` slots
// (ob_rs_sum).  `addend` (optional, local bf16 [M, ldc]) is added to the product before sending.
extern "C" int ob_gemm_rs_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn,
                               const void* addend, const void* const* dst_ptrs, int world, int me, int rows_per_rank,
                               long long ldc, int M, int N, int K, int first_tile_shift, int* status,
                               cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world > 16 || rows_per_rank <= 0 || (long long)rows_per_rank * world < M) return -1;
  CUtensorMap ta, tb;
  int rc;
  if (a_mn) rc = make_tmap_2d(&ta, A, K, M, lda, BK, 64, 2);
  else      rc = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2);
  if (rc) return rc;
  if (b_mn) rc = make_tmap_2d(&tb, B, K, N, ldb, BK, 64, 2);
  else      rc = make_tmap_2d(&tb, B, N, K, ldb, BN, BK, 2);
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = const_cast<void*>(addend); p.accumulate = addend != nullptr; p.ldc = ldc;
  p.alpha = 1.0f; p.status = status;
  p.flag_rows = 1; p.a_flag_rows = 1; p.tile_order = 2; p.first_tile_shift = first_tile_shift;
  for (int i = 0; i < world; ++i) p.rs_dst[i] = const_cast<void*>(dst_ptrs[i]);
  p.rs_rows = rows_per_rank; p.rs_me = me;
  const int sms = sm_count();
  if (!a_mn && !b_mn) return launch<0, 0, 0>(ta, tb, tb, p, sms, stream);
  if (!a_mn && b_mn) return launch<0, 1, 0>(ta, tb, tb, p, sms, stream);
  if (a_mn && !b_mn) return launch<1, 0, 0>(ta, tb, tb, p, sms, stream);
  return launch<1, 1, 0>(ta, tb, tb, p, sms, stream);
}
