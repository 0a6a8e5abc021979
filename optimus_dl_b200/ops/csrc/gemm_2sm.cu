// Launchers of the two-SM persistent GEMM (gemm_2sm.cuh).
#include "gemm_2sm.cuh"
#include "tensormap.cuh"

namespace ob {
namespace gemm2 {

template <int A_MN, int B_MN, int SWIGLU>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
             const __grid_constant__ CUtensorMap tmB2, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  gemm2_cta<A_MN, B_MN, SWIGLU>(&tmA, &tmB, &tmB2, p, blockIdx.x >> 1, gridDim.x >> 1, smem_raw);
}

static int g_max_pairs[4][4] = {};

template <int A_MN, int B_MN, int SWIGLU>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const Params& p, int max_ctas,
                  cudaStream_t stream) {
  auto kern = gemm2_kernel<A_MN, B_MN, SWIGLU>;
  int& max_pairs = g_max_pairs[A_MN * 2 + B_MN][SWIGLU];
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(NUM_THREADS); cfg.dynamicSmemBytes = SMEM_BYTES; cfg.stream = stream;
  cfg.attrs = attr; cfg.numAttrs = 1;
  if (max_pairs == 0) {
    OB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cfg.gridDim = dim3(sms & ~1);
    int n = 0;
    OB_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
    if (n <= 0) return -4;
    max_pairs = n < sms / 2 ? n : sms / 2;
  }
  constexpr int bn = SWIGLU == 1 ? TN / 2 : TN;
  const int tiles = ((p.M + TM - 1) / TM) * ((p.N + bn - 1) / bn);
  int pairs = tiles < max_pairs ? tiles : max_pairs;
  if (max_ctas > 1 && pairs > max_ctas / 2) pairs = max_ctas / 2;
  cfg.gridDim = dim3(2 * pairs);
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, ta, tb, tb2, p));
}

}  // namespace gemm2
}  // namespace ob

using namespace ob;

// Same contract as ob_gemm_bf16 without the operand flags, tile orders and the reduce-scatter epilogue
// (callers that need those use the one-SM kernel).
extern "C" int ob_gemm2_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* C,
                             long long ldc, int M, int N, int K, int out_fp32, int accumulate, const void* bias, int act,
                             float alpha, int max_ctas, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap ta, tb;
  int rc;
  if (a_mn) rc = make_tmap_2d(&ta, A, K, M, lda, gemm2::BK, 64, 2);
  else      rc = make_tmap_2d(&ta, A, M, K, lda, 128, gemm2::BK, 2);
  if (rc) return rc;
  if (b_mn) rc = make_tmap_2d(&tb, B, K, N, ldb, gemm2::BK, 64, 2);
  else      rc = make_tmap_2d(&tb, B, N, K, ldb, 128, gemm2::BK, 2);
  if (rc) return rc;
  gemm::Params p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.bias = bias; p.act = act; p.alpha = alpha; p.status = status; p.flag_rows = 1; p.a_flag_rows = 1;
  if (!a_mn && !b_mn) return gemm2::launch<0, 0, 0>(ta, tb, tb, p, max_ctas, stream);
  if (!a_mn && b_mn) return gemm2::launch<0, 1, 0>(ta, tb, tb, p, max_ctas, stream);
  if (a_mn && !b_mn) return gemm2::launch<1, 0, 0>(ta, tb, tb, p, max_ctas, stream);
  return gemm2::launch<1, 1, 0>(ta, tb, tb, p, max_ctas, stream);
}

// H = silu(X W1^T) * (X W2^T) with the gate rows staged by the pair's first CTA and the up rows by the second.
extern "C" int ob_gemm2_swiglu_bf16(const void* X, long long ldx, const void* W1, const void* W2, long long ldw, void* H,
                                    void* G, void* U, long long ldh, int M, int N, int K, int* status,
                                    cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap ta, tb1, tb2;
  int rc = make_tmap_2d(&ta, X, M, K, ldx, 128, gemm2::BK, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tb1, W1, N, K, ldw, 128, gemm2::BK, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tb2, W2, N, K, ldw, 128, gemm2::BK, 2);
  if (rc) return rc;
  gemm::Params p{};
  p.M = M; p.N = N; p.K = K; p.C = H; p.ldc = ldh; p.G = G; p.U = U; p.alpha = 1.0f; p.status = status;
  p.flag_rows = 1; p.a_flag_rows = 1;
  return gemm2::launch<0, 0, 1>(ta, tb1, tb2, p, 0, stream);
}

// Input gradient of the SwiGLU feed-forward's down projection fused with the activation's backward:
// dh = DY[M, K] WC[K, N] (WC read MN-major) never reaches memory; the epilogue turns it, with g and u read at the
// output coordinates, into dg and du written over g and u (row stride ldg).
extern "C" int ob_gemm2_swiglu_bwd_bf16(const void* DY, long long lddy, const void* WC, long long ldw, void* G, void* U,
                                        long long ldg, int M, int N, int K, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, DY, M, K, lddy, 128, gemm2::BK, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tb, WC, K, N, ldw, gemm2::BK, 64, 2);
  if (rc) return rc;
  gemm::Params p{};
  p.M = M; p.N = N; p.K = K; p.C = nullptr; p.ldc = ldg; p.G = G; p.U = U; p.act = gemm::kActSwigluBwd; p.alpha = 1.0f;
  p.status = status; p.flag_rows = 1; p.a_flag_rows = 1;
  return gemm2::launch<0, 1, 2>(ta, tb, tb, p, 0, stream);
}

// Logits = X[M, K] W[N, K]^T reduced on the fly to per-row cross-entropy statistics (Params::ce_part): nothing of
// size M x N is written.  `part` holds M * tiles_n float4 (16-byte aligned), `part_idx` M * tiles_n ints (tiles_n =
// ceil(N / 256), see ob_gemm2_ce_tiles), `tgt_out` M floats that the caller zeroes first.  ob_ce_stats_merge folds
// the tiles.
extern "C" int ob_gemm2_ce_tiles(int N) { return (N + gemm2::TN - 1) / gemm2::TN; }
extern "C" int ob_gemm2_ce_stats_bf16(const void* X, long long ldx, const void* W, long long ldw, int M, int N, int K,
                                      const void* targets, void* part, void* part_idx, void* tgt_out, int vocab_offset,
                                      int softcap, float cap_c, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, X, M, K, ldx, 128, gemm2::BK, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tb, W, N, K, ldw, 128, gemm2::BK, 2);
  if (rc) return rc;
  gemm::Params p{};
  p.M = M; p.N = N; p.K = K; p.C = nullptr; p.ldc = 0; p.alpha = 1.0f; p.status = status; p.flag_rows = 1; p.a_flag_rows = 1;
  p.ce_targets = (const long long*)targets; p.ce_part = (float*)part; p.ce_part_idx = (int*)part_idx;
  p.ce_tgt = (float*)tgt_out; p.ce_tiles = (N + gemm2::TN - 1) / gemm2::TN; p.ce_vocab_offset = vocab_offset;
  p.ce_softcap = softcap; p.ce_cap = cap_c;
  return gemm2::launch<0, 0, 3>(ta, tb, tb, p, 0, stream);
}
