// Skinny GEMM for decode steps: out[M,N] = x[M,K] W[N,K]^T (+ bias) with M <= 64 rows.
//
// A handful of rows against a whole weight matrix is a weight-streaming problem: every byte of W is needed once
// and the arithmetic is negligible.  The roles are therefore swapped with respect to the training GEMM: a CTA
// takes 128 ROWS OF W as the M side of the tensor-core product (tcgen05.mma, M = 128) and the padded token rows
// (16 / 32 / 64) as its N side, so that one TMA-fed pipeline per SM streams W at memory speed and the small
// activation tile rides along.  The accumulator D[n, m] sits in TMEM with weight rows in lanes; the epilogue
// writes it transposed, which for a fixed token m is a contiguous run of n: coalesced.
// With few weight tiles the reduction dimension is split over the 2, 4 or 8 CTAs of a thread-block cluster: every
// CTA adds its fp32 accumulator into a buffer in the FIRST CTA's shared memory (`red.shared::cluster.add.f32` over
// distributed shared memory), the cluster meets at its hardware barrier, and the first CTA adds the bias and writes
// the bf16 result.  One launch, no global scratch.  All mbarrier waits are bounded as everywhere in this library.
#include "common.cuh"
#include "tensormap.cuh"

namespace ob {
namespace skinny {

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

constexpr int WM = 128;       // weight rows per CTA
constexpr int BK = 64;
constexpr int STAGES = 7;
constexpr int THREADS = 192;  // TMA warp, MMA warp, 4 epilogue warps
constexpr int W_BYTES = WM * BK * 2;

template <int MP>
struct Smem {
  static constexpr int X_BYTES = MP * BK * 2;
  static constexpr int STAGE = W_BYTES + (X_BYTES < 1024 ? 1024 : (X_BYTES + 1023) / 1024 * 1024);
  static constexpr int RED_OFF = STAGES * STAGE;           // [MP][128] fp32 sums (used in the cluster's first CTA)
  static constexpr int BAR_OFF = RED_OFF + MP * WM * 4;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

struct Params {
  int M, N, K;
  __nv_bfloat16* out; long long ldo;
  const __nv_bfloat16* bias;
  int splits;              // CTAs per cluster sharing the reduction dimension (1, 2, 4 or 8)
  int* status;
};

template <int MP>
__global__ void __launch_bounds__(THREADS, 1)
skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const Params p) {
  using L = Smem<MP>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / p.splits, split = blockIdx.x - tile * p.splits;
  const int n0 = tile * WM;
  const int k_tiles = (p.K + BK - 1) / BK;
  const int per = (k_tiles + p.splits - 1) / p.splits;
  const int kt0 = split * per, kt1 = min(k_tiles, kt0 + per);
  const int my_tiles = max(kt1 - kt0, 0);
  constexpr uint32_t TCOLS = MP < 32 ? 32 : MP;

  float* red = reinterpret_cast<float*>(smem + L::RED_OFF);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (p.splits > 1 && split == 0)
    for (int i = threadIdx.x; i < MP * WM; i += THREADS) red[i] = 0.f;
  if (warp == 1) { tmem_alloc(tmem_slot, TCOLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  if (p.splits > 1) cluster_sync_all();      // the first CTA's sums are zero before any peer adds to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmW);
      tma_prefetch_desc(&tmX);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int kt = kt0; kt < kt1 && ok; ++kt) {
        ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status);
        if (!ok) break;
        uint8_t* sW = smem + stage * L::STAGE;
        mbar_arrive_expect_tx(&full_bar[stage], W_BYTES + L::X_BYTES);
        tma_load_2d(sW, &tmW, &full_bar[stage], kt * BK, n0);
        tma_load_2d(sW + W_BYTES, &tmX, &full_bar[stage], kt * BK, 0);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      for (int s = 0; s < STAGES; ++s) {   // drain: no copy is still in flight towards this CTA at exit
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status)) break;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(WM, MP, 0, 0);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int kt = 0; kt < my_tiles && ok; ++kt) {
        ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sW = smem_u32(smem + stage * L::STAGE);
        const uint32_t sX = sW + W_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk)
          umma_f16_ss(tmem_base, make_smem_desc_sw128(sW + kk * 32, 16, 1024), make_smem_desc_sw128(sX + kk * 32, 16, 1024),
                      idesc, (kt | kk) ? 1u : 0u);
        umma_commit(&empty_bar[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    const int quarter = warp & 3;
    const int n = n0 + quarter * 32 + lane;                 // this thread's weight row = output column
    bool ok = my_tiles == 0 ? true : mbar_wait(acc_full, 0, abort_flag, p.status);
    if (ok) {
      tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16);
#pragma unroll
      for (int c = 0; c < MP; c += 16) {
        uint32_t r[16];
        if (my_tiles > 0) { tmem_ld_32x16(t_row + c, r); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = 0u;
        }
        if (p.splits > 1) {
          // add into the first CTA's buffer; rows past M and columns past N carry zeros (TMA fills them)
          const uint32_t local = smem_u32(red + quarter * 32 + lane);
          uint32_t remote;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0));
#pragma unroll
          for (int j = 0; j < 16; ++j)
            asm volatile("red.shared::cluster.add.f32 [%0], %1;" ::"r"(remote + (uint32_t)((c + j) * WM * 4)),
                         "f"(__uint_as_float(r[j]))
                         : "memory");
        } else if (n < p.N) {
          const float b = p.bias ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c + j < p.M) p.out[(long long)(c + j) * p.ldo + n] = __float2bfloat16(__uint_as_float(r[j]) + b);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (p.splits > 1) {
    cluster_sync_all();                        // every CTA's adds have landed
    if (split == 0 && warp >= 2) {
      const int n = n0 + (warp & 3) * 32 + lane;
      if (n < p.N) {
        const float b = p.bias ? __bfloat162float(p.bias[n]) : 0.f;
        for (int m = 0; m < p.M; ++m)
          p.out[(long long)m * p.ldo + n] = __float2bfloat16(red[m * WM + (warp & 3) * 32 + lane] + b);
      }
    }
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TCOLS); }
}


template <int MP>
static int launch(const CUtensorMap& tw, const CUtensorMap& tx, const Params& p, int tiles, cudaStream_t stream) {
  auto kern = skinny_kernel<MP>;
  static bool configured = false;
  if (!configured) {
    OB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<MP>::TOTAL));
    configured = true;
  }
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(tiles * p.splits); cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = Smem<MP>::TOTAL;
  cfg.stream = stream; cfg.attrs = attr; cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, tw, tx, p);
}

}  // namespace skinny
}  // namespace ob

using namespace ob;

// How many CTAs should share the reduction dimension of an [N, K] weight (so that about two waves of CTAs exist).
extern "C" int ob_gemm_skinny_splits(int N, int K) {
  const int tiles = (N + skinny::WM - 1) / skinny::WM;
  const int k_tiles = (K + skinny::BK - 1) / skinny::BK;
  int s = 148 / (tiles > 0 ? tiles : 1);     // about one wave of CTAs
  if (s > k_tiles / 4) s = k_tiles / 4;      // at least four k-tiles per CTA
  return s >= 8 ? 8 : (s >= 4 ? 4 : (s >= 2 ? 2 : 1));   // a portable cluster size
}

// x: [M, K] bf16 (ldx elements between rows), W: [N, K] bf16, out: [M, N] bf16.  M <= 64.
// splits: CTAs per cluster that share the reduction dimension (1, 2, 4 or 8; see ob_gemm_skinny_splits).
extern "C" int ob_gemm_skinny_bf16(const void* x, long long ldx, const void* W, long long ldw, void* out, long long ldo,
                                   int M, int N, int K, const void* bias, int splits, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 64) return -1;
  if (splits < 1) splits = 1;
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return -2;
  const int mp = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  CUtensorMap tw, tx;
  int rc = make_tmap_2d(&tw, W, N, K, ldw, skinny::WM, skinny::BK, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tx, x, M, K, ldx, mp, skinny::BK, 2);
  if (rc) return rc;
  skinny::Params p{M, N, K, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)bias, splits, status};
  const int tiles = (N + skinny::WM - 1) / skinny::WM;
  if (mp == 16) rc = skinny::launch<16>(tw, tx, p, tiles, stream);
  else if (mp == 32) rc = skinny::launch<32>(tw, tx, p, tiles, stream);
  else rc = skinny::launch<64>(tw, tx, p, tiles, stream);
  return rc;
}
