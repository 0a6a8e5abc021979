// Block-scaled e4m3 GEMM for sm_100a and the quantisers that feed it.
//
//   C[M,N] (bf16) = sum over 128-wide k-blocks kb of
//                   sa[kb][m] * sb[n / 128][kb] * ( A8[m, kb] . B8[n, kb] )
//
// A8 [M,K] and B8 [N,K] hold e4m3 values, both with K contiguous.  sa holds one fp32 scale per
// (row, k-block) ("1 x 128" activation scaling, stored k-block-major so that a warp reads
// consecutive rows), sb one scale per 128 x 128 block of B (weight scaling).
//
// Each k-block is one 128-byte swizzle atom of e4m3, i.e. four tcgen05.mma.kind::f8f6f4
// instructions of K = 32.  Because every k-block has its own scale, the tensor core never
// accumulates across k-blocks: the MMA warp writes each k-block's 128 x 256 partial product into one
// of two TMEM slots, and sixteen epilogue warps (four per TMEM lane quarter, 64 columns each) pull
// the partial out with tcgen05.ld, scale it and add it to fp32 accumulators held in registers while
// the tensor core already works on the next k-block in the other slot.  The drain is a chain of
// TMEM-load latencies per warp, so it is spread over many warps to keep it shorter than the MMAs.
//
// Warp roles (576 threads): warp 0 TMA producer, warp 1 MMA issuer / TMEM owner, warps 2..17 epilogue.
#include <cuda_fp8.h>

#include "common.cuh"
#include "tensormap.cuh"

namespace ob {
namespace fp8 {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;       // one scale block = one swizzle atom of 8-bit elements
constexpr int UMMA_K = 32;
constexpr int STAGES = 4;
constexpr int SLOTS = 2;
constexpr int EPI_WARPS = 16;     // four per TMEM lane quarter, 64 columns each
constexpr int NUM_THREADS = 64 + EPI_WARPS * 32;
constexpr int EPI_COLS = BN / (EPI_WARPS / 4);
constexpr int A_TILE_BYTES = BM * BK;
constexpr int B_TILE_BYTES = BN * BK;
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int GROUP_M = 16;

struct Params {
  int M, N, K;
  __nv_bfloat16* C;
  long long ldc;
  const float* sa;    // [K/128][sa_ld]
  long long sa_ld;    // >= M
  const float* sb;    // [ceil(N/128)][K/128]
  int* status;
};

__device__ __forceinline__ void tile_of(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + (r % gm);
  tn = r / gm;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* part_full = bars + 2 * STAGES;
  uint64_t* part_empty = bars + 2 * STAGES + SLOTS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * SLOTS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = p.K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < SLOTS; ++a) { mbar_init(&part_full[a], 1); mbar_init(&part_empty[a], EPI_WARPS); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_of(tile, tiles_m, tiles_n, tm, tn);
        for (int kb = 0; kb < k_blocks && ok; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status);
          if (!ok) break;
          uint8_t* sA = smem + stage * STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
          tma_load_2d(sA, &tmA, &full_bar[stage], kb * BK, tm * BM);
          tma_load_2d(sA + A_TILE_BYTES, &tmB, &full_bar[stage], kb * BK, tn * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      for (int s = 0; s < STAGES; ++s) {   // drain: nothing may still be in flight towards this CTA at exit
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status)) break;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_e4m3(BM, BN);
      int stage = 0; uint32_t phase = 0;
      int slot = 0; uint32_t slot_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < k_blocks && ok; ++kb) {
          ok = mbar_wait(&part_empty[slot], slot_phase ^ 1, abort_flag, p.status);
          if (!ok) break;
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + slot * BN;
          const uint32_t sA = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sB = sA + A_TILE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = make_smem_desc_sw128(sA + kk * 32, 16, 1024);
            const uint64_t db = make_smem_desc_sw128(sB + kk * 32, 16, 1024);
            umma_f8_ss(d_tmem, da, db, idesc, kk ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          umma_commit(&part_full[slot]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if (++slot == SLOTS) { slot = 0; slot_phase ^= 1; }
        }
      }
    }
  } else {
    const int e = warp - 2;                 // 0..EPI_WARPS-1
    const int quarter = warp & 3;           // TMEM lane quarter this warp may read
    const int chunk = e >> 2;               // which EPI_COLS columns of the 256-wide tile
    int slot = 0; uint32_t slot_phase = 0;
    bool ok = true;
    const int sb_ld = k_blocks;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_of(tile, tiles_m, tiles_n, tm, tn);
      const int row = tm * BM + quarter * 32 + lane;
      const int col0 = tn * BN + chunk * EPI_COLS;
      const bool row_ok = row < p.M;
      const bool cols_ok = col0 < p.N;
      const float* sa_row = p.sa + (row_ok ? row : 0);
      const float* sb_row = p.sb + (long long)(cols_ok ? col0 / 128 : 0) * sb_ld;
      float acc[EPI_COLS];
#pragma unroll
      for (int j = 0; j < EPI_COLS; ++j) acc[j] = 0.f;
      // scales are fetched two k-blocks ahead: their global-load latency must not sit between the barrier
      // and the first use
      float sa0 = sa_row[0], sb0 = sb_row[0];
      float sa1 = k_blocks > 1 ? sa_row[p.sa_ld] : 0.f, sb1 = k_blocks > 1 ? sb_row[1] : 0.f;
      for (int kb = 0; kb < k_blocks; ++kb) {
        const float s = sa0 * sb0;
        sa0 = sa1; sb0 = sb1;
        if (kb + 2 < k_blocks) { sa1 = sa_row[(long long)(kb + 2) * p.sa_ld]; sb1 = sb_row[kb + 2]; }
        ok = mbar_wait(&part_full[slot], slot_phase, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + slot * BN + chunk * EPI_COLS;
#pragma unroll
        for (int c = 0; c < EPI_COLS; c += 16) {
          uint32_t r[16];
          tmem_ld_32x16(t_row + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c + j] = fmaf(__uint_as_float(r[j]), s, acc[c + j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&part_empty[slot]);
        if (++slot == SLOTS) { slot = 0; slot_phase ^= 1; }
      }
      if (!ok) break;
      if (row_ok && cols_ok) {
        __nv_bfloat16* crow = p.C + (long long)row * p.ldc + col0;
        const bool vec = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) && col0 + EPI_COLS <= p.N;
        if (vec) {
#pragma unroll
          for (int q = 0; q < EPI_COLS / 8; ++q) {
            uint4 o = make_uint4(pack_bf16x2(acc[8 * q], acc[8 * q + 1]), pack_bf16x2(acc[8 * q + 2], acc[8 * q + 3]),
                                 pack_bf16x2(acc[8 * q + 4], acc[8 * q + 5]), pack_bf16x2(acc[8 * q + 6], acc[8 * q + 7]));
            *reinterpret_cast<uint4*>(crow + 8 * q) = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < EPI_COLS; ++j)
            if (col0 + j < p.N) crow[j] = __float2bfloat16(acc[j]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// Quantisers.  e4m3 has a largest finite value of 448; scale = amax / 448 (1 when the block is all
// zero), stored value = x / scale rounded to nearest-even with saturation.
constexpr float E4M3_MAX = 448.0f;

__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

// 1 x 128 blocks along the contiguous dimension of x [rows, cols]: 16 threads per block, 8 elements (one
// 16-byte load) per thread, block maximum by four shuffles inside the half-warp.
// q [rows, cols] e4m3; scales stored [cols/128][scale_ld].
__global__ void __launch_bounds__(256)
quant_rowwise_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                     float* __restrict__ scales, long long scale_ld, int rows, int cols) {
  const int vec_per_row = cols / 8;
  const long long total = (long long)rows * vec_per_row;   // a multiple of 16 (cols % 128 == 0)
  const long long stride = (long long)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  // the loop bound is uniform per warp (all 32 lanes take part in the shuffles); a half-warp past the end idles
  for (long long base = (long long)blockIdx.x * blockDim.x + (threadIdx.x - lane); base < total; base += stride) {
    const long long i = base + lane;
    const bool live = i < total;
    const int row = live ? (int)(i / vec_per_row) : 0;
    const int v = live ? (int)(i - (long long)row * vec_per_row) : 0;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (live) raw = *reinterpret_cast<const uint4*>(x + (long long)row * ldx + v * 8);
    const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y), c = unpack_bf16x2(raw.z), d = unpack_bf16x2(raw.w);
    float amax = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))),
                       fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(d.x), fabsf(d.y))));
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax > 0.f ? amax / E4M3_MAX : 1.0f;
    const float inv = 1.0f / scale;
    uint2 packed;
    packed.x = (uint32_t)to_e4m3(a.x * inv) | ((uint32_t)to_e4m3(a.y * inv) << 8) |
               ((uint32_t)to_e4m3(b.x * inv) << 16) | ((uint32_t)to_e4m3(b.y * inv) << 24);
    packed.y = (uint32_t)to_e4m3(c.x * inv) | ((uint32_t)to_e4m3(c.y * inv) << 8) |
               ((uint32_t)to_e4m3(d.x * inv) << 16) | ((uint32_t)to_e4m3(d.y * inv) << 24);
    if (live) {
      *reinterpret_cast<uint2*>(q + (long long)row * ldq + v * 8) = packed;
      if ((v & 15) == 0) scales[(long long)(v >> 4) * scale_ld + row] = scale;
    }
  }
}

// 128 x 128 blocks of w [rows, cols]: one CTA (256 threads) per block.  Writes q [rows, cols] and,
// when qt != nullptr, the transposed copy qt [cols, rows]; scales [rows/128][cols/128] and the
// transposed table scales_t [cols/128][rows/128].
__global__ void __launch_bounds__(256)
quant_block_kernel(const __nv_bfloat16* __restrict__ w, long long ldw, uint8_t* __restrict__ q, long long ldq,
                   uint8_t* __restrict__ qt, long long ldqt, float* __restrict__ scales, float* __restrict__ scales_t,
                   int rows, int cols) {
  __shared__ float s_red[8];
  __shared__ uint8_t tile[128][132];
  const int bc = blockIdx.x, br = blockIdx.y;
  const int r0 = br * 128, c0 = bc * 128;
  const int tid = threadIdx.x;
  // each thread handles half a row: 64 consecutive elements
  const int lr = tid >> 1, lc = (tid & 1) * 64;
  const int row = r0 + lr;
  float v[64];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 64; j += 8) {
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (row < rows && c0 + lc + j < cols) raw = *reinterpret_cast<const uint4*>(w + (long long)row * ldw + c0 + lc + j);
    const float2 f0 = unpack_bf16x2(raw.x), f1 = unpack_bf16x2(raw.y), f2 = unpack_bf16x2(raw.z), f3 = unpack_bf16x2(raw.w);
    v[j] = f0.x; v[j + 1] = f0.y; v[j + 2] = f1.x; v[j + 3] = f1.y;
    v[j + 4] = f2.x; v[j + 5] = f2.y; v[j + 6] = f3.x; v[j + 7] = f3.y;
#pragma unroll
    for (int e2 = 0; e2 < 8; ++e2) amax = fmaxf(amax, fabsf(v[j + e2]));
  }
  amax = warp_max(amax);
  if ((tid & 31) == 0) s_red[tid >> 5] = amax;
  __syncthreads();
  amax = s_red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, s_red[i]);
  const float scale = amax > 0.f ? amax / E4M3_MAX : 1.0f;
  const float inv = 1.0f / scale;
  if (tid == 0) {
    scales[(long long)br * gridDim.x + bc] = scale;
    if (scales_t) scales_t[(long long)bc * gridDim.y + br] = scale;
  }
  alignas(16) uint8_t out[64];
#pragma unroll
  for (int j = 0; j < 64; ++j) out[j] = to_e4m3(v[j] * inv);
  if (row < rows) {
#pragma unroll
    for (int j = 0; j < 64; j += 16)
      if (c0 + lc + j < cols) *reinterpret_cast<uint4*>(q + (long long)row * ldq + c0 + lc + j) = *reinterpret_cast<uint4*>(out + j);
  }
  if (qt) {
#pragma unroll
    for (int j = 0; j < 64; ++j) tile[lr][lc + j] = out[j];
    __syncthreads();
    // transposed write: thread handles half a column of the block
    const int tc = tid >> 1, tr0 = (tid & 1) * 64;
    if (c0 + tc < cols) {
      alignas(16) uint8_t col[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) col[j] = tile[tr0 + j][tc];
#pragma unroll
      for (int j = 0; j < 64; j += 16)
        if (r0 + tr0 + j < rows)
          *reinterpret_cast<uint4*>(qt + (long long)(c0 + tc) * ldqt + r0 + tr0 + j) = *reinterpret_cast<uint4*>(col + j);
    }
  }
}

}  // namespace fp8
}  // namespace ob

using namespace ob;
using namespace ob::fp8;

// C[M,N] bf16 from e4m3 A8 [M,K], B8 [N,K] with scales sa [K/128][sa_ld], sb [ceil(N/128)][K/128].
// K must be a multiple of 128; lda/ldb multiples of 16 bytes.
extern "C" int ob_gemm_fp8_block(const void* A8, long long lda, const void* sa, long long sa_ld, const void* B8,
                                 long long ldb, const void* sb, void* C, long long ldc, int M, int N, int K,
                                 int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % BK != 0) return -1;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, A8, M, K, lda, BM, BK, 1);
  if (rc) return rc;
  rc = make_tmap_2d(&tb, B8, N, K, ldb, BN, BK, 1);
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = (__nv_bfloat16*)C; p.ldc = ldc; p.sa = (const float*)sa; p.sa_ld = sa_ld;
  p.sb = (const float*)sb; p.status = status;
  static bool configured = false;
  if (!configured) {
    OB_CUDA_CHECK(cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  if (grid > sms) grid = sms;
  gemm_fp8_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

// x [rows, cols] bf16 -> q e4m3 [rows, cols] (ldq), scales [cols/128][scale_ld].  cols % 128 == 0.
extern "C" int ob_quant_fp8_rowwise(const void* x, long long ldx, void* q, long long ldq, void* scales,
                                    long long scale_ld, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 128 != 0 || ldx % 8 != 0 || ldq % 8 != 0) return -1;
  const long long vecs = (long long)rows * (cols / 8);
  long long blocks = (vecs + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  quant_rowwise_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, (float*)scales,
                                                        scale_ld, rows, cols);
  return (int)cudaGetLastError();
}

// w [rows, cols] bf16 -> q [rows, cols], optional transposed qt [cols, rows], scales [ceil(rows/128)][ceil(cols/128)],
// optional scales_t (transposed table).  cols % 16 == 0 and rows % 16 == 0.
extern "C" int ob_quant_fp8_block(const void* w, long long ldw, void* q, long long ldq, void* qt, long long ldqt,
                                  void* scales, void* scales_t, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 16 != 0 || rows % 16 != 0 || ldw % 8 != 0 || ldq % 16 != 0 || (qt && ldqt % 16 != 0)) return -1;
  dim3 grid((cols + 127) / 128, (rows + 127) / 128);
  quant_block_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)w, ldw, (uint8_t*)q, ldq, (uint8_t*)qt, ldqt,
                                               (float*)scales, (float*)scales_t, rows, cols);
  return (int)cudaGetLastError();
}
