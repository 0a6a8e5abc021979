// e4m3 GEMMs for sm_100a (block-scaled and per-tensor-scaled), their quantisers, and the tensor-parallel forms that
// fuse the GEMM with its collective.  Contents:
//   gemm_fp8_kernel<PER_TENSOR>      the GEMM itself (description below; PER_TENSOR accumulates all of K in TMEM)
//   gemm_fp8_ag_kernel               quantise + e4m3 all-gather (peer stores, flags) + GEMM in one launch
//   gemm_fp8_rs_kernel               GEMM whose epilogue sends bf16 partial tiles to the owner rank (reduce-scatter)
//   quant_rowwise / quant_block      1 x 128 and 128 x 128 block quantisers
//   amax_scale / quant_tensor / quant_tensor_t / delayed_update   per-tensor scaling (current and delayed)
//
// Block-scaled product:
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

#include "comm.cuh"
#include "common.cuh"
#include "gemm_core.cuh"
#include "tensormap.cuh"

namespace ob {
namespace fp8 {

using gemm::wait_flag;

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
  int accumulate;     // C += product (C is read in the epilogue)
  // Gathered-A mode: rows of A8 (and their scales) are being written by other CTAs / other GPUs during this
  // launch; a_flags[m / 128] >= a_flag_value publishes a 128-row group.  Tiles then run m-major, starting at
  // m-tile first_m_tile (the rows that arrive first).
  const int* a_flags;
  int a_flag_value;
  int first_m_tile;
  int m_major;        // tiles run m-major starting at first_m_tile (gathered-A and reduce-scatter modes)
  // Reduce-scatter mode (rs_rows > 0, a multiple of 128): the bf16 tile goes to rank (row / rs_rows)'s staging
  // buffer, slot rs_me, instead of C: rs_dst[owner] + (rs_me * rs_rows + row % rs_rows) * ldc + col.
  void* rs_dst[comm::MAX_RANKS];
  int rs_rows;
  int rs_me;
};

constexpr int RS_STAGE_PER_WARP = 2048;   // 32 rows x 64 bytes, staged per epilogue warp
constexpr int SMEM_RS_BYTES = SMEM_BYTES + EPI_WARPS * RS_STAGE_PER_WARP;

__device__ __forceinline__ void tile_of(const Params& p, int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  if (p.m_major) {   // m-major, rotated so that the rows that are ready (or wanted) first come first
    tm = (tile / tiles_n + p.first_m_tile) % tiles_m;
    tn = tile % tiles_n;
    return;
  }
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + (r % gm);
  tn = r / gm;
}

// PER_TENSOR = false: block-scaled product (each 128-wide k-block is drained from TMEM and scaled in registers).
// PER_TENSOR = true: one scale per operand (p.sa[0] * p.sb[0]); the tensor core accumulates over all of K in
// TMEM and the epilogue drains each tile once, so the main loop runs at the plain e4m3 rate.
template <bool PER_TENSOR, bool RS = false>
__device__ __forceinline__ void fp8_cta(const CUtensorMap* tmA_p, const CUtensorMap* tmB_p, const Params& p,
                                        const int cta, const int n_ctas, uint8_t* smem_raw) {
  const CUtensorMap& tmA = *tmA_p;
  const CUtensorMap& tmB = *tmB_p;
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
      for (int tile = cta; tile < num_tiles && ok; tile += n_ctas) {
        int tm, tn;
        tile_of(p, tile, tiles_m, tiles_n, tm, tn);
        if (p.a_flags) {
          ok = wait_flag(p.a_flags + tm, p.a_flag_value, abort_flag, p.status);
          if (!ok) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");   // rows written by plain stores, read by TMA
        }
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
      for (int tile = cta; tile < num_tiles && ok; tile += n_ctas) {
        if (PER_TENSOR) ok = mbar_wait(&part_empty[slot], slot_phase ^ 1, abort_flag, p.status);
        for (int kb = 0; kb < k_blocks && ok; ++kb) {
          if (!PER_TENSOR) ok = mbar_wait(&part_empty[slot], slot_phase ^ 1, abort_flag, p.status);
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
            umma_f8_ss(d_tmem, da, db, idesc, (kk != 0 || (PER_TENSOR && kb != 0)) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if (!PER_TENSOR || kb == k_blocks - 1) {
            umma_commit(&part_full[slot]);
            if (++slot == SLOTS) { slot = 0; slot_phase ^= 1; }
          }
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
    const int drains = PER_TENSOR ? 1 : k_blocks;
    const float tensor_scale = PER_TENSOR ? p.sa[0] * p.sb[0] : 0.f;
    for (int tile = cta; tile < num_tiles && ok; tile += n_ctas) {
      int tm, tn;
      tile_of(p, tile, tiles_m, tiles_n, tm, tn);
      const int row = tm * BM + quarter * 32 + lane;
      const int col0 = tn * BN + chunk * EPI_COLS;
      const bool row_ok = row < p.M;
      const bool cols_ok = col0 < p.N;
      const float* sa_row = p.sa + (row_ok && !PER_TENSOR ? row : 0);
      const float* sb_row = p.sb + (PER_TENSOR ? 0 : (long long)(cols_ok ? col0 / 128 : 0) * sb_ld);
      float acc[EPI_COLS];
#pragma unroll
      for (int j = 0; j < EPI_COLS; ++j) acc[j] = 0.f;
      if (!PER_TENSOR && p.a_flags) {
        // the row group's scales were written by the same remote stores as its values: acquire before reading
        int okf = 1;
        if (lane == 0) okf = wait_flag(p.a_flags + tm, p.a_flag_value, abort_flag, p.status) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, okf, 0) != 0;
        if (!ok) break;
      }
      // scales are fetched two k-blocks ahead: their global-load latency must not sit between the barrier
      // and the first use
      float sa0 = sa_row[0], sb0 = sb_row[0];
      float sa1 = drains > 1 ? sa_row[p.sa_ld] : 0.f, sb1 = drains > 1 ? sb_row[1] : 0.f;
      for (int kb = 0; kb < drains; ++kb) {
        const float s = PER_TENSOR ? tensor_scale : sa0 * sb0;
        sa0 = sa1; sb0 = sb1;
        if (kb + 2 < drains) { sa1 = sa_row[(long long)(kb + 2) * p.sa_ld]; sb1 = sb_row[kb + 2]; }
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
      if (RS) {
        // Each lane holds 64 columns of its own row.  Sending them as they are would make every 16-byte store
        // its own NVLink transaction, so the warp stages 32 columns at a time in shared memory (chunks swizzled
        // by row pair: conflict-free both ways) and sends 64-byte row segments, eight rows per instruction.
        uint8_t* stg = smem + STAGES * STAGE_BYTES + 256 + e * RS_STAGE_PER_WARP;
        const int tile_row0 = tm * BM;
        const int owner = tile_row0 / p.rs_rows;
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.rs_dst[owner]) +
                             ((long long)p.rs_me * p.rs_rows + (tile_row0 - owner * p.rs_rows)) * p.ldc;
#pragma unroll
        for (int h = 0; h < EPI_COLS / 32; ++h) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int j = 32 * h + 8 * q;
            const uint4 o = make_uint4(pack_bf16x2(acc[j], acc[j + 1]), pack_bf16x2(acc[j + 2], acc[j + 3]),
                                       pack_bf16x2(acc[j + 4], acc[j + 5]), pack_bf16x2(acc[j + 6], acc[j + 7]));
            *reinterpret_cast<uint4*>(stg + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) = o;
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int r = 8 * it + (lane >> 2), c = lane & 3;
            const uint4 v = *reinterpret_cast<const uint4*>(stg + r * 64 + ((c ^ ((r >> 1) & 3)) << 4));
            const int lrow = quarter * 32 + r;
            const int col = col0 + 32 * h + 8 * c;
            if (tile_row0 + lrow < p.M && col < p.N)
              *reinterpret_cast<uint4*>(dst + (long long)lrow * p.ldc + col) = v;
          }
          __syncwarp();
        }
      } else if (row_ok && cols_ok) {
        __nv_bfloat16* crow = p.C + (long long)row * p.ldc + col0;
        const bool vec = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) && col0 + EPI_COLS <= p.N;
        if (vec) {
#pragma unroll
          for (int q = 0; q < EPI_COLS / 8; ++q) {
            if (p.accumulate) {
              const uint4 old = *reinterpret_cast<const uint4*>(crow + 8 * q);
              const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y), o2 = unpack_bf16x2(old.z),
                           o3 = unpack_bf16x2(old.w);
              acc[8 * q] += o0.x; acc[8 * q + 1] += o0.y; acc[8 * q + 2] += o1.x; acc[8 * q + 3] += o1.y;
              acc[8 * q + 4] += o2.x; acc[8 * q + 5] += o2.y; acc[8 * q + 6] += o3.x; acc[8 * q + 7] += o3.y;
            }
            uint4 o = make_uint4(pack_bf16x2(acc[8 * q], acc[8 * q + 1]), pack_bf16x2(acc[8 * q + 2], acc[8 * q + 3]),
                                 pack_bf16x2(acc[8 * q + 4], acc[8 * q + 5]), pack_bf16x2(acc[8 * q + 6], acc[8 * q + 7]));
            *reinterpret_cast<uint4*>(crow + 8 * q) = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < EPI_COLS; ++j)
            if (col0 + j < p.N) crow[j] = __float2bfloat16(acc[j] + (p.accumulate ? __bfloat162float(crow[j]) : 0.f));
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

template <bool PER_TENSOR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  fp8_cta<PER_TENSOR>(&tmA, &tmB, p, blockIdx.x, gridDim.x, smem_raw);
}

// ---------------------------------------------------------------------------------------------
// Quantisers.  e4m3 has a largest finite value of 448; scale = amax / 448 (1 when the block is all
// zero), stored value = x / scale rounded to nearest-even with saturation.
constexpr float E4M3_MAX = 448.0f;

__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

// four values -> four e4m3 bytes (a in the low byte) with two paired conversions
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// Thread layout shared by the row-streaming quantisers: a 256-thread block covers 256 / tpr rows with tpr threads
// each (tpr = 16 .. 256, a power of two, chosen by the host from the row width), so no index needs a division.
struct RowTiling {
  int tpr_log2;   // log2(threads per row)
};

static RowTiling row_tiling(int vec_per_row) {
  int l = 4;                                  // at least one 16-lane group per row
  while (l < 8 && (1 << (l + 1)) <= vec_per_row) ++l;
  return RowTiling{l};
}

// 1 x 128 blocks along the contiguous dimension of x [rows, cols]: 16 threads per block, 8 elements (one
// 16-byte load) per thread, block maximum by four shuffles inside the half-warp.
// q [rows, cols] e4m3; scales stored [cols/128][scale_ld].
__global__ void __launch_bounds__(256)
quant_rowwise_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                     float* __restrict__ scales, long long scale_ld, int rows, int cols, RowTiling t) {
  const int vec_per_row = cols >> 3;          // a multiple of 16 (cols % 128 == 0)
  const int tpr = 1 << t.tpr_log2;
  const int tx = threadIdx.x & (tpr - 1), ty = threadIdx.x >> t.tpr_log2;
  const int rows_per_block = 256 >> t.tpr_log2;
  // loop bounds are uniform per warp (all 32 lanes take part in the shuffles); lanes past the end idle
  for (int row0 = blockIdx.x * rows_per_block; row0 < rows; row0 += gridDim.x * rows_per_block) {
    const int row = row0 + ty;
    const bool row_live = row < rows;
    const __nv_bfloat16* xr = x + (long long)(row_live ? row : 0) * ldx;
    uint8_t* qr = q + (long long)(row_live ? row : 0) * ldq;
    for (int v0 = 0; v0 < vec_per_row; v0 += tpr) {
      const int v = v0 + tx;
      const bool live = row_live && v < vec_per_row;
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (live) raw = *reinterpret_cast<const uint4*>(xr + v * 8);
      const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y), c = unpack_bf16x2(raw.z), d = unpack_bf16x2(raw.w);
      float amax = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))),
                         fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(d.x), fabsf(d.y))));
#pragma unroll
      for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float scale = amax > 0.f ? amax / E4M3_MAX : 1.0f;
      const float inv = 1.0f / scale;
      if (live) {
        uint2 packed;
        packed.x = e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
        packed.y = e4m3x4(c.x * inv, c.y * inv, d.x * inv, d.y * inv);
        *reinterpret_cast<uint2*>(qr + v * 8) = packed;
        if ((v & 15) == 0) scales[(long long)(v >> 4) * scale_ld + row] = scale;
      }
    }
  }
}

// 128 x 128 blocks of w [rows, cols]: one CTA (256 threads) per block.  Writes q [rows, cols] and,
// when qt != nullptr, the transposed copy qt [cols, rows]; scales [rows/128][cols/128] and the
// transposed table scales_t [cols/128][rows/128].  With tensor_scale != nullptr every block uses that one scale
// (per-tensor scaling) and no scale table is written; amax_rec then receives the tensor's |w| maximum (float
// bits, atomic maximum).
__global__ void __launch_bounds__(256)
quant_block_kernel(const __nv_bfloat16* __restrict__ w, long long ldw, uint8_t* __restrict__ q, long long ldq,
                   uint8_t* __restrict__ qt, long long ldqt, float* __restrict__ scales, float* __restrict__ scales_t,
                   int rows, int cols, const float* __restrict__ tensor_scale, unsigned* __restrict__ amax_rec) {
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
  const float scale = tensor_scale ? *tensor_scale : (amax > 0.f ? amax / E4M3_MAX : 1.0f);
  const float inv = 1.0f / scale;
  if (tid == 0 && amax_rec && amax > 0.f) atomicMax(amax_rec, __float_as_uint(amax));
  if (tid == 0 && scales) {
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


// ---------------------------------------------------------------------------------------------
// Per-tensor scaling: one fp32 scale for the whole tensor (current scaling: from this tensor's own maximum;
// delayed scaling: from a history of earlier maxima).

__device__ __forceinline__ float amax8(const uint4& raw) {
  const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y), c = unpack_bf16x2(raw.z), d = unpack_bf16x2(raw.w);
  return fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))),
               fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(d.x), fabsf(d.y))));
}

__device__ __forceinline__ float block_max_256(float v, float* s_red) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
  __syncthreads();
  float m = s_red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) m = fmaxf(m, s_red[i]);
  return m;
}

// |x| maximum of x [rows, cols] -> *scale_out = max / 448 * margin_mul (1 when the tensor is all zero).
// ws = {running maximum (float bits), ticket}; both are zero on entry and are left zero by the last block.
__global__ void __launch_bounds__(256)
amax_scale_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int rows, int cols, unsigned* __restrict__ ws,
                  float* __restrict__ scale_out, float margin_mul, RowTiling t) {
  __shared__ float s_red[8];
  const int vec_per_row = cols >> 3;
  const int tpr = 1 << t.tpr_log2;
  const int tx = threadIdx.x & (tpr - 1), ty = threadIdx.x >> t.tpr_log2;
  const int rows_per_block = 256 >> t.tpr_log2;
  float m = 0.f;
  for (int row = blockIdx.x * rows_per_block + ty; row < rows; row += gridDim.x * rows_per_block) {
    const __nv_bfloat16* xr = x + (long long)row * ldx;
    for (int v = tx; v < vec_per_row; v += tpr) m = fmaxf(m, amax8(*reinterpret_cast<const uint4*>(xr + v * 8)));
  }
  m = block_max_256(m, s_red);
  if (threadIdx.x == 0) {
    atomicMax(&ws[0], __float_as_uint(m));     // non-negative floats order like their bit patterns
    __threadfence();
    const unsigned ticket = atomicAdd(&ws[1], 1u);
    if (ticket == gridDim.x - 1) {
      __threadfence();
      const float amax = __uint_as_float(atomicExch(&ws[0], 0u));
      ws[1] = 0u;
      *scale_out = amax > 0.f ? amax / E4M3_MAX * margin_mul : 1.0f;
    }
  }
}

// q = e4m3(x / *scale); when amax_rec != nullptr the tensor's |x| maximum is also folded into *amax_rec
// (float bits, atomic maximum) for the delayed-scaling history.
__global__ void __launch_bounds__(256)
quant_tensor_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                    const float* __restrict__ scale, unsigned* __restrict__ amax_rec, int rows, int cols,
                    RowTiling t) {
  __shared__ float s_red[8];
  const int vec_per_row = cols >> 3;
  const int tpr = 1 << t.tpr_log2;
  const int tx = threadIdx.x & (tpr - 1), ty = threadIdx.x >> t.tpr_log2;
  const int rows_per_block = 256 >> t.tpr_log2;
  const float inv = 1.0f / *scale;
  float m = 0.f;
  for (int row = blockIdx.x * rows_per_block + ty; row < rows; row += gridDim.x * rows_per_block) {
    const __nv_bfloat16* xr = x + (long long)row * ldx;
    uint8_t* qr = q + (long long)row * ldq;
    for (int v = tx; v < vec_per_row; v += tpr) {
      const uint4 raw = *reinterpret_cast<const uint4*>(xr + v * 8);
      if (amax_rec) m = fmaxf(m, amax8(raw));
      const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y), c = unpack_bf16x2(raw.z), d = unpack_bf16x2(raw.w);
      uint2 packed;
      packed.x = e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
      packed.y = e4m3x4(c.x * inv, c.y * inv, d.x * inv, d.y * inv);
      *reinterpret_cast<uint2*>(qr + v * 8) = packed;
    }
  }
  if (amax_rec) {
    m = block_max_256(m, s_red);
    if (threadIdx.x == 0 && m > 0.f) atomicMax(amax_rec, __float_as_uint(m));
  }
}

// Per-tensor quantiser that also writes the transposed copy: q [rows, cols] and qt [cols, rows] from one read of
// x, with the given scale.  One CTA per 128 x 128 tile in two 64-row passes; a thread converts a 4 x 8 patch
// (four 16-byte loads), stores its four 8-byte rows of q, transposes the patch in registers (byte permutes)
// into eight 32-bit words (4 rows of one column each) and parks them in shared memory [col][row / 4]; after
// both passes every qt row of the tile leaves as one 128-byte segment.  rows % 16 == 0, cols % 8 == 0.

constexpr int QT_PITCH = 33;   // words per column row of the staging tile (32 + 1: column neighbours shift one bank)

__global__ void __launch_bounds__(256)
quant_tensor_t_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                      uint8_t* __restrict__ qt, long long ldqt, const float* __restrict__ scale,
                      unsigned* __restrict__ amax_rec, int rows, int cols) {
  __shared__ uint32_t tile[128 * QT_PITCH];
  __shared__ float s_red[8];
  const int tid = threadIdx.x;
  const int r0 = blockIdx.y * 128, c0 = blockIdx.x * 128;
  const float inv = 1.0f / *scale;
  const int ci = tid & 15;          // 8-column group
  const int rg = tid >> 4;          // 4-row group within a pass (0..15)
  const int col = c0 + ci * 8;
  const int sw = (ci >> 2) & 3;     // word swizzle: the four column groups that would share a bank take different words
  float amax = 0.f;
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int rgg = pass * 16 + rg;           // 4-row group within the tile (0..31)
    const int row = r0 + rgg * 4;
    uint32_t lo[4], hi[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      uint4 raw = make_uint4(0, 0, 0, 0);
      const bool ok = row + r < rows && col < cols;
      if (ok) raw = *reinterpret_cast<const uint4*>(x + (long long)(row + r) * ldx + col);
      const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y), c = unpack_bf16x2(raw.z), d = unpack_bf16x2(raw.w);
      if (amax_rec)
        amax = fmaxf(amax, fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))),
                                 fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(d.x), fabsf(d.y)))));
      lo[r] = e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
      hi[r] = e4m3x4(c.x * inv, c.y * inv, d.x * inv, d.y * inv);
      if (ok) *reinterpret_cast<uint2*>(q + (long long)(row + r) * ldq + col) = make_uint2(lo[r], hi[r]);
    }
    // 4 x 4 byte transposes: word k holds rows 0..3 of column k
    uint32_t w[8];
    {
      const uint32_t t0 = __byte_perm(lo[0], lo[1], 0x5140), t1 = __byte_perm(lo[2], lo[3], 0x5140);
      const uint32_t t2 = __byte_perm(lo[0], lo[1], 0x7362), t3 = __byte_perm(lo[2], lo[3], 0x7362);
      w[0] = __byte_perm(t0, t1, 0x5410); w[1] = __byte_perm(t0, t1, 0x7632);
      w[2] = __byte_perm(t2, t3, 0x5410); w[3] = __byte_perm(t2, t3, 0x7632);
      const uint32_t u0 = __byte_perm(hi[0], hi[1], 0x5140), u1 = __byte_perm(hi[2], hi[3], 0x5140);
      const uint32_t u2 = __byte_perm(hi[0], hi[1], 0x7362), u3 = __byte_perm(hi[2], hi[3], 0x7362);
      w[4] = __byte_perm(u0, u1, 0x5410); w[5] = __byte_perm(u0, u1, 0x7632);
      w[6] = __byte_perm(u2, u3, 0x5410); w[7] = __byte_perm(u2, u3, 0x7632);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) tile[(ci * 8 + k) * QT_PITCH + (rgg ^ sw)] = w[k];
  }
  __syncthreads();
  // transposed rows: 8 lanes x 16 bytes = the tile's 128 rows of one column
  const int l8 = tid & 7;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = (tid >> 3) + 32 * i;
    const int s = (c >> 5) & 3;
    const uint32_t* src = tile + c * QT_PITCH;
    const uint4 v = make_uint4(src[(4 * l8 + 0) ^ s], src[(4 * l8 + 1) ^ s], src[(4 * l8 + 2) ^ s], src[(4 * l8 + 3) ^ s]);
    if (c0 + c < cols && r0 + 16 * l8 < rows)
      *reinterpret_cast<uint4*>(qt + (long long)(c0 + c) * ldqt + r0 + 16 * l8) = v;
  }
  if (amax_rec) {
    amax = block_max_256(amax, s_red);
    if (tid == 0 && amax > 0.f) atomicMax(amax_rec, __float_as_uint(amax));
  }
}

// Delayed-scaling bookkeeping, one block per tensor.  state[i] = {scale, recorded maximum (float bits), hist[H]}:
// the recorded maximum moves into hist[pos], is cleared, and the scale becomes max(hist) / 448 * margin_mul
// (use_max) or the newest maximum / 448 * margin_mul; a tensor that recorded nothing keeps its scale.
__global__ void __launch_bounds__(128)
delayed_update_kernel(float* __restrict__ state, int H, int pos, float margin_mul, int use_max) {
  __shared__ float s_red[4];
  float* st = state + (long long)blockIdx.x * (2 + H);
  if (threadIdx.x == 0) {
    st[2 + pos] = __uint_as_float(reinterpret_cast<unsigned*>(st)[1]);
    reinterpret_cast<unsigned*>(st)[1] = 0u;
  }
  __syncthreads();
  float m = 0.f;
  if (use_max) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) m = fmaxf(m, st[2 + i]);
  } else if (threadIdx.x == 0) {
    m = st[2 + pos];
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    m = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
    if (m > 0.f) st[0] = m / E4M3_MAX * margin_mul;
  }
}

// ---------------------------------------------------------------------------------------------
// All-gather of a sequence-parallel activation fused with its quantisation and the FP8 GEMM that consumes it.
//
// Every rank holds `rows` rows of the bf16 activation.  The first n_copy CTAs of the launch quantise this rank's
// rows 128 at a time (1 x 128 scales, or one given scale in per-tensor mode), store the e4m3 values -- and in
// block mode the scales -- into EVERY rank's gathered operand (this rank's own included) with plain peer
// stores, and then release that row group's flag on each rank.  The remaining CTAs run the GEMM over the
// gathered operand, m-major from this rank's own rows, and acquire a row group's flag before its first TMA
// load.  NVLink carries one byte per element instead of two, and no separate quantiser launch is needed.
struct AgQuant {
  const __nv_bfloat16* x;   // this rank's rows [rows, K], row stride ldx
  long long ldx;
  int rows, K, me, world;
  comm::PeerPtrs a8;        // gathered e4m3 operand [world * rows, K] on every rank
  comm::PeerPtrs sa;        // scale table [K / 128][sa_ld] on every rank (block mode)
  long long sa_ld;
  comm::PeerPtrs flags;     // one int per 128 rows of the gathered operand, on every rank
  int epoch;
  const float* tensor_scale;   // per-tensor mode: the scale to use
  unsigned* amax_rec;          // per-tensor mode, optional: receives max|x| of this rank's rows
};

template <bool PER_TENSOR>
__device__ __forceinline__ void quant_push(const AgQuant& a, int first, int stride, uint8_t* smem_raw) {
  float* s_scales = reinterpret_cast<float*>(smem_raw);   // [K / 128][128] (block mode)
  __shared__ float s_red[8];
  const int tid = threadIdx.x;
  const bool worker = tid < 512;            // 16 warps quantise; the rest of the block only joins the barriers
  const int kbs = a.K / 128;
  const int lane16 = tid & 15;
  const int blk = tid >> 4;                 // 0..31: which 1 x 128 block of the current group of 32
  const float inv_t = PER_TENSOR ? 1.0f / *a.tensor_scale : 0.f;
  float amax_all = 0.f;
  const int chunks = a.rows / 128;
  for (int ch = first; ch < chunks; ch += stride) {
    const int row0 = ch * 128;                       // within this rank's rows
    const long long grow0 = (long long)a.me * a.rows + row0;   // within the gathered operand
    const int n_blocks = 128 * kbs;
    if (worker) {
      constexpr int U = 8;   // loads in flight per thread: the copy CTAs are few, so each must keep many bytes moving
      for (int b0 = 0; b0 < n_blocks; b0 += 32 * U) {
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int b = b0 + 32 * u + blk;             // blocks run along K first: 32 of them are 8 KB of one row
          const int r = b / kbs, kb = b - r * kbs;
          raw[u] = make_uint4(0, 0, 0, 0);
          if (b < n_blocks)
            raw[u] = *reinterpret_cast<const uint4*>(a.x + (long long)(row0 + r) * a.ldx + kb * 128 + lane16 * 8);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int b = b0 + 32 * u + blk;
          const bool live = b < n_blocks;                // uniform per half-warp (a block is 16 lanes)
          const int r = live ? b / kbs : 0, kb = live ? b - r * kbs : 0;
          const float2 f0 = unpack_bf16x2(raw[u].x), f1 = unpack_bf16x2(raw[u].y), f2 = unpack_bf16x2(raw[u].z),
                       f3 = unpack_bf16x2(raw[u].w);
          float inv = inv_t;
          if (!PER_TENSOR || a.amax_rec) {
            float amax = fmaxf(fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f1.x), fabsf(f1.y))),
                               fmaxf(fmaxf(fabsf(f2.x), fabsf(f2.y)), fmaxf(fabsf(f3.x), fabsf(f3.y))));
            if (PER_TENSOR) {
              amax_all = fmaxf(amax_all, amax);
            } else {
#pragma unroll
              for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
              const float scale = amax > 0.f ? amax / E4M3_MAX : 1.0f;
              inv = 1.0f / scale;
              if (live && lane16 == 0) s_scales[kb * 128 + r] = scale;
            }
          }
          uint2 packed;
          packed.x = e4m3x4(f0.x * inv, f0.y * inv, f1.x * inv, f1.y * inv);
          packed.y = e4m3x4(f2.x * inv, f2.y * inv, f3.x * inv, f3.y * inv);
          const long long off = (grow0 + r) * (long long)a.K + kb * 128 + lane16 * 8;
          if (live)
            for (int pr = 0; pr < a.world; ++pr)
              *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(a.a8.p[pr]) + off) = packed;
        }
      }
    }
    if (!PER_TENSOR) {
      __syncthreads();
      // scale rows: 128 consecutive floats per k-block and rank
      if (worker) {
        for (int i = tid; i < kbs * 128; i += 512) {
          const int kb = i >> 7, r = i & 127;
          const float v = s_scales[i];
          for (int pr = 0; pr < a.world; ++pr)
            reinterpret_cast<float*>(a.sa.p[pr])[(long long)kb * a.sa_ld + grow0 + r] = v;
        }
      }
    }
    // all of this CTA's stores for the group are visible system-wide before the flags go out
    __threadfence_system();
    __syncthreads();
    if (tid < a.world) {
      int* f = reinterpret_cast<int*>(a.flags.p[tid]) + (int)(grow0 / 128);
      asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f), "r"(a.epoch) : "memory");
    }
    __syncthreads();   // s_scales is reused by the next group
  }
  if (PER_TENSOR && a.amax_rec) {
    amax_all = warp_max(amax_all);
    if (worker && (tid & 31) == 0 && amax_all > 0.f) atomicMax(a.amax_rec, __float_as_uint(amax_all));
  }
  (void)s_red;
}

template <bool PER_TENSOR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_rs_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p) {
  extern __shared__ uint8_t smem_raw[];   // SMEM_RS_BYTES: the ring plus the epilogue warps' staging
  fp8_cta<PER_TENSOR, true>(&tmA, &tmB, p, blockIdx.x, gridDim.x, smem_raw);
}

template <bool PER_TENSOR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_ag_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p,
                   const AgQuant a, const int n_copy) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x < n_copy) {
    quant_push<PER_TENSOR>(a, blockIdx.x, n_copy, smem_raw);
    return;
  }
  fp8_cta<PER_TENSOR>(&tmA, &tmB, p, blockIdx.x - n_copy, gridDim.x - n_copy, smem_raw);
}

}  // namespace fp8
}  // namespace ob

using namespace ob;
using namespace ob::fp8;

// C[M,N] bf16 from e4m3 A8 [M,K], B8 [N,K] with scales sa [K/128][sa_ld], sb [ceil(N/128)][K/128].
// K must be a multiple of 128; lda/ldb multiples of 16 bytes.
template <bool PER_TENSOR>
static int launch_fp8(const void* A8, long long lda, const void* sa, long long sa_ld, const void* B8, long long ldb,
                      const void* sb, void* C, long long ldc, int M, int N, int K, int accumulate, int* status,
                      cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % BK != 0) return -1;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, A8, M, K, lda, BM, BK, 1);
  if (rc) return rc;
  rc = make_tmap_2d(&tb, B8, N, K, ldb, BN, BK, 1);
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = (__nv_bfloat16*)C; p.ldc = ldc; p.sa = (const float*)sa; p.sa_ld = sa_ld;
  p.sb = (const float*)sb; p.status = status; p.accumulate = accumulate;
  static bool configured = false;
  if (!configured) {
    OB_CUDA_CHECK(cudaFuncSetAttribute(gemm_fp8_kernel<PER_TENSOR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       SMEM_BYTES));
    configured = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  if (grid > sms) grid = sms;
  gemm_fp8_kernel<PER_TENSOR><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

extern "C" int ob_gemm_fp8_block(const void* A8, long long lda, const void* sa, long long sa_ld, const void* B8,
                                 long long ldb, const void* sb, void* C, long long ldc, int M, int N, int K,
                                 int* status, cudaStream_t stream) {
  return launch_fp8<false>(A8, lda, sa, sa_ld, B8, ldb, sb, C, ldc, M, N, K, 0, status, stream);
}

// C[M,N] bf16 (+)= (*sa * *sb) * A8 [M,K] . B8 [N,K]^T with one device-resident fp32 scale per operand.
extern "C" int ob_gemm_fp8_tensor(const void* A8, long long lda, const void* sa, const void* B8, long long ldb,
                                  const void* sb, void* C, long long ldc, int M, int N, int K, int accumulate,
                                  int* status, cudaStream_t stream) {
  return launch_fp8<true>(A8, lda, sa, 0, B8, ldb, sb, C, ldc, M, N, K, accumulate, status, stream);
}

// Fused quantise + all-gather + FP8 GEMM (see gemm_fp8_ag_kernel).  x: this rank's bf16 rows [rows, K];
// a8_ptrs / sa_ptrs / flag_ptrs: every rank's gathered operand, scale table and flag words (index `me` = local);
// C [world * rows, N] = gathered(x) . B8^T.  per_tensor != 0: scales are *tensor_scale (the same value on every
// rank) and *sb; otherwise 1 x 128 scales travel with the rows and sb is the 128 x 128 table of B.
// rows % 128 == 0, K % 128 == 0.
extern "C" int ob_gemm_fp8_ag(const void* x, long long ldx, int rows, const void* const* a8_ptrs,
                              const void* const* sa_ptrs, long long sa_ld, const void* const* flag_ptrs, int world,
                              int me, int epoch, const void* B8, long long ldb, const void* sb, void* C, long long ldc,
                              int N, int K, int per_tensor, const void* tensor_scale, void* amax_rec, int n_copy,
                              int* status, cudaStream_t stream) {
  if (rows <= 0 || N <= 0 || K <= 0) return 0;
  // distinct codes per failed precondition: the caller reports the number
  if (rows % 128 != 0) return -11;
  if (K % BK != 0) return -12;
  if (ldx % 8 != 0) return -13;
  if (world < 1 || world > comm::MAX_RANKS || me < 0 || me >= world) return -14;
  if ((long long)K * 4 > (long long)STAGES * STAGE_BYTES) return -15;   // scale staging of one row group
  const int M = rows * world;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, a8_ptrs[me], M, K, K, BM, BK, 1);
  if (rc) return rc - 1000;
  rc = make_tmap_2d(&tb, B8, N, K, ldb, BN, BK, 1);
  if (rc) return rc - 2000;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = (__nv_bfloat16*)C; p.ldc = ldc;
  p.sa = per_tensor ? (const float*)tensor_scale : (const float*)sa_ptrs[me];
  p.sa_ld = sa_ld; p.sb = (const float*)sb; p.status = status; p.accumulate = 0;
  p.a_flags = (const int*)flag_ptrs[me]; p.a_flag_value = epoch; p.first_m_tile = (me * rows) / BM; p.m_major = 1;
  AgQuant a{};
  a.x = (const __nv_bfloat16*)x; a.ldx = ldx; a.rows = rows; a.K = K; a.me = me; a.world = world;
  for (int i = 0; i < world; ++i) {
    a.a8.p[i] = const_cast<void*>(a8_ptrs[i]);
    a.sa.p[i] = per_tensor ? nullptr : const_cast<void*>(sa_ptrs[i]);
    a.flags.p[i] = const_cast<void*>(flag_ptrs[i]);
  }
  a.sa_ld = sa_ld; a.epoch = epoch; a.tensor_scale = (const float*)tensor_scale; a.amax_rec = (unsigned*)amax_rec;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (n_copy < 1) n_copy = 1;
  if (n_copy > rows / 128) n_copy = rows / 128;
  if (n_copy > sms / 2) n_copy = sms / 2;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int gemm_ctas = sms - n_copy;
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  // every CTA of the launch must be resident at once (GEMM CTAs wait for copy CTAs): grid <= SM count, one CTA per SM
  if (per_tensor) {
    static bool configured = false;
    if (!configured) {
      OB_CUDA_CHECK(cudaFuncSetAttribute(gemm_fp8_ag_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
      configured = true;
    }
    gemm_fp8_ag_kernel<true><<<n_copy + gemm_ctas, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p, a, n_copy);
  } else {
    static bool configured = false;
    if (!configured) {
      OB_CUDA_CHECK(cudaFuncSetAttribute(gemm_fp8_ag_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
      configured = true;
    }
    gemm_fp8_ag_kernel<false><<<n_copy + gemm_ctas, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p, a, n_copy);
  }
  return (int)cudaGetLastError();
}

// Row-parallel FP8 GEMM whose epilogue is the send half of a reduce-scatter: the bf16 partial product
// A8 [M,K] . B8 [N,K]^T of this rank goes, tile by tile, into slot `me` of the owner rank's staging buffer
// (dst_ptrs[owner], [world][rows_per_rank][ldc]); a following ob_rs_sum adds the slots.  per_tensor selects
// the scale scheme as in ob_gemm_fp8_tensor / ob_gemm_fp8_block.  rows_per_rank % 128 == 0, N % 8 == 0.
extern "C" int ob_gemm_fp8_rs(const void* A8, long long lda, const void* sa, long long sa_ld, const void* B8,
                              long long ldb, const void* sb, const void* const* dst_ptrs, int world, int me,
                              int rows_per_rank, long long ldc, int M, int N, int K, int per_tensor,
                              int first_tile_shift, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % BK != 0 || rows_per_rank % BM != 0 || N % 8 != 0 || ldc % 8 != 0 || world < 1 || world > comm::MAX_RANKS ||
      M != rows_per_rank * world)
    return -1;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, A8, M, K, lda, BM, BK, 1);
  if (rc) return rc;
  rc = make_tmap_2d(&tb, B8, N, K, ldb, BN, BK, 1);
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = nullptr; p.ldc = ldc; p.sa = (const float*)sa; p.sa_ld = sa_ld;
  p.sb = (const float*)sb; p.status = status;
  p.m_major = 1; p.first_m_tile = first_tile_shift; p.rs_rows = rows_per_rank; p.rs_me = me;
  for (int i = 0; i < world; ++i) p.rs_dst[i] = const_cast<void*>(dst_ptrs[i]);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  if (grid > sms) grid = sms;
  if (per_tensor) {
    static bool configured = false;
    if (!configured) {
      OB_CUDA_CHECK(cudaFuncSetAttribute(gemm_fp8_rs_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_RS_BYTES));
      configured = true;
    }
    gemm_fp8_rs_kernel<true><<<grid, NUM_THREADS, SMEM_RS_BYTES, stream>>>(ta, tb, p);
  } else {
    static bool configured = false;
    if (!configured) {
      OB_CUDA_CHECK(cudaFuncSetAttribute(gemm_fp8_rs_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_RS_BYTES));
      configured = true;
    }
    gemm_fp8_rs_kernel<false><<<grid, NUM_THREADS, SMEM_RS_BYTES, stream>>>(ta, tb, p);
  }
  return (int)cudaGetLastError();
}

static int quant_grid(int rows, const RowTiling& t) {
  const int rows_per_block = 256 >> t.tpr_log2;
  long long blocks = ((long long)rows + rows_per_block - 1) / rows_per_block;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return (int)blocks;
}

// *scale_out = max|x| / 448 * margin_mul.  ws: two zeroed 32-bit words reused from call to call (per stream).
extern "C" int ob_fp8_amax_scale(const void* x, long long ldx, int rows, int cols, void* ws, void* scale_out,
                                 float margin_mul, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return -1;
  if (cols % 8 != 0 || ldx % 8 != 0) return -1;
  const RowTiling t = row_tiling(cols / 8);
  amax_scale_kernel<<<quant_grid(rows, t), 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, rows, cols, (unsigned*)ws,
                                                             (float*)scale_out, margin_mul, t);
  return (int)cudaGetLastError();
}

// q = e4m3(x / *scale); optional amax_rec (see quant_tensor_kernel).
extern "C" int ob_quant_fp8_tensor(const void* x, long long ldx, void* q, long long ldq, const void* scale,
                                   void* amax_rec, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 8 != 0 || ldx % 8 != 0 || ldq % 8 != 0) return -1;
  const RowTiling t = row_tiling(cols / 8);
  quant_tensor_kernel<<<quant_grid(rows, t), 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq,
                                                               (const float*)scale, (unsigned*)amax_rec, rows, cols, t);
  return (int)cudaGetLastError();
}

// q [rows, cols] and qt [cols, rows] = e4m3(x / *scale); optional amax_rec.  rows % 16 == 0, cols % 16 == 0.
extern "C" int ob_quant_fp8_tensor_t(const void* x, long long ldx, void* q, long long ldq, void* qt, long long ldqt,
                                     const void* scale, void* amax_rec, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 16 != 0 || rows % 16 != 0 || ldx % 8 != 0 || ldq % 8 != 0 || ldqt % 16 != 0) return -1;
  dim3 grid((cols + 127) / 128, (rows + 127) / 128);
  quant_tensor_t_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, (uint8_t*)qt, ldqt,
                                                  (const float*)scale, (unsigned*)amax_rec, rows, cols);
  return (int)cudaGetLastError();
}

// state [n][2 + H] fp32 (see delayed_update_kernel); pos in [0, H).
extern "C" int ob_fp8_delayed_update(void* state, int n, int H, int pos, float margin_mul, int use_max,
                                     cudaStream_t stream) {
  if (n <= 0) return 0;
  if (H <= 0 || pos < 0 || pos >= H) return -1;
  delayed_update_kernel<<<n, 128, 0, stream>>>((float*)state, H, pos, margin_mul, use_max);
  return (int)cudaGetLastError();
}

// x [rows, cols] bf16 -> q e4m3 [rows, cols] (ldq), scales [cols/128][scale_ld].  cols % 128 == 0.
extern "C" int ob_quant_fp8_rowwise(const void* x, long long ldx, void* q, long long ldq, void* scales,
                                    long long scale_ld, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 128 != 0 || ldx % 8 != 0 || ldq % 8 != 0) return -1;
  const RowTiling t = row_tiling(cols / 8);
  const int rows_per_block = 256 >> t.tpr_log2;
  long long blocks = ((long long)rows + rows_per_block - 1) / rows_per_block;
  if (blocks > 148 * 16) blocks = 148 * 16;
  quant_rowwise_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, (float*)scales,
                                                        scale_ld, rows, cols, t);
  return (int)cudaGetLastError();
}

// w [rows, cols] bf16 -> q [rows, cols], optional transposed qt [cols, rows], scales [ceil(rows/128)][ceil(cols/128)],
// optional scales_t (transposed table); or, with tensor_scale, one given scale and no tables.  cols % 16 == 0 and
// rows % 16 == 0.
extern "C" int ob_quant_fp8_block(const void* w, long long ldw, void* q, long long ldq, void* qt, long long ldqt,
                                  void* scales, void* scales_t, int rows, int cols, const void* tensor_scale,
                                  void* amax_rec, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 16 != 0 || rows % 16 != 0 || ldw % 8 != 0 || ldq % 16 != 0 || (qt && ldqt % 16 != 0)) return -1;
  dim3 grid((cols + 127) / 128, (rows + 127) / 128);
  quant_block_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)w, ldw, (uint8_t*)q, ldq, (uint8_t*)qt, ldqt,
                                               (float*)scales, (float*)scales_t, rows, cols,
                                               (const float*)tensor_scale, (unsigned*)amax_rec);
  return (int)cudaGetLastError();
}
