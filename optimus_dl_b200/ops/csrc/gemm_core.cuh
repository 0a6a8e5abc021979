// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[M,N] = epilogue( A[M,K] * B[N,K]^T )
//
// Operands arrive through TMA into 128-byte-swizzled shared-memory tiles, the
// product is accumulated by tcgen05.mma into TMEM (two 128x256 fp32 accumulators,
// so that the epilogue of tile i overlaps the main loop of tile i+1), and the
// epilogue reads TMEM with tcgen05.ld.
//
// Either operand may be "K-major" (reduction dimension contiguous in global
// memory: A stored [M,K], B stored [N,K]) or "MN-major" (A stored [K,M], B stored
// [K,N]).  With both forms available the forward (x W^T), input-gradient (dy W)
// and weight-gradient (dy^T x) products of a linear layer run without a transpose.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
// owner, warps 2..5 = epilogue (each owns the TMEM lane quarter warp_id % 4).
#pragma once
#include "common.cuh"

namespace ob {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;      // one 128-byte swizzle atom of bf16 along K
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int ACC_STAGES = 2;
constexpr int NUM_THREADS = 192;
constexpr int A_TILE_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_TILE_BYTES = BN * BK * 2;   // 32 KB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
// Reduce-scatter epilogue: each epilogue warp stages 32 rows x 64 bf16 columns (rows padded to 144 bytes,
// conflict-free for 16-byte accesses) so that peer stores leave as 128-byte row segments.
constexpr int RS_ROW_ELEMS = 72;
constexpr int RS_STAGE_BYTES = 4 * 32 * RS_ROW_ELEMS * 2;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + RS_STAGE_BYTES;
constexpr int GROUP_M = 16;

enum Act : int { kActNone = 0, kActGelu = 1, kActRelu2 = 2, kActSilu = 3, kActSwigluBwd = 4 };

struct Params {
  int M, N, K;
  void* C;               // output, row-major [M, ldc]
  long long ldc;
  int out_fp32;          // 0: bf16 output, 1: fp32 output
  int accumulate;        // 1: C += result (same dtype as output)
  const void* bias;      // optional [N] (bf16), added before the activation
  int act;               // Act
  float alpha;           // scale applied to the accumulator
  // SwiGLU mode (template flag): B tile = 128 rows of B (gate) followed by 128 rows
  // of B2 (up); outputs h = silu(g)*u to C (width N) and, when set, g and u.
  // With act == kActSwigluBwd (plain mode) the product is dh, the gradient of h = silu(g) * u: the epilogue reads
  // g and u at the output coordinates from G and U (row stride ldc), overwrites them with dg and du, and writes
  // nothing to C.
  void* G;
  void* U;
  // Optional readiness flags, one per group of `flag_rows` rows of the B operand
  // (K-major B only).  The producer waits until flags[row / flag_rows] >= flag_value
  // before it loads a B tile.  Used by kernels that land B in local memory from
  // peers while the product runs.
  const int* b_flags;
  int flag_rows;
  int flag_value;
  // Same for the A operand (rows of A), K-major A only.
  const int* a_flags;
  int a_flag_rows;
  int a_flag_value;
  int* status;           // error word (see StatusCode)
  int tile_order;        // 0: grouped-M raster, 1: flag-friendly order starting at first_n_tile
  int first_tile_shift;  // rotates the n-tile (or m-tile) order so locally owned chunks go first
  // Reduce-scatter push (bf16 output only): when rs_rows > 0 the output row `r` belongs to rank
  // r / rs_rows and is stored, straight from the epilogue, into that rank's staging buffer
  // rs_dst[owner] at slot `rs_me` (layout [world][rs_rows][ldc]) over NVLink peer stores.  The
  // owner adds the `world` slots afterwards (ob_rs_sum).  With `accumulate`, the local C[M,ldc]
  // is added to the product before it is sent.
  void* rs_dst[16];
  int rs_rows;
  int rs_me;
  // Cross-entropy statistics epilogue (own kernel instantiation): the product is a block of logits that is never
  // stored.  Per output row and 256-column tile the epilogue leaves max, sum exp(z - max), sum z and the largest
  // value as one float4 in ce_part[row * ce_tiles + tile_n], its column in ce_part_idx[row * ce_tiles + tile_n], and
  // the logit of the row's target (when the target lies in the tile) in ce_tgt[row].  z is the bf16-rounded logit after the optional
  // soft cap (ce_softcap: 0 none, 1 c tanh(x / c), 2 23 sigmoid((x + 5) / 7.5)).
  const long long* ce_targets;
  float* ce_part;
  int* ce_part_idx;
  float* ce_tgt;
  int ce_tiles;          // 256-column tiles per row = ceil(N / 256)
  int ce_vocab_offset;
  int ce_softcap;
  float ce_cap;
};

struct TileCoord {
  int m, n;
};

__device__ __forceinline__ TileCoord tile_coord(int tile, int tiles_m, int tiles_n, const Params& p) {
  TileCoord c;
  if (p.tile_order == 1) {
    // n-major order (all m-tiles of one n-tile before the next), rotated: tiles that
    // read rows already resident run first while the rest is still arriving.
    int n = tile / tiles_m;
    c.m = tile - n * tiles_m;
    c.n = (n + p.first_tile_shift) % tiles_n;
    return c;
  }
  if (p.tile_order == 2) {
    // m-major rotated order, for a gathered A operand.
    int m = tile / tiles_n;
    c.n = tile - m * tiles_n;
    c.m = (m + p.first_tile_shift) % tiles_m;
    return c;
  }
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, tiles_m - first_m);
  const int r = tile - g * per_group;
  c.m = first_m + (r % gm);
  c.n = r / gm;
  return c;
}

#ifndef OB_FLAG_WAIT_NS
#define OB_FLAG_WAIT_NS 2000000000ULL   // a flag that is not set within two seconds is reported, not waited for
#endif
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait for `*flag >= value`.  On expiry (or when another role of the CTA already gave up) returns false
// after raising the CTA's abort flag and recording kStatusFlagTimeout; the caller unwinds normally.
__device__ __forceinline__ bool wait_flag(const int* flag, int value, volatile int* abort_flag, int* status) {
  const unsigned long long t0 = global_ns();
  for (uint32_t it = 0;; ++it) {
    int v;
    // system scope: the flag (and the data it covers) may have been written by another GPU
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= value) return true;
    if ((it & 0x3f) == 0x3f) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > OB_FLAG_WAIT_NS) break;
      __nanosleep(64);
    }
  }
  *abort_flag = 1;
  if (status) atomicCAS(status, kStatusOk, kStatusFlagTimeout);
  return false;
}

__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case kActGelu: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
    case kActRelu2: { float r = fmaxf(x, 0.0f); return r * r; }
    case kActSilu: return x / (1.0f + __expf(-x));
    default: return x;
  }
}

// Epilogue of the fused "input gradient of the down projection + SwiGLU backward" product: the accumulator tile is
// dh; g and u are read at the output coordinates (thread = row, 32 columns = 64 bytes per step, the next step's
// reads in flight under the current step's arithmetic) and overwritten with
//   dg = dh u s(g) (1 + g (1 - s(g))),  du = dh g s(g),   s = logistic function.
// dh is rounded to bf16 first, as the two-kernel path (GEMM, then the elementwise kernel) does.
__device__ __forceinline__ void epilogue_swiglu_bwd(const Params& p, int m0, int n0, uint32_t t_row, int warp, int lane,
                                                    bool vec_ok) {
  const int row = m0 + (warp & 3) * 32 + lane;
  const bool row_ok = row < p.M;
  __nv_bfloat16* grow = reinterpret_cast<__nv_bfloat16*>(p.G) + (long long)(row_ok ? row : 0) * p.ldc + n0;
  __nv_bfloat16* urow = reinterpret_cast<__nv_bfloat16*>(p.U) + (long long)(row_ok ? row : 0) * p.ldc + n0;
  auto grads = [](float d, float g, float u, float& dg, float& du) {
    d = __bfloat162float(__float2bfloat16(d));
    const float sg = 1.0f / (1.0f + __expf(-g));
    dg = d * u * sg * (1.0f + g * (1.0f - sg));
    du = d * g * sg;
  };
  const bool fast = vec_ok && n0 + BN <= p.N;      // warp-uniform
  if (fast) {
    // full tile: the reads of g and u run DEPTH steps ahead of the arithmetic (L2 latency under the main loop's
    // operand traffic is a few thousand cycles, one step of arithmetic a few hundred)
    constexpr int DEPTH = 3, STEPS = BN / 32;
    uint4 gq[DEPTH][4], uq[DEPTH][4];
    auto fetch = [&](int step, int slot) {
      if (row_ok) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          gq[slot][q] = *reinterpret_cast<const uint4*>(grow + step * 32 + 8 * q);
          uq[slot][q] = *reinterpret_cast<const uint4*>(urow + step * 32 + 8 * q);
        }
      }
    };
#pragma unroll
    for (int s0 = 0; s0 < DEPTH; ++s0) fetch(s0, s0);
#pragma unroll
    for (int st = 0; st < STEPS; ++st) {
      const int slot = st % DEPTH, c = st * 32;
      uint32_t r[32];
      tmem_ld_32x32(t_row + c, r);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t gw[4] = {gq[slot][q].x, gq[slot][q].y, gq[slot][q].z, gq[slot][q].w};
          const uint32_t uw[4] = {uq[slot][q].x, uq[slot][q].y, uq[slot][q].z, uq[slot][q].w};
          uint32_t og[4], ou[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 g2 = unpack_bf16x2(gw[j]), u2 = unpack_bf16x2(uw[j]);
            float dg0, du0, dg1, du1;
            grads(__uint_as_float(r[8 * q + 2 * j]), g2.x, u2.x, dg0, du0);
            grads(__uint_as_float(r[8 * q + 2 * j + 1]), g2.y, u2.y, dg1, du1);
            og[j] = pack_bf16x2(dg0, dg1);
            ou[j] = pack_bf16x2(du0, du1);
          }
          *reinterpret_cast<uint4*>(grow + c + 8 * q) = make_uint4(og[0], og[1], og[2], og[3]);
          *reinterpret_cast<uint4*>(urow + c + 8 * q) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
        }
      }
      if (st + DEPTH < STEPS) fetch(st + DEPTH, slot);
    }
    return;
  }
#pragma unroll 1
  for (int c = 0; c < BN; c += 32) {
    if (n0 + c >= p.N) break;   // warp-uniform
    uint32_t r[32];
    tmem_ld_32x32(t_row + c, r);
    tmem_ld_wait();
    if (!row_ok) continue;
    for (int j = 0; j < 32; ++j) {
      if (n0 + c + j < p.N) {
        float dg, du;
        grads(__uint_as_float(r[j]), __bfloat162float(grow[c + j]), __bfloat162float(urow[c + j]), dg, du);
        grow[c + j] = __float2bfloat16(dg);
        urow[c + j] = __float2bfloat16(du);
      }
    }
  }
}

// Epilogue of the "linear layer + cross-entropy statistics" product (see Params::ce_part).  Thread = row; the 256
// columns of the tile go by in eight steps of 32 with a running (max, sum-exp) pair that is rescaled once per step.
__device__ __forceinline__ void epilogue_ce_stats(const Params& p, int m0, int n0, uint32_t t_row, int warp, int lane) {
  const int row = m0 + (warp & 3) * 32 + lane;
  const bool row_ok = row < p.M;
  long long y = -1;
  if (row_ok) y = p.ce_targets[row] - p.ce_vocab_offset;        // outside [0, N): not in this slice (or ignored)
  float m = -INFINITY, s = 0.f, sum = 0.f, best = -INFINITY, tgt = 0.f;
  int best_idx = 0x7fffffff;
  bool has_tgt = false;
  auto capf = [&](float x) {
    x = __bfloat162float(__float2bfloat16(x));
    if (p.ce_softcap == 1) return p.ce_cap * tanhf(x / p.ce_cap);
    if (p.ce_softcap == 2) return 23.0f / (1.0f + __expf(-(x + 5.0f) / 7.5f));
    return x;
  };
  auto step = [&](const uint32_t* r, int c) {
    const int col = n0 + c;
    const int ncols = min(32, p.N - col);    // warp-uniform
    float z[32];
    float cm = -INFINITY;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      z[j] = j < ncols ? capf(__uint_as_float(r[j])) : -INFINITY;
      cm = fmaxf(cm, z[j]);
    }
    if (cm > m) { s *= __expf(m - cm); m = cm; }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      s += __expf(z[j] - m);                 // -inf for the columns past N: adds 0
      sum += j < ncols ? z[j] : 0.f;
      if (z[j] > best) { best = z[j]; best_idx = col + j; }
      if ((long long)(col + j) == y) { tgt = z[j]; has_tgt = true; }
    }
  };
  // two register buffers: the TMEM read of the next 32 columns is in flight while the current ones are reduced (a
  // read waits behind the accumulator traffic of the running MMAs for a few thousand cycles)
  uint32_t ra[32], rb[32];
  tmem_ld_32x32(t_row, ra);
  tmem_ld_wait32(ra);
#pragma unroll 1
  for (int c = 0; c < BN; c += 64) {
    const bool has_b = n0 + c + 32 < p.N;                 // all warp-uniform
    const bool has_next = c + 64 < BN && n0 + c + 64 < p.N;
    if (has_b) tmem_ld_32x32(t_row + c + 32, rb);
    step(ra, c);
    if (!has_b) break;
    tmem_ld_wait32(rb);
    if (has_next) tmem_ld_32x32(t_row + c + 64, ra);
    step(rb, c + 32);
    if (!has_next) break;
    tmem_ld_wait32(ra);
  }
  if (row_ok) {
    const long long slot = (long long)row * p.ce_tiles + n0 / BN;
    reinterpret_cast<float4*>(p.ce_part)[slot] = make_float4(m, s, sum, best);
    p.ce_part_idx[slot] = best_idx;
    if (has_tgt) p.ce_tgt[row] = tgt;
  }
}

// Epilogue of one 128 x 256 accumulator tile, executed by one epilogue warp for its 32 TMEM lanes:
// `t_row` is the TMEM address of the warp's first lane at the tile's first column, (m0, n0) the tile origin in C.
template <int SWIGLU>
__device__ __forceinline__ void epilogue_tile(const Params& p, int m0, int n0, uint32_t t_row, int warp, int lane,
                                              bool vec_ok, __nv_bfloat16* rs_stage_base) {
  const int quarter = warp & 3;
  const int row = m0 + quarter * 32 + lane;
  if (SWIGLU == 1) {
    // columns [0,128) hold the gate product, [128,256) the up product
#pragma unroll 1
    for (int c = 0; c < 128; c += 32) {
      uint32_t g[32], u[32];
      tmem_ld_32x32(t_row + c, g);
      tmem_ld_32x32(t_row + 128 + c, u);
      tmem_ld_wait();
      if (row < p.M) {
        const int col = n0 + c;
        __nv_bfloat16* hrow = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col;
        __nv_bfloat16* grow = p.G ? reinterpret_cast<__nv_bfloat16*>(p.G) + (long long)row * p.ldc + col : nullptr;
        __nv_bfloat16* urow = p.U ? reinterpret_cast<__nv_bfloat16*>(p.U) + (long long)row * p.ldc + col : nullptr;
        if (vec_ok && col + 32 <= p.N) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t hp[4], gp[4], up[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              // round the gate and up products to bf16 first, as the unfused path does
              float g0 = __bfloat162float(__float2bfloat16(__uint_as_float(g[v * 8 + 2 * j])));
              float g1 = __bfloat162float(__float2bfloat16(__uint_as_float(g[v * 8 + 2 * j + 1])));
              float u0 = __bfloat162float(__float2bfloat16(__uint_as_float(u[v * 8 + 2 * j])));
              float u1 = __bfloat162float(__float2bfloat16(__uint_as_float(u[v * 8 + 2 * j + 1])));
              gp[j] = pack_bf16x2(g0, g1);
              up[j] = pack_bf16x2(u0, u1);
              hp[j] = pack_bf16x2(g0 / (1.0f + __expf(-g0)) * u0, g1 / (1.0f + __expf(-g1)) * u1);
            }
            *reinterpret_cast<uint4*>(hrow + v * 8) = make_uint4(hp[0], hp[1], hp[2], hp[3]);
            if (grow) *reinterpret_cast<uint4*>(grow + v * 8) = make_uint4(gp[0], gp[1], gp[2], gp[3]);
            if (urow) *reinterpret_cast<uint4*>(urow + v * 8) = make_uint4(up[0], up[1], up[2], up[3]);
          }
        } else {
          for (int j = 0; j < 32; ++j) {
            if (col + j < p.N) {
              float g0 = __bfloat162float(__float2bfloat16(__uint_as_float(g[j])));
              float u0 = __bfloat162float(__float2bfloat16(__uint_as_float(u[j])));
              hrow[j] = __float2bfloat16(g0 / (1.0f + __expf(-g0)) * u0);
              if (grow) grow[j] = __float2bfloat16(g0);
              if (urow) urow[j] = __float2bfloat16(u0);
            }
          }
        }
      }
    }
  } else {
    if (SWIGLU == 2) { epilogue_swiglu_bwd(p, m0, n0, t_row, warp, lane, vec_ok); return; }
    if (SWIGLU == 3) { epilogue_ce_stats(p, m0, n0, t_row, warp, lane); return; }
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      const int col = n0 + c;
      if (col >= p.N) break;   // warp-uniform
      uint32_t r[32];
      tmem_ld_32x32(t_row + c, r);
      tmem_ld_wait();
      if (row < p.M) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        if (p.bias) {
          const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col;
#pragma unroll
          for (int j = 0; j < 32; ++j) if (col + j < p.N) v[j] += __bfloat162float(b[j]);
        }
        if (p.act != kActNone) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], p.act);
        }
        if (p.out_fp32) {
          float* crow = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col;
          if ((p.ldc % 4 == 0) && col + 32 <= p.N && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0)) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 o = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
              if (p.accumulate) {
                float4 old = *reinterpret_cast<float4*>(crow + 4 * q);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(crow + 4 * q) = o;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col + j < p.N) crow[j] = p.accumulate ? crow[j] + v[j] : v[j];
          }
        } else {
          __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col;
          // with `accumulate` the addend is always read from the local C, also in reduce-scatter mode
          const __nv_bfloat16* srow = crow;
          if (p.rs_rows > 0) {
            // reduce-scatter mode: park the 32 columns in this warp's staging rows; the flush below
            // (outside the row guard, all lanes take part) sends them as 128-byte segments
            if (p.accumulate) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col + j < p.N) v[j] += __bfloat162float(srow[j]);
            }
            __nv_bfloat16* st = rs_stage_base + ((warp & 3) * 32 + lane) * RS_ROW_ELEMS + ((c >> 5) & 1) * 32;
#pragma unroll
            for (int q = 0; q < 4; ++q)
              *reinterpret_cast<uint4*>(st + 8 * q) =
                  make_uint4(pack_bf16x2(v[8 * q], v[8 * q + 1]), pack_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                             pack_bf16x2(v[8 * q + 4], v[8 * q + 5]), pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
          } else
          if (vec_ok && col + 32 <= p.N) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (p.accumulate) {
                uint4 old = *reinterpret_cast<const uint4*>(srow + 8 * q);
                float2 a0 = unpack_bf16x2(old.x), a1 = unpack_bf16x2(old.y), a2 = unpack_bf16x2(old.z),
                       a3 = unpack_bf16x2(old.w);
                v[8 * q] += a0.x; v[8 * q + 1] += a0.y; v[8 * q + 2] += a1.x; v[8 * q + 3] += a1.y;
                v[8 * q + 4] += a2.x; v[8 * q + 5] += a2.y; v[8 * q + 6] += a3.x; v[8 * q + 7] += a3.y;
              }
              uint4 o = make_uint4(pack_bf16x2(v[8 * q], v[8 * q + 1]), pack_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                                   pack_bf16x2(v[8 * q + 4], v[8 * q + 5]), pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
              *reinterpret_cast<uint4*>(crow + 8 * q) = o;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col + j < p.N)
                crow[j] = __float2bfloat16(p.accumulate ? __bfloat162float(srow[j]) + v[j] : v[j]);
          }
        }
      }
      if (p.rs_rows > 0 && (((c >> 5) & 1) == 1 || c + 32 >= BN || n0 + c + 32 >= p.N)) {
        __syncwarp();
        const __nv_bfloat16* stw = rs_stage_base + (warp & 3) * 32 * RS_ROW_ELEMS;
        const int seg = lane & 7;
        const int colg = n0 + (c & ~63) + seg * 8;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int rr = it * 4 + (lane >> 3);
          const int rowg = m0 + quarter * 32 + rr;
          if (rowg < p.M && colg < p.N && (colg < n0 + c + 32)) {
            const int owner = rowg / p.rs_rows;
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.rs_dst[owner]) +
                                 ((long long)p.rs_me * p.rs_rows + (rowg - owner * p.rs_rows)) * p.ldc + colg;
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(stw + rr * RS_ROW_ELEMS + seg * 8);
          }
        }
        __syncwarp();
      }
    }
  }
}

// One CTA's share of the persistent GEMM. `first_tile`/`tile_stride` give the static
// tile schedule (callers with extra non-GEMM CTAs pass the GEMM CTA index and count).
template <int A_MN, int B_MN, int SWIGLU>
__device__ __forceinline__ void gemm_cta(const CUtensorMap* tmA, const CUtensorMap* tmB, const CUtensorMap* tmB2,
                                         const Params& p, int first_tile, int tile_stride, uint8_t* smem_raw) {
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                          // [STAGES]
  uint64_t* empty_bar = bars + STAGES;                // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;             // [ACC_STAGES]
  uint64_t* acc_empty = bars + 2 * STAGES + ACC_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * ACC_STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __nv_bfloat16* rs_stage_base = reinterpret_cast<__nv_bfloat16*>(smem + STAGES * STAGE_BYTES + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + (SWIGLU ? BN / 2 : BN) - 1) / (SWIGLU ? BN / 2 : BN);
  const int num_tiles = tiles_m * tiles_n;
  const int k_tiles = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < ACC_STAGES; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
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
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(tmA);
      tma_prefetch_desc(tmB);
      if (SWIGLU) tma_prefetch_desc(tmB2);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_stride) {
        TileCoord tc = tile_coord(tile, tiles_m, tiles_n, p);
        const int m0 = tc.m * BM;
        const int n0 = tc.n * (SWIGLU ? BN / 2 : BN);
        if (p.b_flags) {
          const int f0 = n0 / p.flag_rows;
          const int f1 = (min(n0 + (SWIGLU ? BN / 2 : BN), p.N) - 1) / p.flag_rows;
          for (int f = f0; f <= f1 && ok; ++f) ok = wait_flag(p.b_flags + f, p.flag_value, abort_flag, p.status);
        }
        if (p.a_flags) {
          const int f0 = m0 / p.a_flag_rows;
          const int f1 = (min(m0 + BM, p.M) - 1) / p.a_flag_rows;
          for (int f = f0; f <= f1 && ok; ++f) ok = wait_flag(p.a_flags + f, p.a_flag_value, abort_flag, p.status);
        }
        if (p.b_flags || p.a_flags) asm volatile("fence.proxy.async.global;" ::: "memory");
        for (int kt = 0; kt < k_tiles && ok; ++kt) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status);
          if (!ok) break;
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_TILE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
          const int k0 = kt * BK;
          if (A_MN) {
            // global A is [K, M]: boxes of 64 (m) x 64 (k), one per 64 columns of the tile
            tma_load_2d(sA, tmA, &full_bar[stage], m0, k0);
            tma_load_2d(sA + 8192, tmA, &full_bar[stage], m0 + 64, k0);
          } else {
            tma_load_2d(sA, tmA, &full_bar[stage], k0, m0);
          }
          if (SWIGLU) {
            tma_load_2d(sB, tmB, &full_bar[stage], k0, n0);
            tma_load_2d(sB + B_TILE_BYTES / 2, tmB2, &full_bar[stage], k0, n0);
          } else if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sB + c * 8192, tmB, &full_bar[stage], n0 + c * 64, k0);
          } else {
            tma_load_2d(sB, tmB, &full_bar[stage], k0, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // Drain: wait (bounded) until every stage this thread filled has been consumed, so
      // that no copy is still in flight towards this CTA's shared memory at exit.
      for (int s = 0; s < STAGES; ++s) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status)) break;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_stride) {
        ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kt = 0; kt < k_tiles; ++kt) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sB = sA + A_TILE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // K-major: step 32 bytes inside the swizzle atom; MN-major: step 16 k-rows of 128 bytes.
            const uint64_t da = A_MN ? make_smem_desc_sw128(sA + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sA + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(sB + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sB + kk * 32, 16, 1024);
            umma_f16_ss(d_tmem, da, db, idesc, (kt | kk) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);   // frees this smem stage once the MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&acc_full[acc]);        // accumulator complete
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;            // TMEM lanes [32*quarter, 32*quarter+32)
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    const bool vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    for (int tile = first_tile; tile < num_tiles && ok; tile += tile_stride) {
      TileCoord tc = tile_coord(tile, tiles_m, tiles_n, p);
      const int m0 = tc.m * BM;
      const int n0 = tc.n * (SWIGLU ? BN / 2 : BN);
      ok = mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status);
      if (!ok) break;
      tc_fence_after();
      epilogue_tile<SWIGLU>(p, m0, n0, tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN, warp, lane, vec_ok,
                            rs_stage_base);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace gemm
}  // namespace ob
