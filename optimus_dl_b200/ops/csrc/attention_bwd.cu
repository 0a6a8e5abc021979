// Flash-attention backward for sm_100a (same masking rule as attention_fwd.cu).
//
// Three launches:
//   delta kernel : delta[h, i] = sum_c dO[i,h,c] * O[i,h,c]
//   dQ kernel    : one CTA per (128-query tile, head); loops over key tiles:
//                    S = Q K^T, dP = dO V^T (tcgen05, operands in smem) -> TMEM
//                    dS = exp2(S*scale - lse) * (dP - delta)           (thread per query row)
//                    dQ += dS K   (dS from TMEM, K tile re-read as an MN-major operand)
//   dKV kernel   : one CTA per (128-key tile, kv head); loops over the query heads of the group
//                  and the query tiles that can see these keys, transposed problem:
//                    S^T = K Q^T, dP^T = V dO^T -> TMEM (thread per key row)
//                    dV += P^T dO, dK += dS^T Q  (P^T / dS^T from TMEM, dO / Q tiles MN-major)
// Recomputing S and dP in both kernels costs two extra products but needs no atomics: every
// output element is written by exactly one CTA in a fixed order (bitwise reproducible).
//
// Pipelining: every 128-wide tile is processed as two 64-wide halves with their own TMEM
// regions and barriers.  Two compute warpgroups (one per half) turn S/dP into P/dS while the
// MMA warp already issues the products of the other half and of the next tile, so the tensor
// pipe and the softmax arithmetic overlap.  The softmax scale is applied once in the epilogue
// (dQ and dK), not per score.
#include "common.cuh"
#include "tensormap.cuh"

namespace ob {
namespace attnb {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int HALF = 64;
constexpr int STAGES = 2;
constexpr uint32_t DESC_HI = smem_desc_hi_sw128(1024);   // every operand tile: 128-byte swizzle, 8-row groups of 1024 bytes
constexpr int THREADS = 384;      // 8 compute warps + TMA warp + MMA warp + 2 warps that only give up registers
constexpr float LOG2E = 1.4426950408889634f;

struct BwdParams {
  int N, Hq, Hk, window;
  float scale, scale_log2;
  const int* doc_start;
  const float* lse;        // [Hq, N]
  const float* delta;      // [Hq, N]
  __nv_bfloat16* dq; __nv_bfloat16* dk; __nv_bfloat16* dv;
  long long dqkv_stride;   // token stride of dq / dk / dv (elements)
  const int* kv_last_q;    // [key tiles] last query index that can attend a key of the tile
  int* status;
};

__global__ void delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                             long long out_stride, long long dout_stride, float* __restrict__ delta, int N, int Hq,
                             int hd) {
  const int lane = threadIdx.x & 31;
  const long long total = (long long)N * Hq;
  for (long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); item < total;
       item += (long long)gridDim.x * (blockDim.x >> 5)) {
    const int i = (int)(item / Hq), h = (int)(item % Hq);
    const __nv_bfloat16* o = out + i * out_stride + (long long)h * hd;
    const __nv_bfloat16* d = dout + i * dout_stride + (long long)h * hd;
    float s = 0.f;
    for (int c = lane * 2; c < hd; c += 64) {
      float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(o + c));
      float2 b = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(d + c));
      s += a.x * b.x + a.y * b.y;
    }
    s = warp_sum(s);
    if (lane == 0) delta[(long long)h * N + i] = s;
  }
}

// last query that may attend any key of tile t: largest i with max(doc_start[i], i-window+1) <= k_hi
__global__ void kv_last_q_kernel(const int* __restrict__ doc_start, int N, int window, int* __restrict__ out,
                                 int n_tiles) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tiles) return;
  const int k_hi = min(t * BN + BN - 1, N - 1);
  int lo = k_hi, hi = N - 1;   // the key itself is always attendable by query k_hi
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    int l = doc_start[mid];
    if (window > 0) l = max(l, mid - window + 1);
    if (l <= k_hi) lo = mid; else hi = mid - 1;
  }
  out[t] = lo;
}

__device__ __forceinline__ void store_row_bf16(__nv_bfloat16* drow, const uint32_t* o, float mul) {
#pragma unroll
  for (int v = 0; v < 4; ++v)
    *reinterpret_cast<uint4*>(drow + 8 * v) =
        make_uint4(pack_bf16x2(__uint_as_float(o[8 * v]) * mul, __uint_as_float(o[8 * v + 1]) * mul),
                   pack_bf16x2(__uint_as_float(o[8 * v + 2]) * mul, __uint_as_float(o[8 * v + 3]) * mul),
                   pack_bf16x2(__uint_as_float(o[8 * v + 4]) * mul, __uint_as_float(o[8 * v + 5]) * mul),
                   pack_bf16x2(__uint_as_float(o[8 * v + 6]) * mul, __uint_as_float(o[8 * v + 7]) * mul));
}

// ============================================================================ dQ kernel
// Measured on B200: one tcgen05.mma takes about 70 cycles when it extends the accumulation chain of the MMA before
// it, and never less than about 49, whatever its width; a 128-wide MMA needs 64 cycles of tensor time anyway, a
// 64-wide one only 32.  So every product here is 128 wide, and the two independent products of a tile (S and dP)
// are issued alternately, k-step by k-step, so that neither waits for its own previous step.
//
// Per key tile: S = Q K^T and dP = dO V^T land in TMEM; the two compute warpgroups (64 key columns each) pull
// their halves into registers and release the two regions at once, so the MMA warp issues the NEXT tile's S / dP
// while this tile's dS = P * (dP - delta) is still being computed; dS goes to its own TMEM columns and feeds
// dQ += dS K.  Q lives in TMEM as an A operand (each thread stores its own row once).
constexpr int DQ_STAGES = 3;

template <int HD>
struct SmemQ {
  static constexpr int TILE = BM * HD * 2;
  static constexpr int DO_OFF = 0, K_OFF = TILE, V_OFF = K_OFF + DQ_STAGES * TILE;
  static constexpr int BAR_OFF = V_OFF + DQ_STAGES * TILE;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

// TMEM columns: S [0,128) dP [128,256) dQ [256,256+HD) dS (bf16 pairs) [384,448) Q (bf16 pairs) [448,448+HD/2)
template <int HD>
__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const __grid_constant__ CUtensorMap tmDO, const __nv_bfloat16* __restrict__ qg, long long q_stride,
                   const BwdParams p) {
  using L = SmemQ<HD>;
  constexpr int SLABS = HD / 64;
  constexpr int SLAB_BYTES = BM * 128;
  constexpr int T_S = 0, T_DP = BN, T_DQ = 2 * BN, T_DS = 384, T_QA = 448;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* k_full = bars; uint64_t* k_empty = bars + DQ_STAGES;
  uint64_t* v_full = bars + 2 * DQ_STAGES; uint64_t* v_empty = bars + 3 * DQ_STAGES;
  uint64_t* misc = bars + 4 * DQ_STAGES;
  uint64_t* sdp_full = misc;          // S and dP of a tile are complete (one commit per tile)
  uint64_t* sdp_free = misc + 1;      // both warpgroups hold their halves in registers (8 warps)
  uint64_t* ds_ready = misc + 2;      // dS of a tile is in TMEM (8 warps)
  uint64_t* dq_done = misc + 3;       // the dQ product of a tile has read dS and K (one commit per tile)
  uint64_t* a_ready = misc + 4;       // Q rows are in TMEM (4 warps)
  uint64_t* do_full = misc + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qtiles = (p.N + BM - 1) / BM;
  const int h = blockIdx.x % p.Hq;
  const int qt = n_qtiles - 1 - blockIdx.x / p.Hq;
  const int kvh = h / (p.Hq / p.Hk);
  const int q_lo = qt * BM, q_hi = min(q_lo + BM - 1, p.N - 1);
  int lo_first = p.doc_start[q_lo], lo_last = p.doc_start[q_hi];
  if (p.window > 0) { lo_first = max(lo_first, q_lo - p.window + 1); lo_last = max(lo_last, q_hi - p.window + 1); }
  const int j_lo = lo_first / BN, j_hi = q_hi / BN;
  const int n_tiles = j_hi - j_lo + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < DQ_STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    mbar_init(sdp_full, 1); mbar_init(sdp_free, 8); mbar_init(ds_ready, 8); mbar_init(dq_done, 1);
    mbar_init(a_ready, 4); mbar_init(do_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // The third warpgroup (two single-thread roles and two idle warps) hands registers to the two compute
  // warpgroups, whose threads hold a whole row of a tile.
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
    if (warp == 8) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        mbar_arrive_expect_tx(do_full, L::TILE);
#pragma unroll
        for (int s = 0; s < SLABS; ++s) tma_load_2d(smem + L::DO_OFF + s * SLAB_BYTES, &tmDO, do_full, h * HD + s * 64, q_lo);
        bool ok = true;
        for (int t = 0; t < n_tiles && ok; ++t) {
          const int st = t % DQ_STAGES, j = j_lo + t;
          const uint32_t ph = (t / DQ_STAGES) & 1;
          ok = mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status);
          if (!ok) break;
          mbar_arrive_expect_tx(&k_full[st], L::TILE);
#pragma unroll
          for (int s = 0; s < SLABS; ++s)
            tma_load_2d(smem + L::K_OFF + st * L::TILE + s * SLAB_BYTES, &tmK, &k_full[st], kvh * HD + s * 64, j * BN);
          ok = mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status);
          if (!ok) break;
          mbar_arrive_expect_tx(&v_full[st], L::TILE);
#pragma unroll
          for (int s = 0; s < SLABS; ++s)
            tma_load_2d(smem + L::V_OFF + st * L::TILE + s * SLAB_BYTES, &tmV, &v_full[st], kvh * HD + s * 64, j * BN);
        }
      }
    } else if (warp == 9) {
      // ------------------------------------------------------------------ MMA issuer
      {   // all 32 lanes run the issue loop; the MMA and commit forms elect one lane
        constexpr uint32_t idesc_s = make_idesc_bf16(BM, BN, 0, 0);
        constexpr uint32_t idesc_dq = make_idesc_bf16(BM, HD, 0, 1);
        const uint32_t sDO = smem_u32(smem + L::DO_OFF);
        const uint32_t sK = smem_u32(smem + L::K_OFF), sV = smem_u32(smem + L::V_OFF);
        bool ok = mbar_wait(a_ready, 0, abort_flag, p.status);
        if (ok) ok = mbar_wait(do_full, 0, abort_flag, p.status);

        auto issue_sdp = [&](int t) -> bool {
          const int st = t % DQ_STAGES;
          const uint32_t ph = (t / DQ_STAGES) & 1;
          if (!mbar_wait(&k_full[st], ph, abort_flag, p.status)) return false;
          if (!mbar_wait(&v_full[st], ph, abort_flag, p.status)) return false;
          tc_fence_after();
          const uint32_t k_lo = smem_desc_lo(sK + st * L::TILE, 16), v_lo = smem_desc_lo(sV + st * L::TILE, 16);
          const uint32_t do_lo = smem_desc_lo(sDO, 16);
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t off = ((kk / 4) * SLAB_BYTES + (kk % 4) * 32) >> 4;
            umma_f16_ts_lh(tmem_base + T_S, tmem_base + T_QA + kk * 8, k_lo + off, DESC_HI, idesc_s, kk ? 1u : 0u);
            umma_f16_ss_lh(tmem_base + T_DP, do_lo + off, v_lo + off, DESC_HI, idesc_s, kk ? 1u : 0u);
          }
          umma_commit_elect(sdp_full);
          umma_commit_elect(&v_empty[st]);
          return true;
        };

        if (ok) ok = issue_sdp(0);
        for (int t = 0; t < n_tiles && ok; ++t) {
          const int st = t % DQ_STAGES;
          if (t + 1 < n_tiles) {
            ok = mbar_wait(sdp_free, t & 1, abort_flag, p.status);
            if (ok) ok = issue_sdp(t + 1);
            if (!ok) break;
          }
          ok = mbar_wait(ds_ready, t & 1, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t kt_lo = smem_desc_lo(sK + st * L::TILE, SLAB_BYTES);     // K read MN-major: 16 keys = 2048 bytes
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk)
            umma_f16_ts_lh(tmem_base + T_DQ, tmem_base + T_DS + kk * 8, kt_lo + ((kk * 2048) >> 4), DESC_HI, idesc_dq,
                           (t > 0 || kk) ? 1u : 0u);
          umma_commit_elect(dq_done);
          umma_commit_elect(&k_empty[st]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warpgroups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    const int hf = warp >> 2;                 // which 64 key columns of every tile this warpgroup owns
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int qi = q_lo + row;
    const bool row_valid = qi < p.N;
    const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16);
    if (hf == 0) {
      // Q rows into TMEM as the A operand of S = Q K^T: 16 bf16 pairs per tcgen05.st, zeros past the end
      const __nv_bfloat16* src = qg + (long long)qi * q_stride + (long long)h * HD;
#pragma unroll
      for (int c = 0; c < HD / 2; c += 16) {
        uint32_t r[16];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 u = make_uint4(0u, 0u, 0u, 0u);
          if (row_valid) u = *reinterpret_cast<const uint4*>(src + 2 * c + 8 * v);
          r[4 * v] = u.x; r[4 * v + 1] = u.y; r[4 * v + 2] = u.z; r[4 * v + 3] = u.w;
        }
        tmem_st_32x16(t_row + T_QA + c, r);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(a_ready);
    }
    int lo_row = 0;
    float lse2 = 0.f, dl = 0.f;
    if (row_valid) {
      lo_row = p.doc_start[qi];
      if (p.window > 0) lo_row = max(lo_row, qi - p.window + 1);
      lse2 = p.lse[(long long)h * p.N + qi] * LOG2E;
      dl = p.delta[(long long)h * p.N + qi];
    }
    const uint32_t t_s = t_row + T_S + hf * HALF, t_dp = t_row + T_DP + hf * HALF, t_ds = t_row + T_DS + hf * (HALF / 2);
    bool ok = true;
    for (int t = 0; t < n_tiles && ok; ++t) {
      ok = mbar_wait(sdp_full, t & 1, abort_flag, p.status);
      if (!ok) break;
      tc_fence_after();
      uint32_t s[HALF], dp[HALF], pk[HALF / 2];
      tmem_ld_32x32(t_s, s);
      tmem_ld_32x32(t_s + 32, s + 32);
      tmem_ld_32x32(t_dp, dp);
      tmem_ld_32x32(t_dp + 32, dp + 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sdp_free);     // the S / dP columns may be overwritten by the next tile
      const int k0 = (j_lo + t) * BN + hf * HALF;
      const bool need_mask = (k0 + HALF - 1 > q_lo) || (k0 < lo_last);
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < HALF; e += 2) {
          const int kj = k0 + e;
          const bool v0 = row_valid && kj <= qi && kj >= lo_row;
          const bool v1 = row_valid && kj + 1 <= qi && kj + 1 >= lo_row;
          const float p0 = v0 ? exp2f(fmaf(__uint_as_float(s[e]), p.scale_log2, -lse2)) : 0.f;
          const float p1 = v1 ? exp2f(fmaf(__uint_as_float(s[e + 1]), p.scale_log2, -lse2)) : 0.f;
          pk[e / 2] = pack_bf16x2(p0 * (__uint_as_float(dp[e]) - dl), p1 * (__uint_as_float(dp[e + 1]) - dl));
        }
      } else {
        // packed pairs: one fused multiply-add, one add and one multiply per TWO scores around the two exponentials
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nl2 = make_float2(-lse2, -lse2), nd2 = make_float2(-dl, -dl);
#pragma unroll
        for (int e = 0; e < HALF; e += 2) {
          const float2 t = ffma2(u2f2(s[e], s[e + 1]), sc2, nl2);
          const float2 pr = make_float2(exp2f(t.x), exp2f(t.y));
          const float2 r = fmul2(pr, fadd2(u2f2(dp[e], dp[e + 1]), nd2));
          pk[e / 2] = pack_bf16x2(r.x, r.y);
        }
      }
      if (t > 0) {                               // the previous tile's dQ product has finished reading dS
        ok = mbar_wait(dq_done, (t - 1) & 1, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
      }
      tmem_st_32x16(t_ds, pk);
      tmem_st_32x16(t_ds + 16, pk + 16);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
    if (ok) ok = mbar_wait(dq_done, (n_tiles - 1) & 1, abort_flag, p.status);
    if (ok) {
      tc_fence_after();
      // the two warpgroups split the head dimension of the output
      __nv_bfloat16* drow = p.dq + (long long)qi * p.dqkv_stride + h * HD;
#pragma unroll
      for (int c = hf * (HD / 2); c < (hf + 1) * (HD / 2); c += 32) {
        uint32_t o[32];
        tmem_ld_32x32(t_row + T_DQ + c, o);
        tmem_ld_wait();
        if (row_valid) store_row_bf16(drow + c, o, p.scale);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ============================================================================ dK/dV kernel
// Transposed problem (key rows in TMEM lanes).  All 512 TMEM columns are taken by the two accumulators and the
// S^T / dP^T of one 128-query tile, so the tile is processed as two 64-query halves with their own columns and
// barriers: while one warpgroup turns its half into P^T / dS^T the tensor cores run the other half's products.
// (A form with 128-wide S^T / dP^T and nothing else in flight measured 16 % slower: the round trips between the
// MMA warp and the compute warps, a few hundred cycles each, were then all on the critical path.)
// The per-query terms of P^T = exp2(S^T scale log2e - lse log2e) and dS^T = P^T (dP^T - delta) enter through the
// tensor core: one more K step appends to K and V a block of ones (three columns) and to Q and dO the three-way
// bf16 split of -lse / scale and of -delta, so that the accumulators already hold S^T - lse / scale and
// dP^T - delta.  The compute warps then need one multiply, one exponential and one multiply per element; reading
// the two vectors from shared memory inside that loop had doubled its time (the reads share the issue path of the
// exponentials).
template <int HD>
struct SmemKV {
  static constexpr int TILE = BM * HD * 2;
  static constexpr int K_OFF = 0, V_OFF = TILE, Q_OFF = 2 * TILE, DO_OFF = Q_OFF + STAGES * TILE;
  static constexpr int VEC_OFF = DO_OFF + STAGES * TILE;            // [8 warps][HALF] lowest attendable key per query
  static constexpr int ONES_OFF = VEC_OFF + 8 * HALF * 4;           // [BN x 16] bf16, columns 0..2 = 1 (no swizzle)
  static constexpr int AUG_OFF = ONES_OFF + BN * 32;                // [2][BM x 16] bf16: -lse/scale and -delta, split
  static constexpr int BAR_OFF = AUG_OFF + 2 * BM * 32;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

// TMEM columns: S^T_a [0,64) S^T_b [64,128) dP^T_a [128,192) dP^T_b [192,256) dV [256,384) dK [384,512)
template <int HD>
__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const BwdParams p) {
  using L = SmemKV<HD>;
  constexpr int SLABS = HD / 64;
  constexpr int SLAB_BYTES = BM * 128;
  constexpr int HALF_BYTES = HALF * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1; uint64_t* q_empty = bars + 3;
  uint64_t* sdp_full = bars + 5;      // [2]
  uint64_t* pds_ready = bars + 7;     // [2]
  uint64_t* final_bar = bars + 9;
  uint64_t* aug_init = bars + 10;     // ones block and the first tile's vectors are in shared memory (8 warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* vec = reinterpret_cast<int*>(smem + L::VEC_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.x % p.Hk;
  const int kt = blockIdx.x / p.Hk;               // early key tiles see the most queries: they go first
  const int G = p.Hq / p.Hk;
  const int k0 = kt * BN;
  const int i_lo = k0 / BM;
  const int i_hi = p.kv_last_q[kt] / BM;
  const int n_i = i_hi - i_lo + 1;
  const int n_iter = G * n_i;
  const int n_steps = 2 * n_iter;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&sdp_full[s], 1); mbar_init(&pds_ready[s], 4); }
    mbar_init(final_bar, 1);
    mbar_init(aug_init, 8);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // As in the dQ kernel: the third warpgroup hands registers to the two compute warpgroups.
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
    if (warp == 8) {
      if (lane == 0) {
        mbar_arrive_expect_tx(kv_full, 2 * L::TILE);
#pragma unroll
        for (int s = 0; s < SLABS; ++s) {
          tma_load_2d(smem + L::K_OFF + s * SLAB_BYTES, &tmK, kv_full, kvh * HD + s * 64, k0);
          tma_load_2d(smem + L::V_OFF + s * SLAB_BYTES, &tmV, kv_full, kvh * HD + s * 64, k0);
        }
        bool ok = true;
        for (int it = 0; it < n_iter && ok; ++it) {
          const int g = it / n_i, i = i_lo + it % n_i, h = kvh * G + g;
          const int st = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(&q_empty[st], ph ^ 1, abort_flag, p.status);
          if (!ok) break;
          mbar_arrive_expect_tx(&q_full[st], 2 * L::TILE);
#pragma unroll
          for (int s = 0; s < SLABS; ++s) {
            tma_load_2d(smem + L::Q_OFF + st * L::TILE + s * SLAB_BYTES, &tmQ, &q_full[st], h * HD + s * 64, i * BM);
            tma_load_2d(smem + L::DO_OFF + st * L::TILE + s * SLAB_BYTES, &tmDO, &q_full[st], h * HD + s * 64, i * BM);
          }
        }
      }
    } else if (warp == 9) {
      {   // all 32 lanes run the issue loop; the MMA and commit forms elect one lane
        constexpr uint32_t idesc_s = make_idesc_bf16(BN, HALF, 0, 0);
        constexpr uint32_t idesc_o = make_idesc_bf16(BN, HD, 0, 1);
        const uint32_t sK = smem_u32(smem + L::K_OFF), sV = smem_u32(smem + L::V_OFF);
        const uint32_t sQ = smem_u32(smem + L::Q_OFF), sDO = smem_u32(smem + L::DO_OFF);
        const uint32_t sOnes = smem_u32(smem + L::ONES_OFF), sAug = smem_u32(smem + L::AUG_OFF);
        constexpr uint32_t DESC_HI_AUG = smem_desc_hi_noswizzle(256);
        bool ok = mbar_wait(kv_full, 0, abort_flag, p.status);
        if (ok) ok = mbar_wait(aug_init, 0, abort_flag, p.status);

        auto issue_sdp = [&](int s) -> bool {
          const int hf = s & 1, it = s >> 1, st = it % STAGES;
          if (hf == 0 && !mbar_wait(&q_full[st], (it / STAGES) & 1, abort_flag, p.status)) return false;
          tc_fence_after();
          const uint32_t k_lo = smem_desc_lo(sK, 16), v_lo = smem_desc_lo(sV, 16);
          const uint32_t ones_lo = smem_desc_lo(sOnes, 128);
          const uint32_t augl_lo = smem_desc_lo(sAug + hf * (HALF / 8) * 256, 128);
          const uint32_t augd_lo = smem_desc_lo(sAug + BM * 32 + hf * (HALF / 8) * 256, 128);
          const uint32_t q_lo_d = smem_desc_lo(sQ + st * L::TILE + hf * HALF_BYTES, 16);
          const uint32_t do_lo = smem_desc_lo(sDO + st * L::TILE + hf * HALF_BYTES, 16);
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {      // the two independent chains alternate (see the dQ kernel)
            const uint32_t off = ((kk / 4) * SLAB_BYTES + (kk % 4) * 32) >> 4;
            umma_f16_ss_lh(tmem_base + hf * HALF, k_lo + off, q_lo_d + off, DESC_HI, idesc_s, kk ? 1u : 0u);
            umma_f16_ss_lh(tmem_base + BM + hf * HALF, v_lo + off, do_lo + off, DESC_HI, idesc_s, kk ? 1u : 0u);
          }
          // the appended K step: ones x (-lse / scale) and ones x (-delta)
          umma_f16_ss_lh(tmem_base + hf * HALF, ones_lo, augl_lo, DESC_HI_AUG, idesc_s, 1u);
          umma_f16_ss_lh(tmem_base + BM + hf * HALF, ones_lo, augd_lo, DESC_HI_AUG, idesc_s, 1u);
          umma_commit_elect(&sdp_full[hf]);
          return true;
        };

        if (ok) ok = issue_sdp(0);
        if (ok && n_steps > 1) ok = issue_sdp(1);
        for (int s = 0; s < n_steps && ok; ++s) {
          const int hf = s & 1, it = s >> 1, st = it % STAGES;
          ok = mbar_wait(&pds_ready[hf], it & 1, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t dot_lo = smem_desc_lo(sDO + st * L::TILE + hf * HALF_BYTES, SLAB_BYTES);   // MN-major reads
          const uint32_t qt_lo = smem_desc_lo(sQ + st * L::TILE + hf * HALF_BYTES, SLAB_BYTES);
#pragma unroll
          for (int kk = 0; kk < HALF / 16; ++kk) {
            const uint32_t off = (kk * 2048) >> 4;
            umma_f16_ts_lh(tmem_base + 2 * BM, tmem_base + hf * HALF + kk * 8, dot_lo + off, DESC_HI, idesc_o,         // dV += P^T dO
                           (s > 0 || kk) ? 1u : 0u);
            umma_f16_ts_lh(tmem_base + 3 * BM, tmem_base + BM + hf * HALF + kk * 8, qt_lo + off, DESC_HI, idesc_o,    // dK += dS^T Q
                           (s > 0 || kk) ? 1u : 0u);
          }
          if (hf == 1) umma_commit_elect(&q_empty[st]);
          if (s + 2 < n_steps) ok = issue_sdp(s + 2);
        }
        umma_commit_elect(final_bar);
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    const int hf = warp >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;        // key row == TMEM lane
    const int kj = k0 + row;
    const bool key_valid = kj < p.N;
    const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16);
    const uint32_t t_s = t_row + hf * HALF, t_dp = t_row + BM + hf * HALF;
    int* lo_s = vec + warp * HALF;              // this warp's copy of the lowest attendable key of each query
    bool ok = true;
    // Per-query values of a tile half, fetched from global memory one iteration ahead into registers.  Every lane
    // keeps the lowest attendable key of two queries (masked tiles); in addition thread (quarter, lane) owns ONE
    // row of the appended operand block: quarters 0 / 1 write -lse / scale of queries lane / 32 + lane, quarters
    // 2 / 3 write -delta of the same queries.
    constexpr int VPL = HALF / 32;               // values per lane
    int nx_lo[VPL];
    float nx_val;
    const int aug_q = (quarter & 1) * 32 + lane;                     // query inside the half
    const int aug_row = hf * HALF + aug_q;                           // row of the appended block
    uint8_t* aug_dst = smem + L::AUG_OFF + (quarter >> 1) * (BM * 32) + (aug_row / 8) * 256 + (aug_row % 8) * 16;
    const float inv_scale = 1.0f / p.scale;
    auto fetch_vec = [&](int it) {
      const int g = it / n_i, i = i_lo + it % n_i, h = kvh * G + g;
#pragma unroll
      for (int u = 0; u < VPL; ++u) {
        const int qi = i * BM + hf * HALF + lane + 32 * u;
        nx_lo[u] = 0x7fffffff;
        if (qi < p.N) nx_lo[u] = p.doc_start[qi];
      }
      const int qa = i * BM + hf * HALF + aug_q;
      nx_val = 0.f;       // raw value: nothing may depend on the load before write_aug(), a whole tile later
      if (qa < p.N) nx_val = (quarter < 2) ? p.lse[(long long)h * p.N + qa] : p.delta[(long long)h * p.N + qa];
    };
    auto write_aug = [&]() {                     // three-way bf16 split: the products with 1.0 add up in fp32
      const float x = (quarter < 2) ? -nx_val * inv_scale : -nx_val;
      const __nv_bfloat16 b0 = __float2bfloat16(x);
      const float r1 = x - __bfloat162float(b0);
      const __nv_bfloat16 b1 = __float2bfloat16(r1);
      const __nv_bfloat16 b2 = __float2bfloat16(r1 - __bfloat162float(b1));
      const uint32_t w0 = (uint32_t)__bfloat16_as_ushort(b0) | ((uint32_t)__bfloat16_as_ushort(b1) << 16);
      *reinterpret_cast<uint4*>(aug_dst) = make_uint4(w0, (uint32_t)__bfloat16_as_ushort(b2), 0u, 0u);
    };
    {
      // once per CTA: the ones block (row = TMEM lane of this thread's quarter / lane, written by warpgroup 0), the
      // zero upper halves of the appended rows, and the first tile's vectors
      if (hf == 0) {
        uint8_t* o = smem + L::ONES_OFF + (row / 8) * 256 + (row % 8) * 16;
        *reinterpret_cast<uint4*>(o) = make_uint4(0x3f803f80u, 0x00003f80u, 0u, 0u);
        *reinterpret_cast<uint4*>(o + 128) = make_uint4(0u, 0u, 0u, 0u);
      }
      *reinterpret_cast<uint4*>(aug_dst + 128) = make_uint4(0u, 0u, 0u, 0u);
      if (n_iter > 0) { fetch_vec(0); write_aug(); }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(aug_init);
    }
    for (int it = 0; it < n_iter && ok; ++it) {
      const int i = i_lo + it % n_i;
      const int q_first = i * BM + hf * HALF;
      __syncwarp();                              // the previous iteration's reads of lo_s are done
#pragma unroll
      for (int u = 0; u < VPL; ++u) {
        int lo = nx_lo[u];
        if (p.window > 0 && lo != 0x7fffffff) lo = max(lo, q_first + lane + 32 * u - p.window + 1);
        lo_s[lane + 32 * u] = lo;
      }
      __syncwarp();
      if (it + 1 < n_iter) fetch_vec(it + 1);
      ok = mbar_wait(&sdp_full[hf], it & 1, abort_flag, p.status);
      if (!ok) break;
      tc_fence_after();
      uint32_t s[HALF], dp[HALF], pk[HALF / 2], dk_[HALF / 2];
      tmem_ld_32x32(t_s, s);
      tmem_ld_32x32(t_s + 32, s + 32);
      tmem_ld_32x32(t_dp, dp);
      tmem_ld_32x32(t_dp + 32, dp + 32);
      tmem_ld_wait();
      const bool need_mask = (q_first < k0 + BN - 1) || (lo_s[HALF - 1] > k0) || (k0 + BN > p.N);
      // the accumulators hold S^T - lse / scale and dP^T - delta
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < HALF; e += 4) {
          const int4 lo4 = *reinterpret_cast<const int4*>(lo_s + e);
          const int lov[4] = {lo4.x, lo4.y, lo4.z, lo4.w};
          float pr[4], ds[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int qi = q_first + e + u;
            const bool valid = key_valid && kj <= qi && kj >= lov[u];
            pr[u] = valid ? exp2f(__uint_as_float(s[e + u]) * p.scale_log2) : 0.f;
            ds[u] = pr[u] * __uint_as_float(dp[e + u]);
          }
          pk[e / 2] = pack_bf16x2(pr[0], pr[1]); pk[e / 2 + 1] = pack_bf16x2(pr[2], pr[3]);
          dk_[e / 2] = pack_bf16x2(ds[0], ds[1]); dk_[e / 2 + 1] = pack_bf16x2(ds[2], ds[3]);
        }
      } else {
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
#pragma unroll
        for (int e = 0; e < HALF; e += 2) {
          const float2 t = fmul2(u2f2(s[e], s[e + 1]), sc2);
          const float2 pr = make_float2(exp2f(t.x), exp2f(t.y));
          const float2 r = fmul2(pr, u2f2(dp[e], dp[e + 1]));
          pk[e / 2] = pack_bf16x2(pr.x, pr.y);
          dk_[e / 2] = pack_bf16x2(r.x, r.y);
        }
      }
      // the next tile's vectors for this half: the products that read the current ones have completed (sdp_full),
      // and the arrival below orders these writes in front of the next S^T / dP^T of this half
      if (it + 1 < n_iter) { write_aug(); fence_proxy_async(); }
      tmem_st_32x16(t_s, pk);
      tmem_st_32x16(t_s + 16, pk + 16);
      tmem_st_32x16(t_dp, dk_);
      tmem_st_32x16(t_dp + 16, dk_ + 16);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_ready[hf]);
    }
    if (ok) ok = mbar_wait(final_bar, 0, abort_flag, p.status);
    if (ok) {
      tc_fence_after();
      // warpgroup 0 writes dV, warpgroup 1 writes dK (scaled)
      __nv_bfloat16* drow = (hf == 0 ? p.dv : p.dk) + (long long)kj * p.dqkv_stride + kvh * HD;
      const uint32_t t_acc = t_row + (2 + hf) * BM;
      const float mul = hf == 0 ? 1.0f : p.scale;
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t o[32];
        tmem_ld_32x32(t_acc + c, o);
        tmem_ld_wait();
        if (key_valid) store_row_bf16(drow + c, o, mul);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace attnb
}  // namespace ob

using namespace ob;
using namespace ob::attnb;

template <int HD>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                      const __nv_bfloat16* qg, long long q_stride, const __nv_bfloat16* dog, long long do_stride,
                      const BwdParams& p, cudaStream_t stream) {
  auto kq = attn_bwd_dq_kernel<HD>;
  auto kkv = attn_bwd_dkv_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    OB_CUDA_CHECK(cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemQ<HD>::TOTAL));
    OB_CUDA_CHECK(cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemKV<HD>::TOTAL));
    configured = true;
  }
  const int n_qtiles = (p.N + BM - 1) / BM, n_ktiles = (p.N + BN - 1) / BN;
  kkv<<<n_ktiles * p.Hk, THREADS, SmemKV<HD>::TOTAL, stream>>>(tq, tk, tv, tdo, p);
  kq<<<n_qtiles * p.Hq, THREADS, SmemQ<HD>::TOTAL, stream>>>(tk, tv, tdo, qg, q_stride, p);
  return (int)cudaGetLastError();
}

// q, k, v: post-RoPE projections (views of one buffer, token stride qkv_stride); out / dout: [N, Hq*hd]
// (token stride out_stride); lse: fp32 [Hq, N] from the forward; delta: fp32 scratch [Hq, N];
// dq, dk, dv: views of one gradient buffer with token stride dqkv_stride; kv_last: int32 scratch
// of ceil(N / 128) entries.
extern "C" int ob_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                           const void* lse, void* delta, void* dq, void* dk, void* dv, const void* doc_start,
                           void* kv_last, int N, int Hq, int Hk, int hd, long long qkv_stride, long long out_stride,
                           long long dqkv_stride, float scale, int window, int* status, cudaStream_t stream) {
  if (N <= 0) return 0;
  if (hd != 64 && hd != 128) return -1;
  CUtensorMap tq, tk, tv, tdo;
  int rc = make_tmap_2d(&tq, q, N, (uint64_t)Hq * hd, qkv_stride, BM, 64, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tk, k, N, (uint64_t)Hk * hd, qkv_stride, BN, 64, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tv, v, N, (uint64_t)Hk * hd, qkv_stride, BN, 64, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tdo, dout, N, (uint64_t)Hq * hd, out_stride, BM, 64, 2);
  if (rc) return rc;
  const int n_ktiles = (N + BN - 1) / BN;
  long long items = (long long)N * Hq;
  int grid = (int)((items + 7) / 8 < 148 * 16 ? (items + 7) / 8 : 148 * 16);
  delta_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)dout, out_stride, out_stride,
                                         (float*)delta, N, Hq, hd);
  kv_last_q_kernel<<<(n_ktiles + 127) / 128, 128, 0, stream>>>((const int*)doc_start, N, window, (int*)kv_last, n_ktiles);
  BwdParams p{N, Hq, Hk, window, scale, scale * LOG2E, (const int*)doc_start, (const float*)lse, (const float*)delta,
              (__nv_bfloat16*)dq, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, dqkv_stride, (const int*)kv_last, status};
  const __nv_bfloat16* qg = (const __nv_bfloat16*)q;
  const __nv_bfloat16* dog = (const __nv_bfloat16*)dout;
  return hd == 128 ? launch_bwd<128>(tq, tk, tv, tdo, qg, qkv_stride, dog, out_stride, p, stream)
                   : launch_bwd<64>(tq, tk, tv, tdo, qg, qkv_stride, dog, out_stride, p, stream);
}
