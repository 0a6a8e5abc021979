// Flash-attention forward for sm_100a: causal, document-masked, sliding-window, GQA.
//
// Tokens form one flat stream of N positions (batches and packed documents are described by
// doc_start[i] = index of the first token of i's document).  Query i attends keys j with
//     max(doc_start[i], i - window + 1) <= j <= i          (window = 0: no window)
//
// One CTA handles two 128-row query tiles of one head (256 queries) against 128-key tiles:
//   warps 0-3 / 4-7 : softmax warpgroups, one per query tile; thread t owns query row t
//                     (TMEM lane t): reads S with tcgen05.ld, keeps running max / sum, writes
//                     P (bf16) back into TMEM over S, rescales O lazily
//   warp 8          : TMA producer (Q once, then K and V tiles through 2-stage rings)
//   warp 9          : MMA issuer: S = Q K^T (operands in smem), O += P V (P from TMEM, V in smem
//                     read as an MN-major operand), interleaved so that one warpgroup's softmax
//                     overlaps the other tile's tensor-core work
// TMEM: S0 | S1 | O0 | O1, 128 fp32 columns each.  Key tiles that are fully masked for a query
// tile are skipped; masks are applied only on boundary tiles.
#include "common.cuh"
#include "tensormap.cuh"

namespace ob {
namespace attn {

constexpr int BM = 128;       // query rows per tile
constexpr int BN = 128;       // keys per tile
constexpr int NQ = 2;         // query tiles per CTA
constexpr int KV_STAGES = 2;
constexpr int THREADS = 384;      // 8 softmax warps + TMA warp + MMA warp + 2 warps that only give up registers
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr float RESCALE_THRESHOLD = 8.0f;   // in log2 units

struct FwdParams {
  int N, Hq, Hk, window;
  float scale_log2;           // softmax scale * log2(e)
  const int* doc_start;
  __nv_bfloat16* out;
  long long out_stride;       // elements between tokens of out
  float* lse;                 // [Hq, N], natural log
  int* status;
};

template <int HD>
struct Smem {
  static constexpr int TILE = BM * HD * 2;                 // bytes of one 128 x HD bf16 tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = NQ * TILE;
  static constexpr int V_OFF = K_OFF + KV_STAGES * TILE;
  static constexpr int BAR_OFF = V_OFF + KV_STAGES * TILE;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

struct TileRange {
  int lo, hi;   // inclusive key-tile range; lo > hi means inactive
  int q_lo, q_hi;
  int lo_first, lo_last;   // lowest attendable key of the first / last row of the tile
};

__device__ __forceinline__ TileRange tile_range(int q0, int q, const FwdParams& p) {
  TileRange r;
  r.q_lo = q0 + q * BM;
  if (r.q_lo >= p.N) { r.lo = 1; r.hi = 0; r.q_hi = r.q_lo; r.lo_first = r.lo_last = 0; return r; }
  r.q_hi = min(r.q_lo + BM - 1, p.N - 1);
  int lf = p.doc_start[r.q_lo], ll = p.doc_start[r.q_hi];
  if (p.window > 0) { lf = max(lf, r.q_lo - p.window + 1); ll = max(ll, r.q_hi - p.window + 1); }
  r.lo_first = lf; r.lo_last = ll;
  r.lo = lf / BN;
  r.hi = r.q_hi / BN;
  return r;
}

template <int HD>
__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  using L = Smem<HD>;
  constexpr int SLABS = HD / 64;            // 64-column (128-byte) slabs per tile
  constexpr int SLAB_BYTES = BM * 128;      // 16 KB
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;                   // [1]
  uint64_t* k_full = bars + 1;               // [KV_STAGES]
  uint64_t* k_empty = bars + 3;
  uint64_t* v_full = bars + 5;
  uint64_t* v_empty = bars + 7;
  uint64_t* s_full = bars + 9;               // [NQ]
  uint64_t* p_ready = bars + 11;             // [NQ]
  uint64_t* o_final = bars + 13;             // [NQ]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qblocks = (p.N + NQ * BM - 1) / (NQ * BM);
  const int h = blockIdx.x % p.Hq;
  const int qb = n_qblocks - 1 - blockIdx.x / p.Hq;     // heaviest (latest) query blocks first
  const int kvh = h / (p.Hq / p.Hk);
  const int q0 = qb * NQ * BM;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    for (int q = 0; q < NQ; ++q) { mbar_init(&s_full[q], 1); mbar_init(&p_ready[q], 4); mbar_init(&o_final[q], 1); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  TileRange tr[NQ];
#pragma unroll
  for (int q = 0; q < NQ; ++q) tr[q] = tile_range(q0, q, p);
  int jmin = 1 << 30, jmax = -1;
#pragma unroll
  for (int q = 0; q < NQ; ++q) if (tr[q].lo <= tr[q].hi) { jmin = min(jmin, tr[q].lo); jmax = max(jmax, tr[q].hi); }

  // The third warpgroup (two single-thread roles and two idle warps) hands registers to the two compute
  // warpgroups, whose threads hold a whole row of a tile.
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
    if (warp == 8) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0 && jmax >= jmin) {
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
        mbar_arrive_expect_tx(q_full, NQ * L::TILE);
#pragma unroll
        for (int q = 0; q < NQ; ++q)
#pragma unroll
          for (int s = 0; s < SLABS; ++s)
            tma_load_2d(smem + L::Q_OFF + q * L::TILE + s * SLAB_BYTES, &tmQ, q_full, h * HD + s * 64, q0 + q * BM);
        bool ok = true;
        for (int j = jmin; j <= jmax && ok; ++j) {
          const int t = j - jmin, st = t % KV_STAGES;
          const uint32_t ph = (t / KV_STAGES) & 1;
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
      if (jmax >= jmin) {   // all 32 lanes run the issue loop; the MMA and commit forms elect one lane
        constexpr uint32_t idesc_s = make_idesc_bf16(BM, BN, 0, 0);
        constexpr uint32_t idesc_pv = make_idesc_bf16(BM, HD, 0, 1);
        const uint32_t sQ = smem_u32(smem + L::Q_OFF), sK = smem_u32(smem + L::K_OFF), sV = smem_u32(smem + L::V_OFF);
        uint32_t p_phase[NQ] = {0, 0};
        bool ok = mbar_wait(q_full, 0, abort_flag, p.status);

        constexpr uint32_t DESC_HI = smem_desc_hi_sw128(1024);
        auto issue_s = [&](int q, int j) {
          const int st = (j - jmin) % KV_STAGES;
          const uint32_t a_lo = smem_desc_lo(sQ + q * L::TILE, 16), b_lo = smem_desc_lo(sK + st * L::TILE, 16);
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t off = ((kk / 4) * SLAB_BYTES + (kk % 4) * 32) >> 4;
            umma_f16_ss_lh(tmem_base + q * BN, a_lo + off, b_lo + off, DESC_HI, idesc_s, kk ? 1u : 0u);
          }
          umma_commit_elect(&s_full[q]);
        };
        auto issue_pv = [&](int q, int j, bool accumulate) {
          const int st = (j - jmin) % KV_STAGES;
          // A: P in TMEM, 16 bf16 per 8 columns; B: V tile read MN-major (hd contiguous), 16 keys = 2048 bytes
          const uint32_t b_lo = smem_desc_lo(sV + st * L::TILE, SLAB_BYTES);
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk)
            umma_f16_ts_lh(tmem_base + 2 * BN + q * BN, tmem_base + q * BN + kk * 8, b_lo + ((kk * 2048) >> 4), DESC_HI,
                           idesc_pv, (accumulate || kk) ? 1u : 0u);
        };
        auto active = [&](int q, int j) { return tr[q].lo <= tr[q].hi && j >= tr[q].lo && j <= tr[q].hi; };
        auto kv_wait = [&](uint64_t* bar, int j) {
          const int t = j - jmin;
          return mbar_wait(&bar[t % KV_STAGES], (t / KV_STAGES) & 1, abort_flag, p.status);
        };

        if (ok) ok = kv_wait(k_full, jmin);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int q = 0; q < NQ; ++q) if (active(q, jmin)) issue_s(q, jmin);
          umma_commit_elect(&k_empty[0]);
        }
        for (int j = jmin; j <= jmax && ok; ++j) {
          ok = kv_wait(v_full, j);
          if (ok && j + 1 <= jmax) ok = kv_wait(k_full, j + 1);
          if (!ok) break;
#pragma unroll
          for (int q = 0; q < NQ; ++q) {
            if (active(q, j)) {
              ok = mbar_wait(&p_ready[q], p_phase[q], abort_flag, p.status);
              if (!ok) break;
              p_phase[q] ^= 1;
              tc_fence_after();
              issue_pv(q, j, j > tr[q].lo);
            }
            if (j + 1 <= jmax && active(q, j + 1)) issue_s(q, j + 1);
          }
          if (!ok) break;
          umma_commit_elect(&v_empty[(j - jmin) % KV_STAGES]);
          if (j + 1 <= jmax) umma_commit_elect(&k_empty[(j + 1 - jmin) % KV_STAGES]);
        }
#pragma unroll
        for (int q = 0; q < NQ; ++q) if (tr[q].lo <= tr[q].hi) umma_commit_elect(&o_final[q]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    const int q = warp >> 2;                 // query tile of this warpgroup
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;     // row inside the tile == TMEM lane
    const TileRange r = tr[q];
    if (r.lo <= r.hi) {
      const int qi = r.q_lo + row;
      const bool row_valid = qi < p.N;
      int lo_row = 0;
      if (row_valid) {
        lo_row = p.doc_start[qi];
        if (p.window > 0) lo_row = max(lo_row, qi - p.window + 1);
      }
      const uint32_t t_s = tmem_base + (uint32_t(quarter * 32) << 16) + q * BN;
      const uint32_t t_o = tmem_base + (uint32_t(quarter * 32) << 16) + 2 * BN + q * BN;
      float m_run = -INFINITY, l_run = 0.f;
      uint32_t s_phase = 0;
      bool ok = true;
      for (int j = r.lo; j <= r.hi && ok; ++j) {
        ok = mbar_wait(&s_full[q], s_phase, abort_flag, p.status);
        if (!ok) break;
        s_phase ^= 1;
        tc_fence_after();
        float s[BN];
#pragma unroll
        for (int c = 0; c < BN; c += 32) tmem_ld_32x32(t_s + c, reinterpret_cast<uint32_t*>(s + c));
        tmem_ld_wait();
        const int k0 = j * BN;
        const bool need_mask = (k0 + BN - 1 > r.q_lo) || (k0 < r.lo_last);
        // Unmasked tiles work on the raw scores: the maximum commutes with the (positive) scale, and scale and
        // reference maximum fold into one fused multiply-add per PAIR of scores in front of the exponential.
        float mx = -INFINITY;
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < BN; ++c) {
            const int kj = k0 + c;
            const bool valid = row_valid && kj <= qi && kj >= lo_row;
            s[c] = valid ? s[c] : -INFINITY;
            mx = fmaxf(mx, s[c]);
          }
        } else {
          float mx2 = -INFINITY;
#pragma unroll
          for (int c = 0; c < BN; c += 4) { mx = fmax3(mx, s[c], s[c + 1]); mx2 = fmax3(mx2, s[c + 2], s[c + 3]); }
          mx = fmaxf(mx, mx2);
        }
        mx *= p.scale_log2;          // -inf stays -inf
        // lazy rescale: keep the old reference max unless the new one is much larger
        float alpha = 1.0f;
        const float m_new = fmaxf(m_run, mx);
        const bool bump = (m_new > m_run + RESCALE_THRESHOLD) || (m_run == -INFINITY && m_new > -INFINITY);
        if (bump) {
          alpha = (m_run == -INFINITY) ? 0.0f : exp2f(m_run - m_new);
          m_run = m_new;
          l_run *= alpha;
        }
        const float m_use = (m_run == -INFINITY) ? 0.0f : m_run;
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(-m_use, -m_use);
        float2 sum2 = make_float2(0.f, 0.f), sum2b = make_float2(0.f, 0.f);   // two chains of packed adds
        // P (bf16) goes back over S in four stores of 16 columns as it is produced: the thread holds all of S in
        // registers by now, and at most 16 packed results at a time
#pragma unroll
        for (int cc = 0; cc < BN; cc += 32) {
          uint32_t pk[16];
#pragma unroll
          for (int c = cc; c < cc + 32; c += 4) {
            const float2 t0 = ffma2(make_float2(s[c], s[c + 1]), sc2, nm2);     // masked scores: -inf * scale = -inf
            const float2 t1 = ffma2(make_float2(s[c + 2], s[c + 3]), sc2, nm2);
            const float2 e0 = make_float2(exp2f(t0.x), exp2f(t0.y));
            const float2 e1 = make_float2(exp2f(t1.x), exp2f(t1.y));
            sum2 = fadd2(sum2, e0);
            sum2b = fadd2(sum2b, e1);
            pk[(c - cc) / 2] = pack_bf16x2(e0.x, e0.y);
            pk[(c - cc) / 2 + 1] = pack_bf16x2(e1.x, e1.y);
          }
          tmem_st_32x16(t_s + cc / 2, pk);
        }
        sum2 = fadd2(sum2, sum2b);
        const float sum = sum2.x + sum2.y;
        l_run += sum;
        if (j > r.lo && __any_sync(0xffffffffu, bump)) {
          // O of this tile was produced with the old reference max: scale it (whole warp takes part)
#pragma unroll
          for (int c = 0; c < HD; c += 16) {
            uint32_t o[16];
            tmem_ld_32x16(t_o + c, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st_32x16(t_o + c, o);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[q]);
      }
      if (ok) ok = mbar_wait(&o_final[q], 0, abort_flag, p.status);
      if (ok) {
        tc_fence_after();
        const float inv_l = l_run > 0.f ? 1.0f / l_run : 0.f;
        if (row_valid) p.lse[(long long)h * p.N + qi] = (l_run > 0.f) ? (m_run + log2f(l_run)) * LN2 : -INFINITY;
        __nv_bfloat16* orow = p.out + (long long)qi * p.out_stride + h * HD;
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32(t_o + c, o);
          tmem_ld_wait();
          if (row_valid) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(o[8 * v]) * inv_l, __uint_as_float(o[8 * v + 1]) * inv_l);
              w.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * inv_l, __uint_as_float(o[8 * v + 3]) * inv_l);
              w.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * inv_l, __uint_as_float(o[8 * v + 5]) * inv_l);
              w.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * inv_l, __uint_as_float(o[8 * v + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + c + 8 * v) = w;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace attn
}  // namespace ob

using namespace ob;
using namespace ob::attn;

template <int HD>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& p,
                      cudaStream_t stream) {
  auto kern = attn_fwd_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    OB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<HD>::TOTAL));
    configured = true;
  }
  const int n_qblocks = (p.N + NQ * BM - 1) / (NQ * BM);
  kern<<<n_qblocks * p.Hq, THREADS, Smem<HD>::TOTAL, stream>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

// q, k, v: bf16 [N, H*, hd] views with token strides (elements); heads contiguous.
// out: bf16 [N, Hq*hd] with token stride out_stride; lse: fp32 [Hq, N].
extern "C" int ob_attn_fwd(const void* q, const void* k, const void* v, void* out, void* lse, const void* doc_start,
                           int N, int Hq, int Hk, int hd, long long q_stride, long long kv_stride, long long out_stride,
                           float scale, int window, int* status, cudaStream_t stream) {
  if (N <= 0) return 0;
  if (hd != 64 && hd != 128) return -1;
  if (Hq % Hk != 0) return -2;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_2d(&tq, q, N, (uint64_t)Hq * hd, q_stride, BM, 64, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tk, k, N, (uint64_t)Hk * hd, kv_stride, BN, 64, 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tv, v, N, (uint64_t)Hk * hd, kv_stride, BN, 64, 2);
  if (rc) return rc;
  FwdParams p{N, Hq, Hk, window, scale * LOG2E, (const int*)doc_start, (__nv_bfloat16*)out, out_stride, (float*)lse,
              status};
  return hd == 128 ? launch_fwd<128>(tq, tk, tv, p, stream) : launch_fwd<64>(tq, tk, tv, p, stream);
}
