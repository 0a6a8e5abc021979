// Single-query ("decode") attention against a key/value cache, with the cache append fused in.
//
//   q        [B, Hq, HD]     bf16, row stride q_stride (it usually lives inside the fused qkv row)
//   k_new    [B, Hk, HD]     bf16, the current token's key (already normalised / rotated); v_new alike
//   k_cache  logical [B, Tmax, Hk, HD] bf16 with arbitrary batch / token / head strides (v_cache alike;
//            a head-major allocation gives every CTA one contiguous stream); sequence b holds seq_lens[b] tokens *including*
//            the current one, whose row (seq_lens[b] - 1) this kernel writes before it attends
//   out      [B, Hq, HD]     bf16
//
// The kernel is bound by the cache read, so it is organised around keeping loads in flight rather
// than around tensor cores: one CTA per (kv head, sequence, split of the sequence) streams 64-token
// K and V tiles through shared memory with cp.async double buffering; all query heads that share
// the kv head (GQA group, up to 8) are served from the same tile.  With more than one split the
// partial (max, sum, accumulator) triples are merged by a second small kernel.
#include "common.cuh"

namespace ob {
namespace decode {

constexpr int TILE = 64;
constexpr int THREADS = 128;
constexpr int MAX_REP = 8;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int HD>
struct Smem {
  static constexpr int KPAD = HD + 8;  // 16-byte skew per row: conflict-free 16-byte row reads
  __nv_bfloat16 k[2][TILE][KPAD];
  __nv_bfloat16 v[2][TILE][HD];
  float q[MAX_REP][HD];
  float s[MAX_REP][TILE];
  float m[MAX_REP], l[MAX_REP], alpha[MAX_REP];
  float red[THREADS / HD > 1 ? MAX_REP * THREADS : 1];
};

template <int HD>
__device__ __forceinline__ void load_tile(Smem<HD>& sm, int buf, const __nv_bfloat16* kbase, const __nv_bfloat16* vbase,
                                          long long tok_stride, int t_first, int t_end) {
  constexpr int CH = HD / 8;  // 16-byte chunks per row
  for (int i = threadIdx.x; i < TILE * CH; i += THREADS) {
    const int r = i / CH, c = i - r * CH;
    const int t = t_first + r;
    if (t < t_end) {
      cp_async_16(&sm.k[buf][r][c * 8], kbase + (long long)t * tok_stride + c * 8);
      cp_async_16(&sm.v[buf][r][c * 8], vbase + (long long)t * tok_stride + c * 8);
    }
  }
}

template <int HD>
__global__ void __launch_bounds__(THREADS, 3)
decode_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ k_new,
              const __nv_bfloat16* __restrict__ v_new, long long new_stride, __nv_bfloat16* __restrict__ k_cache,
              __nv_bfloat16* __restrict__ v_cache, long long batch_stride, long long tok_stride, long long head_stride,
              const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ out, long long out_stride,
              float* __restrict__ part_o, float* __restrict__ part_ml, int Hq, int Hk, int n_splits, int t_max,
              float scale_log2, int window) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  Smem<HD>& sm = *reinterpret_cast<Smem<HD>*>(smem_raw);
  const int hk = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int n_rep = Hq / Hk;
  const int tid = threadIdx.x;
  int len = seq_lens[b];
  if (len > t_max) len = t_max;
  if (len < 0) len = 0;  // an empty sequence still writes zeros / empty partials
  __nv_bfloat16* kc = k_cache + (long long)b * batch_stride + (long long)hk * head_stride;
  __nv_bfloat16* vc = v_cache + (long long)b * batch_stride + (long long)hk * head_stride;
  const int start = (window > 0 && len > window) ? len - window : 0;
  const int span = len - start;
  const int per = ((span + n_splits - 1) / n_splits + TILE - 1) / TILE * TILE;
  const int t0 = start + split * per;
  const int t1 = min(len, t0 + per);

  // fused append: the CTA whose range ends at the current token stores it into the cache first
  if (k_new != nullptr && t1 == len && t0 < t1) {
    if (tid < HD / 8) {
      const uint4 kv = *reinterpret_cast<const uint4*>(k_new + (long long)b * new_stride + (long long)hk * HD + tid * 8);
      *reinterpret_cast<uint4*>(kc + (long long)(len - 1) * tok_stride + tid * 8) = kv;
    } else if (tid < HD / 4) {
      const int c = tid - HD / 8;
      const uint4 vv = *reinterpret_cast<const uint4*>(v_new + (long long)b * new_stride + (long long)hk * HD + c * 8);
      *reinterpret_cast<uint4*>(vc + (long long)(len - 1) * tok_stride + c * 8) = vv;
    }
  }
  for (int i = tid; i < n_rep * HD; i += THREADS) {
    const int r = i / HD, d = i - r * HD;
    sm.q[r][d] = __bfloat162float(q[(long long)b * q_stride + (long long)(hk * n_rep + r) * HD + d]) * scale_log2;
  }
  if (tid < MAX_REP) { sm.m[tid] = -INFINITY; sm.l[tid] = 0.f; sm.alpha[tid] = 1.f; }
  __syncthreads();  // also orders the appended row before the cp.async reads below

  constexpr int SUB = THREADS / HD;       // position subsets in the PV phase (1 for HD 128, 2 for HD 64)
  const int d = tid % HD, sub = tid / HD;
  float acc[MAX_REP];
#pragma unroll
  for (int r = 0; r < MAX_REP; ++r) acc[r] = 0.f;

  const int n_tiles = t0 < t1 ? (t1 - t0 + TILE - 1) / TILE : 0;
  if (n_tiles > 0) load_tile<HD>(sm, 0, kc, vc, tok_stride, t0, t1);
  cp_async_commit();
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < n_tiles) load_tile<HD>(sm, buf ^ 1, kc, vc, tok_stride, t0 + (tile + 1) * TILE, t1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int valid = min(TILE, t1 - (t0 + tile * TILE));
    // scores: one (query head, position) pair per work item
    for (int item = tid; item < n_rep * TILE; item += THREADS) {
      const int r = item / TILE, t = item - r * TILE;
      float dot = -INFINITY;
      if (t < valid) {
        // four independent partial sums: one serial chain of 128 dependent FMAs would cost more than the loads
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
        const uint4* krow = reinterpret_cast<const uint4*>(&sm.k[buf][t][0]);
        const float4* qrow = reinterpret_cast<const float4*>(&sm.q[r][0]);
#pragma unroll
        for (int c = 0; c < HD / 8; ++c) {
          const uint4 kk = krow[c];
          const float4 qa = qrow[2 * c], qb = qrow[2 * c + 1];
          const float2 k0 = unpack_bf16x2(kk.x), k1 = unpack_bf16x2(kk.y), k2 = unpack_bf16x2(kk.z), k3 = unpack_bf16x2(kk.w);
          d0 = fmaf(qa.x, k0.x, d0); d1 = fmaf(qa.y, k0.y, d1); d2 = fmaf(qa.z, k1.x, d2); d3 = fmaf(qa.w, k1.y, d3);
          d0 = fmaf(qb.x, k2.x, d0); d1 = fmaf(qb.y, k2.y, d1); d2 = fmaf(qb.z, k3.x, d2); d3 = fmaf(qb.w, k3.y, d3);
        }
        dot = (d0 + d1) + (d2 + d3);
      }
      sm.s[r][t] = dot;
    }
    __syncthreads();
    // online softmax bookkeeping: warp w owns query heads w, w + 4
    {
      const int warp = tid >> 5, lane = tid & 31;
      for (int r = warp; r < n_rep; r += THREADS / 32) {
        const float s0 = sm.s[r][lane], s1 = sm.s[r][lane + 32];
        const float m_old = sm.m[r];
        const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
        const float p0 = exp2f(s0 - m_new), p1 = exp2f(s1 - m_new);
        sm.s[r][lane] = p0;
        sm.s[r][lane + 32] = p1;
        const float sum = warp_sum(p0 + p1);
        if (lane == 0) {
          const float a = exp2f(m_old - m_new);
          sm.alpha[r] = a;
          sm.l[r] = sm.l[r] * a + sum;
          sm.m[r] = m_new;
        }
      }
    }
    __syncthreads();
    // P V: thread owns output dimension d (and every SUB-th position)
#pragma unroll
    for (int r = 0; r < MAX_REP; ++r)
      if (r < n_rep) acc[r] *= sm.alpha[r];
    {
      // positions in groups of four: the probabilities come as one float4 (broadcast) per query head,
      // and the four products per head are summed as a tree before they join the accumulator
      const int t_end4 = (SUB == 1) ? (valid & ~3) : 0;
      for (int t = 0; t < t_end4; t += 4) {
        const float v0 = __bfloat162float(sm.v[buf][t][d]), v1 = __bfloat162float(sm.v[buf][t + 1][d]);
        const float v2 = __bfloat162float(sm.v[buf][t + 2][d]), v3 = __bfloat162float(sm.v[buf][t + 3][d]);
#pragma unroll
        for (int r = 0; r < MAX_REP; ++r)
          if (r < n_rep) {
            const float4 p4 = *reinterpret_cast<const float4*>(&sm.s[r][t]);
            acc[r] += (p4.x * v0 + p4.y * v1) + (p4.z * v2 + p4.w * v3);
          }
      }
      for (int t = t_end4 + sub; t < valid; t += SUB) {
        const float vv = __bfloat162float(sm.v[buf][t][d]);
#pragma unroll
        for (int r = 0; r < MAX_REP; ++r)
          if (r < n_rep) acc[r] += sm.s[r][t] * vv;
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  if (SUB > 1) {
#pragma unroll
    for (int r = 0; r < MAX_REP; ++r)
      if (r < n_rep) sm.red[r * THREADS + tid] = acc[r];
    __syncthreads();
    if (sub == 0) {
#pragma unroll
      for (int r = 0; r < MAX_REP; ++r)
        if (r < n_rep)
          for (int s2 = 1; s2 < SUB; ++s2) acc[r] += sm.red[r * THREADS + s2 * HD + d];
    }
  }
  if (sub != 0) return;
#pragma unroll
  for (int r = 0; r < MAX_REP; ++r) {
    if (r >= n_rep) break;
    const int hq = hk * n_rep + r;
    if (n_splits == 1) {
      const float l = sm.l[r];
      out[(long long)b * out_stride + (long long)hq * HD + d] = __float2bfloat16(l > 0.f ? acc[r] / l : 0.f);
    } else {
      const long long slot = ((long long)b * Hq + hq) * n_splits + split;
      part_o[slot * HD + d] = acc[r];
      if (d == 0) { part_ml[slot * 2] = sm.m[r]; part_ml[slot * 2 + 1] = sm.l[r]; }
    }
  }
}

template <int HD>
__global__ void __launch_bounds__(HD)
combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
               long long out_stride, int Hq, int n_splits) {
  const int hq = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const long long base = ((long long)b * Hq + hq) * n_splits;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[(base + s) * 2]);
  float num = 0.f, den = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    if (ms == -INFINITY) continue;
    const float w = exp2f(ms - m);
    num += w * part_o[(base + s) * HD + d];
    den += w * part_ml[(base + s) * 2 + 1];
  }
  out[(long long)b * out_stride + (long long)hq * HD + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
}

template <int HD>
static int launch(const void* q, long long q_stride, const void* k_new, const void* v_new, long long new_stride,
                  void* k_cache, void* v_cache, long long batch_stride, long long tok_stride, long long head_stride,
                  const int* seq_lens, void* out, long long out_stride, float* part_o, float* part_ml, int B, int Hq, int Hk, int n_splits,
                  int t_max, float scale, int window, cudaStream_t stream) {
  auto kern = decode_kernel<HD>;
  static bool configured = false;
  const int smem = (int)sizeof(Smem<HD>);
  if (!configured) {
    OB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  dim3 grid(Hk, B, n_splits);
  kern<<<grid, THREADS, smem, stream>>>((const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_new,
                                        (const __nv_bfloat16*)v_new, new_stride, (__nv_bfloat16*)k_cache,
                                        (__nv_bfloat16*)v_cache, batch_stride, tok_stride, head_stride, seq_lens,
                                        (__nv_bfloat16*)out, out_stride, part_o, part_ml, Hq, Hk, n_splits, t_max,
                                        scale * 1.4426950408889634f, window);
  int rc = (int)cudaGetLastError();
  if (rc || n_splits == 1) return rc;
  combine_kernel<HD><<<dim3(Hq, B), HD, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, out_stride, Hq, n_splits);
  return (int)cudaGetLastError();
}

}  // namespace decode
}  // namespace ob

// n_splits > 1 needs part_o [B*Hq*n_splits*hd] and part_ml [B*Hq*n_splits*2] fp32 workspaces.
// k_new / v_new may be null when the cache already holds the current token.
extern "C" int ob_attn_decode(const void* q, long long q_stride, const void* k_new, const void* v_new,
                              long long new_stride, void* k_cache, void* v_cache, long long batch_stride,
                              long long tok_stride, long long head_stride, const void* seq_lens, void* out, long long out_stride,
                              void* part_o, void* part_ml, int B, int Hq, int Hk, int hd, int n_splits, int t_max,
                              float scale, int window, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (Hk <= 0 || Hq % Hk != 0 || Hq / Hk > ob::decode::MAX_REP || n_splits < 1) return -1;
  if (n_splits > 1 && (part_o == nullptr || part_ml == nullptr)) return -2;
  if ((q_stride | new_stride | batch_stride | tok_stride | head_stride | out_stride) % 8 != 0) return -3;
  if (hd == 128)
    return ob::decode::launch<128>(q, q_stride, k_new, v_new, new_stride, k_cache, v_cache, batch_stride, tok_stride, head_stride,
                                   (const int*)seq_lens, out, out_stride, (float*)part_o, (float*)part_ml, B, Hq, Hk,
                                   n_splits, t_max, scale, window, stream);
  if (hd == 64)
    return ob::decode::launch<64>(q, q_stride, k_new, v_new, new_stride, k_cache, v_cache, batch_stride, tok_stride, head_stride,
                                  (const int*)seq_lens, out, out_stride, (float*)part_o, (float*)part_ml, B, Hq, Hk,
                                  n_splits, t_max, scale, window, stream);
  return -4;
}
