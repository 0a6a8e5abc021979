// Single-query ("decode") attention against a key/value cache, with the cache append fused in.
//
//   q        [B, Hq, HD]     bf16, row stride q_stride (it usually lives inside the fused qkv row)
//   k_new    [B, Hk, HD]     bf16, the current token's key (already normalised / rotated); v_new alike
//   k_cache  logical [B, Tmax, Hk, HD] bf16 with arbitrary batch / token / head strides (v_cache alike;
//            a head-major allocation gives every CTA one contiguous stream); sequence b holds seq_lens[b] tokens *including*
//            the current one, whose row (seq_lens[b] - 1) this kernel writes before it attends
//   out      [B, Hq, HD]     bf16
//
// The kernel is bound by the cache read: one CTA per (kv head, sequence, split of the sequence) streams 64-token
// K and V tiles through shared memory with cp.async double buffering; all query heads that share the kv head (GQA
// group, up to 8) are served from the same tile as the rows of small tensor-core products, so the instruction count
// per cached byte stays low.  With more than one split the partial (max, sum, accumulator) triples are merged by a
// second small kernel.
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

// Shared memory: K and V tiles with rows padded by 16 bytes (conflict-free ldmatrix), the query group as a
// 16-row bf16 matrix (rows beyond the group are zero), and after the main loop the per-warp partial results.
template <int HD>
struct Smem {
  static constexpr int PAD = HD + 8;
  __nv_bfloat16 k[2][TILE][PAD];
  __nv_bfloat16 v[2][TILE][PAD];
  __nv_bfloat16 q[16][PAD];
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
    } else {
      // rows past the end must be finite: their probabilities are zero, but 0 * NaN would poison the sums
      *reinterpret_cast<uint4*>(&sm.k[buf][r][c * 8]) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(&sm.v[buf][r][c * 8]) = make_uint4(0, 0, 0, 0);
    }
  }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
// D (16x8, fp32) += A (16x16, bf16, row) * B (16x8, bf16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The GQA group (up to 8 query heads that share this kv head) is the M dimension of small tensor-core products
// (legacy mma.sync: the tiles are far too small for tcgen05 and the kernel is bound by the cache stream, not by
// math).  Each of the four warps owns 16 of the 64 positions of a tile and keeps its own running maximum, sum and
// 16 x HD output accumulator, so no cross-warp step happens per tile; the four partial results are merged once at
// the end, like split partials.
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
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
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
  // query group -> 16 x HD bf16 matrix in shared memory (zero rows beyond the group)
  for (int i = tid; i < 16 * (HD / 8); i += THREADS) {
    const int r = i / (HD / 8), c = i - r * (HD / 8);
    uint4 val = make_uint4(0, 0, 0, 0);
    if (r < n_rep) val = *reinterpret_cast<const uint4*>(q + (long long)b * q_stride + (long long)(hk * n_rep + r) * HD + c * 8);
    *reinterpret_cast<uint4*>(&sm.q[r][c * 8]) = val;
  }
  __syncthreads();  // also orders the appended row before the cp.async reads below

  // A fragments of Q for every 16-wide k-step, kept in registers for the whole kernel
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int s = 0; s < HD / 16; ++s)
    ldmatrix_x4(qf[s], &sm.q[(lane & 7) + ((lane >> 3) & 1) * 8][s * 16 + (lane >> 4) * 8]);

  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows lane/4 and lane/4 + 8

  const int n_tiles = t0 < t1 ? (t1 - t0 + TILE - 1) / TILE : 0;
  if (n_tiles > 0) load_tile<HD>(sm, 0, kc, vc, tok_stride, t0, t1);
  cp_async_commit();
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < n_tiles) load_tile<HD>(sm, buf ^ 1, kc, vc, tok_stride, t0 + (tile + 1) * TILE, t1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int p0 = warp * 16;                                   // this warp's positions inside the tile
    const int valid = t1 - (t0 + tile * TILE);                  // positions of the tile that exist
    if (p0 < valid) {
      // S = Q K^T for 16 positions: two 16x8 accumulators
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < HD / 16; ++s) {
        uint32_t kf[4];
        ldmatrix_x4(kf, &sm.k[buf][p0 + (lane & 7) + (lane >> 4) * 8][s * 16 + ((lane >> 3) & 1) * 8]);
        mma_16816(s0, qf[s], kf[0], kf[1]);
        mma_16816(s1, qf[s], kf[2], kf[3]);
      }
      // scale, mask the tail, online softmax per row (rows r = lane/4 and r + 8; 4 columns each per thread)
      const int c0 = p0 + 2 * (lane & 3);
      float e[8] = {s0[0], s0[1], s1[0], s1[1], s0[2], s0[3], s1[2], s1[3]};   // row r: e[0..3], row r+8: e[4..7]
      const int cols[4] = {c0, c0 + 1, c0 + 8, c0 + 9};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool okc = cols[i] < valid;
        e[i] = okc ? e[i] * scale_log2 : -INFINITY;
        e[4 + i] = okc ? e[4 + i] * scale_log2 : -INFINITY;
      }
      float mx0 = fmaxf(fmaxf(e[0], e[1]), fmaxf(e[2], e[3])), mx1 = fmaxf(fmaxf(e[4], e[5]), fmaxf(e[6], e[7]));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);     // finite: position p0 of this warp exists
      const float a0 = exp2f(m0 - n0), a1 = exp2f(m1 - n1);
      m0 = n0; m1 = n1;
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        e[i] = exp2f(e[i] - n0); sum0 += e[i];
        e[4 + i] = exp2f(e[4 + i] - n1); sum1 += e[4 + i];
      }
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
      l0 = l0 * a0 + sum0;
      l1 = l1 * a1 + sum1;
      // P as the A fragment of the second product (accumulator layout of two n-tiles = A layout of one k-step)
      uint32_t pf[4];
      pf[0] = pack_bf16x2(e[0], e[1]);   // row r,     k 0..7 part
      pf[1] = pack_bf16x2(e[4], e[5]);   // row r + 8, k 0..7 part
      pf[2] = pack_bf16x2(e[2], e[3]);   // row r,     k 8..15 part
      pf[3] = pack_bf16x2(e[6], e[7]);   // row r + 8, k 8..15 part
#pragma unroll
      for (int j = 0; j < HD / 16; ++j) {
        o[2 * j][0] *= a0; o[2 * j][1] *= a0; o[2 * j][2] *= a1; o[2 * j][3] *= a1;
        o[2 * j + 1][0] *= a0; o[2 * j + 1][1] *= a0; o[2 * j + 1][2] *= a1; o[2 * j + 1][3] *= a1;
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, &sm.v[buf][p0 + (lane & 7) + ((lane >> 3) & 1) * 8][j * 16 + (lane >> 4) * 8]);
        mma_16816(o[2 * j], pf, vf[0], vf[1]);
        mma_16816(o[2 * j + 1], pf, vf[2], vf[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // merge the four warps (fixed order).  The K/V tile memory is free now and holds the partials:
  //   po[warp][row][HD] fp32, pm[warp][row], pl[warp][row]
  float* po = reinterpret_cast<float*>(smem_raw);
  float* pm = po + 4 * 16 * HD;
  float* pl = pm + 4 * 16;
  const int r0 = lane >> 2, cq = 2 * (lane & 3);
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) {
    float* base0 = po + (warp * 16 + r0) * HD + j * 8 + cq;
    float* base1 = po + (warp * 16 + r0 + 8) * HD + j * 8 + cq;
    base0[0] = o[j][0]; base0[1] = o[j][1];
    base1[0] = o[j][2]; base1[1] = o[j][3];
  }
  if ((lane & 3) == 0) {
    pm[warp * 16 + r0] = m0; pl[warp * 16 + r0] = l0;
    pm[warp * 16 + r0 + 8] = m1; pl[warp * 16 + r0 + 8] = l1;
  }
  __syncthreads();
  for (int i = tid; i < n_rep * HD; i += THREADS) {
    const int r = i / HD, d = i - r * HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, pm[w * 16 + r]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = pm[w * 16 + r];
      if (mw == -INFINITY) continue;
      const float f = exp2f(mw - mm);
      num += f * po[(w * 16 + r) * HD + d];
      den += f * pl[w * 16 + r];
    }
    const int hq = hk * n_rep + r;
    if (n_splits == 1) {
      out[(long long)b * out_stride + (long long)hq * HD + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
    } else {
      const long long slot = ((long long)b * Hq + hq) * n_splits + split;
      part_o[slot * HD + d] = num;
      if (d == 0) { part_ml[slot * 2] = mm; part_ml[slot * 2 + 1] = den; }
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
