// Fused next-token sampler: temperature, top-k, top-p and the categorical draw in one launch.
//
// One CTA per row of logits [B, V].  Nothing is sorted and no probability vector is written:
//   * top-k: radix select (4 passes of 8 bits over order-preserving keys) finds the k-th largest
//     scaled logit; everything >= it is kept (ties are kept, like a `logits < kth` mask);
//   * top-p: an element is in the nucleus iff the mass of strictly larger elements is <= top_p (the
//     usual shifted rule).  The kernel draws from the candidates, tests that condition for the draw
//     with one summation pass, and on failure discards everything at or below the draw and repeats
//     (rejection sampling; the accepted draw is an exact sample of the renormalised nucleus);
//   * the draw is arg max (z_i + Gumbel_i) over the kept set, which is an exact sample from
//     softmax(z) restricted to that set; the noise is a counter-based hash of (seed, offset, row, i).
// With neither top-k nor top-p the whole thing is a single pass over the row.
#include "common.cuh"

namespace ob {
namespace sampler {

constexpr int THREADS = 1024;

__device__ __forceinline__ uint32_t f2key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint32_t hash32(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL;
  x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL;
  x ^= x >> 33;
  return (uint32_t)x;
}

__device__ __forceinline__ float gumbel(uint64_t seed, uint64_t offset, int row, int i) {
  const uint64_t ctr = (seed * 0x9E3779B97F4A7C15ULL) ^ (offset * 0xD1B54A32D192ED03ULL) ^
                       ((uint64_t)(uint32_t)row << 32) ^ (uint32_t)i;
  const float u = ((float)(hash32(ctr) >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
  return -__logf(-__logf(u));
}

template <typename T> __device__ __forceinline__ float ldz(const T* p, int i);
template <> __device__ __forceinline__ float ldz<float>(const float* p, int i) { return p[i]; }
template <> __device__ __forceinline__ float ldz<__nv_bfloat16>(const __nv_bfloat16* p, int i) { return __bfloat162float(p[i]); }

struct ArgMax { float v; int i; };

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i && b.i >= 0)) return b;
  return a;
}

__device__ ArgMax block_argmax(ArgMax x, ArgMax* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  if (warp == 0) {
    ArgMax y = lane < THREADS / 32 ? scratch[lane] : ArgMax{-INFINITY, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax z;
      z.v = __shfl_xor_sync(0xffffffffu, y.v, o);
      z.i = __shfl_xor_sync(0xffffffffu, y.i, o);
      y = better(y, z);
    }
    if (lane == 0) scratch[0] = y;
  }
  __syncthreads();
  return scratch[0];
}

__device__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < THREADS / 32; ++w) t += scratch[w];   // same order in every thread
  return t;
}

__device__ float block_max(float v, float* scratch) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = scratch[0];
  for (int w = 1; w < THREADS / 32; ++w) t = fmaxf(t, scratch[w]);
  return t;
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
sample_kernel(const T* __restrict__ logits, long long row_stride, int V, float inv_temp, int top_k, float top_p,
              int greedy, unsigned long long seed, unsigned long long offset, long long* __restrict__ out) {
  __shared__ ArgMax scratch[THREADS / 32];
  __shared__ uint32_t hist_n[256];
  __shared__ uint32_t s_prefix, s_k;
  __shared__ float s_fscratch[THREADS / 32];
  const int row = blockIdx.x, tid = threadIdx.x;
  const T* z_row = logits + (long long)row * row_stride;

  if (greedy) {
    ArgMax best{-INFINITY, -1};
    for (int i = tid; i < V; i += THREADS) best = better(best, ArgMax{ldz(z_row, i), i});
    best = block_argmax(best, scratch);
    if (tid == 0) out[row] = best.i;
    return;
  }
  uint32_t thr_key = 0;  // keep elements with key >= thr_key
  const bool use_k = top_k > 0 && top_k < V;
  const bool use_p = top_p > 0.f && top_p < 1.f;
  if (use_k) {
    uint32_t prefix = 0, mask = 0;
    uint32_t k_left = (uint32_t)top_k;
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int i = tid; i < 256; i += THREADS) hist_n[i] = 0;
      __syncthreads();
      for (int i = tid; i < V; i += THREADS) {
        const uint32_t key = f2key(ldz(z_row, i) * inv_temp);
        if ((key & mask) == prefix) atomicAdd(&hist_n[(key >> shift) & 0xFF], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        uint32_t cum = 0;
        int bin = 255;
        for (; bin > 0; --bin) {
          if (cum + hist_n[bin] >= k_left) break;
          cum += hist_n[bin];
        }
        s_prefix = prefix | ((uint32_t)bin << shift);
        s_k = k_left - cum;
      }
      __syncthreads();
      prefix = s_prefix;
      k_left = s_k;
      mask |= 0xFFu << shift;
    }
    thr_key = prefix;
  }
  if (use_p) {
    // Nucleus sampling by rejection: draw from the current candidates; the draw is inside the nucleus iff
    // the probability mass of strictly larger candidates is at most top_p.  Otherwise everything at or
    // below the draw lies outside the nucleus (the nucleus is closed upwards), is removed, and we draw
    // again.  Every round is two plain passes over the row; no sorting, no histogram.
    float mx = -INFINITY;
    for (int i = tid; i < V; i += THREADS) mx = fmaxf(mx, ldz(z_row, i) * inv_temp);
    mx = block_max(mx, s_fscratch);
    float zsum = 0.f;
    for (int i = tid; i < V; i += THREADS) {
      const float z = ldz(z_row, i) * inv_temp;
      if (f2key(z) >= thr_key) zsum += __expf(z - mx);
    }
    zsum = block_sum(zsum, s_fscratch);
    const float target = top_p * zsum;
    float low = -INFINITY;   // candidates must have z > low
    int chosen = -1;
    for (int round = 0; round < 32 && chosen < 0; ++round) {
      ArgMax cand{-INFINITY, -1};
      for (int i = tid; i < V; i += THREADS) {
        const float z = ldz(z_row, i) * inv_temp;
        if (f2key(z) >= thr_key && z > low)
          cand = better(cand, ArgMax{z + gumbel(seed + 0x632BE59BD9B4E019ULL * (round + 1), offset, row, i), i});
      }
      cand = block_argmax(cand, scratch);
      if (cand.i < 0) break;
      const float zj = ldz(z_row, cand.i) * inv_temp;
      float above = 0.f;
      for (int i = tid; i < V; i += THREADS) {
        const float z = ldz(z_row, i) * inv_temp;
        if (f2key(z) >= thr_key && z > zj) above += __expf(z - mx);
      }
      above = block_sum(above, s_fscratch);
      if (above <= target) chosen = cand.i;
      else low = zj;
    }
    if (chosen < 0) {   // numerically empty candidate set: fall back to the most likely candidate
      ArgMax top{-INFINITY, -1};
      for (int i = tid; i < V; i += THREADS) {
        const float z = ldz(z_row, i) * inv_temp;
        if (f2key(z) >= thr_key) top = better(top, ArgMax{z, i});
      }
      chosen = block_argmax(top, scratch).i;
    }
    if (tid == 0) out[row] = chosen;
    return;
  }
  ArgMax best{-INFINITY, -1};
  for (int i = tid; i < V; i += THREADS) {
    const float z = ldz(z_row, i) * inv_temp;
    if (f2key(z) >= thr_key) best = better(best, ArgMax{z + gumbel(seed, offset, row, i), i});
  }
  best = block_argmax(best, scratch);
  if (tid == 0) out[row] = best.i;
}

}  // namespace sampler
}  // namespace ob

// logits: [B, V] fp32 (is_bf16 = 0) or bf16 (is_bf16 = 1) with the given row stride (elements);
// out: int64 [B].  temperature <= 0 or greedy != 0 gives arg max.  `offset` should advance by
// one per call so that successive steps draw independent noise from the same seed.
extern "C" int ob_sample(const void* logits, int is_bf16, long long row_stride, int B, int V, float temperature,
                         int top_k, float top_p, int greedy, unsigned long long seed, unsigned long long offset,
                         void* out, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (V <= 0) return -1;
  if (temperature <= 0.f) greedy = 1;
  const float inv_temp = greedy ? 1.0f : 1.0f / temperature;
  using namespace ob::sampler;
  if (is_bf16)
    sample_kernel<__nv_bfloat16><<<B, THREADS, 0, stream>>>((const __nv_bfloat16*)logits, row_stride, V, inv_temp,
                                                            top_k, top_p, greedy, seed, offset, (long long*)out);
  else
    sample_kernel<float><<<B, THREADS, 0, stream>>>((const float*)logits, row_stride, V, inv_temp, top_k, top_p, greedy,
                                                    seed, offset, (long long*)out);
  return (int)cudaGetLastError();
}
