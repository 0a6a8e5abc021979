// Cross-entropy over a chunk of bf16 logits [rows, V_local] (row stride ld), in two kernels
// so that a vocabulary-sharded (tensor-parallel) loss can exchange per-row statistics
// between them:
//   ce_stats : per row, over this rank's vocabulary slice: max, sum exp(z - max), sum z,
//              z[target] (when the target falls in the slice), arg max.
//   ce_grad  : given the global log-sum-exp of each row, overwrite the logits in place with
//              d loss / d logits = (softmax - (1-s) onehot - s/V) * scale * softcap'(z).
// Supports ignore_index, label smoothing s and two soft-capping forms applied to the raw
// logits first: z = c tanh(x / c) and z = 23 sigmoid((x + 5) / 7.5).
// The caller produces the chunk with the GEMM (x_chunk @ W^T) and feeds the in-place
// gradient to two more GEMMs (dX and dW), so full [tokens, vocab] logits never exist.
// Semantics follow optimus_dl/modules/criterion/cross_entropy.py:191-267.
#include "common.cuh"

namespace ob {
namespace ce {

constexpr int THREADS = 256;
enum Softcap : int { kNone = 0, kTanh = 1, kSigmoid = 2 };

__device__ __forceinline__ float cap(float x, int mode, float c) {
  if (mode == kTanh) return c * tanhf(x / c);
  if (mode == kSigmoid) return 23.0f / (1.0f + __expf(-(x + 5.0f) / 7.5f));
  return x;
}
__device__ __forceinline__ float cap_grad(float x, int mode, float c) {
  if (mode == kTanh) { float t = tanhf(x / c); return 1.0f - t * t; }
  if (mode == kSigmoid) { float s = 1.0f / (1.0f + __expf(-(x + 5.0f) / 7.5f)); return 23.0f / 7.5f * s * (1.0f - s); }
  return 1.0f;
}

struct Stat {
  float m, s, sum, best;
  int best_idx;
};
__device__ __forceinline__ void stat_add(Stat& st, float z, int idx) {
  if (z > st.m) { st.s = st.s * __expf(st.m - z) + 1.0f; st.m = z; } else { st.s += __expf(z - st.m); }
  st.sum += z;
  if (z > st.best) { st.best = z; st.best_idx = idx; }
}
__device__ __forceinline__ void stat_merge(Stat& a, const Stat& b) {
  const float m = fmaxf(a.m, b.m);
  const float sa = (a.m == -INFINITY) ? 0.f : a.s * __expf(a.m - m);
  const float sb = (b.m == -INFINITY) ? 0.f : b.s * __expf(b.m - m);
  a.s = sa + sb; a.m = m; a.sum += b.sum;
  if (b.best > a.best || (b.best == a.best && b.best_idx < a.best_idx)) { a.best = b.best; a.best_idx = b.best_idx; }
}

__global__ void __launch_bounds__(THREADS)
ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, const long long* __restrict__ targets,
                float* __restrict__ row_max, float* __restrict__ row_sumexp, float* __restrict__ row_sum,
                float* __restrict__ row_tgt, float* __restrict__ row_best, int* __restrict__ row_best_idx, int rows,
                int V, int vocab_offset, int softcap, float cap_c) {
  __shared__ Stat red[THREADS / 32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* z = logits + (long long)row * ld;
    Stat st{-INFINITY, 0.f, 0.f, -INFINITY, 0x7fffffff};
    const bool vec = (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
    const int nv = vec ? V / 8 : 0;
    for (int i = threadIdx.x; i < nv; i += THREADS) {
      uint4 u = reinterpret_cast<const uint4*>(z)[i];
      uint32_t* p = &u.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(p[j]);
        stat_add(st, cap(f.x, softcap, cap_c), i * 8 + 2 * j);
        stat_add(st, cap(f.y, softcap, cap_c), i * 8 + 2 * j + 1);
      }
    }
    for (int i = nv * 8 + threadIdx.x; i < V; i += THREADS) stat_add(st, cap(__bfloat162float(z[i]), softcap, cap_c), i);
    // warp then block merge
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Stat other;
      other.m = __shfl_xor_sync(0xffffffffu, st.m, o);
      other.s = __shfl_xor_sync(0xffffffffu, st.s, o);
      other.sum = __shfl_xor_sync(0xffffffffu, st.sum, o);
      other.best = __shfl_xor_sync(0xffffffffu, st.best, o);
      other.best_idx = __shfl_xor_sync(0xffffffffu, st.best_idx, o);
      stat_merge(st, other);
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = st;
    __syncthreads();
    if (threadIdx.x == 0) {
      Stat t = red[0];
      for (int w = 1; w < THREADS / 32; ++w) stat_merge(t, red[w]);
      row_max[row] = t.m;
      row_sumexp[row] = t.s;
      row_sum[row] = t.sum;
      row_best[row] = t.best;
      row_best_idx[row] = t.best_idx + vocab_offset;
      const long long y = targets[row] - vocab_offset;
      row_tgt[row] = (y >= 0 && y < V) ? cap(__bfloat162float(z[y]), softcap, cap_c) : 0.f;
    }
  }
}

__global__ void __launch_bounds__(THREADS)
ce_grad_kernel(__nv_bfloat16* __restrict__ logits, long long ld, const long long* __restrict__ targets,
               const float* __restrict__ row_lse, int rows, int V, int vocab_offset, int total_vocab,
               long long ignore_index, float smoothing, const float* __restrict__ scale_ptr, float scale_mul,
               int softcap, float cap_c, const float* __restrict__ row_weight) {
  const float scale0 = (scale_ptr ? *scale_ptr : 1.0f) * scale_mul;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float scale = row_weight ? scale0 * row_weight[row] : scale0;
    __nv_bfloat16* z = logits + (long long)row * ld;
    const long long tgt = targets[row];
    const bool ignored = (tgt == ignore_index);
    const long long y = tgt - vocab_offset;
    const float lse = row_lse[row];
    const float uni = smoothing / total_vocab;
    const bool vec = (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
    const int nv = vec ? V / 8 : 0;
    for (int i = threadIdx.x; i < nv; i += THREADS) {
      uint4 u = reinterpret_cast<uint4*>(z)[i];
      uint32_t* p = &u.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(p[j]);
        float o[2];
        float raw[2] = {f.x, f.y};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int idx = i * 8 + 2 * j + e;
          const float zc = cap(raw[e], softcap, cap_c);
          float g = __expf(zc - lse) - uni - ((idx == y) ? (1.0f - smoothing) : 0.f);
          g *= scale * cap_grad(raw[e], softcap, cap_c);
          o[e] = ignored ? 0.f : g;
        }
        p[j] = pack_bf16x2(o[0], o[1]);
      }
      reinterpret_cast<uint4*>(z)[i] = u;
    }
    for (int i = nv * 8 + threadIdx.x; i < V; i += THREADS) {
      const float raw = __bfloat162float(z[i]);
      const float zc = cap(raw, softcap, cap_c);
      float g = __expf(zc - lse) - uni - ((i == y) ? (1.0f - smoothing) : 0.f);
      g *= scale * cap_grad(raw, softcap, cap_c);
      z[i] = __float2bfloat16(ignored ? 0.f : g);
    }
  }
}

// Folds the per-tile statistics of the fused "linear + statistics" product (gemm::Params::ce_part: one float4 and one
// column index per row and 256-column tile, a row's tiles contiguous) into the same per-row outputs as
// ce_stats_kernel.  One warp per row; equal maxima keep the lowest column.
__global__ void __launch_bounds__(THREADS)
ce_stats_merge_kernel(const float4* __restrict__ part, const int* __restrict__ part_idx, int rows, int tiles_n,
                      float* __restrict__ row_max, float* __restrict__ row_sumexp, float* __restrict__ row_sum,
                      float* __restrict__ row_best, int* __restrict__ row_best_idx, int vocab_offset) {
  const int row = blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  Stat st{-INFINITY, 0.f, 0.f, -INFINITY, 0x7fffffff};
  for (int t = lane; t < tiles_n; t += 32) {
    const float4 v = part[(long long)row * tiles_n + t];
    Stat o{v.x, v.y, v.z, v.w, part_idx[(long long)row * tiles_n + t]};
    stat_merge(st, o);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Stat other;
    other.m = __shfl_xor_sync(0xffffffffu, st.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, st.s, o);
    other.sum = __shfl_xor_sync(0xffffffffu, st.sum, o);
    other.best = __shfl_xor_sync(0xffffffffu, st.best, o);
    other.best_idx = __shfl_xor_sync(0xffffffffu, st.best_idx, o);
    stat_merge(st, other);
  }
  if (lane == 0) {
    row_max[row] = st.m;
    row_sumexp[row] = st.s;
    row_sum[row] = st.sum;
    row_best[row] = st.best;
    row_best_idx[row] = st.best_idx + vocab_offset;
  }
}

}  // namespace ce
}  // namespace ob

extern "C" int ob_ce_stats_merge(const void* part, const void* part_idx, int rows, int tiles_n, void* row_max,
                                 void* row_sumexp, void* row_sum, void* row_best, void* row_best_idx, int vocab_offset,
                                 cudaStream_t stream) {
  if (rows <= 0) return 0;
  constexpr int rows_per_block = ob::ce::THREADS / 32;
  ob::ce::ce_stats_merge_kernel<<<(rows + rows_per_block - 1) / rows_per_block, ob::ce::THREADS, 0, stream>>>(
      (const float4*)part, (const int*)part_idx, rows, tiles_n, (float*)row_max, (float*)row_sumexp, (float*)row_sum,
      (float*)row_best, (int*)row_best_idx, vocab_offset);
  return (int)cudaGetLastError();
}


using namespace ob::ce;

extern "C" int ob_ce_stats(const void* logits, long long ld, const void* targets, void* row_max, void* row_sumexp,
                           void* row_sum, void* row_tgt, void* row_best, void* row_best_idx, int rows, int V,
                           int vocab_offset, int softcap, float cap_c, cudaStream_t stream) {
  if (rows == 0) return 0;
  ce_stats_kernel<<<rows, THREADS, 0, stream>>>((const __nv_bfloat16*)logits, ld, (const long long*)targets,
                                                (float*)row_max, (float*)row_sumexp, (float*)row_sum, (float*)row_tgt,
                                                (float*)row_best, (int*)row_best_idx, rows, V, vocab_offset, softcap,
                                                cap_c);
  return (int)cudaGetLastError();
}

extern "C" int ob_ce_grad(void* logits, long long ld, const void* targets, const void* row_lse, int rows, int V,
                          int vocab_offset, int total_vocab, long long ignore_index, float smoothing,
                          const void* scale_ptr, float scale_mul, int softcap, float cap_c, const void* row_weight,
                          cudaStream_t stream) {
  if (rows == 0) return 0;
  ce_grad_kernel<<<rows, THREADS, 0, stream>>>((__nv_bfloat16*)logits, ld, (const long long*)targets,
                                               (const float*)row_lse, rows, V, vocab_offset, total_vocab, ignore_index,
                                               smoothing, (const float*)scale_ptr, scale_mul, softcap, cap_c,
                                               (const float*)row_weight);
  return (int)cudaGetLastError();
}
