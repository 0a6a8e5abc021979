// Bandwidth-bound helpers: SwiGLU (elementwise form), fused AdamW over flat shards,
// sum of squares for the gradient norm, embedding gather / scatter-add.
// All loops are grid-stride with 128-bit accesses; tails are handled element-wise.
#include "common.cuh"

namespace ob {
namespace ew {

// fast reciprocal: the results are rounded to bf16, an IEEE division would only cost issue slots
__device__ __forceinline__ float sigmoidf_(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// h = silu(g) * u
__global__ void swiglu_fwd_kernel(const uint4* __restrict__ g, const uint4* __restrict__ u, uint4* __restrict__ h,
                                  long long nvec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    uint4 a = g[i], b = u[i], o;
    uint32_t* ap = &a.x; uint32_t* bp = &b.x; uint32_t* op = &o.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 gv = unpack_bf16x2(ap[j]), uv = unpack_bf16x2(bp[j]);
      op[j] = pack_bf16x2(gv.x * sigmoidf_(gv.x) * uv.x, gv.y * sigmoidf_(gv.y) * uv.y);
    }
    h[i] = o;
  }
}

// dg = dh * u * s(g) * (1 + g (1 - s(g))), du = dh * silu(g); optionally recomputes h.
// dg/du may alias g/u (in-place).
__global__ void swiglu_bwd_kernel(const uint4* __restrict__ dh, const uint4* g, const uint4* u, uint4* dg, uint4* du,
                                  uint4* __restrict__ h_out, long long nvec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    uint4 a = g[i], b = u[i], d = dh[i], og, ou, oh;
    uint32_t* ap = &a.x; uint32_t* bp = &b.x; uint32_t* dp = &d.x;
    uint32_t* ogp = &og.x; uint32_t* oup = &ou.x; uint32_t* ohp = &oh.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 gv = unpack_bf16x2(ap[j]), uv = unpack_bf16x2(bp[j]), dv = unpack_bf16x2(dp[j]);
      float s0 = sigmoidf_(gv.x), s1 = sigmoidf_(gv.y);
      float si0 = gv.x * s0, si1 = gv.y * s1;
      ogp[j] = pack_bf16x2(dv.x * uv.x * s0 * (1.0f + gv.x * (1.0f - s0)), dv.y * uv.y * s1 * (1.0f + gv.y * (1.0f - s1)));
      oup[j] = pack_bf16x2(dv.x * si0, dv.y * si1);
      ohp[j] = pack_bf16x2(si0 * uv.x, si1 * uv.y);
    }
    dg[i] = og;
    du[i] = ou;
    if (h_out) h_out[i] = oh;
  }
}

// Fused AdamW on a flat shard.  master/m/v are fp32; grad is bf16 or fp32; the updated
// parameter is also written in bf16 (the copy that forward/backward read).
//   g_eff = grad * grad_scale * clip,   clip = min(1, max_norm / (sqrt(*sumsq * norm_scale) + 1e-6))
// when sumsq != nullptr (the squared global gradient norm, accumulated on the device).
template <typename GradT>
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             const GradT* __restrict__ grad, __nv_bfloat16* __restrict__ param_bf16, long long n,
                             float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                             float grad_scale, const float* __restrict__ sumsq, float max_norm) {
  float scale = grad_scale;
  if (sumsq) {
    const float norm = sqrtf(*sumsq) * grad_scale;
    const float clip = fminf(1.0f, max_norm / (norm + 1e-6f));
    scale *= clip;
  }
  const float step = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const float decay = 1.0f - lr * wd;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float g;
    if constexpr (sizeof(GradT) == 2) g = __bfloat162float(grad[i]); else g = grad[i];
    g *= scale;
    float p = master[i] * decay;
    const float mi = beta1 * m[i] + (1.0f - beta1) * g;
    const float vi = beta2 * v[i] + (1.0f - beta2) * g * g;
    const float denom = sqrtf(vi) * inv_sqrt_bc2 + eps;
    p -= step * mi / denom;
    master[i] = p; m[i] = mi; v[i] = vi;
    if (param_bf16) param_bf16[i] = __float2bfloat16(p);
  }
}

// Deterministic sum of squares: per-block partials, the last block adds them in order.
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, long long n, float* __restrict__ partials,
                             unsigned int* __restrict__ counter, float* __restrict__ out, int accumulate) {
  __shared__ float red[32];
  __shared__ bool last;
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v;
    if constexpr (sizeof(T) == 2) v = __bfloat162float(x[i]); else v = x[i];
    s += v * v;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) {
      partials[blockIdx.x] = t;
      __threadfence();
      unsigned int done = atomicAdd(counter, 1u);
      last = (done == gridDim.x - 1);
    }
  }
  __syncthreads();
  if (last && threadIdx.x == 0) {
    __threadfence();
    float t = 0.f;
    for (unsigned int b = 0; b < gridDim.x; ++b) t += reinterpret_cast<volatile float*>(partials)[b];
    *out = accumulate ? *out + t : t;
    *counter = 0;
  }
}

// out[t, :] = table[ids[t], :]
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long T, int D, int V) {
  const int nvec = D / 8;
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    long long id = ids[t];
    if (id < 0 || id >= V) id = 0;
    const uint4* src = reinterpret_cast<const uint4*>(table + id * D);
    uint4* dst = reinterpret_cast<uint4*>(out + t * D);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = src[i];
  }
}

// dtable[id, :] (+)= sum over the tokens with that id of dout[token, :].
// `sorted_ids` is ascending and `perm[i]` is the token index of sorted position i, so the
// rows of one id are added by one CTA in a fixed order (bitwise reproducible, no atomics).
__global__ void embedding_bwd_kernel(const long long* __restrict__ sorted_ids, const long long* __restrict__ perm,
                                     const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dtable,
                                     long long T, int D, int V, int pad_id, int accumulate) {
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    const long long id = sorted_ids[t];
    if (id < 0 || id >= V || id == pad_id) continue;
    if (t > 0 && sorted_ids[t - 1] == id) continue;  // not the first row of its segment
    long long end = t + 1;
    while (end < T && sorted_ids[end] == id) ++end;
    __nv_bfloat16* dst = dtable + id * D;
    for (int i = threadIdx.x * 2; i < D; i += blockDim.x * 2) {
      float2 acc = accumulate ? unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dst + i)) : make_float2(0.f, 0.f);
      for (long long r = t; r < end; ++r) {
        float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dout + perm[r] * D + i));
        acc.x += v.x; acc.y += v.y;
      }
      *reinterpret_cast<uint32_t*>(dst + i) = pack_bf16x2(acc.x, acc.y);
    }
  }
}

// bf16 <-> fp32 flat helpers with scale (used when folding fp32 side buffers into bf16 gradients)
__global__ void add_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n,
                                       int accumulate) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16(accumulate ? __bfloat162float(dst[i]) + src[i] : src[i]);
}

}  // namespace ew
}  // namespace ob

using namespace ob::ew;

static int ew_grid(long long n, int threads) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long need = (n + threads - 1) / threads;
  long long cap = (long long)sms * 16;
  return (int)(need < cap ? (need > 0 ? need : 1) : cap);
}

extern "C" int ob_swiglu_fwd(const void* g, const void* u, void* h, long long n, cudaStream_t stream) {
  if (n % 8) return -1;
  if (n == 0) return 0;
  swiglu_fwd_kernel<<<ew_grid(n / 8, 256), 256, 0, stream>>>((const uint4*)g, (const uint4*)u, (uint4*)h, n / 8);
  return (int)cudaGetLastError();
}

extern "C" int ob_swiglu_bwd(const void* dh, const void* g, const void* u, void* dg, void* du, void* h_out, long long n,
                             cudaStream_t stream) {
  if (n % 8) return -1;
  if (n == 0) return 0;
  swiglu_bwd_kernel<<<ew_grid(n / 8, 256), 256, 0, stream>>>((const uint4*)dh, (const uint4*)g, (const uint4*)u,
                                                             (uint4*)dg, (uint4*)du, (uint4*)h_out, n / 8);
  return (int)cudaGetLastError();
}

extern "C" int ob_adamw(void* master, void* m, void* v, const void* grad, int grad_is_fp32, void* param_bf16,
                        long long n, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                        float grad_scale, const void* sumsq, float max_norm, cudaStream_t stream) {
  if (n == 0) return 0;
  const int grid = ew_grid(n, 256);
  if (grad_is_fp32)
    adamw_kernel<float><<<grid, 256, 0, stream>>>((float*)master, (float*)m, (float*)v, (const float*)grad,
                                                  (__nv_bfloat16*)param_bf16, n, lr, beta1, beta2, eps, wd, bc1, bc2,
                                                  grad_scale, (const float*)sumsq, max_norm);
  else
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((float*)master, (float*)m, (float*)v,
                                                          (const __nv_bfloat16*)grad, (__nv_bfloat16*)param_bf16, n, lr,
                                                          beta1, beta2, eps, wd, bc1, bc2, grad_scale,
                                                          (const float*)sumsq, max_norm);
  return (int)cudaGetLastError();
}

// scratch: at least 1024 floats followed by one zero-initialised uint32 counter (4100 bytes).
extern "C" int ob_sumsq(const void* x, long long n, int is_fp32, void* scratch, void* out, int accumulate,
                        cudaStream_t stream) {
  int grid = ew_grid(n, 256);
  if (grid > 1024) grid = 1024;
  float* partials = (float*)scratch;
  unsigned int* counter = (unsigned int*)(partials + 1024);
  if (is_fp32)
    sumsq_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, n, partials, counter, (float*)out, accumulate);
  else
    sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, n, partials, counter, (float*)out,
                                                          accumulate);
  return (int)cudaGetLastError();
}

extern "C" int ob_embedding_fwd(const void* ids, const void* table, void* out, long long T, int D, int V,
                                cudaStream_t stream) {
  if (D % 8) return -1;
  if (T == 0) return 0;
  int grid = T < 148 * 16 ? (int)T : 148 * 16;
  embedding_fwd_kernel<<<grid, 128, 0, stream>>>((const long long*)ids, (const __nv_bfloat16*)table,
                                                 (__nv_bfloat16*)out, T, D, V);
  return (int)cudaGetLastError();
}

extern "C" int ob_embedding_bwd(const void* sorted_ids, const void* perm, const void* dout, void* dtable, long long T,
                                int D, int V, int pad_id, int accumulate, cudaStream_t stream) {
  if (D % 2) return -1;
  if (T == 0) return 0;
  int grid = T < 148 * 16 ? (int)T : 148 * 16;
  embedding_bwd_kernel<<<grid, 256, 0, stream>>>((const long long*)sorted_ids, (const long long*)perm,
                                                 (const __nv_bfloat16*)dout, (__nv_bfloat16*)dtable, T, D, V, pad_id,
                                                 accumulate);
  return (int)cudaGetLastError();
}

extern "C" int ob_add_f32_to_bf16(const void* src, void* dst, long long n, int accumulate, cudaStream_t stream) {
  if (n == 0) return 0;
  add_f32_to_bf16_kernel<<<ew_grid(n, 256), 256, 0, stream>>>((const float*)src, (__nv_bfloat16*)dst, n, accumulate);
  return (int)cudaGetLastError();
}
