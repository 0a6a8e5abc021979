// RMSNorm and LayerNorm, forward and backward, for bf16 activations with fp32 math.
//
// One CTA of 256 threads handles one row at a time; each thread keeps its slice of the
// row in registers (D <= 8192, D % 8 == 0), so x is read from HBM once per pass.
//   forward : y = x_hat * w (+ b),  x_hat = (x - mean) * rstd   (mean = 0 for RMSNorm)
//             optional fused residual add: h = x + residual is written out and normalised
//   backward: dx = rstd * (g - x_hat * mean(g * x_hat) - mean(g)),  g = dy * w
//             dw = sum_rows(dy * x_hat), db = sum_rows(dy): each CTA accumulates its rows
//             in registers, writes one partial row into a scratch buffer [grid, D], and a
//             second kernel adds the partials in a fixed order (bitwise reproducible).
// Math follows the fp32 ("gemma" casting) convention of the reference's RMSNorm
// (optimus_dl/modules/model/blocks/layer_norms.py:86-120).
#include <cuda_fp8.h>

#include "common.cuh"

namespace ob {
namespace norm {

constexpr int THREADS = 256;
constexpr int MAX_VEC = 4;  // uint4 (8 bf16) per thread per slot -> D <= 256 * 8 * 4

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}

// QUANT: besides y the kernel writes e4m3(y) with one scale per 1 x 128 block (q [rows, D], scales
// [D / 128][scale_ld]): a block is 16 consecutive threads' vectors, so its maximum is a half-warp reduction of
// values the thread already holds, and the linear layer that consumes y needs no quantiser pass.  The quantised
// values are taken from y as stored (rounded to bf16), exactly what a separate quantiser would read.  D % 128 == 0.
template <bool LAYERNORM, int NVEC, bool QUANT = false>
__global__ void __launch_bounds__(THREADS, NVEC <= 2 ? 6 : 2)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out,
                float* __restrict__ mean_out, int rows, int D, float eps, uint8_t* __restrict__ q = nullptr,
                float* __restrict__ scales = nullptr, long long scale_ld = 0) {
  __shared__ float red[THREADS / 32];
  const int nvec = D / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * D);
    const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + (size_t)row * D) : nullptr;
    float v[NVEC][8];
    float s = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int idx = threadIdx.x + i * THREADS;
      if (idx < nvec) {
        uint4 u = xr[idx];
        float2 a = unpack_bf16x2(u.x), bq = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        v[i][0] = a.x; v[i][1] = a.y; v[i][2] = bq.x; v[i][3] = bq.y; v[i][4] = c.x; v[i][5] = c.y; v[i][6] = d.x; v[i][7] = d.y;
        if (rr) {
          uint4 r = rr[idx];
          float2 ra = unpack_bf16x2(r.x), rb = unpack_bf16x2(r.y), rc = unpack_bf16x2(r.z), rd = unpack_bf16x2(r.w);
          v[i][0] += ra.x; v[i][1] += ra.y; v[i][2] += rb.x; v[i][3] += rb.y; v[i][4] += rc.x; v[i][5] += rc.y; v[i][6] += rd.x; v[i][7] += rd.y;
          // the residual stream is stored in bf16: normalise what the next layer will read
          uint4 o = make_uint4(pack_bf16x2(v[i][0], v[i][1]), pack_bf16x2(v[i][2], v[i][3]),
                               pack_bf16x2(v[i][4], v[i][5]), pack_bf16x2(v[i][6], v[i][7]));
          reinterpret_cast<uint4*>(h_out + (size_t)row * D)[idx] = o;
          float2 t0 = unpack_bf16x2(o.x), t1 = unpack_bf16x2(o.y), t2 = unpack_bf16x2(o.z), t3 = unpack_bf16x2(o.w);
          v[i][0] = t0.x; v[i][1] = t0.y; v[i][2] = t1.x; v[i][3] = t1.y; v[i][4] = t2.x; v[i][5] = t2.y; v[i][6] = t3.x; v[i][7] = t3.y;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) { s += v[i][j]; s2 += v[i][j] * v[i][j]; }
      }
    }
    float mean = 0.f;
    if (LAYERNORM) {
      mean = block_sum(s, red) / D;
      float var = 0.f;
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        const int idx = threadIdx.x + i * THREADS;
        if (idx < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) { float d = v[i][j] - mean; var += d * d; }
        }
      }
      s2 = var;
    }
    const float tot = block_sum(s2, red);
    const float rstd = rsqrtf(tot / D + eps);
    if (threadIdx.x == 0) {
      if (rstd_out) rstd_out[row] = rstd;
      if (LAYERNORM && mean_out) mean_out[row] = mean;
    }
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * D);
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int idx = threadIdx.x + i * THREADS;
      uint4 packed = make_uint4(0, 0, 0, 0);
      if (idx < nvec) {
        uint4 wu = reinterpret_cast<const uint4*>(w)[idx];
        float2 w0 = unpack_bf16x2(wu.x), w1 = unpack_bf16x2(wu.y), w2 = unpack_bf16x2(wu.z), w3 = unpack_bf16x2(wu.w);
        float ww[8] = {w0.x, w0.y, w1.x, w1.y, w2.x, w2.y, w3.x, w3.y};
        float bb[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (LAYERNORM && b) {
          uint4 bu = reinterpret_cast<const uint4*>(b)[idx];
          float2 b0 = unpack_bf16x2(bu.x), b1 = unpack_bf16x2(bu.y), b2 = unpack_bf16x2(bu.z), b3 = unpack_bf16x2(bu.w);
          bb[0] = b0.x; bb[1] = b0.y; bb[2] = b1.x; bb[3] = b1.y; bb[4] = b2.x; bb[5] = b2.y; bb[6] = b3.x; bb[7] = b3.y;
        }
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * ww[j] + bb[j];
        packed = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]),
                            pack_bf16x2(o[6], o[7]));
        yr[idx] = packed;
      }
      if (QUANT) {
        // nvec is a multiple of 16 here, so a half-warp is wholly inside or wholly outside the row; all 32 lanes
        // take part in the shuffles either way
        const float2 f0 = unpack_bf16x2(packed.x), f1 = unpack_bf16x2(packed.y), f2 = unpack_bf16x2(packed.z),
                     f3 = unpack_bf16x2(packed.w);
        float amax = fmaxf(fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f1.x), fabsf(f1.y))),
                           fmaxf(fmaxf(fabsf(f2.x), fabsf(f2.y)), fmaxf(fabsf(f3.x), fabsf(f3.y))));
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float scale = amax > 0.f ? amax / 448.0f : 1.0f;
        const float inv = 1.0f / scale;
        if (idx < nvec) {
          uint2 e;
          e.x = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(f0.x * inv, f0.y * inv), __NV_SATFINITE, __NV_E4M3) |
                ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(f1.x * inv, f1.y * inv), __NV_SATFINITE, __NV_E4M3) << 16);
          e.y = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(f2.x * inv, f2.y * inv), __NV_SATFINITE, __NV_E4M3) |
                ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(f3.x * inv, f3.y * inv), __NV_SATFINITE, __NV_E4M3) << 16);
          reinterpret_cast<uint2*>(q + (size_t)row * D)[idx] = e;
          if ((idx & 15) == 0) scales[(long long)(idx >> 4) * scale_ld + row] = scale;
        }
      }
    }
  }
}

// NVEC = uint4 slots per thread (1, 2 or 4): register arrays are sized for the row width actually used,
// which decides how many rows an SM keeps in flight.
template <bool LAYERNORM, int NVEC>
__global__ void __launch_bounds__(THREADS, NVEC <= 2 ? 3 : 1)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                const float* __restrict__ mean_in, const __nv_bfloat16* __restrict__ dres,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, float* __restrict__ db_partial,
                int rows, int D) {
  __shared__ float red[THREADS / 32];
  const int nvec = D / 8;
  float dw_acc[NVEC][8], db_acc[NVEC][8], ww[NVEC][8];
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int idx = threadIdx.x + i * THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) { dw_acc[i][j] = 0.f; db_acc[i][j] = 0.f; ww[i][j] = 0.f; }
    if (idx < nvec) {
      uint4 wu = reinterpret_cast<const uint4*>(w)[idx];
      float2 w0 = unpack_bf16x2(wu.x), w1 = unpack_bf16x2(wu.y), w2 = unpack_bf16x2(wu.z), w3 = unpack_bf16x2(wu.w);
      ww[i][0] = w0.x; ww[i][1] = w0.y; ww[i][2] = w1.x; ww[i][3] = w1.y; ww[i][4] = w2.x; ww[i][5] = w2.y; ww[i][6] = w3.x; ww[i][7] = w3.y;
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rstd = rstd_in[row];
    const float mean = LAYERNORM ? mean_in[row] : 0.f;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * D);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * D);
    float xh[NVEC][8], g[NVEC][8];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int idx = threadIdx.x + i * THREADS;
      if (idx < nvec) {
        uint4 xu = xr[idx], gu = gr[idx];
        float2 x0 = unpack_bf16x2(xu.x), x1 = unpack_bf16x2(xu.y), x2 = unpack_bf16x2(xu.z), x3 = unpack_bf16x2(xu.w);
        float2 g0 = unpack_bf16x2(gu.x), g1 = unpack_bf16x2(gu.y), g2 = unpack_bf16x2(gu.z), g3 = unpack_bf16x2(gu.w);
        float xv[8] = {x0.x, x0.y, x1.x, x1.y, x2.x, x2.y, x3.x, x3.y};
        float gv[8] = {g0.x, g0.y, g1.x, g1.y, g2.x, g2.y, g3.x, g3.y};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mean) * rstd;
          dw_acc[i][j] += gv[j] * xh[i][j];
          db_acc[i][j] += gv[j];
          g[i][j] = gv[j] * ww[i][j];
          c1 += g[i][j] * xh[i][j];
          c2 += g[i][j];
        }
      }
    }
    c1 = block_sum(c1, red) / D;
    c2 = LAYERNORM ? block_sum(c2, red) / D : 0.f;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * D);
    const uint4* drr = dres ? reinterpret_cast<const uint4*>(dres + (size_t)row * D) : nullptr;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int idx = threadIdx.x + i * THREADS;
      if (idx < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * c1 - c2);
        if (drr) {
          uint4 r = drr[idx];
          float2 r0 = unpack_bf16x2(r.x), r1 = unpack_bf16x2(r.y), r2 = unpack_bf16x2(r.z), r3 = unpack_bf16x2(r.w);
          o[0] += r0.x; o[1] += r0.y; o[2] += r1.x; o[3] += r1.y; o[4] += r2.x; o[5] += r2.y; o[6] += r3.x; o[7] += r3.y;
        }
        dxr[idx] = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]),
                              pack_bf16x2(o[6], o[7]));
      }
    }
  }
  float* dwp = dw_partial + (size_t)blockIdx.x * D;
  float* dbp = (LAYERNORM && db_partial) ? db_partial + (size_t)blockIdx.x * D : nullptr;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      reinterpret_cast<float4*>(dwp)[idx * 2] = make_float4(dw_acc[i][0], dw_acc[i][1], dw_acc[i][2], dw_acc[i][3]);
      reinterpret_cast<float4*>(dwp)[idx * 2 + 1] = make_float4(dw_acc[i][4], dw_acc[i][5], dw_acc[i][6], dw_acc[i][7]);
      if (dbp) {
        reinterpret_cast<float4*>(dbp)[idx * 2] = make_float4(db_acc[i][0], db_acc[i][1], db_acc[i][2], db_acc[i][3]);
        reinterpret_cast<float4*>(dbp)[idx * 2 + 1] = make_float4(db_acc[i][4], db_acc[i][5], db_acc[i][6], db_acc[i][7]);
      }
    }
  }
}

// out[c] (+)= sum_p partial[p, c], fixed summation order.  A CTA owns 32 columns; its 8 warps each add every
// eighth partial row (coalesced 128-byte reads), then the 8 sub-sums are added in warp order.
__global__ void __launch_bounds__(256)
reduce_partials_kernel(const float* __restrict__ partial, int nparts, int D, __nv_bfloat16* __restrict__ out_bf16,
                       float* __restrict__ out_f32, int accumulate) {
  __shared__ float sub[8][32];
  const int cg = threadIdx.x & 31, rg = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cg;
  float s = 0.f;
  if (c < D)
    for (int p = rg; p < nparts; p += 8) s += partial[(size_t)p * D + c];
  sub[rg][cg] = s;
  __syncthreads();
  if (rg == 0 && c < D) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) t += sub[r][cg];
    if (out_f32) out_f32[c] = accumulate ? out_f32[c] + t : t;
    if (out_bf16) out_bf16[c] = __float2bfloat16(accumulate ? __bfloat162float(out_bf16[c]) + t : t);
  }
}

}  // namespace norm
}  // namespace ob

using namespace ob::norm;

static int sm_count_() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}
// Resident CTAs per SM follow the launch bounds of the kernels (backward: 3, forward: 6 for rows up to 4096 wide),
// so every CTA of the grid is running and each keeps one row in flight.
static int norm_grid(int rows) {
  const int g = sm_count_() * 3;
  return rows < g ? rows : g;
}
static int norm_fwd_grid(int rows) {
  const int g = sm_count_() * 6;
  return rows < g ? rows : g;
}

extern "C" int ob_norm_bwd_grid(int rows) { return norm_grid(rows); }

#define OB_NORM_FWD_LAUNCH(LN, D, grid, ...)                                              \
  do {                                                                                     \
    if ((D) <= THREADS * 8) norm_fwd_kernel<LN, 1><<<grid, THREADS, 0, stream>>>(__VA_ARGS__);            \
    else if ((D) <= THREADS * 16) norm_fwd_kernel<LN, 2><<<grid, THREADS, 0, stream>>>(__VA_ARGS__);      \
    else norm_fwd_kernel<LN, 4><<<grid, THREADS, 0, stream>>>(__VA_ARGS__);                               \
  } while (0)

#define OB_NORM_BWD_LAUNCH(LN, D, ...)                                                     \
  do {                                                                                     \
    if ((D) <= THREADS * 8) norm_bwd_kernel<LN, 1><<<grid, THREADS, 0, stream>>>(__VA_ARGS__);            \
    else if ((D) <= THREADS * 16) norm_bwd_kernel<LN, 2><<<grid, THREADS, 0, stream>>>(__VA_ARGS__);      \
    else norm_bwd_kernel<LN, 4><<<grid, THREADS, 0, stream>>>(__VA_ARGS__);                               \
  } while (0)

static bool norm_args_ok(int D) { return D % 8 == 0 && D <= THREADS * 8 * MAX_VEC; }

// y = rmsnorm(x [+ residual]) * w.  h_out receives x + residual when residual is given.
extern "C" int ob_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out, void* rstd,
                              int rows, int D, float eps, cudaStream_t stream) {
  if (!norm_args_ok(D)) return -1;
  if (rows == 0) return 0;
  OB_NORM_FWD_LAUNCH(false, D, norm_fwd_grid(rows), (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w, nullptr, (__nv_bfloat16*)y,
      (__nv_bfloat16*)h_out, (float*)rstd, nullptr, rows, D, eps);
  return (int)cudaGetLastError();
}

// As ob_rmsnorm_fwd, and also q = e4m3(y) with 1 x 128 scales [D / 128][scale_ld] (scale_ld >= rows).  D % 128 == 0.
extern "C" int ob_rmsnorm_fwd_fp8(const void* x, const void* residual, const void* w, void* y, void* h_out, void* rstd,
                                  void* q, void* scales, long long scale_ld, int rows, int D, float eps,
                                  cudaStream_t stream) {
  if (!norm_args_ok(D) || D % 128 != 0 || scale_ld < rows) return -1;
  if (rows == 0) return 0;
  const int grid = norm_fwd_grid(rows);
#define OB_NORM_FP8_ARGS                                                                                             \
  (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w, nullptr, (__nv_bfloat16*)y,      \
      (__nv_bfloat16*)h_out, (float*)rstd, nullptr, rows, D, eps, (uint8_t*)q, (float*)scales, scale_ld
  if (D <= THREADS * 8) norm_fwd_kernel<false, 1, true><<<grid, THREADS, 0, stream>>>(OB_NORM_FP8_ARGS);
  else if (D <= THREADS * 16) norm_fwd_kernel<false, 2, true><<<grid, THREADS, 0, stream>>>(OB_NORM_FP8_ARGS);
  else norm_fwd_kernel<false, 4, true><<<grid, THREADS, 0, stream>>>(OB_NORM_FP8_ARGS);
#undef OB_NORM_FP8_ARGS
  return (int)cudaGetLastError();
}

// dx = rmsnorm_bwd(dy, x, w, rstd) [+ dres];  dw (bf16 and/or fp32) = sum over rows.
// `partial` is scratch of ob_norm_bwd_grid(rows) * D floats.
extern "C" int ob_rmsnorm_bwd(const void* dy, const void* x, const void* w, const void* rstd, const void* dres,
                              void* dx, void* partial, void* dw_bf16, void* dw_f32, int accumulate, int rows, int D,
                              cudaStream_t stream) {
  if (!norm_args_ok(D)) return -1;
  if (rows == 0) return 0;
  const int grid = norm_grid(rows);
  OB_NORM_BWD_LAUNCH(false, D, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                       (const __nv_bfloat16*)w, (const float*)rstd, nullptr,
                                                       (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx,
                                                       (float*)partial, nullptr, rows, D);
  reduce_partials_kernel<<<(D + 31) / 32, 256, 0, stream>>>((const float*)partial, grid, D, (__nv_bfloat16*)dw_bf16,
                                                              (float*)dw_f32, accumulate);
  return (int)cudaGetLastError();
}

extern "C" int ob_layernorm_fwd(const void* x, const void* w, const void* b, void* y, void* mean, void* rstd, int rows,
                                int D, float eps, cudaStream_t stream) {
  if (!norm_args_ok(D)) return -1;
  if (rows == 0) return 0;
  OB_NORM_FWD_LAUNCH(true, D, norm_fwd_grid(rows), (const __nv_bfloat16*)x, nullptr, (const __nv_bfloat16*)w, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, nullptr,
      (float*)rstd, (float*)mean, rows, D, eps);
  return (int)cudaGetLastError();
}

// `partial` is scratch of 2 * ob_norm_bwd_grid(rows) * D floats (dw partials, then db partials).
extern "C" int ob_layernorm_bwd(const void* dy, const void* x, const void* w, const void* mean, const void* rstd,
                                void* dx, void* partial, void* dw_bf16, void* db_bf16, int rows, int D,
                                cudaStream_t stream) {
  if (!norm_args_ok(D)) return -1;
  if (rows == 0) return 0;
  const int grid = norm_grid(rows);
  float* dwp = (float*)partial;
  float* dbp = dwp + (size_t)grid * D;
  OB_NORM_BWD_LAUNCH(true, D, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                      (const __nv_bfloat16*)w, (const float*)rstd, (const float*)mean,
                                                      nullptr, (__nv_bfloat16*)dx, dwp, dbp, rows, D);
  reduce_partials_kernel<<<(D + 31) / 32, 256, 0, stream>>>(dwp, grid, D, (__nv_bfloat16*)dw_bf16, nullptr, 0);
  reduce_partials_kernel<<<(D + 31) / 32, 256, 0, stream>>>(dbp, grid, D, (__nv_bfloat16*)db_bf16, nullptr, 0);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate (declared in rmsnorm_bwd_noalloc.h).
//
// Same math and kernels as ob_rmsnorm_bwd, but the per-CTA weight-gradient partials live in a
// fixed array inside this library instead of a buffer the caller allocates.
#include "rmsnorm_bwd_noalloc.h"

#include <cstdio>
#include <mutex>

// 128 CTAs x 8192 columns x 4 bytes = 4 MiB per GPU that loads the library, held until exit.
static __device__ __align__(256) float g_rmsnorm_bwd_partials[OB_RMSNORM_NOALLOC_MAX_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_partials_ptr[kMaxDevices] = {};
std::mutex g_partials_mutex;

// Device address of the array on the current device; looked up once per device (the array's
// name is only a host-side handle and must never be handed to a kernel directly).
int partials_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return OB_RMSNORM_NOALLOC_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_partials_mutex);
  if (g_partials_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_rmsnorm_bwd_partials);
    if (e != cudaSuccess) return (int)e;
    g_partials_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_partials_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int ob_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const void* rstd, void* dx,
                                      void* dw_bf16, int rows, int D, cudaStream_t stream) {
  if (rows < 0) {
    std::fprintf(stderr, "ob_rmsnorm_bwd_noalloc: negative row count %d\n", rows);
    return OB_RMSNORM_NOALLOC_ERR_SHAPE;
  }
  if (D <= 0 || !norm_args_ok(D)) {
    std::fprintf(stderr, "ob_rmsnorm_bwd_noalloc: unsupported width D=%d (need D %% 8 == 0 and D <= %d)\n", D,
                 THREADS * 8 * MAX_VEC);
    return OB_RMSNORM_NOALLOC_ERR_SHAPE;
  }
  if (rows == 0) return 0;
  const int grid = rows < OB_RMSNORM_NOALLOC_MAX_CTAS ? rows : OB_RMSNORM_NOALLOC_MAX_CTAS;
  if ((long long)grid * D > (long long)OB_RMSNORM_NOALLOC_MAX_FLOATS) {
    std::fprintf(stderr, "ob_rmsnorm_bwd_noalloc: %d CTAs x D=%d needs %lld floats of scratch, the built-in array holds %d\n",
                 grid, D, (long long)grid * D, OB_RMSNORM_NOALLOC_MAX_FLOATS);
    return OB_RMSNORM_NOALLOC_ERR_TOO_LARGE;
  }
  float* partial = nullptr;
  const int rc = partials_for_current_device(&partial);
  if (rc != 0) return rc;
  // every CTA overwrites its whole row of partials, so nothing has to be cleared between calls
  OB_NORM_BWD_LAUNCH(false, D, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                       (const __nv_bfloat16*)w, (const float*)rstd, nullptr, nullptr,
                                                       (__nv_bfloat16*)dx, partial, nullptr, rows, D);
  reduce_partials_kernel<<<(D + 31) / 32, 256, 0, stream>>>(partial, grid, D, (__nv_bfloat16*)dw_bf16, nullptr, 0);
  return (int)cudaGetLastError();
}
