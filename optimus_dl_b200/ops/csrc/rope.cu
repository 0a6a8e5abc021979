// Fused per-head QK-norm + rotary embedding, forward and backward.
//
// q and k live as head slices of one activation row (the fused QKV projection output
// [T, (Hq + 2 Hkv) * hd], or separate tensors with a token stride).  One warp handles one
// (token, head) pair: each lane owns hd/32 consecutive elements, i.e. whole rotation pairs.
//   forward : x_hat = x * rsqrt(mean(x^2) + eps) * w      (only when norm weights are given)
//             out[2i]   = x_hat[2i] * cos - x_hat[2i+1] * sin
//             out[2i+1] = x_hat[2i] * sin + x_hat[2i+1] * cos        (interleaved pairs)
//   backward: inverse rotation of the incoming gradient, then the RMSNorm backward;
//             the norm-weight gradient is accumulated per CTA and written as a partial row.
// cos/sin come from a table [max_pos, hd/2, 2] (fp32) indexed by position id.
// Semantics follow optimus_dl/modules/model/blocks/rope.py:181-253 and the QK-norm order of
// optimus_dl/modules/model/blocks/attention.py:317-335 (norm before rotation, fp32 math).
#include "common.cuh"

namespace ob {
namespace rope {

constexpr int WARPS = 8;

template <int HD>
__global__ void __launch_bounds__(WARPS * 32)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                       long long in_tok_stride, long long out_tok_stride, const float* __restrict__ freqs,
                       const int* __restrict__ pos_ids, const __nv_bfloat16* __restrict__ qw,
                       const __nv_bfloat16* __restrict__ kw, float* __restrict__ rstd_out, int T, int Hq, int Hk,
                       int seq_len, float eps) {
  constexpr int E = HD / 32;  // elements per lane (2, 4 or 8)
  const int lane = threadIdx.x & 31;
  const int H = Hq + Hk;
  const long long total = (long long)T * H;
  for (long long item = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5); item < total;
       item += (long long)gridDim.x * WARPS) {
    const int t = (int)(item / H);
    const int h = (int)(item - (long long)t * H);
    const __nv_bfloat16* src = in + t * in_tok_stride + (long long)h * HD + lane * E;
    __nv_bfloat16* dst = out + t * out_tok_stride + (long long)h * HD + lane * E;
    float v[E];
    if constexpr (E == 2) {
      float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src));
      v[0] = a.x; v[1] = a.y;
    } else if constexpr (E == 4) {
      uint2 u = *reinterpret_cast<const uint2*>(src);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
      v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    } else {
      uint4 u = *reinterpret_cast<const uint4*>(src);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4 % E] = c.x; v[5 % E] = c.y; v[6 % E] = d.x; v[7 % E] = d.y;
    }
    const __nv_bfloat16* nw = (h < Hq) ? qw : kw;
    if (nw) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < E; ++j) ss += v[j] * v[j];
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / HD + eps);
      if (rstd_out && lane == 0) rstd_out[item] = rstd;
#pragma unroll
      for (int j = 0; j < E; ++j) {
        // round like the unfused path: the normalised value is produced in the activation dtype
        float xn = v[j] * rstd * __bfloat162float(nw[lane * E + j]);
        v[j] = __bfloat162float(__float2bfloat16(xn));
      }
    }
    const int pos = pos_ids ? pos_ids[t] : (t % seq_len);
    const float* f = freqs + ((long long)pos * (HD / 2) + lane * (E / 2)) * 2;
    float o[E];
#pragma unroll
    for (int j = 0; j < E / 2; ++j) {
      const float c = f[2 * j], s = f[2 * j + 1];
      o[2 * j] = v[2 * j] * c - v[2 * j + 1] * s;
      o[2 * j + 1] = v[2 * j] * s + v[2 * j + 1] * c;
    }
    if constexpr (E == 2) {
      *reinterpret_cast<uint32_t*>(dst) = pack_bf16x2(o[0], o[1]);
    } else if constexpr (E == 4) {
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]),
                                                  pack_bf16x2(o[4 % E], o[5 % E]), pack_bf16x2(o[6 % E], o[7 % E]));
    }
  }
}

// Backward.  `x_in` is the pre-norm input saved by the forward (only needed with norm weights).
template <int HD>
__global__ void __launch_bounds__(WARPS * 32)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ din,
                       long long dout_tok_stride, long long din_tok_stride, const __nv_bfloat16* __restrict__ x_in,
                       long long x_tok_stride, const float* __restrict__ freqs, const int* __restrict__ pos_ids,
                       const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
                       const float* __restrict__ rstd_in, float* __restrict__ dw_partial, int T, int Hq, int Hk,
                       int seq_len) {
  constexpr int E = HD / 32;
  __shared__ float sdw[2][WARPS][HD];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int H = Hq + Hk;
  const long long total = (long long)T * H;
  float dwq[E], dwk[E];
#pragma unroll
  for (int j = 0; j < E; ++j) { dwq[j] = 0.f; dwk[j] = 0.f; }
  for (long long item = (long long)blockIdx.x * WARPS + warp; item < total; item += (long long)gridDim.x * WARPS) {
    const int t = (int)(item / H);
    const int h = (int)(item - (long long)t * H);
    const __nv_bfloat16* gsrc = dout + t * dout_tok_stride + (long long)h * HD + lane * E;
    __nv_bfloat16* gdst = din + t * din_tok_stride + (long long)h * HD + lane * E;
    float g[E];
#pragma unroll
    for (int j = 0; j < E / 2; ++j) {
      float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(gsrc + 2 * j));
      g[2 * j] = a.x; g[2 * j + 1] = a.y;
    }
    const int pos = pos_ids ? pos_ids[t] : (t % seq_len);
    const float* f = freqs + ((long long)pos * (HD / 2) + lane * (E / 2)) * 2;
    float gi[E];
#pragma unroll
    for (int j = 0; j < E / 2; ++j) {
      const float c = f[2 * j], s = f[2 * j + 1];
      gi[2 * j] = g[2 * j] * c + g[2 * j + 1] * s;
      gi[2 * j + 1] = -g[2 * j] * s + g[2 * j + 1] * c;
    }
    const __nv_bfloat16* nw = (h < Hq) ? qw : kw;
    if (nw) {
      const float rstd = rstd_in[item];
      const __nv_bfloat16* xs = x_in + t * x_tok_stride + (long long)h * HD + lane * E;
      float xh[E], gw[E];
      float c1 = 0.f;
#pragma unroll
      for (int j = 0; j < E; ++j) {
        xh[j] = __bfloat162float(xs[j]) * rstd;
        gw[j] = gi[j] * __bfloat162float(nw[lane * E + j]);
        c1 += gw[j] * xh[j];
        if (h < Hq) dwq[j] += gi[j] * xh[j]; else dwk[j] += gi[j] * xh[j];
      }
      c1 = warp_sum(c1) / HD;
#pragma unroll
      for (int j = 0; j < E; ++j) gi[j] = rstd * (gw[j] - xh[j] * c1);
    }
#pragma unroll
    for (int j = 0; j < E / 2; ++j) *reinterpret_cast<uint32_t*>(gdst + 2 * j) = pack_bf16x2(gi[2 * j], gi[2 * j + 1]);
  }
  if (dw_partial) {
#pragma unroll
    for (int j = 0; j < E; ++j) { sdw[0][warp][lane * E + j] = dwq[j]; sdw[1][warp][lane * E + j] = dwk[j]; }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * HD; i += blockDim.x) {
      const int which = i / HD, c = i - which * HD;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) s += sdw[which][w][c];
      dw_partial[((size_t)blockIdx.x * 2 + which) * HD + c] = s;
    }
  }
}

}  // namespace rope
}  // namespace ob

using namespace ob::rope;

static int rope_grid(long long items) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long need = (items + WARPS - 1) / WARPS;
  long long g = (long long)sms * 8;
  return (int)(need < g ? need : g);
}
extern "C" int ob_rope_grid(long long items) { return rope_grid(items); }

// In-place capable (in == out) when no norm weights are given.
extern "C" int ob_qknorm_rope_fwd(const void* in, void* out, long long in_tok_stride, long long out_tok_stride,
                                  const void* freqs, const void* pos_ids, const void* qw, const void* kw, void* rstd,
                                  int T, int Hq, int Hk, int hd, int seq_len, float eps, cudaStream_t stream) {
  const long long items = (long long)T * (Hq + Hk);
  if (items == 0) return 0;
  const int grid = rope_grid(items);
#define OB_LAUNCH(HD)                                                                                              \
  qknorm_rope_fwd_kernel<HD><<<grid, WARPS * 32, 0, stream>>>(                                                     \
      (const __nv_bfloat16*)in, (__nv_bfloat16*)out, in_tok_stride, out_tok_stride, (const float*)freqs,           \
      (const int*)pos_ids, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, (float*)rstd, T, Hq, Hk, seq_len, eps)
  if (hd == 64) OB_LAUNCH(64);
  else if (hd == 128) OB_LAUNCH(128);
  else if (hd == 256) OB_LAUNCH(256);
  else return -1;
#undef OB_LAUNCH
  return (int)cudaGetLastError();
}

// dw_partial: scratch of ob_rope_grid(T*(Hq+Hk)) * 2 * hd floats when norm weights are given.
extern "C" int ob_qknorm_rope_bwd(const void* dout, void* din, long long dout_tok_stride, long long din_tok_stride,
                                  const void* x_in, long long x_tok_stride, const void* freqs, const void* pos_ids,
                                  const void* qw, const void* kw, const void* rstd, void* dw_partial, int T, int Hq,
                                  int Hk, int hd, int seq_len, cudaStream_t stream) {
  const long long items = (long long)T * (Hq + Hk);
  if (items == 0) return 0;
  const int grid = rope_grid(items);
#define OB_LAUNCH(HD)                                                                                              \
  qknorm_rope_bwd_kernel<HD><<<grid, WARPS * 32, 0, stream>>>(                                                     \
      (const __nv_bfloat16*)dout, (__nv_bfloat16*)din, dout_tok_stride, din_tok_stride, (const __nv_bfloat16*)x_in, \
      x_tok_stride, (const float*)freqs, (const int*)pos_ids, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw,  \
      (const float*)rstd, (float*)dw_partial, T, Hq, Hk, seq_len)
  if (hd == 64) OB_LAUNCH(64);
  else if (hd == 128) OB_LAUNCH(128);
  else if (hd == 256) OB_LAUNCH(256);
  else return -1;
#undef OB_LAUNCH
  return (int)cudaGetLastError();
}
