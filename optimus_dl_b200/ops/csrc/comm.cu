// Collective kernels that run over NVLink peer memory (see comm.cuh):
//   ob_barrier       : bounded cross-GPU barrier on a symmetric flag array
//   ob_pull          : all-gather as P2P pulls of copy tasks (no staging, lands in place)
//   ob_rs_adamw      : gradient reduce-scatter fused with bf16->fp32 cast, scaling, optional
//                      fp32 accumulation and the sharded AdamW update (three modes)
// The GEMM that overlaps an all-gather with its own tiles lives in gemm_ag.cu.
#include "comm.cuh"

namespace ob {
namespace comm {

// Poll limit of the cross-GPU flag waits in this file (about 100 ns per poll: the default is roughly two seconds).
// The host may lower it (ob_set_flag_wait_iters) so that a test can let a wait run out quickly.
__device__ unsigned int g_flag_wait_iters = 1u << 24;

// flags: this rank's symmetric int array [MAX_RANKS]; peers.p[r] = rank r's array.
// Rank `me` writes `epoch` into slot `me` of every rank, then waits for all slots of its own array.
__global__ void barrier_kernel(PeerPtrs peers, int me, int world, int epoch, int* status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  int* remote = reinterpret_cast<int*>(peers.p[r]) + me;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const int* mine = reinterpret_cast<const int*>(peers.p[me]) + r;
  bool ok = false;
  const uint32_t limit = g_flag_wait_iters;
  for (uint32_t it = 0; it < limit; ++it) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v >= epoch) { ok = true; break; }
    __nanosleep(100);
  }
  if (!ok && status) atomicCAS(status, kStatusOk, kStatusFlagTimeout);
  __threadfence_system();
}

__global__ void __launch_bounds__(1024)
pull_kernel(const CopyTask* __restrict__ tasks, int n_tasks, PeerPtrs src, __nv_bfloat16* dst, int* flags, int epoch) {
  run_copy_tasks(tasks, n_tasks, blockIdx.x, gridDim.x, src, dst, flags, epoch);
}

// One owned slice of a parameter: `numel` elements that sit at `grad_off` in every rank's (symmetric) gradient
// buffer, at `param_off` in this rank's bf16 parameter shard and at `shard_off` in its fp32 shard state.
struct Segment {
  long long grad_off;
  long long param_off;
  long long shard_off;
  int numel;
  float weight_decay;
  float lr_scale;
  int pad;
};

struct AdamArgs {
  float lr, beta1, beta2, eps, bc1, bc2;
  float grad_scale;        // e.g. 1 / (world * accumulation steps)
  float max_norm;          // > 0: clip with *sumsq_in
  const float* sumsq_in;   // squared global gradient norm (before grad_scale), device scalar
};

enum Mode : int { kFused = 0, kReduceOnly = 1, kUpdateOnly = 2 };

// Sum of the ranks' bf16 gradients for 8 consecutive elements, in fixed rank order (every owner adds in the same
// order, so results are reproducible).  The loads of up to four ranks are issued before the first add; they are
// weak, non-allocating loads: the data was published before the barrier this launch is ordered after.
__device__ __forceinline__ void reduce_peers_8(const PeerPtrs& grads, int world, long long off, int i, float* g) {
  for (int r0 = 0; r0 < world; r0 += 4) {
    uint4 u[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (r0 + j < world)
        u[j] = ld_peer_bulk_16(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(grads.p[r0 + j]) + off) + i);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (r0 + j < world) {
        const float2 a0 = unpack_bf16x2(u[j].x), a1 = unpack_bf16x2(u[j].y), a2 = unpack_bf16x2(u[j].z), a3 = unpack_bf16x2(u[j].w);
        g[0] += a0.x; g[1] += a0.y; g[2] += a1.x; g[3] += a1.y; g[4] += a2.x; g[5] += a2.y; g[6] += a3.x; g[7] += a3.y;
      }
  }
}

// MODE kFused     : g = [grad_shard +] sum_r peer_grad[r]  -> AdamW -> master/m/v, bf16 shard out
// MODE kReduceOnly: grad_shard = [grad_shard +] sum_r peer_grad[r]            (fp32 accumulation over micro-batches)
// MODE kUpdateOnly: g = grad_shard -> AdamW (with clip) -> master/m/v, bf16 shard out
// `acc_in` selects the bracketed term.
template <int MODE>
__global__ void __launch_bounds__(256)
rs_adamw_kernel(const Segment* __restrict__ segs, int n_segs, PeerPtrs grads, int world,
                float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                float* __restrict__ grad_shard, __nv_bfloat16* __restrict__ param_out, AdamArgs a, int acc_in,
                const int* __restrict__ status) {
  // A step whose barrier (or any earlier kernel) reported a failed wait must not be committed: the peers'
  // gradient buffers may be half written. The status word is sticky until the host reads and clears it.
  if (MODE != kReduceOnly && status != nullptr && *reinterpret_cast<const volatile int*>(status) != kStatusOk) return;
  float scale = a.grad_scale;
  if (MODE != kReduceOnly && a.sumsq_in && a.max_norm > 0.f) {
    const float norm = sqrtf(*a.sumsq_in) * a.grad_scale;
    scale *= fminf(1.0f, a.max_norm / (norm + 1e-6f));
  }
  const float inv_sqrt_bc2 = rsqrtf(a.bc2);
  for (int s = 0; s < n_segs; ++s) {
    const Segment seg = segs[s];
    const bool aligned = (seg.grad_off % 8 == 0) && (seg.param_off % 8 == 0) && (seg.shard_off % 4 == 0);
    const int nvec = aligned ? seg.numel / 8 : 0;
    const float lr = a.lr * seg.lr_scale;
    const float step = lr / a.bc1;
    const float decay = 1.0f - lr * seg.weight_decay;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += gridDim.x * blockDim.x) {
      float g[8];
      float4* gs = reinterpret_cast<float4*>(grad_shard + seg.shard_off) + 2 * i;
      if (MODE == kUpdateOnly || acc_in) {
        const float4 g0 = gs[0], g1 = gs[1];
        g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = 0.f;
      }
      if (MODE != kUpdateOnly) reduce_peers_8(grads, world, seg.grad_off, i, g);
      if (MODE == kReduceOnly) {
        gs[0] = make_float4(g[0], g[1], g[2], g[3]);
        gs[1] = make_float4(g[4], g[5], g[6], g[7]);
        continue;
      }
      float4* mp = reinterpret_cast<float4*>(master + seg.shard_off) + 2 * i;
      float4* mm = reinterpret_cast<float4*>(m + seg.shard_off) + 2 * i;
      float4* vv = reinterpret_cast<float4*>(v + seg.shard_off) + 2 * i;
      float4 p0 = mp[0], p1 = mp[1], m0 = mm[0], m1 = mm[1], v0 = vv[0], v1 = vv[1];
      float p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
      float mo[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
      float vo[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gj = g[j] * scale;
        mo[j] = a.beta1 * mo[j] + (1.0f - a.beta1) * gj;
        vo[j] = a.beta2 * vo[j] + (1.0f - a.beta2) * gj * gj;
        p[j] = p[j] * decay - step * mo[j] / (sqrtf(vo[j]) * inv_sqrt_bc2 + a.eps);
      }
      mp[0] = make_float4(p[0], p[1], p[2], p[3]); mp[1] = make_float4(p[4], p[5], p[6], p[7]);
      mm[0] = make_float4(mo[0], mo[1], mo[2], mo[3]); mm[1] = make_float4(mo[4], mo[5], mo[6], mo[7]);
      vv[0] = make_float4(vo[0], vo[1], vo[2], vo[3]); vv[1] = make_float4(vo[4], vo[5], vo[6], vo[7]);
      reinterpret_cast<uint4*>(param_out + seg.param_off)[i] =
          make_uint4(pack_bf16x2(p[0], p[1]), pack_bf16x2(p[2], p[3]), pack_bf16x2(p[4], p[5]), pack_bf16x2(p[6], p[7]));
    }
    // scalar tail (segments whose length is not a multiple of 8)
    for (int i = nvec * 8 + blockIdx.x * blockDim.x + threadIdx.x; i < seg.numel; i += gridDim.x * blockDim.x) {
      const long long k = seg.shard_off + i;
      float g = (MODE == kUpdateOnly || acc_in) ? grad_shard[k] : 0.f;
      if (MODE != kUpdateOnly) {
        for (int r = 0; r < world; ++r)
          g += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grads.p[r])[seg.grad_off + i]);
      }
      if (MODE == kReduceOnly) { grad_shard[k] = g; continue; }
      const float gj = g * scale;
      const float mo = a.beta1 * m[k] + (1.0f - a.beta1) * gj;
      const float vo = a.beta2 * v[k] + (1.0f - a.beta2) * gj * gj;
      const float p = master[k] * decay - step * mo / (sqrtf(vo) * inv_sqrt_bc2 + a.eps);
      master[k] = p; m[k] = mo; v[k] = vo;
      param_out[seg.param_off + i] = __float2bfloat16(p);
    }
  }
}

}  // namespace comm
}  // namespace ob

using namespace ob;
using namespace ob::comm;

// Receive half of a reduce-scatter whose send half ran in a GEMM epilogue (ob_gemm_rs_bf16):
// cross-GPU barrier, then out[r][c] = residual[r][c] + sum_s staging[s][r][c] (fp32, fixed slot
// order, one rounding to bf16).  The barrier is part of the kernel: block 0 publishes this rank's
// arrival, every block waits (bounded) until all ranks have arrived before it touches `staging`.
__global__ void __launch_bounds__(256)
rs_sum_kernel(PeerPtrs flag_peers, int me, int world, int epoch, const __nv_bfloat16* __restrict__ staging, int rows,
              int D, long long ld, const __nv_bfloat16* __restrict__ residual, long long res_ld,
              __nv_bfloat16* __restrict__ out, long long out_ld, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (flag_peers.p[me] != nullptr && world > 1) {
    if (blockIdx.x == 0 && (int)threadIdx.x < world) {
      __threadfence_system();
      int* remote = reinterpret_cast<int*>(flag_peers.p[threadIdx.x]) + me;
      asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    }
    if ((int)threadIdx.x < world) {
      const int* mine = reinterpret_cast<const int*>(flag_peers.p[me]) + threadIdx.x;
      bool ok = false;
      const uint32_t limit = g_flag_wait_iters;
      for (uint32_t it = 0; it < limit; ++it) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if (v >= epoch) { ok = true; break; }
        __nanosleep(100);
      }
      if (!ok) {
        s_ok = 0;
        if (status) atomicCAS(status, kStatusOk, kStatusFlagTimeout);
      }
    }
    __syncthreads();
    if (!s_ok) return;
  }
  const int vec_per_row = D / 8;
  const long long total = (long long)rows * vec_per_row;
  const long long slot = (long long)rows * ld;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / vec_per_row);
    const int c = (int)(i - (long long)r * vec_per_row) * 8;
    float acc[8];
    if (residual) {
      const uint4 u = *reinterpret_cast<const uint4*>(residual + (long long)r * res_ld + c);
      const float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y), a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
      acc[0] = a0.x; acc[1] = a0.y; acc[2] = a1.x; acc[3] = a1.y; acc[4] = a2.x; acc[5] = a2.y; acc[6] = a3.x; acc[7] = a3.y;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
    for (int s = 0; s < world; ++s) {
      const uint4 u = ld_peer_16(staging + s * slot + (long long)r * ld + c);
      const float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y), a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
      acc[0] += a0.x; acc[1] += a0.y; acc[2] += a1.x; acc[3] += a1.y; acc[4] += a2.x; acc[5] += a2.y; acc[6] += a3.x; acc[7] += a3.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + (long long)r * out_ld + c) = o;
  }
}

// Vocabulary-parallel embedding without partial sums: this rank owns table rows
// [voff, voff + v_local); for every token whose id falls in that range it stores the row into
// the activation buffer of the rank that holds the token (token t lives on rank t / rows_per_rank).
// One warp per token; ids outside the range are another rank's job.
__global__ void __launch_bounds__(256)
embedding_push_kernel(const long long* __restrict__ ids, int T, const __nv_bfloat16* __restrict__ table, int v_local,
                      int voff, int D, PeerPtrs dst, int rows_per_rank) {
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    const long long id = ids[t] - voff;
    if (id < 0 || id >= v_local) continue;
    const int owner = t / rows_per_rank;
    const uint4* src = reinterpret_cast<const uint4*>(table + id * D);
    uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[owner]) +
                                          (long long)(t - owner * rows_per_rank) * D);
    for (int i = lane; i < D / 8; i += 32) out[i] = src[i];
  }
}

static PeerPtrs make_peers(const void* const* ptrs, int world) {
  PeerPtrs p{};
  for (int i = 0; i < world && i < MAX_RANKS; ++i) p.p[i] = const_cast<void*>(ptrs[i]);
  return p;
}

// Poll limit of ob_barrier / ob_rs_sum waits on the current device (0 restores the default).
extern "C" int ob_set_flag_wait_iters(unsigned int iters) {
  if (iters == 0) iters = 1u << 24;
  return (int)cudaMemcpyToSymbol(g_flag_wait_iters, &iters, sizeof(iters));
}

extern "C" int ob_barrier(const void* const* flag_ptrs, int me, int world, int epoch, int* status,
                          cudaStream_t stream) {
  if (world > MAX_RANKS) return -1;
  barrier_kernel<<<1, 32, 0, stream>>>(make_peers(flag_ptrs, world), me, world, epoch, status);
  return (int)cudaGetLastError();
}

// tasks: device array of CopyTask (24 bytes each).  dst is this rank's buffer, src_ptrs the peers'.
extern "C" int ob_pull(const void* tasks, int n_tasks, const void* const* src_ptrs, int world, void* dst, int* flags,
                       int epoch, int n_ctas, cudaStream_t stream) {
  if (world > MAX_RANKS) return -1;
  if (n_tasks == 0) return 0;
  if (n_ctas <= 0) n_ctas = 32;
  if (n_ctas > n_tasks) n_ctas = n_tasks;
  pull_kernel<<<n_ctas, 1024, 0, stream>>>((const CopyTask*)tasks, n_tasks, make_peers(src_ptrs, world),
                                           (__nv_bfloat16*)dst, flags, epoch);
  return (int)cudaGetLastError();
}

// mode: 0 reduce + AdamW in one pass, 1 reduce into the fp32 gradient shard, 2 AdamW from the gradient shard.
// acc_in (modes 0 and 1): start from the gradient shard instead of zero (gradient accumulation in fp32).
// The update modes do nothing while *status is non-zero (a failed wait earlier in the step).
extern "C" int ob_rs_adamw(int mode, const void* segs, int n_segs, const void* const* grad_ptrs, int world,
                           void* master, void* m, void* v, void* grad_shard, void* param_out, float lr, float beta1,
                           float beta2, float eps, float bc1, float bc2, float grad_scale, float max_norm,
                           const void* sumsq_in, int acc_in, int n_ctas, const int* status, cudaStream_t stream) {
  if (world > MAX_RANKS) return -1;
  if (n_segs == 0) return 0;
  if ((mode != kFused || acc_in) && grad_shard == nullptr) return -2;
  if (n_ctas <= 0) n_ctas = 148 * 6;
  AdamArgs a{lr, beta1, beta2, eps, bc1, bc2, grad_scale, max_norm, (const float*)sumsq_in};
  PeerPtrs g = make_peers(grad_ptrs, world);
  if (mode == kFused)
    rs_adamw_kernel<kFused><<<n_ctas, 256, 0, stream>>>((const Segment*)segs, n_segs, g, world, (float*)master,
                                                        (float*)m, (float*)v, (float*)grad_shard,
                                                        (__nv_bfloat16*)param_out, a, acc_in, status);
  else if (mode == kReduceOnly)
    rs_adamw_kernel<kReduceOnly><<<n_ctas, 256, 0, stream>>>((const Segment*)segs, n_segs, g, world, nullptr, nullptr,
                                                             nullptr, (float*)grad_shard, nullptr, a, acc_in, status);
  else
    rs_adamw_kernel<kUpdateOnly><<<n_ctas, 256, 0, stream>>>((const Segment*)segs, n_segs, g, world, (float*)master,
                                                             (float*)m, (float*)v, (float*)grad_shard,
                                                             (__nv_bfloat16*)param_out, a, 0, status);
  return (int)cudaGetLastError();
}

// staging: this rank's buffer [world][rows][ld] (bf16) that the peers' GEMM epilogues filled.
// flag_ptrs may be null (or world == 1) to skip the built-in barrier.
extern "C" int ob_rs_sum(const void* const* flag_ptrs, int me, int world, int epoch, const void* staging, int rows,
                         int D, long long ld, const void* residual, long long res_ld, void* out, long long out_ld,
                         int n_ctas, int* status, cudaStream_t stream) {
  if (world > MAX_RANKS || D % 8 != 0 || ld % 8 != 0 || out_ld % 8 != 0 || (residual && res_ld % 8 != 0)) return -1;
  if (rows <= 0) return 0;
  PeerPtrs fp{};
  if (flag_ptrs) fp = make_peers(flag_ptrs, world);
  if (n_ctas <= 0) n_ctas = 296;
  rs_sum_kernel<<<n_ctas, 256, 0, stream>>>(fp, me, world, epoch, (const __nv_bfloat16*)staging, rows, D, ld,
                                            (const __nv_bfloat16*)residual, res_ld, (__nv_bfloat16*)out, out_ld,
                                            status);
  return (int)cudaGetLastError();
}

// ids: int64 [T] (the same on every rank); table: this rank's [v_local, D] bf16 rows.
extern "C" int ob_embedding_push(const void* ids, int T, const void* table, int v_local, int voff, int D,
                                 const void* const* dst_ptrs, int world, int rows_per_rank, cudaStream_t stream) {
  if (world > MAX_RANKS || D % 8 != 0 || rows_per_rank <= 0) return -1;
  if (T <= 0) return 0;
  int blocks = (T + 7) / 8;
  if (blocks > 1184) blocks = 1184;
  embedding_push_kernel<<<blocks, 256, 0, stream>>>((const long long*)ids, T, (const __nv_bfloat16*)table, v_local, voff,
                                                    D, make_peers(dst_ptrs, world), rows_per_rank);
  return (int)cudaGetLastError();
}
