// Device-side pieces of the NVLink data plane: peer copy tasks, flags and bounded barriers.
//
// Every rank maps every peer's symmetric buffers, so a kernel addresses peer memory with
// ordinary loads and stores (system scope where ordering matters).  No bulk-tensor copy with a
// cluster-wide broadcast is used anywhere in this data plane.
#pragma once
#include "common.cuh"

namespace ob {
namespace comm {

constexpr int MAX_RANKS = 16;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

// One unit of copy work: `numel` bf16 elements pulled from element offset `src_offset` of rank `peer`'s buffer
// to element offset `offset` of the local one (the push form uses `offset` on the peer's side).  `flag` >= 0
// names a readiness flag that is set to the launch's epoch when the chunk has landed.
struct CopyTask {
  long long offset;
  long long src_offset;
  int numel;
  short peer;
  short pad;
  int flag;
};

// Bulk data loads from a peer.  The data was published before a barrier that this launch is ordered after, so
// a weak load is enough; it must not allocate in L1 (the line could survive into a later launch) and, unlike a
// system-scope relaxed load, it may be issued back to back with its neighbours.
__device__ __forceinline__ uint4 ld_peer_bulk_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__device__ __forceinline__ uint4 ld_peer_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Executed by a whole CTA: copy tasks [first, n) with stride `stride`.  UNROLL 16-byte loads per thread are
// issued before the first store, i.e. blockDim.x * UNROLL * 16 bytes are in flight per CTA.
template <int UNROLL = 8>
__device__ __forceinline__ void run_copy_tasks(const CopyTask* tasks, int n_tasks, int first, int stride,
                                               const PeerPtrs& src, __nv_bfloat16* dst, int* flags, int epoch) {
  for (int t = first; t < n_tasks; t += stride) {
    const CopyTask task = tasks[t];
    const __nv_bfloat16* s = reinterpret_cast<const __nv_bfloat16*>(src.p[task.peer]) + task.src_offset;
    __nv_bfloat16* d = dst + task.offset;
    const int nvec = (task.offset % 8 == 0 && task.src_offset % 8 == 0) ? task.numel / 8 : 0;
    int i = threadIdx.x;
    for (; i + (UNROLL - 1) * (int)blockDim.x < nvec; i += UNROLL * blockDim.x) {
      uint4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) v[u] = ld_peer_bulk_16(reinterpret_cast<const uint4*>(s) + i + u * blockDim.x);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) reinterpret_cast<uint4*>(d)[i + u * blockDim.x] = v[u];
    }
    for (; i < nvec; i += blockDim.x) reinterpret_cast<uint4*>(d)[i] = ld_peer_bulk_16(reinterpret_cast<const uint4*>(s) + i);
    for (int j = nvec * 8 + threadIdx.x; j < task.numel; j += blockDim.x) d[j] = s[j];
    if (task.flag >= 0) {
      // the consumer reads these bytes through TMA (async proxy): order our generic-proxy stores
      asm volatile("fence.proxy.async.global;" ::: "memory");
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();
        asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flags + task.flag), "r"(epoch) : "memory");
      }
    }
  }
}

// Push variant: the chunks of this rank's own slice (`src`, local) are stored into the peers' operand buffers
// and the peers' row flags are raised.  task.offset is the element offset inside the peer's buffer, the source
// element offset is task.offset - slice_base.  Stores over NVLink are posted, so a few CTAs saturate the link
// where loads would wait a round trip each.
template <int UNROLL = 8>
__device__ __forceinline__ void run_push_tasks(const CopyTask* tasks, int n_tasks, int first, int stride,
                                               const __nv_bfloat16* src, long long slice_base, const PeerPtrs& dst,
                                               const PeerPtrs& flag_ptrs, int epoch) {
  for (int t = first; t < n_tasks; t += stride) {
    const CopyTask task = tasks[t];
    const uint4* s = reinterpret_cast<const uint4*>(src + (task.offset - slice_base));
    uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[task.peer]) + task.offset);
    const int nvec = task.numel / 8;   // chunks are whole rows of a width that is a multiple of 8
    int i = threadIdx.x;
    for (; i + (UNROLL - 1) * (int)blockDim.x < nvec; i += UNROLL * blockDim.x) {
      uint4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) v[u] = s[i + u * blockDim.x];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) d[i + u * blockDim.x] = v[u];
    }
    for (; i < nvec; i += blockDim.x) d[i] = s[i];
    // make this CTA's stores visible at system scope, then publish the chunk on the peer
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && task.flag >= 0) {
      int* f = reinterpret_cast<int*>(flag_ptrs.p[task.peer]) + task.flag;
      asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
    }
  }
}

}  // namespace comm
}  // namespace ob
