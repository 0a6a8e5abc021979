// Two-SM form of the persistent bf16 GEMM: a pair of CTAs on neighbouring SMs (a cluster of two) computes one
// 256 x 256 output tile with `tcgen05.mma.cta_group::2`.
//
// Why a pair: with one CTA per 128 x 256 tile every k-step of 16 reads 4 KB of A and 8 KB of B from shared
// memory, and TMA writes the same amount again, which is more than one SM's shared memory delivers at full
// tensor rate.  In the paired form each CTA stages its own 128 rows of A and only HALF of the B tile (128 of the
// 256 columns); the tensor cores of the pair read the two halves from both shared memories.  Shared-memory
// traffic per SM drops by a third and six pipeline stages fit where four did.
//
// Roles per CTA (192 threads, as in the one-SM kernel): warp 0 = TMA producer, warp 1 = TMEM owner (and, in the
// pair's leader CTA only, the MMA issuer), warps 2..5 = epilogue for this CTA's 128 accumulator rows.
//   * both producers issue their loads with `.cta_group::2` and name the LEADER's "full" barrier, so the leader's
//     MMA thread sees one barrier complete when both halves have landed (the leader's producer posts the
//     expected byte count for both CTAs);
//   * the leader's MMA thread frees a stage, and publishes a finished accumulator, with a commit that arrives on
//     the same barrier in both CTAs (`tcgen05.commit ... multicast::cluster`, CTA mask 0b11);
//   * the epilogue warps of both CTAs release an accumulator stage by arriving on the leader's barrier.
// No load uses a cluster-wide broadcast: each CTA fetches its own tiles.  Every wait is bounded (common.cuh); the
// CTAs of a pair leave together through a cluster barrier so that neither exits while its peer may still signal it.
#pragma once
#include "gemm_core.cuh"

namespace ob {
namespace gemm2 {

using gemm::Params;
using gemm::TileCoord;

constexpr int TM = 256;               // rows of the pair's tile (128 per CTA)
constexpr int TN = 256;               // columns of the pair's tile (each CTA stages 128 of the B rows)
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int ACC_STAGES = 2;
constexpr int NUM_THREADS = 192;
constexpr int A_BYTES = 128 * BK * 2;   // 16 KB per CTA
constexpr int B_BYTES = 128 * BK * 2;   // 16 KB per CTA (half of the B tile)
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;   // clears the CTA-rank bit of a shared::cluster address: the pair's even CTA

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Tiled load into THIS CTA's shared memory whose completion bytes are counted on the pair leader's barrier.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar) & kPeerMask), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma2_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in both CTAs of the pair once all MMAs issued so far are done.
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & kPeerMask) : "memory");
}

// One CTA's share of the paired persistent GEMM: `pair` / `n_pairs` give the static tile schedule of the CTA pair
// this CTA belongs to (callers with extra non-GEMM CTAs in the grid pass the GEMM pair index and count).
template <int A_MN, int B_MN, int SWIGLU>
__device__ __forceinline__ void gemm2_cta(const CUtensorMap* tmA_, const CUtensorMap* tmB_, const CUtensorMap* tmB2_,
                                          const Params& p, int pair, int n_pairs, uint8_t* smem_raw) {
  const CUtensorMap& tmA = *tmA_;
  const CUtensorMap& tmB = *tmB_;
  const CUtensorMap& tmB2 = *tmB2_;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                          // [STAGES]      used in the leader CTA
  uint64_t* empty_bar = bars + STAGES;                // [STAGES]      one set per CTA
  uint64_t* acc_full = bars + 2 * STAGES;             // [ACC_STAGES]  one set per CTA
  uint64_t* acc_empty = bars + 2 * STAGES + ACC_STAGES;   //           used in the leader CTA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * ACC_STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  constexpr bool DUAL = SWIGLU == 1;                   // 1: dual-B SwiGLU forward, 2: SwiGLU-backward epilogue,
                                                       // 3: cross-entropy statistics epilogue (no output tensor)
  constexpr int bn = DUAL ? TN / 2 : TN;               // output columns per tile
  const int tiles_m = (p.M + TM - 1) / TM;
  const int tiles_n = (p.N + bn - 1) / bn;
  const int num_tiles = tiles_m * tiles_n;
  const int k_tiles = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < ACC_STAGES; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 8); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();       // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      if (DUAL) tma_prefetch_desc(&tmB2);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        const TileCoord tc = gemm::tile_coord(tile, tiles_m, tiles_n, p);
        const int m0 = tc.m * TM + (int)rank * 128;          // this CTA's rows of A
        const int n0 = tc.n * bn;
        const int nb = DUAL ? n0 : n0 + (int)rank * 128;     // this CTA's rows of B
        const CUtensorMap* tb = (DUAL && rank == 1) ? &tmB2 : &tmB;
        if (p.b_flags) {
          // rows of B that another part of this launch is still landing in local memory (fused all-gather)
          const int f0 = nb / p.flag_rows;
          const int f1 = (min(nb + 128, p.N) - 1) / p.flag_rows;
          for (int f = f0; f <= f1 && ok; ++f) ok = gemm::wait_flag(p.b_flags + f, p.flag_value, abort_flag, p.status);
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kt = 0; kt < k_tiles && ok; ++kt) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status);
          if (!ok) break;
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
          const int k0 = kt * BK;
          if (A_MN) {
            tma_load_2d_pair(sA, &tmA, &full_bar[stage], m0, k0);
            tma_load_2d_pair(sA + 8192, &tmA, &full_bar[stage], m0 + 64, k0);
          } else {
            tma_load_2d_pair(sA, &tmA, &full_bar[stage], k0, m0);
          }
          if (B_MN && !DUAL) {
            tma_load_2d_pair(sB, tb, &full_bar[stage], nb, k0);
            tma_load_2d_pair(sB + 8192, tb, &full_bar[stage], nb + 64, k0);
          } else {
            tma_load_2d_pair(sB, tb, &full_bar[stage], k0, nb);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // drain: every stage this thread filled has been consumed, so no copy is in flight towards this CTA
      for (int s = 0; s < STAGES; ++s) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status)) break;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TM, TN, A_MN, B_MN && !DUAL);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TN;
        for (int kt = 0; kt < k_tiles; ++kt) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sB = sA + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(sA + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sA + kk * 32, 16, 1024);
            const uint64_t db = (B_MN && !DUAL) ? make_smem_desc_sw128(sB + kk * 2048, 8192, 1024)
                                                  : make_smem_desc_sw128(sB + kk * 32, 16, 1024);
            umma2_f16_ss(d_tmem, da, db, idesc, (kt | kk) ? 1u : 0u);
          }
          umma2_commit_both(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma2_commit_both(&acc_full[acc]);
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
      // Wait (bounded) until both CTAs' epilogues have drained every accumulator stage, so that nothing reads
      // TMEM, and no commit is still on its way to a barrier, when the pair leaves.
      for (int a = 0; a < ACC_STAGES && ok; ++a) {
        ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status);
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quarter = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    const bool vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(SWIGLU == 2 ? p.G : p.C) & 15) == 0) &&
                        (SWIGLU != 2 || (reinterpret_cast<uintptr_t>(p.U) & 15) == 0);
    // SwiGLU-backward epilogue: g and u of a tile are read by thread = row in 64-byte pieces, which DRAM serves
    // badly (one short burst per 28 KB-strided row).  Each thread therefore asks L2 for the whole 512-byte extent
    // of its row one tile ahead, while the tensor cores still work on that tile; the epilogue's reads then hit L2.
    auto prefetch_gu = [&](int t) {
      if (SWIGLU != 2 || t >= num_tiles) return;
      const TileCoord pc = gemm::tile_coord(t, tiles_m, tiles_n, p);
      const int prow = pc.m * TM + (int)rank * 128 + quarter * 32 + lane, pn0 = pc.n * bn;
      if (prow >= p.M) return;
      const __nv_bfloat16* pg = reinterpret_cast<const __nv_bfloat16*>(p.G) + (long long)prow * p.ldc + pn0;
      const __nv_bfloat16* pu = reinterpret_cast<const __nv_bfloat16*>(p.U) + (long long)prow * p.ldc + pn0;
#pragma unroll
      for (int c = 0; c < TN; c += 64) {
        if (pn0 + c < p.N) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(pg + c));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(pu + c));
        }
      }
    };
    prefetch_gu(pair);
    for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
      const TileCoord tc = gemm::tile_coord(tile, tiles_m, tiles_n, p);
      const int m0 = tc.m * TM + (int)rank * 128;
      const int n0 = tc.n * bn;
      prefetch_gu(tile + n_pairs);
      ok = mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status);
      if (!ok) break;
      tc_fence_after();
      gemm::epilogue_tile<SWIGLU>(p, m0, n0, tmem_base + (uint32_t(quarter * 32) << 16) + acc * TN, warp, lane, vec_ok,
                                  nullptr);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&acc_empty[acc]);
      if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();       // both CTAs are done with TMEM and with each other's barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}


}  // namespace gemm2
}  // namespace ob
