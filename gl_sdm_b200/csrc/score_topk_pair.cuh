// Dense-key routing, CTA-pair variant: two CTAs of a cluster work on one unit of 256 query
// rows. Each CTA keeps its own 128 query rows and loads HALF of every 256-slot key tile; one
// thread of the leader CTA issues tcgen05.mma.cta_group::2 (M = 256 across the pair, N = 256),
// so every key sub-tile is read from shared memory once per 256 rows instead of once per 128.
// That halves the shared-memory operand traffic per MMA, which is what limits the single-CTA
// kernel (128x128x16 MMAs stream 128 B/clk). Accumulators: 128 lanes x 256 columns x 2
// buffers of each CTA's tensor memory. Scanning, queues and inserters are as in the
// wide-tile kernel, per CTA, over 128 rows (8 scanner warps, 4 inserter warps).
//
// Cross-CTA signalling: both CTAs' TMA loads complete transactions on the LEADER's full
// barriers; the leader's commits are multicast to the barrier at the same offset in both CTAs
// (accumulator full, stage empty, query tile empty); scanner warps of both CTAs arrive on the
// leader's accumulator-empty barrier. No TMA load is multicast. Every wait is bounded.
#pragma once

#include "score_topk.cuh"

namespace glsdm {
namespace dense {

constexpr int kPairTileCols = 256;               // slots per key tile of the pair (MMA N)
constexpr int kPairStages = 4;
constexpr int kPairScanWarps = 8;                // 4 lane quarters x 2 column halves
constexpr int kPairInsertWarps = 4;              // one per lane quarter (32 rows), fed by its two scanner warps
constexpr int kPairThreads = 32 * (2 + kPairScanWarps + kPairInsertWarps);
constexpr uint32_t kPairInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kPairTileCols >> 3) << 17) |
                                    ((256 >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(leader_bar)
      : "memory");
}

__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kPairInstrDesc), "r"(acc)
      : "memory");
}

// Arrive on the barrier at this offset in BOTH CTAs once all prior MMAs have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t both = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(both)
      : "memory");
}

struct PairBarriers {
  uint64_t a_full;                     // leader: both CTAs' query tiles have landed
  uint64_t a_empty;                    // each CTA: the MMAs have finished with the query tile
  uint64_t b_full[kPairStages];        // leader: both halves of the key tile have landed
  uint64_t b_empty[kPairStages];       // each CTA: the stage may be overwritten
  uint64_t acc_full[2];                // each CTA: accumulator buffer complete
  uint64_t acc_empty[2];               // leader: all 16 scanner warps of the pair are done with it
  uint32_t tmem_base;
  int abort_flag;
};

template <int KB>
struct PairLayout {
  static constexpr int kA = KB * kSubTileBytes;                    // 128 rows
  static constexpr int kB = kPairStages * KB * kSubTileBytes;      // 128 key rows per stage
  static constexpr int kListOffset = kA + kB;
  static constexpr int kListBytes = 8 * 32 * kBlockRows;
  __host__ __device__ static constexpr int total() {
    return kListOffset + kListBytes + static_cast<int>(sizeof(PairBarriers)) + 4 * kBlockRows +
           kPairInsertWarps * static_cast<int>(sizeof(Queue)) + 64;
  }
};

template <int KB>
__global__ void __launch_bounds__(kPairThreads, 1)
score_topk_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, Params p) {
  extern __shared__ __align__(1024) uint8_t raw_smem[];
  uint8_t* smem_a = raw_smem;
  uint8_t* smem_b = raw_smem + PairLayout<KB>::kA;
  uint64_t* all_lists = reinterpret_cast<uint64_t*>(raw_smem + PairLayout<KB>::kListOffset);
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(raw_smem + PairLayout<KB>::kListOffset + PairLayout<KB>::kListBytes);
  float* floors = reinterpret_cast<float*>(bars + 1);
  Queue* queues = reinterpret_cast<Queue*>(floors + kBlockRows);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    mbar_init(&bars->a_full, 1);
    mbar_init(&bars->a_empty, 1);
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&bars->b_full[s], 1);
      mbar_init(&bars->b_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], 2 * kPairScanWarps);
    }
    bars->abort_flag = (smem_u32(raw_smem) & 1023u) ? 1 : 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i < kPairInsertWarps * static_cast<int>(sizeof(Queue) / 4); i += kPairThreads)
    reinterpret_cast<uint32_t*>(queues)[i] = 0;
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                           // the peer's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  const int units = p.unit_pairs * p.splits;
  const int cluster_id = blockIdx.x >> 1, clusters = gridDim.x >> 1;
  constexpr uint32_t kTileBytes = KB * kSubTileBytes;   // what ONE CTA loads per key tile / query tile
  uint32_t issued_mask = 0, issued_parity = 0;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      const uint32_t leader_a_full = map_to_cta(smem_u32(&bars->a_full), 0);
      uint32_t stage = 0, b_phase = 0, a_phase = 0;
      bool ok = true;
      for (int unit = cluster_id; unit < units && ok; unit += clusters) {
        const int split = unit / p.unit_pairs, pair = unit % p.unit_pairs;
        if (unit != cluster_id) {
          ok = mbar_wait(&bars->a_empty, a_phase, abort_flag);
          a_phase ^= 1u;
          if (!ok) break;
        }
        if (leader) mbar_expect_tx(&bars->a_full, 2 * kTileBytes);
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d_pair(smem_a + kb * kSubTileBytes, &map_q, kb * kAtomK,
                           pair * kUnitRows + static_cast<int>(rank) * kBlockRows, leader_a_full);
        const int t0 = split * p.tiles_per_split;
        const int t1 = min(t0 + p.tiles_per_split, p.tiles_total);
        for (int t = t0; t < t1; ++t) {
          ok = mbar_wait(&bars->b_empty[stage], b_phase ^ 1u, abort_flag);
          if (!ok) break;
          if (leader) mbar_expect_tx(&bars->b_full[stage], 2 * kTileBytes);
          const uint32_t leader_full = map_to_cta(smem_u32(&bars->b_full[stage]), 0);
          for (int kb = 0; kb < KB; ++kb)
            tma_load_2d_pair(smem_b + (stage * KB + kb) * kSubTileBytes, &map_k, kb * kAtomK,
                             t * kPairTileCols + static_cast<int>(rank) * kBlockRows, leader_full);
          issued_mask |= 1u << stage;
          issued_parity = (issued_parity & ~(1u << stage)) | (b_phase << stage);
          if (++stage == kPairStages) { stage = 0; b_phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      uint32_t stage = 0, b_phase = 0, a_phase = 0, acc_phase[2] = {0, 0};
      uint32_t tile_counter = 0;
      bool ok = true;
      int done = 0;
      for (int unit = cluster_id; unit < units && ok; unit += clusters) {
        const int split = unit / p.unit_pairs;
        ok = mbar_wait(&bars->a_full, a_phase, abort_flag);
        a_phase ^= 1u;
        if (!ok) break;
        const int t0 = split * p.tiles_per_split;
        const int t1 = min(t0 + p.tiles_per_split, p.tiles_total);
        for (int t = t0; t < t1; ++t, ++tile_counter) {
          const uint32_t buf = tile_counter & 1u;
          ok = mbar_wait(&bars->b_full[stage], b_phase, abort_flag);
          if (!ok) break;
          ok = mbar_wait(&bars->acc_empty[buf], acc_phase[buf] ^ 1u, abort_flag);
          if (!ok) break;
          acc_phase[buf] ^= 1u;
          tc_fence_after();
          const uint32_t d = tmem_base + buf * kPairTileCols;
#pragma unroll
          for (int kk = 0; kk < KB * 4; ++kk) {
            const uint32_t a_addr = smem_u32(smem_a + (kk / 4) * kSubTileBytes) + (kk % 4) * 32;
            const uint32_t b_addr = smem_u32(smem_b + (stage * KB + kk / 4) * kSubTileBytes) + (kk % 4) * 32;
            umma_bf16_pair(d, umma_desc(a_addr), umma_desc(b_addr), kk > 0);
          }
          umma_commit_pair(&bars->b_empty[stage]);
          umma_commit_pair(&bars->acc_full[buf]);
          if (++stage == kPairStages) { stage = 0; b_phase ^= 1u; }
        }
        umma_commit_pair(&bars->a_empty);
        ++done;
      }
      if (ok && done > 0) mbar_wait(&bars->a_empty, static_cast<uint32_t>(done - 1) & 1u, abort_flag);
    }
  } else if (warp < 2 + kPairScanWarps) {
    // ---------------------------------------------------------------- scanners
    const int quarter = warp & 3;               // tensor-memory lane quarter this warp may read
    const int col_half = (warp - 2) >> 2;       // which 128 of the tile's 256 columns
    const int row = quarter * 32 + lane;        // row of this CTA's 128
    Queue* q = queues + quarter;
    volatile float* my_floor = floors + row;
    const uint32_t row_tag = static_cast<uint32_t>(lane) << 24;
    const uint32_t leader_empty[2] = {map_to_cta(smem_u32(&bars->acc_empty[0]), 0),
                                      map_to_cta(smem_u32(&bars->acc_empty[1]), 0)};
    uint32_t acc_phase[2] = {0, 0};
    uint32_t tile_counter = 0, unit_local = 0;
    bool ok = true;
    for (int unit = cluster_id; unit < units && ok; unit += clusters, ++unit_local) {
      const int split = unit / p.unit_pairs;
      for (uint32_t spin = 0; *reinterpret_cast<volatile uint32_t*>(&q->epoch) < unit_local; ++spin)
        if (spin >= kSpinLimit || ((spin & 1023u) == 1023u && *abort_flag)) { *abort_flag = 1; ok = false; break; }
      if (!__all_sync(kFullMask, ok)) { ok = false; break; }
      const int t0 = split * p.tiles_per_split;
      const int t1 = min(t0 + p.tiles_per_split, p.tiles_total);
      for (int t = t0; t < t1 && ok; ++t, ++tile_counter) {
        const uint32_t buf = tile_counter & 1u;
        ok = mbar_wait(&bars->acc_full[buf], acc_phase[buf], abort_flag);
        if (!ok) break;
        acc_phase[buf] ^= 1u;
        tc_fence_after();
        const int64_t col0 = static_cast<int64_t>(t) * kPairTileCols + col_half * 128;
        const int64_t left = p.slots - col0;
        const int live_cols = left < 128 ? static_cast<int>(left < 0 ? 0 : left) : 128;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kPairTileCols +
                               col_half * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[64];
          tmem_load32(taddr + h * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
          tmem_load32(taddr + h * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
          tmem_wait_loads();
          const float floor = *my_floor;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const float best = max_of_32(&r[c * 32]);
            if (!__any_sync(kFullMask, best >= floor)) continue;
            const int first = h * 64 + c * 32;
            uint32_t mine = 0;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              mine |= (__uint_as_float(r[c * 32 + i]) >= floor && first + i < live_cols) ? (1u << i) : 0u;
            uint32_t cols = __reduce_or_sync(kFullMask, mine);
            const uint32_t slot0 = static_cast<uint32_t>(col0) + first;
            while (cols && ok) {
              const int i = __ffs(cols) - 1;
              cols &= cols - 1;
              const float v = __uint_as_float(tmem_load1(taddr + first + i));
              const bool pass = (mine >> i) & 1u;
              const unsigned m = __ballot_sync(kFullMask, pass);
              ok = queue_push(q, m, pass, pack_key(orderable_bits(v), row_tag | (slot0 + i)), lane, abort_flag);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_empty[buf]);
      }
      __threadfence_block();
      __syncwarp();
      if (lane == 0) atomicAdd(&q->done, 1u);
    }
  } else {
    // ---------------------------------------------------------------- inserters
    const int iw = warp - 2 - kPairScanWarps;   // rows [32*iw, 32*iw + 32) of this CTA: lane quarter iw
    Queue* q = queues + iw;
    uint64_t* lists = all_lists + static_cast<size_t>(iw) * 32 * 32;
    float* floor_s = floors + iw * 32;
    const int K = p.width;
    uint32_t head = 0, units_done = 0;
    bool ok = true;
    for (int r = 0; r < 32; ++r) lists[r * 32 + lane] = 0;
    floor_s[lane] = -INFINITY;
    __syncwarp();
    for (int unit = cluster_id; unit < units && ok; unit += clusters) {
      const int split = unit / p.unit_pairs, pair = unit % p.unit_pairs;
      uint32_t idle = 0;
      for (;;) {
        const uint64_t e = *reinterpret_cast<volatile uint64_t*>(&q->slot[(head + lane) & (kQueueSlots - 1)]);
        const unsigned ready = __ballot_sync(kFullMask, e != 0);
        const int count = (ready == kFullMask) ? 32 : __ffs(~ready) - 1;
        if (count == 0) {
          const uint32_t finished = *reinterpret_cast<volatile uint32_t*>(&q->done);
          const uint32_t tail = *reinterpret_cast<volatile uint32_t*>(&q->tail);
          // two scanner warps feed a queue: the two column halves of this lane quarter
          if (finished == 2u * (units_done + 1u) && tail == head) break;
          if (++idle >= kIdleLimit || ((idle & 1023u) == 0 && *abort_flag)) { *abort_flag = 1; ok = false; break; }
          __nanosleep(kIdleNanoseconds);   // an idle poll loop costs issue slots and, under the power cap, clock
          continue;
        }
        idle = 0;
        for (int j = 0; j < count; ++j) {
          const uint64_t entry = shfl_u64(e, j);
          const int row = static_cast<int>(entry >> 24) & 31;
          const uint64_t key = (entry & 0xffffffff00000000ull) | (entry & 0xffffffull);
          uint64_t* row_list = lists + row * 32;
          const uint64_t cur = row_list[lane];
          const int pos = __popc(__ballot_sync(kFullMask, cur > key));
          if (pos < K) {
            const uint64_t up = __shfl_up_sync(kFullMask, cur, 1);
            const uint64_t ne = lane < pos ? cur : (lane == pos ? key : up);
            row_list[lane] = ne;
            if (lane == K - 1)
              *reinterpret_cast<volatile float*>(&floor_s[row]) =
                  ne ? from_orderable_bits(static_cast<uint32_t>(ne >> 32)) : -INFINITY;
          }
        }
        if (lane < count) *reinterpret_cast<volatile uint64_t*>(&q->slot[(head + lane) & (kQueueSlots - 1)]) = 0;
        __threadfence_block();
        __syncwarp();
        head += count;
        if (lane == 0) *reinterpret_cast<volatile uint32_t*>(&q->head) = head;
      }
      if (!ok) break;
      __syncwarp();
      for (int r = 0; r < 32; ++r) {
        const int64_t row = static_cast<int64_t>(pair) * kUnitRows + static_cast<int64_t>(rank) * kBlockRows + iw * 32 + r;
        const uint64_t e = lists[r * 32 + lane];
        if (row < p.rows && lane < K) {
          const int64_t at = (static_cast<int64_t>(split) * p.rows + row) * K + lane;
          p.out_score[at] = e ? from_orderable_bits(static_cast<uint32_t>(e >> 32)) : -INFINITY;
          p.out_slot[at] = e ? static_cast<int32_t>(p.col_base + static_cast<int64_t>(e & 0xffffffull)) : -1;
        }
        lists[r * 32 + lane] = 0;
      }
      floor_s[lane] = -INFINITY;
      __threadfence_block();
      __syncwarp();
      ++units_done;
      if (lane == 0) *reinterpret_cast<volatile uint32_t*>(&q->epoch) = units_done;
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.device_status != nullptr) atomicOr(p.device_status, GLSDM_DEV_WAIT_EXPIRED);
    // this CTA's own key-tile requests (they write THIS CTA's shared memory) must have landed;
    // their completion is visible on the leader's barrier only, so the peer just waits a while
    if (threadIdx.x == 0) {
      for (int s = 0; s < kPairStages; ++s) {
        if (!(issued_mask & (1u << s))) continue;
        for (uint32_t spin = 0; spin < (1u << 20); ++spin)
          if (leader ? mbar_try_wait(&bars->b_full[s], (issued_parity >> s) & 1u) : (spin > (1u << 16))) break;
      }
    }
    __syncthreads();
  }
  // neither CTA may leave (or free tensor memory) while the other can still signal its barriers
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols));
  }
}

}  // namespace dense
}  // namespace glsdm
