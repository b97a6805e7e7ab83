// Dense-key routing, wide-tile variant: one CTA per unit of 128 query rows, key tiles of 256
// slots, tcgen05.mma of shape 128 x 256 x 16 (cta_group::1). An MMA of N = 256 reads its A
// operand once for twice the columns, so the tensor pipe asks shared memory for 96 bytes per
// clock instead of the 128 of two N = 128 instructions - measured on B200 the bare MMA + TMA
// pipeline rises from 1120 to 1320 TFLOP/s. The price is that a key tile now serves 128 rows
// instead of 256, i.e. twice the L2-to-shared traffic per FLOP (64 B/clk per SM at full rate).
// Accumulators: 128 lanes x 256 columns x 2 buffers of tensor memory. Scanning, queues and
// inserters are the single-CTA kernel's: 8 scanner warps (4 lane quarters x 2 column halves,
// thread = one row x 128 columns), 4 inserter warps (32 rows each). Every wait is bounded.
#pragma once

#include "score_topk.cuh"

namespace glsdm {
namespace dense {

constexpr int kWideTileCols = 256;                 // slots per key tile (MMA N)
constexpr int kWideSubTileBytes = kWideTileCols * 128;   // one [256 x 64] bf16 sub-tile, 32 KB
constexpr int kWideStages = 2;
constexpr int kWideScanWarps = 8;
constexpr int kWideInsertWarps = 4;                 // one per lane quarter (32 rows), fed by its two scanner warps
constexpr int kWideThreads = 32 * (2 + kWideScanWarps + kWideInsertWarps);
constexpr uint32_t kWideInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kWideTileCols >> 3) << 17) |
                                    ((kBlockRows >> 4) << 24);

__device__ __forceinline__ void umma_bf16_wide(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kWideInstrDesc), "r"(acc)
      : "memory");
}

struct WideBarriers {
  uint64_t a_full;
  uint64_t a_empty;
  uint64_t b_full[kWideStages];
  uint64_t b_empty[kWideStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Shared memory: [A: kb sub-tiles of 128 rows][B: stages x kb sub-tiles of 256 rows][lists][barriers]
template <int KB>
struct WideLayout {
  static constexpr int kA = KB * kSubTileBytes;
  static constexpr int kB = kWideStages * KB * kWideSubTileBytes;
  static constexpr int kListOffset = kA + kB;
  static constexpr int kListBytes = 8 * 32 * kBlockRows;
  __host__ __device__ static constexpr int total() {
    return kListOffset + kListBytes + static_cast<int>(sizeof(WideBarriers)) + 4 * kBlockRows +
           kWideInsertWarps * static_cast<int>(sizeof(Queue)) + 64;
  }
};

// One exchange of bounds for the 32 rows of an inserter warp (lane r: row r): store the K-th best
// score the row has reached where it rose since the last time, raise the floor to what the peers
// have stored. Out of line: it runs a few hundred times per unit, the kernel around it is tuned.
__device__ __noinline__ void exchange_row_bounds(const Params& p, const uint64_t* lists, float* floor_s, int block,
                                                 int iw, int lane, int K, float& seed, float& told) {
  const int64_t row = static_cast<int64_t>(block) * kBlockRows + iw * 32 + lane;
  if (row >= p.rows) return;
  const int64_t name = (row + p.row_shift) % p.rows;
  const uint64_t last = lists[lane * 32 + K - 1];
  const float mine = last ? from_orderable_bits(static_cast<uint32_t>(last >> 32)) : -INFINITY;
  if (mine > told) {
    told = mine;
    for (int peer = 0; peer < p.floor_peers; ++peer) p.floor_out[peer][name] = mine;
  }
  float bound = seed;
  for (int src = 0; src < p.floor_sources; ++src)
    bound = fmaxf(bound, __ldcg(p.floor_in + static_cast<int64_t>(src) * p.rows + name));
  if (bound > seed) {
    seed = bound;
    if (bound > mine) *reinterpret_cast<volatile float*>(&floor_s[lane]) = bound;
  }
}

// kBounds: the instantiation that takes and gives row bounds (row_floor, floor_in, floor_out).
// The plain one is compiled without any of it, so a single GPU runs exactly the kernel it ran
// before bounds existed.
template <int KB, bool kBounds>
__global__ void __launch_bounds__(kWideThreads, 1)
score_topk_wide_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, Params p) {
  extern __shared__ __align__(1024) uint8_t raw_smem[];
  uint8_t* smem_a = raw_smem;
  uint8_t* smem_b = raw_smem + WideLayout<KB>::kA;
  uint64_t* all_lists = reinterpret_cast<uint64_t*>(raw_smem + WideLayout<KB>::kListOffset);
  WideBarriers* bars = reinterpret_cast<WideBarriers*>(raw_smem + WideLayout<KB>::kListOffset + WideLayout<KB>::kListBytes);
  float* floors = reinterpret_cast<float*>(bars + 1);
  Queue* queues = reinterpret_cast<Queue*>(floors + kBlockRows);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&bars->a_full, 1);
    mbar_init(&bars->a_empty, 1);
    for (int s = 0; s < kWideStages; ++s) {
      mbar_init(&bars->b_full[s], 1);
      mbar_init(&bars->b_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], kWideScanWarps);
    }
    bars->abort_flag = (smem_u32(raw_smem) & 1023u) ? 1 : 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i < kWideInsertWarps * static_cast<int>(sizeof(Queue) / 4); i += kWideThreads)
    reinterpret_cast<uint32_t*>(queues)[i] = 0;
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  const int units = unit_count(p);
  const int first_unit = blockIdx.x, unit_stride = gridDim.x;
  constexpr uint32_t kQueryBytes = KB * kSubTileBytes;          // 128 query rows
  constexpr uint32_t kKeyBytes = KB * kWideSubTileBytes;        // 256 key rows
  uint32_t issued_mask = 0, issued_parity = 0;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t stage = 0, b_phase = 0, a_phase = 0;
      bool ok = true;
      for (int unit = first_unit; unit < units && ok; unit += unit_stride) {
        const UnitSpan span = unit_span(p, unit);
        const int pair = span.block;
        if (unit != first_unit) {
          ok = mbar_wait(&bars->a_empty, a_phase, abort_flag);
          a_phase ^= 1u;
          if (!ok) break;
        }
        mbar_expect_tx(&bars->a_full, kQueryBytes);
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d(smem_a + kb * kSubTileBytes, &map_q, kb * kAtomK, pair * kBlockRows, &bars->a_full);
        const int t0 = span.t0, t1 = span.t1;
        for (int t = t0; t < t1; ++t) {
          ok = mbar_wait(&bars->b_empty[stage], b_phase ^ 1u, abort_flag);
          if (!ok) break;
          mbar_expect_tx(&bars->b_full[stage], kKeyBytes);
          for (int kb = 0; kb < KB; ++kb)
            tma_load_2d(smem_b + (stage * KB + kb) * kWideSubTileBytes, &map_k, kb * kAtomK, t * kWideTileCols,
                        &bars->b_full[stage]);
          issued_mask |= 1u << stage;
          issued_parity = (issued_parity & ~(1u << stage)) | (b_phase << stage);
          if (++stage == kWideStages) { stage = 0; b_phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t stage = 0, b_phase = 0, a_phase = 0, acc_phase[2] = {0, 0};
      uint32_t tile_counter = 0;
      bool ok = true;
      int done = 0;
      for (int unit = first_unit; unit < units && ok; unit += unit_stride) {
        const UnitSpan span = unit_span(p, unit);
        ok = mbar_wait(&bars->a_full, a_phase, abort_flag);
        a_phase ^= 1u;
        if (!ok) break;
        const int t0 = span.t0, t1 = span.t1;
        for (int t = t0; t < t1; ++t, ++tile_counter) {
          const uint32_t buf = tile_counter & 1u;
          ok = mbar_wait(&bars->b_full[stage], b_phase, abort_flag);
          if (!ok) break;
          ok = mbar_wait(&bars->acc_empty[buf], acc_phase[buf] ^ 1u, abort_flag);
          if (!ok) break;
          acc_phase[buf] ^= 1u;
          tc_fence_after();
          const uint32_t d = tmem_base + buf * kWideTileCols;
#pragma unroll
          for (int kk = 0; kk < KB * 4; ++kk) {
            const uint32_t a_addr = smem_u32(smem_a + (kk / 4) * kSubTileBytes) + (kk % 4) * 32;
            const uint32_t b_addr = smem_u32(smem_b + (stage * KB + kk / 4) * kWideSubTileBytes) + (kk % 4) * 32;
            umma_bf16_wide(d, umma_desc(a_addr), umma_desc(b_addr), kk > 0);
          }
          umma_commit(&bars->b_empty[stage]);
          umma_commit(&bars->acc_full[buf]);
          if (++stage == kWideStages) { stage = 0; b_phase ^= 1u; }
        }
        umma_commit(&bars->a_empty);
        ++done;
      }
      if (ok && done > 0) mbar_wait(&bars->a_empty, static_cast<uint32_t>(done - 1) & 1u, abort_flag);
    }
  } else if (warp < 2 + kWideScanWarps) {
    // ---------------------------------------------------------------- scanners
    const int quarter = warp & 3;               // tensor-memory lane quarter this warp may read
    const int col_half = (warp - 2) >> 2;       // which 128 of the tile's 256 columns
    const int row = quarter * 32 + lane;        // row of this CTA's 128
    Queue* q = queues + quarter;
    volatile float* my_floor = floors + row;
    const uint32_t row_tag = static_cast<uint32_t>(lane) << 24;
    uint32_t acc_phase[2] = {0, 0};
    uint32_t tile_counter = 0, unit_local = 0;
    bool ok = true;
    for (int unit = first_unit; unit < units && ok; unit += unit_stride, ++unit_local) {
      const UnitSpan span = unit_span(p, unit);
      for (uint32_t spin = 0; *reinterpret_cast<volatile uint32_t*>(&q->epoch) < unit_local; ++spin)
        if (spin >= kSpinLimit || ((spin & 1023u) == 1023u && *abort_flag)) { *abort_flag = 1; ok = false; break; }
      if (!__all_sync(kFullMask, ok)) { ok = false; break; }
      const int t0 = span.t0, t1 = span.t1;
      // Rows past the end of the batch are zero-filled by the tile load: all their scores are
      // equal, and with ties preferring the larger slot EVERY column would replace the one
      // before it in their lists (measured: 5.8 ms instead of 0.1 ms for 96 rows x 2,048
      // slots). Their floor is +inf, so nothing of them is ever queued.
      const bool row_live = static_cast<int64_t>(span.block) * kBlockRows + row < p.rows;
      for (int t = t0; t < t1 && ok; ++t, ++tile_counter) {
        const uint32_t buf = tile_counter & 1u;
        ok = mbar_wait(&bars->acc_full[buf], acc_phase[buf], abort_flag);
        if (!ok) break;
        acc_phase[buf] ^= 1u;
        tc_fence_after();
        const int64_t col0 = static_cast<int64_t>(t) * kWideTileCols + col_half * 128;
        const int64_t left = p.slots - col0;
        const int live_cols = left < 128 ? static_cast<int>(left < 0 ? 0 : left) : 128;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kWideTileCols +
                               col_half * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[64];
          tmem_load32(taddr + h * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
          tmem_load32(taddr + h * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
          tmem_wait_loads();
          const float floor = row_live ? *my_floor : INFINITY;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            float group[11];
            const float best = max_of_32(&r[c * 32], group);
            if (!__any_sync(kFullMask, best >= floor)) continue;
            // Rare path: one bit per passing column (looking only into the three-column groups
            // whose maximum passes in some row), then a loop over the columns that passed in
            // any row, re-reading that single column from tensor memory.
            const int first = h * 64 + c * 32;
            uint32_t mine = 0;
#pragma unroll
            for (int j = 0; j < 11; ++j) {
              if (!__any_sync(kFullMask, group[j] >= floor)) continue;
#pragma unroll
              for (int i = 3 * j; i < (j < 10 ? 3 * j + 3 : 32); ++i)
                mine |= (__uint_as_float(r[c * 32 + i]) >= floor) ? (1u << i) : 0u;
            }
            if (live_cols < 128) {              // the ragged last tile: columns past the end never count
              const int valid = live_cols - first;
              mine &= valid >= 32 ? 0xffffffffu : (valid <= 0 ? 0u : (1u << valid) - 1u);
            }
            uint32_t cols = __reduce_or_sync(kFullMask, mine);
            const uint32_t slot0 = static_cast<uint32_t>(col0) + first;
            while (cols && ok) {
              const int i = __ffs(cols) - 1;
              cols &= cols - 1;
              const float v = __uint_as_float(tmem_load1(taddr + first + i));
              // the floor may have risen since the chunk was tested: a fresh look spares the
              // inserter candidates it would only throw away (6 % less start-up time per unit)
              const bool pass = ((mine >> i) & 1u) && v >= *my_floor;
              const unsigned m = __ballot_sync(kFullMask, pass);
              ok = queue_push(q, m, pass, pack_key(orderable_bits(v), row_tag | (slot0 + i)), lane, abort_flag);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->acc_empty[buf]);
      }
      __threadfence_block();
      __syncwarp();
      if (lane == 0) atomicAdd(&q->done, 1u);
    }
  } else {
    // ---------------------------------------------------------------- inserters
    const int iw = warp - 2 - kWideScanWarps;   // rows [32*iw, 32*iw + 32) of the unit: lane quarter iw
    Queue* q = queues + iw;
    uint64_t* lists = all_lists + static_cast<size_t>(iw) * 32 * 32;
    float* floor_s = floors + iw * 32;
    const int K = p.width;
    uint32_t head = 0, units_done = 0;
    bool ok = true;
    for (int r = 0; r < 32; ++r) lists[r * 32 + lane] = 0;
    // A caller may know a score that the K-th best of a row is sure to reach (row_floor): the
    // row's floor starts there instead of at -inf, and candidates below it are never queued.
    auto seed_for = [&](int unit_index) -> float {
      if constexpr (!kBounds) return -INFINITY;
      if ((p.row_floor == nullptr && p.floor_sources == 0) || unit_index >= units) return -INFINITY;
      const UnitSpan s = unit_span(p, unit_index);
      const int64_t r = static_cast<int64_t>(s.block) * kBlockRows + iw * 32 + lane;
      if (r >= p.rows) return -INFINITY;
      float bound = p.row_floor != nullptr ? p.row_floor[r] : -INFINITY;
      const int64_t name = (r + p.row_shift) % p.rows;
      for (int src = 0; src < p.floor_sources; ++src)    // peers write these while we run: read past L1
        bound = fmaxf(bound, __ldcg(p.floor_in + static_cast<int64_t>(src) * p.rows + name));
      return bound;
    };
    float seed = seed_for(first_unit);
    floor_s[lane] = seed;
    __syncwarp();
    // While a unit runs, the shards that scan the same rows at the same time (their first waves
    // overlap) keep each other informed: every so many looks at its queue this warp stores the K-th best
    // score its 32 rows have reached so far where it rose, and raises its floors to what the
    // peers have stored. A bound above the row's own K-th entry simply closes the row earlier.
    const bool sharing = kBounds && (p.floor_peers > 0 || p.floor_sources > 0);
    float told = -INFINITY;    // lane r: the last bound stored for row r of this unit
    uint32_t batches = 0;
    auto refresh_bounds = [&](int block) { exchange_row_bounds(p, lists, floor_s, block, iw, lane, K, seed, told); };
    for (int unit = first_unit; unit < units && ok; unit += unit_stride) {
      const UnitSpan span = unit_span(p, unit);
      const int pair = span.block;
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
          if (sharing && (idle & p.floor_refresh_mask) == 0) refresh_bounds(pair);
          // Nothing queued: most of a unit is like this. Polling flat out would spend issue
          // slots and, on a power-capped part, clock rate that the tensor pipe can use
          // (measured: 1166 -> 1197 TFLOP/s sustained on 65,536 rows x 16.7M slots).
          __nanosleep(kIdleNanoseconds);
          continue;
        }
        idle = 0;
        // One insertion: the warp holds the row's list (lane j = entry j, best first), finds the
        // key's place with a ballot and shifts the tail down by one lane.
        auto insert_one = [&](uint64_t entry) {
          const int row = static_cast<int>(entry >> 24) & 31;
          const uint64_t key = (entry & 0xffffffff00000000ull) | (entry & 0xffffffull);
          uint64_t* row_list = lists + row * 32;
          const uint64_t cur = row_list[lane];
          const int pos = __popc(__ballot_sync(kFullMask, cur > key));
          float row_seed = -INFINITY;
          if constexpr (kBounds) row_seed = __shfl_sync(kFullMask, seed, row);
          if (pos < K) {
            const uint64_t up = __shfl_up_sync(kFullMask, cur, 1);
            const uint64_t ne = lane < pos ? cur : (lane == pos ? key : up);
            row_list[lane] = ne;
            if (lane == K - 1)
              *reinterpret_cast<volatile float*>(&floor_s[row]) =
                  ne ? (kBounds ? fmaxf(from_orderable_bits(static_cast<uint32_t>(ne >> 32)), row_seed)
                                : from_orderable_bits(static_cast<uint32_t>(ne >> 32)))
                     : row_seed;
          }
        };
        // Entries of four different rows are independent: their list loads, ballots and
        // stores are issued together, which hides the shared-memory and vote latencies that a
        // single insertion spends waiting (the start of a unit is nothing but insertions).
        int j = 0;
        for (; j + 4 <= count; j += 4) {
          uint64_t entry[4];
          int row[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            entry[i] = shfl_u64(e, j + i);
            row[i] = static_cast<int>(entry[i] >> 24) & 31;
          }
          const bool distinct = row[0] != row[1] && row[0] != row[2] && row[0] != row[3] && row[1] != row[2] &&
                                row[1] != row[3] && row[2] != row[3];
          if (!distinct) {
#pragma unroll
            for (int i = 0; i < 4; ++i) insert_one(entry[i]);
            continue;
          }
          uint64_t key[4], cur[4];
          int pos[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            key[i] = (entry[i] & 0xffffffff00000000ull) | (entry[i] & 0xffffffull);
            cur[i] = lists[row[i] * 32 + lane];
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) pos[i] = __popc(__ballot_sync(kFullMask, cur[i] > key[i]));
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint64_t up = __shfl_up_sync(kFullMask, cur[i], 1);
            float row_seed = -INFINITY;
            if constexpr (kBounds) row_seed = __shfl_sync(kFullMask, seed, row[i]);
            if (pos[i] < K) {
              const uint64_t ne = lane < pos[i] ? cur[i] : (lane == pos[i] ? key[i] : up);
              lists[row[i] * 32 + lane] = ne;
              if (lane == K - 1)
                *reinterpret_cast<volatile float*>(&floor_s[row[i]]) =
                    ne ? (kBounds ? fmaxf(from_orderable_bits(static_cast<uint32_t>(ne >> 32)), row_seed)
                                  : from_orderable_bits(static_cast<uint32_t>(ne >> 32)))
                       : row_seed;
            }
          }
        }
        for (; j < count; ++j) insert_one(shfl_u64(e, j));
        if (lane < count) *reinterpret_cast<volatile uint64_t*>(&q->slot[(head + lane) & (kQueueSlots - 1)]) = 0;
        __threadfence_block();
        __syncwarp();
        head += count;
        if (lane == 0) *reinterpret_cast<volatile uint32_t*>(&q->head) = head;
        // the start of a unit is all insertions and no idle look: exchange there too
        if (sharing && (++batches & p.floor_refresh_mask) == 0) refresh_bounds(pair);
      }
      if (!ok) break;
      __syncwarp();
      float reached = -INFINITY;   // lane r: the K-th best score row r ended with (-inf: fewer than K qualified)
      for (int r = 0; r < 32; ++r) {
        const int64_t row = static_cast<int64_t>(pair) * kBlockRows + iw * 32 + r;
        const uint64_t e = lists[r * 32 + lane];
        if (kBounds && p.floor_peers > 0) {
          const uint64_t last = shfl_u64(e, K - 1);
          if (lane == r && last != 0) reached = from_orderable_bits(static_cast<uint32_t>(last >> 32));
        }
        if (row < p.rows && lane < K) {
          const float score = e ? from_orderable_bits(static_cast<uint32_t>(e >> 32)) : -INFINITY;
          const int32_t slot = e ? static_cast<int32_t>(p.col_base + static_cast<int64_t>(e & 0xffffffull)) : -1;
          if (span.tail) {
            const int64_t tail_rows = p.rows - static_cast<int64_t>(p.unit_pairs) * kBlockRows;
            const int64_t at = (static_cast<int64_t>(span.part) * tail_rows +
                                (row - static_cast<int64_t>(p.unit_pairs) * kBlockRows)) * K + lane;
            p.tail_score[at] = score;
            p.tail_slot[at] = slot;
          } else {
            const int64_t at = (static_cast<int64_t>(span.part) * p.rows + row) * K + lane;
            p.out_score[at] = score;
            p.out_slot[at] = slot;
          }
        }
        lists[r * 32 + lane] = 0;
      }
      if (kBounds && p.floor_peers > 0 && reached > told) {
        // The K-th best over a part of the bank never exceeds the K-th best over all of it: a
        // valid bound for every other shard, whichever part of the slot range this unit covered.
        const int64_t row = static_cast<int64_t>(pair) * kBlockRows + iw * 32 + lane;
        if (row < p.rows) {
          const int64_t name = (row + p.row_shift) % p.rows;
          for (int peer = 0; peer < p.floor_peers; ++peer) p.floor_out[peer][name] = reached;
        }
      }
      told = -INFINITY;
      seed = seed_for(unit + unit_stride);
      floor_s[lane] = seed;
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
    // Key tiles that were requested but never consumed still write shared memory: give
    // the latest request of each stage a bounded chance to land before the CTA exits.
    if (threadIdx.x == 0) {
      for (int s = 0; s < kWideStages; ++s) {
        if (!(issued_mask & (1u << s))) continue;
        for (uint32_t spin = 0; spin < (1u << 20); ++spin)
          if (mbar_try_wait(&bars->b_full[s], (issued_parity >> s) & 1u)) break;
      }
    }
    __syncthreads();
  }
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols));
  }
}

}  // namespace dense
}  // namespace glsdm
