// Dense-key routing: scores = queries x keys^T on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory), fused with a running per-row top-k in the
// epilogue, so the [rows, slots] score matrix never leaves the SM.
//
// One persistent CTA per SM, 14 warps:
//   warp 0     TMA producer: the unit's query tile (2 x 128 rows) once, then key tiles of
//              128 slots through a 3-stage shared-memory ring (128-byte swizzle, K-major)
//   warp 1     allocates tensor memory (512 columns) and issues tcgen05.mma from one thread:
//              per key tile, 2 row blocks x dk/16 instructions of shape 128 x 128 x 16
//              (bf16 in, fp32 accumulate); accumulators are double-buffered in tensor memory
//   warps 2-9  scanners: thread = one query row; tcgen05.ld moves 64 columns at a time to
//              registers, a running max against the row's floor (its current k-th score)
//              rejects most 32-column groups with one compare; survivors are pushed into a
//              small shared-memory queue and the accumulator buffer goes back to the MMA warp
//   warps 10-13 inserters: each drains the queue of two scanner warps (64 rows) and inserts
//              the candidates into the rows' sorted lists in shared memory, the whole warp
//              working on one list at a time; they publish the new floors to the scanners.
//              Scanning thus never waits for an insertion (only for queue space).
// A unit is (pair of 128-row blocks, one split of the slot range). Each unit writes its
// rows' best `width` (score, slot) pairs; with more than one split a small merge kernel
// reduces the splits. Units are ordered split-major so that the CTAs running at the same time
// stream the same keys and share them through L2.
//
// Every wait on an mbarrier is bounded: when a wait runs out the CTA raises a shared abort
// flag, sets GLSDM_DEV_WAIT_EXPIRED in the caller's status word, drains its outstanding
// loads (bounded again), frees its tensor memory and returns.
//
// Tie rule (gl_sdm/memory/routing.py:21-24): equal scores prefer the larger slot. Slots are
// scanned in ascending order, so a score equal to the current k-th one replaces it.
#include "score_topk.cuh"
#include "score_topk_wide.cuh"

namespace glsdm {
namespace {

using namespace dense;

struct Barriers {
  uint64_t a_full;
  uint64_t a_empty;
  uint64_t b_full[kStages];
  uint64_t b_empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Shared memory: [A: 2 row blocks x kb sub-tiles][B: stages x kb sub-tiles][lists][barriers]
template <int KB>
struct Layout {
  static constexpr int kA = 2 * KB * kSubTileBytes;
  static constexpr int kB = kStages * KB * kSubTileBytes;
  static constexpr int kListOffset = kA + kB;
  __host__ __device__ static constexpr int list_bytes(int) { return 8 * 32 * 32 * kEpilogueWarps; }
  __host__ __device__ static constexpr int total(int width) {
    return kListOffset + list_bytes(width) + static_cast<int>(sizeof(Barriers)) + 4 * 32 * kEpilogueWarps +
           kInsertWarps * static_cast<int>(sizeof(Queue)) + 64;
  }
};

template <int KB>
__global__ void __launch_bounds__(kThreads, 1)
score_topk_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, Params p) {
  // The 128-byte-swizzled tiles need a 1024-byte aligned base; dynamic shared memory starts
  // at the alignment the declaration asks for (checked below, the kernel refuses otherwise).
  extern __shared__ __align__(1024) uint8_t raw_smem[];
  uint8_t* smem = raw_smem;
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + Layout<KB>::kA;
  float* list_val = reinterpret_cast<float*>(smem + Layout<KB>::kListOffset);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + Layout<KB>::kListOffset + Layout<KB>::list_bytes(p.width));
  float* floors = reinterpret_cast<float*>(bars + 1);                       // [256] current k-th score per row
  Queue* queues = reinterpret_cast<Queue*>(floors + 32 * kEpilogueWarps);   // [kInsertWarps]
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&bars->a_full, 1);
    mbar_init(&bars->a_empty, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->b_full[s], 1);
      mbar_init(&bars->b_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], kEpilogueWarps);
    }
    bars->abort_flag = (smem_u32(raw_smem) & 1023u) ? 1 : 0;   // misaligned base: every role leaves at once
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i < kInsertWarps * static_cast<int>(sizeof(Queue) / 4); i += kThreads)
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

  const int units = p.unit_pairs * p.splits;
  constexpr uint32_t kTileBytes = KB * kSubTileBytes;
  // Thread 0 only: for every stage, whether a key tile was ever requested and under which
  // barrier parity the latest request completes (used to drain loads after an abort).
  uint32_t issued_mask = 0, issued_parity = 0;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t stage = 0, b_phase = 0, a_phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        const int split = unit / p.unit_pairs, pair = unit % p.unit_pairs;
        // the previous unit's MMAs must have finished reading the query tile
        if (unit != static_cast<int>(blockIdx.x)) {
          ok = mbar_wait(&bars->a_empty, a_phase, abort_flag);
          a_phase ^= 1u;
          if (!ok) break;
        }
        mbar_expect_tx(&bars->a_full, 2 * kTileBytes);
        for (int mb = 0; mb < 2; ++mb)
          for (int kb = 0; kb < KB; ++kb)
            tma_load_2d(smem_a + (mb * KB + kb) * kSubTileBytes, &map_q, kb * kAtomK,
                        pair * kUnitRows + mb * kBlockRows, &bars->a_full);
        const int t0 = split * p.tiles_per_split;
        const int t1 = min(t0 + p.tiles_per_split, p.tiles_total);
        for (int t = t0; t < t1; ++t) {
          ok = mbar_wait(&bars->b_empty[stage], b_phase ^ 1u, abort_flag);
          if (!ok) break;
          mbar_expect_tx(&bars->b_full[stage], kTileBytes);
          for (int kb = 0; kb < KB; ++kb)
            tma_load_2d(smem_b + (stage * KB + kb) * kSubTileBytes, &map_k, kb * kAtomK, t * kTileCols,
                        &bars->b_full[stage]);
          issued_mask |= 1u << stage;
          issued_parity = (issued_parity & ~(1u << stage)) | (b_phase << stage);
          if (++stage == kStages) { stage = 0; b_phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t stage = 0, b_phase = 0, a_phase = 0, acc_phase[2] = {0, 0};
      uint32_t tile_counter = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
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
#pragma unroll
          for (int mb = 0; mb < 2; ++mb) {
            const uint32_t d = tmem_base + buf * (2 * kTileCols) + mb * kTileCols;
#pragma unroll
            for (int kk = 0; kk < KB * 4; ++kk) {
              const uint32_t a_addr = smem_u32(smem_a + (mb * KB + kk / 4) * kSubTileBytes) + (kk % 4) * 32;
              const uint32_t b_addr = smem_u32(smem_b + (stage * KB + kk / 4) * kSubTileBytes) + (kk % 4) * 32;
              umma_bf16(d, umma_desc(a_addr), umma_desc(b_addr), kk > 0);
            }
          }
          umma_commit(&bars->b_empty[stage]);   // the stage is free once these MMAs have read it
          umma_commit(&bars->acc_full[buf]);    // the accumulators are complete
          if (++stage == kStages) { stage = 0; b_phase ^= 1u; }
        }
        umma_commit(&bars->a_empty);            // the query tile may be overwritten
      }
      // The last commit's arrival must land before this CTA's shared memory is released.
      if (ok && static_cast<int>(blockIdx.x) < units) {
        const int done = (units - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1;
        mbar_wait(&bars->a_empty, static_cast<uint32_t>(done - 1) & 1u, abort_flag);
      }
    }
  } else if (warp < 2 + kEpilogueWarps) {
    // ---------------------------------------------------------------- scanners
    // Scanner: lane = one query row of the unit. Row lists live with the inserter; the
    // scanner only compares against the row's published floor and queues what passes.
    const int ew = warp - 2;                    // 0..7
    const int mb = ew >> 2;                     // row block of this warp
    const int quarter = warp & 3;               // tensor-memory lane quarter this warp may read
    Queue* q = queues + (ew >> 1);
    volatile float* my_floor = floors + ew * 32 + lane;
    const uint32_t row_tag = static_cast<uint32_t>((ew & 1) * 32 + lane) << 24;
    uint32_t acc_phase[2] = {0, 0};
    uint32_t tile_counter = 0, unit_local = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++unit_local) {
      const int split = unit / p.unit_pairs;
      // the inserter must have written out and reset the previous unit's lists
      for (uint32_t spin = 0; *reinterpret_cast<volatile uint32_t*>(&q->epoch) < unit_local; ++spin)
        if (spin >= kSpinLimit || ((spin & 1023u) == 1023u && *abort_flag)) { *abort_flag = 1; ok = false; break; }
      if (!__all_sync(kFullMask, ok)) { ok = false; break; }
      const int t0 = split * p.tiles_per_split;
      const int t1 = min(t0 + p.tiles_per_split, p.tiles_total);
      // rows past the end of the batch (zero-filled, all scores equal) never queue anything
      const bool row_live = static_cast<int64_t>(unit % p.unit_pairs) * kUnitRows + mb * kBlockRows + quarter * 32 + lane < p.rows;
      for (int t = t0; t < t1 && ok; ++t, ++tile_counter) {
        const uint32_t buf = tile_counter & 1u;
        ok = mbar_wait(&bars->acc_full[buf], acc_phase[buf], abort_flag);
        if (!ok) break;
        acc_phase[buf] ^= 1u;
        tc_fence_after();
        const int64_t col0 = static_cast<int64_t>(t) * kTileCols;
        const int64_t left = p.slots - col0;
        const int live_cols = left < kTileCols ? static_cast<int>(left) : kTileCols;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * (2 * kTileCols) +
                               mb * kTileCols;
#pragma unroll
        for (int h = 0; h < 2; ++h) {           // two halves of 64 columns
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
            // Rare path. Registers cannot be indexed by a run-time column, and handling every
            // column inline would bloat the loop, so: one bit per passing column - looking only
            // into the three-column groups whose maximum passes in some row - then a short
            // loop over the columns that passed in any row, re-reading that single column
            // from tensor memory (the buffer is released only after the tile's events).
            const int first = h * 64 + c * 32;
            uint32_t mine = 0;
#pragma unroll
            for (int j = 0; j < 11; ++j) {
              if (!__any_sync(kFullMask, group[j] >= floor)) continue;
#pragma unroll
              for (int i = 3 * j; i < (j < 10 ? 3 * j + 3 : 32); ++i)
                mine |= (__uint_as_float(r[c * 32 + i]) >= floor) ? (1u << i) : 0u;
            }
            if (live_cols < kTileCols) {        // the ragged last tile: columns past the end never count
              const int valid = live_cols - first;
              mine &= valid >= 32 ? 0xffffffffu : (valid <= 0 ? 0u : (1u << valid) - 1u);
            }
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
        if (lane == 0) mbar_arrive(&bars->acc_empty[buf]);
      }
      // this warp has pushed everything of the unit
      __threadfence_block();
      __syncwarp();
      if (lane == 0) atomicAdd(&q->done, 1u);
    }
  } else {
    // ---------------------------------------------------------------- inserters
    // Inserter: drains one queue, keeps the sorted lists of its 64 rows (32 entries each, best
    // first; lane j holds entry j of the list being updated), publishes floors, and at the end
    // of a unit writes the lists out and resets them.
    const int iw = warp - 2 - kEpilogueWarps;   // 0..3
    Queue* q = queues + iw;
    uint64_t* lists = reinterpret_cast<uint64_t*>(list_val) + static_cast<size_t>(iw) * 64 * 32;
    float* floor_s = floors + iw * 64;
    const int K = p.width;
    uint32_t head = 0, units_done = 0;
    bool ok = true;
    for (int r = 0; r < 64; ++r) lists[r * 32 + lane] = 0;
    floor_s[lane] = -INFINITY;
    floor_s[32 + lane] = -INFINITY;
    __syncwarp();
    for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
      const int split = unit / p.unit_pairs, pair = unit % p.unit_pairs;
      uint32_t idle = 0;
      for (;;) {
        const uint64_t e = *reinterpret_cast<volatile uint64_t*>(&q->slot[(head + lane) & (kQueueSlots - 1)]);
        const unsigned ready = __ballot_sync(kFullMask, e != 0);
        const int count = (ready == kFullMask) ? 32 : __ffs(~ready) - 1;   // contiguous ready prefix
        if (count == 0) {
          const uint32_t finished = *reinterpret_cast<volatile uint32_t*>(&q->done);
          const uint32_t tail = *reinterpret_cast<volatile uint32_t*>(&q->tail);
          if (finished == 2u * (units_done + 1u) && tail == head) break;    // unit complete, queue empty
          if (++idle >= kIdleLimit || ((idle & 1023u) == 0 && *abort_flag)) { *abort_flag = 1; ok = false; break; }
          __nanosleep(kIdleNanoseconds);   // an idle poll loop costs issue slots and, under the power cap, clock
          continue;
        }
        idle = 0;
        for (int j = 0; j < count; ++j) {
          const uint64_t entry = shfl_u64(e, j);
          const int row = static_cast<int>(entry >> 24) & 63;
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
      // lane j writes entry j of each row: coalesced [row][width] stores, then reset the list
      for (int r = 0; r < 64; ++r) {
        const int ew = 2 * iw + (r >> 5);
        const int64_t row = static_cast<int64_t>(pair) * kUnitRows + (ew >> 2) * kBlockRows + ((ew + 2) & 3) * 32 + (r & 31);
        const uint64_t e = lists[r * 32 + lane];
        if (row < p.rows && lane < K) {
          const int64_t at = (static_cast<int64_t>(split) * p.rows + row) * K + lane;
          p.out_score[at] = e ? from_orderable_bits(static_cast<uint32_t>(e >> 32)) : -INFINITY;
          p.out_slot[at] = e ? static_cast<int32_t>(p.col_base + static_cast<int64_t>(e & 0xffffffull)) : -1;
        }
        lists[r * 32 + lane] = 0;
      }
      floor_s[lane] = -INFINITY;
      floor_s[32 + lane] = -INFINITY;
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
      for (int s = 0; s < kStages; ++s) {
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

// Merge of the per-split candidate lists of each row, best first (score desc, slot desc).
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
split_merge_kernel(const float* __restrict__ cand_score, const int32_t* __restrict__ cand_slot, int splits,
                   int64_t rows, int width, float* __restrict__ out_score, int32_t* __restrict__ out_slot) {
  __shared__ uint64_t stage[kWarpsPerBlock][kStageSlots];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (row >= rows) return;
  WarpSelect sel;
  sel.init(stage[warp], width, lane);
  for (int s = 0; s < splits; ++s) {
    const int64_t at = (static_cast<int64_t>(s) * rows + row) * width + lane;
    uint64_t key = 0;
    if (lane < width) {
      const int32_t slot = cand_slot[at];
      if (slot >= 0) key = pack_key(orderable_bits(cand_score[at]), static_cast<uint32_t>(slot));
    }
    sel.offer(key);
  }
  sel.finish();
  if (lane < width) {
    const bool live = sel.list != 0;
    out_score[row * width + lane] = live ? from_orderable_bits(static_cast<uint32_t>(sel.list >> 32)) : -INFINITY;
    out_slot[row * width + lane] = live ? static_cast<int32_t>(static_cast<uint32_t>(sel.list)) : -1;
  }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) == cudaSuccess &&
        res == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(sym);
  }
  return fn;
}

// 2-D bf16 tensor [rows, dk] with a row pitch of `pitch` elements; boxes of [box_rows x 64].
bool make_map(CUtensorMap* map, const void* base, int64_t rows, int dk, int64_t pitch, int box_rows = kBlockRows) {
  EncodeTiled enc = encode_tiled();
  if (enc == nullptr) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(dk), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch) * 2};
  const cuuint32_t box[2] = {kAtomK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Plan {
  int unit_pairs, tiles_total, splits, tiles_per_split;
  int tail_blocks = 0, tail_splits = 0, tail_tiles_per_split = 0;   // see Params
  int64_t tail_rows = 0;
};

// Pick the number of slot-range splits. Every split restarts its rows' lists from nothing and
// pays the insert-heavy start again (about k*ln(columns/k) inserts per row, measured at
// roughly 220*k key-tile times per unit), so the model is
//   time(s) = waves(s) * (tiles per split + 220*k),  waves = ceil(row pairs * s / SMs),
// minimised over s with at least 1024 key tiles per split; ties prefer fewer splits.
Plan make_plan(int64_t rows, int64_t slots, int sms, int width, int tile_cols = kTileCols, int unit_rows = kUnitRows,
               int restart_per_width = 220) {
  Plan pl;
  pl.unit_pairs = static_cast<int>((rows + unit_rows - 1) / unit_rows);
  pl.tiles_total = static_cast<int>((slots + tile_cols - 1) / tile_cols);
  const int64_t restart = static_cast<int64_t>(restart_per_width) * width;
  int best = 1;
  int64_t best_cost = -1;
  for (int s = 1; s <= 64; ++s) {
    const int64_t per = (pl.tiles_total + s - 1) / s;
    if (s > 1 && per < 1024) break;
    const int64_t units = static_cast<int64_t>(pl.unit_pairs) * s;
    const int64_t waves = (units + sms - 1) / sms;
    const int64_t cost = waves * (per + restart);
    if (best_cost < 0 || cost * 100 < best_cost * 97) { best_cost = cost; best = s; }
  }
  pl.splits = best;
  pl.tiles_per_split = (pl.tiles_total + best - 1) / best;
  pl.splits = (pl.tiles_total + pl.tiles_per_split - 1) / pl.tiles_per_split;
  return pl;
}

// Start-up of a unit of the wide-tile kernel in key-tile times per route kept (one wave of
// 128-row units over 512..16384 tiles of 256 slots, top-32: time = 1.05 us x tiles + start-up).
constexpr int kWideRestartPerWidth = 47;

// The wide-tile kernel may also keep one split for the row blocks that fill whole waves of
// CTAs and cut only the blocks of the last, partly filled wave (their lists are merged
// afterwards): time = full waves * (tiles + restart) + (tiles / tail splits + restart).
Plan make_plan_with_tail(int64_t rows, int64_t slots, int sms, int width, int tile_cols, int unit_rows) {
  Plan pl = make_plan(rows, slots, sms, width, tile_cols, unit_rows, kWideRestartPerWidth);
  const int blocks = pl.unit_pairs;
  const int full = blocks / sms * sms, tail = blocks - full;
  if (full == 0 || tail == 0) return pl;
  const int64_t restart = static_cast<int64_t>(kWideRestartPerWidth) * width;
  int parts = sms / tail;
  while (parts > 1 && (pl.tiles_total + parts - 1) / parts < 1024) --parts;
  if (parts < 2) return pl;
  const int64_t per = (pl.tiles_total + parts - 1) / parts;
  const int64_t uniform_units = static_cast<int64_t>(blocks) * pl.splits;
  const int64_t uniform_cost = (uniform_units + sms - 1) / sms * (pl.tiles_per_split + restart);
  const int64_t tail_cost = static_cast<int64_t>(full / sms) * (pl.tiles_total + restart) + per + restart;
  if (tail_cost * 100 >= uniform_cost * 98) return pl;
  pl.unit_pairs = full;
  pl.splits = 1;
  pl.tiles_per_split = pl.tiles_total;
  pl.tail_blocks = tail;
  pl.tail_tiles_per_split = static_cast<int>(per);
  pl.tail_splits = static_cast<int>((pl.tiles_total + per - 1) / per);
  pl.tail_rows = rows - static_cast<int64_t>(full) * unit_rows;
  return pl;
}

int sm_count_cached() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
      sms = 148;
  }
  return sms;
}

// Which kernel runs: 0 = one CTA per 256 rows, key tiles of 128 slots (128x128x16 MMAs);
// 2 = one CTA per 128 rows, key tiles of 256 slots (128x256x16 MMAs). Set by
// glsdm_score_topk_variant() or GLSDM_SCORE_TOPK_VARIANT. (1 named a CTA-pair kernel that
// measured slower than both and was removed; the number is kept free.)
constexpr int kDefaultVariant = 2;
int g_variant = -1;

int variant() {
  if (g_variant < 0) {
    const char* env = getenv("GLSDM_SCORE_TOPK_VARIANT");
    g_variant = (env != nullptr && (env[0] == '0' || env[0] == '2')) ? env[0] - '0' : kDefaultVariant;
  }
  return g_variant;
}

Plan plan_for(int64_t rows, int64_t slots, int width) {
  switch (variant()) {
    case 2: return make_plan_with_tail(rows, slots, sm_count_cached(), width, kWideTileCols, kBlockRows);
    default: return make_plan(rows, slots, sm_count_cached(), width);
  }
}


}  // namespace
}  // namespace glsdm

using namespace glsdm;

extern "C" int glsdm_score_topk_variant(int which) {
  const int before = variant();
  if (which == 0 || which == 2) g_variant = which;
  return before;
}

extern "C" int glsdm_score_topk_plan(int64_t rows, int64_t slots, int32_t width, int32_t which, int32_t sms,
                                     int32_t* out) {
  if (rows < 1 || slots < 1 || width < 1 || sms < 1 || out == nullptr || (which != 0 && which != 2)) return GLSDM_ERR_ARGUMENT;
  const Plan pl = which == 2 ? make_plan_with_tail(rows, slots, sms, width, kWideTileCols, kBlockRows)
                             : make_plan(rows, slots, sms, width);
  out[0] = pl.unit_pairs;
  out[1] = pl.splits;
  out[2] = pl.tiles_per_split;
  out[3] = pl.tiles_total;
  out[4] = pl.tail_blocks;
  out[5] = pl.tail_splits;
  out[6] = pl.tail_tiles_per_split;
  out[7] = which == 2 ? kBlockRows : kUnitRows;
  return GLSDM_OK;
}

// GLSDM_FLOOR_REFRESH: looks at the queue between two exchanges of bounds inside a unit (a power
// of two; 0 = only when a unit starts and ends).
static uint32_t floor_refresh_mask() {
  static const uint32_t mask = [] {
    const char* v = std::getenv("GLSDM_FLOOR_REFRESH");
    const long n = (v == nullptr || v[0] == '\0') ? static_cast<long>(kFloorRefresh) : std::atol(v);
    if (n <= 0) return 0xffffffffu;
    uint32_t pow2 = 1;
    while (pow2 < static_cast<uint32_t>(n) && pow2 < (1u << 30)) pow2 <<= 1;
    return pow2 - 1u;
  }();
  return mask;
}

extern "C" size_t glsdm_score_topk_workspace_bytes(int64_t rows, int64_t slots, int32_t dk, int32_t width) {
  (void)dk;
  if (rows < 1 || slots < 1 || width < 1) return 0;
  const Plan pl = plan_for(rows, slots, width);
  if (pl.tail_blocks > 0) return static_cast<size_t>(pl.tail_splits) * pl.tail_rows * width * 8 + 512;
  if (pl.splits <= 1) return 256;
  return static_cast<size_t>(pl.splits) * rows * width * 8 + 512;
}

extern "C" int glsdm_score_topk(const void* queries, const void* keys, int64_t rows, int64_t slots, int32_t dk,
                                int32_t width, int64_t col_base, float* out_score, int32_t* out_slot,
                                void* workspace, size_t workspace_bytes, uint32_t* device_status,
                                glsdm_stream_t stream) {
  return glsdm_score_topk_pitched(queries, dk, keys, dk, rows, slots, dk, width, col_base, out_score, out_slot,
                                  workspace, workspace_bytes, device_status, stream);
}

extern "C" int glsdm_score_topk_pitched(const void* queries, int64_t query_pitch, const void* keys,
                                        int64_t key_pitch, int64_t rows, int64_t slots, int32_t dk, int32_t width,
                                        int64_t col_base, float* out_score, int32_t* out_slot, void* workspace,
                                        size_t workspace_bytes, uint32_t* device_status, glsdm_stream_t stream) {
  return glsdm_score_topk_bounded(queries, query_pitch, keys, key_pitch, rows, slots, dk, width, col_base, nullptr,
                                  out_score, out_slot, workspace, workspace_bytes, device_status, stream);
}

extern "C" int glsdm_score_topk_bounded(const void* queries, int64_t query_pitch, const void* keys,
                                        int64_t key_pitch, int64_t rows, int64_t slots, int32_t dk, int32_t width,
                                        int64_t col_base, const float* row_floor, float* out_score,
                                        int32_t* out_slot, void* workspace, size_t workspace_bytes,
                                        uint32_t* device_status, glsdm_stream_t stream) {
  return glsdm_score_topk_shared(queries, query_pitch, keys, key_pitch, rows, slots, dk, width, col_base, row_floor,
                                 0, nullptr, 0, nullptr, 0, out_score, out_slot, workspace, workspace_bytes,
                                 device_status, stream);
}

extern "C" int glsdm_score_topk_shared(const void* queries, int64_t query_pitch, const void* keys,
                                       int64_t key_pitch, int64_t rows, int64_t slots, int32_t dk, int32_t width,
                                       int64_t col_base, const float* row_floor, int64_t row_shift,
                                       const float* floor_in, int32_t floor_sources, float* const* floor_out,
                                       int32_t floor_peers, float* out_score, int32_t* out_slot, void* workspace,
                                       size_t workspace_bytes, uint32_t* device_status, glsdm_stream_t stream) {
  if (floor_sources < 0 || floor_peers < 0 || row_shift < 0 || (rows > 0 && row_shift >= rows)) return GLSDM_ERR_ARGUMENT;
  if (floor_peers > kMaxFloorPeers) return GLSDM_ERR_LIMIT;
  if ((floor_sources > 0 && floor_in == nullptr) || (floor_peers > 0 && floor_out == nullptr)) return GLSDM_ERR_ARGUMENT;
  for (int i = 0; i < floor_peers; ++i)
    if (floor_out[i] == nullptr) return GLSDM_ERR_ARGUMENT;
  if (query_pitch < dk || key_pitch < dk || (query_pitch % 8) || (key_pitch % 8)) return GLSDM_ERR_ARGUMENT;
  if (queries == nullptr || keys == nullptr || out_score == nullptr || out_slot == nullptr) return GLSDM_ERR_ARGUMENT;
  if (rows < 0 || slots < 1 || width < 1 || col_base < 0) return GLSDM_ERR_ARGUMENT;
  if (dk != 64 && dk != 128) return GLSDM_ERR_UNSUPPORTED;
  if (width > 32 || col_base + slots > 0x7fffffffll || slots > kMaxSlotsPerCall) return GLSDM_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(queries) | reinterpret_cast<uintptr_t>(keys)) & 15u) return GLSDM_ERR_ARGUMENT;
  if (rows == 0) return GLSDM_OK;
  const int sms = sm_count_cached();
  const bool wide = variant() == 2;
  const Plan pl = plan_for(rows, slots, width);
  Params p;
  p.rows = rows;
  p.slots = slots;
  p.col_base = col_base;
  p.dk = dk;
  p.width = width;
  p.splits = pl.splits;
  p.tiles_per_split = pl.tiles_per_split;
  p.tiles_total = pl.tiles_total;
  p.unit_pairs = pl.unit_pairs;
  p.device_status = device_status;
  p.row_floor = row_floor;
  p.floor_in = floor_in;
  p.floor_sources = floor_sources;
  p.floor_peers = floor_peers;
  p.row_shift = row_shift;
  p.floor_refresh_mask = floor_refresh_mask();
  for (int i = 0; i < kMaxFloorPeers; ++i) p.floor_out[i] = i < floor_peers ? floor_out[i] : nullptr;
  p.tail_blocks = pl.tail_blocks;
  p.tail_splits = pl.tail_splits;
  p.tail_tiles_per_split = pl.tail_tiles_per_split;
  p.tail_score = nullptr;
  p.tail_slot = nullptr;
  if (pl.tail_blocks > 0) {
    const size_t cells = static_cast<size_t>(pl.tail_splits) * pl.tail_rows * width;
    if (workspace == nullptr || workspace_bytes < cells * 8) return GLSDM_ERR_WORKSPACE;
    p.tail_score = static_cast<float*>(workspace);
    p.tail_slot = reinterpret_cast<int32_t*>(static_cast<float*>(workspace) + cells);
    p.out_score = out_score;
    p.out_slot = out_slot;
  } else if (pl.splits > 1) {
    const size_t need = static_cast<size_t>(pl.splits) * rows * width * 8;
    if (workspace == nullptr || workspace_bytes < need) return GLSDM_ERR_WORKSPACE;
    p.out_score = static_cast<float*>(workspace);
    p.out_slot = reinterpret_cast<int32_t*>(static_cast<float*>(workspace) + static_cast<size_t>(pl.splits) * rows * width);
  } else {
    p.out_score = out_score;
    p.out_slot = out_slot;
  }
  CUtensorMap map_q, map_k;
  if (!make_map(&map_q, queries, rows, dk, query_pitch) ||
      !make_map(&map_k, keys, slots, dk, key_pitch, wide ? kWideTileCols : kBlockRows)) {
    note_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled");
    return GLSDM_ERR_CUDA;
  }
  const int units = pl.unit_pairs * pl.splits + pl.tail_blocks * pl.tail_splits;
  const int grid = units < sms ? units : sms;
  if (wide) {
    const bool bounds = row_floor != nullptr || floor_sources > 0 || floor_peers > 0;
#define GLSDM_WIDE(KB, BOUNDS)                                                                              \
  do {                                                                                                      \
    const int smem = WideLayout<KB>::total();                                                               \
    GLSDM_CUDA_OK(cudaFuncSetAttribute(score_topk_wide_kernel<KB, BOUNDS>,                                  \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem),                  \
                  "score_topk shared memory");                                                              \
    score_topk_wide_kernel<KB, BOUNDS><<<grid, kWideThreads, smem, stream>>>(map_q, map_k, p);              \
  } while (0)
    if (dk == 128) {
      if (bounds) GLSDM_WIDE(2, true); else GLSDM_WIDE(2, false);
    } else {
      if (bounds) GLSDM_WIDE(1, true); else GLSDM_WIDE(1, false);
    }
#undef GLSDM_WIDE
  } else if (dk == 128) {
    const int smem = Layout<2>::total(width);
    GLSDM_CUDA_OK(cudaFuncSetAttribute(score_topk_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                  "score_topk shared memory");
    score_topk_kernel<2><<<grid, kThreads, smem, stream>>>(map_q, map_k, p);
  } else {
    const int smem = Layout<1>::total(width);
    GLSDM_CUDA_OK(cudaFuncSetAttribute(score_topk_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                  "score_topk shared memory");
    score_topk_kernel<1><<<grid, kThreads, smem, stream>>>(map_q, map_k, p);
  }
  GLSDM_CUDA_OK(cudaGetLastError(), "score_topk launch");
  count_launches(1);
  if (pl.tail_blocks > 0) {
    const int64_t first = rows - pl.tail_rows;
    split_merge_kernel<<<blocks_for(pl.tail_rows, kWarpsPerBlock), kWarpsPerBlock * 32, 0, stream>>>(
        p.tail_score, p.tail_slot, pl.tail_splits, pl.tail_rows, width, out_score + first * width,
        out_slot + first * width);
    GLSDM_CUDA_OK(cudaGetLastError(), "score_topk tail merge launch");
    count_launches(1);
  } else if (pl.splits > 1) {
    split_merge_kernel<<<blocks_for(rows, kWarpsPerBlock), kWarpsPerBlock * 32, 0, stream>>>(
        p.out_score, p.out_slot, pl.splits, rows, width, out_score, out_slot);
    GLSDM_CUDA_OK(cudaGetLastError(), "score_topk merge launch");
    count_launches(1);
  }
  return GLSDM_OK;
}
