// Building blocks shared by the dense-key routing kernels (score_topk.cu: 128x128x16 MMAs over
// 256 rows; score_topk_wide.cuh: 128x256x16 MMAs over 128 rows): mbarrier / TMA / tcgen05
// wrappers, the shared-memory matrix descriptor, and the scanner -> inserter candidate queue.
#pragma once

#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"

namespace glsdm {
namespace dense {

constexpr int kBlockRows = 128;                 // rows of one MMA (M)
constexpr int kUnitRows = 2 * kBlockRows;       // rows handled by one CTA unit
constexpr int kTileCols = 128;                  // slots per key tile (MMA N)
constexpr int kStages = 3;
constexpr int kAtomK = 64;                      // bf16 elements per 128-byte swizzle row
constexpr int kSubTileBytes = kBlockRows * 128; // one [128 x 64] bf16 sub-tile, 16 KB
constexpr int kEpilogueWarps = 8;                // scanner warps
constexpr int kInsertWarps = 4;                  // one per pair of scanner warps (64 rows)
constexpr int kThreads = 32 * (2 + kEpilogueWarps + kInsertWarps);
constexpr int kQueueSlots = 32;                  // entries per inserter queue (one per lane)
constexpr int64_t kMaxSlotsPerCall = 1 << 24;    // a queue entry carries a 24-bit slot
constexpr int kTmemCols = 512;
constexpr uint32_t kSpinLimit = 1u << 24;
constexpr unsigned kIdleNanoseconds = 1000;      // an idle inserter sleeps this long between looks at its queue
constexpr uint32_t kFloorRefresh = 64;           // idle looks between two exchanges of bounds with the peers (a power of two)
constexpr uint32_t kIdleLimit = 1u << 22;        // idle looks before an inserter gives up (about four seconds)

constexpr int kMaxFloorPeers = 7;

struct Params {
  int64_t rows;
  int64_t slots;
  int64_t col_base;
  int dk;
  int width;
  int splits;
  int tiles_per_split;
  int tiles_total;
  int unit_pairs;       // row blocks that take the uniform splits (all of them unless there is a tail)
  float* out_score;     // [splits][rows][width] (or the final output when splits == 1)
  int32_t* out_slot;
  uint32_t* device_status;
  const float* row_floor;   // [rows] a score every row's K-th best is known to reach, or null
  // Bounds exchanged with the other shards WHILE they scan (all optional). floor_in
  // [floor_sources][rows]: what the peers have reached so far, written by their kernels into
  // this GPU's memory; read when a unit starts. floor_out[i] [rows]: this shard's place in peer
  // i's floor_in; when a unit ends, the K-th best score of each of its rows is stored there
  // (plain stores, nobody waits for anybody: a bound that has not arrived yet is only a
  // missed saving). Rows are addressed as (row + row_shift) % rows, so that shards which walk
  // the rows in different orders (rotated copies of the queries) agree on their names.
  const float* floor_in;
  int floor_sources;
  float* floor_out[kMaxFloorPeers];
  int floor_peers;
  int64_t row_shift;
  uint32_t floor_refresh_mask;   // bounds are exchanged inside a unit every (mask + 1) looks at the queue
  // Tail (wide-tile kernel only): the row blocks left over after the last full wave of CTAs
  // have their slot range cut in tail_splits parts, so the last wave is short instead of
  // mostly idle. Their partial lists go to tail_score/tail_slot [part][tail row][width].
  int tail_blocks;
  int tail_splits;
  int tail_tiles_per_split;
  float* tail_score;
  int32_t* tail_slot;
};

// One unit of work: a block of query rows against the key tiles [t0, t1); `part` numbers the
// pieces of the block's slot range, `tail` says which output the piece belongs to.
struct UnitSpan {
  int block, part, t0, t1;
  bool tail;
};

__device__ __forceinline__ int unit_count(const Params& p) {
  return p.unit_pairs * p.splits + p.tail_blocks * p.tail_splits;
}

// Units are numbered part-major, so the CTAs that run at the same time stream the same keys.
__device__ __forceinline__ UnitSpan unit_span(const Params& p, int unit) {
  UnitSpan u;
  const int uniform = p.unit_pairs * p.splits;
  if (unit < uniform) {
    u.tail = false;
    u.part = unit / p.unit_pairs;
    u.block = unit % p.unit_pairs;
    u.t0 = u.part * p.tiles_per_split;
    u.t1 = min(u.t0 + p.tiles_per_split, p.tiles_total);
  } else {
    const int j = unit - uniform;
    u.tail = true;
    u.part = j / p.tail_blocks;
    u.block = p.unit_pairs + j % p.tail_blocks;
    u.t0 = u.part * p.tail_tiles_per_split;
    u.t1 = min(u.t0 + p.tail_tiles_per_split, p.tiles_total);
  }
  return u;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait. Returns false when the wait ran out or another role has aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 bytes apart,
// 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);        // start address, bits [0,14)
  d |= static_cast<uint64_t>(1) << 16;                            // leading byte offset (unused with swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                    // stride byte offset, bits [32,46)
  d |= static_cast<uint64_t>(1) << 46;                            // version
  d |= static_cast<uint64_t>(2) << 61;                            // SWIZZLE_128B
  return d;
}

// Instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, M = 128, N = 128.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kTileCols >> 3) << 17) |
                                ((kBlockRows >> 4) << 24);

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kInstrDesc), "r"(acc)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

__device__ __forceinline__ uint32_t tmem_load1(uint32_t taddr) {
  uint32_t r;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  return r;
}

// Largest of 32 accumulator values with the three-input max of sm_100 (16 instructions).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// m[j] = largest of columns 3j..3j+2 for j < 10, m[10] = larger of columns 30 and 31; returns
// the largest of all 32. The group maxima let the rare path look only at groups that matter.
__device__ __forceinline__ float max_of_32(const uint32_t* r, float (&m)[11]) {
#pragma unroll
  for (int j = 0; j < 10; ++j)
    m[j] = max3(__uint_as_float(r[3 * j]), __uint_as_float(r[3 * j + 1]), __uint_as_float(r[3 * j + 2]));
  m[10] = fmaxf(__uint_as_float(r[30]), __uint_as_float(r[31]));
  const float a = max3(m[0], m[1], m[2]), b = max3(m[3], m[4], m[5]), c = max3(m[6], m[7], m[8]);
  return fmaxf(max3(a, b, c), fmaxf(m[9], m[10]));
}

__device__ __forceinline__ float max_of_32(const uint32_t* r) {
  float groups[11];
  return max_of_32(r, groups);
}

__device__ __forceinline__ void tmem_wait_loads() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Candidate queue of one inserter warp (multi-producer: two scanner warps; one consumer).
// An entry is orderable score << 32 | row (6 bits) << 24 | slot (24 bits); 0 = empty slot.
struct Queue {
  uint64_t slot[kQueueSlots];
  uint32_t tail;    // entries reserved so far (producers, atomicAdd)
  uint32_t head;    // entries consumed so far (consumer)
  uint32_t done;    // scanner warps that have finished pushing, summed over units
  uint32_t epoch;   // units whose lists the consumer has written out and reset
};

// Push the entries of the lanes in `m` (warp-uniform). Space is reserved with one atomic per
// call; a lane waits (bounded) until the consumer has freed the ring slot it was given.
__device__ __forceinline__ bool queue_push(Queue* q, unsigned m, bool pass, uint64_t entry, int lane,
                                           volatile int* abort_flag) {
  uint32_t base = 0;
  if (lane == 0) base = atomicAdd(&q->tail, static_cast<uint32_t>(__popc(m)));
  base = __shfl_sync(kFullMask, base, 0);
  bool ok = true;
  if (pass) {
    const uint32_t at = base + __popc(m & ((1u << lane) - 1u));
    uint32_t spin = 0;
    while (static_cast<int32_t>(at - *reinterpret_cast<volatile uint32_t*>(&q->head)) >= kQueueSlots) {
      if (++spin >= kSpinLimit || ((spin & 1023u) == 0 && *abort_flag)) { ok = false; break; }
    }
    if (ok) *reinterpret_cast<volatile uint64_t*>(&q->slot[at & (kQueueSlots - 1)]) = entry;
  }
  if (!__all_sync(kFullMask, ok)) { *abort_flag = 1; return false; }
  return true;
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }


}  // namespace dense
}  // namespace glsdm
