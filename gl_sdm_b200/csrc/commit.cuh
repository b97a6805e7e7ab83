// Shared pieces of the buffered commit: scratch layout, the stable LSD radix sort of
// (key, entry id) pairs, and the per-lane row slices the reducers work on. Included by the
// translation units that finish the commit in different ways (materialised delta rows in
// commit.cu, deltas rebuilt from their factors in commit_factored.cu).
#pragma once

#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>

#include "common.cuh"
#include "glsdm.h"

namespace glsdm {
namespace {

constexpr int kRadixBits = 8;
constexpr int kRadix = 1 << kRadixBits;
constexpr int kDigits = 64 / kRadixBits;
constexpr int kSortThreads = 256;
constexpr int kItems = 8;                           // keys per thread in a tile
constexpr int kTile = kSortThreads * kItems;        // 2048 keys per block
constexpr int kLongSegment = 256;                   // entries summed strictly in sequence

struct Plan {
  uint32_t skip[kDigits];    // 1 = all keys share this digit
  uint32_t source[kDigits];  // buffer (0/1) holding the input of this pass
  uint32_t final_buffer;     // buffer holding the fully sorted order
  uint32_t last_pass;        // the last pass that moves keys; the gather rides on it
  uint32_t long_count;       // queued long segments
  uint32_t chunk_cursor;     // partial-sum rows handed out so far
  uint32_t ticket[kDigits];  // next tile of each pass (tiles are taken in this order)
  uint32_t entry_ticket;     // next block of the entry stage
  uint32_t done;             // blocks of the entry stage that have finished
  uint32_t pad[2];
};

struct Workspace {
  uint64_t* keys[2];
  uint32_t* ids[2];
  int64_t* sorted_address;
  uint32_t* histogram;          // [kDigits][kRadix]
  Plan* plan;
  unsigned long long* status;   // [tiles][kRadix] look-back words of the pass in flight
  uint2* long_list;             // (start, length) of queued segments
  float* partial;               // [partial_rows][dim]
  int64_t partial_rows;
  int64_t long_capacity;
  int tiles;
  // histogram, plan and status lie together and must be zero when a commit starts: one clear.
  void* zero_from;
  size_t zero_bytes;
  // When set, the number of live entries is read on the device (a list whose length the
  // host does not know): grids stay sized for the capacity, blocks past the end do nothing.
  const uint32_t* live;
  uint32_t* device_status;      // where a wait that ran out is reported (may be null)
};

__device__ __forceinline__ int64_t live_entries(const uint32_t* live, int64_t capacity) {
  return live != nullptr ? static_cast<int64_t>(*live) : capacity;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t carve(Workspace* w, char* base, int64_t entries, int32_t dim) {
  size_t at = 0;
  auto take = [&](size_t bytes) {
    char* p = base ? base + at : nullptr;
    at += align_up(bytes, 256);
    return p;
  };
  const int tiles = static_cast<int>((entries + kTile - 1) / kTile);
  const int64_t long_capacity = entries / kLongSegment + 1;
  const int64_t partial_rows = 2 * (entries / kLongSegment) + 2;
  Workspace local;
  Workspace* o = w ? w : &local;
  o->tiles = tiles;
  o->live = nullptr;
  o->device_status = nullptr;
  o->long_capacity = long_capacity;
  o->partial_rows = partial_rows;
  o->keys[0] = reinterpret_cast<uint64_t*>(take(sizeof(uint64_t) * entries));
  o->keys[1] = reinterpret_cast<uint64_t*>(take(sizeof(uint64_t) * entries));
  o->ids[0] = reinterpret_cast<uint32_t*>(take(sizeof(uint32_t) * entries));
  o->ids[1] = reinterpret_cast<uint32_t*>(take(sizeof(uint32_t) * entries));
  o->sorted_address = reinterpret_cast<int64_t*>(take(sizeof(int64_t) * entries));
  o->long_list = reinterpret_cast<uint2*>(take(sizeof(uint2) * long_capacity));
  o->partial = reinterpret_cast<float*>(take(sizeof(float) * partial_rows * dim));
  // The zeroed region comes last, so that zeroed scratch of a caller can follow it directly.
  const size_t zero_at = at;
  o->histogram = reinterpret_cast<uint32_t*>(take(sizeof(uint32_t) * kDigits * kRadix));
  o->plan = reinterpret_cast<Plan*>(take(sizeof(Plan)));
  o->status = reinterpret_cast<unsigned long long*>(
      take(sizeof(unsigned long long) * kRadix * static_cast<size_t>(tiles)));
  o->zero_from = base ? base + zero_at : nullptr;
  o->zero_bytes = at - zero_at;
  return at;
}

__device__ __forceinline__ uint32_t digit_of(uint64_t key, int pass) {
  return static_cast<uint32_t>(key >> (pass * kRadixBits)) & (kRadix - 1);
}

// ---- words that one block publishes and later blocks poll ------------------------------------
//
// A word carries a 32-bit count, the pass it belongs to and its kind in ONE 64-bit value, so a
// reader needs no ordering beyond the load itself: kind 0 = nothing yet, kAggregate = the count
// of this block alone, kPrefix = the count of this block and every block before it. Blocks
// take their place in a chain from a ticket counter, so every block a reader waits for has
// already started running; the wait is bounded all the same and, when it runs out, reports
// GLSDM_DEV_WAIT_EXPIRED and goes on with what it has (the result is then wrong and flagged).
constexpr unsigned long long kAggregate = 1ull << 62;
constexpr unsigned long long kPrefix = 2ull << 62;
constexpr int kPollLimit = 1 << 20;

__device__ __forceinline__ unsigned long long chain_word(unsigned long long kind, int tag, uint32_t count) {
  return kind | (static_cast<unsigned long long>(tag & 63) << 56) | count;
}

__device__ __forceinline__ void chain_publish(unsigned long long* slot, unsigned long long word) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(slot), "l"(word) : "memory");
}

__device__ __forceinline__ unsigned long long chain_peek(const unsigned long long* slot) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(slot) : "memory");
  return v;
}

// Sum of the counts of chain positions [0, position) of one chain whose words lie `stride`
// apart: walks back over aggregates until it meets a prefix. Eight words are requested at a
// time, so a walk over many aggregates costs one memory latency per eight positions.
__device__ __forceinline__ uint32_t chain_look_back(const unsigned long long* words, size_t stride,
                                                    int64_t position, int tag, uint32_t* device_status) {
  constexpr int kWindow = 8;
  uint32_t before = 0;
  for (int64_t t = position - 1; t >= 0; t -= kWindow) {
    unsigned long long v[kWindow];
#pragma unroll
    for (int j = 0; j < kWindow; ++j)
      v[j] = t - j >= 0 ? chain_peek(words + static_cast<size_t>(t - j) * stride) : 0ull;
#pragma unroll
    for (int j = 0; j < kWindow; ++j) {
      if (t - j < 0) return before;
      int polls = 0;
      while ((v[j] >> 62) == 0 || static_cast<int>((v[j] >> 56) & 63) != (tag & 63)) {
        if (++polls > kPollLimit) {
          if (device_status != nullptr) atomicOr(device_status, GLSDM_DEV_WAIT_EXPIRED);
          return before;
        }
        __nanosleep(20);
        v[j] = chain_peek(words + static_cast<size_t>(t - j) * stride);
      }
      before += static_cast<uint32_t>(v[j]);
      if ((v[j] >> 62) == 2) return before;
    }
  }
  return before;
}

// ---- entry stage: order-preserving keys, entry ids, digit histograms, the plan ------------------

// The sort's plan from the finished histogram, by one whole block: a digit on which every key
// agrees needs no pass; pass 0 always runs, so that some pass carries the gather. Only the
// fields of the plan that describe the passes are written.
__device__ __forceinline__ void write_plan(const uint32_t* histogram, int passes, int64_t entries, Plan* plan) {
  __shared__ uint32_t uniform[kDigits];
  if (threadIdx.x < kDigits) uniform[threadIdx.x] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < passes * kRadix; i += blockDim.x)
    if (__ldcg(histogram + i) == static_cast<uint32_t>(entries)) uniform[i / kRadix] = 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t buffer = 0, last = 0;
    for (int p = 0; p < kDigits; ++p) {
      const uint32_t skip = (p >= passes) ? 1u : (p == 0 ? 0u : uniform[p]);
      plan->skip[p] = skip;
      plan->source[p] = buffer;
      if (!skip) {
        buffer ^= 1u;
        last = p;
      }
    }
    plan->final_buffer = buffer;
    plan->last_pass = last;
  }
  __syncthreads();
}

// End of the entry stage, called by every block with its own digit counts in shared memory:
// adds them to the global histogram; the block that finishes last writes the plan (a digit on
// which every key agrees needs no pass; pass 0 always runs, so that some pass carries the
// gather). `entries_known` is the entry count when the host knows it, else w.live is read.
__device__ __forceinline__ void finish_entry_stage(const Workspace& w, int passes, int64_t entries_known,
                                                   const uint32_t (*local)[kRadix]) {
  __shared__ int is_last;
  __syncthreads();
  for (int i = threadIdx.x; i < passes * kRadix; i += blockDim.x) {
    const uint32_t c = (&local[0][0])[i];
    if (c) atomicAdd(w.histogram + i, c);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&w.plan->done, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int64_t entries = w.live != nullptr
                              ? static_cast<int64_t>(*reinterpret_cast<const volatile uint32_t*>(w.live))
                              : entries_known;
  write_plan(w.histogram, passes, entries, w.plan);
}

// Tile `tile` of the caller's keys: order-preserving keys, entry ids, digit counts into `local`.
__device__ __forceinline__ void prepare_tile(const int64_t* __restrict__ keys, int64_t entries, int passes,
                                             const Workspace& w, int64_t tile, uint32_t (*local)[kRadix]) {
  const int64_t base = tile * kTile;
  for (int r = 0; r < kItems; ++r) {
    const int64_t i = base + r * kSortThreads + threadIdx.x;
    if (i < entries) {
      const uint64_t k = static_cast<uint64_t>(keys[i]) ^ 0x8000000000000000ull;
      w.keys[0][i] = k;
      w.ids[0][i] = static_cast<uint32_t>(i);
      for (int p = 0; p < passes; ++p) atomicAdd(&local[p][digit_of(k, p)], 1u);
    }
  }
}

__global__ void __launch_bounds__(kSortThreads)
prepare_kernel(const int64_t* __restrict__ keys, int64_t entries, int passes, Workspace w) {
  __shared__ uint32_t local[kDigits][kRadix];
  for (int i = threadIdx.x; i < kDigits * kRadix; i += kSortThreads) (&local[0][0])[i] = 0;
  __syncthreads();
  prepare_tile(keys, entries, passes, w, blockIdx.x, local);
  finish_entry_stage(w, passes, entries, local);
}

// What rides on the last pass: the address (and, for the factored commit, the 16-byte
// record) of every entry, written at the entry's sorted position.
struct SortGather {
  const int64_t* addresses;  // [entries] by entry id
  const uint4* records;      // [entries] by entry id, or null
  uint4* sorted_records;     // [entries] by sorted position
};

// One tile (2048 keys) of one radix pass, in three steps that share the block's scratch:
//   count    a warp owns 256 consecutive keys and takes them 32 at a time, so (warp, round,
//            lane) order is input order; ranks inside a round come from match_any;
//   place    thread d turns the warps' counts of digit d into offsets inside the tile, and
//            learns how many keys with digit d the EARLIER tiles hold by looking back along
//            the chain of published words;
//   scatter  stable: smaller digits first, then earlier tiles, then earlier keys of the tile.
struct SortScratch {
  uint32_t warp_count[kSortThreads / 32][kRadix];
  uint32_t digit_base[kRadix];
  uint32_t scan_carry[kSortThreads / 32];
};

struct TileKeys {
  uint64_t key[kItems];
  uint32_t id[kItems];
  uint32_t rank[kItems];
};

__device__ __forceinline__ void tile_count(const Workspace& w, const Plan& plan, int64_t entries, int pass,
                                           int64_t tile, SortScratch& sh, TileKeys& k) {
  constexpr int kWarps = kSortThreads / 32;
  __syncthreads();   // the previous tile of this block is done with the scratch
  for (int i = threadIdx.x; i < kWarps * kRadix; i += kSortThreads) (&sh.warp_count[0][0])[i] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t src = plan.source[pass];
  const uint64_t* __restrict__ keys = w.keys[src];
  const uint32_t* __restrict__ ids = w.ids[src];
  const int64_t base = tile * kTile + warp * (kItems * 32);
#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    const int64_t i = base + r * 32 + lane;
    const bool live = i < entries;
    k.key[r] = live ? keys[i] : 0;
    k.id[r] = live ? ids[i] : 0;
    const uint32_t d = live ? digit_of(k.key[r], pass) : kRadix;  // dead lanes match only each other
    const unsigned peers = __match_any_sync(kFullMask, d);
    const uint32_t before = __popc(peers & ((1u << lane) - 1u));
    uint32_t prior = 0;
    if (live) prior = sh.warp_count[warp][d];
    __syncwarp();
    if (live && before == 0) sh.warp_count[warp][d] = prior + __popc(peers);
    __syncwarp();
    k.rank[r] = prior + before;
  }
  __syncthreads();
}

// Thread d: the tile's count of digit d; the warps' counts become their offsets inside the tile.
__device__ __forceinline__ uint32_t tile_total(SortScratch& sh) {
  const int d = threadIdx.x;  // kSortThreads == kRadix: thread d owns digit d
  uint32_t total = 0;
  for (int q = 0; q < kSortThreads / 32; ++q) {
    const uint32_t c = sh.warp_count[q][d];
    sh.warp_count[q][d] = total;
    total += c;
  }
  return total;
}

// Thread d, given the count of digit d in earlier tiles: where digit d of this tile starts.
__device__ __forceinline__ void tile_place(const Workspace& w, int pass, uint32_t earlier, SortScratch& sh) {
  const int d = threadIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // keys with a smaller digit, over the whole input: exclusive scan of this pass's histogram
  const uint32_t h = __ldcg(w.histogram + pass * kRadix + d);
  uint32_t inclusive = h;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(kFullMask, inclusive, o);
    if (lane >= o) inclusive += t;
  }
  if (lane == 31) sh.scan_carry[warp] = inclusive;
  __syncthreads();
  uint32_t smaller = inclusive - h;
  for (int q = 0; q < warp; ++q) smaller += sh.scan_carry[q];
  sh.digit_base[d] = smaller + earlier;
  __syncthreads();
}

__device__ __forceinline__ void tile_scatter(const Workspace& w, const Plan& plan, int64_t entries, int pass,
                                             const SortGather& g, int64_t tile, const SortScratch& sh,
                                             const TileKeys& k) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t src = plan.source[pass];
  uint64_t* __restrict__ out_keys = w.keys[src ^ 1u];
  uint32_t* __restrict__ out_ids = w.ids[src ^ 1u];
  const int64_t base = tile * kTile + warp * (kItems * 32);
  const bool last = static_cast<uint32_t>(pass) == plan.last_pass && g.addresses != nullptr;
#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    const int64_t i = base + r * 32 + lane;
    if (i < entries) {
      const uint32_t d = digit_of(k.key[r], pass);
      const uint32_t at = sh.digit_base[d] + sh.warp_count[warp][d] + k.rank[r];
      out_keys[at] = k.key[r];
      out_ids[at] = k.id[r];
      if (last) {
        w.sorted_address[at] = g.addresses[k.id[r]];
        if (g.records != nullptr) g.sorted_records[at] = g.records[k.id[r]];
      }
    }
  }
}

// The three steps joined by the look-back chain.
__device__ __forceinline__ void radix_pass_tile(const Workspace& w, const Plan& plan, int64_t entries, int pass,
                                                const SortGather& g, int64_t tile, SortScratch& sh) {
  TileKeys k;
  tile_count(w, plan, entries, pass, tile, sh, k);
  const uint32_t total = tile_total(sh);
  unsigned long long* mine = w.status + static_cast<size_t>(tile) * kRadix + threadIdx.x;
  const int tag = pass + 1;
  uint32_t earlier = 0;
  if (tile == 0) {
    chain_publish(mine, chain_word(kPrefix, tag, total));
  } else {
    chain_publish(mine, chain_word(kAggregate, tag, total));
    earlier = chain_look_back(w.status + threadIdx.x, kRadix, tile, tag, w.device_status);
    chain_publish(mine, chain_word(kPrefix, tag, earlier + total));
  }
  tile_place(w, pass, earlier, sh);
  tile_scatter(w, plan, entries, pass, g, tile, sh, k);
}

__global__ void __launch_bounds__(kSortThreads)
radix_pass_kernel(Workspace w, int64_t entries, int pass, SortGather g) {
  if (w.plan->skip[pass]) return;
  __shared__ uint32_t my_tile;
  entries = live_entries(w.live, entries);
  if (threadIdx.x == 0) my_tile = atomicAdd(&w.plan->ticket[pass], 1u);
  __syncthreads();
  __shared__ SortScratch scratch;
  const int64_t tile = my_tile;
  if (tile * kTile >= entries) return;
  radix_pass_tile(w, *w.plan, entries, pass, g, tile, scratch);
}

// Per-lane slice of a dim-wide fp32 row: lanes own column blocks of 32*V floats.
template <int V>
struct Slice {
  float v[V];
};

template <int V>
__device__ __forceinline__ void zero(Slice<V>& s) {
#pragma unroll
  for (int i = 0; i < V; ++i) s.v[i] = 0.f;
}

// Column layout per lane for V in {1,2,4,8}: V<=4 -> V consecutive floats at lane*V;
// V==8 -> two float4 at lane*4 and 128+lane*4 (keeps every warp load contiguous).
template <int V>
__device__ __forceinline__ void load_delta(Slice<V>& s, const float* __restrict__ row, int lane) {
  if constexpr (V == 1) {
    s.v[0] = __ldg(row + lane);
  } else if constexpr (V == 2) {
    const float2 t = __ldg(reinterpret_cast<const float2*>(row) + lane);
    s.v[0] = t.x; s.v[1] = t.y;
  } else if constexpr (V == 4) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(row) + lane);
    s.v[0] = t.x; s.v[1] = t.y; s.v[2] = t.z; s.v[3] = t.w;
  } else {
    const float4 a = __ldg(reinterpret_cast<const float4*>(row) + lane);
    const float4 b = __ldg(reinterpret_cast<const float4*>(row) + 32 + lane);
    s.v[0] = a.x; s.v[1] = a.y; s.v[2] = a.z; s.v[3] = a.w;
    s.v[4] = b.x; s.v[5] = b.y; s.v[6] = b.z; s.v[7] = b.w;
  }
}

// Ask for a row of `floats` fp32 values to be brought into L1: the in-order sum of a long
// segment reads one row after another, and what it waits for is each row's latency.
__device__ __forceinline__ void prefetch_row(const float* row, int floats) {
  for (int c = 0; c < floats; c += 32) asm volatile("prefetch.global.L1 [%0];" ::"l"(row + c));
}

template <int V>
__device__ __forceinline__ int column_of(int lane, int i) {
  if constexpr (V == 8) return (i < 4) ? lane * 4 + i : 128 + lane * 4 + (i - 4);
  return lane * V + i;
}

template <int V>
__device__ __forceinline__ void add(Slice<V>& acc, const Slice<V>& x) {
#pragma unroll
  for (int i = 0; i < V; ++i) acc.v[i] = __fadd_rn(acc.v[i], x.v[i]);
}

template <typename T>
__device__ __forceinline__ float load_value(const T* p);
template <>
__device__ __forceinline__ float load_value<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_value<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <typename T>
__device__ __forceinline__ void store_value(T* p, float v);
template <>
__device__ __forceinline__ void store_value<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_value<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&p);
}

// new_row = old_row + acc (one rounding to the bank dtype), for this lane's columns, moved
// in the widest unit the lane's column group allows (4 columns: 16 B fp32 / 8 B bf16).
template <typename T, int V>
__device__ __forceinline__ void apply_row(const T* in_row, T* out_row, const Slice<V>& acc, int lane) {
  if constexpr (V % 4 == 0) {
#pragma unroll
    for (int c = 0; c < V / 4; ++c) {
      const int col = column_of<V>(lane, c * 4);
      const float* a = acc.v + c * 4;
      if constexpr (sizeof(T) == 4) {
        const float4 o = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(in_row) + col);
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(out_row) + col) =
            make_float4(__fadd_rn(o.x, a[0]), __fadd_rn(o.y, a[1]), __fadd_rn(o.z, a[2]), __fadd_rn(o.w, a[3]));
      } else {
        const uint2 o = *reinterpret_cast<const uint2*>(in_row + col);
        uint2 n;
        n.x = pack_bf16x2(__fadd_rn(bf16_lo(o.x), a[0]), __fadd_rn(bf16_hi(o.x), a[1]));
        n.y = pack_bf16x2(__fadd_rn(bf16_lo(o.y), a[2]), __fadd_rn(bf16_hi(o.y), a[3]));
        *reinterpret_cast<uint2*>(out_row + col) = n;
      }
    }
  } else if constexpr (V == 2) {
    const int col = lane * 2;
    if constexpr (sizeof(T) == 4) {
      const float2 o = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(in_row) + col);
      *reinterpret_cast<float2*>(reinterpret_cast<float*>(out_row) + col) =
          make_float2(__fadd_rn(o.x, acc.v[0]), __fadd_rn(o.y, acc.v[1]));
    } else {
      const uint32_t o = *reinterpret_cast<const uint32_t*>(in_row + col);
      *reinterpret_cast<uint32_t*>(out_row + col) =
          pack_bf16x2(__fadd_rn(bf16_lo(o), acc.v[0]), __fadd_rn(bf16_hi(o), acc.v[1]));
    }
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = column_of<V>(lane, i);
      store_value<T>(out_row + c, __fadd_rn(load_value<T>(in_row + c), acc.v[i]));
    }
  }
}

// The same update split in two, so that several rows' old values can be in flight at once:
// load_bank returns this lane's columns of a bank row as fp32, store_bank rounds and stores.
template <typename T, int V>
__device__ __forceinline__ void load_bank(const T* row, Slice<V>& out, int lane) {
  if constexpr (V % 4 == 0) {
#pragma unroll
    for (int c = 0; c < V / 4; ++c) {
      const int col = column_of<V>(lane, c * 4);
      if constexpr (sizeof(T) == 4) {
        const float4 o = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(row) + col);
        out.v[c * 4] = o.x; out.v[c * 4 + 1] = o.y; out.v[c * 4 + 2] = o.z; out.v[c * 4 + 3] = o.w;
      } else {
        const uint2 o = *reinterpret_cast<const uint2*>(row + col);
        out.v[c * 4] = bf16_lo(o.x); out.v[c * 4 + 1] = bf16_hi(o.x);
        out.v[c * 4 + 2] = bf16_lo(o.y); out.v[c * 4 + 3] = bf16_hi(o.y);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) out.v[i] = load_value<T>(row + column_of<V>(lane, i));
  }
}

template <typename T, int V>
__device__ __forceinline__ void store_bank(T* row, const Slice<V>& in, int lane) {
  if constexpr (V % 4 == 0) {
#pragma unroll
    for (int c = 0; c < V / 4; ++c) {
      const int col = column_of<V>(lane, c * 4);
      if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(row) + col) =
            make_float4(in.v[c * 4], in.v[c * 4 + 1], in.v[c * 4 + 2], in.v[c * 4 + 3]);
      } else {
        uint2 n;
        n.x = pack_bf16x2(in.v[c * 4], in.v[c * 4 + 1]);
        n.y = pack_bf16x2(in.v[c * 4 + 2], in.v[c * 4 + 3]);
        *reinterpret_cast<uint2*>(row + col) = n;
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) store_value<T>(row + column_of<V>(lane, i), in.v[i]);
  }
}

// Length of the segment starting at sorted position `start` (address `a`).
__device__ __forceinline__ int64_t segment_length(const int64_t* __restrict__ sorted, int64_t start,
                                                  int64_t entries, int64_t a, int lane) {
  int64_t len = 1;
  for (;;) {
    const int64_t at = start + len + lane;
    const bool same = at < entries && sorted[at] == a;
    const unsigned m = __ballot_sync(kFullMask, same);
    if (m == kFullMask) { len += 32; continue; }
    len += __ffs(~m) - 1;
    return len;
  }
}

// Everything a commit polls or counts starts at zero; `extra_bytes` extends the clear over
// zeroed scratch the caller placed directly behind the workspace.
inline int clear_sort_state(const Workspace& w, size_t extra_bytes, glsdm_stream_t stream) {
  GLSDM_CUDA_OK(cudaMemsetAsync(w.zero_from, 0, w.zero_bytes + extra_bytes, stream), "commit state clear");
  return GLSDM_OK;
}

// The passes of the sort, after an entry stage has written w.keys[0], w.ids[0], the histogram
// and the plan: one launch per digit (a digit all keys agree on returns at once). Afterwards
// w.ids[w.plan->final_buffer] holds the entry ids in stable key order, w.sorted_address the
// address of every sorted position (and g.sorted_records its record).
inline int run_passes(const Workspace& w, int64_t entries, int passes, const SortGather& g,
                      glsdm_stream_t stream) {
  for (int p = 0; p < passes; ++p)
    radix_pass_kernel<<<w.tiles, kSortThreads, 0, stream>>>(w, entries, p, g);
  GLSDM_CUDA_OK(cudaGetLastError(), "commit sort launch");
  count_launches(passes);
  return GLSDM_OK;
}

// The same sort in ONE cooperative launch (a grid small enough to be resident at once, with a
// grid-wide barrier where a launch boundary would be): clear | prepare | plan (every block
// computes the same one) | pass, pass, ... Small and medium sorts are bound by dependent
// launches, not bytes. Blocks walk the tiles in increasing order, so every tile a look-back
// waits for belongs to a resident block that reaches it no later.
__global__ void __launch_bounds__(kSortThreads)
sort_all_kernel(const int64_t* __restrict__ keys, int64_t entries, int passes, Workspace w, SortGather g) {
  cooperative_groups::grid_group grid = cooperative_groups::this_grid();
  __shared__ uint32_t local[kDigits][kRadix];
  __shared__ Plan plan;
  __shared__ SortScratch scratch;
  {
    uint4* zero = static_cast<uint4*>(w.zero_from);
    const size_t cells = w.zero_bytes / sizeof(uint4);
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < cells;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
      zero[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  for (int i = threadIdx.x; i < kDigits * kRadix; i += blockDim.x) (&local[0][0])[i] = 0;
  grid.sync();
  const int64_t tiles = (entries + kTile - 1) / kTile;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) prepare_tile(keys, entries, passes, w, tile, local);
  __syncthreads();
  for (int i = threadIdx.x; i < passes * kRadix; i += blockDim.x) {
    const uint32_t c = (&local[0][0])[i];
    if (c) atomicAdd(w.histogram + i, c);
  }
  grid.sync();
  write_plan(w.histogram, passes, entries, &plan);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (int p = 0; p < kDigits; ++p) {
      w.plan->skip[p] = plan.skip[p];
      w.plan->source[p] = plan.source[p];
    }
    w.plan->final_buffer = plan.final_buffer;
    w.plan->last_pass = plan.last_pass;
  }
  for (int p = 0; p < passes; ++p) {
    if (plan.skip[p]) continue;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x)
      radix_pass_tile(w, plan, entries, p, g, tile, scratch);
    if (static_cast<uint32_t>(p) != plan.last_pass) grid.sync();
  }
}

constexpr int64_t kSortAllMaxEntries = int64_t{1} << 20;   // beyond it every pass wants the whole GPU

// Blocks of sort_all_kernel that are resident at once on the current device (two per SM at
// most), or -1 where a cooperative launch is not possible.
inline int sort_all_resident() {
  static thread_local int resident[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return -1;
  if (resident[device] == 0) {
    int cooperative = 0, sms = 0, per_sm = 0;
    if (cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sort_all_kernel, kSortThreads, 0) != cudaSuccess)
      return -1;
    resident[device] = cooperative && per_sm > 0 ? sms * (per_sm < 2 ? per_sm : 2) : -1;
  }
  return resident[device];
}

// Sort (keys[i], i) for i in [0, entries): one cooperative launch where that pays and is
// possible (GLSDM_ORDER_ALL=0 switches it off), else clear, prepare and one launch per pass.
inline int run_sort(const Workspace& w, const int64_t* keys, int64_t entries, int passes,
                    const SortGather& g, glsdm_stream_t stream) {
  static const bool one_launch = [] {
    const char* v = getenv("GLSDM_ORDER_ALL");
    return v == nullptr || v[0] != '0';
  }();
  const int resident = (one_launch && entries <= kSortAllMaxEntries) ? sort_all_resident() : -1;
  if (resident > 0) {
    const int grid = w.tiles < resident ? (w.tiles < 1 ? 1 : w.tiles) : resident;
    Workspace ws = w;
    SortGather gs = g;
    void* args[] = {&keys, &entries, &passes, &ws, &gs};
    GLSDM_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(sort_all_kernel), dim3(grid), dim3(kSortThreads),
                                              args, 0, stream),
                  "commit sort launch");
    count_launches(1);
    return GLSDM_OK;
  }
  if (int s = clear_sort_state(w, 0, stream)) return s;
  prepare_kernel<<<w.tiles, kSortThreads, 0, stream>>>(keys, entries, passes, w);
  GLSDM_CUDA_OK(cudaGetLastError(), "commit prepare launch");
  count_launches(1);
  return run_passes(w, entries, passes, g, stream);
}

// Keys are compared as signed 64-bit integers: the top digit always carries the sign.
inline int sort_passes(int32_t key_bits) {
  return (key_bits == 0 || key_bits == 64) ? kDigits : (key_bits + kRadixBits - 1) / kRadixBits;
}

}  // namespace
}  // namespace glsdm
