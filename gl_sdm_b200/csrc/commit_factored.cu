// Commit of a write proposal that is never written out as delta rows.
//
// A proposal entry is delta_k = mass * ((decay - 1) * row_k + w_k * err), with
// err = beta * (target - decay * prediction) one vector per token
// (gl_sdm/runtime/dense.py:11-14, built in gl_sdm/layers/global_layer.py:44-51 and summed per
// address by gl_sdm/memory/transactions.py:90-96). row_k is the bank row the commit is about to
// update, so the reducer already holds it: it needs only the token's error vector and three
// scalars per entry to rebuild the delta in registers. The [entries, dim] fp32 delta array of
// the materialised path (4*dim bytes written by the proposal and read back by the commit,
// plus the proposal's second read of the bank rows) disappears; what crosses HBM per entry is
// its 8-byte key, 8-byte address and a 16-byte descriptor, plus one read-modify-write per
// touched bank row. Error vectors are shared by a token's K entries and stay in L2.
//
// The arithmetic is the materialised path's, operation for operation (same fp32 products,
// sums and order), so both commits produce bit-identical banks.
#include <cooperative_groups.h>

#include <atomic>
#include <cstdlib>

#include "commit.cuh"
#include "route.cuh"

namespace glsdm {
namespace {

// What the reducer needs to rebuild one entry's delta row.
struct __align__(16) Descriptor {
  uint32_t error_at;  // float offset of the token's error row in the error array
  float weight;       // w_k
  float gate;         // decay - 1
  float mass;
};

struct FactoredScratch {
  int64_t* addresses;     // [entries] shard-local row of every listed entry
  Descriptor* described;  // [entries] by entry
  Descriptor* sorted;     // [entries] in key order
  // Single-writer path only (all three are cleared with the sort state they follow in memory):
  unsigned long long* chain;  // [row blocks] look-back words of the compaction
  uint32_t* seen;         // [bits / 32] an entry has this address (modulo bits)
  uint32_t* twice;        // [bits / 32] a second entry had it too
  uint32_t* live;         // [1] how many entries need the sort
  uint32_t bit_mask;      // bits - 1
  size_t zero_chain;      // bytes of chain and live behind the workspace's zeroed region ...
  size_t zero_extra;      // ... and of the maps as well
};

constexpr int kEntryRows = 4;   // routing rows per warp of the entry stage

// Bits of each address map: a power of two >= 16 per entry. A bank with more rows than bits
// folds several addresses onto one bit; they then all take the sorted path, which is always correct.
int64_t address_bits_for(int64_t entries) {
  int64_t bits = 1 << 16;
  while (bits < 16 * entries && bits < (int64_t{1} << 31)) bits <<= 1;
  return bits;
}

size_t carve_factored(Workspace* w, FactoredScratch* f, char* base, int64_t entries, int32_t dim) {
  size_t at = carve(w, base, entries, dim);
  auto take = [&](size_t bytes) {
    char* p = base ? base + at : nullptr;
    at += align_up(bytes, 256);
    return p;
  };
  FactoredScratch local;
  FactoredScratch* o = f ? f : &local;
  // zeroed scratch first: it continues the zeroed region that ends the workspace
  const size_t zero_at = at;
  o->chain = reinterpret_cast<unsigned long long*>(
      take(sizeof(unsigned long long) * (entries / (kWarpsPerBlock * kEntryRows) + 2)));
  o->live = reinterpret_cast<uint32_t*>(take(sizeof(uint32_t)));
  o->zero_chain = at - zero_at;
  const int64_t bits = address_bits_for(entries);
  o->bit_mask = static_cast<uint32_t>(bits - 1);
  o->seen = reinterpret_cast<uint32_t*>(take(static_cast<size_t>(bits / 8) * 2));   // seen and twice
  o->twice = o->seen != nullptr ? o->seen + bits / 32 : nullptr;
  o->zero_extra = at - zero_at;
  o->addresses = reinterpret_cast<int64_t*>(take(sizeof(int64_t) * entries));
  o->described = reinterpret_cast<Descriptor*>(take(sizeof(Descriptor) * entries));
  o->sorted = reinterpret_cast<Descriptor*>(take(sizeof(Descriptor) * entries));
  return at;
}

struct EntryArgs {
  const int32_t* index;     // write routes, blocks of block_rows rows, route_stride apart
  const float* weights;
  const float* error;       // per block: [block_rows, dim] error rows then [block_rows] decay-1
  const float* mass;        // per token or null
  const uint32_t* offsets;  // first entry of every row, or null: entry = row * width + route
  int64_t rows, block_rows, route_stride, error_stride, tokens, sequences;
  int64_t chunk_offset, key_stride;
  int width, num_layers, layer_index;
};

__device__ __forceinline__ Descriptor shfl_descriptor(const Descriptor& d, int src) {
  Descriptor o;
  o.error_at = __shfl_sync(kFullMask, d.error_at, src);
  o.weight = __shfl_sync(kFullMask, d.weight, src);
  o.gate = __shfl_sync(kFullMask, d.gate, src);
  o.mass = __shfl_sync(kFullMask, d.mass, src);
  return o;
}

// delta = mass * (gate * old + weight * err), the products and the sum rounded one by one as
// the materialised proposal kernels do.
template <int V>
__device__ __forceinline__ void rebuild(Slice<V>& delta, const Descriptor& d, const Slice<V>& err,
                                        const Slice<V>& old) {
#pragma unroll
  for (int i = 0; i < V; ++i)
    delta.v[i] = __fmul_rn(d.mass, __fadd_rn(__fmul_rn(d.gate, old.v[i]), __fmul_rn(d.weight, err.v[i])));
}

// Sum entries [start, start+count) of the sorted order, strictly left to right.
template <int V>
__device__ __forceinline__ void sum_factored(Slice<V>& acc, const Descriptor* __restrict__ sorted,
                                             const float* __restrict__ error, const Slice<V>& old,
                                             int64_t start, int64_t count, int lane) {
  for (int64_t done = 0; done < count; done += 32) {
    const int n = (count - done < 32) ? static_cast<int>(count - done) : 32;
    Descriptor mine = {0u, 0.f, 0.f, 0.f};
    if (lane < n) mine = sorted[start + done + lane];
    if (count > 8 && lane < n) prefetch_row(error + mine.error_at, 32 * V);   // lane t: the row of entry t
    constexpr int kAhead = V >= 8 ? 2 : 4;   // error rows requested before the first is used
    int t = 0;
    for (; t + kAhead <= n; t += kAhead) {
      Slice<V> e[kAhead];
      Descriptor d[kAhead];
#pragma unroll
      for (int j = 0; j < kAhead; ++j) {
        d[j] = shfl_descriptor(mine, t + j);
        load_delta<V>(e[j], error + d[j].error_at, lane);
      }
#pragma unroll
      for (int j = 0; j < kAhead; ++j) {
        Slice<V> x;
        rebuild<V>(x, d[j], e[j], old);
        add<V>(acc, x);
      }
    }
    for (; t < n; ++t) {
      const Descriptor d = shfl_descriptor(mine, t);
      Slice<V> e, x;
      load_delta<V>(e, error + d.error_at, lane);
      rebuild<V>(x, d, e, old);
      add<V>(acc, x);
    }
  }
}

// Any-width variant over the 8 column blocks [c0, c0+256): lanes stride the columns.
template <typename T>
__device__ __forceinline__ void sum_factored_generic(float (&acc)[8], const float (&old)[8],
                                                     const Descriptor* __restrict__ sorted,
                                                     const float* __restrict__ error, int dim, int c0,
                                                     int64_t start, int64_t count, int lane) {
  for (int64_t t = 0; t < count; ++t) {
    const Descriptor d = sorted[start + t];
    const float* __restrict__ erow = error + d.error_at;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + j * 32 + lane;
      if (c < dim) {
        const float x = __fmul_rn(d.mass, __fadd_rn(__fmul_rn(d.gate, old[j]), __fmul_rn(d.weight, __ldg(erow + c))));
        acc[j] = __fadd_rn(acc[j], x);
      }
    }
  }
}

struct FactoredArgs {
  void* values;           // shard rows [bank_rows, dim], updated in place
  const float* error;
  const Descriptor* sorted;
  int64_t entries;
  int64_t bank_rows;
  int dim;
  uint32_t* device_status;
};

// Single-entry rows in flight per warp: 2 for 256-wide rows (as in the delta-row reducer); narrower
// rows leave registers for more, which is what a latency-bound warp needs.
template <int V>
struct FactoredBatch {
  static constexpr int value = V >= 8 ? 2 : (V >= 4 ? 4 : 8);
};

template <typename T, int V>
__device__ __forceinline__ void reduce_factored_block(const Workspace& w, const FactoredArgs& a, int64_t block) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t first = (block * kWarpsPerBlock + warp) * 32;
  const int64_t entries = live_entries(w.live, a.entries);
  if (first >= entries) return;
  const int64_t* __restrict__ sorted = w.sorted_address;
  const int64_t at = first + lane;
  const int64_t mine = at < entries ? sorted[at] : -1;
  const int64_t prev = (at > 0 && at < entries) ? sorted[at - 1] : -2;
  const bool is_head = at < entries && (at == 0 || mine != prev);
  const unsigned all_heads = __ballot_sync(kFullMask, is_head);
  unsigned heads = all_heads;
  T* __restrict__ values = static_cast<T*>(a.values);
  if constexpr (V > 0) {
    const int64_t next = (at + 1 < entries) ? sorted[at + 1] : -3;
    Descriptor my_d = {0u, 0.f, 0.f, 0.f};
    if (at < entries) my_d = a.sorted[at];
    unsigned singles = __ballot_sync(kFullMask, is_head && mine != next && mine >= 0 && mine < a.bank_rows);
    heads &= ~singles;
    constexpr int kFactoredBatch = FactoredBatch<V>::value;
    while (singles) {
      int pick[kFactoredBatch];
#pragma unroll
      for (int j = 0; j < kFactoredBatch; ++j) {
        pick[j] = singles ? __ffs(singles) - 1 : -1;
        if (singles) singles &= singles - 1;
      }
      Slice<V> err[kFactoredBatch], old[kFactoredBatch];
      Descriptor d[kFactoredBatch];
      int64_t where[kFactoredBatch];
#pragma unroll
      for (int j = 0; j < kFactoredBatch; ++j) {
        if (pick[j] < 0) continue;
        d[j] = shfl_descriptor(my_d, pick[j]);
        where[j] = __shfl_sync(kFullMask, mine, pick[j]);
        load_delta<V>(err[j], a.error + d[j].error_at, lane);
        load_bank<T, V>(values + where[j] * a.dim, old[j], lane);
      }
#pragma unroll
      for (int j = 0; j < kFactoredBatch; ++j) {
        if (pick[j] < 0) continue;
        Slice<V> x;
        rebuild<V>(x, d[j], err[j], old[j]);
#pragma unroll
        for (int i = 0; i < V; ++i) old[j].v[i] = __fadd_rn(old[j].v[i], __fadd_rn(0.f, x.v[i]));
        store_bank<T, V>(values + where[j] * a.dim, old[j], lane);
      }
    }
  }
  while (heads) {
    const int h = __ffs(heads) - 1;
    heads &= heads - 1;
    const int64_t start = first + h;
    const int64_t local = __shfl_sync(kFullMask, mine, h);
    if (local < 0 || local >= a.bank_rows) {
      if (lane == 0 && a.device_status) atomicOr(a.device_status, GLSDM_DEV_ADDRESS_OUT_OF_RANGE);
      continue;
    }
    int64_t len;
    const unsigned later = h == 31 ? 0u : (all_heads & (0xffffffffu << (h + 1)));
    if (later) {
      len = (__ffs(later) - 1) - h;
    } else {
      const int64_t tail = first + 32 < entries ? first + 32 : entries;
      len = tail - start;
      if (tail < entries) len = segment_length(sorted, tail - 1, entries, local, lane) + (tail - 1 - start);
    }
    if (len > kLongSegment) {
      if (lane == 0) {
        const uint32_t slot = atomicAdd(&w.plan->long_count, 1u);
        w.long_list[slot] = make_uint2(static_cast<uint32_t>(start), static_cast<uint32_t>(len));
      }
      continue;
    }
    T* row = values + local * a.dim;
    if constexpr (V > 0) {
      Slice<V> old, acc;
      load_bank<T, V>(row, old, lane);
      zero<V>(acc);
      sum_factored<V>(acc, a.sorted, a.error, old, start, len, lane);
#pragma unroll
      for (int i = 0; i < V; ++i) old.v[i] = __fadd_rn(old.v[i], acc.v[i]);
      store_bank<T, V>(row, old, lane);
    } else {
      for (int c0 = 0; c0 < a.dim; c0 += 256) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        float old[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int c = c0 + j * 32 + lane;
          old[j] = c < a.dim ? load_value<T>(row + c) : 0.f;
        }
        sum_factored_generic<T>(acc, old, a.sorted, a.error, a.dim, c0, start, len, lane);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int c = c0 + j * 32 + lane;
          if (c < a.dim) store_value<T>(row + c, __fadd_rn(old[j], acc[j]));
        }
      }
    }
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, 4)
reduce_factored_kernel(Workspace w, FactoredArgs a) {
  reduce_factored_block<T, V>(w, a, blockIdx.x);
}

// One block per queued long segment: 256-entry chunks summed in order by warps (each warp
// reads the old row itself), chunk sums added in chunk order, row updated once. The block
// must finish reading the old row before anyone overwrites it: the update happens after the
// barrier that ends the chunk loop.
template <typename T, int V>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
long_factored_kernel(Workspace w, FactoredArgs a) {
  __shared__ uint32_t partial_base;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t count = w.plan->long_count;
  for (uint32_t s = blockIdx.x; s < count; s += gridDim.x) {
    const uint2 seg = w.long_list[s];
    const int64_t start = seg.x, len = seg.y;
    const int chunks = static_cast<int>((len + kLongSegment - 1) / kLongSegment);
    __syncthreads();
    if (threadIdx.x == 0) partial_base = atomicAdd(&w.plan->chunk_cursor, static_cast<uint32_t>(chunks));
    __syncthreads();
    float* __restrict__ partial = w.partial + static_cast<int64_t>(partial_base) * a.dim;
    T* row = static_cast<T*>(a.values) + w.sorted_address[start] * a.dim;
    for (int c = warp; c < chunks; c += kWarpsPerBlock) {
      const int64_t cs = start + static_cast<int64_t>(c) * kLongSegment;
      const int64_t cn = (len - static_cast<int64_t>(c) * kLongSegment < kLongSegment)
                             ? len - static_cast<int64_t>(c) * kLongSegment : kLongSegment;
      float* prow = partial + static_cast<int64_t>(c) * a.dim;
      if constexpr (V > 0) {
        Slice<V> old, acc;
        load_bank<T, V>(row, old, lane);
        zero<V>(acc);
        sum_factored<V>(acc, a.sorted, a.error, old, cs, cn, lane);
#pragma unroll
        for (int i = 0; i < V; ++i) prow[column_of<V>(lane, i)] = acc.v[i];
      } else {
        for (int c0 = 0; c0 < a.dim; c0 += 256) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          float old[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int col = c0 + j * 32 + lane;
            old[j] = col < a.dim ? load_value<T>(row + col) : 0.f;
          }
          sum_factored_generic<T>(acc, old, a.sorted, a.error, a.dim, c0, cs, cn, lane);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int col = c0 + j * 32 + lane;
            if (col < a.dim) prow[col] = acc[j];
          }
        }
      }
    }
    __syncthreads();
    for (int col = threadIdx.x; col < a.dim; col += blockDim.x) {
      float total = 0.f;
      for (int c = 0; c < chunks; ++c) total = __fadd_rn(total, partial[static_cast<int64_t>(c) * a.dim + col]);
      store_value<T>(row + col, __fadd_rn(load_value<T>(row + col), total));
    }
  }
}

// ---- dense numbering: rows written once skip the sort ------------------------------------------
//
// Most addresses of a commit epoch are written by exactly one entry (a 16M-slot bank and 1M
// entries: ~97 %). Such an entry has nothing to be ordered against: its row can be updated
// straight from the routes, in whatever order the entries come. Two bit maps over the
// addresses find them (first writer sets `seen`, any later one sets `twice`); only the entries
// of addresses marked `twice` are compacted, in entry order, into the list that is sorted and
// reduced as before. The list's length stays on the device.

struct DenseLane {
  int64_t address;   // shard-local row, or -1 when the slot is outside the bank
  int64_t slot;
  float weight;
  bool valid;        // lane holds a route
};

// Row `major` of the token-major numbering ((position, sequence, head)) in the caller's
// [sequence, token, head] layout.
__device__ __forceinline__ int64_t caller_row(const BankView& bank, const EntryArgs& a, int64_t major) {
  const int64_t head = major % bank.heads, ps = major / bank.heads;
  const int64_t sequence = ps % a.sequences, position = ps / a.sequences;
  return (sequence * a.tokens + position) * bank.heads + head;
}

__device__ __forceinline__ DenseLane dense_lane(const BankView& bank, const EntryArgs& a, int64_t row, int lane) {
  DenseLane l;
  l.valid = lane < a.width;
  l.address = -1;
  l.slot = -1;
  l.weight = 0.f;
  if (l.valid) {
    const int64_t block = row / a.block_rows, inner = row % a.block_rows;
    const int64_t at = block * a.route_stride + inner * a.width + lane;
    l.slot = a.index[at];
    l.weight = a.weights[at];
    if (l.slot >= bank.slot_lo && l.slot < bank.slot_hi)
      l.address = (row % bank.heads) * bank.part_stride_rows + (l.slot - bank.slot_lo);
  }
  return l;
}

__device__ __forceinline__ bool written_twice(const FactoredScratch& f, int64_t address) {
  const uint32_t h = static_cast<uint32_t>(address) & f.bit_mask;
  return (f.twice[h >> 5] >> (h & 31)) & 1u;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
mark_addresses_kernel(BankView bank, EntryArgs a, FactoredScratch f) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (row >= a.rows) return;
  const DenseLane l = dense_lane(bank, a, row, lane);
  if (l.address < 0) return;
  const uint32_t h = static_cast<uint32_t>(l.address) & f.bit_mask;
  const uint32_t bit = 1u << (h & 31);
  if (atomicOr(&f.seen[h >> 5], bit) & bit) atomicOr(&f.twice[h >> 5], bit);
}

// ---- entry stage ---------------------------------------------------------------------------
//
// One launch lists the entries the sort has to order - address, order-preserving key, entry id
// and descriptor of each - and counts their digits for every pass (the block that finishes
// last writes the sort's plan). Which routes are listed, and where, depends on the numbering:
//   kEveryRoute       one shard owns the bank and every entry is sorted: entry = token-major
//                     row * width + route. The canonical order inside an address is (position,
//                     layer, arrival = sequence), so a stable sort by the ADDRESS alone yields
//                     it and the key needs no position bits. A slot outside the bank takes the
//                     key one past the last address, sorts last, and is dropped (and reported)
//                     by the reducer through its out-of-range row.
//   kOwnedRoutes      a shard of several: the routes this shard owns, at offsets[row] + rank
//                     among the row's owned routes; keys carry (address, position, layer) as
//                     in gl_sdm/layers/global_layer.py:45,52-53.
//   kOwnedCompact     a shard of several, without a host-side count: the routes whose slot this
//                     shard owns, compacted in token-major order like kSharedAddresses (so the
//                     address alone is the key); the list's length stays on the device.
//   kSharedAddresses  single-writer path: only entries whose address is written more than
//                     once (and, on a shard, owned), compacted in token-major order. A block learns how many entries
//                     the earlier blocks list by looking back along a chain of published
//                     counts (blocks take their rows from a ticket counter, so every block it
//                     waits for is already running); the list's length stays on the device.
enum EntryMode { kEveryRoute = 0, kOwnedRoutes = 1, kSharedAddresses = 2, kOwnedCompact = 3 };

// The rows of entry block `logical` (of `blocks`): lists their entries and adds their digits to
// the block's counts in `local`.
template <int MODE>
__device__ __forceinline__ void entry_rows(const BankView& bank, const EntryArgs& a, const FactoredScratch& f,
                                           const Workspace& w, int passes, uint32_t* device_status, int64_t logical,
                                           int64_t blocks, uint32_t (*local)[kRadix]) {
  constexpr bool kCompacts = MODE == kSharedAddresses || MODE == kOwnedCompact;
  __shared__ uint32_t per_warp[kWarpsPerBlock];
  __shared__ uint32_t block_first;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();   // the previous block of rows is done with the shared words
  DenseLane l[kEntryRows];
  int64_t row[kEntryRows];
  unsigned mask[kEntryRows];
  uint32_t listed = 0;
#pragma unroll
  for (int r = 0; r < kEntryRows; ++r) {
    const int64_t major = (logical * kWarpsPerBlock + warp) * kEntryRows + r;
    mask[r] = 0;
    row[r] = 0;
    l[r].address = -1; l[r].slot = -1; l[r].weight = 0.f; l[r].valid = false;
    if (major < a.rows) {
      row[r] = MODE == kOwnedRoutes ? major : caller_row(bank, a, major);
      l[r] = dense_lane(bank, a, row[r], lane);
      bool list = l[r].valid;
      if (MODE == kOwnedRoutes || MODE == kOwnedCompact) list = l[r].address >= 0;
      if (MODE == kSharedAddresses) list = l[r].address >= 0 && written_twice(f, l[r].address);
      if (kCompacts && l[r].valid && (l[r].slot < 0 || l[r].slot >= bank.slots) && device_status != nullptr)
        atomicOr(device_status, GLSDM_DEV_ADDRESS_OUT_OF_RANGE);   // not a slot of any shard
      mask[r] = __ballot_sync(kFullMask, list);
      listed += __popc(mask[r]);
    }
  }
  uint32_t warp_first = 0;
  if (kCompacts) {
    if (lane == 0) per_warp[warp] = listed;
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t total = 0;
#pragma unroll
      for (int q = 0; q < kWarpsPerBlock; ++q) total += per_warp[q];
      uint32_t before = 0;
      unsigned long long* mine = f.chain + logical;
      if (logical == 0) {
        chain_publish(mine, chain_word(kPrefix, 1, total));
      } else {
        chain_publish(mine, chain_word(kAggregate, 1, total));
        before = chain_look_back(f.chain, 1, logical, 1, device_status);
        chain_publish(mine, chain_word(kPrefix, 1, before + total));
      }
      block_first = before;
      if (logical == blocks - 1) *f.live = before + total;
    }
    __syncthreads();
    warp_first = block_first;
    for (int q = 0; q < warp; ++q) warp_first += per_warp[q];
  }
#pragma unroll
  for (int r = 0; r < kEntryRows; ++r) {
    if ((mask[r] >> lane) & 1u) {
      const int64_t major = (logical * kWarpsPerBlock + warp) * kEntryRows + r;
      const uint32_t rank = __popc(mask[r] & ((1u << lane) - 1u));
      const int64_t head = row[r] % bank.heads, token = row[r] / bank.heads;
      const int64_t block = row[r] / a.block_rows, inner = row[r] % a.block_rows;
      int64_t at, key;
      if (MODE == kEveryRoute) {
        at = major * a.width + lane;
        key = l[r].address >= 0 ? head * bank.slots + l[r].slot : static_cast<int64_t>(bank.heads) * bank.slots;
      } else if (MODE == kOwnedRoutes) {
        at = static_cast<int64_t>(a.offsets[row[r]]) + rank;
        const int64_t position = a.chunk_offset + token % a.tokens;
        key = (head * bank.slots + l[r].slot) * a.key_stride + position * a.num_layers + a.layer_index;
      } else {
        at = static_cast<int64_t>(warp_first) + rank;
        key = head * bank.slots + l[r].slot;
      }
      Descriptor d;
      d.error_at = static_cast<uint32_t>(block * a.error_stride + inner * bank.dim);
      d.weight = l[r].weight;
      d.gate = a.error[block * a.error_stride + a.block_rows * bank.dim + inner];
      d.mass = a.mass != nullptr ? a.mass[token] : 1.0f;
      f.addresses[at] = l[r].address;
      f.described[at] = d;
      const uint64_t k = static_cast<uint64_t>(key) ^ 0x8000000000000000ull;
      w.keys[0][at] = k;
      w.ids[0][at] = static_cast<uint32_t>(at);
      for (int p = 0; p < passes; ++p) atomicAdd(&local[p][digit_of(k, p)], 1u);
    }
    if (kCompacts) warp_first += __popc(mask[r]);
  }
}

template <int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
entry_stage_kernel(BankView bank, EntryArgs a, FactoredScratch f, Workspace w, int passes, int64_t entries_known,
                   uint32_t* device_status) {
  constexpr bool kCompacts = MODE == kSharedAddresses || MODE == kOwnedCompact;
  __shared__ uint32_t local[kDigits][kRadix];
  __shared__ uint32_t logical_block;
  for (int i = threadIdx.x; i < kDigits * kRadix; i += blockDim.x) (&local[0][0])[i] = 0;
  if (threadIdx.x == 0)
    logical_block = kCompacts ? atomicAdd(&w.plan->entry_ticket, 1u) : blockIdx.x;
  __syncthreads();
  entry_rows<MODE>(bank, a, f, w, passes, device_status, logical_block, gridDim.x, local);
  finish_entry_stage(w, passes, entries_known, local);
}

// ---- the whole ordering phase in ONE launch ---------------------------------------------------
//
// Small and medium commits are bound by launches, not by bytes: clear, entry stage and three to
// five passes are as many dependent launches of a few microseconds of work each. This kernel
// runs them back to back on a grid small enough to be resident at once (a cooperative
// launch), with a grid-wide barrier where a launch boundary used to be: clear | entry stage |
// plan (every block computes the same one for itself) | pass, pass, ... Blocks walk the entry
// blocks and the tiles in increasing order, so every block a look-back waits for belongs to
// a resident block that reaches it no later.
template <int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
order_all_kernel(BankView bank, EntryArgs a, FactoredScratch f, Workspace w, int passes, int64_t entries_known,
                 size_t zero_extra, uint32_t* device_status, SortGather g) {
  cooperative_groups::grid_group grid = cooperative_groups::this_grid();
  __shared__ uint32_t local[kDigits][kRadix];
  __shared__ Plan plan;
  {
    uint4* zero = static_cast<uint4*>(w.zero_from);
    const size_t cells = (w.zero_bytes + zero_extra) / sizeof(uint4);
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < cells;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
      zero[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  for (int i = threadIdx.x; i < kDigits * kRadix; i += blockDim.x) (&local[0][0])[i] = 0;
  grid.sync();
  const int64_t blocks = (a.rows + kWarpsPerBlock * kEntryRows - 1) / (kWarpsPerBlock * kEntryRows);
  for (int64_t logical = blockIdx.x; logical < blocks; logical += gridDim.x)
    entry_rows<MODE>(bank, a, f, w, passes, device_status, logical, blocks, local);
  __syncthreads();
  for (int i = threadIdx.x; i < passes * kRadix; i += blockDim.x) {
    const uint32_t c = (&local[0][0])[i];
    if (c) atomicAdd(w.histogram + i, c);
  }
  grid.sync();
  const int64_t entries = w.live != nullptr
                              ? static_cast<int64_t>(*reinterpret_cast<const volatile uint32_t*>(w.live))
                              : entries_known;
  write_plan(w.histogram, passes, entries, &plan);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (int p = 0; p < kDigits; ++p) {
      w.plan->skip[p] = plan.skip[p];
      w.plan->source[p] = plan.source[p];
    }
    w.plan->final_buffer = plan.final_buffer;
    w.plan->last_pass = plan.last_pass;
  }
  __shared__ SortScratch scratch;
  const int64_t tiles = (entries + kTile - 1) / kTile;
  // (Replacing the look-back by a table of the tiles' counts, a grid-wide barrier and a plain
  // sum was measured slower: a barrier over ~256 blocks costs more than the walk it saves.)
  for (int p = 0; p < passes; ++p) {
    if (plan.skip[p]) continue;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x)
      radix_pass_tile(w, plan, entries, p, g, tile, scratch);
    if (static_cast<uint32_t>(p) != plan.last_pass) grid.sync();
  }
}


// Rows written by one entry only, updated straight from the routes: the token's error row is
// read once per warp, the arithmetic is the single-entry case of the reducer.
constexpr int kOnceBatch = 4;   // bank rows in flight per warp (2 measures the same, 8 is 40 % slower)

template <typename T, int V>
__device__ __forceinline__ void apply_once_block(const BankView& bank, const EntryArgs& a, const FactoredScratch& f,
                                                 void* bank_values, int64_t block_index) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t major = block_index * kWarpsPerBlock + warp;
  if (major >= a.rows) return;
  const int64_t row = caller_row(bank, a, major);
  const DenseLane l = dense_lane(bank, a, row, lane);
  unsigned once = __ballot_sync(kFullMask, l.address >= 0 && !written_twice(f, l.address));
  if (once == 0) return;
  const int64_t block = row / a.block_rows, inner = row % a.block_rows;
  Descriptor d;
  d.error_at = 0;
  d.gate = a.error[block * a.error_stride + a.block_rows * bank.dim + inner];
  d.mass = a.mass != nullptr ? a.mass[row / bank.heads] : 1.0f;
  Slice<V> err;
  load_delta<V>(err, a.error + block * a.error_stride + inner * bank.dim, lane);
  T* __restrict__ values = static_cast<T*>(bank_values);
  while (once) {
    int pick[kOnceBatch];
#pragma unroll
    for (int j = 0; j < kOnceBatch; ++j) {
      pick[j] = once ? __ffs(once) - 1 : -1;
      if (once) once &= once - 1;
    }
    Slice<V> old[kOnceBatch];
    int64_t where[kOnceBatch];
    float weight[kOnceBatch];
#pragma unroll
    for (int j = 0; j < kOnceBatch; ++j) {
      if (pick[j] < 0) continue;
      where[j] = __shfl_sync(kFullMask, l.address, pick[j]);
      weight[j] = __shfl_sync(kFullMask, l.weight, pick[j]);
      load_bank<T, V>(values + where[j] * bank.dim, old[j], lane);
    }
#pragma unroll
    for (int j = 0; j < kOnceBatch; ++j) {
      if (pick[j] < 0) continue;
      d.weight = weight[j];
      Slice<V> x;
      rebuild<V>(x, d, err, old[j]);
#pragma unroll
      for (int i = 0; i < V; ++i) old[j].v[i] = __fadd_rn(old[j].v[i], __fadd_rn(0.f, x.v[i]));
      store_bank<T, V>(values + where[j] * bank.dim, old[j], lane);
    }
  }
}

// Both kinds of rows in one launch: the first `shared_blocks` blocks reduce the sorted list of
// the shared addresses (few entries, but each segment is summed in sequence: started first,
// they finish under the bulk), the others update the single-writer rows. The two sets of rows
// are disjoint.
template <typename T, int V>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, 4)
apply_split_kernel(Workspace w, FactoredArgs a, BankView bank, EntryArgs e, FactoredScratch f, int shared_blocks) {
  if (static_cast<int>(blockIdx.x) < shared_blocks) reduce_factored_block<T, V>(w, a, blockIdx.x);
  else apply_once_block<T, V>(bank, e, f, a.values, static_cast<int64_t>(blockIdx.x) - shared_blocks);
}

template <typename T, int V>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, 4)
apply_once_kernel(FactoredArgs a, BankView bank, EntryArgs e, FactoredScratch f) {
  apply_once_block<T, V>(bank, e, f, a.values, blockIdx.x);
}

// The same update with the rows moved by bulk copies (cp.async.bulk): every lane asks for the
// bank row of its own route, whole rows land in shared memory (up to 32 x 512 bytes per warp
// in flight, held by no register), the warp updates them there and bulk-stores them back. A
// warp handles one routing row, so nothing in a block waits for anything but its own copies;
// that wait is bounded.
constexpr int kBulkWarps = 4;

__device__ __forceinline__ uint32_t shared_address(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

template <typename T, int V>
__global__ void __launch_bounds__(kBulkWarps * 32)
apply_once_bulk_kernel(FactoredArgs a, BankView bank, EntryArgs e, FactoredScratch f) {
  constexpr int kRowBytes = 32 * V * static_cast<int>(sizeof(T));
  extern __shared__ __align__(128) unsigned char staging[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* rows_s = staging + warp * (32 * kRowBytes);
  uint64_t* bar = reinterpret_cast<uint64_t*>(staging + kBulkWarps * 32 * kRowBytes) + warp;
  if (lane == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(shared_address(bar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  const int64_t major = static_cast<int64_t>(blockIdx.x) * kBulkWarps + warp;
  if (major >= e.rows) return;
  const int64_t row = caller_row(bank, e, major);
  const DenseLane l = dense_lane(bank, e, row, lane);
  const unsigned once = __ballot_sync(kFullMask, l.address >= 0 && !written_twice(f, l.address));
  if (once == 0) return;
  const bool mine = (once >> lane) & 1u;
  const int place = __popc(once & ((1u << lane) - 1u));
  T* __restrict__ values = static_cast<T*>(a.values);
  if (lane == 0) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(shared_address(bar)),
                 "r"(static_cast<uint32_t>(__popc(once) * kRowBytes))
                 : "memory");
  }
  __syncwarp();
  if (mine) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     shared_address(rows_s + place * kRowBytes)),
                 "l"(values + l.address * bank.dim), "r"(kRowBytes), "r"(shared_address(bar))
                 : "memory");
  }
  // the token's error row and scalars, while the rows travel
  const int64_t block = row / e.block_rows, inner = row % e.block_rows;
  Descriptor d;
  d.error_at = 0;
  d.gate = e.error[block * e.error_stride + e.block_rows * bank.dim + inner];
  d.mass = e.mass != nullptr ? e.mass[row / bank.heads] : 1.0f;
  Slice<V> err;
  load_delta<V>(err, e.error + block * e.error_stride + inner * bank.dim, lane);
  bool landed = false;
  for (int round = 0; round < 2 && !landed; ++round) {
    for (uint32_t spin = 0; spin < (1u << 20) && !landed; ++spin) {
      uint32_t done;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(done)
          : "r"(shared_address(bar))
          : "memory");
      landed = done != 0;
    }
    // a first wait that runs out is reported; the second only keeps the shared memory alive
    // for copies that may still arrive
    if (!landed && round == 0 && lane == 0 && a.device_status != nullptr)
      atomicOr(a.device_status, GLSDM_DEV_WAIT_EXPIRED);
  }
  if (!landed) return;
  int at = 0;
  for (unsigned m = once; m; m &= m - 1, ++at) {
    d.weight = __shfl_sync(kFullMask, l.weight, __ffs(m) - 1);
    T* row_s = reinterpret_cast<T*>(rows_s + at * kRowBytes);
    Slice<V> old, x;
    load_bank<T, V>(row_s, old, lane);
    rebuild<V>(x, d, err, old);
#pragma unroll
    for (int i = 0; i < V; ++i) old.v[i] = __fadd_rn(old.v[i], __fadd_rn(0.f, x.v[i]));
    store_bank<T, V>(row_s, old, lane);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  if (mine) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(values + l.address * bank.dim),
                 "r"(shared_address(rows_s + place * kRowBytes)), "r"(kRowBytes)
                 : "memory");
  }
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// 0 = rows through registers, 1 = rows through bulk copies (GLSDM_ONCE_BULK overrides the default).
bool once_bulk() {
  static const bool on = [] {
    const char* v = std::getenv("GLSDM_ONCE_BULK");
    return v == nullptr || v[0] == '\0' ? true : v[0] != '0';
  }();
  return on;
}

template <typename T, int V>
int launch_once(const FactoredArgs& a, const BankView& v, const EntryArgs& e, const FactoredScratch& f,
                glsdm_stream_t stream) {
  if (once_bulk()) {
    constexpr int kBytes = kBulkWarps * 32 * 32 * V * static_cast<int>(sizeof(T)) + 64;
    GLSDM_CUDA_OK(cudaFuncSetAttribute(apply_once_bulk_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes),
                  "factored single-writer shared memory");
    apply_once_bulk_kernel<T, V><<<blocks_for(e.rows, kBulkWarps), kBulkWarps * 32, kBytes, stream>>>(a, v, e, f);
  } else {
    apply_once_kernel<T, V><<<blocks_for(e.rows, kWarpsPerBlock), kWarpsPerBlock * 32, 0, stream>>>(a, v, e, f);
  }
  GLSDM_CUDA_OK(cudaGetLastError(), "factored single-writer apply launch");
  count_launches(1);
  return GLSDM_OK;
}

// A second stream per (host thread, device) for the one call that both orders and applies: the
// single-writer rows need only the address maps, so they are updated on the caller's stream
// while the shared-address entries are listed and sorted here; the caller's stream waits for
// this one before it reduces them. Streams and events are created on first use and kept.
struct SideLane {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};

int side_lane(SideLane** out) {
  constexpr int kMaxDevices = 64;
  static thread_local SideLane lanes[kMaxDevices];
  int device = -1;
  GLSDM_CUDA_OK(cudaGetDevice(&device), "factored commit cudaGetDevice");
  if (device < 0 || device >= kMaxDevices) return GLSDM_ERR_LIMIT;
  SideLane& lane = lanes[device];
  if (lane.stream == nullptr) {
    // Highest priority: its few small kernels must not queue behind the thousands of blocks of
    // the row update that runs beside them.
    int least = 0, greatest = 0;
    GLSDM_CUDA_OK(cudaDeviceGetStreamPriorityRange(&least, &greatest), "factored commit stream priorities");
    GLSDM_CUDA_OK(cudaStreamCreateWithPriority(&lane.stream, cudaStreamNonBlocking, greatest),
                  "factored commit side stream");
    GLSDM_CUDA_OK(cudaEventCreateWithFlags(&lane.fork, cudaEventDisableTiming), "factored commit event");
    GLSDM_CUDA_OK(cudaEventCreateWithFlags(&lane.join, cudaEventDisableTiming), "factored commit event");
  }
  *out = &lane;
  return GLSDM_OK;
}

template <typename T, int V>
int launch_split(const Workspace& w, const FactoredArgs& a, const BankView& v, const EntryArgs& e,
                 const FactoredScratch& f, glsdm_stream_t stream) {
  const int shared_blocks = blocks_for((a.entries + 31) / 32, kWarpsPerBlock);
  const int long_grid = static_cast<int>(w.long_capacity < 1184 ? w.long_capacity : 1184);
  apply_split_kernel<T, V><<<shared_blocks + blocks_for(e.rows, kWarpsPerBlock), kWarpsPerBlock * 32, 0, stream>>>(
      w, a, v, e, f, shared_blocks);
  GLSDM_CUDA_OK(cudaGetLastError(), "factored split apply launch");
  long_factored_kernel<T, V><<<long_grid, kWarpsPerBlock * 32, 0, stream>>>(w, a);
  GLSDM_CUDA_OK(cudaGetLastError(), "factored long-segment launch");
  count_launches(2);
  return GLSDM_OK;
}

// Largest list the one-launch ordering takes: beyond it the passes want the whole GPU each.
constexpr int64_t kOrderAllMaxEntries = int64_t{1} << 20;

// GLSDM_ORDER_ALL=0 keeps one launch per stage (for comparisons).
bool order_all_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("GLSDM_ORDER_ALL");
    return v == nullptr || v[0] == '\0' ? true : v[0] != '0';
  }();
  return on;
}

// Returns GLSDM_OK when the one-launch ordering ran, a negative value when it cannot run here
// (the caller then takes the launch-per-stage path), or an error.
template <int MODE>
int launch_order_all(BankView v, EntryArgs e, FactoredScratch f, Workspace w, int passes, int64_t entries,
                     size_t zero_extra, uint32_t* device_status, SortGather g, glsdm_stream_t stream) {
  static thread_local int resident[64] = {};
  int device = 0;
  GLSDM_CUDA_OK(cudaGetDevice(&device), "factored commit cudaGetDevice");
  if (device < 0 || device >= 64) return -1;
  if (resident[device] == 0) {
    int cooperative = 0, sms = 0, per_sm = 0;
    GLSDM_CUDA_OK(cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device), "cooperative launch attribute");
    GLSDM_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "SM count");
    GLSDM_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, order_all_kernel<MODE>, kWarpsPerBlock * 32, 0),
                  "order_all occupancy");
    resident[device] = cooperative && per_sm > 0 ? sms * (per_sm < 2 ? per_sm : 2) : -1;
  }
  if (resident[device] < 0) return -1;
  const int64_t row_blocks = (e.rows + kWarpsPerBlock * kEntryRows - 1) / (kWarpsPerBlock * kEntryRows);
  int64_t want = row_blocks > w.tiles ? row_blocks : w.tiles;
  if (want < 1) want = 1;
  const int grid = static_cast<int>(want < resident[device] ? want : resident[device]);
  void* args[] = {&v, &e, &f, &w, &passes, &entries, &zero_extra, &device_status, &g};
  GLSDM_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(order_all_kernel<MODE>), dim3(grid),
                                            dim3(kWarpsPerBlock * 32), args, 0, stream),
                "factored ordering launch");
  count_launches(1);
  return GLSDM_OK;
}

// -1 = decide from the sizes, 0 = sort every entry, 1 = single-writer rows skip the sort.
// GLSDM_FACTORED_ONCE in the environment sets the initial value.
std::atomic<int>& once_mode() {
  static std::atomic<int> mode = [] {
    const char* v = std::getenv("GLSDM_FACTORED_ONCE");
    return (v == nullptr || v[0] == '\0') ? -1 : (v[0] == '0' ? 0 : 1);
  }();
  return mode;
}

// The bit maps and the compaction cost ~6 launches more than they save: they pay once the
// sort they avoid is large (entries) and most rows have one writer (bank rows per entry).
// Measured with 512-byte rows: even at 524,288 entries, 4-8 % faster at 1,048,576 entries with
// 4 to 16 bank rows per entry, 3-20 % slower at 262,144 entries and below.
bool once_path_pays(int64_t entries, int64_t bank_rows) {
  const int mode = once_mode().load();
  if (mode >= 0) return mode == 1;
  return entries >= 3 * (int64_t{1} << 18) && bank_rows >= 4 * entries;
}

template <typename T>
int launch_factored(const Workspace& w, const FactoredArgs& a, bool aligned, glsdm_stream_t stream) {
  const int grid = blocks_for((a.entries + 31) / 32, kWarpsPerBlock);
  const int long_grid = static_cast<int>(w.long_capacity < 1184 ? w.long_capacity : 1184);
#define GLSDM_FACTORED(V)                                                                   \
  do {                                                                                      \
    reduce_factored_kernel<T, V><<<grid, kWarpsPerBlock * 32, 0, stream>>>(w, a);           \
    GLSDM_CUDA_OK(cudaGetLastError(), "factored reduce launch");                            \
    long_factored_kernel<T, V><<<long_grid, kWarpsPerBlock * 32, 0, stream>>>(w, a);        \
    GLSDM_CUDA_OK(cudaGetLastError(), "factored long-segment launch");                      \
    count_launches(2);                                                                      \
  } while (0)
  if (aligned && a.dim == 32) GLSDM_FACTORED(1);
  else if (aligned && a.dim == 64) GLSDM_FACTORED(2);
  else if (aligned && a.dim == 128) GLSDM_FACTORED(4);
  else if (aligned && a.dim == 256) GLSDM_FACTORED(8);
  else GLSDM_FACTORED(0);
#undef GLSDM_FACTORED
  return GLSDM_OK;
}

}  // namespace
}  // namespace glsdm

using namespace glsdm;

extern "C" int glsdm_commit_factored_mode(int mode) {
  const int before = once_mode().load();
  if (mode >= -1 && mode <= 1) once_mode().store(mode);
  return before;
}

extern "C" size_t glsdm_commit_factored_workspace_bytes(int64_t entries, int32_t dim) {
  if (entries < 0 || dim < 1) return 0;
  return carve_factored(nullptr, nullptr, nullptr, entries < 1 ? 1 : entries, dim);
}

extern "C" int glsdm_commit_factored(const glsdm_bank* bank, const int32_t* index, const float* weights,
                                     const float* error, const float* mass, const uint32_t* offsets,
                                     int64_t entries, int64_t rows, int64_t block_rows,
                                     int64_t route_stride, int64_t error_stride, int64_t tokens,
                                     int32_t width, int64_t chunk_offset, int64_t chunk_size,
                                     int32_t num_layers, int32_t layer_index, int32_t key_bits,
                                     void* workspace, size_t workspace_bytes, uint32_t* device_status,
                                     glsdm_stream_t stream) {
  return glsdm_commit_factored_phased(bank, index, weights, error, mass, offsets, entries, rows, block_rows,
                                      route_stride, error_stride, tokens, width, chunk_offset, chunk_size,
                                      num_layers, layer_index, key_bits, GLSDM_COMMIT_ORDER | GLSDM_COMMIT_APPLY,
                                      workspace, workspace_bytes, device_status, stream);
}

extern "C" int glsdm_commit_factored_phased(const glsdm_bank* bank, const int32_t* index, const float* weights,
                                            const float* error, const float* mass, const uint32_t* offsets,
                                            int64_t entries, int64_t rows, int64_t block_rows,
                                            int64_t route_stride, int64_t error_stride, int64_t tokens,
                                            int32_t width, int64_t chunk_offset, int64_t chunk_size,
                                            int32_t num_layers, int32_t layer_index, int32_t key_bits,
                                            int32_t phases, void* workspace, size_t workspace_bytes,
                                            uint32_t* device_status, glsdm_stream_t stream) {
  if ((phases & ~(GLSDM_COMMIT_ORDER | GLSDM_COMMIT_APPLY)) != 0 || phases == 0) return GLSDM_ERR_ARGUMENT;
  if (rows == 0 || entries == 0) return GLSDM_OK;
  if (bank == nullptr || bank->values == nullptr) return GLSDM_ERR_ARGUMENT;
  if (bank->dtype != GLSDM_F32 && bank->dtype != GLSDM_BF16) return GLSDM_ERR_ARGUMENT;
  if (index == nullptr || weights == nullptr || error == nullptr || workspace == nullptr) return GLSDM_ERR_ARGUMENT;
  if (rows < 0 || entries < 0 || tokens < 1 || width < 1 || chunk_size < 1 || num_layers < 1 || layer_index < 0 ||
      layer_index >= num_layers || chunk_offset < 0 || block_rows < 1 || route_stride < 0 || error_stride < 0)
    return GLSDM_ERR_ARGUMENT;
  if (key_bits < 0 || key_bits > 64) return GLSDM_ERR_ARGUMENT;
  if (width > 32 || bank->banks != 1) return GLSDM_ERR_UNSUPPORTED;
  if (entries > 0xfffffff0ll) return GLSDM_ERR_LIMIT;
  if (offsets == nullptr && (entries != rows * width || rows % (static_cast<int64_t>(bank->heads) * tokens) != 0))
    return GLSDM_ERR_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return GLSDM_ERR_ARGUMENT;
  const BankView v = make_view(*bank);
  // Descriptors address error rows with 32 bits.
  const int64_t blocks = (rows + block_rows - 1) / block_rows;
  if ((blocks - 1) * error_stride + block_rows * static_cast<int64_t>(v.dim + 1) > 0xffffffffll) return GLSDM_ERR_LIMIT;
  Workspace w;
  FactoredScratch f;
  const size_t need = carve_factored(&w, &f, static_cast<char*>(workspace), entries, v.dim);
  if (workspace_bytes < need) return GLSDM_ERR_WORKSPACE;

  // 16-byte loads of error rows and bank rows need aligned bases and row offsets.
  const bool aligned = (reinterpret_cast<uintptr_t>(error) & 15u) == 0 &&
                       (reinterpret_cast<uintptr_t>(bank->values) & 15u) == 0 &&
                       (error_stride % 4 == 0 || block_rows >= rows) && v.dim % 4 == 0;
  // A shard of several owns only some of the routes it is shown: about entries * (its slots / all).
  const bool shard = v.slot_lo != 0 || v.slot_hi != v.slots;
  const int64_t expected = shard ? entries * (v.slot_hi - v.slot_lo) / v.slots : entries;
  const bool once = offsets == nullptr && aligned &&
                    once_path_pays(expected, static_cast<int64_t>(v.heads) * v.part_stride_rows) &&
                    (v.dim == 32 || v.dim == 64 || v.dim == 128 || v.dim == 256);
  const bool compact_owned = offsets == nullptr && shard && !once;
  if (once || compact_owned) w.live = f.live;
  EntryArgs e;
  {
  e.index = index; e.weights = weights; e.error = error; e.mass = mass; e.offsets = offsets;
  e.rows = rows; e.block_rows = block_rows; e.route_stride = route_stride; e.error_stride = error_stride;
  e.tokens = tokens; e.sequences = rows / (static_cast<int64_t>(v.heads) * tokens); e.chunk_offset = chunk_offset; e.key_stride = chunk_size * num_layers;
  e.width = width; e.num_layers = num_layers; e.layer_index = layer_index;
  }
  w.device_status = device_status;
  // One call doing both phases on the single-writer path: list and sort the shared-address
  // entries on a second stream while the caller's stream updates the single-writer rows.
  const bool overlap = once && phases == (GLSDM_COMMIT_ORDER | GLSDM_COMMIT_APPLY);
  SideLane* side = nullptr;
  if (phases & GLSDM_COMMIT_ORDER) {
    // Dense numbering sorts by address alone (one value past the last address marks a slot
    // outside the bank; the compacted list of the single-writer path holds no such slot).
    const int64_t largest_key = static_cast<int64_t>(v.heads) * v.slots - ((once || compact_owned) ? 1 : 0);
    int address_bits = 1;
    while (largest_key >> address_bits) ++address_bits;
    const int passes = sort_passes(offsets == nullptr ? address_bits : key_bits);
    const int row_blocks = blocks_for(rows, kWarpsPerBlock * kEntryRows);
    const SortGather gather = {f.addresses, reinterpret_cast<const uint4*>(f.described),
                               reinterpret_cast<uint4*>(f.sorted)};
    int ordered = -1;
    if (!once && entries <= kOrderAllMaxEntries && order_all_enabled()) {
      if (compact_owned)
        ordered = launch_order_all<kOwnedCompact>(v, e, f, w, passes, entries, f.zero_chain, device_status, gather, stream);
      else if (offsets == nullptr)
        ordered = launch_order_all<kEveryRoute>(v, e, f, w, passes, entries, 0, device_status, gather, stream);
      else
        ordered = launch_order_all<kOwnedRoutes>(v, e, f, w, passes, entries, 0, device_status, gather, stream);
      if (ordered > 0) return ordered;
    }
    if (ordered != GLSDM_OK) {
    if (int s = clear_sort_state(w, once ? f.zero_extra : (compact_owned ? f.zero_chain : 0), stream)) return s;
    glsdm_stream_t order_stream = stream;
    if (once) {
      mark_addresses_kernel<<<blocks_for(rows, kWarpsPerBlock), kWarpsPerBlock * 32, 0, stream>>>(v, e, f);
      count_launches(1);
      if (overlap) {
        if (int s = side_lane(&side)) return s;
        GLSDM_CUDA_OK(cudaEventRecord(side->fork, stream), "factored commit fork");
        GLSDM_CUDA_OK(cudaStreamWaitEvent(side->stream, side->fork, 0), "factored commit fork wait");
        order_stream = side->stream;
      }
      entry_stage_kernel<kSharedAddresses><<<row_blocks, kWarpsPerBlock * 32, 0, order_stream>>>(
          v, e, f, w, passes, entries, device_status);
      count_launches(1);
    } else if (compact_owned) {
      entry_stage_kernel<kOwnedCompact><<<row_blocks, kWarpsPerBlock * 32, 0, stream>>>(
          v, e, f, w, passes, entries, device_status);
      count_launches(1);
    } else if (offsets == nullptr) {
      entry_stage_kernel<kEveryRoute><<<row_blocks, kWarpsPerBlock * 32, 0, stream>>>(
          v, e, f, w, passes, entries, device_status);
      count_launches(1);
    } else {
      entry_stage_kernel<kOwnedRoutes><<<row_blocks, kWarpsPerBlock * 32, 0, stream>>>(
          v, e, f, w, passes, entries, device_status);
      count_launches(1);
    }
    GLSDM_CUDA_OK(cudaGetLastError(), "factored entry stage launch");
    if (int s = run_passes(w, entries, passes, gather, order_stream)) return s;
    }
  }
  if (!(phases & GLSDM_COMMIT_APPLY)) return GLSDM_OK;

  FactoredArgs a;
  a.values = const_cast<void*>(bank->values);
  a.error = error;
  a.sorted = f.sorted;
  a.entries = entries;
  a.bank_rows = static_cast<int64_t>(v.heads) * v.part_stride_rows;
  a.dim = v.dim;
  a.device_status = device_status;
  // Single-writer rows on the caller's stream, the shared addresses' rows (other rows) beside
  // them on the side stream: in the one-call form that stream has just sorted them; when only
  // the apply phase was asked for it is forked here.
  if (overlap || (once && once_bulk())) {
    if (side == nullptr) {
      if (int s = side_lane(&side)) return s;
      GLSDM_CUDA_OK(cudaEventRecord(side->fork, stream), "factored commit fork");
      GLSDM_CUDA_OK(cudaStreamWaitEvent(side->stream, side->fork, 0), "factored commit fork wait");
    }
    const bool f32 = bank->dtype == GLSDM_F32;
    int status;
    switch (v.dim) {
      case 32: status = f32 ? launch_once<float, 1>(a, v, e, f, stream) : launch_once<__nv_bfloat16, 1>(a, v, e, f, stream); break;
      case 64: status = f32 ? launch_once<float, 2>(a, v, e, f, stream) : launch_once<__nv_bfloat16, 2>(a, v, e, f, stream); break;
      case 128: status = f32 ? launch_once<float, 4>(a, v, e, f, stream) : launch_once<__nv_bfloat16, 4>(a, v, e, f, stream); break;
      default: status = f32 ? launch_once<float, 8>(a, v, e, f, stream) : launch_once<__nv_bfloat16, 8>(a, v, e, f, stream); break;
    }
    if (status) return status;
    // the shared addresses' rows are other rows than the single-writer ones: their reduction
    // follows the sort on the side stream and the caller's stream only waits for its end
    status = bank->dtype == GLSDM_F32 ? launch_factored<float>(w, a, aligned, side->stream)
                                      : launch_factored<__nv_bfloat16>(w, a, aligned, side->stream);
    if (status) return status;
    GLSDM_CUDA_OK(cudaEventRecord(side->join, side->stream), "factored commit join");
    GLSDM_CUDA_OK(cudaStreamWaitEvent(stream, side->join, 0), "factored commit join wait");
    return GLSDM_OK;
  }
  if (once) {
    const bool f32 = bank->dtype == GLSDM_F32;
    switch (v.dim) {
      case 32: return f32 ? launch_split<float, 1>(w, a, v, e, f, stream) : launch_split<__nv_bfloat16, 1>(w, a, v, e, f, stream);
      case 64: return f32 ? launch_split<float, 2>(w, a, v, e, f, stream) : launch_split<__nv_bfloat16, 2>(w, a, v, e, f, stream);
      case 128: return f32 ? launch_split<float, 4>(w, a, v, e, f, stream) : launch_split<__nv_bfloat16, 4>(w, a, v, e, f, stream);
      default: return f32 ? launch_split<float, 8>(w, a, v, e, f, stream) : launch_split<__nv_bfloat16, 8>(w, a, v, e, f, stream);
    }
  }
  if (bank->dtype == GLSDM_F32) return launch_factored<float>(w, a, aligned, stream);
  return launch_factored<__nv_bfloat16>(w, a, aligned, stream);
}
