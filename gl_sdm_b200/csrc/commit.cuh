// Shared pieces of the buffered commit: scratch layout, the stable LSD radix sort of
// (key, entry id) pairs, and the per-lane row slices the reducers work on. Included by the
// translation units that finish the commit in different ways (materialised delta rows in
// commit.cu, deltas rebuilt from their factors in commit_factored.cu).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

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
  uint32_t long_count;       // queued long segments
  uint32_t chunk_cursor;     // partial-sum rows handed out so far
  uint32_t pad;
};

struct Workspace {
  uint64_t* keys[2];
  uint32_t* ids[2];
  int64_t* sorted_address;
  uint32_t* histogram;   // [kDigits][kRadix]
  uint32_t* tile_count;  // [kRadix][tiles], scanned in place
  Plan* plan;
  uint2* long_list;      // (start, length) of queued segments
  float* partial;        // [partial_rows][dim]
  int64_t partial_rows;
  int64_t long_capacity;
  int tiles;
  // When set, the number of live entries is read on the device (a list whose length the
  // host does not know): grids stay sized for the capacity, blocks past the end do nothing.
  const uint32_t* live;
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
  o->long_capacity = long_capacity;
  o->partial_rows = partial_rows;
  o->keys[0] = reinterpret_cast<uint64_t*>(take(sizeof(uint64_t) * entries));
  o->keys[1] = reinterpret_cast<uint64_t*>(take(sizeof(uint64_t) * entries));
  o->ids[0] = reinterpret_cast<uint32_t*>(take(sizeof(uint32_t) * entries));
  o->ids[1] = reinterpret_cast<uint32_t*>(take(sizeof(uint32_t) * entries));
  o->sorted_address = reinterpret_cast<int64_t*>(take(sizeof(int64_t) * entries));
  o->histogram = reinterpret_cast<uint32_t*>(take(sizeof(uint32_t) * kDigits * kRadix));
  o->tile_count = reinterpret_cast<uint32_t*>(take(sizeof(uint32_t) * kRadix * static_cast<size_t>(tiles)));
  o->plan = reinterpret_cast<Plan*>(take(sizeof(Plan)));
  o->long_list = reinterpret_cast<uint2*>(take(sizeof(uint2) * long_capacity));
  o->partial = reinterpret_cast<float*>(take(sizeof(float) * partial_rows * dim));
  return at;
}

__device__ __forceinline__ uint32_t digit_of(uint64_t key, int pass) {
  return static_cast<uint32_t>(key >> (pass * kRadixBits)) & (kRadix - 1);
}

__global__ void __launch_bounds__(kSortThreads)
prepare_kernel(const int64_t* __restrict__ keys, int64_t entries, const uint32_t* live, int passes,
               uint64_t* __restrict__ out_keys, uint32_t* __restrict__ out_ids,
               uint32_t* __restrict__ histogram) {
  __shared__ uint32_t local[kDigits][kRadix];
  entries = live_entries(live, entries);
  if (static_cast<int64_t>(blockIdx.x) * kTile >= entries) return;
  for (int i = threadIdx.x; i < kDigits * kRadix; i += kSortThreads) (&local[0][0])[i] = 0;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile;
  for (int r = 0; r < kItems; ++r) {
    const int64_t i = base + r * kSortThreads + threadIdx.x;
    if (i < entries) {
      const uint64_t k = static_cast<uint64_t>(keys[i]) ^ 0x8000000000000000ull;
      out_keys[i] = k;
      out_ids[i] = static_cast<uint32_t>(i);
      for (int p = 0; p < passes; ++p) atomicAdd(&local[p][digit_of(k, p)], 1u);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < passes * kRadix; i += kSortThreads) {
    const uint32_t c = (&local[0][0])[i];
    if (c) atomicAdd(histogram + i, c);
  }
}

__global__ void plan_kernel(const uint32_t* __restrict__ histogram, int64_t entries, const uint32_t* live,
                            int passes, Plan* plan) {
  __shared__ uint32_t uniform[kDigits];
  entries = live_entries(live, entries);
  if (threadIdx.x < kDigits) uniform[threadIdx.x] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < passes * kRadix; i += blockDim.x)
    if (histogram[i] == static_cast<uint32_t>(entries)) uniform[i / kRadix] = 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t buffer = 0;
    for (int p = 0; p < kDigits; ++p) {
      const uint32_t skip = (p >= passes) ? 1u : uniform[p];
      plan->skip[p] = skip;
      plan->source[p] = buffer;
      if (!skip) buffer ^= 1u;
    }
    plan->final_buffer = buffer;
    plan->long_count = 0;
    plan->chunk_cursor = 0;
  }
}

__global__ void __launch_bounds__(kSortThreads)
count_kernel(Workspace w, int64_t entries, int pass) {
  if (w.plan->skip[pass]) return;
  __shared__ uint32_t local[kRadix];
  entries = live_entries(w.live, entries);
  // With a device-side count the scan reads only the tiles that hold live entries.
  if (w.live != nullptr && static_cast<int64_t>(blockIdx.x) * kTile >= entries) return;
  local[threadIdx.x] = 0;
  __syncthreads();
  const uint64_t* __restrict__ keys = w.keys[w.plan->source[pass]];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile;
  for (int r = 0; r < kItems; ++r) {
    const int64_t i = base + r * kSortThreads + threadIdx.x;
    if (i < entries) atomicAdd(&local[digit_of(keys[i], pass)], 1u);
  }
  __syncthreads();
  w.tile_count[static_cast<size_t>(threadIdx.x) * w.tiles + blockIdx.x] = local[threadIdx.x];
}

// Exclusive scan of tile_count ([digit][tile] flattened): block d owns digit d. Its base is
// the number of keys with a smaller digit (from the global histogram of this pass); inside
// the digit the tiles are scanned 256 at a time with a running carry.
__global__ void __launch_bounds__(kSortThreads)
scan_kernel(Workspace w, int pass) {
  if (w.plan->skip[pass]) return;
  __shared__ uint32_t part[kSortThreads];
  __shared__ uint32_t carry;
  const int d = blockIdx.x;
  const uint32_t* __restrict__ hist = w.histogram + pass * kRadix;
  part[threadIdx.x] = (static_cast<int>(threadIdx.x) < d) ? hist[threadIdx.x] : 0u;
  __syncthreads();
  for (int off = kSortThreads / 2; off > 0; off >>= 1) {
    if (static_cast<int>(threadIdx.x) < off) part[threadIdx.x] += part[threadIdx.x + off];
    __syncthreads();
  }
  if (threadIdx.x == 0) carry = part[0];
  __syncthreads();
  uint32_t* __restrict__ row = w.tile_count + static_cast<size_t>(d) * w.tiles;
  int tiles = w.tiles;   // only the tiles that hold live entries need their bases
  if (w.live != nullptr) {
    const int64_t used = (static_cast<int64_t>(*w.live) + kTile - 1) / kTile;
    if (used < tiles) tiles = static_cast<int>(used);
  }
  for (int t0 = 0; t0 < tiles; t0 += kSortThreads) {
    const int t = t0 + threadIdx.x;
    const uint32_t c = t < tiles ? row[t] : 0u;
    part[threadIdx.x] = c;
    __syncthreads();
    for (int off = 1; off < kSortThreads; off <<= 1) {
      const uint32_t add = (static_cast<int>(threadIdx.x) >= off) ? part[threadIdx.x - off] : 0u;
      __syncthreads();
      part[threadIdx.x] += add;
      __syncthreads();
    }
    const uint32_t base = carry;
    if (t < tiles) row[t] = base + part[threadIdx.x] - c;
    __syncthreads();
    if (threadIdx.x == kSortThreads - 1) carry = base + part[threadIdx.x];
    __syncthreads();
  }
}

// Stable scatter of one tile. A warp owns 256 consecutive keys and takes them 32 at a time,
// so (warp, round, lane) order is input order; ranks inside a round come from match_any.
__global__ void __launch_bounds__(kSortThreads)
scatter_kernel(Workspace w, int64_t entries, int pass) {
  if (w.plan->skip[pass]) return;
  entries = live_entries(w.live, entries);
  if (static_cast<int64_t>(blockIdx.x) * kTile >= entries) return;
  constexpr int kWarps = kSortThreads / 32;
  __shared__ uint32_t warp_count[kWarps][kRadix];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kWarps * kRadix; i += kSortThreads) (&warp_count[0][0])[i] = 0;
  __syncthreads();
  const uint32_t src = w.plan->source[pass];
  const uint64_t* __restrict__ keys = w.keys[src];
  const uint32_t* __restrict__ ids = w.ids[src];
  uint64_t* __restrict__ out_keys = w.keys[src ^ 1u];
  uint32_t* __restrict__ out_ids = w.ids[src ^ 1u];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile + warp * (kItems * 32);
  uint64_t key[kItems];
  uint32_t id[kItems];
  uint32_t rank[kItems];
#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    const int64_t i = base + r * 32 + lane;
    const bool live = i < entries;
    key[r] = live ? keys[i] : 0;
    id[r] = live ? ids[i] : 0;
    const uint32_t d = live ? digit_of(key[r], pass) : kRadix;  // dead lanes match only each other
    const unsigned peers = __match_any_sync(kFullMask, d);
    const uint32_t before = __popc(peers & ((1u << lane) - 1u));
    uint32_t prior = 0;
    if (live) prior = warp_count[warp][d];
    __syncwarp();
    if (live && before == 0) warp_count[warp][d] = prior + __popc(peers);
    __syncwarp();
    rank[r] = prior + before;
  }
  __syncthreads();
  {
    const int d = threadIdx.x;  // kSortThreads == kRadix
    uint32_t run = w.tile_count[static_cast<size_t>(d) * w.tiles + blockIdx.x];
    for (int q = 0; q < kWarps; ++q) {
      const uint32_t c = warp_count[q][d];
      warp_count[q][d] = run;
      run += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    const int64_t i = base + r * 32 + lane;
    if (i < entries) {
      const uint32_t at = warp_count[warp][digit_of(key[r], pass)] + rank[r];
      out_keys[at] = key[r];
      out_ids[at] = id[r];
    }
  }
}

__global__ void gather_address_kernel(Workspace w, const int64_t* __restrict__ addresses,
                                      int64_t entries) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= live_entries(w.live, entries)) return;
  const uint32_t* __restrict__ ids = w.ids[w.plan->final_buffer];
  w.sorted_address[i] = addresses[ids[i]];
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

// Sort (keys[i], i) for i in [0, entries): prepare -> plan -> one count/scan/scatter round per
// digit that is not uniform. Afterwards w.ids[w.plan->final_buffer] holds the entry ids in
// stable key order; the callers gather what their reducer needs from it.
inline int run_sort(const Workspace& w, const int64_t* keys, int64_t entries, int passes,
                    glsdm_stream_t stream) {
  GLSDM_CUDA_OK(cudaMemsetAsync(w.histogram, 0, sizeof(uint32_t) * kDigits * kRadix, stream),
                "commit histogram clear");
  prepare_kernel<<<w.tiles, kSortThreads, 0, stream>>>(keys, entries, w.live, passes, w.keys[0], w.ids[0],
                                                       w.histogram);
  GLSDM_CUDA_OK(cudaGetLastError(), "commit prepare launch");
  plan_kernel<<<1, 256, 0, stream>>>(w.histogram, entries, w.live, passes, w.plan);
  GLSDM_CUDA_OK(cudaGetLastError(), "commit plan launch");
  for (int p = 0; p < passes; ++p) {
    count_kernel<<<w.tiles, kSortThreads, 0, stream>>>(w, entries, p);
    scan_kernel<<<kRadix, kSortThreads, 0, stream>>>(w, p);
    scatter_kernel<<<w.tiles, kSortThreads, 0, stream>>>(w, entries, p);
    GLSDM_CUDA_OK(cudaGetLastError(), "commit sort launch");
  }
  count_launches(2 + 3 * passes);
  return GLSDM_OK;
}

// Keys are compared as signed 64-bit integers: the top digit always carries the sign.
inline int sort_passes(int32_t key_bits) {
  return (key_bits == 0 || key_bits == 64) ? kDigits : (key_bits + kRadixBits - 1) / kRadixBits;
}

}  // namespace
}  // namespace glsdm
