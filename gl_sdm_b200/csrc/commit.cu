// Buffered commit: stable LSD radix sort of the entries by key, segmented fp32 reduction
// per address in sorted order, one read-modify-write per touched bank row.
// Replaces gl_sdm/memory/transactions.py:69-97 and gl_sdm/memory/backends/commit.py:12-58.
//
// Phases (all on the caller's stream, no host synchronisation, no float atomics):
//   1. clear       one memset of the histogram, the plan and the look-back words
//   2. prepare     keys -> order-preserving u64, entry ids, per-digit histograms (8 x 256);
//                  the block that finishes last writes the plan (a digit on which every key
//                  agrees needs no pass)
//   3. per digit   ONE launch: each tile counts its digits, learns the counts of the earlier
//                  tiles by looking back along a chain of published words, and scatters
//                  stably, ping-ponging two buffers; the last pass also writes the sorted
//                  address of every position
//   4. reduce      one warp per 32 sorted positions; each segment head sums its segment
//                  left to right and updates its bank row; segments longer than
//                  kLongSegment are queued
//   5. long        one block per queued segment: fixed 256-entry chunks summed left to
//                  right by warps, chunk sums added left to right, row updated
#include <mutex>

#include "commit.cuh"

namespace glsdm {
namespace {

// Sum entries [start, start+count) of the sorted order, strictly left to right.
template <int V>
__device__ __forceinline__ void sum_run(Slice<V>& acc, const uint32_t* __restrict__ ids,
                                        const float* __restrict__ deltas, int dim, int64_t start,
                                        int64_t count, int lane) {
  for (int64_t done = 0; done < count; done += 32) {
    const int n = (count - done < 32) ? static_cast<int>(count - done) : 32;
    const uint32_t mine = (lane < n) ? ids[start + done + lane] : 0u;
    if (count > 8 && lane < n) prefetch_row(deltas + static_cast<int64_t>(mine) * dim, dim);   // lane t: entry t's row
    int t = 0;
    for (; t + 4 <= n; t += 4) {
      Slice<V> x[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t e = __shfl_sync(kFullMask, mine, t + j);
        load_delta<V>(x[j], deltas + static_cast<int64_t>(e) * dim, lane);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) add<V>(acc, x[j]);
    }
    for (; t < n; ++t) {
      Slice<V> x;
      const uint32_t e = __shfl_sync(kFullMask, mine, t);
      load_delta<V>(x, deltas + static_cast<int64_t>(e) * dim, lane);
      add<V>(acc, x);
    }
  }
}

// Generic-width variant: any dim, lanes stride the columns, 8 column blocks per sweep.
__device__ __forceinline__ void sum_run_generic(float (&acc)[8], const uint32_t* __restrict__ ids,
                                                const float* __restrict__ deltas, int dim, int c0,
                                                int64_t start, int64_t count, int lane) {
  for (int64_t t = 0; t < count; ++t) {
    const float* row = deltas + static_cast<int64_t>(ids[start + t]) * dim;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + j * 32 + lane;
      if (c < dim) acc[j] = __fadd_rn(acc[j], __ldg(row + c));
    }
  }
}

struct ReduceArgs {
  const void* values_in;
  void* values_out;
  const float* deltas;
  int64_t entries;
  int64_t row_base;
  int64_t bank_rows;
  int dim;
  uint32_t* device_status;
  // Optional undo log: the row each touched address held BEFORE this commit, stored at the
  // sorted position of the address's first entry (other positions stay unwritten).
  void* undo_rows;
};

// Rows of the single-entry fast path in flight per warp, and resident blocks per SM the
// compiler must leave room for. Measured on B200 (1,048,576 entries into a 16,777,216 x 256
// bf16 bank): 2 rows x 4 blocks (64 registers, 32 warps per SM) 609 us per commit against
// 706 us for 4 rows x 2 blocks and 996 us for 8 rows: the kernel wants resident warps, not
// deeper batches.
#ifndef GLSDM_SINGLES_BATCH
#define GLSDM_SINGLES_BATCH 2
#endif
#ifndef GLSDM_REDUCE_MIN_BLOCKS
#define GLSDM_REDUCE_MIN_BLOCKS 4
#endif
template <typename T, int V>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, GLSDM_REDUCE_MIN_BLOCKS)
reduce_kernel(Workspace w, ReduceArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t first = (static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp) * 32;
  if (first >= a.entries) return;
  const int64_t* __restrict__ sorted = w.sorted_address;
  const uint32_t* __restrict__ ids = w.ids[w.plan->final_buffer];
  const int64_t at = first + lane;
  const int64_t mine = at < a.entries ? sorted[at] : -1;
  const int64_t prev = (at > 0 && at < a.entries) ? sorted[at - 1] : -2;
  const bool is_head = at < a.entries && (at == 0 || mine != prev);
  const unsigned all_heads = __ballot_sync(kFullMask, is_head);
  unsigned heads = all_heads;
  // An undo log is searched by bisection later: say so now if its addresses ever descend.
  if (a.undo_rows != nullptr && a.device_status != nullptr && at > 0 && at < a.entries && prev > mine)
    atomicOr(a.device_status, GLSDM_DEV_LOG_NOT_ASCENDING);
  if constexpr (V > 0) {
    // Fast path for addresses that received exactly one entry (the common case): a few such
    // rows at a time, all their delta rows and old bank rows requested before any is used.
    const int64_t next = (at + 1 < a.entries) ? sorted[at + 1] : -3;
    const int64_t mine_local = mine - a.row_base;
    const uint32_t my_id = at < a.entries ? ids[at] : 0u;
    unsigned singles = __ballot_sync(kFullMask, is_head && mine != next && mine_local >= 0 && mine_local < a.bank_rows);
    heads &= ~singles;
    // narrower rows leave registers for more rows in flight (what a latency-bound warp needs)
    constexpr int kB = V >= 8 ? GLSDM_SINGLES_BATCH : (V >= 4 ? 2 * GLSDM_SINGLES_BATCH : 4 * GLSDM_SINGLES_BATCH);
    while (singles) {
      int pick[kB];
#pragma unroll
      for (int j = 0; j < kB; ++j) {
        pick[j] = singles ? __ffs(singles) - 1 : -1;
        if (singles) singles &= singles - 1;
      }
      Slice<V> delta[kB], old[kB];
      int64_t where[kB];
#pragma unroll
      for (int j = 0; j < kB; ++j) {
        if (pick[j] < 0) continue;
        const uint32_t e = __shfl_sync(kFullMask, my_id, pick[j]);
        where[j] = __shfl_sync(kFullMask, mine_local, pick[j]);
        load_delta<V>(delta[j], a.deltas + static_cast<int64_t>(e) * a.dim, lane);
        load_bank<T, V>(static_cast<const T*>(a.values_in) + where[j] * a.dim, old[j], lane);
      }
      if (a.undo_rows != nullptr) {
#pragma unroll
        for (int j = 0; j < kB; ++j) {
          if (pick[j] < 0) continue;
          store_bank<T, V>(static_cast<T*>(a.undo_rows) + (first + pick[j]) * a.dim, old[j], lane);
        }
      }
#pragma unroll
      for (int j = 0; j < kB; ++j) {
        if (pick[j] < 0) continue;
#pragma unroll
        for (int i = 0; i < V; ++i) old[j].v[i] = __fadd_rn(old[j].v[i], __fadd_rn(0.f, delta[j].v[i]));
        store_bank<T, V>(static_cast<T*>(a.values_out) + where[j] * a.dim, old[j], lane);
      }
    }
  }
  while (heads) {
    const int h = __ffs(heads) - 1;
    heads &= heads - 1;
    const int64_t start = first + h;
    const int64_t address = __shfl_sync(kFullMask, mine, h);
    const int64_t local = address - a.row_base;
    if (local < 0 || local >= a.bank_rows) {
      if (lane == 0 && a.device_status) atomicOr(a.device_status, GLSDM_DEV_ADDRESS_OUT_OF_RANGE);
      continue;
    }
    // The next head inside this warp's 32 positions ends the segment; only a segment that
    // runs to the end of the batch has to look at the following positions.
    int64_t len;
    const unsigned later = h == 31 ? 0u : (all_heads & (0xffffffffu << (h + 1)));
    if (later) {
      len = (__ffs(later) - 1) - h;
    } else {
      const int64_t tail = first + 32 < a.entries ? first + 32 : a.entries;
      len = tail - start;
      if (tail < a.entries) len = segment_length(sorted, tail - 1, a.entries, address, lane) + (tail - 1 - start);
    }
    if (len > kLongSegment) {
      if (lane == 0) {
        const uint32_t slot = atomicAdd(&w.plan->long_count, 1u);
        w.long_list[slot] = make_uint2(static_cast<uint32_t>(start), static_cast<uint32_t>(len));
      }
      continue;
    }
    const T* in_row = static_cast<const T*>(a.values_in) + local * a.dim;
    T* out_row = static_cast<T*>(a.values_out) + local * a.dim;
    if constexpr (V > 0) {
      Slice<V> acc;
      zero<V>(acc);
      sum_run<V>(acc, ids, a.deltas, a.dim, start, len, lane);
      if (a.undo_rows != nullptr) {
        Slice<V> old;
        load_bank<T, V>(in_row, old, lane);
        store_bank<T, V>(static_cast<T*>(a.undo_rows) + start * a.dim, old, lane);
#pragma unroll
        for (int i = 0; i < V; ++i) old.v[i] = __fadd_rn(old.v[i], acc.v[i]);
        store_bank<T, V>(out_row, old, lane);
      } else {
        apply_row<T, V>(in_row, out_row, acc, lane);
      }
    } else {
      for (int c0 = 0; c0 < a.dim; c0 += 256) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        sum_run_generic(acc, ids, a.deltas, a.dim, c0, start, len, lane);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int c = c0 + j * 32 + lane;
          if (c < a.dim) {
            const float o = load_value<T>(in_row + c);
            if (a.undo_rows != nullptr) store_value<T>(static_cast<T*>(a.undo_rows) + start * a.dim + c, o);
            store_value<T>(out_row + c, __fadd_rn(o, acc[j]));
          }
        }
      }
    }
  }
}

// One block per queued long segment. Chunk c covers entries [c*256, c*256+256) of the
// segment; warp (c % warps) sums it in order and stores the partial; warp 0 then adds the
// partials in chunk order. The grouping depends only on the segment's length.
template <typename T, int V>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
long_segment_kernel(Workspace w, ReduceArgs a) {
  __shared__ uint32_t partial_base;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t* __restrict__ ids = w.ids[w.plan->final_buffer];
  const uint32_t count = w.plan->long_count;
  for (uint32_t s = blockIdx.x; s < count; s += gridDim.x) {
    const uint2 seg = w.long_list[s];
    const int64_t start = seg.x, len = seg.y;
    const int chunks = static_cast<int>((len + kLongSegment - 1) / kLongSegment);
    __syncthreads();
    if (threadIdx.x == 0) partial_base = atomicAdd(&w.plan->chunk_cursor, static_cast<uint32_t>(chunks));
    __syncthreads();
    float* __restrict__ partial = w.partial + static_cast<int64_t>(partial_base) * a.dim;
    const int64_t local = w.sorted_address[start] - a.row_base;
    const T* in_row = static_cast<const T*>(a.values_in) + local * a.dim;
    T* out_row = static_cast<T*>(a.values_out) + local * a.dim;
    for (int c = warp; c < chunks; c += kWarpsPerBlock) {
      const int64_t cs = start + static_cast<int64_t>(c) * kLongSegment;
      const int64_t cn = (len - static_cast<int64_t>(c) * kLongSegment < kLongSegment)
                             ? len - static_cast<int64_t>(c) * kLongSegment : kLongSegment;
      float* prow = partial + static_cast<int64_t>(c) * a.dim;
      if constexpr (V > 0) {
        Slice<V> acc;
        zero<V>(acc);
        sum_run<V>(acc, ids, a.deltas, a.dim, cs, cn, lane);
#pragma unroll
        for (int i = 0; i < V; ++i) prow[column_of<V>(lane, i)] = acc.v[i];
      } else {
        for (int c0 = 0; c0 < a.dim; c0 += 256) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          sum_run_generic(acc, ids, a.deltas, a.dim, c0, cs, cn, lane);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int col = c0 + j * 32 + lane;
            if (col < a.dim) prow[col] = acc[j];
          }
        }
      }
    }
    __syncthreads();
    // Columns are spread over the whole block for the in-order sum of the chunk partials.
    for (int col = threadIdx.x; col < a.dim; col += blockDim.x) {
      float total = 0.f;
      for (int c = 0; c < chunks; ++c) total = __fadd_rn(total, partial[static_cast<int64_t>(c) * a.dim + col]);
      const float o = load_value<T>(in_row + col);
      if (a.undo_rows != nullptr) store_value<T>(static_cast<T*>(a.undo_rows) + start * a.dim + col, o);
      store_value<T>(out_row + col, __fadd_rn(o, total));
    }
  }
}

template <typename T>
int launch_reduce(const Workspace& w, const ReduceArgs& a, glsdm_stream_t stream) {
  const int grid = blocks_for((a.entries + 31) / 32, kWarpsPerBlock);
  const int long_grid = static_cast<int>(w.long_capacity < 1184 ? w.long_capacity : 1184);
  const bool aligned = (reinterpret_cast<uintptr_t>(a.deltas) & 15u) == 0 &&
                       (reinterpret_cast<uintptr_t>(a.values_in) & 15u) == 0 &&
                       (reinterpret_cast<uintptr_t>(a.values_out) & 15u) == 0 &&
                       (reinterpret_cast<uintptr_t>(a.undo_rows) & 15u) == 0;
#define GLSDM_REDUCE(V)                                                                     \
  do {                                                                                      \
    reduce_kernel<T, V><<<grid, kWarpsPerBlock * 32, 0, stream>>>(w, a);                    \
    GLSDM_CUDA_OK(cudaGetLastError(), "commit reduce launch");                              \
    long_segment_kernel<T, V><<<long_grid, kWarpsPerBlock * 32, 0, stream>>>(w, a);         \
    GLSDM_CUDA_OK(cudaGetLastError(), "commit long-segment launch");                        \
    count_launches(2);                                                                      \
  } while (0)
  if (aligned && a.dim == 32) GLSDM_REDUCE(1);
  else if (aligned && a.dim == 64) GLSDM_REDUCE(2);
  else if (aligned && a.dim == 128) GLSDM_REDUCE(4);
  else if (aligned && a.dim == 256) GLSDM_REDUCE(8);
  else GLSDM_REDUCE(0);
#undef GLSDM_REDUCE
  return GLSDM_OK;
}

}  // namespace
}  // namespace glsdm

using namespace glsdm;

extern "C" size_t glsdm_commit_workspace_bytes(int64_t entries, int32_t dim) {
  if (entries < 0 || dim < 1) return 0;
  return carve(nullptr, nullptr, entries < 1 ? 1 : entries, dim);
}

namespace glsdm {
namespace {
int commit_impl(const void* values_in, void* values_out, int dtype, int64_t row_base,
                int64_t bank_rows, int32_t dim, const int64_t* addresses,
                const float* deltas, const int64_t* keys, int64_t entries,
                int32_t key_bits, void* workspace, size_t workspace_bytes,
                int64_t* undo_addresses, void* undo_rows,
                uint32_t* device_status, glsdm_stream_t stream) {
  if (values_in == nullptr || bank_rows < 1 || dim < 1 || entries < 0) return GLSDM_ERR_ARGUMENT;
  if (dtype != GLSDM_F32 && dtype != GLSDM_BF16) return GLSDM_ERR_ARGUMENT;
  if (entries > 0xfffffff0ll) return GLSDM_ERR_LIMIT;
  if (key_bits < 0 || key_bits > 64) return GLSDM_ERR_ARGUMENT;
  const size_t elem = dtype == GLSDM_F32 ? 4 : 2;
  if (values_out == nullptr) values_out = const_cast<void*>(values_in);
  Workspace w;
  if (entries > 0) {
    // every check comes before the first byte of values_out is written
    if (addresses == nullptr || deltas == nullptr || workspace == nullptr) return GLSDM_ERR_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return GLSDM_ERR_ARGUMENT;
    const size_t need = carve(&w, static_cast<char*>(workspace), entries, dim);
    if (workspace_bytes < need) return GLSDM_ERR_WORKSPACE;
  }
  if (values_out != values_in) {
    GLSDM_CUDA_OK(cudaMemcpyAsync(values_out, values_in, elem * bank_rows * dim,
                                  cudaMemcpyDeviceToDevice, stream), "commit bank copy");
  }
  if (entries == 0) return GLSDM_OK;
  if (keys == nullptr) keys = addresses;
  w.device_status = device_status;
  const SortGather gather = {addresses, nullptr, nullptr};
  if (int s = run_sort(w, keys, entries, sort_passes(key_bits), gather, stream)) return s;

  ReduceArgs a;
  a.values_in = values_in;
  a.values_out = values_out;
  a.deltas = deltas;
  a.entries = entries;
  a.row_base = row_base;
  a.bank_rows = bank_rows;
  a.dim = dim;
  a.device_status = device_status;
  a.undo_rows = undo_rows;
  if (undo_addresses != nullptr) {
    GLSDM_CUDA_OK(cudaMemcpyAsync(undo_addresses, w.sorted_address, sizeof(int64_t) * entries,
                                  cudaMemcpyDeviceToDevice, stream), "commit undo addresses");
  }
  if (dtype == GLSDM_F32) return launch_reduce<float>(w, a, stream);
  return launch_reduce<__nv_bfloat16>(w, a, stream);
}

// One warp per log position: the first position of every address run holds that address's
// row from before the commit; copy it back into the bank.
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
undo_apply_kernel(T* __restrict__ values, int64_t row_base, int64_t bank_rows, int dim,
                  const int64_t* __restrict__ log_addresses, const T* __restrict__ log_rows,
                  int64_t entries) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t at = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (at >= entries) return;
  const int64_t address = log_addresses[at];
  if (at > 0 && log_addresses[at - 1] == address) return;
  const int64_t local = address - row_base;
  if (local < 0 || local >= bank_rows) return;
  const T* src = log_rows + at * dim;
  T* dst = values + local * dim;
  for (int c = lane; c < dim; c += 32) dst[c] = src[c];
}
}  // namespace
}  // namespace glsdm

extern "C" int glsdm_commit(const void* values_in, void* values_out, int dtype, int64_t row_base,
                            int64_t bank_rows, int32_t dim, const int64_t* addresses,
                            const float* deltas, const int64_t* keys, int64_t entries,
                            int32_t key_bits, void* workspace, size_t workspace_bytes,
                            uint32_t* device_status, glsdm_stream_t stream) {
  return commit_impl(values_in, values_out, dtype, row_base, bank_rows, dim, addresses, deltas, keys,
                     entries, key_bits, workspace, workspace_bytes, nullptr, nullptr, device_status, stream);
}

extern "C" int glsdm_commit_undo(void* values, int dtype, int64_t row_base, int64_t bank_rows,
                                 int32_t dim, const int64_t* addresses, const float* deltas,
                                 const int64_t* keys, int64_t entries, int32_t key_bits,
                                 void* workspace, size_t workspace_bytes, int64_t* undo_addresses,
                                 void* undo_rows, uint32_t* device_status, glsdm_stream_t stream) {
  if (entries > 0 && (undo_addresses == nullptr || undo_rows == nullptr)) return GLSDM_ERR_ARGUMENT;
  return commit_impl(values, values, dtype, row_base, bank_rows, dim, addresses, deltas, keys, entries,
                     key_bits, workspace, workspace_bytes, undo_addresses, undo_rows, device_status, stream);
}

extern "C" int glsdm_undo_apply(void* values, int dtype, int64_t row_base, int64_t bank_rows,
                                int32_t dim, const int64_t* undo_addresses, const void* undo_rows,
                                int64_t entries, glsdm_stream_t stream) {
  if (entries < 0 || bank_rows < 1 || dim < 1) return GLSDM_ERR_ARGUMENT;
  if (dtype != GLSDM_F32 && dtype != GLSDM_BF16) return GLSDM_ERR_ARGUMENT;
  if (entries == 0) return GLSDM_OK;
  if (values == nullptr || undo_addresses == nullptr || undo_rows == nullptr) return GLSDM_ERR_ARGUMENT;
  const int grid = blocks_for(entries, kWarpsPerBlock);
  if (dtype == GLSDM_F32) {
    undo_apply_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        static_cast<float*>(values), row_base, bank_rows, dim, undo_addresses,
        static_cast<const float*>(undo_rows), entries);
  } else {
    undo_apply_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        static_cast<__nv_bfloat16*>(values), row_base, bank_rows, dim, undo_addresses,
        static_cast<const __nv_bfloat16*>(undo_rows), entries);
  }
  GLSDM_CUDA_OK(cudaGetLastError(), "undo_apply launch");
  count_launches(1);
  return GLSDM_OK;
}

// ---- the bounded wait on its own -------------------------------------------------------------
namespace glsdm {
namespace {
__global__ void wait_probe_kernel(const unsigned long long* words, int64_t position, uint32_t* device_status,
                                  uint32_t* out_count) {
  const uint32_t before = chain_look_back(words, 1, position, 1, device_status);
  if (out_count != nullptr) *out_count = before;
}
}  // namespace
}  // namespace glsdm

extern "C" int glsdm_wait_probe(const void* words, int64_t position, uint32_t* device_status, uint32_t* out_count,
                                glsdm_stream_t stream) {
  if (words == nullptr || position < 0 || (reinterpret_cast<uintptr_t>(words) & 7u)) return GLSDM_ERR_ARGUMENT;
  wait_probe_kernel<<<1, 1, 0, stream>>>(static_cast<const unsigned long long*>(words), position, device_status, out_count);
  GLSDM_CUDA_OK(cudaGetLastError(), "wait probe launch");
  count_launches(1);
  return GLSDM_OK;
}

// ---- commit without a caller-provided workspace -------------------------------------------
//
// Some hosts of this library have nowhere to get the commit's scratch from. A plain C or C++
// embedder of the C ABI has no tensor allocator to size a workspace with; and a serving loop
// that shares the GPU with other streams must keep cudaMalloc/cudaFree out of its request path,
// because those calls synchronise the whole device and stall everybody else's work. For them
// the scratch lives in the library image itself: a fixed array in device memory that every
// GPU which loads the library carries until the process exits.
namespace glsdm {
namespace {

constexpr int64_t kStaticMaxEntries = 65536;   // entries per commit the built-in scratch covers
constexpr int32_t kStaticMaxDim = 256;         // widest value row it covers
constexpr size_t kStaticScratchBytes = 4u << 20;

static __device__ __align__(256) unsigned char g_commit_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_address[kMaxDevices] = {};

// In host code `g_commit_scratch` is only a handle for the symbol, not a device address;
// the address each device gave the array has to be asked for, once, with that device current.
int static_scratch(void** out) {
  int device = -1;
  GLSDM_CUDA_OK(cudaGetDevice(&device), "commit_static cudaGetDevice");
  if (device < 0 || device >= kMaxDevices) return GLSDM_ERR_LIMIT;
  std::lock_guard<std::mutex> hold(g_scratch_mutex);
  if (g_scratch_address[device] == nullptr) {
    void* address = nullptr;
    GLSDM_CUDA_OK(cudaGetSymbolAddress(&address, g_commit_scratch), "commit_static cudaGetSymbolAddress");
    if (address == nullptr) return GLSDM_ERR_CUDA;
    g_scratch_address[device] = address;
  }
  *out = g_scratch_address[device];
  return GLSDM_OK;
}

}  // namespace
}  // namespace glsdm

extern "C" int glsdm_commit_static(const void* values_in, void* values_out, int dtype, int64_t row_base,
                                   int64_t bank_rows, int32_t dim, const int64_t* addresses,
                                   const float* deltas, const int64_t* keys, int64_t entries,
                                   int32_t key_bits, uint32_t* device_status, glsdm_stream_t stream) {
  if (entries < 0 || dim < 1) return GLSDM_ERR_ARGUMENT;
  if (entries > kStaticMaxEntries || dim > kStaticMaxDim) return GLSDM_ERR_LIMIT;
  if (carve(nullptr, nullptr, entries < 1 ? 1 : entries, dim) > kStaticScratchBytes) return GLSDM_ERR_LIMIT;
  void* scratch = nullptr;
  if (int s = static_scratch(&scratch)) return s;
  // The array still holds whatever the previous call left; glsdm_commit clears the digit
  // histogram, the plan (queue counters, tickets) and the look-back words with one memset,
  // nothing else is read before it is written.
  return glsdm_commit(values_in, values_out, dtype, row_base, bank_rows, dim, addresses, deltas, keys, entries,
                      key_bits, scratch, kStaticScratchBytes, device_status, stream);
}

extern "C" int64_t glsdm_commit_static_max_entries(void) { return glsdm::kStaticMaxEntries; }
