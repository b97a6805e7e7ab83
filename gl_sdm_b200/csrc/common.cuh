// Shared device helpers: order-preserving score keys, the warp-wide streaming top-k
// selector used by every routing kernel, and small launch utilities.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "glsdm.h"

namespace glsdm {

constexpr unsigned kFullMask = 0xffffffffu;
constexpr int kWarpsPerBlock = 8;
constexpr int kStageKeys = 64;   // staged candidate keys per warp (shared memory, 8 bytes each)
// Per-warp selection scratch in 8-byte units: the staged keys, then 256 16-bit lane slots of
// the two-pass factor selection.
constexpr int kStageSlots = kStageKeys + 64;

// Thread-local record of the last CUDA failure, for glsdm_last_cuda_error().
void note_cuda_error(cudaError_t err, const char* where);
// Process-wide count of kernels this library has launched (glsdm_kernel_launches()).
void count_launches(int n);

#define GLSDM_CUDA_OK(expr, where)                  \
  do {                                              \
    cudaError_t e__ = (expr);                       \
    if (e__ != cudaSuccess) {                       \
      ::glsdm::note_cuda_error(e__, where);         \
      return GLSDM_ERR_CUDA;                        \
    }                                               \
  } while (0)

// Map an fp32 score to a uint32 whose unsigned order is the float order, with -0.0 == +0.0
// (the reference compares scores with torch sorts, for which the two zeros tie) and every
// NaN folded to one value above +inf (torch sorts NaN as the largest value).
__device__ __forceinline__ uint32_t orderable_bits(float v) {
  uint32_t b = __float_as_uint(__fadd_rn(v, 0.0f));
  if ((b & 0x7fffffffu) > 0x7f800000u) b = 0x7fc00000u;
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float from_orderable_bits(uint32_t o) {
  return __uint_as_float((o & 0x80000000u) ? (o ^ 0x80000000u) : ~o);
}

__device__ __forceinline__ uint64_t pack_key(uint32_t hi, uint32_t lo) {
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

__device__ __forceinline__ uint64_t shfl_u64(uint64_t v, int src) {
  return __shfl_sync(kFullMask, v, src);
}

__device__ __forceinline__ uint64_t shfl_xor_u64(uint64_t v, int mask) {
  return __shfl_xor_sync(kFullMask, v, mask);
}

// One compare-exchange step across lanes: the lane keeps the larger of (own, partner) when
// keep_max, else the smaller.
__device__ __forceinline__ uint64_t exchange_step(uint64_t x, int j, bool keep_max) {
  const uint64_t y = shfl_xor_u64(x, j);
  const bool take = (y > x) == keep_max;  // equal keys (both empty): either choice is the same
  return take ? y : x;
}

// Bitonic sort of one 64-bit key per lane, descending (lane 0 ends with the largest).
__device__ __forceinline__ uint64_t warp_sort_desc(uint64_t x, int lane) {
#pragma unroll
  for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      const bool up = (lane & k) == 0;
      const bool lower = (lane & j) == 0;
      x = exchange_step(x, j, up == lower);
    }
  }
  return x;
}

// Merge two descending 32-lists (one key per lane each) and keep the 32 largest, descending.
__device__ __forceinline__ uint64_t warp_merge_desc(uint64_t list, uint64_t sorted, int lane) {
  const uint64_t rev = shfl_u64(sorted, 31 - lane);
  uint64_t x = list > rev ? list : rev;  // bitonic, holds the 32 largest of the union
#pragma unroll
  for (int j = 16; j > 0; j >>= 1) x = exchange_step(x, j, (lane & j) == 0);
  return x;
}

// Streaming selection of the `keep` (<= 32) largest distinct 64-bit keys offered to a warp.
// Key 0 means "nothing". Keys above the running threshold are staged in shared memory;
// every 32 staged keys are sorted and merged into the lane-resident list. Because keys
// carry the element's index in their low bits they are distinct, so the result does not
// depend on the order in which they were offered.
struct WarpSelect {
  uint64_t list;    // lane i: i-th largest key so far
  uint64_t thresh;  // key held by lane keep-1 (warp-uniform)
  uint64_t* stage;  // kStageSlots entries owned by this warp
  int staged;       // warp-uniform
  int keep;
  int lane;

  __device__ __forceinline__ void init(uint64_t* stage_, int keep_, int lane_) {
    list = 0;
    thresh = 0;
    stage = stage_;
    staged = 0;
    keep = keep_;
    lane = lane_;
  }

  __device__ __forceinline__ void merge_staged32() {
    __syncwarp();
    const uint64_t x = stage[lane];
    const int rest = staged - 32;
    const uint64_t tail = (lane < rest) ? stage[32 + lane] : 0;
    __syncwarp();
    if (lane < rest) stage[lane] = tail;
    staged = rest;
    list = warp_merge_desc(list, warp_sort_desc(x, lane), lane);
    thresh = shfl_u64(list, keep - 1);
  }

  __device__ __forceinline__ void offer(uint64_t key) {
    const bool pass = key > thresh;
    const unsigned mask = __ballot_sync(kFullMask, pass);
    if (mask == 0) return;
    const int rank = __popc(mask & ((1u << lane) - 1u));
    if (pass) stage[staged + rank] = key;
    staged += __popc(mask);
    if (staged >= 32) merge_staged32();
  }

  __device__ __forceinline__ void finish() {
    if (staged > 0) {
      __syncwarp();
      const uint64_t x = (lane < staged) ? stage[lane] : 0;
      __syncwarp();
      staged = 0;
      list = warp_merge_desc(list, warp_sort_desc(x, lane), lane);
      thresh = shfl_u64(list, keep - 1);
    }
  }
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, o));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
  return v;
}

// Turn the selector's final list (key = orderable score << 32 | slot, best first) into the
// reference's output order: slots ascending, weights = softmax of the selected scores in
// that order (gl_sdm/memory/routing.py:25-26). Lanes >= count receive slot 0, weight 0.
__device__ __forceinline__ void canonical_routes(uint64_t list, int count, int lane,
                                                 uint32_t& slot, float& weight, float& score) {
  const uint64_t by_slot =
      (lane < count) ? pack_key(static_cast<uint32_t>(list), static_cast<uint32_t>(list >> 32))
                     : ~0ull;
  // Ascending by slot == descending by the complement; unused lanes (0) sink to the end.
  const uint64_t sorted = ~warp_sort_desc(~by_slot, lane);
  const bool live = lane < count;
  slot = live ? static_cast<uint32_t>(sorted >> 32) : 0u;
  score = live ? from_orderable_bits(static_cast<uint32_t>(sorted)) : -INFINITY;
  const float top = warp_max(score);
  const float e = live ? expf(score - top) : 0.0f;
  const float total = warp_sum(e);
  weight = live ? e / total : 0.0f;
}

inline int blocks_for(int64_t items, int per_block) {
  return static_cast<int>((items + per_block - 1) / per_block);
}

}  // namespace glsdm
