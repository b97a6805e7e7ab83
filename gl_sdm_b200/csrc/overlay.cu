// Reads of an OLDER bank version through undo logs.
//
// A copy-free commit (glsdm_commit_undo) updates the bank in place and writes down, for every
// address it touches, the row that address held before. A snapshot taken before that commit
// stays readable without a copy of the bank: a row of the old version is the row recorded by
// the EARLIEST later commit that touched its address, or the bank's current row if none did.
// This is the reference's planned "immutable base + versioned touched-row updates"
// (projects/gl-sdm/OPTIMIZATION_PLAN.md, item "Represent commits as compact overlays"; the
// per-commit bank clone it replaces is gl_sdm/memory/transactions.py:96 and state.py:61-62),
// turned around so that the newest version — the one every layer reads — is the plain bank.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"
#include "glsdm.h"
#include "overlay.cuh"
#include "route.cuh"

namespace glsdm {
namespace {

// The weighted gather of route.cuh's gather_units with each route's row given by pointer
// (resolved through the logs) instead of by slot; same grouping, same order of additions, so
// a read through empty logs is bit-identical to snapshot_read.
template <typename T>
__device__ __forceinline__ void gather_units_at(uint64_t row_ptr, float weight, int count, int lane,
                                                int units, int ub, float (&acc)[Unit<T>::kElems]) {
  constexpr int E = Unit<T>::kElems;
  const int here = units < 32 ? units : 32;
  const int groups = 32 / here;
  const int g = lane / here;
  const int u = ub * 32 + (lane % here);
#pragma unroll
  for (int i = 0; i < E; ++i) acc[i] = 0.f;
  for (int k0 = 0; k0 < count; k0 += groups * 4) {
    uint4 raw[4];
    float wk[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + j * groups + g;
      const uint64_t p = shfl_u64(row_ptr, k & 31);
      const float w = __shfl_sync(kFullMask, weight, k & 31);
      const bool live = k < count && p != 0;
      wk[j] = live ? w : 0.f;
      raw[j] = make_uint4(0u, 0u, 0u, 0u);
      if (live) raw[j] = __ldg(reinterpret_cast<const uint4*>(p) + u);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v[E];
      Unit<T>::decode(raw[j], v);
#pragma unroll
      for (int i = 0; i < E; ++i) acc[i] = fmaf(wk[j], v[i], acc[i]);
    }
  }
  for (int off = here; off < 32; off <<= 1) {
#pragma unroll
    for (int i = 0; i < E; ++i) acc[i] += __shfl_xor_sync(kFullMask, acc[i], off);
  }
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
overlay_read_kernel(BankView bank, const void* __restrict__ index, int i64,
                    const float* __restrict__ weights, int64_t rows, int64_t rows_per_bank,
                    int width, bool vec, UndoChain chain, float* __restrict__ out_read,
                    uint32_t* device_status) {
  constexpr int E = Unit<T>::kElems;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (row >= rows) return;
  const int dim = bank.dim;
  const int64_t part = partition_of(bank, row, rows_per_bank, nullptr);
  uint64_t row_ptr = 0;
  float weight = 0.f;
  if (lane < width) {
    const int64_t at = row * width + lane;
    const int64_t s = i64 ? static_cast<const int64_t*>(index)[at]
                          : static_cast<int64_t>(static_cast<const int32_t*>(index)[at]);
    if (s < 0 || s >= bank.slots) {
      if (device_status != nullptr) atomicOr(device_status, GLSDM_DEV_ADDRESS_OUT_OF_RANGE);
    } else {
      weight = weights[at];
      const int64_t flat = part * bank.slots + s;
      const T* src = version_row<T>(chain, flat, dim, static_cast<const T*>(bank.values) + flat * dim);
      row_ptr = reinterpret_cast<uint64_t>(src);
    }
  }
  float* __restrict__ out_row = out_read + row * dim;
  if (vec) {
    const int units = dim / E;
    const int passes = units <= 32 ? 1 : units / 32;
    const int here = units < 32 ? units : 32;
    for (int ub = 0; ub < passes; ++ub) {
      float acc[E];
      gather_units_at<T>(row_ptr, weight, width, lane, units, ub, acc);
      if (lane < here) {
        float4* dst = reinterpret_cast<float4*>(out_row + (ub * 32 + lane) * E);
        dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        if constexpr (E == 8) dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
      }
    }
  } else {
    for (int d0 = 0; d0 < dim; d0 += 32) {
      const int d = d0 + lane;
      float acc = 0.f;
      for (int k = 0; k < width; ++k) {
        const uint64_t p = shfl_u64(row_ptr, k);
        const float w = __shfl_sync(kFullMask, weight, k);
        if (p != 0 && d < dim) acc = fmaf(w, Unit<T>::scalar(reinterpret_cast<const T*>(p) + d), acc);
      }
      if (d < dim) out_row[d] = acc;
    }
  }
}

}  // namespace
}  // namespace glsdm

using namespace glsdm;

extern "C" int glsdm_overlay_read(const glsdm_bank* bank, const void* index, int index_i64,
                                  const float* weights, int64_t rows, int64_t rows_per_bank,
                                  int32_t width, int32_t n_logs, const int64_t* const* log_addresses,
                                  const void* const* log_rows, const int64_t* log_entries,
                                  float* out_read, uint32_t* device_status, glsdm_stream_t stream) {
  if (rows == 0) return GLSDM_OK;
  if (bank == nullptr || bank->values == nullptr) return GLSDM_ERR_ARGUMENT;
  if (bank->dtype != GLSDM_F32 && bank->dtype != GLSDM_BF16) return GLSDM_ERR_ARGUMENT;
  if (index == nullptr || weights == nullptr || out_read == nullptr || rows < 0 || rows_per_bank < 1)
    return GLSDM_ERR_ARGUMENT;
  if (width < 1) return GLSDM_ERR_ARGUMENT;
  if (bank->banks < 1 || (bank->banks > 1 && rows > bank->banks * rows_per_bank)) return GLSDM_ERR_ARGUMENT;
  if (width > 32) return GLSDM_ERR_UNSUPPORTED;
  if (bank->slot_lo != 0 || bank->slot_hi != bank->slots) return GLSDM_ERR_UNSUPPORTED;
  UndoChain chain;
  bool rows_aligned = true;
  if (int s = make_chain(n_logs, log_addresses, log_rows, log_entries, &chain, &rows_aligned)) return s;
  const BankView v = make_view(*bank);
  const int grid = blocks_for(rows, kWarpsPerBlock);
  const bool out_aligned = (reinterpret_cast<uintptr_t>(out_read) & 15u) == 0;
  if (bank->dtype == GLSDM_F32) {
    const bool vec = vector_rows<float>(v.dim, v.values) && out_aligned && rows_aligned;
    overlay_read_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        v, index, index_i64, weights, rows, rows_per_bank, width, vec, chain, out_read, device_status);
  } else {
    const bool vec = vector_rows<__nv_bfloat16>(v.dim, v.values) && out_aligned && rows_aligned;
    overlay_read_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        v, index, index_i64, weights, rows, rows_per_bank, width, vec, chain, out_read, device_status);
  }
  GLSDM_CUDA_OK(cudaGetLastError(), "overlay_read launch");
  count_launches(1);
  return GLSDM_OK;
}
