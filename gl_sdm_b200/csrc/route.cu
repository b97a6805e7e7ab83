// Routing and snapshot-read kernels (one warp per (request, token, head) row) and their
// C entry points: glsdm_pk_select, glsdm_snapshot_read, glsdm_pk_select_read,
// glsdm_pk_propose.
#include "overlay.cuh"
#include "route.cuh"

// Resident blocks per SM the selection kernels are compiled for: with 4 (a 64-register budget)
// the fused route + read measured 336 us at 32,768 rows of 2 x 4096 scores against 355 us
// without a bound, 353 us with 6 and 400 us with 8 (spills).
#ifndef GLSDM_SELECT_MIN_BLOCKS
#define GLSDM_SELECT_MIN_BLOCKS 4
#endif

namespace glsdm {
namespace {

__device__ __forceinline__ void store_routes(void* out_index, bool i64, float* out_weights,
                                             int64_t row, int kout, int lane, uint32_t slot,
                                             float weight) {
  if (lane >= kout) return;
  const int64_t at = row * kout + lane;
  if (out_index != nullptr) {
    if (i64) {
      static_cast<int64_t*>(out_index)[at] = static_cast<int64_t>(slot);
    } else {
      static_cast<int32_t*>(out_index)[at] = static_cast<int32_t>(slot);
    }
  }
  if (out_weights != nullptr) out_weights[at] = weight;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32, GLSDM_SELECT_MIN_BLOCKS)
pk_select_kernel(const float* __restrict__ scores, int64_t rows, int half, int kf, int kout,
                 void* out_index, int i64, float* out_weights) {
  __shared__ uint64_t stage[kWarpsPerBlock][kStageSlots];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (row >= rows) return;
  uint32_t slot;
  float weight;
  pk_route_row(scores + row * 2 * half, half, kf, kout, stage[warp], lane, slot, weight);
  store_routes(out_index, i64 != 0, out_weights, row, kout, lane, slot, weight);
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, GLSDM_SELECT_MIN_BLOCKS)
pk_select_read_kernel(BankView bank, const float* __restrict__ scores, int64_t rows,
                      int64_t rows_per_bank, int half, int kf, int kout, bool vec,
                      float* __restrict__ out_read, void* out_index, int i64,
                      float* out_weights) {
  __shared__ uint64_t stage[kWarpsPerBlock][kStageSlots];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (row >= rows) return;
  uint32_t slot;
  float weight;
  pk_route_row(scores + row * 2 * half, half, kf, kout, stage[warp], lane, slot, weight);
  store_routes(out_index, i64 != 0, out_weights, row, kout, lane, slot, weight);
  const int64_t part = partition_of(bank, row, rows_per_bank, nullptr);
  const T* base = static_cast<const T*>(bank.values) + part * bank.part_stride_rows * bank.dim;
  read_row<T>(base, bank, slot, weight, kout, lane, vec, out_read + row * bank.dim);
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
snapshot_read_kernel(BankView bank, const void* __restrict__ index, int i64,
                     const float* __restrict__ weights, const int64_t* __restrict__ requests,
                     int64_t rows, int64_t rows_per_bank, int width, bool vec,
                     float* __restrict__ out_read, uint32_t* device_status, int64_t block_rows,
                     int64_t block_stride) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (row >= rows) return;
  uint32_t slot = 0;
  float weight = 0.f;
  if (lane < width) {
    // Routes may arrive as per-rank blocks of an all-gather: block b holds block_rows rows
    // starting block_stride elements after block b-1. A plain [rows, width] array is one block.
    const int64_t at = (row / block_rows) * block_stride + (row % block_rows) * width + lane;
    const int64_t s = i64 ? static_cast<const int64_t*>(index)[at]
                          : static_cast<int64_t>(static_cast<const int32_t*>(index)[at]);
    weight = weights[at];
    if (s < 0 || s >= bank.slots) {
      if (device_status != nullptr) atomicOr(device_status, GLSDM_DEV_ADDRESS_OUT_OF_RANGE);
      weight = 0.f;
    } else {
      slot = static_cast<uint32_t>(s);
    }
  }
  int64_t part = partition_of(bank, row, rows_per_bank, requests);
  if (part < 0 || part >= bank.banks * bank.heads) {
    if (lane == 0 && device_status != nullptr) atomicOr(device_status, GLSDM_DEV_ADDRESS_OUT_OF_RANGE);
    part = row % bank.heads;
    weight = 0.f;
  }
  const T* base = static_cast<const T*>(bank.values) + part * bank.part_stride_rows * bank.dim;
  read_row<T>(base, bank, slot, weight, width, lane, vec, out_read + row * bank.dim);
}

// Fused write proposal for one row: route, prediction read, then one delta row per route
//   delta_k = mass * ((decay - 1) * row_k + w_k * beta * (target - decay * prediction))
// (reference gl_sdm/runtime/dense.py:11-14) plus the flat address and canonical sort key
// (reference gl_sdm/layers/global_layer.py:45,52-53). The selected rows are read twice; the
// second read of the same 16-byte units by the same lanes is served from L1/L2.
template <typename T, typename TT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
pk_propose_kernel(BankView bank, const float* __restrict__ scores, const TT* __restrict__ target,
                  const float* __restrict__ beta, const float* __restrict__ log_decay,
                  const float* __restrict__ mass, int64_t rows, int64_t rows_per_bank,
                  int64_t tokens, int half, int kf, int kout, bool vec, int64_t chunk_offset,
                  int64_t key_stride, int num_layers, int layer_index,
                  int64_t* __restrict__ out_addresses, float* __restrict__ out_deltas,
                  int64_t* __restrict__ out_keys) {
  __shared__ uint64_t stage[kWarpsPerBlock][kStageSlots];
  constexpr int E = Unit<T>::kElems;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (row >= rows) return;
  uint32_t slot;
  float weight;
  pk_route_row(scores + row * 2 * half, half, kf, kout, stage[warp], lane, slot, weight);

  const int dim = bank.dim;
  const int64_t part = partition_of(bank, row, rows_per_bank, nullptr);
  const T* base = static_cast<const T*>(bank.values) + part * bank.part_stride_rows * dim;
  const int64_t token = row / bank.heads;
  const float decay = expf(log_decay[row]);
  const float gate = beta[row];
  const float m = mass != nullptr ? mass[token] : 1.0f;
  const float decay_m1 = __fadd_rn(decay, -1.0f);
  float* __restrict__ drows = out_deltas + row * kout * dim;
  const TT* __restrict__ trow = target + row * dim;

  if (lane < kout) {
    const int64_t address = part * bank.slots + slot;
    const int64_t position = chunk_offset + token % tokens;
    out_addresses[row * kout + lane] = address;
    out_keys[row * kout + lane] = address * key_stride + position * num_layers + layer_index;
  }

  if (vec) {
    const int units = dim / E;
    const int passes = units <= 32 ? 1 : units / 32;
    const int here = units < 32 ? units : 32;
    const int groups = 32 / here;
    const int g = lane / here;
    const uint4* __restrict__ rows4 = reinterpret_cast<const uint4*>(base);
    for (int ub = 0; ub < passes; ++ub) {
      float pred[E];
      gather_units<T>(base, bank, slot, weight, kout, lane, units, ub, pred);
      const int u = ub * 32 + (lane % here);
      float err[E];
#pragma unroll
      for (int i = 0; i < E; ++i) {
        const float t = Unit<TT>::scalar(trow + u * E + i);
        err[i] = __fmul_rn(gate, __fadd_rn(t, -__fmul_rn(decay, pred[i])));
      }
      for (int k0 = 0; k0 < kout; k0 += groups) {
        const int k = k0 + g;
        const uint32_t a = __shfl_sync(kFullMask, slot, k & 31);
        const float w = __shfl_sync(kFullMask, weight, k & 31);
        if (k < kout) {
          float v[E];
          const int64_t local = static_cast<int64_t>(a) - bank.slot_lo;
          const bool owned = local >= 0 && local < bank.part_stride_rows;
          uint4 raw = make_uint4(0u, 0u, 0u, 0u);
          if (owned) raw = __ldg(rows4 + local * units + u);
          Unit<T>::decode(raw, v);
          float d[E];
#pragma unroll
          for (int i = 0; i < E; ++i)
            d[i] = __fmul_rn(m, __fadd_rn(__fmul_rn(decay_m1, v[i]), __fmul_rn(w, err[i])));
          float4* dst = reinterpret_cast<float4*>(drows + static_cast<int64_t>(k) * dim + u * E);
          dst[0] = make_float4(d[0], d[1], d[2], d[3]);
          if constexpr (E == 8) dst[1] = make_float4(d[4], d[5], d[6], d[7]);
        }
      }
    }
  } else {
    for (int d0 = 0; d0 < dim; d0 += 32) {
      const int d = d0 + lane;
      float pred = 0.f;
      for (int k = 0; k < kout; ++k) {
        const uint32_t a = __shfl_sync(kFullMask, slot, k);
        const float w = __shfl_sync(kFullMask, weight, k);
        const int64_t local = static_cast<int64_t>(a) - bank.slot_lo;
        if (d < dim && local >= 0 && local < bank.part_stride_rows)
          pred = fmaf(w, Unit<T>::scalar(base + local * dim + d), pred);
      }
      const float t = d < dim ? Unit<TT>::scalar(trow + d) : 0.f;
      const float err = __fmul_rn(gate, __fadd_rn(t, -__fmul_rn(decay, pred)));
      for (int k = 0; k < kout; ++k) {
        const uint32_t a = __shfl_sync(kFullMask, slot, k);
        const float w = __shfl_sync(kFullMask, weight, k);
        const int64_t local = static_cast<int64_t>(a) - bank.slot_lo;
        if (d < dim) {
          const float v = (local >= 0 && local < bank.part_stride_rows)
                              ? Unit<T>::scalar(base + local * dim + d) : 0.f;
          drows[static_cast<int64_t>(k) * dim + d] =
              __fmul_rn(m, __fadd_rn(__fmul_rn(decay_m1, v), __fmul_rn(w, err)));
        }
      }
    }
  }
}

// Row copy out[n] = flat[address[n]] (reference gl_sdm/memory/routing.py:37-42 and
// gl_sdm/memory/backends/primitives.py:14-20). `unit` bytes move per thread.
template <typename U>
__global__ void gather_rows_kernel(const U* __restrict__ flat, const int64_t* __restrict__ address,
                                   int64_t count, int64_t bank_rows, int units,
                                   U* __restrict__ out, uint32_t* device_status) {
  const int64_t total = count * units;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t n = i / units;
    const int u = static_cast<int>(i - n * units);
    const int64_t a = address[n];
    if (a < 0 || a >= bank_rows) {
      if (device_status != nullptr) atomicOr(device_status, GLSDM_DEV_ADDRESS_OUT_OF_RANGE);
      continue;
    }
    out[i] = flat[a * units + u];
  }
}

// Token-clock write proposal (reference gl_sdm/memory/transactions.py:38-59), one warp per
// (active request, head): rows decay first, the retrieval is the weighted sum of the
// decayed rows, and each route receives (decayed - row) + w * beta * (target - retrieved),
// scaled by the request's mass. Operation order follows the reference expression.
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
token_propose_kernel(const T* __restrict__ values, int64_t banks, int heads, int64_t slots, int dim,
                     const int64_t* __restrict__ requests, const void* __restrict__ index, int i64,
                     const float* __restrict__ weights, const float* __restrict__ target,
                     const float* __restrict__ beta, const float* __restrict__ log_decay,
                     const float* __restrict__ mass, int64_t rows, int width,
                     int64_t* __restrict__ out_addresses, float* __restrict__ out_deltas,
                     uint32_t* device_status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (row >= rows) return;
  const int64_t active = row / heads;
  const int head = static_cast<int>(row % heads);
  const int64_t request = requests[active];
  const bool request_ok = request >= 0 && request < banks;
  const int64_t part = (request_ok ? request : 0) * heads + head;
  const float decay = expf(log_decay[row]);
  const float gate = beta[row];
  const float m = mass[active];
  for (int k = lane; k < width; k += 32) {
    const int64_t at = row * width + k;
    const int64_t s = i64 ? static_cast<const int64_t*>(index)[at]
                          : static_cast<int64_t>(static_cast<const int32_t*>(index)[at]);
    out_addresses[at] = part * slots + s;
    if ((s < 0 || s >= slots || !request_ok) && device_status != nullptr)
      atomicOr(device_status, GLSDM_DEV_ADDRESS_OUT_OF_RANGE);
  }
  for (int d = lane; d < dim; d += 32) {
    float retrieved = 0.f;
    for (int k = 0; k < width; ++k) {
      const int64_t at = row * width + k;
      const int64_t s = i64 ? static_cast<const int64_t*>(index)[at]
                            : static_cast<int64_t>(static_cast<const int32_t*>(index)[at]);
      const bool ok = request_ok && s >= 0 && s < slots;
      const float v = ok ? Unit<T>::scalar(values + (part * slots + s) * dim + d) : 0.f;
      retrieved = __fadd_rn(retrieved, __fmul_rn(__fmul_rn(v, decay), weights[at]));
    }
    const float err = __fmul_rn(gate, __fadd_rn(target[row * dim + d], -retrieved));
    for (int k = 0; k < width; ++k) {
      const int64_t at = row * width + k;
      const int64_t s = i64 ? static_cast<const int64_t*>(index)[at]
                            : static_cast<int64_t>(static_cast<const int32_t*>(index)[at]);
      const bool ok = request_ok && s >= 0 && s < slots;
      const float v = ok ? Unit<T>::scalar(values + (part * slots + s) * dim + d) : 0.f;
      const float moved = __fadd_rn(__fmul_rn(v, decay), -v);
      out_deltas[at * dim + d] = __fmul_rn(__fadd_rn(moved, __fmul_rn(weights[at], err)), m);
    }
  }
}

// Product-key routing from per-factor candidate lists (the output of two glsdm_score_topk
// calls, one per sub-key codebook): combine, select, canonical order, softmax.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
pk_combine_kernel(const float* __restrict__ left_score, const int32_t* __restrict__ left_index,
                  const float* __restrict__ right_score, const int32_t* __restrict__ right_index,
                  int64_t rows, int half, int kf, int kout, void* out_index, int i64, float* out_weights) {
  __shared__ uint64_t stage[kWarpsPerBlock][kStageSlots];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (row >= rows) return;
  uint64_t left = 0, right = 0;
  if (lane < kf) {
    const int64_t at = row * kf + lane;
    left = pack_key(orderable_bits(left_score[at]), static_cast<uint32_t>(left_index[at]));
    right = pack_key(orderable_bits(right_score[at]), static_cast<uint32_t>(right_index[at]));
  }
  uint32_t slot;
  float weight;
  pk_combine_lists(left, right, half, kf, kout, stage[warp], lane, slot, weight);
  store_routes(out_index, i64 != 0, out_weights, row, kout, lane, slot, weight);
}

// Softmax backward of one row's routes, scattered to the factor scores: gs_k = w_k * (gw_k -
// sum_j w_j gw_j) is added at left_k and at half + right_k. Routes of the row that share a factor
// index are summed in route order by one lane, so the result does not depend on scheduling; the
// row of 2 * half gradients is written whole (zeros elsewhere).
__device__ __forceinline__ void scatter_score_gradients(float gw, float w, int64_t slot, int width, int half,
                                                        float* __restrict__ srow, int lane) {
  const float mean = warp_sum(lane < width ? w * gw : 0.f);
  const float gs = lane < width ? w * (gw - mean) : 0.f;
  for (int c = lane; c < 2 * half; c += 32) srow[c] = 0.f;
  __syncwarp();
  const int left = static_cast<int>(slot / half), right = static_cast<int>(slot % half);
  for (int f = 0; f < 2; ++f) {
    const int mine = lane < width ? (f == 0 ? left : right) : -1 - lane;   // unused lanes match nobody
    const unsigned peers = __match_any_sync(kFullMask, mine);
    // every lane walks all routes (the shuffle needs the whole warp) and keeps its peers' terms
    float sum = 0.f;
    for (int k = 0; k < width; ++k) {
      const float term = __shfl_sync(kFullMask, gs, k);
      if ((peers >> k) & 1u) sum += term;
    }
    if (lane < width && (peers & ((1u << lane) - 1u)) == 0) srow[f * half + mine] = sum;
  }
}

// Backward of the routed read (reference: autograd through gl_sdm/memory/routing.py:19-28;
// native counterparts gl_sdm/memory/backends/token.py:69-82,134-144). One warp per row.
//   gw_k   = <g, row_k>                       (gradient of the softmax weights)
//   gs_k   = w_k * (gw_k - sum_j w_j gw_j)    (softmax backward = gradient of the selected sums)
//   grad_scores[row, left_k] += gs_k,  grad_scores[row, half + right_k] += gs_k
//   grad_rows[row*K + k, :] = w_k * g         (compact bank gradient: one row per route)
// Routes of one row that share a factor index are summed in route order by one lane, so the
// result does not depend on scheduling. grad_scores is written whole (zeros elsewhere).
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
read_backward_kernel(BankView bank, const float* __restrict__ grad_out, const float* __restrict__ grad_weights,
                     const void* __restrict__ index, int i64, const float* __restrict__ weights, int64_t rows, int64_t rows_per_bank, int width, int half,
                     float* __restrict__ grad_scores, float* __restrict__ grad_rows,
                     int64_t* __restrict__ out_addresses, UndoChain chain) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (row >= rows) return;
  const int dim = bank.dim;
  const int64_t part = partition_of(bank, row, rows_per_bank, nullptr);
  const T* base = static_cast<const T*>(bank.values) + part * bank.part_stride_rows * dim;
  const float* __restrict__ g = grad_out + row * dim;
  int64_t slot = 0;
  float w = 0.f;
  uint64_t row_ptr = 0;   // the row as the version that was read held it
  if (lane < width) {
    const int64_t at = row * width + lane;
    slot = i64 ? static_cast<const int64_t*>(index)[at] : static_cast<int64_t>(static_cast<const int32_t*>(index)[at]);
    w = weights[at];
    const int64_t flat = part * bank.slots + slot;
    out_addresses[at] = flat;
    row_ptr = reinterpret_cast<uint64_t>(version_row<T>(chain, flat, dim, base + slot * dim));
  }
  float gw = 0.f;
  for (int k = 0; k < width; ++k) {
    const float wk = __shfl_sync(kFullMask, w, k);
    const T* vrow = reinterpret_cast<const T*>(shfl_u64(row_ptr, k));
    float* grow = grad_rows + (row * width + k) * dim;
    float partial = 0.f;
    for (int d = lane; d < dim; d += 32) {
      const float gd = g[d];
      partial = fmaf(gd, Unit<T>::scalar(vrow + d), partial);
      grow[d] = __fmul_rn(wk, gd);
    }
    const float total = warp_sum(partial);
    if (lane == k) gw = total;
  }
  // the weights are an output too (the write proposal uses them): add their own gradient
  if (grad_weights != nullptr && lane < width) gw += grad_weights[row * width + lane];
  scatter_score_gradients(gw, w, slot, width, half, grad_scores + row * 2 * half, lane);
}

// Backward of the fused write proposal (glsdm_pk_propose): reference autograd through
// gl_sdm/layers/global_layer.py:41-51 and gl_sdm/runtime/dense.py:11-14. One warp per row; G_k is
// the gradient arriving at delta row k.
//   delta_k = m * ((decay - 1) * row_k + w_k * err),  err = beta * (target - decay * pred),
//   pred = sum_j w_j row_j,  w = softmax of the selected sums
//   g_err    = m * sum_k w_k G_k            g_target = beta * g_err
//   g_beta   = <g_err, target - decay * pred>
//   g_pred   = -beta * decay * g_err
//   g_decay  = m * sum_k <G_k, row_k> - beta * <g_err, pred>;   g_log_decay = decay * g_decay
//   g_w_k    = m * <G_k, err> + <g_pred, row_k>     (then the softmax backward, scattered to the factors)
//   g_row_k  = m * (decay - 1) * G_k + w_k * g_pred (compact bank gradient, one row per route)
// The weights are recomputed from the scores and the routes the forward chose; the rows are
// those of the version the forward read (undo chain). Rows of up to 256 values.
template <typename T, typename TT, int kCols>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
pk_propose_backward_kernel(BankView bank, UndoChain chain, const float* __restrict__ scores,
                           const TT* __restrict__ target, const float* __restrict__ beta,
                           const float* __restrict__ log_decay, const float* __restrict__ mass,
                           const int64_t* __restrict__ addresses, const float* __restrict__ grad_deltas,
                           int64_t rows, int64_t rows_per_bank, int half, int width,
                           float* __restrict__ grad_scores, float* __restrict__ grad_target,
                           float* __restrict__ grad_beta, float* __restrict__ grad_log_decay,
                           float* __restrict__ grad_rows) {
  // kCols columns per lane: rows of at most 32 * kCols values (2, 4 or 8: up to 256)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (row >= rows) return;
  const int dim = bank.dim;
  const int64_t part = partition_of(bank, row, rows_per_bank, nullptr);
  const T* base = static_cast<const T*>(bank.values) + part * bank.part_stride_rows * dim;
  const float* __restrict__ srow = scores + row * 2 * half;
  int64_t slot = 0;
  float sum = -INFINITY;
  uint64_t row_ptr = 0;
  if (lane < width) {
    const int64_t flat = addresses[row * width + lane];
    slot = flat - part * bank.slots;
    if (slot < 0 || slot >= bank.slots) {
      slot = 0;                                  // not a route of this row's bank: weight 0, no access outside it
      row_ptr = reinterpret_cast<uint64_t>(base);
    } else {
      sum = __fadd_rn(srow[slot / half], srow[half + slot % half]);
      row_ptr = reinterpret_cast<uint64_t>(version_row<T>(chain, flat, dim, base + slot * dim));
    }
  }
  float top = sum;
  for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(kFullMask, top, o));
  const float e = lane < width ? expf(sum - top) : 0.f;
  const float w = e / warp_sum(e);

  const float decay = expf(log_decay[row]);
  const float b = beta[row];
  const float m = mass != nullptr ? mass[row / bank.heads] : 1.0f;
  float pred[kCols], resid[kCols], gerr[kCols];
#pragma unroll
  for (int c = 0; c < kCols; ++c) pred[c] = gerr[c] = 0.f;
  for (int k = 0; k < width; ++k) {
    const T* vrow = reinterpret_cast<const T*>(shfl_u64(row_ptr, k));
    const float wk = __shfl_sync(kFullMask, w, k);
#pragma unroll
    for (int c = 0; c < kCols; ++c) {
      const int d = c * 32 + lane;
      if (d < dim) pred[c] = fmaf(wk, Unit<T>::scalar(vrow + d), pred[c]);
    }
  }
  const TT* __restrict__ trow = target + row * dim;
#pragma unroll
  for (int c = 0; c < kCols; ++c) {
    const int d = c * 32 + lane;
    resid[c] = d < dim ? Unit<TT>::scalar(trow + d) - decay * pred[c] : 0.f;
  }
  const float* __restrict__ grow = grad_deltas + row * width * dim;
  float with_err = 0.f;      // lane k: <G_k, err>
  float with_rows = 0.f;     // sum_k <G_k, row_k>
  for (int k = 0; k < width; ++k) {
    const T* vrow = reinterpret_cast<const T*>(shfl_u64(row_ptr, k));
    const float wk = __shfl_sync(kFullMask, w, k);
    float p_err = 0.f, p_rows = 0.f;
#pragma unroll
    for (int c = 0; c < kCols; ++c) {
      const int d = c * 32 + lane;
      if (d < dim) {
        const float g = grow[k * dim + d];
        gerr[c] = fmaf(wk, g, gerr[c]);
        p_err = fmaf(g, b * resid[c], p_err);
        p_rows = fmaf(g, Unit<T>::scalar(vrow + d), p_rows);
      }
    }
    const float t_err = warp_sum(p_err);
    with_rows += p_rows;                 // this lane's columns; summed over the lanes once, below
    if (lane == k) with_err = t_err;
  }
  with_rows = warp_sum(with_rows);
  float p_beta = 0.f, p_pred = 0.f;
  float gpred[kCols];
  float* __restrict__ gt = grad_target + row * dim;
#pragma unroll
  for (int c = 0; c < kCols; ++c) {
    const int d = c * 32 + lane;
    gerr[c] *= m;
    gpred[c] = -b * decay * gerr[c];
    p_beta = fmaf(gerr[c], resid[c], p_beta);
    p_pred = fmaf(gerr[c], pred[c], p_pred);
    if (d < dim) gt[d] = b * gerr[c];
  }
  const float g_beta = warp_sum(p_beta);
  const float g_decay = m * with_rows - b * warp_sum(p_pred);
  if (lane == 0) {
    grad_beta[row] = g_beta;
    grad_log_decay[row] = g_decay * decay;
  }
  const float keep = m * (decay - 1.0f);
  float gw = 0.f;
  for (int k = 0; k < width; ++k) {
    const T* vrow = reinterpret_cast<const T*>(shfl_u64(row_ptr, k));
    const float wk = __shfl_sync(kFullMask, w, k);
    float* __restrict__ out = grad_rows + (row * width + k) * dim;
    float p = 0.f;
#pragma unroll
    for (int c = 0; c < kCols; ++c) {
      const int d = c * 32 + lane;
      if (d < dim) {
        p = fmaf(gpred[c], Unit<T>::scalar(vrow + d), p);
        out[d] = fmaf(keep, grow[k * dim + d], wk * gpred[c]);
      }
    }
    const float t = warp_sum(p);
    if (lane == k) gw = m * with_err + t;
  }
  scatter_score_gradients(gw, w, slot, width, half, grad_scores + row * 2 * half, lane);
}

int route_shape(int32_t half, int32_t width, int* kf, int* kout) {
  if (half < 1 || width < 1) return GLSDM_ERR_ARGUMENT;
  if (half > 65536) return GLSDM_ERR_UNSUPPORTED;
  const int f = width < half ? width : half;
  if (f > 32) return GLSDM_ERR_UNSUPPORTED;
  const int64_t cand = static_cast<int64_t>(f) * f;
  const int o = width < cand ? width : static_cast<int>(cand);
  if (o > 32) return GLSDM_ERR_UNSUPPORTED;
  *kf = f;
  *kout = o;
  return GLSDM_OK;
}

}  // namespace
}  // namespace glsdm

using namespace glsdm;

extern "C" int glsdm_pk_select(const float* scores, int64_t rows, int32_t half, int32_t width,
                               void* out_index, int index_i64, float* out_weights,
                               glsdm_stream_t stream) {
  if (rows == 0) return GLSDM_OK;   // nothing to do: pointers of empty arrays may be null
  int kf, kout;
  if (int s = route_shape(half, width, &kf, &kout)) return s;
  if (rows < 0 || scores == nullptr) return GLSDM_ERR_ARGUMENT;
  if ((half & 3) == 0 && (reinterpret_cast<uintptr_t>(scores) & 15u)) return GLSDM_ERR_ARGUMENT;
  if (rows == 0) return GLSDM_OK;
  pk_select_kernel<<<blocks_for(rows, kWarpsPerBlock), kWarpsPerBlock * 32, 0, stream>>>(
      scores, rows, half, kf, kout, out_index, index_i64, out_weights);
  GLSDM_CUDA_OK(cudaGetLastError(), "pk_select launch");
  count_launches(1);
  return GLSDM_OK;
}

extern "C" int glsdm_snapshot_read(const glsdm_bank* bank, const void* index, int index_i64,
                                   const float* weights, const int64_t* requests, int64_t rows,
                                   int64_t rows_per_bank, int32_t width, float* out_read,
                                   uint32_t* device_status, glsdm_stream_t stream) {
  if (rows == 0) return GLSDM_OK;   // nothing to do: pointers of empty arrays may be null
  if (int s = check_bank(bank)) return s;
  if (index == nullptr || weights == nullptr || out_read == nullptr || rows < 0) return GLSDM_ERR_ARGUMENT;
  if (width < 1 || rows_per_bank < 1) return GLSDM_ERR_ARGUMENT;
  if (requests == nullptr) {
    if (int s = check_rows(bank, rows, rows_per_bank)) return s;
  }
  if (width > 32) return GLSDM_ERR_UNSUPPORTED;
  if (rows == 0) return GLSDM_OK;
  const BankView v = make_view(*bank);
  const int grid = blocks_for(rows, kWarpsPerBlock);
  if (bank->dtype == GLSDM_F32) {
    const bool vec = vector_rows<float>(v.dim, v.values) && (reinterpret_cast<uintptr_t>(out_read) & 15u) == 0;
    snapshot_read_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        v, index, index_i64, weights, requests, rows, rows_per_bank, width, vec, out_read, device_status, rows, 0);
  } else {
    const bool vec = vector_rows<__nv_bfloat16>(v.dim, v.values) && (reinterpret_cast<uintptr_t>(out_read) & 15u) == 0;
    snapshot_read_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        v, index, index_i64, weights, requests, rows, rows_per_bank, width, vec, out_read, device_status, rows, 0);
  }
  GLSDM_CUDA_OK(cudaGetLastError(), "snapshot_read launch");
  count_launches(1);
  return GLSDM_OK;
}

extern "C" int glsdm_shard_read(const glsdm_bank* bank, const int32_t* index, const float* weights,
                                int64_t rows, int64_t block_rows, int64_t block_stride, int32_t width,
                                float* out_partial, uint32_t* device_status, glsdm_stream_t stream) {
  if (rows == 0) return GLSDM_OK;   // nothing to do: pointers of empty arrays may be null
  if (int s = check_bank(bank)) return s;
  if (index == nullptr || weights == nullptr || out_partial == nullptr || rows < 0) return GLSDM_ERR_ARGUMENT;
  if (width < 1 || block_rows < 1 || block_stride < 0) return GLSDM_ERR_ARGUMENT;
  if (width > 32 || bank->banks != 1) return GLSDM_ERR_UNSUPPORTED;
  if (rows == 0) return GLSDM_OK;
  const BankView v = make_view(*bank);
  const int grid = blocks_for(rows, kWarpsPerBlock);
  if (bank->dtype == GLSDM_F32) {
    const bool vec = vector_rows<float>(v.dim, v.values) && (reinterpret_cast<uintptr_t>(out_partial) & 15u) == 0;
    snapshot_read_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        v, index, 0, weights, nullptr, rows, rows, width, vec, out_partial, device_status, block_rows, block_stride);
  } else {
    const bool vec = vector_rows<__nv_bfloat16>(v.dim, v.values) && (reinterpret_cast<uintptr_t>(out_partial) & 15u) == 0;
    snapshot_read_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        v, index, 0, weights, nullptr, rows, rows, width, vec, out_partial, device_status, block_rows, block_stride);
  }
  GLSDM_CUDA_OK(cudaGetLastError(), "shard_read launch");
  count_launches(1);
  return GLSDM_OK;
}

extern "C" int glsdm_pk_select_read(const glsdm_bank* bank, const float* scores, int64_t rows,
                                    int64_t rows_per_bank, int32_t half, int32_t width,
                                    float* out_read, void* out_index, int index_i64,
                                    float* out_weights, uint32_t* device_status,
                                    glsdm_stream_t stream) {
  if (rows == 0) return GLSDM_OK;   // nothing to do: pointers of empty arrays may be null
  (void)device_status;
  if (int s = check_bank(bank)) return s;
  int kf, kout;
  if (int s = route_shape(half, width, &kf, &kout)) return s;
  if (scores == nullptr || out_read == nullptr || rows < 0 || rows_per_bank < 1) return GLSDM_ERR_ARGUMENT;
  if (int s = check_rows(bank, rows, rows_per_bank)) return s;
  if (static_cast<int64_t>(half) * half != bank->slots) return GLSDM_ERR_ARGUMENT;
  if ((half & 3) == 0 && (reinterpret_cast<uintptr_t>(scores) & 15u)) return GLSDM_ERR_ARGUMENT;
  if (rows == 0) return GLSDM_OK;
  const BankView v = make_view(*bank);
  const int grid = blocks_for(rows, kWarpsPerBlock);
  if (bank->dtype == GLSDM_F32) {
    const bool vec = vector_rows<float>(v.dim, v.values) && (reinterpret_cast<uintptr_t>(out_read) & 15u) == 0;
    pk_select_read_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        v, scores, rows, rows_per_bank, half, kf, kout, vec, out_read, out_index, index_i64, out_weights);
  } else {
    const bool vec = vector_rows<__nv_bfloat16>(v.dim, v.values) && (reinterpret_cast<uintptr_t>(out_read) & 15u) == 0;
    pk_select_read_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        v, scores, rows, rows_per_bank, half, kf, kout, vec, out_read, out_index, index_i64, out_weights);
  }
  GLSDM_CUDA_OK(cudaGetLastError(), "pk_select_read launch");
  count_launches(1);
  return GLSDM_OK;
}

template <typename T, typename TT>
static void launch_propose(const BankView& v, const float* scores, const void* target,
                           const float* beta, const float* log_decay, const float* mass,
                           int64_t rows, int64_t rows_per_bank, int64_t tokens, int half, int kf,
                           int kout, int64_t chunk_offset, int64_t chunk_size, int num_layers,
                           int layer_index, int64_t* out_addresses, float* out_deltas,
                           int64_t* out_keys, glsdm_stream_t stream) {
  const bool vec = vector_rows<T>(v.dim, v.values) &&
                   (reinterpret_cast<uintptr_t>(out_deltas) & 15u) == 0;
  pk_propose_kernel<T, TT><<<blocks_for(rows, kWarpsPerBlock), kWarpsPerBlock * 32, 0, stream>>>(
      v, scores, static_cast<const TT*>(target), beta, log_decay, mass, rows, rows_per_bank, tokens,
      half, kf, kout, vec, chunk_offset, chunk_size * num_layers, num_layers, layer_index,
      out_addresses, out_deltas, out_keys);
}

extern "C" int glsdm_pk_propose(const glsdm_bank* bank, const float* scores, const void* target,
                                int target_dtype, const float* beta, const float* log_decay,
                                const float* mass, int64_t rows, int64_t rows_per_bank,
                                int64_t tokens, int32_t half, int32_t width, int64_t chunk_offset,
                                int64_t chunk_size, int32_t num_layers, int32_t layer_index,
                                int64_t* out_addresses, float* out_deltas, int64_t* out_keys,
                                uint32_t* device_status, glsdm_stream_t stream) {
  if (rows == 0) return GLSDM_OK;   // nothing to do: pointers of empty arrays may be null
  (void)device_status;
  if (int s = check_bank(bank)) return s;
  int kf, kout;
  if (int s = route_shape(half, width, &kf, &kout)) return s;
  if (scores == nullptr || target == nullptr || beta == nullptr || log_decay == nullptr ||
      out_addresses == nullptr || out_deltas == nullptr || out_keys == nullptr)
    return GLSDM_ERR_ARGUMENT;
  if (rows < 0 || rows_per_bank < 1 || tokens < 1 || chunk_size < 1 || num_layers < 1 ||
      layer_index < 0 || layer_index >= num_layers || chunk_offset < 0)
    return GLSDM_ERR_ARGUMENT;
  if (int s = check_rows(bank, rows, rows_per_bank)) return s;
  if (static_cast<int64_t>(half) * half != bank->slots) return GLSDM_ERR_ARGUMENT;
  if (bank->slot_lo != 0 || bank->slot_hi != bank->slots) return GLSDM_ERR_UNSUPPORTED;
  if (target_dtype != GLSDM_F32 && target_dtype != GLSDM_BF16) return GLSDM_ERR_ARGUMENT;
  if ((half & 3) == 0 && (reinterpret_cast<uintptr_t>(scores) & 15u)) return GLSDM_ERR_ARGUMENT;
  if (rows == 0) return GLSDM_OK;
  const BankView v = make_view(*bank);
#define GLSDM_PROPOSE(T, TT)                                                                   \
  launch_propose<T, TT>(v, scores, target, beta, log_decay, mass, rows, rows_per_bank, tokens, \
                        half, kf, kout, chunk_offset, chunk_size, num_layers, layer_index,     \
                        out_addresses, out_deltas, out_keys, stream)
  if (bank->dtype == GLSDM_F32) {
    if (target_dtype == GLSDM_F32) GLSDM_PROPOSE(float, float);
    else GLSDM_PROPOSE(float, __nv_bfloat16);
  } else {
    if (target_dtype == GLSDM_F32) GLSDM_PROPOSE(__nv_bfloat16, float);
    else GLSDM_PROPOSE(__nv_bfloat16, __nv_bfloat16);
  }
#undef GLSDM_PROPOSE
  GLSDM_CUDA_OK(cudaGetLastError(), "pk_propose launch");
  count_launches(1);
  return GLSDM_OK;
}

extern "C" int glsdm_pk_propose_backward(const glsdm_bank* bank, const float* scores, const void* target,
                                         int target_dtype, const float* beta, const float* log_decay,
                                         const float* mass, const int64_t* addresses, const float* grad_deltas,
                                         int64_t rows, int64_t rows_per_bank, int32_t half, int32_t width,
                                         int32_t n_logs, const int64_t* const* log_addresses,
                                         const void* const* log_rows, const int64_t* log_entries,
                                         float* grad_scores, float* grad_target, float* grad_beta,
                                         float* grad_log_decay, float* grad_rows, glsdm_stream_t stream) {
  if (rows == 0) return GLSDM_OK;   // nothing to do: pointers of empty arrays may be null
  if (int s = check_bank(bank)) return s;
  int kf, kout;
  if (int s = route_shape(half, width, &kf, &kout)) return s;
  if (scores == nullptr || target == nullptr || beta == nullptr || log_decay == nullptr || addresses == nullptr ||
      grad_deltas == nullptr || grad_scores == nullptr || grad_target == nullptr || grad_beta == nullptr ||
      grad_log_decay == nullptr || grad_rows == nullptr)
    return GLSDM_ERR_ARGUMENT;
  if (rows < 0 || rows_per_bank < 1) return GLSDM_ERR_ARGUMENT;
  if (int s = check_rows(bank, rows, rows_per_bank)) return s;
  if (static_cast<int64_t>(half) * half != bank->slots) return GLSDM_ERR_ARGUMENT;
  if (bank->slot_lo != 0 || bank->slot_hi != bank->slots) return GLSDM_ERR_UNSUPPORTED;
  if (bank->dim > 256) return GLSDM_ERR_UNSUPPORTED;
  if (target_dtype != GLSDM_F32 && target_dtype != GLSDM_BF16) return GLSDM_ERR_ARGUMENT;
  UndoChain chain;
  if (int s = make_chain(n_logs, log_addresses, log_rows, log_entries, &chain, nullptr)) return s;
  const BankView v = make_view(*bank);
  const int grid = blocks_for(rows, kWarpsPerBlock);
#define GLSDM_PROPOSE_BACKWARD_COLS(T, TT, COLS)                                                            \
  pk_propose_backward_kernel<T, TT, COLS><<<grid, kWarpsPerBlock * 32, 0, stream>>>(                        \
      v, chain, scores, static_cast<const TT*>(target), beta, log_decay, mass, addresses, grad_deltas, rows, \
      rows_per_bank, half, kout, grad_scores, grad_target, grad_beta, grad_log_decay, grad_rows)
#define GLSDM_PROPOSE_BACKWARD(T, TT)                                 \
  do {                                                                \
    if (v.dim <= 64) GLSDM_PROPOSE_BACKWARD_COLS(T, TT, 2);           \
    else if (v.dim <= 128) GLSDM_PROPOSE_BACKWARD_COLS(T, TT, 4);     \
    else GLSDM_PROPOSE_BACKWARD_COLS(T, TT, 8);                       \
  } while (0)
  if (bank->dtype == GLSDM_F32) {
    if (target_dtype == GLSDM_F32) GLSDM_PROPOSE_BACKWARD(float, float);
    else GLSDM_PROPOSE_BACKWARD(float, __nv_bfloat16);
  } else {
    if (target_dtype == GLSDM_F32) GLSDM_PROPOSE_BACKWARD(__nv_bfloat16, float);
    else GLSDM_PROPOSE_BACKWARD(__nv_bfloat16, __nv_bfloat16);
  }
#undef GLSDM_PROPOSE_BACKWARD
#undef GLSDM_PROPOSE_BACKWARD_COLS
  GLSDM_CUDA_OK(cudaGetLastError(), "pk_propose_backward launch");
  count_launches(1);
  return GLSDM_OK;
}

extern "C" int glsdm_gather_rows(const void* flat, int dtype, int64_t bank_rows, int32_t dim,
                                 const int64_t* addresses, int64_t count, void* out,
                                 uint32_t* device_status, glsdm_stream_t stream) {
  if (flat == nullptr || addresses == nullptr || out == nullptr) return GLSDM_ERR_ARGUMENT;
  if (bank_rows < 1 || dim < 1 || count < 0) return GLSDM_ERR_ARGUMENT;
  if (dtype != GLSDM_F32 && dtype != GLSDM_BF16) return GLSDM_ERR_ARGUMENT;
  if (count == 0) return GLSDM_OK;
  const int64_t row_bytes = static_cast<int64_t>(dim) * (dtype == GLSDM_F32 ? 4 : 2);
  const bool wide = row_bytes % 16 == 0 && ((reinterpret_cast<uintptr_t>(flat) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
  const int64_t unit = wide ? 16 : (dtype == GLSDM_F32 ? 4 : 2);
  const int units = static_cast<int>(row_bytes / unit);
  const int64_t total = count * units;
  const int grid = static_cast<int>(total / 256 + 1 < 148 * 32 ? total / 256 + 1 : 148 * 32);
  if (unit == 16)
    gather_rows_kernel<uint4><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(flat), addresses, count, bank_rows, units, static_cast<uint4*>(out), device_status);
  else if (unit == 4)
    gather_rows_kernel<uint32_t><<<grid, 256, 0, stream>>>(static_cast<const uint32_t*>(flat), addresses, count, bank_rows, units, static_cast<uint32_t*>(out), device_status);
  else
    gather_rows_kernel<uint16_t><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(flat), addresses, count, bank_rows, units, static_cast<uint16_t*>(out), device_status);
  GLSDM_CUDA_OK(cudaGetLastError(), "gather_rows launch");
  count_launches(1);
  return GLSDM_OK;
}

extern "C" int glsdm_token_propose(const glsdm_bank* bank, const int64_t* requests, const void* index,
                                   int index_i64, const float* weights, const float* target,
                                   const float* beta, const float* log_decay, const float* mass,
                                   int64_t rows, int32_t width, int64_t* out_addresses,
                                   float* out_deltas, uint32_t* device_status,
                                   glsdm_stream_t stream) {
  if (rows == 0) return GLSDM_OK;   // nothing to do: pointers of empty arrays may be null
  if (int s = check_bank(bank)) return s;
  if (requests == nullptr || index == nullptr || weights == nullptr || target == nullptr ||
      beta == nullptr || log_decay == nullptr || mass == nullptr || out_addresses == nullptr ||
      out_deltas == nullptr)
    return GLSDM_ERR_ARGUMENT;
  if (rows < 0 || width < 1) return GLSDM_ERR_ARGUMENT;
  if (bank->slot_lo != 0 || bank->slot_hi != bank->slots) return GLSDM_ERR_UNSUPPORTED;
  if (rows == 0) return GLSDM_OK;
  const int grid = blocks_for(rows, kWarpsPerBlock);
  if (bank->dtype == GLSDM_F32)
    token_propose_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        static_cast<const float*>(bank->values), bank->banks, bank->heads, bank->slots, bank->dim, requests,
        index, index_i64, weights, target, beta, log_decay, mass, rows, width, out_addresses, out_deltas, device_status);
  else
    token_propose_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(bank->values), bank->banks, bank->heads, bank->slots, bank->dim, requests,
        index, index_i64, weights, target, beta, log_decay, mass, rows, width, out_addresses, out_deltas, device_status);
  GLSDM_CUDA_OK(cudaGetLastError(), "token_propose launch");
  count_launches(1);
  return GLSDM_OK;
}

extern "C" int glsdm_pk_combine(const float* left_score, const int32_t* left_index, const float* right_score,
                                const int32_t* right_index, int64_t rows, int32_t half, int32_t width,
                                void* out_index, int index_i64, float* out_weights, glsdm_stream_t stream) {
  if (rows == 0) return GLSDM_OK;   // nothing to do: pointers of empty arrays may be null
  int kf, kout;
  if (int s = route_shape(half, width, &kf, &kout)) return s;
  if (left_score == nullptr || left_index == nullptr || right_score == nullptr || right_index == nullptr ||
      out_index == nullptr || out_weights == nullptr || rows < 0)
    return GLSDM_ERR_ARGUMENT;
  if (rows == 0) return GLSDM_OK;
  pk_combine_kernel<<<blocks_for(rows, kWarpsPerBlock), kWarpsPerBlock * 32, 0, stream>>>(
      left_score, left_index, right_score, right_index, rows, half, kf, kout, out_index, index_i64, out_weights);
  GLSDM_CUDA_OK(cudaGetLastError(), "pk_combine launch");
  count_launches(1);
  return GLSDM_OK;
}

extern "C" int glsdm_read_backward_version(const glsdm_bank* bank, const float* grad_out, const float* grad_weights,
                                           const void* index, int index_i64, const float* weights, int64_t rows,
                                           int64_t rows_per_bank, int32_t width, int32_t half, int32_t n_logs,
                                           const int64_t* const* log_addresses, const void* const* log_rows,
                                           const int64_t* log_entries, float* grad_scores, float* grad_rows,
                                           int64_t* out_addresses, glsdm_stream_t stream) {
  if (rows == 0) return GLSDM_OK;   // nothing to do: pointers of empty arrays may be null
  if (int s = check_bank(bank)) return s;
  if (grad_out == nullptr || index == nullptr || weights == nullptr || grad_scores == nullptr ||
      grad_rows == nullptr || out_addresses == nullptr)
    return GLSDM_ERR_ARGUMENT;
  if (rows < 0 || rows_per_bank < 1 || width < 1 || half < 1) return GLSDM_ERR_ARGUMENT;
  if (int s = check_rows(bank, rows, rows_per_bank)) return s;
  if (width > 32) return GLSDM_ERR_UNSUPPORTED;
  if (static_cast<int64_t>(half) * half != bank->slots) return GLSDM_ERR_ARGUMENT;
  if (bank->slot_lo != 0 || bank->slot_hi != bank->slots) return GLSDM_ERR_UNSUPPORTED;
  UndoChain chain;
  if (int s = make_chain(n_logs, log_addresses, log_rows, log_entries, &chain, nullptr)) return s;
  const BankView v = make_view(*bank);
  const int grid = blocks_for(rows, kWarpsPerBlock);
  if (bank->dtype == GLSDM_F32)
    read_backward_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        v, grad_out, grad_weights, index, index_i64, weights, rows, rows_per_bank, width, half, grad_scores, grad_rows,
        out_addresses, chain);
  else
    read_backward_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        v, grad_out, grad_weights, index, index_i64, weights, rows, rows_per_bank, width, half, grad_scores, grad_rows,
        out_addresses, chain);
  GLSDM_CUDA_OK(cudaGetLastError(), "read_backward launch");
  count_launches(1);
  return GLSDM_OK;
}

extern "C" int glsdm_read_backward(const glsdm_bank* bank, const float* grad_out, const float* grad_weights,
                                   const void* index, int index_i64,
                                   const float* weights, int64_t rows, int64_t rows_per_bank, int32_t width,
                                   int32_t half, float* grad_scores, float* grad_rows, int64_t* out_addresses,
                                   glsdm_stream_t stream) {
  return glsdm_read_backward_version(bank, grad_out, grad_weights, index, index_i64, weights, rows, rows_per_bank,
                                     width, half, 0, nullptr, nullptr, nullptr, grad_scores, grad_rows,
                                     out_addresses, stream);
}
