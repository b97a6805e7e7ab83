// Kernels of the slot-sharded bank: the write proposal is split between the rank that owns
// a token (routes, prediction error) and the rank that owns a slot (delta rows, commit).
//   token owner:  err = beta * (target - decay * prediction)            (write_error)
//   slot owner :  delta_k = mass * ((decay - 1) * row_k + w_k * err)     (shard_propose)
// which is gl_sdm/runtime/dense.py:11-14 with the two factors computed where their
// operands live; addresses and keys follow gl_sdm/layers/global_layer.py:45,52-53.
#include "route.cuh"

namespace glsdm {
namespace {

template <typename TT>
__global__ void write_error_kernel(const float* __restrict__ prediction, const TT* __restrict__ target,
                                   const float* __restrict__ beta, const float* __restrict__ log_decay,
                                   int64_t rows, int dim, float* __restrict__ err,
                                   float* __restrict__ decay_m1) {
  const int64_t total = rows * dim;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / dim;
    const float decay = expf(log_decay[row]);
    const float t = Unit<TT>::scalar(target + i);
    err[i] = __fmul_rn(beta[row], __fadd_rn(t, -__fmul_rn(decay, prediction[i])));
    if (i == row * dim) decay_m1[row] = __fadd_rn(decay, -1.0f);
  }
}

// counts[row] = number of this row's routes whose slot lies in [slot_lo, slot_hi).
__global__ void owned_count_kernel(const int32_t* __restrict__ index, int64_t rows, int width,
                                   int64_t block_rows, int64_t block_stride, int64_t slot_lo,
                                   int64_t slot_hi, uint32_t* __restrict__ counts) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const int64_t at = (row / block_rows) * block_stride + (row % block_rows) * width;
  uint32_t c = 0;
  for (int k = 0; k < width; ++k) {
    const int64_t s = index[at + k];
    c += (s >= slot_lo && s < slot_hi) ? 1u : 0u;
  }
  counts[row] = c;
}

// In-place exclusive scan of counts[rows] by one block; total written to counts[rows].
// 1024 counts per round, read and written coalesced: a shuffle scan inside each warp, one
// more over the 32 warp totals, and a running carry from round to round.
__global__ void __launch_bounds__(1024) offsets_scan_kernel(uint32_t* counts, int64_t rows) {
  __shared__ uint32_t warp_total[32];
  __shared__ uint32_t carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < rows; base += 1024) {
    const int64_t i = base + threadIdx.x;
    const uint32_t c = i < rows ? counts[i] : 0u;
    uint32_t incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t n = __shfl_up_sync(kFullMask, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) warp_total[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const uint32_t t = warp_total[lane];
      uint32_t run = t;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t n = __shfl_up_sync(kFullMask, run, o);
        if (lane >= o) run += n;
      }
      warp_total[lane] = run - t;          // exclusive offset of every warp within the round
    }
    __syncthreads();
    const uint32_t before = carry + warp_total[warp] + incl - c;
    if (i < rows) counts[i] = before;
    __syncthreads();
    if (threadIdx.x == 1023) carry = before + c;
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[rows] = carry;
}

// One warp per routing row: expand the owned routes into delta rows at the row's offset.
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
shard_propose_kernel(BankView bank, const int32_t* __restrict__ index, const float* __restrict__ weights,
                     const float* __restrict__ err, const float* __restrict__ decay_m1,
                     const float* __restrict__ mass, const uint32_t* __restrict__ offsets,
                     int64_t rows, int64_t block_rows, int64_t route_stride, int64_t error_stride,
                     int64_t tokens, int width, bool vec, int64_t chunk_offset,
                     int64_t key_stride, int num_layers, int layer_index,
                     int64_t* __restrict__ out_addresses, float* __restrict__ out_deltas,
                     int64_t* __restrict__ out_keys) {
  constexpr int E = Unit<T>::kElems;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (row >= rows) return;
  const int dim = bank.dim;
  int64_t slot = -1;
  float w = 0.f;
  const int64_t block = row / block_rows, inner = row % block_rows;
  if (lane < width) {
    slot = index[block * route_stride + inner * width + lane];
    w = weights[block * route_stride + inner * width + lane];
  }
  const bool owned = slot >= bank.slot_lo && slot < bank.slot_hi;
  const unsigned mask = __ballot_sync(kFullMask, owned);
  if (mask == 0) return;
  const int64_t head = row % bank.heads;
  const int64_t token = row / bank.heads;
  const int64_t base_entry = offsets[row];
  const int rank = __popc(mask & ((1u << lane) - 1u));
  if (owned) {
    const int64_t address = head * bank.slots + slot;  // one shared bank: partition = head
    const int64_t position = chunk_offset + token % tokens;
    // The address is the row of this rank's shard; the key keeps the bank-wide address so
    // the canonical (address, position, layer) order is that of the unsharded bank.
    out_addresses[base_entry + rank] = head * bank.part_stride_rows + (slot - bank.slot_lo);
    out_keys[base_entry + rank] = address * key_stride + position * num_layers + layer_index;
  }
  // error rows [block_rows, dim] then decay-1 [block_rows] per block, error_stride apart
  const float* __restrict__ eblock = err + block * error_stride;
  const float gate = decay_m1[block * error_stride + inner];
  const float m = mass != nullptr ? mass[token] : 1.0f;
  const T* part = static_cast<const T*>(bank.values) + head * bank.part_stride_rows * dim;
  const float* __restrict__ erow = eblock + inner * dim;
  int entry = 0;
  for (unsigned left = mask; left; left &= left - 1, ++entry) {
    const int k = __ffs(left) - 1;
    const int64_t s = __shfl_sync(kFullMask, slot, k);
    const float wk = __shfl_sync(kFullMask, w, k);
    const T* src = part + (s - bank.slot_lo) * dim;
    float* dst = out_deltas + (base_entry + entry) * dim;
    if (vec) {
      const int units = dim / E;
      for (int u = lane; u < units; u += 32) {
        float v[E];
        Unit<T>::decode(__ldg(reinterpret_cast<const uint4*>(src) + u), v);
        float d[E];
#pragma unroll
        for (int i = 0; i < E; i += 4) {
          const float4 e4 = __ldg(reinterpret_cast<const float4*>(erow + u * E + i));
          d[i] = __fmul_rn(m, __fadd_rn(__fmul_rn(gate, v[i]), __fmul_rn(wk, e4.x)));
          d[i + 1] = __fmul_rn(m, __fadd_rn(__fmul_rn(gate, v[i + 1]), __fmul_rn(wk, e4.y)));
          d[i + 2] = __fmul_rn(m, __fadd_rn(__fmul_rn(gate, v[i + 2]), __fmul_rn(wk, e4.z)));
          d[i + 3] = __fmul_rn(m, __fadd_rn(__fmul_rn(gate, v[i + 3]), __fmul_rn(wk, e4.w)));
        }
        float4* out4 = reinterpret_cast<float4*>(dst + u * E);
        out4[0] = make_float4(d[0], d[1], d[2], d[3]);
        if constexpr (E == 8) out4[1] = make_float4(d[4], d[5], d[6], d[7]);
      }
    } else {
      for (int c = lane; c < dim; c += 32)
        dst[c] = __fmul_rn(m, __fadd_rn(__fmul_rn(gate, Unit<T>::scalar(src + c)), __fmul_rn(wk, erow[c])));
    }
  }
}

}  // namespace
}  // namespace glsdm

using namespace glsdm;

extern "C" int glsdm_write_error(const float* prediction, const void* target, int target_dtype,
                                 const float* beta, const float* log_decay, int64_t rows, int32_t dim,
                                 float* out_error, float* out_decay_m1, glsdm_stream_t stream) {
  if (rows == 0) return GLSDM_OK;   // nothing to do: pointers of empty arrays may be null
  if (prediction == nullptr || target == nullptr || beta == nullptr || log_decay == nullptr ||
      out_error == nullptr || out_decay_m1 == nullptr)
    return GLSDM_ERR_ARGUMENT;
  if (rows < 0 || dim < 1) return GLSDM_ERR_ARGUMENT;
  if (target_dtype != GLSDM_F32 && target_dtype != GLSDM_BF16) return GLSDM_ERR_ARGUMENT;
  if (rows == 0) return GLSDM_OK;
  const int64_t total = rows * dim;
  const int grid = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  if (target_dtype == GLSDM_F32)
    write_error_kernel<float><<<grid, 256, 0, stream>>>(prediction, static_cast<const float*>(target), beta,
                                                        log_decay, rows, dim, out_error, out_decay_m1);
  else
    write_error_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        prediction, static_cast<const __nv_bfloat16*>(target), beta, log_decay, rows, dim, out_error, out_decay_m1);
  GLSDM_CUDA_OK(cudaGetLastError(), "write_error launch");
  count_launches(1);
  return GLSDM_OK;
}

extern "C" int glsdm_shard_offsets(const int32_t* index, int64_t rows, int64_t block_rows,
                                   int64_t block_stride, int32_t width, int64_t slot_lo,
                                   int64_t slot_hi, uint32_t* offsets, glsdm_stream_t stream) {
  if (index == nullptr || offsets == nullptr || rows < 0 || width < 1 || slot_lo > slot_hi ||
      block_rows < 1 || block_stride < 0)
    return GLSDM_ERR_ARGUMENT;
  if (rows * static_cast<int64_t>(width) > 0xfffffff0ll) return GLSDM_ERR_LIMIT;
  if (rows > 0) {
    owned_count_kernel<<<blocks_for(rows, 256), 256, 0, stream>>>(index, rows, width, block_rows, block_stride,
                                                                  slot_lo, slot_hi, offsets);
    GLSDM_CUDA_OK(cudaGetLastError(), "shard count launch");
  }
  offsets_scan_kernel<<<1, 1024, 0, stream>>>(offsets, rows);
  GLSDM_CUDA_OK(cudaGetLastError(), "shard scan launch");
  count_launches(2);
  return GLSDM_OK;
}

extern "C" int glsdm_shard_propose(const glsdm_bank* bank, const int32_t* index, const float* weights,
                                   const float* error, const float* decay_m1, const float* mass,
                                   const uint32_t* offsets, int64_t rows, int64_t block_rows,
                                   int64_t route_stride, int64_t error_stride, int64_t tokens,
                                   int32_t width, int64_t chunk_offset, int64_t chunk_size, int32_t num_layers,
                                   int32_t layer_index, int64_t* out_addresses, float* out_deltas,
                                   int64_t* out_keys, glsdm_stream_t stream) {
  if (rows == 0) return GLSDM_OK;   // nothing to do: pointers of empty arrays may be null
  if (int s = check_bank(bank)) return s;
  if (index == nullptr || weights == nullptr || error == nullptr || decay_m1 == nullptr ||
      offsets == nullptr || out_addresses == nullptr || out_deltas == nullptr || out_keys == nullptr)
    return GLSDM_ERR_ARGUMENT;
  if (rows < 0 || tokens < 1 || width < 1 || chunk_size < 1 || num_layers < 1 || layer_index < 0 ||
      layer_index >= num_layers || chunk_offset < 0 || block_rows < 1 || route_stride < 0 || error_stride < 0)
    return GLSDM_ERR_ARGUMENT;
  if (width > 32) return GLSDM_ERR_UNSUPPORTED;
  if (bank->banks != 1) return GLSDM_ERR_UNSUPPORTED;
  if (rows == 0) return GLSDM_OK;
  const BankView v = make_view(*bank);
  const int grid = blocks_for(rows, kWarpsPerBlock);
  const bool aligned = ((reinterpret_cast<uintptr_t>(error) | reinterpret_cast<uintptr_t>(out_deltas)) & 15u) == 0 &&
                       (error_stride % 4 == 0 || block_rows >= rows);
  if (bank->dtype == GLSDM_F32) {
    const bool vec = aligned && v.dim % 4 == 0 && (reinterpret_cast<uintptr_t>(v.values) & 15u) == 0;
    shard_propose_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        v, index, weights, error, decay_m1, mass, offsets, rows, block_rows, route_stride, error_stride, tokens,
        width, vec, chunk_offset,
        chunk_size * num_layers, num_layers, layer_index, out_addresses, out_deltas, out_keys);
  } else {
    const bool vec = aligned && v.dim % 8 == 0 && (reinterpret_cast<uintptr_t>(v.values) & 15u) == 0;
    shard_propose_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        v, index, weights, error, decay_m1, mass, offsets, rows, block_rows, route_stride, error_stride, tokens,
        width, vec, chunk_offset,
        chunk_size * num_layers, num_layers, layer_index, out_addresses, out_deltas, out_keys);
  }
  GLSDM_CUDA_OK(cudaGetLastError(), "shard_propose launch");
  count_launches(1);
  return GLSDM_OK;
}
