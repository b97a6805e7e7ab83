// Warp-level building blocks of the routed read: product-key selection of one
// (request, token, head) row and the weighted gather of its selected bank rows.
#pragma once

#include "common.cuh"

namespace glsdm {

// Bank geometry as the kernels see it (device copy of glsdm_bank plus derived strides).
struct BankView {
  const void* values;
  int64_t banks;
  int64_t slots;
  int64_t slot_lo;
  int64_t slot_hi;
  int64_t part_stride_rows;  // rows between consecutive (bank, head) partitions of this shard
  int32_t heads;
  int32_t dim;
};

inline BankView make_view(const glsdm_bank& b) {
  BankView v;
  v.values = b.values;
  v.banks = b.banks;
  v.slots = b.slots;
  v.slot_lo = b.slot_lo;
  v.slot_hi = b.slot_hi;
  v.part_stride_rows = b.slot_hi - b.slot_lo;
  v.heads = b.heads;
  v.dim = b.dim;
  return v;
}

inline int check_bank(const glsdm_bank* b) {
  if (b == nullptr || b->values == nullptr) return GLSDM_ERR_ARGUMENT;
  if (b->banks < 1 || b->heads < 1 || b->slots < 1 || b->dim < 1) return GLSDM_ERR_ARGUMENT;
  if (b->slot_lo < 0 || b->slot_hi > b->slots || b->slot_lo >= b->slot_hi) return GLSDM_ERR_ARGUMENT;
  if (b->dtype != GLSDM_F32 && b->dtype != GLSDM_BF16) return GLSDM_ERR_ARGUMENT;
  if (b->slots > 0xffffffffll) return GLSDM_ERR_UNSUPPORTED;
  return GLSDM_OK;
}

// Offer one factor's `half` scores (fp32, contiguous) to a selector; key = score | index.
// (Measured on B200: pre-filtering with a float compare, or unrolling four loads ahead, were
// both slower than this plain loop; the kernel is bound by instruction issue, not by loads.)
__device__ __forceinline__ void offer_factor(WarpSelect& sel, const float* __restrict__ s,
                                             int half, int lane) {
  if ((half & 3) == 0) {
    for (int base = 0; base < half; base += 128) {
      const int i = base + lane * 4;
      const bool live = i < half;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (live) v = __ldg(reinterpret_cast<const float4*>(s + i));
      sel.offer(live ? pack_key(orderable_bits(v.x), i) : 0ull);
      sel.offer(live ? pack_key(orderable_bits(v.y), i + 1) : 0ull);
      sel.offer(live ? pack_key(orderable_bits(v.z), i + 2) : 0ull);
      sel.offer(live ? pack_key(orderable_bits(v.w), i + 3) : 0ull);
    }
  } else {
    for (int base = 0; base < half; base += 32) {
      const int i = base + lane;
      const bool live = i < half;
      const float v = live ? __ldg(s + i) : 0.f;
      sel.offer(live ? pack_key(orderable_bits(v), i) : 0ull);
    }
  }
  sel.finish();
}

__device__ __forceinline__ void pk_combine_lists(uint64_t left, uint64_t right, int half, int kf, int kout,
                                                 uint64_t* stage, int lane, uint32_t& slot, float& weight);

// Product-key selection for one row (reference gl_sdm/memory/routing.py:10-26).
//   per factor: the kf = min(width, half) best (score desc, index desc);
//   candidates: all kf*kf sums left[i] + right[j] (one fp32 add) at slot i*half + j;
//   result: the kout best (sum desc, slot desc), returned slot-ascending with softmax
//   weights in lanes [0, kout).
__device__ __forceinline__ void pk_route_row(const float* __restrict__ row_scores, int half,
                                             int kf, int kout, uint64_t* stage, int lane,
                                             uint32_t& slot, float& weight) {
  WarpSelect sel;
  sel.init(stage, kf, lane);
  offer_factor(sel, row_scores, half, lane);
  const uint64_t left = sel.list;
  sel.init(stage, kf, lane);
  offer_factor(sel, row_scores + half, half, lane);
  const uint64_t right = sel.list;
  pk_combine_lists(left, right, half, kf, kout, stage, lane, slot, weight);
}

// Second stage of the product-key selection: lanes [0, kf) hold the factor lists (key =
// orderable score << 32 | factor index, best first). All kf*kf sums left[i] + right[j] (one
// fp32 add) at slot i*half + j compete; the kout best (sum desc, slot desc) come back
// slot-ascending with softmax weights (reference gl_sdm/memory/routing.py:19-26).
__device__ __forceinline__ void pk_combine_lists(uint64_t left, uint64_t right, int half, int kf, int kout,
                                                 uint64_t* stage, int lane, uint32_t& slot, float& weight) {
  WarpSelect sel;
  const bool right_live = lane < kf;
  const float right_score = from_orderable_bits(static_cast<uint32_t>(right >> 32));
  const uint32_t right_index = static_cast<uint32_t>(right);
  sel.init(stage, kout, lane);
  for (int i = 0; i < kf; ++i) {
    const uint64_t l = shfl_u64(left, i);
    const float sum = __fadd_rn(from_orderable_bits(static_cast<uint32_t>(l >> 32)), right_score);
    const uint32_t address = static_cast<uint32_t>(l) * static_cast<uint32_t>(half) + right_index;
    sel.offer(right_live ? pack_key(orderable_bits(sum), address) : 0ull);
  }
  sel.finish();
  float score;
  canonical_routes(sel.list, kout, lane, slot, weight, score);
}

template <typename T>
struct Unit;  // one 16-byte unit of a bank row, decoded to fp32

template <>
struct Unit<float> {
  static constexpr int kElems = 4;
  __device__ static __forceinline__ void decode(const uint4& raw, float (&out)[4]) {
    out[0] = __uint_as_float(raw.x);
    out[1] = __uint_as_float(raw.y);
    out[2] = __uint_as_float(raw.z);
    out[3] = __uint_as_float(raw.w);
  }
  __device__ static __forceinline__ float scalar(const float* p) { return __ldg(p); }
};

template <>
struct Unit<__nv_bfloat16> {
  static constexpr int kElems = 8;
  __device__ static __forceinline__ void decode(const uint4& raw, float (&out)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static __forceinline__ float scalar(const __nv_bfloat16* p) {
    return __uint_as_float(static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned short*>(p))) << 16);
  }
};

// True when rows can be moved as 16-byte units by the vector path.
template <typename T>
__host__ __device__ inline bool vector_rows(int dim, const void* base) {
  constexpr int e = Unit<T>::kElems;
  if (dim % e != 0) return false;
  const int units = dim / e;
  const bool pow2 = (units & (units - 1)) == 0;
  if (!((units <= 32 && pow2) || (units % 32 == 0))) return false;
  return (reinterpret_cast<uintptr_t>(base) & 15u) == 0;
}

// Weighted sum of the selected rows of one partition (reference routing.py:27-28):
// lanes [0, count) hold (slot, weight); every lane returns, in acc, the sum over routes of
// weight * row[unit elements] for the unit it owns in unit block `ub` (lane % units_here).
// Rows whose slot is outside [slot_lo, slot_hi) contribute nothing.
template <typename T>
__device__ __forceinline__ void gather_units(const T* __restrict__ part, const BankView& bank,
                                             uint32_t slot, float weight, int count, int lane,
                                             int units, int ub,
                                             float (&acc)[Unit<T>::kElems]) {
  constexpr int E = Unit<T>::kElems;
  const int here = units < 32 ? units : 32;  // units handled per pass
  const int groups = 32 / here;
  const int g = lane / here;
  const int u = ub * 32 + (lane % here);
#pragma unroll
  for (int i = 0; i < E; ++i) acc[i] = 0.f;
  const uint4* __restrict__ rows = reinterpret_cast<const uint4*>(part);
  for (int k0 = 0; k0 < count; k0 += groups * 4) {
    uint4 raw[4];
    float wk[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + j * groups + g;
      const uint32_t a = __shfl_sync(kFullMask, slot, k & 31);
      const float w = __shfl_sync(kFullMask, weight, k & 31);
      const bool live = k < count && static_cast<int64_t>(a) >= bank.slot_lo &&
                        static_cast<int64_t>(a) < bank.slot_hi;
      wk[j] = live ? w : 0.f;
      raw[j] = make_uint4(0u, 0u, 0u, 0u);
      if (live) raw[j] = __ldg(rows + (static_cast<int64_t>(a) - bank.slot_lo) * units + u);
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

// Readings of one row into out_row[dim] (fp32). Vector path when rows are 16-byte tileable,
// element-strided path otherwise.
template <typename T>
__device__ __forceinline__ void read_row(const T* __restrict__ part, const BankView& bank,
                                         uint32_t slot, float weight, int count, int lane,
                                         bool vec, float* __restrict__ out_row) {
  constexpr int E = Unit<T>::kElems;
  const int dim = bank.dim;
  if (vec) {
    const int units = dim / E;
    const int passes = units <= 32 ? 1 : units / 32;
    const int here = units < 32 ? units : 32;
    for (int ub = 0; ub < passes; ++ub) {
      float acc[E];
      gather_units<T>(part, bank, slot, weight, count, lane, units, ub, acc);
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
      for (int k = 0; k < count; ++k) {
        const uint32_t a = __shfl_sync(kFullMask, slot, k);
        const float w = __shfl_sync(kFullMask, weight, k);
        const bool live = static_cast<int64_t>(a) >= bank.slot_lo &&
                          static_cast<int64_t>(a) < bank.slot_hi && d < dim;
        if (live) acc = fmaf(w, Unit<T>::scalar(part + (static_cast<int64_t>(a) - bank.slot_lo) * dim + d), acc);
      }
      if (d < dim) out_row[d] = acc;
    }
  }
}

// Partition (bank, head) that routing row `row` reads, and the base of its shard.
__device__ __forceinline__ int64_t partition_of(const BankView& bank, int64_t row,
                                                int64_t rows_per_bank,
                                                const int64_t* __restrict__ requests) {
  const int64_t head = row % bank.heads;
  int64_t b = 0;
  if (requests != nullptr) {
    b = requests[row / bank.heads];
  } else if (bank.banks > 1) {
    b = row / rows_per_bank;
  }
  return b * bank.heads + head;
}

}  // namespace glsdm
