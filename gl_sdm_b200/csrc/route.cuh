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

// Routing rows are laid out [bank, token, head]: with per-request banks, row r reads bank
// r / rows_per_bank, so more rows than banks * rows_per_bank would index past the last bank.
// (A single shared bank serves any number of rows; a request table is checked on the device.)
inline int check_rows(const glsdm_bank* b, int64_t rows, int64_t rows_per_bank) {
  if (rows < 0 || rows_per_bank < 1) return GLSDM_ERR_ARGUMENT;
  if (b->banks > 1 && rows > b->banks * rows_per_bank) return GLSDM_ERR_ARGUMENT;
  return GLSDM_OK;
}

// Offer one factor's `half` scores (fp32, contiguous) to a selector; key = score | index.
// This is the general path (any length, any alignment, any score distribution); the bounded
// selections below take the common shapes and fall back to it.
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

// Bitonic sort of one float per lane, descending (no NaNs among the inputs).
__device__ __forceinline__ float warp_sort_desc_f32(float v, int lane) {
#pragma unroll
  for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      const float p = __shfl_xor_sync(kFullMask, v, j);
      const bool keep_max = ((lane & k) == 0) == ((lane & j) == 0);
      v = keep_max ? fmaxf(v, p) : fminf(v, p);
    }
  }
  return v;
}

#ifndef GLSDM_TWO_PASS_MIN_HALF
#define GLSDM_TWO_PASS_MIN_HALF 256
#endif
#ifndef GLSDM_SELECT_AHEAD
#define GLSDM_SELECT_AHEAD 4
#endif
#ifndef GLSDM_SELECT_AHEAD2
#define GLSDM_SELECT_AHEAD2 2
#endif
constexpr int kLaneSlots = 8;   // candidates one lane may note down in the second pass

// Common end of the bounded selections: every lane has noted `count` element indices in its
// slots; build their exact keys, sort once (twice and a merge above 32 candidates) and keep
// the 32 best. False when the candidates do not fit (the caller falls back).
__device__ __forceinline__ bool finish_candidates(const float* __restrict__ s, uint64_t* stage, int count,
                                                  int lane, uint64_t& list) {
  const uint16_t* __restrict__ slots = reinterpret_cast<const uint16_t*>(stage + kStageKeys);
  int upto = count;   // inclusive prefix over lanes
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(kFullMask, upto, o);
    if (lane >= o) upto += n;
  }
  const int total = __shfl_sync(kFullMask, upto, 31);
  if (__any_sync(kFullMask, count > kLaneSlots) || total > kStageKeys) return false;
  const int first = upto - count;
  for (int c = 0; c < count; ++c) {
    const uint32_t i = slots[c * 32 + lane];
    stage[first + c] = pack_key(orderable_bits(__ldg(s + i)), i);
  }
  __syncwarp();
  const uint64_t k0 = lane < total ? stage[lane] : 0ull;
  const uint64_t k1 = 32 + lane < total ? stage[32 + lane] : 0ull;
  __syncwarp();
  list = warp_sort_desc(k0, lane);
  if (total > 32) list = warp_merge_desc(list, warp_sort_desc(k1, lane), lane);
  return true;
}

// Two-pass selection of one factor's kf best scores, for long factors (reference rule as in
// offer_factor: score descending, larger index first on equal scores, NaN above everything).
//   pass 1  every lane keeps the maxima of two interleaved groups of its elements; the kf-th
//           largest of those 64 group maxima is a score that at least kf elements reach, so
//           nothing below it can be selected;
//   pass 2  re-read the factor (L1/L2) and note the index of every element not below that
//           bound - a few more than kf for any score distribution without long runs of ties;
//   finish  build the exact 64-bit keys of the noted elements, one bitonic sort (two and a
//           merge above 32 candidates), keep the best 32.
// The streaming selector pays a sort and a merge for every 32 elements that beat its running
// threshold (K*ln(half/K) of them); this pays one. Returns false, having selected nothing,
// when more than 64 elements reach the bound or one lane meets more than kLaneSlots of them:
// the caller then runs the streaming selector, so the result never depends on this path.
__device__ __forceinline__ bool select_factor_two_pass(const float* __restrict__ s, int half, int kf,
                                                       uint64_t* stage, int lane, uint64_t& list) {
  float a0 = -INFINITY, a1 = -INFINITY;
  // kAhead 16-byte loads per lane are requested before the first is used: the kernel lives on
  // memory-level parallelism per warp, not on many resident warps (the factor must still be in
  // L2 when the second pass comes back for it).
  constexpr int kAhead = GLSDM_SELECT_AHEAD;
  for (int base = 0; base < half; base += 128 * kAhead) {
    float4 v[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int i = base + u * 128 + lane * 4;
      v[u] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      if (i < half) v[u] = __ldg(reinterpret_cast<const float4*>(s + i));
    }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const float m = fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w));     // fmaxf skips NaNs
      if (u & 1) a1 = fmaxf(a1, m); else a0 = fmaxf(a0, m);
    }
  }
  // The 32 largest of the 64 group maxima, descending; lane kf-1 holds the bound.
  a0 = warp_sort_desc_f32(a0, lane);
  a1 = warp_sort_desc_f32(a1, lane);
  float top = fmaxf(a0, __shfl_sync(kFullMask, a1, 31 - lane));
#pragma unroll
  for (int j = 16; j > 0; j >>= 1) {
    const float p = __shfl_xor_sync(kFullMask, top, j);
    top = (lane & j) == 0 ? fmaxf(top, p) : fminf(top, p);
  }
  const float bound = __shfl_sync(kFullMask, top, kf - 1);

  uint16_t* __restrict__ slots = reinterpret_cast<uint16_t*>(stage + kStageKeys);   // [kLaneSlots][32]
  int count = 0;
  auto note = [&](bool pass, int index) {
    if (pass) {
      if (count < kLaneSlots) slots[count * 32 + lane] = static_cast<uint16_t>(index);
      ++count;
    }
  };
  constexpr int kAhead2 = GLSDM_SELECT_AHEAD2;
  for (int base = 0; base < half; base += 128 * kAhead2) {
    float4 v[kAhead2];
#pragma unroll
    for (int u = 0; u < kAhead2; ++u) {
      const int i = base + u * 128 + lane * 4;
      v[u] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);   // never reaches a finite bound ...
      if (i < half) v[u] = __ldg(reinterpret_cast<const float4*>(s + i));
    }
#pragma unroll
    for (int u = 0; u < kAhead2; ++u) {
      const int i = base + u * 128 + lane * 4;
      const bool live = i < half;                                          // ... and is masked for an infinite one
      const bool p0 = live && !(v[u].x < bound), p1 = live && !(v[u].y < bound);   // NaN passes
      const bool p2 = live && !(v[u].z < bound), p3 = live && !(v[u].w < bound);
      if (p0 | p1 | p2 | p3) {
        note(p0, i);
        note(p1, i + 1);
        note(p2, i + 2);
        note(p3, i + 3);
      }
    }
  }
  return finish_candidates(s, stage, count, lane, list);
}

// max that returns NaN when either input is NaN (fmaxf would drop it).
__device__ __forceinline__ float max_keep_nan(float a, float b) {
  float d;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}

constexpr int kGroupSteps = 16;   // 8-element groups one lane can keep in registers

// The same bounded selection for factors of 256..4096 scores (a multiple of 256): one pass
// over memory. A lane reads 8 consecutive scores per step (one 32-byte sector) and keeps the
// maximum of each such group in a register. The bound is taken from those maxima as in the
// two-pass selection; afterwards only the groups whose maximum reaches it - about as many as
// there are winners - are read again, one sector each, instead of the whole factor.
__device__ __forceinline__ bool select_factor_groups(const float* __restrict__ s, int half, int kf,
                                                     uint64_t* stage, int lane, uint64_t& list) {
  const int steps = half >> 8;
  float group[kGroupSteps];
  float a0 = -INFINITY, a1 = -INFINITY;
  const float4* __restrict__ mine = reinterpret_cast<const float4*>(s) + lane * 2;
#pragma unroll
  for (int u0 = 0; u0 < kGroupSteps; u0 += 4) {
    if (u0 < steps) {                       // steps is a multiple of 4 only above 1024 scores: guard each load
      float4 lo[4], hi[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bool live = u0 + j < steps;
        lo[j] = hi[j] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        if (live) {
          lo[j] = __ldg(mine + (u0 + j) * 64);
          hi[j] = __ldg(mine + (u0 + j) * 64 + 1);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float m = max_keep_nan(max_keep_nan(max_keep_nan(lo[j].x, lo[j].y), max_keep_nan(lo[j].z, lo[j].w)),
                                     max_keep_nan(max_keep_nan(hi[j].x, hi[j].y), max_keep_nan(hi[j].z, hi[j].w)));
        group[u0 + j] = m;
        if (j & 1) a1 = fmaxf(a1, m); else a0 = fmaxf(a0, m);     // fmaxf: a NaN group is left out of the bound
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) group[u0 + j] = -INFINITY;
    }
  }
  a0 = warp_sort_desc_f32(a0, lane);
  a1 = warp_sort_desc_f32(a1, lane);
  float top = fmaxf(a0, __shfl_sync(kFullMask, a1, 31 - lane));
#pragma unroll
  for (int j = 16; j > 0; j >>= 1) {
    const float p = __shfl_xor_sync(kFullMask, top, j);
    top = (lane & j) == 0 ? fmaxf(top, p) : fminf(top, p);
  }
  const float bound = __shfl_sync(kFullMask, top, kf - 1);

  uint16_t* __restrict__ slots = reinterpret_cast<uint16_t*>(stage + kStageKeys);   // [kLaneSlots][32]
  int count = 0;
  auto note = [&](bool pass, int index) {
    if (pass) {
      if (count < kLaneSlots) slots[count * 32 + lane] = static_cast<uint16_t>(index);
      ++count;
    }
  };
  // Each lane walks only its own groups that reach the bound (a NaN maximum passes): the warp
  // loops as often as its busiest lane has such groups, not once per group.
  unsigned hits = 0;
#pragma unroll
  for (int u = 0; u < kGroupSteps; ++u)
    if (u < steps && !(group[u] < bound)) hits |= 1u << u;
  while (hits) {
    const int u = __ffs(hits) - 1;
    hits &= hits - 1;
    const float4 lo = __ldg(mine + u * 64), hi = __ldg(mine + u * 64 + 1);
    const int i = u * 256 + lane * 8;
    note(!(lo.x < bound), i);
    note(!(lo.y < bound), i + 1);
    note(!(lo.z < bound), i + 2);
    note(!(lo.w < bound), i + 3);
    note(!(hi.x < bound), i + 4);
    note(!(hi.y < bound), i + 5);
    note(!(hi.z < bound), i + 6);
    note(!(hi.w < bound), i + 7);
  }
  return finish_candidates(s, stage, count, lane, list);
}

// The bounded selection for a factor of at most 128 scores (a multiple of 4): a lane holds its
// four scores in registers, the groups are those fours, and nothing is read twice.
__device__ __forceinline__ bool select_factor_small(const float* __restrict__ s, int half, int kf,
                                                    uint64_t* stage, int lane, uint64_t& list) {
  const int i = lane * 4;
  const bool live = i < half;
  float4 v = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
  if (live) v = __ldg(reinterpret_cast<const float4*>(s + i));
  float m = max_keep_nan(max_keep_nan(v.x, v.y), max_keep_nan(v.z, v.w));
  m = m != m ? INFINITY : m;            // a group holding a NaN outranks every finite bound
  const float bound = __shfl_sync(kFullMask, warp_sort_desc_f32(m, lane), kf - 1);
  uint16_t* __restrict__ slots = reinterpret_cast<uint16_t*>(stage + kStageKeys);
  int count = 0;
  auto note = [&](bool pass, int index) {
    if (pass) {
      slots[count * 32 + lane] = static_cast<uint16_t>(index);
      ++count;
    }
  };
  if (live) {
    note(!(v.x < bound), i);
    note(!(v.y < bound), i + 1);
    note(!(v.z < bound), i + 2);
    note(!(v.w < bound), i + 3);
  }
  return finish_candidates(s, stage, count, lane, list);
}

// Product-key selection for one row (reference gl_sdm/memory/routing.py:10-26).
//   per factor: the kf = min(width, half) best (score desc, index desc);
//   candidates: all kf*kf sums left[i] + right[j] (one fp32 add) at slot i*half + j;
//   result: the kout best (sum desc, slot desc), returned slot-ascending with softmax
//   weights in lanes [0, kout).
__device__ __forceinline__ void pk_route_row(const float* __restrict__ row_scores, int half,
                                             int kf, int kout, uint64_t* stage, int lane,
                                             uint32_t& slot, float& weight) {
  // Three bounded selections by factor length (registers only up to 128 scores, register
  // group maxima up to 4096, two passes over memory beyond); each declines a row it cannot
  // finish in one sort, and those rows - like odd lengths - stream through the selector.
  const bool two_pass = half >= GLSDM_TWO_PASS_MIN_HALF && (half & 3) == 0 && half <= 65536 &&
                        (reinterpret_cast<uintptr_t>(row_scores) & 15u) == 0;
  const bool small = half <= 128 && (half & 3) == 0 && (reinterpret_cast<uintptr_t>(row_scores) & 15u) == 0;
  const bool in_registers = (half & 255) == 0 && half <= 256 * kGroupSteps &&
                            (reinterpret_cast<uintptr_t>(row_scores) & 31u) == 0;
  uint64_t lists[2];
#pragma unroll
  for (int f = 0; f < 2; ++f) {
    const float* __restrict__ factor = row_scores + f * half;
    const bool done = small ? select_factor_small(factor, half, kf, stage, lane, lists[f])
                      : !two_pass ? false
                      : in_registers ? select_factor_groups(factor, half, kf, stage, lane, lists[f])
                                     : select_factor_two_pass(factor, half, kf, stage, lane, lists[f]);
    if (!done) {
      WarpSelect sel;
      sel.init(stage, kf, lane);
      offer_factor(sel, factor, half, lane);
      lists[f] = sel.list;
    }
  }
  pk_combine_lists(lists[0], lists[1], half, kf, kout, stage, lane, slot, weight);
}

// The pairs (i, j) of list positions with (i+1)*(j+1) <= 32, as i << 8 | j (0xffff = unused).
// With both lists descending, exact arithmetic puts the 32 largest sums among these 119.
static __device__ const uint16_t kHyperbola[128] = {
    0x0000, 0x0001, 0x0002, 0x0003, 0x0004, 0x0005, 0x0006, 0x0007, 0x0008, 0x0009, 0x000a, 0x000b,
    0x000c, 0x000d, 0x000e, 0x000f, 0x0010, 0x0011, 0x0012, 0x0013, 0x0014, 0x0015, 0x0016, 0x0017,
    0x0018, 0x0019, 0x001a, 0x001b, 0x001c, 0x001d, 0x001e, 0x001f, 0x0100, 0x0101, 0x0102, 0x0103,
    0x0104, 0x0105, 0x0106, 0x0107, 0x0108, 0x0109, 0x010a, 0x010b, 0x010c, 0x010d, 0x010e, 0x010f,
    0x0200, 0x0201, 0x0202, 0x0203, 0x0204, 0x0205, 0x0206, 0x0207, 0x0208, 0x0209, 0x0300, 0x0301,
    0x0302, 0x0303, 0x0304, 0x0305, 0x0306, 0x0307, 0x0400, 0x0401, 0x0402, 0x0403, 0x0404, 0x0405,
    0x0500, 0x0501, 0x0502, 0x0503, 0x0504, 0x0600, 0x0601, 0x0602, 0x0603, 0x0700, 0x0701, 0x0702,
    0x0703, 0x0800, 0x0801, 0x0802, 0x0900, 0x0901, 0x0902, 0x0a00, 0x0a01, 0x0b00, 0x0b01, 0x0c00,
    0x0c01, 0x0d00, 0x0d01, 0x0e00, 0x0e01, 0x0f00, 0x0f01, 0x1000, 0x1100, 0x1200, 0x1300, 0x1400,
    0x1500, 0x1600, 0x1700, 0x1800, 0x1900, 0x1a00, 0x1b00, 0x1c00, 0x1d00, 0x1e00, 0x1f00, 0xffff,
    0xffff, 0xffff, 0xffff, 0xffff, 0xffff, 0xffff, 0xffff, 0xffff};

// Second stage of the product-key selection: lanes [0, kf) hold the factor lists (key =
// orderable score << 32 | factor index, best first). All kf*kf sums left[i] + right[j] (one
// fp32 add) at slot i*half + j compete; the kout best (sum desc, slot desc) come back
// slot-ascending with softmax weights (reference gl_sdm/memory/routing.py:19-26).
// This is the plain form: every sum is offered to the streaming selector.
__device__ __forceinline__ uint64_t pk_combine_streaming(uint64_t left, uint64_t right, int half, int kf, int kout,
                                                        uint64_t* stage, int lane) {
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
  return sel.list;
}

// The 32 largest of two descending float lists (one value per lane each), descending.
__device__ __forceinline__ float warp_merge_desc_f32(float a, float b, int lane) {
  float x = fmaxf(a, __shfl_sync(kFullMask, b, 31 - lane));
#pragma unroll
  for (int j = 16; j > 0; j >>= 1) {
    const float p = __shfl_xor_sync(kFullMask, x, j);
    x = (lane & j) == 0 ? fmaxf(x, p) : fminf(x, p);
  }
  return x;
}

// The bounded form. The kout-th largest of the sums on the hyperbola (i+1)*(j+1) <= kout is a
// value that kout sums reach, and in exact arithmetic it IS the kout-th largest of all kf*kf
// sums; under fp32 rounding a sum outside the hyperbola can tie with it (and win on its
// address), so every sum that is not below the bound is collected - row by row, stopping at
// the first row where none is, since both lists descend - and ranked with the exact keys.
// Normally that is kout sums and they need no ranking at all. Too many candidates (long runs
// of ties, NaN scores): false, and the caller streams all sums through the selector.
__device__ __forceinline__ bool pk_combine_bounded(uint64_t left, uint64_t right, int half, int kf, int kout,
                                                   uint64_t* stage, int lane, uint64_t& list, int& count) {
  const float l_score = from_orderable_bits(static_cast<uint32_t>(left >> 32));
  const float r_score = from_orderable_bits(static_cast<uint32_t>(right >> 32));
  float v[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const uint32_t pair = __ldg(kHyperbola + r * 32 + lane);
    const int i = pair >> 8, j = pair & 0xff;
    const float sum = __fadd_rn(__shfl_sync(kFullMask, l_score, i & 31), __shfl_sync(kFullMask, r_score, j & 31));
    const bool valid = pair != 0xffffu && (i + 1) * (j + 1) <= kout && i < kf && j < kf;
    v[r] = !valid ? -INFINITY : (sum != sum ? INFINITY : sum);      // a NaN sum ranks above everything
    v[r] = warp_sort_desc_f32(v[r], lane);
  }
  const float top = warp_merge_desc_f32(warp_merge_desc_f32(v[0], v[1], lane), warp_merge_desc_f32(v[2], v[3], lane), lane);
  const float bound = __shfl_sync(kFullMask, top, kout - 1);

  const uint32_t right_index = static_cast<uint32_t>(right);
  count = 0;
  for (int i = 0; i < kf; ++i) {
    const float sum = __fadd_rn(__shfl_sync(kFullMask, l_score, i), r_score);
    const uint32_t left_index = __shfl_sync(kFullMask, static_cast<uint32_t>(left), i);
    const bool pass = lane < kf && !(sum < bound);
    const unsigned mask = __ballot_sync(kFullMask, pass);
    if (mask == 0) break;               // sums only get smaller down the list
    const int at = count + __popc(mask & ((1u << lane) - 1u));
    if (pass && at < kStageKeys) stage[at] = pack_key(orderable_bits(sum), left_index * static_cast<uint32_t>(half) + right_index);
    count += __popc(mask);
  }
  if (count > kStageKeys || count < kout) return false;
  __syncwarp();
  const uint64_t k0 = lane < count ? stage[lane] : 0ull;
  const uint64_t k1 = 32 + lane < count ? stage[32 + lane] : 0ull;
  __syncwarp();
  if (count == kout) {                  // exactly the winners: no ranking needed
    list = k0;
    return true;
  }
  list = warp_sort_desc(k0, lane);
  if (count > 32) list = warp_merge_desc(list, warp_sort_desc(k1, lane), lane);
  return true;
}

__device__ __forceinline__ void pk_combine_lists(uint64_t left, uint64_t right, int half, int kf, int kout,
                                                 uint64_t* stage, int lane, uint32_t& slot, float& weight) {
  uint64_t list;
  int count;
#ifndef GLSDM_COMBINE_BOUNDED
#define GLSDM_COMBINE_BOUNDED 1
#endif
  if (!GLSDM_COMBINE_BOUNDED || !pk_combine_bounded(left, right, half, kf, kout, stage, lane, list, count))
    list = pk_combine_streaming(left, right, half, kf, kout, stage, lane);
  float score;
  canonical_routes(list, kout, lane, slot, weight, score);
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
