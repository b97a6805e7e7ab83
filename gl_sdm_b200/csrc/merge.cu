// Merge of per-shard route candidates into the global routes of a slot-sharded bank.
// Every rank runs this on the same all-gathered candidate lists, so every rank derives the
// same routes. Tie rule and softmax: gl_sdm/memory/routing.py:21-26.
#include "common.cuh"

namespace glsdm {
namespace {

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
topk_merge_kernel(const float* __restrict__ cand_score, const int32_t* __restrict__ cand_slot,
                  int parts, int64_t part_stride, int64_t rows, int width, void* out_index, int i64,
                  float* __restrict__ out_weights) {
  __shared__ uint64_t stage[kWarpsPerBlock][kStageSlots];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (row >= rows) return;
  auto key_of = [&](int p) -> uint64_t {
    const int64_t at = static_cast<int64_t>(p) * part_stride + row * width + lane;
    if (lane >= width) return 0ull;
    const int32_t slot = cand_slot[at];
    // A shard with fewer than `width` slots pads its list with slot -1.
    return slot >= 0 ? pack_key(orderable_bits(cand_score[at]), static_cast<uint32_t>(slot)) : 0ull;
  };
  // Candidate lists normally arrive best first (that is how the scoring kernels write them):
  // then each one is a single bitonic merge into the running list. A list that is not in
  // that order sends the whole row through the general selector instead.
  uint64_t list = 0;
  bool in_order = true;
  for (int p = 0; p < parts && in_order; ++p) {
    const uint64_t key = key_of(p);
    const uint64_t next = __shfl_down_sync(kFullMask, key, 1);
    in_order = __all_sync(kFullMask, lane == 31 || key >= next);
    if (in_order) list = p == 0 ? key : warp_merge_desc(list, key, lane);
  }
  if (!in_order) {
    WarpSelect sel;
    sel.init(stage[warp], width, lane);
    for (int p = 0; p < parts; ++p) sel.offer(key_of(p));
    sel.finish();
    list = sel.list;
  }
  uint32_t slot;
  float weight, score;
  canonical_routes(list, width, lane, slot, weight, score);
  if (lane < width) {
    const int64_t at = row * width + lane;
    if (i64) static_cast<int64_t*>(out_index)[at] = slot;
    else static_cast<int32_t*>(out_index)[at] = static_cast<int32_t>(slot);
    out_weights[at] = weight;
  }
}

}  // namespace
}  // namespace glsdm

using namespace glsdm;

extern "C" int glsdm_topk_merge(const float* cand_score, const int32_t* cand_slot, int32_t parts,
                                int64_t rows, int32_t width, void* out_index, int index_i64,
                                float* out_weights, glsdm_stream_t stream) {
  return glsdm_topk_merge_strided(cand_score, cand_slot, parts, rows * width, rows, width, out_index, index_i64,
                                  out_weights, stream);
}

extern "C" int glsdm_topk_merge_strided(const float* cand_score, const int32_t* cand_slot, int32_t parts,
                                        int64_t part_stride, int64_t rows, int32_t width, void* out_index,
                                        int index_i64, float* out_weights, glsdm_stream_t stream) {
  if (cand_score == nullptr || cand_slot == nullptr || out_index == nullptr || out_weights == nullptr)
    return GLSDM_ERR_ARGUMENT;
  if (parts < 1 || rows < 0 || width < 1 || part_stride < rows * width) return GLSDM_ERR_ARGUMENT;
  if (width > 32) return GLSDM_ERR_UNSUPPORTED;
  if (rows == 0) return GLSDM_OK;
  topk_merge_kernel<<<blocks_for(rows, kWarpsPerBlock), kWarpsPerBlock * 32, 0, stream>>>(
      cand_score, cand_slot, parts, part_stride, rows, width, out_index, index_i64, out_weights);
  GLSDM_CUDA_OK(cudaGetLastError(), "topk_merge launch");
  count_launches(1);
  return GLSDM_OK;
}
