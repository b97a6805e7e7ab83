#include "common.cuh"
extern "C" size_t glsdm_score_topk_workspace_bytes(int64_t, int64_t, int32_t, int32_t) { return 0; }
extern "C" int glsdm_score_topk(const void*, const void*, int64_t, int64_t, int32_t, int32_t, int64_t,
                                float*, int32_t*, void*, size_t, uint32_t*, glsdm_stream_t) {
  return GLSDM_ERR_UNSUPPORTED;
}
