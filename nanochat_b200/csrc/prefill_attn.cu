// Kernel (d) placeholder while the tcgen05 tile kernel is being brought up.
#include "nckv_common.cuh"

extern "C" int nckv_prefill_attn(const void *q, const void *k, const void *v, const int32_t *cache_seqlens,
                                 void *out, int B, int T_new, int Hq, int Hkv, int D, int T_k,
                                 int64_t kv_batch_stride, int64_t kv_token_stride, int window_left,
                                 int32_t *status, void *stream) {
    nckv::set_error("prefill_attn: not built yet");
    return NCKV_E_UNSUPPORTED;
}
