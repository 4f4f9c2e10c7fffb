// Host-side plumbing of libnckv: error text, device queries, tensor-map encoding, status word.
#include <stdarg.h>
#include <string.h>

#include "nckv_common.cuh"

namespace nckv {

static thread_local char g_err[512] = {0};

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return NCKV_E_CUDA;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || p == nullptr) {
        set_error("cuTensorMapEncodeTiled is not available from this driver (%d)", (int)e);
        return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
    return fn;
}

// A (B, T, Hkv, 128) bf16 view seen as a 4-D tensor (d, h, t, b); one box is
// 64 channels x 1 head x box_tokens tokens, written to shared memory with the 128-byte
// swizzle so that 8 consecutive token rows land in 8 distinct 16-byte bank groups.
int make_kv_tensor_map(CUtensorMap *map, const void *base, int B, int T, int Hkv,
                       int64_t batch_stride, int64_t token_stride, int box_tokens) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return NCKV_E_CUDA;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) {
        set_error("cache base pointer is not 16-byte aligned");
        return NCKV_E_ARG;
    }
    if (token_stride < (int64_t)Hkv * NCKV_D || (token_stride % 8) != 0 || (batch_stride % 8) != 0) {
        set_error("cache strides must be multiples of 8 elements and token_stride >= Hkv*D");
        return NCKV_E_ARG;
    }
    cuuint64_t dims[4] = {(cuuint64_t)NCKV_D, (cuuint64_t)Hkv, (cuuint64_t)T, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)NCKV_D * 2, (cuuint64_t)token_stride * 2,
                             (cuuint64_t)batch_stride * 2};
    cuuint32_t box[4] = {64u, 1u, (cuuint32_t)box_tokens, 1u};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    if (B == 1) strides[2] = (cuuint64_t)T * token_stride * 2;  // unused dim still needs a legal stride
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (B=%d T=%d Hkv=%d bs=%lld ts=%lld)",
                  (int)r, B, T, Hkv, (long long)batch_stride, (long long)token_stride);
        return NCKV_E_CUDA;
    }
    return NCKV_OK;
}

// The same view as a 5-D tensor (d_lo[64], t, d_hi[2], h, b): one box of 64 x box_tokens x 2 brings both
// 64-channel halves of a tile with a single copy instruction and lays them out exactly like two
// 4-D boxes would ([half][token][128 B], 128-byte swizzle).  Returns NCKV_E_CUDA if the driver
// refuses the (non-monotonic) stride order; callers then fall back to make_kv_tensor_map.
int make_kv_tensor_map_5d(CUtensorMap *map, const void *base, int B, int T, int Hkv,
                          int64_t batch_stride, int64_t token_stride, int box_tokens) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return NCKV_E_CUDA;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || token_stride < (int64_t)Hkv * NCKV_D ||
        (token_stride % 8) != 0 || (batch_stride % 8) != 0) {
        set_error("cache pointer/strides unsuitable for a tensor map");
        return NCKV_E_ARG;
    }
    cuuint64_t dims[5] = {64, (cuuint64_t)T, 2, (cuuint64_t)Hkv, (cuuint64_t)B};
    cuuint64_t strides[4] = {(cuuint64_t)token_stride * 2, 128, (cuuint64_t)NCKV_D * 2,
                             B == 1 ? (cuuint64_t)T * token_stride * 2 : (cuuint64_t)batch_stride * 2};
    cuuint32_t box[5] = {64u, (cuuint32_t)box_tokens, 2u, 1u, 1u};
    cuuint32_t estr[5] = {1u, 1u, 1u, 1u, 1u};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (5-D) failed with CUresult %d", (int)r);
        return NCKV_E_CUDA;
    }
    return NCKV_OK;
}

}  // namespace nckv

extern "C" {

int nckv_version(void) { return 100; }
const char *nckv_arch(void) { return "sm_100a"; }
const char *nckv_last_error(void) { return nckv::g_err; }

int nckv_read_status(void *status_word, int clear, void *stream) {
    if (!status_word) {
        nckv::set_error("nckv_read_status: null status word");
        return NCKV_E_ARG;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int32_t v = 0;
    NCKV_CUDA_CHECK(cudaMemcpyAsync(&v, status_word, sizeof(v), cudaMemcpyDeviceToHost, s));
    NCKV_CUDA_CHECK(cudaStreamSynchronize(s));
    if (clear && v != 0) {
        NCKV_CUDA_CHECK(cudaMemsetAsync(status_word, 0, sizeof(v), s));
    }
    return (int)(v & 0x7fffffff);
}

}  // extern "C"
