// Log-sum-exp combine of partial attention results computed over disjoint key ranges
// (the exchange step of the sequence-split long-context path).  One warp per output row;
// lane owns 4 of the 128 channels.  The reference never splits keys, so this has no
// counterpart there; it computes exactly what a single softmax over the union would.
#include <math.h>

#include "nckv_common.cuh"

namespace nckv {

__global__ void __launch_bounds__(256) lse_combine_kernel(const float *__restrict__ parts_o,
                                                         const float *__restrict__ parts_lse,
                                                         int n_parts, int rows, long long stride_o,
                                                         long long stride_lse,
                                                         __nv_bfloat16 *__restrict__ out,
                                                         float *__restrict__ lse_out) {
    const int lane = threadIdx.x & 31;
    const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (row >= rows) return;
    float M = -INFINITY;
    for (int i = 0; i < n_parts; ++i) M = fmaxf(M, parts_lse[(long long)i * stride_lse + row]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float L = 0.f;
    if (M > -INFINITY) {
        for (int i = 0; i < n_parts; ++i) {
            const float w = expf(parts_lse[(long long)i * stride_lse + row] - M);  // exp(-inf) = 0 drops empty parts
            if (w == 0.f) continue;
            const float4 v = reinterpret_cast<const float4 *>(parts_o + (long long)i * stride_o + row * NCKV_D)[lane];
            L += w;
            acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
        }
        const float inv = 1.f / L;
        acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    }
    uint2 packed;
    packed.x = pack_bf16x2(acc.x, acc.y);
    packed.y = pack_bf16x2(acc.z, acc.w);
    reinterpret_cast<uint2 *>(out + row * NCKV_D)[lane] = packed;
    if (lse_out && lane == 0) lse_out[row] = M > -INFINITY ? M + logf(L) : -INFINITY;
}

// The split bookkeeping as arrays (owned_below: nckv_common.cuh).  This kernel never releases its
// dependents early: a kernel launched behind it with programmatic dependent launch may read its
// outputs before its own grid-dependency wait (the decode kernels read cache_seqlens that early).
__global__ void kv_split_plan_kernel(const int32_t *__restrict__ seqlens, int B, int T_new, int world, int rank,
                                     int block, int32_t *__restrict__ local_len_after,
                                     int32_t *__restrict__ write_slot) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const int L = max(seqlens[b], 0);
    local_len_after[b] = owned_below(L + T_new, world, rank, block);
    // the T_new new tokens are written by this shard only if it owns position L (callers keep
    // T_new == 1 on this path, or chunks that do not straddle a block)
    write_slot[b] = ((L / block) % world == rank) ? owned_below(L, world, rank, block) : -1;
}

}  // namespace nckv

extern "C" int nckv_kv_split_plan(const int32_t *cache_seqlens, int B, int T_new, int world, int rank, int block,
                                  int32_t *local_len_after, int32_t *write_slot, void *stream) {
    using namespace nckv;
    if (!cache_seqlens || !local_len_after || !write_slot) {
        set_error("kv_split_plan: null pointer argument");
        return NCKV_E_ARG;
    }
    if (B <= 0 || T_new <= 0 || world <= 0 || rank < 0 || rank >= world || block <= 0) {
        set_error("kv_split_plan: bad argument (B=%d T_new=%d world=%d rank=%d block=%d)",
                  B, T_new, world, rank, block);
        return NCKV_E_ARG;
    }
    kv_split_plan_kernel<<<(B + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        cache_seqlens, B, T_new, world, rank, block, local_len_after, write_slot);
    NCKV_CUDA_CHECK(cudaGetLastError());
    return NCKV_OK;
}

extern "C" int nckv_lse_combine(const float *parts_o, const float *parts_lse, int n_parts, int rows,
                                int D, int64_t part_stride_o, int64_t part_stride_lse, void *out, float *lse_out,
                                void *stream) {
    using namespace nckv;
    if (!parts_o || !parts_lse || !out) {
        set_error("lse_combine: null pointer argument");
        return NCKV_E_ARG;
    }
    if (n_parts <= 0 || rows <= 0) {
        set_error("lse_combine: non-positive size (n_parts=%d rows=%d)", n_parts, rows);
        return NCKV_E_ARG;
    }
    if (D != NCKV_D) {
        set_error("lse_combine: head_dim %d unsupported (kernels are built for 128)", D);
        return NCKV_E_UNSUPPORTED;
    }
    if (part_stride_o < (int64_t)rows * D || part_stride_lse < rows || (part_stride_o % 4) != 0) {
        set_error("lse_combine: part strides (%lld, %lld) too small or misaligned for %d rows", (long long)part_stride_o,
                  (long long)part_stride_lse, rows);
        return NCKV_E_ARG;
    }
    if (((uintptr_t)parts_o | (uintptr_t)out) & 15) {
        set_error("lse_combine: tensors must be 16-byte aligned");
        return NCKV_E_ARG;
    }
    const int threads = 256;
    const long long blocks = ((long long)rows * 32 + threads - 1) / threads;
    lse_combine_kernel<<<(unsigned)blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        parts_o, parts_lse, n_parts, rows, (long long)part_stride_o, (long long)part_stride_lse,
        static_cast<__nv_bfloat16 *>(out), lse_out);
    NCKV_CUDA_CHECK(cudaGetLastError());
    return NCKV_OK;
}
