// Kernel (c): prefill broadcast — KVCache.prefill (engine.py:123-137).
//
// The batch-1 prompt cache (L, 1, T_src, Hkv, D) is copied into every row of the decode cache
// (L, B, T_dst, Hkv, D) for the first p tokens.  Per (layer, row) that is one contiguous run of
// p*Hkv*D elements, so the copy is pure 16-byte vector traffic: each thread loads a few source
// vectors ONCE and stores them to all B rows (source bytes cross HBM once; the B-fold fan-out is
// all writes, which is what bounds this kernel).  K and V go through the same launch; the new
// cache_seqlens (= p for every row) are written by the first CTA.
#include "nckv_common.cuh"

namespace nckv {

constexpr int BC_THREADS = 256;
constexpr int BC_VEC = 4;  // 16-byte vectors per thread per step (64 B in flight per thread per row)

struct BroadcastParams {
    const uint4 *src[2];
    uint4 *dst[2];
    int32_t *dst_seqlens;
    int L, B, p;
    long long run_vecs;        // p*Hkv*D / 8
    long long src_layer_vecs;  // T_src*Hkv*D / 8
    long long dst_row_vecs;    // T_dst*Hkv*D / 8
};

__global__ void __launch_bounds__(BC_THREADS) prefill_broadcast_kernel(const BroadcastParams q) {
    if (blockIdx.x == 0 && q.dst_seqlens) {
        for (int b = threadIdx.x; b < q.B; b += blockDim.x) q.dst_seqlens[b] = q.p;
    }
    // chunk = BC_THREADS*BC_VEC consecutive vectors of one (tensor, layer) run
    const long long chunk_vecs = (long long)BC_THREADS * BC_VEC;
    const long long chunks_per_run = (q.run_vecs + chunk_vecs - 1) / chunk_vecs;
    const long long n_chunks = 2LL * q.L * chunks_per_run;
    for (long long c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        const int which = (int)(c / (q.L * chunks_per_run));
        const long long rem = c % (q.L * chunks_per_run);
        const int layer = (int)(rem / chunks_per_run);
        const long long v0 = (rem % chunks_per_run) * chunk_vecs;
        const uint4 *s = (which ? q.src[1] : q.src[0]) + layer * q.src_layer_vecs;
        uint4 *d = (which ? q.dst[1] : q.dst[0]) + (long long)layer * q.B * q.dst_row_vecs;
        uint4 regs[BC_VEC];
        bool live[BC_VEC];
#pragma unroll
        for (int i = 0; i < BC_VEC; ++i) {
            const long long v = v0 + (long long)i * BC_THREADS + threadIdx.x;
            live[i] = v < q.run_vecs;
            if (live[i]) regs[i] = __ldg(s + v);
        }
        for (int b = 0; b < q.B; ++b) {
            uint4 *row = d + (long long)b * q.dst_row_vecs;
#pragma unroll
            for (int i = 0; i < BC_VEC; ++i) {
                const long long v = v0 + (long long)i * BC_THREADS + threadIdx.x;
                if (live[i]) __stcs(row + v, regs[i]);
            }
        }
    }
}

// The same prefill into a paged cache.  Pages that hold a whole page of prompt tokens are shared by
// all rows (the block tables point at them), so the copy is a list of jobs "fill page P with n tokens
// of the prompt starting at token t0": one job per shared page plus one per row for the page that
// holds the prompt's tail, which each row needs for itself because it appends there.
struct PagedFillParams {
    const uint4 *src[2];
    uint4 *dst[2];
    const int32_t *jobs;  // n_jobs x (page, first source token, tokens)
    int L, n_pages;
    long long tok_vecs;        // Hkv*D / 8
    long long src_layer_vecs;  // T_src*Hkv*D / 8
    long long page_vecs;       // page_tokens*Hkv*D / 8
};

__global__ void __launch_bounds__(BC_THREADS) paged_fill_kernel(const PagedFillParams q) {
    const int job = blockIdx.y;
    const int which = blockIdx.z & 1, layer = blockIdx.z >> 1;
    const int page = q.jobs[3 * job], t0 = q.jobs[3 * job + 1], n = q.jobs[3 * job + 2];
    if (page < 0 || page >= q.n_pages || n <= 0) return;
    const long long run = (long long)n * q.tok_vecs;
    const uint4 *s = (which ? q.src[1] : q.src[0]) + layer * q.src_layer_vecs + (long long)t0 * q.tok_vecs;
    uint4 *d = (which ? q.dst[1] : q.dst[0]) + ((long long)layer * q.n_pages + page) * q.page_vecs;
    const long long v0 = (long long)blockIdx.x * BC_THREADS * BC_VEC;
#pragma unroll
    for (int i = 0; i < BC_VEC; ++i) {
        const long long v = v0 + (long long)i * BC_THREADS + threadIdx.x;
        if (v < run) __stcs(d + v, __ldg(s + v));
    }
}

}  // namespace nckv

extern "C" int nckv_paged_fill(const void *src_k, const void *src_v, void *k_pool, void *v_pool, const int32_t *jobs,
                               int n_jobs, int L, int Hkv, int D, int T_src, int page_tokens, int n_pages,
                               void *stream) {
    using namespace nckv;
    if (!src_k || !src_v || !k_pool || !v_pool || !jobs) {
        set_error("paged_fill: null pointer argument");
        return NCKV_E_ARG;
    }
    if (n_jobs <= 0 || n_jobs > 65535 || L <= 0 || 2 * L > 65535 || Hkv <= 0 || T_src <= 0 || page_tokens <= 0 || n_pages <= 0) {
        set_error("paged_fill: bad size (n_jobs=%d L=%d Hkv=%d T_src=%d page_tokens=%d n_pages=%d)", n_jobs, L, Hkv, T_src,
                  page_tokens, n_pages);
        return NCKV_E_ARG;
    }
    if ((D % 8) != 0) {
        set_error("paged_fill: head_dim %d must be a multiple of 8", D);
        return NCKV_E_UNSUPPORTED;
    }
    if (((uintptr_t)src_k | (uintptr_t)src_v | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) {
        set_error("paged_fill: tensors must be 16-byte aligned");
        return NCKV_E_ARG;
    }
    PagedFillParams q;
    q.src[0] = static_cast<const uint4 *>(src_k);
    q.src[1] = static_cast<const uint4 *>(src_v);
    q.dst[0] = static_cast<uint4 *>(k_pool);
    q.dst[1] = static_cast<uint4 *>(v_pool);
    q.jobs = jobs;
    q.L = L; q.n_pages = n_pages;
    q.tok_vecs = (long long)Hkv * D / 8;
    q.src_layer_vecs = (long long)T_src * q.tok_vecs;
    q.page_vecs = (long long)page_tokens * q.tok_vecs;
    const long long chunk_vecs = (long long)BC_THREADS * BC_VEC;
    const dim3 grid((unsigned)((q.page_vecs + chunk_vecs - 1) / chunk_vecs), (unsigned)n_jobs, (unsigned)(2 * L));
    paged_fill_kernel<<<grid, BC_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(q);
    NCKV_CUDA_CHECK(cudaGetLastError());
    return NCKV_OK;
}

extern "C" int nckv_prefill_broadcast(const void *src_k, const void *src_v, void *dst_k, void *dst_v,
                                      int32_t *dst_seqlens, int L, int B, int p, int Hkv, int D,
                                      int T_src, int T_dst, void *stream) {
    using namespace nckv;
    if (!src_k || !src_v || !dst_k || !dst_v) {
        set_error("prefill_broadcast: null pointer argument");
        return NCKV_E_ARG;
    }
    if (L <= 0 || B <= 0 || Hkv <= 0 || p < 0 || T_src <= 0 || T_dst <= 0) {
        set_error("prefill_broadcast: bad size (L=%d B=%d p=%d Hkv=%d T_src=%d T_dst=%d)", L, B, p, Hkv, T_src, T_dst);
        return NCKV_E_ARG;
    }
    if ((D % 8) != 0) {
        set_error("prefill_broadcast: head_dim %d must be a multiple of 8", D);
        return NCKV_E_UNSUPPORTED;
    }
    if (p > T_src || p > T_dst) {
        set_error("prefill_broadcast: p=%d exceeds a cache capacity (T_src=%d, T_dst=%d)", p, T_src, T_dst);
        return NCKV_E_CAPACITY;
    }
    if (((uintptr_t)src_k | (uintptr_t)src_v | (uintptr_t)dst_k | (uintptr_t)dst_v) & 15) {
        set_error("prefill_broadcast: tensors must be 16-byte aligned");
        return NCKV_E_ARG;
    }
    BroadcastParams q;
    q.src[0] = static_cast<const uint4 *>(src_k);
    q.src[1] = static_cast<const uint4 *>(src_v);
    q.dst[0] = static_cast<uint4 *>(dst_k);
    q.dst[1] = static_cast<uint4 *>(dst_v);
    q.dst_seqlens = dst_seqlens;
    q.L = L; q.B = B; q.p = p;
    q.run_vecs = (long long)p * Hkv * D / 8;
    q.src_layer_vecs = (long long)T_src * Hkv * D / 8;
    q.dst_row_vecs = (long long)T_dst * Hkv * D / 8;
    const long long chunk_vecs = (long long)BC_THREADS * BC_VEC;
    const long long n_chunks = 2LL * L * ((q.run_vecs + chunk_vecs - 1) / chunk_vecs);
    long long grid = (long long)sm_count() * 8;
    if (n_chunks < grid) grid = n_chunks > 0 ? n_chunks : 1;
    prefill_broadcast_kernel<<<(unsigned)grid, BC_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(q);
    NCKV_CUDA_CHECK(cudaGetLastError());
    return NCKV_OK;
}
