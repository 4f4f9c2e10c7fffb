// Kernel (a): fused RoPE + QK rms-norm + scale + KV append, bit-exact against the eager bf16 path.
//
// One half-warp (16 lanes x 8 bf16 = one 256-byte head row, 16-byte loads and stores) handles
// one (row b, token t, head) of q, k or v.  The arithmetic reproduces, rounding for rounding,
// the reference's op sequence on bf16 tensors:
//   apply_rotary_emb (gpt.py:57-63):  y1 = bf16(bf16(x1*cos) + bf16(x2*sin))
//                                     y2 = bf16(bf16(x1*(-sin)) + bf16(x2*cos))
//   norm (gpt.py:42-43):              z  = bf16(y * rsqrt(mean_fp32(y^2) + eps))
//   scale (gpt.py:101-102):           out = bf16(float(z) * 1.2f)
// The fp32 sum of squares is accumulated in the order of torch's vectorised row kernel for a
// 128-wide row (32 lanes x 4 consecutive elements, sequential within a lane, then a
// shuffle-down tree with offsets 16, 8, 4, 2, 1), so that rstd carries the same last bit.
#include "nckv_common.cuh"

namespace nckv {

struct AppendParams {
    const uint4 *q_in;
    const uint4 *k_in;
    const uint4 *v_in;
    uint4 *q_out;
    __nv_bfloat16 *k_cache;
    __nv_bfloat16 *v_cache;
    const int32_t *cache_seqlens;
    const int32_t *write_slots;  // optional: cache index of token 0 per row (-1: do not write); null = cache_seqlens
    const uint4 *cos;  // (rope_len, 64) bf16 = 8 uint4 per position
    const uint4 *sin;
    int32_t *status;
    int B, T_new, Hq, Hkv, T_max, rope_len;
    int64_t cache_batch_stride, cache_token_stride;
    float qk_scale, eps;
    int transform_k;  // 0: k is stored as given (plain append)
    KvSplit split;    // block > 0: block-cyclic sequence split, the owner of position cache_seqlens[b] stores k/v
    // paged storage (block_table != null): the caches are page pools (n_pages, page_tokens, Hkv, D);
    // T_max is then max_pages * page_tokens and cache_batch_stride the distance between pages
    const int32_t *block_table;
    int page_tokens, max_pages, n_pages;
    // distance between the tokens of q_in / k_in / v_in in 16-byte units (heads of a token are packed); lets the
    // three be column slices of one projection output
    long long q_stride, k_stride, v_stride;
};

__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
    f[0] = bf16lo(v.x); f[1] = bf16hi(v.x);
    f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
    f[4] = bf16lo(v.z); f[5] = bf16hi(v.z);
    f[6] = bf16lo(v.w); f[7] = bf16hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 v;
    v.x = pack_bf16x2(f[0], f[1]);
    v.y = pack_bf16x2(f[2], f[3]);
    v.z = pack_bf16x2(f[4], f[5]);
    v.w = pack_bf16x2(f[6], f[7]);
    return v;
}
__device__ __forceinline__ uint4 shfl_xor_u4(const uint4 &v, int mask) {
    uint4 r;
    r.x = __shfl_xor_sync(0xffffffffu, v.x, mask);
    r.y = __shfl_xor_sync(0xffffffffu, v.y, mask);
    r.z = __shfl_xor_sync(0xffffffffu, v.z, mask);
    r.w = __shfl_xor_sync(0xffffffffu, v.w, mask);
    return r;
}

// RoPE -> rms-norm -> scale on one 128-wide head row held 8 elements per lane by 16 lanes.
// `j` is the lane's index within its half-warp (0..15); all 32 lanes must call this.
__device__ __forceinline__ uint4 rope_norm_scale(const uint4 &xin, const uint4 &cosv,
                                                 const uint4 &sinv, int j, float qk_scale,
                                                 float eps) {
    float own[8], oth[8], c[8], s[8], y[8];
    uint4 partner = shfl_xor_u4(xin, 8);  // channel i <-> i + 64
    unpack8(xin, own);
    unpack8(partner, oth);
    unpack8(cosv, c);
    unpack8(sinv, s);
    const bool first_half = j < 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (first_half) {  // own = x1, oth = x2
            float t1 = round_bf16(__fmul_rn(own[i], c[i]));
            float t2 = round_bf16(__fmul_rn(oth[i], s[i]));
            y[i] = round_bf16(__fadd_rn(t1, t2));
        } else {  // own = x2, oth = x1
            float t3 = round_bf16(__fmul_rn(oth[i], -s[i]));
            float t4 = round_bf16(__fmul_rn(own[i], c[i]));
            y[i] = round_bf16(__fadd_rn(t3, t4));
        }
    }
    // sum of squares: two "virtual lanes" of 4 consecutive elements per real lane
    float e0 = __fmul_rn(y[0], y[0]);
    e0 = __fmaf_rn(y[1], y[1], e0);
    e0 = __fmaf_rn(y[2], y[2], e0);
    e0 = __fmaf_rn(y[3], y[3], e0);
    float e1 = __fmul_rn(y[4], y[4]);
    e1 = __fmaf_rn(y[5], y[5], e1);
    e1 = __fmaf_rn(y[6], y[6], e1);
    e1 = __fmaf_rn(y[7], y[7], e1);
    // virtual shuffle-down tree with offsets 16, 8, 4, 2 (= real-lane offsets 8, 4, 2, 1), then 1
#pragma unroll
    for (int off = 8; off >= 1; off >>= 1) {
        float o0 = __shfl_down_sync(0xffffffffu, e0, off, 16);
        float o1 = __shfl_down_sync(0xffffffffu, e1, off, 16);
        e0 = __fadd_rn(e0, o0);
        e1 = __fadd_rn(e1, o1);
    }
    float total = __fadd_rn(e0, e1);
    total = __shfl_sync(0xffffffffu, total, 0, 16);
    const float rstd = rsqrtf(__fadd_rn(__fdiv_rn(total, 128.0f), eps));
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float z = round_bf16(__fmul_rn(y[i], rstd));
        o[i] = __fmul_rn(z, qk_scale);  // pack8 applies the final bf16 rounding
    }
    return pack8(o);
}

__global__ void __launch_bounds__(256) append_rope_norm_kernel(const AppendParams p) {
    // Programmatic dependent launch: this grid may have been scheduled while its predecessor was
    // still running; its inputs come from that predecessor, so wait before touching anything.
    // The attention kernel that follows may be scheduled right away, even before that wait: it
    // reads only cache_seqlens and older cache rows until it has itself waited for this grid.
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int lane = threadIdx.x & 31;
    const int j = lane & 15;
    const int heads_per_tok = (p.q_in ? p.Hq : 0) + 2 * p.Hkv;
    const int q_heads = p.q_in ? p.Hq : 0;
    const long long total_rows = (long long)p.B * p.T_new * heads_per_tok;
    const long long n_half_warps = ((long long)gridDim.x * blockDim.x) >> 4;
    long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    // rows are padded to an even count per iteration so both half-warps stay convergent
    const long long padded = (total_rows + 1) & ~1LL;
    for (; row < padded; row += n_half_warps) {
        const bool live = row < total_rows;
        const long long r = live ? row : total_rows - 1;
        const int slot = (int)(r % heads_per_tok);
        const long long bt = r / heads_per_tok;
        const int t = (int)(bt % p.T_new);
        const int b = (int)(bt / p.T_new);
        // kind: 0 = q head, 1 = k head, 2 = v head.  The two half-warps of a warp may hold
        // different kinds, so the transform (which shuffles across the warp) runs unconditionally
        // and its result is selected afterwards.
        const int kind = slot < q_heads ? 0 : (slot < q_heads + p.Hkv ? 1 : 2);
        const int h = kind == 0 ? slot : (kind == 1 ? slot - q_heads : slot - q_heads - p.Hkv);
        const bool transform = kind == 0 || (kind == 1 && p.transform_k);
        const uint4 *src = kind == 0 ? p.q_in : (kind == 1 ? p.k_in : p.v_in);
        const long long src_idx = (bt * (kind == 0 ? p.Hq : p.Hkv) + h) * 16 + j;  // packed: where q_out goes
        const long long in_idx = bt * (kind == 0 ? p.q_stride : (kind == 1 ? p.k_stride : p.v_stride)) + h * 16 + j;
        // the input row does not depend on the row's length: its load goes out together with the
        // length's, one round trip ahead of the table rows that do
        uint4 x = make_uint4(0, 0, 0, 0);
        if (live) x = src[in_idx];
        const int len = p.cache_seqlens[b];          // sequence position of token 0 (drives RoPE)
        int wslot = p.write_slots ? p.write_slots[b] : len;  // cache index of token 0
        if (p.split.block > 0 && len >= 0)
            wslot = (len / p.split.block) % p.split.world == p.split.rank
                        ? owned_below(len, p.split.world, p.split.rank, p.split.block) : -1;
        const int pos = len + t;
        bool ok = live;
        if (len < 0 || wslot < -1) {
            if (live && j == 0 && slot == 0 && t == 0) atomicOr(p.status, (int)NCKV_ST_BAD_SEQLEN);
            ok = false;
        } else if ((wslot >= 0 && wslot + p.T_new > p.T_max) || (p.rope_len > 0 && len + p.T_new > p.rope_len)) {
            if (live && j == 0 && slot == 0 && t == 0) atomicOr(p.status, (int)NCKV_ST_OVERFLOW);
            ok = false;
        }
        const bool write_kv = ok && wslot >= 0;  // -1: this row's token belongs to another shard
        const int safe_pos = ok ? pos : 0;
        uint4 cv = make_uint4(0, 0, 0, 0), sv = cv;
        if (!ok) x = cv;
        if (ok && transform) {
            cv = p.cos[(long long)safe_pos * 8 + (j & 7)];
            sv = p.sin[(long long)safe_pos * 8 + (j & 7)];
        }
        uint4 o = rope_norm_scale(x, cv, sv, j, p.qk_scale, p.eps);
        if (!transform) o = x;
        if (ok) {
            if (kind == 0) {
                p.q_out[src_idx] = o;
            } else if (write_kv) {
                __nv_bfloat16 *cache = kind == 1 ? p.k_cache : p.v_cache;
                long long outer = b, tok = wslot + t;
                if (p.block_table) {  // row -> page
                    const int idx = (int)(tok / p.page_tokens);
                    tok -= (long long)idx * p.page_tokens;
                    outer = p.block_table[(long long)b * p.max_pages + idx];
                    if (outer < 0 || outer >= p.n_pages) {
                        if (j == 0 && h == 0 && kind == 1) atomicOr(p.status, (int)NCKV_ST_BAD_PAGE);
                        outer = -1;
                    }
                }
                if (outer >= 0) {
                    uint4 *dst = reinterpret_cast<uint4 *>(cache + outer * p.cache_batch_stride +
                                                           tok * p.cache_token_stride + (long long)h * NCKV_D);
                    dst[j] = o;
                }
            }
        }
    }
}

static int check_common(const void *k_in, const void *v_in, void *k_cache, void *v_cache,
                        const int32_t *cache_seqlens, int B, int T_new, int Hkv, int D, int T_max,
                        int64_t bs, int64_t ts, int32_t *status) {
    if (!k_in || !v_in || !k_cache || !v_cache || !cache_seqlens || !status) {
        set_error("append: null pointer argument");
        return NCKV_E_ARG;
    }
    if (B <= 0 || T_new <= 0 || Hkv <= 0 || T_max <= 0) {
        set_error("append: non-positive size (B=%d T_new=%d Hkv=%d T_max=%d)", B, T_new, Hkv, T_max);
        return NCKV_E_ARG;
    }
    if (D != NCKV_D) {
        set_error("append: head_dim %d unsupported (kernels are built for 128)", D);
        return NCKV_E_UNSUPPORTED;
    }
    if (T_new > T_max) {
        set_error("append: T_new=%d exceeds cache capacity T_max=%d", T_new, T_max);
        return NCKV_E_CAPACITY;
    }
    if (ts < (int64_t)Hkv * D || (ts % 8) != 0 || (bs % 8) != 0) {
        set_error("append: cache strides must be multiples of 8 elements, token stride >= Hkv*D");
        return NCKV_E_ARG;
    }
    const uintptr_t a = (uintptr_t)k_in | (uintptr_t)v_in | (uintptr_t)k_cache | (uintptr_t)v_cache;
    if (a & 15) {
        set_error("append: tensors must be 16-byte aligned");
        return NCKV_E_ARG;
    }
    return NCKV_OK;
}

static int launch_append(const AppendParams &p, cudaStream_t stream) {
    const int heads_per_tok = (p.q_in ? p.Hq : 0) + 2 * p.Hkv;
    const long long rows = (long long)p.B * p.T_new * heads_per_tok;
    const int threads = 256;                                   // 16 head rows per CTA
    long long blocks = (rows + 15) / 16;
    const long long cap = (long long)sm_count() * 8 * 4;       // grid-stride beyond this
    if (blocks > cap) blocks = cap;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NCKV_CUDA_CHECK(cudaLaunchKernelEx(&cfg, append_rope_norm_kernel, p));
    return NCKV_OK;
}

}  // namespace nckv

extern "C" {

static int append_rope_norm_impl(const void *q_in, const void *k_in, const void *v_in, void *q_out,
                                 void *k_cache, void *v_cache, const int32_t *cache_seqlens,
                                 const int32_t *write_slots, nckv::KvSplit split, const void *cos, const void *sin, int B, int T_new,
                                 int Hq, int Hkv, int D, int T_max, int64_t cache_batch_stride,
                                 int64_t cache_token_stride, int rope_len, float qk_scale, float eps,
                                 int32_t *status, void *stream, const int32_t *block_table = nullptr,
                                 int page_tokens = 0, int max_pages = 0, int n_pages = 0, int64_t q_token_stride = 0,
                                 int64_t k_token_stride = 0, int64_t v_token_stride = 0) {
    using namespace nckv;
    if ((q_token_stride && (q_token_stride % 8 || q_token_stride < (int64_t)Hq * D)) ||
        (k_token_stride && (k_token_stride % 8 || k_token_stride < (int64_t)Hkv * D)) ||
        (v_token_stride && (v_token_stride % 8 || v_token_stride < (int64_t)Hkv * D))) {
        set_error("append_rope_norm: token strides must be multiples of 8 elements and span a token's heads");
        return NCKV_E_ARG;
    }
    int rc = check_common(k_in, v_in, k_cache, v_cache, cache_seqlens, B, T_new, Hkv, D, T_max,
                          cache_batch_stride, cache_token_stride, status);
    if (rc != NCKV_OK) return rc;
    if (!cos || !sin || rope_len <= 0) {
        set_error("append_rope_norm: cos/sin tables are required");
        return NCKV_E_ARG;
    }
    if (q_in && (!q_out || Hq <= 0 || (Hq % Hkv) != 0)) {
        set_error("append_rope_norm: q given but q_out missing or Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
        return NCKV_E_ARG;
    }
    if (((uintptr_t)cos | (uintptr_t)sin | (uintptr_t)q_in | (uintptr_t)q_out) & 15) {
        set_error("append_rope_norm: tensors must be 16-byte aligned");
        return NCKV_E_ARG;
    }
    AppendParams p;
    p.q_in = static_cast<const uint4 *>(q_in);
    p.k_in = static_cast<const uint4 *>(k_in);
    p.v_in = static_cast<const uint4 *>(v_in);
    p.q_out = static_cast<uint4 *>(q_out);
    p.k_cache = static_cast<__nv_bfloat16 *>(k_cache);
    p.v_cache = static_cast<__nv_bfloat16 *>(v_cache);
    p.cache_seqlens = cache_seqlens;
    p.write_slots = write_slots;
    p.cos = static_cast<const uint4 *>(cos);
    p.sin = static_cast<const uint4 *>(sin);
    p.status = status;
    p.B = B; p.T_new = T_new; p.Hq = Hq; p.Hkv = Hkv; p.T_max = T_max; p.rope_len = rope_len;
    p.cache_batch_stride = cache_batch_stride;
    p.cache_token_stride = cache_token_stride;
    p.qk_scale = qk_scale;
    p.eps = eps;
    p.transform_k = 1;
    p.split = split;
    p.block_table = block_table;
    p.page_tokens = page_tokens; p.max_pages = max_pages; p.n_pages = n_pages;
    p.q_stride = q_token_stride ? q_token_stride / 8 : (long long)Hq * 16;
    p.k_stride = k_token_stride ? k_token_stride / 8 : (long long)Hkv * 16;
    p.v_stride = v_token_stride ? v_token_stride / 8 : (long long)Hkv * 16;
    return launch_append(p, static_cast<cudaStream_t>(stream));
}

int nckv_append_rope_norm_strided(const void *q_in, const void *k_in, const void *v_in, int64_t q_token_stride,
                                  int64_t k_token_stride, int64_t v_token_stride, void *q_out, void *k_cache,
                                  void *v_cache, const int32_t *cache_seqlens, const void *cos, const void *sin, int B,
                                  int T_new, int Hq, int Hkv, int D, int T_max, int64_t cache_batch_stride,
                                  int64_t cache_token_stride, int rope_len, float qk_scale, float eps, int32_t *status,
                                  void *stream) {
    if (((uintptr_t)k_in | (uintptr_t)v_in) & 15) {
        nckv::set_error("append_rope_norm_strided: tensors must be 16-byte aligned");
        return NCKV_E_ARG;
    }
    return append_rope_norm_impl(q_in, k_in, v_in, q_out, k_cache, v_cache, cache_seqlens, nullptr, nckv::KvSplit{0, 0, 0}, cos,
                                 sin, B, T_new, Hq, Hkv, D, T_max, cache_batch_stride, cache_token_stride, rope_len,
                                 qk_scale, eps, status, stream, nullptr, 0, 0, 0, q_token_stride, k_token_stride,
                                 v_token_stride);
}

int nckv_append_rope_norm(const void *q_in, const void *k_in, const void *v_in, void *q_out,
                          void *k_cache, void *v_cache, const int32_t *cache_seqlens,
                          const void *cos, const void *sin, int B, int T_new, int Hq, int Hkv,
                          int D, int T_max, int64_t cache_batch_stride,
                          int64_t cache_token_stride, int rope_len, float qk_scale, float eps,
                          int32_t *status, void *stream) {
    return append_rope_norm_impl(q_in, k_in, v_in, q_out, k_cache, v_cache, cache_seqlens, nullptr, nckv::KvSplit{0, 0, 0}, cos, sin, B, T_new,
                                 Hq, Hkv, D, T_max, cache_batch_stride, cache_token_stride, rope_len, qk_scale, eps,
                                 status, stream);
}

int nckv_append_rope_norm_at(const void *q_in, const void *k_in, const void *v_in, void *q_out,
                             void *k_cache, void *v_cache, const int32_t *positions, const int32_t *write_slots,
                             const void *cos, const void *sin, int B, int T_new, int Hq, int Hkv,
                             int D, int T_max, int64_t cache_batch_stride, int64_t cache_token_stride,
                             int rope_len, float qk_scale, float eps, int32_t *status, void *stream) {
    if (!write_slots) {
        nckv::set_error("append_rope_norm_at: write_slots is required");
        return NCKV_E_ARG;
    }
    return append_rope_norm_impl(q_in, k_in, v_in, q_out, k_cache, v_cache, positions, write_slots, nckv::KvSplit{0, 0, 0}, cos, sin, B, T_new,
                                 Hq, Hkv, D, T_max, cache_batch_stride, cache_token_stride, rope_len, qk_scale, eps,
                                 status, stream);
}

int nckv_append_rope_norm_split(const void *q_in, const void *k_in, const void *v_in, void *q_out,
                                void *k_cache, void *v_cache, const int32_t *cache_seqlens, const void *cos,
                                const void *sin, int B, int T_new, int Hq, int Hkv, int D, int T_local,
                                int64_t cache_batch_stride, int64_t cache_token_stride, int rope_len,
                                float qk_scale, float eps, int world, int rank, int block, int32_t *status,
                                void *stream) {
    if (world <= 0 || rank < 0 || rank >= world || block <= 0 || T_new != 1) {
        nckv::set_error("append_rope_norm_split: bad split (world=%d rank=%d block=%d) or T_new=%d != 1", world, rank,
                        block, T_new);
        return NCKV_E_ARG;
    }
    return append_rope_norm_impl(q_in, k_in, v_in, q_out, k_cache, v_cache, cache_seqlens, nullptr,
                                 nckv::KvSplit{world, rank, block}, cos, sin, B, T_new, Hq, Hkv, D, T_local,
                                 cache_batch_stride, cache_token_stride, rope_len, qk_scale, eps, status, stream);
}

int nckv_append_rope_norm_paged(const void *q_in, const void *k_in, const void *v_in, void *q_out, void *k_pool,
                                void *v_pool, const int32_t *block_table, const int32_t *cache_seqlens,
                                const void *cos, const void *sin, int B, int T_new, int Hq, int Hkv, int D,
                                int page_tokens, int max_pages, int n_pages, int64_t page_stride, int64_t token_stride,
                                int rope_len, float qk_scale, float eps, int32_t *status, void *stream) {
    if (!block_table || page_tokens <= 0 || max_pages <= 0 || n_pages <= 0 ||
        (long long)page_tokens * max_pages > 0x3fffffffLL) {
        nckv::set_error("append_rope_norm_paged: bad paging (page_tokens=%d max_pages=%d n_pages=%d)", page_tokens,
                        max_pages, n_pages);
        return NCKV_E_ARG;
    }
    return append_rope_norm_impl(q_in, k_in, v_in, q_out, k_pool, v_pool, cache_seqlens, nullptr, nckv::KvSplit{0, 0, 0},
                                 cos, sin, B, T_new, Hq, Hkv, D, page_tokens * max_pages, page_stride, token_stride,
                                 rope_len, qk_scale, eps, status, stream, block_table, page_tokens, max_pages, n_pages);
}

int nckv_append(const void *k_in, const void *v_in, void *k_cache, void *v_cache,
                const int32_t *cache_seqlens, int B, int T_new, int Hkv, int D, int T_max,
                int64_t cache_batch_stride, int64_t cache_token_stride, int32_t *status,
                void *stream) {
    using namespace nckv;
    int rc = check_common(k_in, v_in, k_cache, v_cache, cache_seqlens, B, T_new, Hkv, D, T_max,
                          cache_batch_stride, cache_token_stride, status);
    if (rc != NCKV_OK) return rc;
    AppendParams p;
    p.q_in = nullptr;
    p.k_in = static_cast<const uint4 *>(k_in);
    p.v_in = static_cast<const uint4 *>(v_in);
    p.q_out = nullptr;
    p.k_cache = static_cast<__nv_bfloat16 *>(k_cache);
    p.v_cache = static_cast<__nv_bfloat16 *>(v_cache);
    p.cache_seqlens = cache_seqlens;
    p.write_slots = nullptr;
    p.cos = nullptr;
    p.sin = nullptr;
    p.status = status;
    p.B = B; p.T_new = T_new; p.Hq = 0; p.Hkv = Hkv; p.T_max = T_max; p.rope_len = 0;
    p.cache_batch_stride = cache_batch_stride;
    p.cache_token_stride = cache_token_stride;
    p.qk_scale = 1.0f;
    p.eps = 0.0f;
    p.transform_k = 0;
    p.split = KvSplit{0, 0, 0};
    p.block_table = nullptr;
    p.page_tokens = p.max_pages = p.n_pages = 0;
    p.q_stride = 0;
    p.k_stride = p.v_stride = (long long)Hkv * 16;
    return launch_append(p, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
