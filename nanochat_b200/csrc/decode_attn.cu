// Kernel (b): split-KV decode attention (one query token per row), HBM-bandwidth bound.
//
// Work decomposition.  Keys of row b are cut into tiles of DEC_TILE tokens starting at the first
// visible key; the tiles of all (row, kv-head) pairs form one flat sequence (row outer, head
// middle, tile inner).  Every WARP of the persistent grid (one CTA per SM) takes an equal,
// contiguous slice of that sequence, so ragged cache_seqlens balance to within one tile.  A warp
// is a self-contained stream processor: lane 0 issues TMA tile loads (K and V, 128-byte swizzle)
// into the warp's private ring of DEC_STAGES shared-memory stages, completion is signalled on
// the warp's own mbarriers, and the loads run ahead across pair boundaries.  There is no CTA-wide
// synchronisation after set-up.
//
// Math per tile.  All G = Hq/Hkv query heads that share a kv head are the rows of one
// m16n8k16 tile (rows >= G are zero), so K/V bytes are read once per group.  S = Q K^T and
// O += P V use the warp-level bf16 MMA with fp32 accumulation; running max / sum use quad
// shuffles; P is rounded to bf16 for the second product, as the flash-style library kernels do.
//
// Combine.  A pair whose tiles all fall inside one warp's slice is normalised and written
// directly.  Otherwise each warp writes an un-normalised partial (O, m, l) to the workspace and
// bumps the pair's arrival counter; the last warp to arrive merges the partials with a
// log-sum-exp and resets the counter.  Nothing ever waits on another warp.
//
// Replaces: flash_attention.py:83-89 (Tq == 1 branch of _sdpa_attention) reached through
// flash_attention.py:165-177, with the per-row cache_seqlens contract of flash_attention.py:142.
#include <math.h>

#include "nckv_common.cuh"

namespace nckv {

constexpr int DEC_TILE = 32;    // keys per tile
constexpr int DEC_STAGES = 3;   // tiles in flight per warp
constexpr int DEC_WARPS = 4;    // warps (independent streams) per CTA
constexpr int DEC_MAX_B = 1024; // rows per launch (bounds the shared-memory row tables)
constexpr int DEC_HALF_BYTES = DEC_TILE * 128;        // one 64-channel half of a K or V tile
constexpr int DEC_STAGE_BYTES = 4 * DEC_HALF_BYTES;   // K lo, K hi, V lo, V hi
constexpr int DEC_STATUS_BYTES = 256;

struct DecodeParams {
    const __nv_bfloat16 *q;
    const int32_t *seqlens;
    __nv_bfloat16 *out;
    float *out_f32;
    float *lse;
    int32_t *status;
    int32_t *counters;  // one per (row, kv head); zero on entry, zero on exit
    float *partials;    // 2 records per warp of the grid, rec_floats each
    int B, Hq, Hkv, G, T_max;
    int seqlen_offset, window_left, kv_begin, kv_end;
    int rec_floats;
    float scale_log2;
#ifdef NCKV_TIMELINE
    unsigned long long *timeline;  // 8 stamps per warp of the grid (debug builds only)
#endif
};

struct TileCursor {
    int b, h, j, nt;
};

__device__ __forceinline__ void cursor_advance(TileCursor &c, const int *s_pref, int B, int Hkv) {
    if (++c.j < c.nt) return;
    c.j = 0;
    if (++c.h < Hkv) return;
    c.h = 0;
    int b = c.b + 1;
    while (b < B && s_pref[b + 1] == s_pref[b]) ++b;  // skip rows without visible keys
    c.b = b;
    c.nt = b < B ? s_pref[b + 1] - s_pref[b] : 0;
}

// Largest b with Hkv * pref[b] <= x; the row it names always owns tile x.
__device__ __forceinline__ int find_row(const int *s_pref, int B, int Hkv, int x) {
    int lo = 0, hi = B;  // invariant: Hkv*pref[lo] <= x < Hkv*pref[hi]
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (Hkv * s_pref[mid] <= x) lo = mid; else hi = mid;
    }
    return lo;
}

template <bool GHI>  // GHI: group size 9..16 (rows 8..15 of the MMA tile carry heads too)
__global__ void __launch_bounds__(DEC_WARPS * 32, 1)
decode_attn_kernel(const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const DecodeParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits 4..9
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint8_t *stages = smem;  // [DEC_WARPS][DEC_STAGES][DEC_STAGE_BYTES]
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(stages + DEC_WARPS * DEC_STAGES * DEC_STAGE_BYTES);
    int *s_start = reinterpret_cast<int *>(full_bar + DEC_WARPS * DEC_STAGES);
    int *s_end = s_start + DEC_MAX_B;
    int *s_pref = s_end + DEC_MAX_B;  // B + 1 entries

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int B = p.B, Hkv = p.Hkv, G = p.G;
#ifdef NCKV_TIMELINE
    unsigned long long *tl = p.timeline + ((long long)blockIdx.x * DEC_WARPS + warp) * 8;
    unsigned long long tl_fin = 0;
#define TL_STAMP(i) do { if (lane == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); tl[i] = t_; } } while (0)
#define TL_NOW(v) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v))
    TL_STAMP(0);
#else
#define TL_STAMP(i)
#endif

    // ---- set-up: per-row visible key range and tile counts --------------------------------
    for (int b = tid; b < B; b += blockDim.x) {
        int n = p.seqlens[b] + p.seqlen_offset;
        if (n < 0) {
            if (blockIdx.x == 0) atomicOr(p.status, (int)NCKV_ST_BAD_SEQLEN);
            n = 0;
        }
        if (n > p.T_max) {
            if (blockIdx.x == 0) atomicOr(p.status, (int)NCKV_ST_OVERFLOW);
            n = p.T_max;
        }
        int lo = 0, hi = n;
        if (p.window_left >= 0) lo = max(0, n - 1 - p.window_left);
        if (p.kv_end > p.kv_begin) {
            lo = max(lo, p.kv_begin);
            hi = min(hi, p.kv_end);
        }
        if (hi < lo) hi = lo;
        s_start[b] = lo;
        s_end[b] = hi;
    }
    if (tid == 0) {
        for (int i = 0; i < DEC_WARPS * DEC_STAGES; ++i) mbar_init(&full_bar[i], 1);
        fence_mbar_init();
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
    }
    __syncthreads();
    if (warp == 0) {  // exclusive prefix sum of tiles per row
        const int per = (B + 31) / 32;
        const int b0 = lane * per;
        int local = 0;
        for (int i = 0; i < per; ++i) {
            int b = b0 + i;
            if (b < B) local += (s_end[b] - s_start[b] + DEC_TILE - 1) / DEC_TILE;
        }
        int incl = local;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            int v = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += v;
        }
        int run = incl - local;
        for (int i = 0; i < per; ++i) {
            int b = b0 + i;
            if (b < B) {
                s_pref[b] = run;
                run += (s_end[b] - s_start[b] + DEC_TILE - 1) / DEC_TILE;
            }
        }
        if (lane == 31) s_pref[B] = incl;
    }
    __syncthreads();

    // rows without any visible key: zero output, lse = -inf (only sharded calls can produce them)
    for (int b = blockIdx.x; b < B; b += gridDim.x) {
        if (s_pref[b + 1] != s_pref[b]) continue;
        for (int i = tid; i < p.Hq * NCKV_D; i += blockDim.x) {
            const long long o = (long long)b * p.Hq * NCKV_D + i;
            p.out[o] = __float2bfloat16(0.0f);
            if (p.out_f32) p.out_f32[o] = 0.0f;
        }
        if (p.lse) for (int i = tid; i < p.Hq; i += blockDim.x) p.lse[(long long)b * p.Hq + i] = -INFINITY;
    }

    TL_STAMP(1);
    // Slices: with q = total / W and r = total % W, warp w owns q + (w < r) consecutive tiles
    // starting at w*q + min(w, r).  Everything is 32-bit (the host bounds total below 2^31).
    const int total = Hkv * s_pref[B];
    if (total == 0) return;
    const int W = gridDim.x * DEC_WARPS;
    const int gw = blockIdx.x * DEC_WARPS + warp;
    const int sl_q = total / W, sl_r = total % W;
    const int lo_tile = gw * sl_q + min(gw, sl_r);
    const int n_my = sl_q + (gw < sl_r ? 1 : 0);
    if (n_my == 0) return;
    auto slice_lo = [&](int w) { return w * sl_q + min(w, sl_r); };
    auto warp_of = [&](int x) {  // the warp whose slice holds tile x
        const int big = sl_r * (sl_q + 1);
        return x < big ? x / (sl_q + 1) : sl_r + (x - big) / sl_q;
    };

    uint8_t *my_stages = stages + warp * DEC_STAGES * DEC_STAGE_BYTES;
    uint64_t *my_bar = full_bar + warp * DEC_STAGES;

    TileCursor cons;
    cons.b = find_row(s_pref, B, Hkv, lo_tile);
    cons.nt = s_pref[cons.b + 1] - s_pref[cons.b];
    {
        const int rel = lo_tile - Hkv * s_pref[cons.b];
        cons.h = rel / cons.nt;
        cons.j = rel - cons.h * cons.nt;
    }
    TileCursor prod = cons;

    auto issue_tile = [&](const TileCursor &c, int stage) {
        // lane 0 only
        uint8_t *dst = my_stages + stage * DEC_STAGE_BYTES;
        uint64_t *bar = &my_bar[stage];
        const int key0 = s_start[c.b] + c.j * DEC_TILE;
        fence_proxy_async_smem();
        mbar_arrive_expect_tx(bar, DEC_STAGE_BYTES);
        tma_load_4d(dst, &tmap_k, bar, 0, c.h, key0, c.b);
        tma_load_4d(dst + DEC_HALF_BYTES, &tmap_k, bar, 64, c.h, key0, c.b);
        tma_load_4d(dst + 2 * DEC_HALF_BYTES, &tmap_v, bar, 0, c.h, key0, c.b);
        tma_load_4d(dst + 3 * DEC_HALF_BYTES, &tmap_v, bar, 64, c.h, key0, c.b);
    };

    int issued = 0;
    for (; issued < DEC_STAGES && issued < n_my; ++issued) {
        if (lane == 0) issue_tile(prod, issued);
        cursor_advance(prod, s_pref, B, Hkv);
    }

    TL_STAMP(2);
    const int g = lane >> 2;  // MMA row within 8 (query head within the group)
    const int t4 = lane & 3;
    uint32_t qa[8][GHI ? 4 : 2];  // A fragments of Q for the 8 k-steps over D
    float o_acc[16][4];
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};
    int seg_j0 = 0;
    bool timed_out = false;
    int pend0 = 0, pend1 = 0, n_pend = 0;  // pairs whose partial record awaits its arrival (at most 2 per slice)
#ifdef NCKV_TIMELINE
    unsigned long long tf0s = 0;
#endif

    for (int it = 0; it < n_my; ++it) {
        const int stage = it % DEC_STAGES;
        const uint32_t parity = (uint32_t)((it / DEC_STAGES) & 1);
        const bool seg_begin = (it == 0) || (cons.j == 0);
        if (seg_begin) {
            seg_j0 = cons.j;
            m_run[0] = m_run[1] = -INFINITY;
            l_run[0] = l_run[1] = 0.f;
#pragma unroll
            for (int nd = 0; nd < 16; ++nd)
                o_acc[nd][0] = o_acc[nd][1] = o_acc[nd][2] = o_acc[nd][3] = 0.f;
            const __nv_bfloat16 *qrow = p.q + ((long long)cons.b * p.Hq + (long long)cons.h * G) * NCKV_D;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                const uint32_t *r0 = reinterpret_cast<const uint32_t *>(qrow + (long long)g * NCKV_D + kk * 16 + 2 * t4);
                qa[kk][0] = g < G ? __ldg(r0) : 0u;
                qa[kk][1] = g < G ? __ldg(r0 + 4) : 0u;
                if (GHI) {
                    const uint32_t *r1 = reinterpret_cast<const uint32_t *>(qrow + (long long)(g + 8) * NCKV_D + kk * 16 + 2 * t4);
                    qa[kk][2] = (g + 8) < G ? __ldg(r1) : 0u;
                    qa[kk][3] = (g + 8) < G ? __ldg(r1 + 4) : 0u;
                }
            }
        }

        if (!mbar_wait_bounded(&my_bar[stage], parity)) {
            timed_out = true;
            break;
        }

#ifdef NCKV_TIMELINE
        if (it == 0) TL_STAMP(3);
#endif
        const uint32_t kbase = smem_u32(my_stages + stage * DEC_STAGE_BYTES);
        const uint32_t vbase = kbase + 2 * DEC_HALF_BYTES;
        const int key0 = s_start[cons.b] + cons.j * DEC_TILE;
        const int nvalid = min(DEC_TILE, s_end[cons.b] - key0);

        if (nvalid < DEC_TILE) {
            // Tail tile: rows past the last visible key may hold stale bytes; zero V there so a
            // zero probability never meets a NaN/Inf bit pattern.
            uint8_t *vb = my_stages + stage * DEC_STAGE_BYTES + 2 * DEC_HALF_BYTES;
            if (lane < 16) {
                for (int r = nvalid; r < DEC_TILE; ++r)
                    *reinterpret_cast<uint4 *>(vb + (lane >> 3) * DEC_HALF_BYTES + r * 128 + (lane & 7) * 16) =
                        make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }

        // ---- S = Q K^T  (16 x DEC_TILE) ----
        float s_acc[DEC_TILE / 8][4];
#pragma unroll
        for (int nb = 0; nb < DEC_TILE / 8; ++nb) {
            s_acc[nb][0] = s_acc[nb][1] = s_acc[nb][2] = s_acc[nb][3] = 0.f;
            const int r = nb * 8 + (lane & 7);
#pragma unroll
            for (int kk = 0; kk < 8; kk += 2) {
                const int c = 2 * kk + (lane >> 3);
                const uint32_t addr = kbase + (c >> 3) * DEC_HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, addr);
                if (GHI) {
                    mma_bf16_16816(s_acc[nb][0], s_acc[nb][1], s_acc[nb][2], s_acc[nb][3],
                                   qa[kk][0], qa[kk][GHI ? 2 : 0], qa[kk][1], qa[kk][GHI ? 3 : 1], b0, b1);
                    mma_bf16_16816(s_acc[nb][0], s_acc[nb][1], s_acc[nb][2], s_acc[nb][3],
                                   qa[kk + 1][0], qa[kk + 1][GHI ? 2 : 0], qa[kk + 1][1], qa[kk + 1][GHI ? 3 : 1], b2, b3);
                } else {
                    mma_bf16_16816(s_acc[nb][0], s_acc[nb][1], s_acc[nb][2], s_acc[nb][3],
                                   qa[kk][0], 0u, qa[kk][1], 0u, b0, b1);
                    mma_bf16_16816(s_acc[nb][0], s_acc[nb][1], s_acc[nb][2], s_acc[nb][3],
                                   qa[kk + 1][0], 0u, qa[kk + 1][1], 0u, b2, b3);
                }
            }
        }

        // ---- mask the tail, online softmax (rows g and g+8) ----
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < DEC_TILE / 8; ++nb) {
            const int k0 = nb * 8 + 2 * t4;
            if (k0 >= nvalid) { s_acc[nb][0] = -INFINITY; s_acc[nb][2] = -INFINITY; }
            if (k0 + 1 >= nvalid) { s_acc[nb][1] = -INFINITY; s_acc[nb][3] = -INFINITY; }
            mx0 = fmaxf(mx0, fmaxf(s_acc[nb][0], s_acc[nb][1]));
            if (GHI) mx1 = fmaxf(mx1, fmaxf(s_acc[nb][2], s_acc[nb][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        if (GHI) {
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        }
        const float mn0 = fmaxf(m_run[0], mx0 * p.scale_log2);
        const float mn1 = GHI ? fmaxf(m_run[1], mx1 * p.scale_log2) : 0.f;
        const float alpha0 = exp2f(m_run[0] - mn0);  // first tile: exp2(-inf) = 0
        const float alpha1 = GHI ? exp2f(m_run[1] - mn1) : 0.f;
        m_run[0] = mn0;
        if (GHI) m_run[1] = mn1;
        float rs0 = 0.f, rs1 = 0.f;
        uint32_t pa[DEC_TILE / 8][2];
#pragma unroll
        for (int nb = 0; nb < DEC_TILE / 8; ++nb) {
            const float p0 = exp2f(fmaf(s_acc[nb][0], p.scale_log2, -mn0));
            const float p1 = exp2f(fmaf(s_acc[nb][1], p.scale_log2, -mn0));
            rs0 += p0 + p1;
            pa[nb][0] = pack_bf16x2(p0, p1);
            if (GHI) {
                const float p2 = exp2f(fmaf(s_acc[nb][2], p.scale_log2, -mn1));
                const float p3 = exp2f(fmaf(s_acc[nb][3], p.scale_log2, -mn1));
                rs1 += p2 + p3;
                pa[nb][1] = pack_bf16x2(p2, p3);
            } else {
                pa[nb][1] = 0u;
            }
        }
        l_run[0] = l_run[0] * alpha0 + rs0;  // per-lane partial sums; reduced over the quad at the end
        if (GHI) l_run[1] = l_run[1] * alpha1 + rs1;
#pragma unroll
        for (int nd = 0; nd < 16; ++nd) {
            o_acc[nd][0] *= alpha0;
            o_acc[nd][1] *= alpha0;
            if (GHI) { o_acc[nd][2] *= alpha1; o_acc[nd][3] *= alpha1; }
        }

        // ---- O += P V  (16 x 128) ----
#pragma unroll
        for (int ks = 0; ks < DEC_TILE / 16; ++ks) {
            const int r = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
            for (int nd = 0; nd < 16; nd += 2) {
                const int c = nd + (lane >> 4);
                const uint32_t addr = vbase + (c >> 3) * DEC_HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3, addr);
                mma_bf16_16816(o_acc[nd][0], o_acc[nd][1], o_acc[nd][2], o_acc[nd][3],
                               pa[2 * ks][0], pa[2 * ks][1], pa[2 * ks + 1][0], pa[2 * ks + 1][1], b0, b1);
                mma_bf16_16816(o_acc[nd + 1][0], o_acc[nd + 1][1], o_acc[nd + 1][2], o_acc[nd + 1][3],
                               pa[2 * ks][0], pa[2 * ks][1], pa[2 * ks + 1][0], pa[2 * ks + 1][1], b2, b3);
            }
        }

        // ---- this stage is free again: fetch the tile DEC_STAGES ahead ----
        __syncwarp();
        if (issued < n_my) {
            if (lane == 0) issue_tile(prod, stage);
            cursor_advance(prod, s_pref, B, Hkv);
            ++issued;
        }

        // ---- end of this pair's run inside my slice? ----
        const bool seg_end = (it == n_my - 1) || (cons.j == cons.nt - 1);
        if (seg_end) {
#ifdef NCKV_TIMELINE
            TL_NOW(tf0s);
            if (it == n_my - 1) TL_STAMP(4);
#endif
            float l0 = l_run[0], l1 = l_run[1];
            l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
            l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
            if (GHI) {
                l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
                l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
            }
            const bool complete = (seg_j0 == 0) && (cons.j == cons.nt - 1);
            const long long row_base = (long long)cons.b * p.Hq + (long long)cons.h * G;
            if (complete) {
                const float inv0 = 1.f / l0;
                const float inv1 = GHI ? 1.f / l1 : 0.f;
#pragma unroll
                for (int nd = 0; nd < 16; ++nd) {
                    const int d = nd * 8 + 2 * t4;
                    if (g < G) {
                        const long long o = (row_base + g) * NCKV_D + d;
                        const float v0 = o_acc[nd][0] * inv0, v1 = o_acc[nd][1] * inv0;
                        *reinterpret_cast<uint32_t *>(p.out + o) = pack_bf16x2(v0, v1);
                        if (p.out_f32) *reinterpret_cast<float2 *>(p.out_f32 + o) = make_float2(v0, v1);
                    }
                    if (GHI && g + 8 < G) {
                        const long long o = (row_base + g + 8) * NCKV_D + d;
                        const float v0 = o_acc[nd][2] * inv1, v1 = o_acc[nd][3] * inv1;
                        *reinterpret_cast<uint32_t *>(p.out + o) = pack_bf16x2(v0, v1);
                        if (p.out_f32) *reinterpret_cast<float2 *>(p.out_f32 + o) = make_float2(v0, v1);
                    }
                }
                if (p.lse && t4 == 0) {
                    if (g < G) p.lse[row_base + g] = (m_run[0] + log2f(l0)) * 0.69314718055994531f;
                    if (GHI && g + 8 < G) p.lse[row_base + g + 8] = (m_run[1] + log2f(l1)) * 0.69314718055994531f;
                }
            } else {
                // partial record: [G][128] un-normalised O, then m[G], l[G].  The arrival on the
                // pair's counter is deferred to the end of this warp's slice, so that no fence sits
                // in the middle of the tile stream.
                const int slot = 2 * gw + (seg_j0 == 0 ? 1 : 0);
                float *rec = p.partials + (long long)slot * p.rec_floats;
#pragma unroll
                for (int nd = 0; nd < 16; ++nd) {
                    const int d = nd * 8 + 2 * t4;
                    if (g < G) __stcg(reinterpret_cast<float2 *>(rec + g * NCKV_D + d), make_float2(o_acc[nd][0], o_acc[nd][1]));
                    if (GHI && g + 8 < G)
                        __stcg(reinterpret_cast<float2 *>(rec + (g + 8) * NCKV_D + d), make_float2(o_acc[nd][2], o_acc[nd][3]));
                }
                if (t4 == 0) {
                    if (g < G) { __stcg(rec + G * NCKV_D + g, m_run[0]); __stcg(rec + G * NCKV_D + G + g, l0); }
                    if (GHI && g + 8 < G) { __stcg(rec + G * NCKV_D + g + 8, m_run[1]); __stcg(rec + G * NCKV_D + G + g + 8, l1); }
                }
                if (n_pend == 0) pend0 = cons.b * Hkv + cons.h; else pend1 = cons.b * Hkv + cons.h;
                ++n_pend;
            }
#ifdef NCKV_TIMELINE
            { unsigned long long tf1; TL_NOW(tf1); tl_fin += tf1 - tf0s; }
#endif
        }
        cursor_advance(cons, s_pref, B, Hkv);
    }
#ifdef NCKV_TIMELINE
    unsigned long long tf2; TL_NOW(tf2);
#endif
    // ---- deferred arrivals: publish my partial records, merge the pairs I complete ---------------
    if (n_pend > 0 && !timed_out) {
        __syncwarp();
        if (lane == 0) __threadfence();  // cumulative: orders the whole warp's record stores (after the barrier)
        __syncwarp();
        for (int e = 0; e < n_pend; ++e) {
            const int pair = e == 0 ? pend0 : pend1;
            const int pb = pair / Hkv, ph = pair - pb * Hkv;
            const int nt = s_pref[pb + 1] - s_pref[pb];
            const int P0 = Hkv * s_pref[pb] + ph * nt;
            const int w_first = warp_of(P0), w_last = warp_of(P0 + nt - 1);
            const int nparts = w_last - w_first + 1;  // non-empty slices are contiguous in w
            int old = 0;
            if (lane == 0) old = atomicAdd(&p.counters[pair], 1);
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old != nparts - 1) continue;
            // last arriver: log-sum-exp merge.  Lane i looks after parts i, i+32, ...; for the
            // O rows every lane owns channels 4*lane .. 4*lane+3.
            __threadfence();
            const long long row_base = (long long)pb * p.Hq + (long long)ph * G;
            for (int hg = 0; hg < G; ++hg) {
                float mloc = -INFINITY;
                for (int i = lane; i < nparts; i += 32) {
                    const int w = w_first + i;
                    const float *r2 = p.partials + (long long)(2 * w + (slice_lo(w) <= P0 ? 1 : 0)) * p.rec_floats;
                    mloc = fmaxf(mloc, __ldcg(r2 + G * NCKV_D + hg));
                }
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, off));
                const float M = mloc;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                float Lloc = 0.f;
                for (int base = 0; base < nparts; base += 32) {
                    const int i = base + lane;
                    float sc = 0.f;
                    int my_slot = 0;
                    if (i < nparts) {
                        const int w = w_first + i;
                        my_slot = 2 * w + (slice_lo(w) <= P0 ? 1 : 0);
                        const float *r2 = p.partials + (long long)my_slot * p.rec_floats;
                        sc = exp2f(__ldcg(r2 + G * NCKV_D + hg) - M);
                        Lloc += sc * __ldcg(r2 + G * NCKV_D + G + hg);
                    }
                    const int cnt = min(32, nparts - base);
#pragma unroll 4
                    for (int jn = 0; jn < cnt; ++jn) {
                        const float s_j = __shfl_sync(0xffffffffu, sc, jn);
                        const int slot_j = __shfl_sync(0xffffffffu, my_slot, jn);
                        const float4 v = __ldcg(reinterpret_cast<const float4 *>(p.partials + (long long)slot_j * p.rec_floats + hg * NCKV_D) + lane);
                        acc.x = fmaf(s_j, v.x, acc.x); acc.y = fmaf(s_j, v.y, acc.y);
                        acc.z = fmaf(s_j, v.z, acc.z); acc.w = fmaf(s_j, v.w, acc.w);
                    }
                }
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) Lloc += __shfl_xor_sync(0xffffffffu, Lloc, off);
                const float inv = 1.f / Lloc;
                acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
                const long long o = (row_base + hg) * NCKV_D + lane * 4;
                uint2 packed;
                packed.x = pack_bf16x2(acc.x, acc.y);
                packed.y = pack_bf16x2(acc.z, acc.w);
                *reinterpret_cast<uint2 *>(p.out + o) = packed;
                if (p.out_f32) *reinterpret_cast<float4 *>(p.out_f32 + o) = acc;
                if (p.lse && lane == 0) p.lse[row_base + hg] = (M + log2f(Lloc)) * 0.69314718055994531f;
            }
            if (lane == 0) p.counters[pair] = 0;
        }
    }
    TL_STAMP(5);
#ifdef NCKV_TIMELINE
    if (lane == 0) { unsigned long long tf3; TL_NOW(tf3); tl[6] = tl_fin + (tf3 - tf2); tl[7] = (unsigned long long)n_my; }
#endif

    if (timed_out) {
        if (lane == 0) atomicOr(p.status, (int)NCKV_ST_TIMEOUT);
        // give copies already issued a bounded chance to land before the CTA's memory is released
        for (int s = 0; s < DEC_STAGES; ++s) mbar_wait_bounded(&my_bar[s], 0, 1u << 12);
    }
}

static size_t decode_smem_bytes() {
    return 1024 + (size_t)DEC_WARPS * DEC_STAGES * DEC_STAGE_BYTES + DEC_WARPS * DEC_STAGES * sizeof(uint64_t) +
           (3 * DEC_MAX_B + 4) * sizeof(int);
}

// Workspace layout: [0,256) status; counters (B*Hkv int32, rounded to 256 B); partial records.
static size_t ws_counter_bytes(int B, int Hkv) { return (((size_t)B * Hkv * 4) + 255) & ~(size_t)255; }
// One partial record: [G][128] fp32 O, then m[G] and l[G], padded so records stay 16-byte aligned.
static int rec_floats_for(int G) { return G * NCKV_D + ((2 * G + 3) & ~3); }
static size_t ws_partial_bytes(int G) {
    return (size_t)2 * sm_count() * DEC_WARPS * (size_t)rec_floats_for(G) * sizeof(float);
}

#ifdef NCKV_TIMELINE
static unsigned long long *g_timeline = nullptr;
#endif

}  // namespace nckv

extern "C" {

#ifdef NCKV_TIMELINE
NCKV_API void nckv_debug_set_timeline(void *ptr) { nckv::g_timeline = static_cast<unsigned long long *>(ptr); }
#endif

size_t nckv_workspace_bytes(int B, int Hq, int Hkv, int D) {
    using namespace nckv;
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || D != NCKV_D || Hq % Hkv) return 0;
    return DEC_STATUS_BYTES + ws_counter_bytes(B, Hkv) + ws_partial_bytes(Hq / Hkv);
}

int nckv_decode_attn(const void *q, const void *k_cache, const void *v_cache,
                     const int32_t *cache_seqlens, void *out, float *out_f32, float *lse_out,
                     int B, int Hq, int Hkv, int D, int T_max, int64_t cache_batch_stride,
                     int64_t cache_token_stride, int seqlen_offset, int window_left,
                     int kv_begin, int kv_end, void *workspace, size_t workspace_bytes,
                     void *stream) {
    using namespace nckv;
    if (!q || !k_cache || !v_cache || !cache_seqlens || !out || !workspace) {
        set_error("decode_attn: null pointer argument");
        return NCKV_E_ARG;
    }
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || T_max <= 0) {
        set_error("decode_attn: non-positive size (B=%d Hq=%d Hkv=%d T_max=%d)", B, Hq, Hkv, T_max);
        return NCKV_E_ARG;
    }
    if (D != NCKV_D) {
        set_error("decode_attn: head_dim %d unsupported (kernels are built for 128)", D);
        return NCKV_E_UNSUPPORTED;
    }
    if (Hq % Hkv != 0 || Hq / Hkv > 16) {
        set_error("decode_attn: Hq=%d must be a multiple of Hkv=%d with group size <= 16", Hq, Hkv);
        return NCKV_E_UNSUPPORTED;
    }
    if (B > DEC_MAX_B) {
        set_error("decode_attn: B=%d exceeds %d rows per launch", B, DEC_MAX_B);
        return NCKV_E_UNSUPPORTED;
    }
    if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)out_f32 | (uintptr_t)workspace) & 15) {
        set_error("decode_attn: q/out/workspace must be 16-byte aligned");
        return NCKV_E_ARG;
    }
    if ((long long)B * Hkv * ((T_max + DEC_TILE - 1) / DEC_TILE) >= (1LL << 31) / (sm_count() * DEC_WARPS)) {
        set_error("decode_attn: B*Hkv*T_max too large for 32-bit tile arithmetic");
        return NCKV_E_UNSUPPORTED;
    }
    const size_t need = nckv_workspace_bytes(B, Hq, Hkv, D);
    if (workspace_bytes < need) {
        set_error("decode_attn: workspace of %zu bytes given, %zu needed", workspace_bytes, need);
        return NCKV_E_CAPACITY;
    }
    const int G = Hq / Hkv;
    CUtensorMap mk, mv;
    int rc = make_kv_tensor_map(&mk, k_cache, B, T_max, Hkv, cache_batch_stride, cache_token_stride, DEC_TILE);
    if (rc != NCKV_OK) return rc;
    rc = make_kv_tensor_map(&mv, v_cache, B, T_max, Hkv, cache_batch_stride, cache_token_stride, DEC_TILE);
    if (rc != NCKV_OK) return rc;

    uint8_t *ws = static_cast<uint8_t *>(workspace);
    DecodeParams p;
    p.q = static_cast<const __nv_bfloat16 *>(q);
    p.seqlens = cache_seqlens;
    p.out = static_cast<__nv_bfloat16 *>(out);
    p.out_f32 = out_f32;
    p.lse = lse_out;
    p.status = reinterpret_cast<int32_t *>(ws);
    p.counters = reinterpret_cast<int32_t *>(ws + DEC_STATUS_BYTES);
    p.partials = reinterpret_cast<float *>(ws + DEC_STATUS_BYTES + ws_counter_bytes(B, Hkv));
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.T_max = T_max;
    p.seqlen_offset = seqlen_offset;
    p.window_left = window_left;
    p.kv_begin = kv_begin;
    p.kv_end = kv_end;
    p.rec_floats = rec_floats_for(G);
    p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)D));
#ifdef NCKV_TIMELINE
    p.timeline = g_timeline;
#endif

    const size_t smem = decode_smem_bytes();
    static bool attr_set[64][2] = {{false}};
    int dev = 0;
    NCKV_CUDA_CHECK(cudaGetDevice(&dev));
    const bool ghi = G > 8;
    if (dev < 64 && !attr_set[dev][ghi]) {
        if (ghi)
            NCKV_CUDA_CHECK(cudaFuncSetAttribute(decode_attn_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        else
            NCKV_CUDA_CHECK(cudaFuncSetAttribute(decode_attn_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev][ghi] = true;
    }
    const int grid = sm_count();
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (ghi)
        decode_attn_kernel<true><<<grid, DEC_WARPS * 32, smem, s>>>(mk, mv, p);
    else
        decode_attn_kernel<false><<<grid, DEC_WARPS * 32, smem, s>>>(mk, mv, p);
    NCKV_CUDA_CHECK(cudaGetLastError());
    return NCKV_OK;
}

}  // extern "C"
