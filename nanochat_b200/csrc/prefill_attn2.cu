// Kernel (d): dense causal attention for T_new >= 1 query tokens per row (prefill, chunked prefill,
// flash_attn_func) on the 5th-generation tensor cores: tcgen05.mma with Q, K, V in shared memory
// (TMA, 128-byte swizzle), the scores, the probabilities and the accumulators in tensor memory.
//
// Work item = 256 consecutive query tokens of one (row, q head): two query tiles Q0, Q1 of 128 rows
// that walk the same key tiles of 128 keys, so every K and V tile that reaches shared memory feeds
// two score products and two P V products.  One persistent CTA per SM takes items c, c + grid, ...
// of a list ordered longest first inside groups of (row, head) pairs whose K/V fit in L2 together
// (causal tiles differ in length by the number of query tiles; the order bounds the tail).
//
// Tensor memory (all 512 columns): S0 [0,128)  S1 [128,256)  O0 [256,384)  O1 [384,512); P_i is
// written as packed bf16 over the first 64 columns of S_i.
// Warps: 0-3 softmax of Q0, 4-7 softmax of Q1 (thread r owns query row r = TMEM lane r), 8 issues the
// MMAs, 9 issues the TMA copies; mbarriers only, no CTA-wide barrier after set-up.
// The MMA thread's instruction stream, key tile j ("period" j):
//     PV_0(j)  S_0(j+1)  commit->s_full[0]     PV_1(j)  S_1(j+1)  commit->s_full[1]     commit->rel
// so while softmax group 0 works on S_0(j+1) the tensor pipe runs PV_1(j), S_1(j+1) and vice versa.
// Products issued by one thread execute in order: S_i(j+1) may overwrite the columns P_i(j) was read
// from, and the commit behind S_i(j+1) also tells that PV_i(j) has completed (O_i is quiescent while
// group i handles tile j+1, which is when it may rescale it).  The item stream is flattened: the
// first score products of the next item follow the last P V of the current one, and its Q/K/V are
// requested as soon as the stages they land in are free.
// Softmax: two passes over the 128 scores of a row in TMEM (max, then exp2 + pack), the running max is
// followed lazily (raised, and O rescaled, only when the true max has grown by more than 2^8).
// Every barrier wait is bounded; a wait that runs out sets NCKV_ST_TIMEOUT, the CTA stops issuing
// work, frees its TMEM and returns.
//
// Replaces: the full-causal and explicit-mask branches of _sdpa_attention
// (flash_attention.py:79-80, 92-102) reached from flash_attn_with_kvcache
// (flash_attention.py:165-177) and flash_attn_func (flash_attention.py:107-128).
#include <math.h>

#include "nckv_common.cuh"
#include "tc05.cuh"

namespace nckv {

constexpr int P2_M = 128;                  // rows of a query tile
constexpr int P2_N = 128;                  // keys of a tile
constexpr int P2_KST = 3;                  // K stages
constexpr int P2_VST = 2;                  // V stages
constexpr int P2_SOFTMAX_THREADS = 256;    // two groups of 128
constexpr int P2_THREADS = P2_SOFTMAX_THREADS + 64;
constexpr int P2_Q_BYTES = P2_M * NCKV_D * 2;   // 32 KB per query tile: two 64-channel halves of [128][128 B]
constexpr int P2_KV_BYTES = P2_N * NCKV_D * 2;  // 32 KB per K or V tile
constexpr int P2_TMEM_COLS = 512;
constexpr unsigned long long P2_WAIT_LIMIT = NCKV_WAIT_LIMIT_NS;

struct Prefill2Params {
    const int32_t *seqlens;  // may be null (all zero)
    __nv_bfloat16 *out;
    int32_t *status;
    int B, T_new, Hq, Hkv, T_k;
    int window_left;
    int n_items, n_qpairs, group_pairs;
    float scale_log2;
};

// Everything a role needs to know about one work item; computed identically by every warp.
struct ItemPlan {
    int b, hq, hkv, t0, L;
    int base;         // first key of tile 0
    int jb[2], je[2]; // tiles [jb, je) are the ones query tile i looks at (je == jb: none)
    int kv_hi[2];     // keys at or beyond this position are invisible to every row of tile i
    int n;            // key tiles of the item = max(je)
};

__device__ __forceinline__ ItemPlan plan_item(const Prefill2Params &p, int item) {
    ItemPlan it;
    const int n_pairs = p.Hq * p.B;
    const int per_group = p.group_pairs * p.n_qpairs;
    const int grp = item / per_group;
    const int in_grp = item - grp * per_group;
    const int grp_pairs = min(p.group_pairs, n_pairs - grp * p.group_pairs);
    const int qp = p.n_qpairs - 1 - in_grp / grp_pairs;  // long items first
    const int pair = grp * p.group_pairs + in_grp % grp_pairs;
    it.hq = pair % p.Hq;
    it.b = pair / p.Hq;
    it.hkv = it.hq / (p.Hq / p.Hkv);
    it.t0 = qp * 2 * P2_M;
    int L = p.seqlens ? p.seqlens[it.b] : 0;
    if (L < 0) L = 0;  // reported once, by the set-up code
    it.L = L;
    int Tk = L + p.T_new;
    if (Tk > p.T_k) Tk = p.T_k;
    int lo0 = 0;
    it.n = 0;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r0 = it.t0 + i * P2_M;
        it.jb[i] = it.je[i] = 0;
        it.kv_hi[i] = 0;
        if (r0 >= p.T_new) continue;
        const int last_t = min(r0 + P2_M, p.T_new) - 1;
        const int hi = min(Tk, L + last_t + 1);
        const int lo = p.window_left >= 0 ? max(0, L + r0 - p.window_left) : 0;
        if (i == 0) lo0 = lo;
        it.kv_hi[i] = hi;
        if (hi > lo) {
            it.jb[i] = (lo - lo0) / P2_N;
            it.je[i] = (hi - lo0 + P2_N - 1) / P2_N;
        }
        it.n = max(it.n, it.je[i]);
    }
    it.base = lo0;
    return it;
}

__global__ void __launch_bounds__(P2_THREADS, 1)
prefill_attn2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const Prefill2Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0) {  // uniform; checked rather than assumed
        if (threadIdx.x == 0) atomicOr(p.status, (int)NCKV_ST_TIMEOUT);
        return;
    }
    uint8_t *sQ = smem;                                  // 2 x 32 KB
    uint8_t *sK = sQ + 2 * P2_Q_BYTES;                   // 3 x 32 KB
    uint8_t *sV = sK + P2_KST * P2_KV_BYTES;             // 2 x 32 KB
    uint64_t *bars = reinterpret_cast<uint64_t *>(sV + P2_VST * P2_KV_BYTES);
    uint64_t *bar_q = bars;            // Q0 and Q1 of an item landed
    uint64_t *bar_k = bars + 1;        // [3] K tile landed
    uint64_t *bar_v = bars + 4;        // [2] V tile landed
    uint64_t *bar_s = bars + 6;        // [2] S_i of a tile complete (and every product issued before it)
    uint64_t *bar_o = bars + 8;        // [2] last P V of an item for query tile i complete
    uint64_t *bar_p = bars + 10;       // [2] P_i of a tile is in TMEM (4 arrivals: one per warp of the group)
    uint64_t *bar_rel = bars + 12;     // [2] every product of a period complete (period g on bar_rel[g & 1])
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 14);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    pdl_wait_prior_grids();
    if (tid == 0) {
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
        mbar_init(bar_q, 1);
        for (int s = 0; s < P2_KST; ++s) mbar_init(&bar_k[s], 1);
        for (int s = 0; s < P2_VST; ++s) mbar_init(&bar_v[s], 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar_s[i], 1);
            mbar_init(&bar_o[i], 1);
            mbar_init(&bar_p[i], P2_M / 32);
            mbar_init(&bar_rel[i], 1);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (blockIdx.x == 0 && p.seqlens) {  // lengths out of range: reported once
        for (int b = tid; b < p.B; b += blockDim.x) {
            const int L = p.seqlens[b];
            if (L < 0) atomicOr(p.status, (int)NCKV_ST_BAD_SEQLEN);
            else if (L + p.T_new > p.T_k) atomicOr(p.status, (int)NCKV_ST_OVERFLOW);
        }
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, P2_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    constexpr uint32_t IDESC_S = umma_idesc(P2_M, P2_N, 0, 0);
    constexpr uint32_t IDESC_O = umma_idesc(P2_M, NCKV_D, 0, 1);
    auto timed_out = [&]() {
        *abort_flag = 1;
        atomicOr(p.status, (int)NCKV_ST_TIMEOUT);
    };

    if (warp == P2_SOFTMAX_THREADS / 32 + 1) {
        // =============== one lane moves the tiles ===================================================
        if (lane == 0) {
            long long g0 = 0;        // global index of the item's tile 0 (= of its period 0)
            int q_free = -1;         // global period after which the Q buffers may be overwritten
            long long rel_seen = -1; // highest period known to be complete
            bool ok = true;
            auto wait_rel = [&](long long g) {  // wait until period g has completed (g < 0: nothing to wait for)
                if (!ok || g <= rel_seen) return;
                ok = mbar_wait_bounded(&bar_rel[g & 1], (uint32_t)((g >> 1) & 1), P2_WAIT_LIMIT);
                rel_seen = g;
            };
            int item_no = 0;
            for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++item_no) {
                const ItemPlan it = plan_item(p, item);
                if (it.n == 0) continue;
                auto load_k = [&](int j) {  // K tile j of this item -> stage (g0 + j) % 3, once that stage's last reader is done
                    const long long g = g0 + j;
                    wait_rel(g - 3);
                    if (!ok) return;
                    const int stage = (int)(g % P2_KST), key0 = it.base + j * P2_N;
                    uint8_t *kd = sK + stage * P2_KV_BYTES;
                    mbar_arrive_expect_tx(&bar_k[stage], P2_KV_BYTES);
                    tma_load_4d(kd, &tmap_k, &bar_k[stage], 0, it.hkv, key0, it.b);
                    tma_load_4d(kd + P2_KV_BYTES / 2, &tmap_k, &bar_k[stage], 64, it.hkv, key0, it.b);
                };
                auto load_v = [&](int j) {
                    const long long g = g0 + j;
                    wait_rel(g - 2);
                    if (!ok) return;
                    const int stage = (int)(g % P2_VST), key0 = it.base + j * P2_N;
                    uint8_t *vd = sV + stage * P2_KV_BYTES;
                    mbar_arrive_expect_tx(&bar_v[stage], P2_KV_BYTES);
                    tma_load_4d(vd, &tmap_v, &bar_v[stage], 0, it.hkv, key0, it.b);
                    tma_load_4d(vd + P2_KV_BYTES / 2, &tmap_v, &bar_v[stage], 64, it.hkv, key0, it.b);
                };
                // in the order in which their stages come free
                load_k(0);
                wait_rel(q_free);
                if (!ok) break;
                mbar_arrive_expect_tx(bar_q, 2 * P2_Q_BYTES);
#pragma unroll
                for (int i = 0; i < 2; ++i) {  // rows past T_new are filled with zeros by the copy
                    tma_load_4d(sQ + i * P2_Q_BYTES, &tmap_q, bar_q, 0, it.hq, it.t0 + i * P2_M, it.b);
                    tma_load_4d(sQ + i * P2_Q_BYTES + P2_Q_BYTES / 2, &tmap_q, bar_q, 64, it.hq, it.t0 + i * P2_M, it.b);
                }
                if (it.n > 1) load_k(1);
                load_v(0);
                if (it.n > 2) load_k(2);
                if (it.n > 1) load_v(1);
                for (int t = 0; t < it.n && ok; ++t) {
                    if (t + 3 < it.n) load_k(t + 3);
                    if (t + 2 < it.n) load_v(t + 2);
                }
                // the score products of the item's last tile are issued in its period n - 2 (in its first
                // period if it has a single tile)
                q_free = (int)(g0 + (it.n >= 2 ? it.n - 2 : 0));
                g0 += it.n;
            }
            if (!ok) timed_out();
        }
        __syncwarp();
    } else if (warp == P2_SOFTMAX_THREADS / 32) {
        // =============== one warp feeds the tensor core ============================================
        const bool leader = lane == 0;
        const uint64_t desc_q = smem_desc_sw128(smem_u32(sQ), 16, 1024);
        const uint64_t desc_k = smem_desc_sw128(smem_u32(sK), 16, 1024);
        const uint64_t desc_v = smem_desc_sw128(smem_u32(sV), P2_KV_BYTES / 2, 1024);
        auto wait_all = [&](uint64_t *bar, uint32_t parity) -> bool {
            return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity, P2_WAIT_LIMIT));
        };
        long long g0 = 0;
        unsigned n_p[2] = {0, 0};  // P tiles of group i consumed so far
        int item_no = 0;
        bool ok = true;
        // S_i(j) = Q_i K(j)^T into S_i
        auto issue_s = [&](int i, long long g) -> bool {
            const int stage = (int)(g % P2_KST);
            if (!wait_all(&bar_k[stage], (uint32_t)((g / P2_KST) & 1))) return false;
            tc_fence_after();
            const uint64_t dq = desc_q + (uint64_t)((i * P2_Q_BYTES) >> 4);
            const uint64_t dk = desc_k + (uint64_t)((stage * P2_KV_BYTES) >> 4);
            const uint32_t ds = tmem_base + (uint32_t)i * P2_N;
#pragma unroll
            for (int kk = 0; kk < NCKV_D / 16; ++kk) {
                const uint32_t off = (uint32_t)(kk & 3) * 32;
                const uint64_t da = dq + (uint64_t)(((kk >> 2) * (P2_Q_BYTES / 2) + off) >> 4);
                const uint64_t db = dk + (uint64_t)(((kk >> 2) * (P2_KV_BYTES / 2) + off) >> 4);
                if (leader) umma_bf16(ds, da, db, IDESC_S, kk > 0 ? 1u : 0u);
            }
            return true;
        };
        // O_i (+)= P_i V(j)
        auto issue_pv = [&](int i, long long g, bool accumulate) -> bool {
            const int stage = (int)(g % P2_VST);
            if (!wait_all(&bar_v[stage], (uint32_t)((g / P2_VST) & 1))) return false;
            if (!wait_all(&bar_p[i], n_p[i] & 1u)) return false;
            ++n_p[i];
            tc_fence_after();
            const uint64_t dv = desc_v + (uint64_t)((stage * P2_KV_BYTES) >> 4);
            const uint32_t pbase = tmem_base + (uint32_t)i * P2_N;      // P_i: packed bf16 over S_i's first 64 columns
            const uint32_t dout = tmem_base + 256 + (uint32_t)i * NCKV_D;
#pragma unroll
            for (int ks = 0; ks < P2_N / 16; ++ks) {
                const uint64_t db = dv + (uint64_t)((ks * 16 * 128) >> 4);
                if (leader) umma_bf16_a_tmem(dout, pbase + (uint32_t)ks * 8, db, IDESC_O, (accumulate || ks > 0) ? 1u : 0u);
            }
            return true;
        };
        for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
            const ItemPlan it = plan_item(p, item);
            if (it.n == 0) continue;
            ok = wait_all(bar_q, (uint32_t)(item_no & 1));
            ++item_no;
            // first score products of the item
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (ok && it.je[i] > it.jb[i]) {
                    ok = issue_s(i, g0 + it.jb[i]);
                    if (ok && leader) umma_commit(&bar_s[i]);
                    __syncwarp();
                }
            }
            for (int j = 0; j < it.n && ok; ++j) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (!ok || j < it.jb[i] || j >= it.je[i]) continue;
                    ok = issue_pv(i, g0 + j, j > it.jb[i]);
                    if (!ok) continue;
                    if (j + 1 < it.je[i]) {
                        ok = issue_s(i, g0 + j + 1);
                        if (ok && leader) umma_commit(&bar_s[i]);
                    } else if (leader) {
                        umma_commit(&bar_o[i]);
                    }
                    __syncwarp();
                }
                if (ok && leader) umma_commit(&bar_rel[(g0 + j) & 1]);
                __syncwarp();
            }
            g0 += it.n;
        }
        if (!ok && leader) timed_out();
        __syncwarp();
    } else {
        // =============== softmax groups: one thread per query row ==================================
        const int grp = tid >> 7;            // which query tile
        const int row = tid & (P2_M - 1);    // query row inside the tile == TMEM lane
        const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tmem_s = tmem_base + (uint32_t)grp * P2_N;
        const uint32_t tmem_o = tmem_base + 256 + (uint32_t)grp * NCKV_D;
        unsigned n_s = 0, n_o = 0;  // completions consumed on bar_s[grp] / bar_o[grp]
        long long g0 = 0;
        bool aborted = false;
        for (int item = blockIdx.x; item < p.n_items && !aborted; item += gridDim.x) {
            const ItemPlan it = plan_item(p, item);
            const int r0 = it.t0 + grp * P2_M;
            const int t = r0 + row;
            const int pos = it.L + t;  // absolute position of this row's token
            const int jb = grp ? it.jb[1] : it.jb[0], je = grp ? it.je[1] : it.je[0];
            const int kv_hi = grp ? it.kv_hi[1] : it.kv_hi[0];
            float m_used = -INFINITY, l_run = 0.f;
            for (int j = jb; j < je; ++j) {
                const int key0 = it.base + j * P2_N;
                {
                    const bool ok = *abort_flag == 0 && mbar_wait_bounded(&bar_s[grp], n_s & 1u, P2_WAIT_LIMIT);
                    if (!__all_sync(0xffffffffu, ok)) {
                        aborted = true;
                        break;
                    }
                    ++n_s;
                }
                tc_fence_after();
                // only tiles that touch the causal diagonal, the window edge or the end of the keys need
                // per-element masking (uniform over the group)
                const bool edge = (key0 + P2_N - 1 > it.L + r0) || (key0 + P2_N > kv_hi) ||
                                  (p.window_left >= 0 && key0 < it.L + r0 + P2_M - 1 - p.window_left);
                // pass 1: row max of the raw scores
                float mx_raw = -INFINITY;
#pragma unroll
                for (int ch = 0; ch < P2_N / 32; ++ch) {
                    float c[32];
                    tmem_ld32(tmem_s + lane_sel + ch * 32, c);
                    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int e = 0; e < 32; e += 4) {
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            float sv = c[e + u];
                            if (edge) {
                                const int kk = key0 + ch * 32 + e + u;
                                const bool visible = (kk <= pos) && (kk < kv_hi) && (p.window_left < 0 || pos - kk <= p.window_left);
                                sv = visible ? sv : -INFINITY;
                            }
                            mx4[u] = fmaxf(mx4[u], sv);
                        }
                    }
                    mx_raw = fmaxf(mx_raw, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])));
                }
                const float mx = mx_raw * p.scale_log2;  // the scale is positive
                const bool raise = mx > m_used + 8.f;    // also the first tile that shows this row a key
                const float alpha = raise ? ex2_approx(m_used - mx) : 1.f;
                if (raise) {
                    l_run *= alpha;
                    m_used = mx;
                }
                const float m_use = m_used == -INFINITY ? 0.f : m_used;
                // pass 2: P = 2^(s * scale - m), packed to bf16 over the columns the scores came from.  Chunk
                // ch of 32 scores becomes 16 words; they overwrite columns [16 ch, 16 ch + 16), which hold
                // scores of chunks <= ch / 2: already consumed.
                float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int ch = 0; ch < P2_N / 32; ++ch) {
                    float c[32];
                    tmem_ld32(tmem_s + lane_sel + ch * 32, c);
                    uint32_t pk[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 4) {
                        float pv[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            float sv = c[e + u];
                            if (edge) {
                                const int kk = key0 + ch * 32 + e + u;
                                const bool visible = (kk <= pos) && (kk < kv_hi) && (p.window_left < 0 || pos - kk <= p.window_left);
                                sv = visible ? sv : -INFINITY;
                            }
                            pv[u] = ex2_approx(fmaf(sv, p.scale_log2, -m_use));
                            rs4[u] += pv[u];
                        }
                        pk[e / 2] = pack_bf16x2(pv[0], pv[1]);
                        pk[e / 2 + 1] = pack_bf16x2(pv[2], pv[3]);
                    }
                    tmem_st16_words(tmem_s + lane_sel + ch * 16, pk);
                }
                l_run += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
                // A raised scale: the O row accumulated so far goes to the new scale.  P V of the previous
                // tile has completed (the commit that released this tile's scores was issued behind it) and the
                // next one is not issued before this thread's arrival below.
                if (j > jb && __any_sync(0xffffffffu, raise)) {
#pragma unroll
                    for (int ch = 0; ch < NCKV_D / 32; ++ch) {
                        float c[32];
                        tmem_ld32(tmem_o + lane_sel + ch * 32, c);
#pragma unroll
                        for (int e = 0; e < 32; ++e) c[e] *= alpha;
                        tmem_st32(tmem_o + lane_sel + ch * 32, c);
                    }
                }
                // rows of the V tile past the last key of the item may hold stale bytes: zero them so that a
                // zero probability never multiplies a NaN/Inf bit pattern (both groups do it, each before its
                // own product can be issued)
                const int item_hi = max(it.kv_hi[0], it.kv_hi[1]);
                if (key0 + P2_N > item_hi) {
                    const long long g = g0 + j;
                    const int stage = (int)(g % P2_VST);
                    uint8_t *vd = sV + stage * P2_KV_BYTES;
                    if (mbar_wait_bounded(&bar_v[stage], (uint32_t)((g / P2_VST) & 1), P2_WAIT_LIMIT)) {
                        for (int idx = row; idx < (key0 + P2_N - item_hi) * 16; idx += P2_M) {
                            const int r = (item_hi - key0) + idx / 16, chn = idx % 16;
                            *reinterpret_cast<uint4 *>(vd + (chn >> 3) * (P2_KV_BYTES / 2) + r * 128 + ((chn & 7) << 4)) =
                                make_uint4(0, 0, 0, 0);
                        }
                    }
                    fence_proxy_async_smem();
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_p[grp]);
            }
            if (aborted) break;
            // ---- epilogue of the item ----------------------------------------------------------------
            if (je > jb) {
                const bool ok = mbar_wait_bounded(&bar_o[grp], n_o & 1u, P2_WAIT_LIMIT);
                ++n_o;
                if (!__all_sync(0xffffffffu, ok)) {
                    if (!ok) timed_out();
                    aborted = true;
                    break;
                }
                tc_fence_after();
            }
            if (r0 < p.T_new) {  // uniform over the group
                const float inv = (je > jb && l_run > 0.f) ? 1.f / l_run : 0.f;
                uint4 *dst = reinterpret_cast<uint4 *>(p.out + (((long long)it.b * p.T_new + t) * p.Hq + it.hq) * NCKV_D);
#pragma unroll
                for (int ch = 0; ch < NCKV_D / 32; ++ch) {
                    float c[32];
                    if (je > jb) {
                        tmem_ld32(tmem_o + lane_sel + ch * 32, c);
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e) c[e] = 0.f;
                    }
                    if (t < p.T_new) {  // rows past the end of the sequence are padding
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            uint4 v;
                            v.x = pack_bf16x2(c[8 * e + 0] * inv, c[8 * e + 1] * inv);
                            v.y = pack_bf16x2(c[8 * e + 2] * inv, c[8 * e + 3] * inv);
                            v.z = pack_bf16x2(c[8 * e + 4] * inv, c[8 * e + 5] * inv);
                            v.w = pack_bf16x2(c[8 * e + 6] * inv, c[8 * e + 7] * inv);
                            dst[ch * 4 + e] = v;
                        }
                    }
                }
                // the O columns are read: order those loads before the next item's first P V (which this
                // thread releases with its next arrival on bar_p)
                tc_fence_before();
            }
            g0 += it.n;
        }
        if (aborted && *abort_flag == 0) timed_out();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, P2_TMEM_COLS);
}

static size_t prefill2_smem_bytes() {
    return 2 * P2_Q_BYTES + (P2_KST + P2_VST) * P2_KV_BYTES + 16 * sizeof(uint64_t);
}

}  // namespace nckv

extern "C" int nckv_prefill_attn(const void *q, const void *k, const void *v, const int32_t *cache_seqlens,
                                 void *out, int B, int T_new, int Hq, int Hkv, int D, int T_k,
                                 int64_t kv_batch_stride, int64_t kv_token_stride, int window_left,
                                 int32_t *status, void *stream) {
    using namespace nckv;
    if (!q || !k || !v || !out || !status) {
        set_error("prefill_attn: null pointer argument");
        return NCKV_E_ARG;
    }
    if (B <= 0 || T_new <= 0 || Hq <= 0 || Hkv <= 0 || T_k <= 0) {
        set_error("prefill_attn: non-positive size (B=%d T_new=%d Hq=%d Hkv=%d T_k=%d)", B, T_new, Hq, Hkv, T_k);
        return NCKV_E_ARG;
    }
    if (D != NCKV_D) {
        set_error("prefill_attn: head_dim %d unsupported (kernels are built for 128)", D);
        return NCKV_E_UNSUPPORTED;
    }
    if (Hq % Hkv != 0) {
        set_error("prefill_attn: Hq=%d must be a multiple of Hkv=%d", Hq, Hkv);
        return NCKV_E_UNSUPPORTED;
    }
    if (T_new > T_k) {
        set_error("prefill_attn: T_new=%d exceeds the key capacity T_k=%d", T_new, T_k);
        return NCKV_E_CAPACITY;
    }
    const int n_qpairs = (T_new + 2 * P2_M - 1) / (2 * P2_M);
    if ((long long)n_qpairs * Hq * B > 0x7fffffffLL) {
        set_error("prefill_attn: B=%d x Hq=%d x %d query tiles exceed the item limit", B, Hq, n_qpairs);
        return NCKV_E_UNSUPPORTED;
    }
    if (((uintptr_t)q | (uintptr_t)out) & 15) {
        set_error("prefill_attn: q/out must be 16-byte aligned");
        return NCKV_E_ARG;
    }
    CUtensorMap mq, mk, mv;
    int rc = make_kv_tensor_map(&mq, q, B, T_new, Hq, (int64_t)T_new * Hq * D, (int64_t)Hq * D, P2_M);
    if (rc != NCKV_OK) return rc;
    rc = make_kv_tensor_map(&mk, k, B, T_k, Hkv, kv_batch_stride, kv_token_stride, P2_N);
    if (rc != NCKV_OK) return rc;
    rc = make_kv_tensor_map(&mv, v, B, T_k, Hkv, kv_batch_stride, kv_token_stride, P2_N);
    if (rc != NCKV_OK) return rc;

    Prefill2Params p;
    p.seqlens = cache_seqlens;
    p.out = static_cast<__nv_bfloat16 *>(out);
    p.status = status;
    p.B = B; p.T_new = T_new; p.Hq = Hq; p.Hkv = Hkv; p.T_k = T_k;
    p.window_left = window_left;
    p.n_qpairs = n_qpairs;
    p.n_items = n_qpairs * Hq * B;
    p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)D));
    {
        // pairs per group: about 48 MB of K and V rows (512 B per key and kv head, shared by Hq / Hkv
        // q heads) leaves room in the 126 MB L2 for two groups in flight and everything else
        const long long keys = window_left >= 0 && window_left + 2 * P2_M < T_k ? window_left + 2 * P2_M : T_k;
        const long long bytes_per_pair = keys * 512 / (Hq / Hkv) + 1;
        long long g = (48LL << 20) / bytes_per_pair;
        g -= g % (Hq / Hkv);  // keep the q heads of a kv head in one group
        p.group_pairs = (int)(g < Hq / Hkv ? Hq / Hkv : (g > (long long)Hq * B ? (long long)Hq * B : g));
    }

    const size_t smem = prefill2_smem_bytes();
    static bool attr_set[64] = {false};  // per device; setting the attribute twice from racing threads is harmless
    int dev = 0;
    NCKV_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        NCKV_CUDA_CHECK(cudaFuncSetAttribute(prefill_attn2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev] = true;
    }
    const int grid = p.n_items < sm_count() ? p.n_items : sm_count();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(P2_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NCKV_CUDA_CHECK(cudaLaunchKernelEx(&cfg, prefill_attn2_kernel, mq, mk, mv, p));
    return NCKV_OK;
}
