// Kernel (d): dense causal attention for T_new >= 1 query tokens per row (prefill, chunked
// prefill, flash_attn_func), on the 5th-generation tensor cores: tcgen05.mma with Q, K, V in
// shared memory (TMA, 128-byte swizzle), the probabilities and the accumulators in tensor memory.
//
// One CTA owns a tile of PF_M = 128 query tokens of one (row, q head) and walks the visible keys
// in tiles of PF_N = 64.  Three roles, connected by mbarriers only (no CTA-wide barrier in the loop):
//   producer warp     one lane issues the TMA copies: Q once, K and V through two stages each; a
//                     stage is refilled as soon as the product that read it has completed
//   MMA warp          one lane issues, per tile,
//                       S = Q K^T   8 x tcgen05.mma (M128 N64 K16) into one of two S buffers in
//                                   TMEM (columns [0, 64) and [64, 128)), two tiles ahead of the softmax
//                       O += P V    4 x tcgen05.mma (M128 N128 K16): P is the A operand, read from
//                                   TMEM; V is used in place as an MN-major shared-memory operand;
//                                   the accumulator stays in TMEM columns [128, 256) over all tiles
//                     and signals completion through tcgen05.commit
//   softmax warps     thread r owns query row r = TMEM lane r: tcgen05.ld brings its 64 scores
//                     into registers, causal / window masking is done by index (edge tiles only),
//                     running max and sum are per-thread scalars, P is rounded to bf16 and stored
//                     with tcgen05.st over the first 32 columns of the S buffer it came from.
//                     P is scaled by a running max that is only raised when the true max has
//                     grown by more than 2^8; only then is the O row rescaled in TMEM
//                     (tcgen05.ld / multiply / tcgen05.st), so most tiles neither wait for nor
//                     touch the accumulator.  O is read once, at the end.
// Products issued by one thread execute in order: S of tile it+2 is issued behind O += P V(it)
// and may therefore overwrite the buffer P(it) was read from.
// Two CTAs fit on an SM (about 96 KB of shared memory and 256 of the 512 TMEM columns each), so
// one CTA's softmax overlaps the other's tensor work.
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

constexpr int PF_M = 128;  // query tokens per CTA
constexpr int PF_N = 64;   // keys per tile
constexpr int PF_STAGES = 2;    // K stages
constexpr int PF_VSTAGES = 3;   // V stages
constexpr int PF_SPLIT = 1;                           // softmax threads per query row (2 measured slower)
constexpr int PF_SOFTMAX_THREADS = PF_M * PF_SPLIT;
constexpr int PF_THREADS = PF_SOFTMAX_THREADS + 64;   // + one warp that issues the MMAs + one that issues the TMA copies
constexpr int PF_Q_BYTES = PF_M * NCKV_D * 2;        // 32 KB: two 64-channel halves of [128][128 B]
constexpr int PF_KV_BYTES = PF_N * NCKV_D * 2;       // 16 KB: two halves of [64][128 B]
constexpr int PF_TMEM_COLS = 256;                    // S/P buffers: [0,64), [64,128)   O: [128,256)
constexpr unsigned long long PF_WAIT_LIMIT = NCKV_WAIT_LIMIT_NS;

struct PrefillParams {
    const int32_t *seqlens;  // may be null (all zero)
    __nv_bfloat16 *out;
    int32_t *status;
    int B, T_new, Hq, Hkv, T_k;
    int group_pairs;  // (row, q head) pairs per scheduling group, see the work order in the kernel
    int pair_major;   // order inside a group: 1 pair by pair, 0 longest tiles of all pairs first
    int window_left;
    float scale_log2;
};



__global__ void __launch_bounds__(PF_THREADS, 2)
prefill_attn_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const PrefillParams p) {
    // The swizzled tiles need 1024-byte aligned bases; the dynamic segment is declared with that
    // alignment (no slack bytes: two CTAs must fit in one SM's shared memory).
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0) {  // uniform; checked rather than assumed
        if (threadIdx.x == 0) atomicOr(p.status, (int)NCKV_ST_TIMEOUT);
        return;
    }
    uint8_t *sQ = smem;                                   // 32 KB
    uint8_t *sK = sQ + PF_Q_BYTES;                        // 2 x 16 KB
    uint8_t *sV = sK + PF_STAGES * PF_KV_BYTES;           // 3 x 16 KB
    uint64_t *bars = reinterpret_cast<uint64_t *>(sV + PF_VSTAGES * PF_KV_BYTES);
    uint64_t *bar_q = bars;          // Q landed
    uint64_t *bar_k = bars + 1;      // [PF_STAGES] K tile landed
    uint64_t *bar_v = bars + 3;      // [PF_VSTAGES] V tile landed
    // [2] S(it) = Q K(it)^T complete, on bar_s[it & 1].  Products complete in issue order and S(it) is
    // issued behind O += P V(it-2), so this also says "P V(it-2) complete".
    uint64_t *bar_s = bars + 6;
    // [2] O += P V(it) complete, on bar_o[it & 1]: signalled only for the last two tiles, which no S
    // follows.  Every tcgen05.commit costs tensor-pipe time (measured: groups of 4-8 instructions
    // between commits run at about half the rate of an uninterrupted stream), so a tile gets one.
    uint64_t *bar_o = bars + 8;
    // [2] P(it) in TMEM, S(it) read, O rescaled: one arrival per softmax warp on bar_p[it & 1].  Two
    // barriers because the softmax may finish tile it+1 before the issuer has looked at tile it.
    uint64_t *bar_p = bars + 10;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 12);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    // PF_SPLIT == 2 only: [2 buffers][2][PF_M] row maxima exchanged between the threads of a row
    __nv_bfloat16 *s_xchg = reinterpret_cast<__nv_bfloat16 *>(bars + 13);
    (void)s_xchg;

    const int tid = threadIdx.x, warp = tid >> 5;
    // Work order.  CTAs are handed to the SMs in block-index order, which makes the grid a work queue.
    // Causal query tiles differ in length by up to n_qtiles x, so the order decides both the tail and
    // which tiles share an SM.  The (row, q head) pairs are taken in groups of group_pairs (sized on the
    // host so that a group's K/V stays in L2 while its query tiles reuse it).  Inside a group either
    // pair by pair with a pair's long tiles first (long and short tiles then meet on an SM and fill each
    // other's gaps: best while a pair has few tiles), or all pairs' longest tiles first and their shortest
    // last (bounds the tail when one tile is a large share of an SM's work: long sequences).
    const int n_qtiles = (p.T_new + PF_M - 1) / PF_M;
    const int n_pairs = p.Hq * p.B;
    const int per_group = p.group_pairs * n_qtiles;
    const int grp = (int)blockIdx.x / per_group;
    const int in_grp = (int)blockIdx.x - grp * per_group;
    const int grp_pairs = min(p.group_pairs, n_pairs - grp * p.group_pairs);
    int qt, pair;
    if (p.pair_major) {  // pair by pair, a pair's long tiles first
        pair = grp * p.group_pairs + in_grp / n_qtiles;
        qt = n_qtiles - 1 - in_grp % n_qtiles;
    } else {             // all pairs' longest tiles first, their shortest last
        qt = n_qtiles - 1 - in_grp / grp_pairs;
        pair = grp * p.group_pairs + in_grp % grp_pairs;
    }
    const int hq = pair % p.Hq, b = pair / p.Hq;
    const int hkv = hq / (p.Hq / p.Hkv);
    const int t0 = qt * PF_M;

    pdl_wait_prior_grids();
    int L = p.seqlens ? p.seqlens[b] : 0;
    if (L < 0) {
        if (tid == 0) atomicOr(p.status, (int)NCKV_ST_BAD_SEQLEN);
        L = 0;
    }
    int Tk = L + p.T_new;  // keys present after the append
    if (Tk > p.T_k) {
        if (tid == 0) atomicOr(p.status, (int)NCKV_ST_OVERFLOW);
        Tk = p.T_k;
    }
    // keys any row of this tile may see: [kv_lo, kv_hi)
    const int last_t = min(t0 + PF_M, p.T_new) - 1;
    const int kv_hi = min(Tk, L + last_t + 1);
    const int kv_lo = p.window_left >= 0 ? max(0, L + t0 - p.window_left) : 0;
    const int n_tiles = kv_hi > kv_lo ? (kv_hi - kv_lo + PF_N - 1) / PF_N : 0;

    if (tid == 0) {
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
        mbar_init(bar_q, 1);
        for (int s = 0; s < PF_STAGES; ++s) mbar_init(&bar_k[s], 1);
        for (int s = 0; s < PF_VSTAGES; ++s) mbar_init(&bar_v[s], 1);
        mbar_init(&bar_s[0], 1);
        mbar_init(&bar_s[1], 1);
        mbar_init(&bar_o[0], 1);
        mbar_init(&bar_o[1], 1);
        mbar_init(&bar_p[0], PF_SOFTMAX_THREADS / 32);
        mbar_init(&bar_p[1], PF_SOFTMAX_THREADS / 32);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, PF_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base;          // S buffer 0: columns [0, 64), S buffer 1: columns [64, 128)
    const uint32_t tmem_o = tmem_base + 128;    // columns [128, 256)
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;  // a warp reaches TMEM lanes 32*(warp % 4) ..

    constexpr uint32_t IDESC_S = umma_idesc(PF_M, PF_N, 0, 0);
    constexpr uint32_t IDESC_O = umma_idesc(PF_M, NCKV_D, 0, 1);
    const bool issuer_warp = warp == PF_SOFTMAX_THREADS / 32;
    bool aborted = false;
    auto timed_out = [&]() {
        *abort_flag = 1;
        atomicOr(p.status, (int)NCKV_ST_TIMEOUT);
    };

    if (warp == PF_SOFTMAX_THREADS / 32 + 1) {
        // =============== one lane moves the tiles: Q once, K and V through two stages each =======
        if ((tid & 31) == 0 && n_tiles > 0) {
            auto load_k = [&](int tile) {  // K(tile) -> stage tile % 2
                const int stage = tile % PF_STAGES, key0 = kv_lo + tile * PF_N;
                uint8_t *kd = sK + stage * PF_KV_BYTES;
                mbar_arrive_expect_tx(&bar_k[stage], PF_KV_BYTES);
                tma_load_4d(kd, &tmap_k, &bar_k[stage], 0, hkv, key0, b);
                tma_load_4d(kd + PF_KV_BYTES / 2, &tmap_k, &bar_k[stage], 64, hkv, key0, b);
            };
            auto load_v = [&](int tile) {  // V(tile) -> stage tile % 3
                const int stage = tile % PF_VSTAGES, key0 = kv_lo + tile * PF_N;
                uint8_t *vd = sV + stage * PF_KV_BYTES;
                mbar_arrive_expect_tx(&bar_v[stage], PF_KV_BYTES);
                tma_load_4d(vd, &tmap_v, &bar_v[stage], 0, hkv, key0, b);
                tma_load_4d(vd + PF_KV_BYTES / 2, &tmap_v, &bar_v[stage], 64, hkv, key0, b);
            };
            mbar_arrive_expect_tx(bar_q, PF_Q_BYTES);
            tma_load_4d(sQ, &tmap_q, bar_q, 0, hq, t0, b);
            tma_load_4d(sQ + PF_Q_BYTES / 2, &tmap_q, bar_q, 64, hq, t0, b);
            for (int i = 0; i < PF_STAGES && i < n_tiles; ++i) load_k(i);
            for (int i = 0; i < PF_VSTAGES && i < n_tiles; ++i) load_v(i);
            bool ok = true;
            for (int t = 0; t + 2 < n_tiles && ok; ++t) {
                // S(t) complete: K(t)'s stage is free for K(t+2); and, being issued behind it,
                // O += P V(t-2) is complete too: V(t-2)'s stage is free for V(t+1)
                ok = mbar_wait_bounded(&bar_s[t & 1], (uint32_t)((t >> 1) & 1), PF_WAIT_LIMIT);
                if (!ok) break;
                load_k(t + 2);
                if (t + 1 >= PF_VSTAGES) load_v(t + 1);
            }
            // V of the last tile: its stage is the one of V(n-4), free once S(n-2) has completed
            if (ok && n_tiles - 1 >= PF_VSTAGES && n_tiles >= 2) {
                const int t = n_tiles - 2;
                ok = mbar_wait_bounded(&bar_s[t & 1], (uint32_t)((t >> 1) & 1), PF_WAIT_LIMIT);
                if (ok) load_v(n_tiles - 1);
            }
            if (!ok) timed_out();
        }
        __syncwarp();
    } else if (issuer_warp) {
        // =============== one warp feeds the tensor core ============================================
        // The whole warp runs this loop so that control flow and every MMA operand (descriptors,
        // TMEM addresses) stay warp-uniform; only the tcgen05.mma / tcgen05.commit instructions
        // themselves are executed by a single lane.
        if (n_tiles > 0) {
            const bool leader = (tid & 31) == 0;
            // Descriptors differ only in the start-address field (address >> 4 in the low 14 bits),
            // so they are built once and advanced by adding the byte offset >> 4.
            const uint64_t desc_q = smem_desc_sw128(smem_u32(sQ), 16, 1024);
            const uint64_t desc_k = smem_desc_sw128(smem_u32(sK), 16, 1024);
            const uint64_t desc_v = smem_desc_sw128(smem_u32(sV), PF_KV_BYTES / 2, 1024);
            auto wait_all = [&](uint64_t *bar, uint32_t parity) -> bool {
                return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity, PF_WAIT_LIMIT));
            };
            // S(tile) = Q K(tile)^T into S buffer tile & 1, then arrive on bar_s[tile & 1]
            auto issue_s = [&](int tile) -> bool {
                const int stage = tile % PF_STAGES;
                if (tile == 0 && !wait_all(bar_q, 0)) return false;
                if (!wait_all(&bar_k[stage], (uint32_t)((tile / PF_STAGES) & 1))) return false;
                tc_fence_after();
                const uint64_t dk = desc_k + (uint64_t)((stage * PF_KV_BYTES) >> 4);
                const uint32_t ds = tmem_s + (uint32_t)(tile & 1) * PF_N;
                if (leader) {  // one thread runs the whole burst: nothing diverges and reconverges between the instructions
#pragma unroll
                    for (int kk = 0; kk < NCKV_D / 16; ++kk) {
                        const uint32_t off = (uint32_t)(kk & 3) * 32;
                        const uint64_t da = desc_q + (uint64_t)(((kk >> 2) * (PF_Q_BYTES / 2) + off) >> 4);
                        const uint64_t db = dk + (uint64_t)(((kk >> 2) * (PF_KV_BYTES / 2) + off) >> 4);
                        umma_bf16(ds, da, db, IDESC_S, kk > 0 ? 1u : 0u);
                    }
                    umma_commit(&bar_s[tile & 1]);
                }
                __syncwarp();
                return true;
            };
            // O (+)= P V(tile) into TMEM columns [128, 256), then arrive on bar_o[tile & 1]
            auto issue_pv = [&](int tile, bool commit_now) -> bool {
                const int stage = tile % PF_VSTAGES;
                if (!wait_all(&bar_v[stage], (uint32_t)((tile / PF_VSTAGES) & 1))) return false;
                tc_fence_after();
                // V in place: N (channels) contiguous, the two 64-channel halves PF_KV_BYTES/2 apart
                // (leading offset), 8-key groups 1024 B apart (stride offset)
                const uint64_t dv = desc_v + (uint64_t)((stage * PF_KV_BYTES) >> 4);
                const uint32_t pbase = tmem_s + (uint32_t)(tile & 1) * PF_N;
                if (leader) {
#pragma unroll
                    for (int ks = 0; ks < PF_N / 16; ++ks) {
                        // P(tile) sits in the first 32 columns of its S buffer; 16 keys = 8 columns
                        const uint64_t db = dv + (uint64_t)((ks * 16 * 128) >> 4);
                        umma_bf16_a_tmem(tmem_o, pbase + (uint32_t)ks * 8, db, IDESC_O, (tile > 0 || ks > 0) ? 1u : 0u);
                    }
                    if (commit_now) umma_commit(&bar_o[tile & 1]);
                }
                __syncwarp();
                return true;
            };

            // S runs two tiles ahead of the softmax
            bool ok = issue_s(0);
            if (ok && n_tiles > 1) ok = issue_s(1);
            for (int it = 0; it < n_tiles && ok; ++it) {
                // P(it) is in TMEM, S(it) has been read, O carries the scale P was made with
                ok = wait_all(&bar_p[it & 1], (uint32_t)((it >> 1) & 1));
                if (!ok) break;
                tc_fence_after();
                // S(it+2) goes into the S buffer every thread has just finished reading; its commit also
                // covers O += P V(it).  The last two tiles have no S behind them and signal bar_o.
                const bool s_follows = it + 2 < n_tiles;
                ok = issue_pv(it, !s_follows);
                if (ok && s_follows) ok = issue_s(it + 2);
            }
            if (!ok && leader) timed_out();
        }
        __syncwarp();
    } else {
        // =============== softmax threads: PF_SPLIT per query row =================================
        // Softmax state of this thread's row.  P is scaled by m_used, which follows the true running
        // max lazily: it is only raised (and the O row in TMEM rescaled) when the max has grown by
        // more than 2^8, so exp2(s - m_used) stays <= 256 and most tiles need no rescale at all.
        float m_used = -INFINITY, l_run = 0.f;
        const int row = tid & (PF_M - 1);  // query row inside the tile == TMEM lane
        const int half = tid / PF_M;       // which share of the tile's scores (and of the output channels) is mine
        const int pos = L + t0 + row;      // absolute position of this row's token
        constexpr int HN = PF_N / PF_SPLIT;    // scores per thread and tile
        constexpr int OC = NCKV_D / PF_SPLIT;  // output channels per thread

        for (int it = 0; it < n_tiles; ++it) {
            const int stage = it % PF_VSTAGES;
            const uint32_t kv_parity = (uint32_t)((it / PF_VSTAGES) & 1);
            const int key0 = kv_lo + it * PF_N;
            const uint32_t tmem_s_it = tmem_s + (uint32_t)(it & 1) * PF_N;
            // tcgen05.ld/st are warp-wide (.sync.aligned): every decision that skips them is taken per warp
            {
                const bool ok = *abort_flag == 0 &&
                                mbar_wait_bounded(&bar_s[it & 1], (uint32_t)((it >> 1) & 1), PF_WAIT_LIMIT);
                if (!__all_sync(0xffffffffu, ok)) {
                    aborted = true;
                    break;
                }
            }
            tc_fence_after();

            float s_val[HN];
#pragma unroll
            for (int ch = 0; ch < HN / 32; ++ch) {
                float c[32];
                tmem_ld32(tmem_s_it + lane_sel + half * HN + ch * 32, c);  // raw q.k, scaled inside the exponent
#pragma unroll
                for (int i = 0; i < 32; ++i) s_val[ch * 32 + i] = c[i];
            }
            // only tiles that touch the causal diagonal, the window edge or the end of the keys need
            // per-element masking (uniform over the CTA)
            const bool edge = (key0 + PF_N - 1 > L + t0) || (key0 + PF_N > kv_hi) ||
                              (p.window_left >= 0 && key0 < L + t0 + PF_M - 1 - p.window_left);
            if (edge) {
                // this row sees columns [c_lo, c_hi) of its share of the tile
                const int c_hi = min(pos, kv_hi - 1) - (key0 + half * HN) + 1;
                const int c_lo = p.window_left >= 0 ? pos - p.window_left - (key0 + half * HN) : 0;
#pragma unroll
                for (int c = 0; c < HN; ++c) s_val[c] = (c >= c_lo && c < c_hi) ? s_val[c] : -INFINITY;
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains instead of one
#pragma unroll
            for (int c = 0; c < HN; c += 4) {
                mx4[0] = fmaxf(mx4[0], s_val[c]);
                mx4[1] = fmaxf(mx4[1], s_val[c + 1]);
                mx4[2] = fmaxf(mx4[2], s_val[c + 2]);
                mx4[3] = fmaxf(mx4[3], s_val[c + 3]);
            }
            float mx_raw = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            if (PF_SPLIT == 2) {
                // The row max needs both halves: exchange through shared memory, double buffered
                // because a thread may run up to one tile ahead of its partner.  bf16 rounded UP: the
                // reference point of the exponentials only has to be the same in both threads and
                // not below the true max.
                __nv_bfloat16 *xb = s_xchg + (it & 1) * 2 * PF_M;
                const __nv_bfloat16 mine = __float2bfloat16_ru(mx_raw);
                xb[half * PF_M + row] = mine;
                asm volatile("bar.sync 1, %0;" ::"n"(PF_SOFTMAX_THREADS) : "memory");
                mx_raw = fmaxf(__bfloat162float(mine), __bfloat162float(xb[(half ^ 1) * PF_M + row]));
            }
            // the max is taken on raw scores and scaled once (the scale is positive)
            const float mx = mx_raw * p.scale_log2;
            const bool raise = mx > m_used + 8.f;  // also the first tile that shows this row a key (m_used = -inf)
            const float alpha = raise ? ex2_approx(m_used - mx) : 1.f;  // 2^-inf = 0
            if (raise) {
                l_run *= alpha;
                m_used = mx;
            }
            const float m_use = m_used == -INFINITY ? 0.f : m_used;  // a row that has seen no key yet
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[HN / 2];
#pragma unroll
            for (int c = 0; c < HN; c += 4) {
                // one FFMA and one MUFU.EX2 per score: 2^(s * scale - m)
                const float p0 = ex2_approx(fmaf(s_val[c], p.scale_log2, -m_use));
                const float p1 = ex2_approx(fmaf(s_val[c + 1], p.scale_log2, -m_use));
                const float p2 = ex2_approx(fmaf(s_val[c + 2], p.scale_log2, -m_use));
                const float p3 = ex2_approx(fmaf(s_val[c + 3], p.scale_log2, -m_use));
                rs4[0] += p0; rs4[1] += p1; rs4[2] += p2; rs4[3] += p3;
                pk[c / 2] = pack_bf16x2(p0, p1);
                pk[c / 2 + 1] = pack_bf16x2(p2, p3);
            }
            l_run += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);  // this thread's share of the row sum

            // P row -> TMEM, over the first 32 columns of this tile's S buffer (this lane's own scores,
            // already in registers).  S of tile it+2 is issued behind P V(it) and lands on top of it.
            tmem_st_words(tmem_s_it + lane_sel + half * (HN / 2), pk);
            // A raised scale: O (+)= P V of the previous tile must be complete before the O rows
            // accumulated so far are brought to the new scale (tcgen05.ld / multiply / tcgen05.st).
            // Every lane applies its own factor (1 for rows that keep their scale).
            if (it > 0 && __any_sync(0xffffffffu, raise)) {
                // O += P V(it-1) complete: told by S(it+1), which was issued behind it, or by bar_o
                // when tile it is the last one
                const bool ok = it + 1 < n_tiles
                                    ? mbar_wait_bounded(&bar_s[(it + 1) & 1], (uint32_t)(((it + 1) >> 1) & 1), PF_WAIT_LIMIT)
                                    : mbar_wait_bounded(&bar_o[(it - 1) & 1], 0, PF_WAIT_LIMIT);
                if (!__all_sync(0xffffffffu, ok)) {
                    if (!ok) timed_out();
                    aborted = true;
                    break;
                }
                tc_fence_after();
#pragma unroll
                for (int ch = 0; ch < OC / 32; ++ch) {
                    float c[32];
                    tmem_ld32(tmem_o + lane_sel + half * OC + ch * 32, c);
#pragma unroll
                    for (int i = 0; i < 32; ++i) c[i] *= alpha;
                    tmem_st32(tmem_o + lane_sel + half * OC + ch * 32, c);
                }
            }
            // rows of the V tile past the last key may hold stale bytes: zero them so that a zero
            // probability never multiplies a NaN/Inf bit pattern
            if (key0 + PF_N > kv_hi) {
                uint8_t *vd = sV + stage * PF_KV_BYTES;
                if (mbar_wait_bounded(&bar_v[stage], kv_parity, PF_WAIT_LIMIT)) {
                    for (int idx = tid; idx < (key0 + PF_N - kv_hi) * 16; idx += PF_SOFTMAX_THREADS) {
                        const int r = (kv_hi - key0) + idx / 16, ch = idx % 16;
                        *reinterpret_cast<uint4 *>(vd + (ch >> 3) * (PF_KV_BYTES / 2) + r * 128 + ((ch & 7) << 4)) =
                            make_uint4(0, 0, 0, 0);
                    }
                }
                fence_proxy_async_smem();  // the zeroed V rows must be visible to the tensor core
            }
            tc_fence_before();  // orders this thread's TMEM loads/stores before the next MMAs
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(&bar_p[it & 1]);  // one arrival per warp
        }
        if (aborted && *abort_flag == 0) timed_out();  // a wait ran out in this warp

        // ---- epilogue ---------------------------------------------------------------------------
        const int t = t0 + row;
        if (!aborted && n_tiles > 0) {
            const bool ok = mbar_wait_bounded(&bar_o[(n_tiles - 1) & 1], 0, PF_WAIT_LIMIT);
            if (!ok) timed_out();
            aborted = !__all_sync(0xffffffffu, ok);
            tc_fence_after();
        }
        float l_row = l_run;
        if (PF_SPLIT == 2) {  // the row sum is the sum of the two threads' shares
            // every product has completed (or the CTA has given up): the first K stage is free
            float *s_sum = reinterpret_cast<float *>(sK);
            s_sum[half * PF_M + row] = l_run;
            asm volatile("bar.sync 1, %0;" ::"n"(PF_SOFTMAX_THREADS) : "memory");
            l_row += s_sum[(half ^ 1) * PF_M + row];
        }
        if (!aborted) {  // uniform over the warp: the TMEM loads below are warp-wide instructions
            const float inv = (n_tiles > 0 && l_row > 0.f) ? 1.f / l_row : 0.f;
            uint4 *dst = reinterpret_cast<uint4 *>(p.out + (((long long)b * p.T_new + t) * p.Hq + hq) * NCKV_D + half * OC);
#pragma unroll
            for (int ch = 0; ch < OC / 32; ++ch) {
                float c[32];
                if (n_tiles > 0) {
                    tmem_ld32(tmem_o + lane_sel + half * OC + ch * 32, c);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) c[i] = 0.f;
                }
                if (t < p.T_new) {  // rows past the end of the sequence are padding
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 v;
                        v.x = pack_bf16x2(c[8 * i + 0] * inv, c[8 * i + 1] * inv);
                        v.y = pack_bf16x2(c[8 * i + 2] * inv, c[8 * i + 3] * inv);
                        v.z = pack_bf16x2(c[8 * i + 4] * inv, c[8 * i + 5] * inv);
                        v.w = pack_bf16x2(c[8 * i + 6] * inv, c[8 * i + 7] * inv);
                        dst[ch * 4 + i] = v;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, PF_TMEM_COLS);
}

static size_t prefill_smem_bytes() {
    return PF_Q_BYTES + (PF_STAGES + PF_VSTAGES) * PF_KV_BYTES + 13 * sizeof(uint64_t) +
           (PF_SPLIT == 2 ? 4 * PF_M * sizeof(__nv_bfloat16) : 0);
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
    const int n_qtiles = (T_new + PF_M - 1) / PF_M;
    if ((long long)n_qtiles * Hq * B > 0x7fffffffLL) {
        set_error("prefill_attn: B=%d x Hq=%d x %d query tiles exceed the grid limit", B, Hq, n_qtiles);
        return NCKV_E_UNSUPPORTED;
    }
    if (((uintptr_t)q | (uintptr_t)out) & 15) {
        set_error("prefill_attn: q/out must be 16-byte aligned");
        return NCKV_E_ARG;
    }
    CUtensorMap mq, mk, mv;
    int rc = make_kv_tensor_map(&mq, q, B, T_new, Hq, (int64_t)T_new * Hq * D, (int64_t)Hq * D, PF_M);
    if (rc != NCKV_OK) return rc;
    rc = make_kv_tensor_map(&mk, k, B, T_k, Hkv, kv_batch_stride, kv_token_stride, PF_N);
    if (rc != NCKV_OK) return rc;
    rc = make_kv_tensor_map(&mv, v, B, T_k, Hkv, kv_batch_stride, kv_token_stride, PF_N);
    if (rc != NCKV_OK) return rc;

    PrefillParams p;
    p.seqlens = cache_seqlens;
    p.out = static_cast<__nv_bfloat16 *>(out);
    p.status = status;
    p.B = B; p.T_new = T_new; p.Hq = Hq; p.Hkv = Hkv; p.T_k = T_k;
    p.window_left = window_left;
    p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)D));
    {
        // pairs per group: about 48 MB of K and V rows (512 B per key and kv head, shared by Hq / Hkv
        // q heads) leaves room in the 126 MB L2 for two groups in flight and everything else
        const long long keys = window_left >= 0 && window_left + PF_M < T_k ? window_left + PF_M : T_k;
        const long long bytes_per_pair = keys * 512 / (Hq / Hkv) + 1;
        long long g = (48LL << 20) / bytes_per_pair;
        g -= g % (Hq / Hkv);  // keep the q heads of a kv head in one group
        p.group_pairs = (int)(g < Hq / Hkv ? Hq / Hkv : (g > (long long)Hq * B ? (long long)Hq * B : g));
    }

    p.pair_major = n_qtiles <= 16;  // measured on B200: 2048-token rows and shorter prefer it, 4096 and longer do not

    const size_t smem = prefill_smem_bytes();
    static bool attr_set[64] = {false};
    int dev = 0;
    NCKV_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        NCKV_CUDA_CHECK(cudaFuncSetAttribute(prefill_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n_qtiles * Hq * B));
    cfg.blockDim = dim3(PF_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NCKV_CUDA_CHECK(cudaLaunchKernelEx(&cfg, prefill_attn_kernel, mq, mk, mv, p));
    return NCKV_OK;
}
