// Kernel (d): dense causal attention for T_new >= 1 query tokens per row (prefill, chunked
// prefill, flash_attn_func), on the 5th-generation tensor cores: tcgen05.mma with Q, K, V in
// shared memory (TMA, 128-byte swizzle), the probabilities and the accumulators in tensor memory.
//
// A work item is a tile of PF_M = 128 query tokens of one (row, q head) with the keys it sees, walked
// in tiles of PF_N = 64.  The CTAs are persistent, two per SM, and each works through a fixed list of
// items as ONE stream of key tiles: the copies and the first score products of the next item are
// issued while the softmax of the current item's last tiles and its output are still under way.
// Three roles, connected by mbarriers only (no CTA-wide barrier in the loop):
//   producer warp     one lane issues the TMA copies: Q per item, K through two and V through three
//                     stages; a stage is refilled as soon as the product that read it has completed
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
// Two CTAs fit on an SM (112 KB of shared memory and 256 of the 512 TMEM columns each), so one
// CTA's softmax overlaps the other's tensor work.  mbarrier waits are made by one lane per warp:
// a poll by 32 lanes is served lane after lane, and even a satisfied wait costs about 100 cycles.
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
static_assert(PF_N == 64, "the softmax loads a tile's scores with one 64-column tcgen05.ld");
constexpr int PF_STAGES = 2;    // K stages
constexpr int PF_VSTAGES = 3;   // V stages
constexpr int PF_SOFTMAX_THREADS = PF_M;               // one softmax thread per query row (two, each with half a tile's scores, measured slower)
constexpr int PF_THREADS = PF_SOFTMAX_THREADS + 64;   // + one warp that issues the MMAs + one that issues the TMA copies
constexpr int PF_Q_BYTES = PF_M * NCKV_D * 2;        // 32 KB: two 64-channel halves of [128][128 B]
constexpr int PF_KV_BYTES = PF_N * NCKV_D * 2;       // 16 KB: two halves of [64][128 B]
constexpr int PF_TMEM_COLS = 256;                    // S/P buffers: [0,64), [64,128)   O: [128,256)
constexpr unsigned long long PF_WAIT_LIMIT = NCKV_WAIT_LIMIT_NS;

struct PrefillParams {
    const int32_t *seqlens;  // may be null (all zero)
    __nv_bfloat16 *out;
    float *lse;  // optional (B, Hq, T_new): natural log of each row's sum of exponentials, -inf for a row without keys
    int32_t *status;
    int B, T_new, Hq, Hkv, T_k;
    int n_qtiles, n_items;
    int group_pairs;  // (row, q head) pairs per scheduling group, see the work order below
    int n_groups;     // the last group takes the remaining pairs (fewer than 2 group_pairs)
    int window_left;
    float scale_log2;
};

// One work item: PF_M query tokens of one (row, q head) and the key tiles they see.
struct PfItem {
    int hq, b, hkv, t0, L;
    int kv_lo, kv_hi;  // keys any row of the tile may see: [kv_lo, kv_hi)
    int n_tiles;
};

// Work order.  The CTAs are persistent (two per SM) and each takes a fixed subsequence of the item
// list, so every role of a CTA can enumerate its items without talking to the others.  Causal
// items differ in length by up to n_qtiles x; the list is ordered longest first inside groups of
// group_pairs (row, q head) pairs (sized on the host so that a group's K/V stays in L2 while its
// query tiles reuse it), and the list is dealt out back and forth (round r: item r G + c to CTA c
// when r is even, r G + G - 1 - c when odd), which evens out the sums without a shared counter.
__device__ __forceinline__ int pf_item_index(const PrefillParams &p, int seq) {
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    const long long base = (long long)seq * G;
    const long long idx = base + ((seq & 1) ? G - 1 - c : c);
    return idx < p.n_items ? (int)idx : -1;
}

__device__ __forceinline__ PfItem pf_item(const PrefillParams &p, int idx) {
    PfItem it;
    const int n_pairs = p.Hq * p.B;
    const int per_group = p.group_pairs * p.n_qtiles;
    const int grp = min(idx / per_group, p.n_groups - 1);
    const int in_grp = idx - grp * per_group;
    const int grp_pairs = grp == p.n_groups - 1 ? n_pairs - grp * p.group_pairs : p.group_pairs;
    const int qt = p.n_qtiles - 1 - in_grp / grp_pairs;  // all pairs' longest tiles first
    const int pair = grp * p.group_pairs + in_grp % grp_pairs;
    it.hq = pair % p.Hq;
    it.b = pair / p.Hq;
    it.hkv = it.hq / (p.Hq / p.Hkv);
    it.t0 = qt * PF_M;
    int L = p.seqlens ? p.seqlens[it.b] : 0;
    if (L < 0) L = 0;  // reported once by the set-up code
    it.L = L;
    int Tk = L + p.T_new;  // keys present after the append
    if (Tk > p.T_k) Tk = p.T_k;
    const int last_t = min(it.t0 + PF_M, p.T_new) - 1;
    it.kv_hi = min(Tk, L + last_t + 1);
    it.kv_lo = p.window_left >= 0 ? max(0, L + it.t0 - p.window_left) : 0;
    it.n_tiles = it.kv_hi > it.kv_lo ? (it.kv_hi - it.kv_lo + PF_N - 1) / PF_N : 0;
    return it;
}

// Position in a CTA's stream of key tiles: item number `seq` of the CTA, tile `t` inside it.  Items
// without any visible key are skipped (only the softmax warps look at them, to write zeros).
struct PfCursor {
    PfItem it;
    int seq, t;
    bool valid;
    __device__ __forceinline__ void load(const PrefillParams &p, int from_seq) {  // first non-empty item at or after from_seq
        t = 0;
        for (seq = from_seq;; ++seq) {
            const int idx = pf_item_index(p, seq);
            if (idx < 0) {
                valid = false;
                return;
            }
            it = pf_item(p, idx);
            if (it.n_tiles > 0) {
                valid = true;
                return;
            }
        }
    }
    __device__ __forceinline__ void advance(const PrefillParams &p) {
        if (++t >= it.n_tiles) load(p, seq + 1);
    }
    __device__ __forceinline__ bool last_of_item() const { return t == it.n_tiles - 1; }
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
    // All tile barriers are indexed by the GLOBAL tile number g of the CTA's stream (its items' tiles one
    // after the other): stage g % 2 or g % 3, buffer g & 1, and the phase parity follows from g as well.
    uint64_t *bar_q = bars;          // Q of an item landed (one phase per item)
    uint64_t *bar_k = bars + 1;      // [PF_STAGES] K tile landed
    uint64_t *bar_v = bars + 3;      // [PF_VSTAGES] V tile landed
    // [2] S(g) = Q K(g)^T complete, on bar_s[g & 1].  Products complete in issue order and S(g) is
    // issued behind O += P V(g-2), so this also says "P V(g-2) complete".
    uint64_t *bar_s = bars + 6;
    // [2] O += P V complete for the last (bar_o[0]) and the second last (bar_o[1]) tile of an item: no S
    // of the same item follows them.  One phase per item (bar_o[1]: per item of two or more tiles).
    uint64_t *bar_o = bars + 8;
    // [2] P(g) in TMEM, S(g) read, O rescaled: one arrival per softmax warp on bar_p[g & 1].
    uint64_t *bar_p = bars + 10;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 12);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5;

    pdl_wait_prior_grids();
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
    if (blockIdx.x == 0 && p.seqlens) {  // lengths out of range: reported once
        for (int b = tid; b < p.B; b += blockDim.x) {
            const int L = p.seqlens[b];
            if (L < 0) atomicOr(p.status, (int)NCKV_ST_BAD_SEQLEN);
            else if (L + p.T_new > p.T_k) atomicOr(p.status, (int)NCKV_ST_OVERFLOW);
        }
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
    auto timed_out = [&]() {
        *abort_flag = 1;
        atomicOr(p.status, (int)NCKV_ST_TIMEOUT);
    };
    auto par2 = [](uint32_t g) -> uint32_t { return (g >> 1) & 1u; };  // phase of a barrier indexed g & 1

    if (warp == PF_SOFTMAX_THREADS / 32 + 1) {
        // =============== one lane moves the tiles ===================================================
        if ((tid & 31) == 0) {
            PfCursor kc, vc, wc;  // next K tile to load, next V tile to load, tile whose score product is awaited
            kc.load(p, 0);
            vc = kc;
            wc = kc;
            uint32_t gk = 0, gv = 0;
            auto load_k = [&]() {
                const int stage = (int)(gk % PF_STAGES), key0 = kc.it.kv_lo + kc.t * PF_N;
                uint8_t *kd = sK + stage * PF_KV_BYTES;
                mbar_arrive_expect_tx(&bar_k[stage], PF_KV_BYTES);
                tma_load_4d(kd, &tmap_k, &bar_k[stage], 0, kc.it.hkv, key0, kc.it.b);
                tma_load_4d(kd + PF_KV_BYTES / 2, &tmap_k, &bar_k[stage], 64, kc.it.hkv, key0, kc.it.b);
                kc.advance(p);
                ++gk;
            };
            auto load_v = [&]() {
                const int stage = (int)(gv % PF_VSTAGES), key0 = vc.it.kv_lo + vc.t * PF_N;
                uint8_t *vd = sV + stage * PF_KV_BYTES;
                mbar_arrive_expect_tx(&bar_v[stage], PF_KV_BYTES);
                tma_load_4d(vd, &tmap_v, &bar_v[stage], 0, vc.it.hkv, key0, vc.it.b);
                tma_load_4d(vd + PF_KV_BYTES / 2, &tmap_v, &bar_v[stage], 64, vc.it.hkv, key0, vc.it.b);
                vc.advance(p);
                ++gv;
            };
            auto load_q = [&](const PfItem &it) {
                mbar_arrive_expect_tx(bar_q, PF_Q_BYTES);
                tma_load_4d(sQ, &tmap_q, bar_q, 0, it.hq, it.t0, it.b);
                tma_load_4d(sQ + PF_Q_BYTES / 2, &tmap_q, bar_q, 64, it.hq, it.t0, it.b);
            };
            bool ok = true;
            if (wc.valid) {
                load_q(wc.it);
                while (gk < PF_STAGES && kc.valid) load_k();
                while (gv < PF_VSTAGES && vc.valid) load_v();
                for (uint32_t g = 0; wc.valid && ok; ++g) {
                    // what S(g)'s completion releases: the Q buffer if g ends its item, K(g)'s stage for
                    // K(g+2) and, P V(g-2) being complete too, V(g-2)'s stage for V(g+1)
                    PfCursor nx;
                    nx.valid = false;
                    if (wc.last_of_item()) nx.load(p, wc.seq + 1);
                    if (!kc.valid && !vc.valid && !nx.valid) break;
                    ok = mbar_wait_bounded(&bar_s[g & 1], par2(g), PF_WAIT_LIMIT);
                    if (!ok) break;
                    if (nx.valid) load_q(nx.it);
                    if (kc.valid) load_k();
                    if (vc.valid && gv <= g + 1) load_v();
                    wc.advance(p);
                }
            }
            if (!ok) timed_out();
        }
        __syncwarp();
    } else if (issuer_warp) {
        // =============== one thread feeds the tensor core ==========================================
        // tcgen05.mma / tcgen05.commit are single-thread instructions and an mbarrier poll by 32 lanes
        // is 32 polls, one after the other: lane 0 runs this role alone.
        if ((tid & 31) == 0) {
            // Descriptors differ only in the start-address field (address >> 4 in the low 14 bits),
            // so they are built once and advanced by adding the byte offset >> 4.
            const uint64_t desc_q = smem_desc_sw128(smem_u32(sQ), 16, 1024);
            const uint64_t desc_k = smem_desc_sw128(smem_u32(sK), 16, 1024);
            const uint64_t desc_v = smem_desc_sw128(smem_u32(sV), PF_KV_BYTES / 2, 1024);
            PfCursor sc, pc;  // tile of the next score product, tile of the next P V product
            sc.load(p, 0);
            pc = sc;
            uint32_t gs = 0, gp = 0;
            uint32_t n_q = 0;  // items whose Q has been waited for
            // S(gs) = Q K(gs)^T into S buffer gs & 1, then arrive on bar_s[gs & 1]
            auto issue_s = [&]() -> bool {
                const uint32_t stage = gs % PF_STAGES;
                if (sc.t == 0) {  // first tile of an item: its Q
                    if (!mbar_wait_bounded(bar_q, n_q & 1u, PF_WAIT_LIMIT)) return false;
                    ++n_q;
                }
                if (!mbar_wait_bounded(&bar_k[stage], (gs / PF_STAGES) & 1u, PF_WAIT_LIMIT)) return false;
                tc_fence_after();
                const uint64_t dk = desc_k + (uint64_t)((stage * PF_KV_BYTES) >> 4);
                const uint32_t ds = tmem_s + (gs & 1u) * PF_N;
#pragma unroll
                for (int kk = 0; kk < NCKV_D / 16; ++kk) {
                    const uint32_t off = (uint32_t)(kk & 3) * 32;
                    const uint64_t da = desc_q + (uint64_t)(((kk >> 2) * (PF_Q_BYTES / 2) + off) >> 4);
                    const uint64_t db = dk + (uint64_t)(((kk >> 2) * (PF_KV_BYTES / 2) + off) >> 4);
                    umma_bf16(ds, da, db, IDESC_S, kk > 0 ? 1u : 0u);
                }
                umma_commit(&bar_s[gs & 1u]);
                sc.advance(p);
                ++gs;
                return true;
            };
            // S runs two tiles ahead of the softmax
            bool ok = true;
            if (sc.valid) ok = issue_s();
            if (ok && sc.valid) ok = issue_s();
            while (pc.valid && ok) {
                // P(gp) is in TMEM, S(gp) has been read, O carries the scale P was made with
                const uint32_t vstage = gp % PF_VSTAGES;
                ok = mbar_wait_bounded(&bar_p[gp & 1u], par2(gp), PF_WAIT_LIMIT) &&
                     mbar_wait_bounded(&bar_v[vstage], (gp / PF_VSTAGES) & 1u, PF_WAIT_LIMIT);
                if (!ok) break;
                tc_fence_after();
                // V in place: N (channels) contiguous, the two 64-channel halves PF_KV_BYTES/2 apart
                // (leading offset), 8-key groups 1024 B apart (stride offset)
                const uint64_t dv = desc_v + (uint64_t)((vstage * PF_KV_BYTES) >> 4);
                const uint32_t pbase = tmem_s + (gp & 1u) * PF_N;
#pragma unroll
                for (int ks = 0; ks < PF_N / 16; ++ks) {
                    // P(gp) sits in the first 32 columns of its S buffer; 16 keys = 8 columns
                    const uint64_t db = dv + (uint64_t)((ks * 16 * 128) >> 4);
                    umma_bf16_a_tmem(tmem_o, pbase + (uint32_t)ks * 8, db, IDESC_O, (pc.t > 0 || ks > 0) ? 1u : 0u);
                }
                // S(gp+2), issued behind this product into the S buffer P(gp) sits in, tells of its completion
                // too; the last two tiles of an item tell it themselves (the S behind them belongs to the next
                // item and may have to wait for that item's Q).
                const int from_end = pc.it.n_tiles - 1 - pc.t;
                if (from_end < 2) umma_commit(&bar_o[from_end]);
                if (sc.valid) ok = issue_s();
                pc.advance(p);
                ++gp;
            }
            if (!ok) timed_out();
        }
        __syncwarp();
    } else {
        // =============== softmax threads: one per query row =========================================
        const int row = tid & (PF_M - 1);  // query row inside the tile == TMEM lane
        bool aborted = false;
        uint32_t g = 0;  // global tile number of the current item's tile 0
        uint32_t n_o0 = 0, n_o1 = 0;  // phases of bar_o[0] / bar_o[1] used up by the items before this one
        // one lane polls (32 lanes polling one mbarrier are served one after the other), the warp follows
        auto warp_wait = [&](uint64_t *bar, uint32_t parity) -> bool {
            int ok = 1;
            if ((tid & 31) == 0) ok = mbar_wait_bounded(bar, parity, PF_WAIT_LIMIT) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            __syncwarp();  // orders the lanes' later reads of the tile behind lane 0's observation
            return ok != 0;
        };
        for (int seq = 0; !aborted; ++seq) {
            const int idx = pf_item_index(p, seq);
            if (idx < 0) break;
            const PfItem it = pf_item(p, idx);
            const int n_tiles = it.n_tiles;
            const int pos = it.L + it.t0 + row;  // absolute position of this row's token
            // P V of the item's tile t complete: told by S of tile t+2, issued behind it, or by bar_o for the
            // item's last two tiles
            auto pv_done = [&](int t) -> bool {
                const int from_end = n_tiles - 1 - t;
                const uint32_t x = g + (uint32_t)t;
                return from_end >= 2 ? warp_wait(&bar_s[(x + 2) & 1u], par2(x + 2)) : warp_wait(&bar_o[from_end], (from_end == 0 ? n_o0 : n_o1) & 1u);
            };
            // Softmax state of this thread's row.  P is scaled by m_used, which follows the true running
            // max lazily: it is only raised (and the O row in TMEM rescaled) when the max has grown by
            // more than 2^8, so exp2(s - m_used) stays <= 256 and most tiles need no rescale at all.
            float m_used = -INFINITY, l_run = 0.f;
            for (int t = 0; t < n_tiles; ++t) {
                const uint32_t gt = g + (uint32_t)t;
                const int stage = (int)(gt % PF_VSTAGES);
                const int key0 = it.kv_lo + t * PF_N;
                const uint32_t tmem_s_it = tmem_s + (uint32_t)(gt & 1) * PF_N;
                // tcgen05.ld/st are warp-wide (.sync.aligned): every decision that skips them is taken per warp
                if (*abort_flag != 0 || !warp_wait(&bar_s[gt & 1u], par2(gt))) {  // both uniform over the warp
                    aborted = true;
                    break;
                }
                tc_fence_after();

                float s_val[PF_N];
                tmem_ld64(tmem_s_it + lane_sel, s_val);  // raw q.k, scaled inside the exponent; one load, one wait
                // only tiles that touch the causal diagonal, the window edge or the end of the keys need
                // per-element masking (uniform over the CTA)
                const bool edge = (key0 + PF_N - 1 > it.L + it.t0) || (key0 + PF_N > it.kv_hi) ||
                                  (p.window_left >= 0 && key0 < it.L + it.t0 + PF_M - 1 - p.window_left);
                if (edge) {
                    // this row sees columns [c_lo, c_hi) of the tile
                    const int c_hi = min(pos, it.kv_hi - 1) - key0 + 1;
                    const int c_lo = p.window_left >= 0 ? pos - p.window_left - key0 : 0;
#pragma unroll
                    for (int c = 0; c < PF_N; ++c) s_val[c] = (c >= c_lo && c < c_hi) ? s_val[c] : -INFINITY;
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains instead of one
#pragma unroll
                for (int c = 0; c < PF_N; c += 8) {
                    mx4[0] = fmax3(mx4[0], s_val[c], s_val[c + 1]);
                    mx4[1] = fmax3(mx4[1], s_val[c + 2], s_val[c + 3]);
                    mx4[2] = fmax3(mx4[2], s_val[c + 4], s_val[c + 5]);
                    mx4[3] = fmax3(mx4[3], s_val[c + 6], s_val[c + 7]);
                }
                // the max is taken on raw scores and scaled once (the scale is positive)
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
                const bool raise = mx > m_used + 8.f;  // also the first tile that shows this row a key (m_used = -inf)
                const float alpha = raise ? ex2_approx(m_used - mx) : 1.f;  // 2^-inf = 0
                if (raise) {
                    l_run *= alpha;
                    m_used = mx;
                }
                const float m_use = m_used == -INFINITY ? 0.f : m_used;  // a row that has seen no key yet
                float2 rs01 = make_float2(0.f, 0.f), rs23 = make_float2(0.f, 0.f);
                const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), neg_m2 = make_float2(-m_use, -m_use);
                uint32_t pk[PF_N / 2];
#pragma unroll
                for (int c = 0; c < PF_N; c += 4) {
                    // 2^(s * scale - m): one two-wide FFMA per pair of scores, one MUFU.EX2 per score
                    const float2 x01 = ffma2(make_float2(s_val[c], s_val[c + 1]), scale2, neg_m2);
                    const float2 x23 = ffma2(make_float2(s_val[c + 2], s_val[c + 3]), scale2, neg_m2);
                    const float2 p01 = make_float2(ex2_approx(x01.x), ex2_approx(x01.y));
                    const float2 p23 = make_float2(ex2_approx(x23.x), ex2_approx(x23.y));
                    rs01 = fadd2(rs01, p01);
                    rs23 = fadd2(rs23, p23);
                    pk[c / 2] = pack_bf16x2(p01.x, p01.y);
                    pk[c / 2 + 1] = pack_bf16x2(p23.x, p23.y);
                }
                l_run += (rs01.x + rs01.y) + (rs23.x + rs23.y);

                // P row -> TMEM, over the first 32 columns of this tile's S buffer (this lane's own scores,
                // already in registers).  S of tile g+2 is issued behind P V(g) and lands on top of it.
                tmem_st_words(tmem_s_it + lane_sel, pk);
                // A raised scale: O (+)= P V of the previous tile must be complete before the O rows
                // accumulated so far are brought to the new scale (tcgen05.ld / multiply / tcgen05.st).
                // Every lane applies its own factor (1 for rows that keep their scale).
                if (t > 0 && __any_sync(0xffffffffu, raise)) {
                    if (!pv_done(t - 1)) {
                        timed_out();
                        aborted = true;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int ch = 0; ch < NCKV_D / 32; ++ch) {
                        float c[32];
                        tmem_ld32(tmem_o + lane_sel + ch * 32, c);
#pragma unroll
                        for (int i = 0; i < 32; ++i) c[i] *= alpha;
                        tmem_st32(tmem_o + lane_sel + ch * 32, c);
                    }
                }
                // rows of the V tile past the last key may hold stale bytes: zero them so that a zero
                // probability never multiplies a NaN/Inf bit pattern
                if (key0 + PF_N > it.kv_hi) {
                    uint8_t *vd = sV + stage * PF_KV_BYTES;
                    if (warp_wait(&bar_v[stage], (gt / PF_VSTAGES) & 1u)) {
                        for (int i = tid; i < (key0 + PF_N - it.kv_hi) * 16; i += PF_SOFTMAX_THREADS) {
                            const int r = (it.kv_hi - key0) + i / 16, ch = i % 16;
                            *reinterpret_cast<uint4 *>(vd + (ch >> 3) * (PF_KV_BYTES / 2) + r * 128 + ((ch & 7) << 4)) =
                                make_uint4(0, 0, 0, 0);
                        }
                    }
                    fence_proxy_async_smem();  // the zeroed V rows must be visible to the tensor core
                }
                tc_fence_before();  // orders this thread's TMEM loads/stores before the next MMAs
                __syncwarp();
                if ((tid & 31) == 0) mbar_arrive(&bar_p[gt & 1]);  // one arrival per warp
            }
            if (aborted) break;

            // ---- epilogue of the item -------------------------------------------------------------
            const int tq = it.t0 + row;
            if (n_tiles > 0) {
                if (!pv_done(n_tiles - 1)) {
                    timed_out();
                    aborted = true;
                    break;
                }
                tc_fence_after();
            }
            const float inv = (n_tiles > 0 && l_run > 0.f) ? 1.f / l_run : 0.f;
            if (p.lse && tq < p.T_new)  // m_used and l_run are in powers of two
                p.lse[((long long)it.b * p.Hq + it.hq) * p.T_new + tq] =
                    (n_tiles > 0 && l_run > 0.f) ? (m_used + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
            uint4 *dst = reinterpret_cast<uint4 *>(p.out + (((long long)it.b * p.T_new + tq) * p.Hq + it.hq) * NCKV_D);
#pragma unroll
            for (int ch = 0; ch < NCKV_D / 64; ++ch) {
                float c[64];
                if (n_tiles > 0) {
                    tmem_ld64(tmem_o + lane_sel + ch * 64, c);
                } else {
#pragma unroll
                    for (int i = 0; i < 64; ++i) c[i] = 0.f;
                }
                if (tq < p.T_new) {  // rows past the end of the sequence are padding
#pragma unroll
                    for (int i = 0; i < 4; ++i) {  // 32 bytes per store: whole sectors
                        uint32_t w[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) w[e] = pack_bf16x2(c[16 * i + 2 * e] * inv, c[16 * i + 2 * e + 1] * inv);
                        st_global_v8(dst + (ch * 4 + i) * 2, w);
                    }
                }
            }
            // O is read: order those loads before the first P V of the next item, which overwrites it and
            // is only issued after this thread's next arrival on bar_p
            tc_fence_before();
            g += (uint32_t)n_tiles;
            n_o0 += n_tiles >= 1;
            n_o1 += n_tiles >= 2;
        }
        if (aborted && *abort_flag == 0) timed_out();  // a wait ran out in this warp
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, PF_TMEM_COLS);
}

static size_t prefill_smem_bytes() {
    return PF_Q_BYTES + (PF_STAGES + PF_VSTAGES) * PF_KV_BYTES + 13 * sizeof(uint64_t);
}

}  // namespace nckv


static int prefill_launch(const void *q, const void *k, const void *v, const int32_t *cache_seqlens, void *out,
                          float *lse, int B, int T_new, int Hq, int Hkv, int D, int T_k, int64_t kv_batch_stride,
                          int64_t kv_token_stride, int window_left, int32_t *status, void *stream) {
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
    p.lse = lse;
    p.status = status;
    p.B = B; p.T_new = T_new; p.Hq = Hq; p.Hkv = Hkv; p.T_k = T_k;
    p.window_left = window_left;
    p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)D));
    const int n_items = n_qtiles * Hq * B;
    const int grid = n_items < 2 * sm_count() ? n_items : 2 * sm_count();  // two CTAs per SM, persistent
    p.n_qtiles = n_qtiles;
    p.n_items = n_items;
    {
        // Pairs per group.  Everything in one group when all K and V rows (512 B per key and kv head,
        // shared by Hq / Hkv q heads) are 40 MB or less, a third of L2; else groups of about that size,
        // rounded down to one whose item count is a multiple of twice the grid, so that the
        // back-and-forth deal hands every CTA the same mix of long and short tiles.  The last group
        // takes the remainder as well.
        const long long keys = window_left >= 0 && window_left + PF_M < T_k ? window_left + PF_M : T_k;
        const long long bytes_per_pair = keys * 512 / (Hq / Hkv) + 1;
        const long long pairs = (long long)Hq * B;
        const long long rep = Hq / Hkv;  // keep the q heads of a kv head in one group
        long long g = pairs;
        if (pairs * bytes_per_pair > (40LL << 20)) {
            g = (40LL << 20) / bytes_per_pair;
            g -= g % rep;
            long long a = 2LL * grid, b = n_qtiles;
            while (b) { const long long t = a % b; a = b; b = t; }  // a = gcd(2 grid, n_qtiles)
            long long unit = 2LL * grid / a;                         // pairs per balanced deal
            { long long x = unit, y = rep; while (y) { const long long t = x % y; x = y; y = t; } unit = unit / x * rep; }
            if (g >= unit) g -= g % unit;
            if (g < rep) g = rep;
            if (g > pairs) g = pairs;
        }
        p.n_groups = (int)(pairs / g);  // >= 1; the last group also takes the pairs / g remainder
        p.group_pairs = (int)g;
    }

    const size_t smem = prefill_smem_bytes();
    static bool attr_set[64] = {false};
    int dev = 0;
    NCKV_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        NCKV_CUDA_CHECK(cudaFuncSetAttribute(prefill_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
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

extern "C" int nckv_prefill_attn(const void *q, const void *k, const void *v, const int32_t *cache_seqlens,
                                 void *out, int B, int T_new, int Hq, int Hkv, int D, int T_k,
                                 int64_t kv_batch_stride, int64_t kv_token_stride, int window_left,
                                 int32_t *status, void *stream) {
    return prefill_launch(q, k, v, cache_seqlens, out, nullptr, B, T_new, Hq, Hkv, D, T_k, kv_batch_stride,
                          kv_token_stride, window_left, status, stream);
}

// Forward of flash_attn_func for training: the same kernel over plain (B, T, H, D) tensors, which also
// writes the log-sum-exp of every row for the backward pass.
extern "C" int nckv_flash_attn_fwd(const void *q, const void *k, const void *v, void *out, float *lse, int B, int T,
                                   int Hq, int Hkv, int D, int window_left, int32_t *status, void *stream) {
    if (!lse) {
        nckv::set_error("flash_attn_fwd: null lse pointer");
        return NCKV_E_ARG;
    }
    return prefill_launch(q, k, v, nullptr, out, lse, B, T, Hq, Hkv, D, T, (int64_t)T * Hkv * D, (int64_t)Hkv * D,
                          window_left, status, stream);
}
