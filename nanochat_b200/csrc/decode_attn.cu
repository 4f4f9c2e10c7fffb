// Kernel (b): split-KV decode attention (one query token per row), HBM-bandwidth bound.
//
// Work decomposition.  Keys of row b are cut into tiles of DEC_TILE tokens starting at the first
// visible key; the tiles of all (row, kv-head) pairs form one flat sequence (row outer, head
// middle, tile inner) of `total` tiles.  The sequence is handed out as RUNS of consecutive tiles:
//   * the sequence is cut into one equal slice per warp of the persistent grid (DEC_CTAS_PER_SM CTAs
//     per SM, DEC_WARPS warps each); the first 60% of a slice is that warp's static run, so a warp
//     starts without any global traffic;
//   * the last 40% of every slice is cut into small runs that warps claim from an atomic ticket counter (drawn one
//     run ahead, so the round trip is hidden) when they finish what they have.  SMs do not all
//     see the same HBM bandwidth (two dies, distance to the stacks); the dynamic part lets the
//     fast ones absorb the difference.
// A warp is a self-contained stream processor: lane 0 issues TMA tile loads (K and V, 128-byte
// swizzle, L2 evict-first) into the warp's private ring of DEC_STAGES shared-memory stages (48 keys x
// 512 B = 24 KB each; 2 CTAs x 2 warps x 2 stages = 192 KB in flight per SM; measured best of the
// tile/stage/warp splits of that budget on B200.  Two small CTAs per SM instead of one large one let
// the next launch's CTAs move in, and start their first loads, as soon as half an SM is done),
// completion is signalled on the warp's own mbarriers, and the loads run ahead across pair and
// run boundaries.  There is no CTA-wide synchronisation after set-up and no fence or wait on
// another warp anywhere in the stream.
//
// Math per tile.  All G = Hq/Hkv query heads that share a kv head are the rows of one
// m16n8k16 tile (rows >= G are zero), so K/V bytes are read once per group.  S = Q K^T and
// O += P V use the warp-level bf16 MMA with fp32 accumulation; running max / sum use quad
// shuffles; P is rounded to bf16 for the second product, as the flash-style library kernels do.
//
// Combine.  A pair whose tiles all fall inside one run is normalised and written directly.
// Otherwise every run that touches the pair leaves an un-normalised partial (O, m, l) in the
// workspace; which runs exist is a pure function of cache_seqlens, so a second, tiny kernel
// (decode_merge_kernel, one warp per (row, q head)) recomputes the cut and merges the partials
// with a log-sum-exp.  It is launched with programmatic dependent launch: its set-up overlaps the
// tail of the streaming kernel.
//
// Replaces: flash_attention.py:83-89 (Tq == 1 branch of _sdpa_attention) reached through
// flash_attention.py:165-177, with the per-row cache_seqlens contract of flash_attention.py:142.
#include <math.h>

#include "nckv_common.cuh"

namespace nckv {

#ifndef NCKV_DEC_TILE
#define NCKV_DEC_TILE 48
#endif
#ifndef NCKV_DEC_STAGES
#define NCKV_DEC_STAGES 2
#endif
#ifndef NCKV_DEC_WARPS
#define NCKV_DEC_WARPS 2
#endif
constexpr int DEC_TILE = NCKV_DEC_TILE;      // keys per tile (multiple of 16)
constexpr int DEC_STAGES = NCKV_DEC_STAGES;  // tiles in flight per warp
constexpr int DEC_WARPS = NCKV_DEC_WARPS;    // warps (independent streams) per CTA
#ifndef NCKV_DEC_CTAS_PER_SM
#define NCKV_DEC_CTAS_PER_SM 2
#endif
constexpr int DEC_CTAS_PER_SM = NCKV_DEC_CTAS_PER_SM;  // CTAs of the persistent grid per SM
#ifndef NCKV_DEC_MAX_B
#define NCKV_DEC_MAX_B 1024
#endif
constexpr int DEC_MAX_B = NCKV_DEC_MAX_B; // rows per launch (bounds the shared-memory row tables)
constexpr int DEC_HALF_BYTES = DEC_TILE * 128;        // one 64-channel half of a K or V tile
constexpr int DEC_STAGE_BYTES = 4 * DEC_HALF_BYTES;   // K lo, K hi, V lo, V hi
constexpr int DEC_STATUS_BYTES = 256;                 // status word, then the ticket counter at +16
constexpr int DEC_RING = 4;                           // runs a warp may have claimed but not finished
constexpr int DEC_DYN_PER_WARP = 4;                   // at most this many dynamic runs per warp of the grid
#ifndef NCKV_DEC_STATIC_NUM
#define NCKV_DEC_STATIC_NUM 6
#endif
#ifndef NCKV_DEC_MIN_RUN
#define NCKV_DEC_MIN_RUN 2
#endif
constexpr int DEC_STATIC_NUM = NCKV_DEC_STATIC_NUM, DEC_STATIC_DEN = 10; // statically assigned fraction of a slice
constexpr int DEC_MIN_RUN = NCKV_DEC_MIN_RUN;  // tiles in the smallest dynamic run
#ifndef NCKV_DEC_PREFETCH
#define NCKV_DEC_PREFETCH 2
#endif
constexpr int DEC_PREFETCH = NCKV_DEC_PREFETCH;  // tiles of the static run a warp asks L2 for before it may start
constexpr int MERGE_WARPS = 8;
constexpr int MERGE_BATCH = 16; // O rows fetched per round trip
constexpr int MERGE_PLAN = 4;  // chunks of 32 parts whose record slots a merge warp works out ahead of time

struct DecodeParams {
    const __nv_bfloat16 *q;
    const int32_t *seqlens;
    __nv_bfloat16 *out;
    float *out_f32;
    float *lse;
    int32_t *status;
    int32_t *run_counter;  // dynamic run tickets; zero on entry, zero on exit
    float *partials;       // 2 records per run, rec_floats each
    int B, Hq, Hkv, G, T_max;
    int seqlen_offset, window_left, kv_begin, kv_end;
    KvSplit split;         // block > 0: seqlens are global lengths, the cache holds this shard's block-cyclic part
    // paged storage (block_table != null): the caches are pools of pages (n_pages, page_tokens, Hkv, D);
    // token t of row b lives in page block_table[b * max_pages + t / page_tokens] at t % page_tokens.
    // page_tokens is a multiple of DEC_TILE and tiles are cut on the DEC_TILE grid, so a tile never
    // straddles two pages.
    const int32_t *block_table;
    int page_tokens, max_pages, n_pages;
    int rec_floats;
    int W;                 // warps of the streaming grid (the run geometry depends on it)
    float scale_log2;
};

struct TileCursor {
    int b, h, j, nt;
};

struct RunEntry {  // one claimed run, handed from the issuing side of a warp to its consuming side
    int k, n;      // run id, tiles
    TileCursor start;
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

// Cursor of flat tile index x: the row is the largest b with Hkv * pref[b] <= x.  Called by a whole
// warp: lanes test 32 candidate rows at a time and vote.
__device__ __forceinline__ TileCursor locate_tile(const int *s_pref, int B, int Hkv, int x) {
    const int lane = threadIdx.x & 31;
    int row = 0;
    for (int base = 0; base < B; base += 32) {
        const int b = base + lane;
        const bool le = b < B && Hkv * s_pref[b] <= x;
        const unsigned m = __ballot_sync(0xffffffffu, le);
        if (m == 0) break;            // prefix sums are non-decreasing: nothing further can qualify
        row = base + 31 - __clz(m);   // highest qualifying row of this block
        if (m != 0xffffffffu) break;
    }
    TileCursor c;
    c.b = row;
    c.nt = s_pref[row + 1] - s_pref[row];
    const int rel = x - Hkv * s_pref[row];
    c.h = rel / c.nt;
    c.j = rel - c.h * c.nt;
    return c;
}

// How the flat tile sequence [0, total) is cut into runs.  A pure function of (total, W), so the
// streaming kernel and the merge kernel agree on it.
//   slice w (w < W) = q + (w < r) consecutive tiles, q = total / W, r = total % W
//   static run w    = the first 60% of slice w (all of it when the slice is shorter than 4 tiles)
//   dynamic runs    = the rest of each slice in chunks of CH tiles, numbered in tile order
// Interleaving static and dynamic stretches keeps the number of runs that touch any one
// (row, head) pair small, which bounds the work of the merge.
struct RunGeometry {
    int total, W;
    int q, r;            // slice lengths
    int s_big, s_small;  // static tiles of a slice of q+1 / q tiles
    int d_big, d_small;  // dynamic runs of a slice of q+1 / q tiles
    int CH, n_dyn;

    __device__ __forceinline__ static int static_part(int n) { return n < 4 ? n : (n * DEC_STATIC_NUM) / DEC_STATIC_DEN; }
    __device__ __forceinline__ void init(int total_, int W_) {
        total = total_;
        W = W_;
        q = total / W;
        r = total - q * W;
        s_big = static_part(q + 1);
        s_small = static_part(q);
        const int tail = (q + 1) - s_big;  // the longest dynamic stretch
        CH = max(DEC_MIN_RUN, (tail + DEC_DYN_PER_WARP - 1) / DEC_DYN_PER_WARP);
        d_big = (q + 1 - s_big + CH - 1) / CH;
        d_small = (q - s_small + CH - 1) / CH;
        n_dyn = r * d_big + (W - r) * d_small;
    }
    __device__ __forceinline__ int slice_lo(int w) const { return w * q + min(w, r); }
    __device__ __forceinline__ int slice_len(int w) const { return q + (w < r ? 1 : 0); }
    __device__ __forceinline__ int slice_of(int x) const {
        const int big = r * (q + 1);
        return x < big ? x / (q + 1) : r + (x - big) / q;
    }
    // dynamic run id k >= W  ->  (slice, chunk within the slice's dynamic stretch)
    __device__ __forceinline__ void dyn_split(int k, int &w, int &c) const {
        const int idx = k - W;
        const int big = r * d_big;
        if (idx < big) {
            w = idx / d_big;
            c = idx - w * d_big;
        } else {
            w = r + (idx - big) / d_small;
            c = (idx - big) - (w - r) * d_small;
        }
    }
    __device__ __forceinline__ void run_range(int k, int &lo, int &len) const {
        if (k < W) {
            lo = slice_lo(k);
            len = k < r ? s_big : s_small;
            return;
        }
        int w, c;
        dyn_split(k, w, c);
        const int st = w < r ? s_big : s_small;
        lo = slice_lo(w) + st + c * CH;
        len = min(CH, slice_len(w) - st - c * CH);
    }
    __device__ __forceinline__ int run_of(int x) const {  // the run that holds tile x
        const int w = slice_of(x);
        const int off = x - slice_lo(w);
        const int st = w < r ? s_big : s_small;
        if (off < st) return w;
        const int c = (off - st) / CH;
        return W + (w < r ? w * d_big : r * d_big + (w - r) * d_small) + c;
    }
};

// Entries per shared-memory row table of a launch with B rows (B + 1 are used; a multiple of 32 keeps
// the tables aligned).  Sizing them by the launch instead of by DEC_MAX_B keeps room on the SM for the
// merge grid to be resident beside the streaming CTAs at ordinary batch sizes.
__host__ __device__ inline int table_rows(int B) { return (B + 1 + 31) & ~31; }

// Per-row visible key range [s_start, s_end) and the exclusive prefix sum of tiles per row
// (s_pref, B + 1 entries), computed by a whole CTA.  Ends with a __syncthreads().
// With paged storage s_start is the tile origin (the first visible key rounded down to the tile grid)
// and s_head the number of keys of tile 0 in front of the first visible one (0 otherwise).
__device__ __forceinline__ void build_row_tables(const DecodeParams &p, int *s_start, int *s_end, int *s_pref,
                                                 int *s_head, bool report) {
    const int tid = threadIdx.x, lane = tid & 31, B = p.B;
    for (int b = tid; b < B; b += blockDim.x) {
        int n = p.seqlens[b] + p.seqlen_offset;
        if (n < 0) {
            if (report) atomicOr(p.status, (int)NCKV_ST_BAD_SEQLEN);
            n = 0;
        }
        if (p.split.block > 0) n = owned_below(n, p.split.world, p.split.rank, p.split.block);
        if (n > p.T_max) {
            if (report) atomicOr(p.status, (int)NCKV_ST_OVERFLOW);
            n = p.T_max;
        }
        int lo = 0, hi = n;
        if (p.window_left >= 0) lo = max(0, n - 1 - p.window_left);
        if (p.kv_end > p.kv_begin) {
            lo = max(lo, p.kv_begin);
            hi = min(hi, p.kv_end);
        }
        if (hi < lo) hi = lo;
        const int origin = p.block_table ? (hi > lo ? (lo / DEC_TILE) * DEC_TILE : lo) : lo;
        s_start[b] = origin;
        s_end[b] = hi;
        s_head[b] = lo - origin;
    }
    __syncthreads();
    if (tid < 32) {  // exclusive prefix sum of tiles per row
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
}


// Paged storage: tile starting at key `key0` of row b -> (token inside its page, page).  A page number
// outside the pool is reported and replaced by the pool size, a coordinate the copy fills with zeros.
__device__ __forceinline__ void page_coords(const DecodeParams &p, int b, int key0, int &tok, int &page) {
    const int idx = key0 / p.page_tokens;
    tok = key0 - idx * p.page_tokens;
    page = __ldg(p.block_table + (long long)b * p.max_pages + idx);
    if (page < 0 || page >= p.n_pages) {
        atomicOr(p.status, (int)NCKV_ST_BAD_PAGE);
        page = p.n_pages;
    }
}

// GHI: group size 9..16 (rows 8..15 of the MMA tile carry heads too).  MAP5: the tensor maps are the
// 5-D form (one copy per K or V tile) instead of the 4-D form (one copy per 64-channel half).
// PAGED: block-table storage (always with the 5-D maps, whose outermost coordinate is then the page).
template <bool GHI, bool MAP5, bool PAGED = false>
__global__ void __launch_bounds__(DEC_WARPS * 32, DEC_CTAS_PER_SM)
decode_attn_kernel(const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const DecodeParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits 4..9
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint8_t *stages = smem;  // [DEC_WARPS][DEC_STAGES][DEC_STAGE_BYTES]
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(stages + DEC_WARPS * DEC_STAGES * DEC_STAGE_BYTES);
    RunEntry *rings = reinterpret_cast<RunEntry *>(full_bar + DEC_WARPS * DEC_STAGES);  // [DEC_WARPS][DEC_RING]
    int *s_start = reinterpret_cast<int *>(rings + DEC_WARPS * DEC_RING);  // four tables of table_rows(B) entries
    int *s_end = s_start + table_rows(p.B);
    int *s_pref = s_end + table_rows(p.B);  // B + 1 entries
    int *s_head = s_pref + table_rows(p.B);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int B = p.B, Hkv = p.Hkv, G = p.G;

    // ---- set-up ---------------------------------------------------------------------------------
    if (tid == 0) {
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
        for (int i = 0; i < DEC_WARPS * DEC_STAGES; ++i) mbar_init(&full_bar[i], 1);
        fence_mbar_init();
    }
    // Programmatic dependent launch: this grid may be running while the kernels before it in the
    // stream (the append kernel; the tail and the merge kernel of a previous call) still are.
    // What is read before wait_prior() below is only what none of them writes: cache_seqlens and
    // keys/values older than the last max(seqlen_offset, 1) visible positions of a row (the rows a
    // decode step's append kernel may have written).  q, the appended rows, the run counter
    // and every store come after it.  Dependents (the merge kernel) are released after the wait,
    // so that a grid that can start early always finds its predecessor's predecessors complete.
    build_row_tables(p, s_start, s_end, s_pref, s_head, blockIdx.x == 0);
    bool prior_done = false;
    auto wait_prior = [&]() {  // called warp-uniformly
        if (!prior_done) {
            pdl_wait_prior_grids();
            pdl_launch_dependents();  // the merge kernel may be scheduled and run its own set-up now
            prior_done = true;
        }
    };

    RunGeometry geo;
    geo.init(Hkv * s_pref[B], p.W);
    const int gw = blockIdx.x * DEC_WARPS + warp;

    {
        // rows without any visible key: zero output, lse = -inf (only sharded calls can produce them)
        bool any_empty = false;
        for (int b = blockIdx.x; b < B; b += gridDim.x) any_empty |= s_pref[b + 1] == s_pref[b];
        if (any_empty) {  // uniform over the CTA
            wait_prior();
            for (int b = blockIdx.x; b < B; b += gridDim.x) {
                if (s_pref[b + 1] != s_pref[b]) continue;
                for (int i = tid; i < p.Hq * NCKV_D; i += blockDim.x) {
                    const long long o = (long long)b * p.Hq * NCKV_D + i;
                    if (p.out) p.out[o] = __float2bfloat16(0.0f);
                    if (p.out_f32) p.out_f32[o] = 0.0f;
                }
                if (p.lse) for (int i = tid; i < p.Hq; i += blockDim.x) p.lse[(long long)b * p.Hq + i] = -INFINITY;
            }
        }
    }
    if (geo.total == 0) return;  // every warp of the grid takes this exit together

    uint8_t *my_stages = stages + warp * DEC_STAGES * DEC_STAGE_BYTES;
    uint64_t *my_bar = full_bar + warp * DEC_STAGES;
    RunEntry *my_ring = rings + warp * DEC_RING;
    const uint64_t kv_policy = l2_policy_evict_first();

    // ---- issuing side: claims runs, keeps DEC_STAGES tile loads in flight --------------------
    TileCursor prod = {0, 0, 0, 0};
    int prod_left = 0;       // tiles of the current run not yet issued
    int ring_push = 0, ring_pop = 0;
    int issue_idx = 0;       // tiles issued so far (stage = idx % DEC_STAGES)
    bool first_claim = true, sched_done = false, have_ticket = false;
    unsigned stage_dirty = 0;  // lane 0: stages whose V rows were zeroed by ordinary stores
    int next_ticket = 0;     // lane 0 only: a dynamic ticket drawn ahead of need, so its latency is hidden

    auto claim_run = [&]() -> int {  // next run id for this warp; >= W + n_dyn means "no more"
        if (first_claim) {  // the static run; the first ticket is drawn once its loads are in flight
            first_claim = false;
            return gw;
        }
        if (!have_ticket) {  // only when the static run was empty
            wait_prior();  // the counter belongs to the previous launch until that has completed
            if (lane == 0) next_ticket = atomicAdd(p.run_counter, 1);
            have_ticket = true;
        }
        const int t = __shfl_sync(0xffffffffu, next_ticket, 0);
        // Tickets n_dyn .. n_dyn + W - 1 are the W terminating ones, one per warp (a warp stops
        // drawing at its first); whoever holds the last knows nobody will draw again and re-arms
        // the counter for the next launch.
        if (t < geo.n_dyn) {
            if (lane == 0) next_ticket = atomicAdd(p.run_counter, 1);
        } else if (t == geo.n_dyn + geo.W - 1 && lane == 0) {
            *p.run_counter = 0;
        }
        return geo.W + t;
    };

    auto issue_one = [&]() -> bool {  // issue the next tile load if there is one
        if (prod_left == 0) {
            if (sched_done) return false;
            int k, n, run_lo;
            for (;;) {
                k = claim_run();
                if (k >= geo.W + geo.n_dyn) {
                    sched_done = true;
                    return false;
                }
                geo.run_range(k, run_lo, n);
                if (n > 0) break;  // only a static run can be empty (fewer tiles than warps)
            }
            prod = locate_tile(s_pref, B, Hkv, run_lo);
            prod_left = n;
            if (lane == 0) {
                RunEntry e;
                e.k = k; e.n = n; e.start = prod;
                my_ring[ring_push % DEC_RING] = e;
            }
            ++ring_push;
            __syncwarp();
        }
        const int key0 = s_start[prod.b] + prod.j * DEC_TILE;
        int tok = key0, outer = prod.b;  // token and outermost (row or page) coordinate of the tile
        if (PAGED) page_coords(p, prod.b, key0, tok, outer);
        // A tile that reaches the rows appended by this step has to wait for the append kernel.
        // With seqlen_offset == 0 the caller has already counted the new token in cache_seqlens
        // (the sequence-split path does): the last visible position is then the appended one.
        if (!prior_done && key0 + DEC_TILE > s_end[prod.b] - max(p.seqlen_offset, 1)) wait_prior();
        if (lane == 0) {
            const int stage = issue_idx % DEC_STAGES;
            uint8_t *dst = my_stages + stage * DEC_STAGE_BYTES;
            uint64_t *bar = &my_bar[stage];
            // the only generic-proxy writes to a stage are the zeroed V rows of a tail tile; order
            // them before the bulk copy that reuses the stage
            if (stage_dirty & (1u << stage)) {
                fence_proxy_async_smem();
                stage_dirty &= ~(1u << stage);
            }
            mbar_arrive_expect_tx(bar, DEC_STAGE_BYTES);
            // K/V bytes are used once: evict-first keeps them from flushing q and the partial
            // records out of L2
            if (MAP5) {
                tma_load_5d_hint(dst, &tmap_k, bar, 0, tok, 0, prod.h, outer, kv_policy);
                tma_load_5d_hint(dst + 2 * DEC_HALF_BYTES, &tmap_v, bar, 0, tok, 0, prod.h, outer, kv_policy);
            } else {
                tma_load_4d_hint(dst, &tmap_k, bar, 0, prod.h, key0, prod.b, kv_policy);
                tma_load_4d_hint(dst + DEC_HALF_BYTES, &tmap_k, bar, 64, prod.h, key0, prod.b, kv_policy);
                tma_load_4d_hint(dst + 2 * DEC_HALF_BYTES, &tmap_v, bar, 0, prod.h, key0, prod.b, kv_policy);
                tma_load_4d_hint(dst + 3 * DEC_HALF_BYTES, &tmap_v, bar, 64, prod.h, key0, prod.b, kv_policy);
            }
        }
        ++issue_idx;
        --prod_left;
        cursor_advance(prod, s_pref, B, Hkv);
        return true;
    };

    // The first loads of the static run go out before the wait: they overlap the append kernel and,
    // in back-to-back calls, the tail and the merge of the previous call.
    issue_one();
    while (issue_idx < DEC_STAGES && prod_left > 0 && issue_one()) {
    }
    // The ring is full, yet the kernels in front may need a few more microseconds (and, once this
    // grid may go on, its first loads are behind it): ask L2 for the next tiles of the static run so
    // that HBM keeps working through the hand-over.  Purely a hint; the copies into shared memory
    // are issued as usual and then hit L2.  A prefetched line that the append kernel writes
    // afterwards is updated in L2, which is where every later read of it is served from.
    if (DEC_PREFETCH > 0 && lane == 0) {
        TileCursor pc = prod;
        int left = prod_left;
        for (int i = 0; i < DEC_PREFETCH && left > 0; ++i, --left) {
            const int key0 = s_start[pc.b] + pc.j * DEC_TILE;
            if (MAP5) {
                int tok = key0, outer = pc.b;
                if (PAGED) page_coords(p, pc.b, key0, tok, outer);
                tma_prefetch_l2_5d(&tmap_k, 0, tok, 0, pc.h, outer);
                tma_prefetch_l2_5d(&tmap_v, 0, tok, 0, pc.h, outer);
            } else {
                tma_prefetch_l2_4d(&tmap_k, 0, pc.h, key0, pc.b);
                tma_prefetch_l2_4d(&tmap_k, 64, pc.h, key0, pc.b);
                tma_prefetch_l2_4d(&tmap_v, 0, pc.h, key0, pc.b);
                tma_prefetch_l2_4d(&tmap_v, 64, pc.h, key0, pc.b);
            }
            cursor_advance(pc, s_pref, B, Hkv);
        }
    }
    wait_prior();
    if (!have_ticket) {  // needed once the static run has been issued; by then it has long arrived
        if (lane == 0) next_ticket = atomicAdd(p.run_counter, 1);
        have_ticket = true;
    }
    while (issue_idx < DEC_STAGES && issue_one()) {
    }

    // ---- consuming side -----------------------------------------------------------------------
    const int g = lane >> 2;  // MMA row within 8 (query head within the group)
    const int t4 = lane & 3;
    uint32_t qa[8][GHI ? 4 : 2];  // A fragments of Q for the 8 k-steps over D
    float o_acc[16][4];
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};
    TileCursor cons = {0, 0, 0, 0};
    int cons_left = 0, cons_k = 0;
    int cons_idx = 0;
    int seg_j0 = 0;
    bool run_begin = false, timed_out = false;

    while (cons_idx < issue_idx) {
        if (cons_left == 0) {
            const RunEntry e = my_ring[ring_pop % DEC_RING];
            ++ring_pop;
            cons = e.start;
            cons_k = e.k;
            cons_left = e.n;
            run_begin = true;
        }
        const int stage = cons_idx % DEC_STAGES;
        const uint32_t parity = (uint32_t)((cons_idx / DEC_STAGES) & 1);
        const bool seg_begin = run_begin || (cons.j == 0);
        run_begin = false;
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
                    qa[kk][GHI ? 2 : 0] = (g + 8) < G ? __ldg(r1) : 0u;
                    qa[kk][GHI ? 3 : 1] = (g + 8) < G ? __ldg(r1 + 4) : 0u;
                }
            }
        }

        if (!mbar_wait_bounded(&my_bar[stage], parity)) {
            timed_out = true;
            break;
        }

        const uint32_t kbase = smem_u32(my_stages + stage * DEC_STAGE_BYTES);
        const uint32_t vbase = kbase + 2 * DEC_HALF_BYTES;
        const int key0 = s_start[cons.b] + cons.j * DEC_TILE;
        const int nvalid = min(DEC_TILE, s_end[cons.b] - key0);
        const int nskip = (PAGED && cons.j == 0) ? s_head[cons.b] : 0;  // keys of the tile in front of the window

        if (nvalid < DEC_TILE) {
            // Tail tile: rows past the last visible key may hold stale bytes; zero V there so a
            // zero probability never meets a NaN/Inf bit pattern.
            uint8_t *vb = my_stages + stage * DEC_STAGE_BYTES + 2 * DEC_HALF_BYTES;
            if (lane < 16) {
                for (int r = nvalid; r < DEC_TILE; ++r)
                    *reinterpret_cast<uint4 *>(vb + (lane >> 3) * DEC_HALF_BYTES + r * 128 + (lane & 7) * 16) =
                        make_uint4(0, 0, 0, 0);
            }
            stage_dirty |= 1u << stage;
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
            if (k0 >= nvalid || (PAGED && k0 < nskip)) { s_acc[nb][0] = -INFINITY; s_acc[nb][2] = -INFINITY; }
            if (k0 + 1 >= nvalid || (PAGED && k0 + 1 < nskip)) { s_acc[nb][1] = -INFINITY; s_acc[nb][3] = -INFINITY; }
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

        // ---- this stage is free again: keep the ring of loads full ----
        ++cons_idx;
        --cons_left;
        __syncwarp();
        issue_one();

        // ---- end of this pair's stretch inside the run? ----
        const bool seg_end = (cons_left == 0) || (cons.j == cons.nt - 1);
        if (seg_end) {
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
                        if (p.out) *reinterpret_cast<uint32_t *>(p.out + o) = pack_bf16x2(v0, v1);
                        if (p.out_f32) *reinterpret_cast<float2 *>(p.out_f32 + o) = make_float2(v0, v1);
                    }
                    if (GHI && g + 8 < G) {
                        const long long o = (row_base + g + 8) * NCKV_D + d;
                        const float v0 = o_acc[nd][2] * inv1, v1 = o_acc[nd][3] * inv1;
                        if (p.out) *reinterpret_cast<uint32_t *>(p.out + o) = pack_bf16x2(v0, v1);
                        if (p.out_f32) *reinterpret_cast<float2 *>(p.out_f32 + o) = make_float2(v0, v1);
                    }
                }
                if (p.lse && t4 == 0) {
                    if (g < G) p.lse[row_base + g] = (m_run[0] + log2f(l0)) * 0.69314718055994531f;
                    if (GHI && g + 8 < G) p.lse[row_base + g + 8] = (m_run[1] + log2f(l1)) * 0.69314718055994531f;
                }
            } else {
                // partial record: [G][128] un-normalised O, then m[G], l[G]; a run leaves at most
                // two (one where it starts inside a pair, one where it ends inside a pair).  Plain
                // stores: the merge kernel only runs after this grid has completed.
                const int slot = 2 * cons_k + (seg_j0 == 0 ? 1 : 0);
                float *rec = p.partials + (long long)slot * p.rec_floats;
#pragma unroll
                for (int nd = 0; nd < 16; ++nd) {
                    const int d = nd * 8 + 2 * t4;
                    if (g < G) *reinterpret_cast<float2 *>(rec + g * NCKV_D + d) = make_float2(o_acc[nd][0], o_acc[nd][1]);
                    if (GHI && g + 8 < G)
                        *reinterpret_cast<float2 *>(rec + (g + 8) * NCKV_D + d) = make_float2(o_acc[nd][2], o_acc[nd][3]);
                }
                if (t4 == 0) {
                    if (g < G) { rec[G * NCKV_D + g] = m_run[0]; rec[G * NCKV_D + G + g] = l0; }
                    if (GHI && g + 8 < G) { rec[G * NCKV_D + g + 8] = m_run[1]; rec[G * NCKV_D + G + g + 8] = l1; }
                }
            }
        }
        cursor_advance(cons, s_pref, B, Hkv);
    }

    if (timed_out) {
        if (lane == 0) atomicOr(p.status, (int)NCKV_ST_TIMEOUT);
        // give copies already issued a bounded chance to land before the CTA's memory is released
        for (int s = 0; s < DEC_STAGES; ++s) mbar_wait_bounded(&my_bar[s], 0, 1000000ull);
        // leave the ticket counter consistent: draw (without working on them) until this warp
        // has taken its terminating ticket
        for (int guard = 0; !sched_done && guard < geo.n_dyn + geo.W + 1; ++guard) {
            if (claim_run() >= geo.W + geo.n_dyn) sched_done = true;
        }
    }
}

// The row tables of a launch, copied out for inspection.
__global__ void __launch_bounds__(128) decode_key_ranges_kernel(const DecodeParams p, int32_t *key_begin,
                                                                int32_t *key_end) {
    extern __shared__ int s_tables[];
    int *s_start = s_tables, *s_end = s_start + table_rows(p.B), *s_pref = s_end + table_rows(p.B);
    int *s_head = s_pref + table_rows(p.B);
    build_row_tables(p, s_start, s_end, s_pref, s_head, true);
    for (int b = threadIdx.x; b < p.B; b += blockDim.x) {
        key_begin[b] = s_start[b] + s_head[b];
        key_end[b] = s_end[b];
    }
}

// Where the merged result goes when the keys are split across GPUs: besides the local buffers, the
// packed fp32 partial ([rows][128] output | [rows] log-sum-exp) is stored into slot (step parity,
// rank) of every peer's exchange buffer with plain peer stores, and the last block to finish
// releases the per-(parity, rank) flag on every peer with the step number.  world == 0: off.
struct PushDesc {
    PeerPtrs peers;
    const unsigned *step_counter;  // completed exchange steps (advanced by the wait/combine kernel)
    unsigned *done;                // blocks of the merge grid that have finished; zero on entry and exit
    long long per;                 // floats per (parity, rank) slot
    int world, rank, rows;
};

// Block-table storage of a launch (table == null: dense caches).
struct PagedDesc {
    const int32_t *table;
    int page_tokens, max_pages, n_pages;
};

// Merge of the partial records.  An item is one (row, q head); WPI warps work on it (1: a warp per
// item, for batches of many short pairs; MERGE_WARPS: a block per item, for few long pairs whose
// tiles were spread over dozens of runs).  Which records belong to a pair follows from cache_seqlens
// alone.  The runs that can touch the pair's tile range [P0, P1) are enumerated as CANDIDATES
// (slice w, r) with r = 0 the static run of the slice and r = 1.. its dynamic runs, D1 = 1 + d_big
// per slice; candidate c = 32 * chunk + lane is looked after by one lane, which works out on its own
// (no walk over the runs) whether that run exists and meets the pair, and in which record slot it left
// its partial.  The slots of a warp's first chunks are worked out BEFORE the grid-dependency wait,
// while the streaming kernel is still running; after the wait only loads, shuffles and the store remain.
// Candidates are merged in index order, so the result does not depend on timing.
template <int WPI>
__global__ void __launch_bounds__(MERGE_WARPS * 32) decode_merge_kernel(const DecodeParams p,
                                                                        const __grid_constant__ PushDesc pd) {
    extern __shared__ int s_tables[];
    int *s_start = s_tables, *s_end = s_start + table_rows(p.B), *s_pref = s_end + table_rows(p.B);
    int *s_head = s_pref + table_rows(p.B);
    // WPI > 1: the warps' partial merges (M, L, 128 channels) and their part counts
    float *s_comb = reinterpret_cast<float *>(s_head + table_rows(p.B));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int B = p.B, Hkv = p.Hkv, G = p.G;
    pdl_launch_dependents();  // whatever follows in the stream may be scheduled behind this grid
    // cache_seqlens is stable by now: the streaming kernel only lets this grid start after it has
    // itself waited for its predecessor
    build_row_tables(p, s_start, s_end, s_pref, s_head, false);
    RunGeometry geo;
    geo.init(Hkv * s_pref[B], p.W);
    const int n_items = B * p.Hq;
    const int first_item = WPI == 1 ? blockIdx.x * MERGE_WARPS + warp : blockIdx.x;
    const int item_stride = WPI == 1 ? gridDim.x * MERGE_WARPS : gridDim.x;
    const int sub = WPI == 1 ? 0 : warp;  // this warp's share of an item's chunks: sub, sub + WPI, ...
    const int D1 = 1 + geo.d_big;

    struct ItemRange {
        int P0, P1, w0, n_chunks, hg;
    };
    auto item_range = [&](int item) -> ItemRange {
        ItemRange r;
        const int b = item / p.Hq, hq = item - b * p.Hq;
        const int h = hq / G;
        r.hg = hq - h * G;
        const int nt = s_pref[b + 1] - s_pref[b];
        r.P0 = Hkv * s_pref[b] + h * nt;
        r.P1 = r.P0 + nt;
        r.w0 = 0;
        r.n_chunks = 0;
        if (nt > 0 && geo.total > 0) {  // nt == 0: no visible key, the streaming kernel wrote zeros
            r.w0 = geo.slice_of(r.P0);
            r.n_chunks = ((geo.slice_of(r.P1 - 1) - r.w0 + 1) * D1 + 31) >> 5;
        }
        return r;
    };
    // record slot of candidate `cand` of the item, or -1 if that run does not exist or misses the pair
    auto cand_slot = [&](const ItemRange &r, int cand) -> int {
        const int w = r.w0 + cand / D1, rr = cand - (cand / D1) * D1;
        if (w >= geo.W) return -1;
        const int st = w < geo.r ? geo.s_big : geo.s_small;
        const int slice_lo = geo.slice_lo(w), slice_len = geo.slice_len(w);
        int k, lo, len;
        if (rr == 0) {
            k = w;
            lo = slice_lo;
            len = st;
        } else {
            const int c = rr - 1;
            if (c >= (w < geo.r ? geo.d_big : geo.d_small)) return -1;
            k = geo.W + (w < geo.r ? w * geo.d_big : geo.r * geo.d_big + (w - geo.r) * geo.d_small) + c;
            lo = slice_lo + st + c * geo.CH;
            len = min(geo.CH, slice_len - st - c * geo.CH);
        }
        if (len <= 0 || lo >= r.P1 || lo + len <= r.P0) return -1;
        return 2 * k + (lo <= r.P0 ? 1 : 0);
    };

    ItemRange cur = {0, 0, 0, 0, 0};
    int plan_slots[MERGE_PLAN];
#pragma unroll
    for (int c = 0; c < MERGE_PLAN; ++c) plan_slots[c] = -1;
    if (first_item < n_items) {
        cur = item_range(first_item);
#pragma unroll
        for (int c = 0; c < MERGE_PLAN; ++c) {
            const int chunk = sub + c * WPI;
            if (chunk < cur.n_chunks) plan_slots[c] = cand_slot(cur, chunk * 32 + lane);
        }
    }

    pdl_wait_prior_grids();  // the streaming kernel has completed and its records are visible
    const bool push = pd.world > 0;
    if (geo.total == 0 && !push) return;
    // The exchange step this call belongs to.  The counter is only advanced by the wait/combine
    // kernel of the previous step, which completed before the kernels in front of this grid ran.
    const unsigned step = push ? *pd.step_counter + 1u : 0u;
    const long long push_off = push ? ((long long)(step & 1u) * pd.world + pd.rank) * pd.per : 0;
    auto push_row = [&](int item, const float4 &row, float lse_v) {
        for (int r = 0; r < pd.world; ++r) {
            float *dst = pd.peers.buf[r] + push_off;
            reinterpret_cast<float4 *>(dst + (long long)item * NCKV_D)[lane] = row;
            if (lane == 0) dst[(long long)pd.rows * NCKV_D + item] = lse_v;
        }
    };

    for (int item = first_item; item < n_items; item += item_stride) {
        if (item != first_item) cur = item_range(item);
        const int hg = cur.hg;
        float M = -INFINITY, L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int nparts = 0;
        for (int ci = 0, chunk = sub; chunk < cur.n_chunks; ++ci, chunk += WPI) {
            int my_slot;
            if (item == first_item && ci < MERGE_PLAN) {
                my_slot = plan_slots[0];
#pragma unroll
                for (int c = 1; c < MERGE_PLAN; ++c)
                    if (ci == c) my_slot = plan_slots[c];
            } else {
                my_slot = cand_slot(cur, chunk * 32 + lane);
            }
            const unsigned live = __ballot_sync(0xffffffffu, my_slot >= 0);
            if (live == 0) continue;
            nparts += __popc(live);
            float m_i = -INFINITY, l_i = 0.f;
            if (my_slot >= 0) {
                const float *r2 = p.partials + (long long)my_slot * p.rec_floats;
                m_i = __ldcg(r2 + G * NCKV_D + hg);
                l_i = __ldcg(r2 + G * NCKV_D + G + hg);
            }
            // O rows of the live candidates in batches of MERGE_BATCH loads issued back to back (one round
            // trip per batch instead of one per part); the first batch is in flight during the reductions
            float4 v[MERGE_BATCH];
            unsigned todo = live;
            int src[MERGE_BATCH];
            auto fetch = [&]() {
#pragma unroll
                for (int u = 0; u < MERGE_BATCH; ++u) {
                    src[u] = todo ? __ffs(todo) - 1 : -1;
                    if (todo) todo &= todo - 1;
                    const int slot_j = __shfl_sync(0xffffffffu, my_slot, src[u] < 0 ? 0 : src[u]);
                    v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (src[u] >= 0)
                        v[u] = __ldcg(reinterpret_cast<const float4 *>(p.partials + (long long)slot_j * p.rec_floats + hg * NCKV_D) + lane);
                }
            };
            fetch();
            float cm = m_i;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, off));
            const float newM = fmaxf(M, cm);
            const float rescale = exp2f(M - newM);  // first chunk: exp2(-inf) = 0
            const float sc = my_slot >= 0 ? exp2f(m_i - newM) : 0.f;
            float cl = sc * l_i;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) cl += __shfl_xor_sync(0xffffffffu, cl, off);
            L = L * rescale + cl;
            acc.x *= rescale; acc.y *= rescale; acc.z *= rescale; acc.w *= rescale;
            M = newM;
            for (;;) {
#pragma unroll
                for (int u = 0; u < MERGE_BATCH; ++u) {
                    const float s_j = __shfl_sync(0xffffffffu, sc, src[u] < 0 ? 0 : src[u]);
                    if (src[u] >= 0) {
                        acc.x = fmaf(s_j, v[u].x, acc.x); acc.y = fmaf(s_j, v[u].y, acc.y);
                        acc.z = fmaf(s_j, v[u].z, acc.z); acc.w = fmaf(s_j, v[u].w, acc.w);
                    }
                }
                if (todo == 0) break;
                fetch();
            }
        }
        if (WPI > 1) {
            // combine the warps' shares in warp order: [warp][M, L, count, pad, 128 channels]
            float *mine = s_comb + warp * (NCKV_D + 4);
            if (lane == 0) { mine[0] = M; mine[1] = L; mine[2] = (float)nparts; }
            reinterpret_cast<float4 *>(mine + 4)[lane] = acc;
            __syncthreads();
            if (warp == 0) {
                M = -INFINITY; L = 0.f; nparts = 0;
                acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int w2 = 0; w2 < WPI; ++w2) {
                    const float *o = s_comb + w2 * (NCKV_D + 4);
                    const float m2 = o[0], l2 = o[1];
                    nparts += (int)o[2];
                    if (m2 == -INFINITY) continue;
                    const float newM = fmaxf(M, m2);
                    const float ra = exp2f(M - newM), rb = exp2f(m2 - newM);
                    const float4 v2 = reinterpret_cast<const float4 *>(o + 4)[lane];
                    acc.x = acc.x * ra + v2.x * rb; acc.y = acc.y * ra + v2.y * rb;
                    acc.z = acc.z * ra + v2.z * rb; acc.w = acc.w * ra + v2.w * rb;
                    L = L * ra + l2 * rb;
                    M = newM;
                }
            }
            __syncthreads();
            if (warp != 0) continue;
        }
        if (nparts <= 1) {
            // written by the streaming kernel itself (one run held the whole pair, or no key is visible)
            if (push)
                push_row(item, __ldcg(reinterpret_cast<const float4 *>(p.out_f32 + (long long)item * NCKV_D) + lane),
                         __ldcg(p.lse + item));
            continue;
        }
        const float inv = 1.f / L;
        acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
        const long long o = (long long)item * NCKV_D + lane * 4;
        uint2 packed;
        packed.x = pack_bf16x2(acc.x, acc.y);
        packed.y = pack_bf16x2(acc.z, acc.w);
        if (p.out) *reinterpret_cast<uint2 *>(p.out + o) = packed;
        if (p.out_f32) *reinterpret_cast<float4 *>(p.out_f32 + o) = acc;
        const float lse_v = (M + log2f(L)) * 0.69314718055994531f;
        if (p.lse && lane == 0) p.lse[item] = lse_v;
        if (push) push_row(item, acc, lse_v);
    }
    if (push) {
        // every block's peer stores are ordered before its count; the last block orders all counts
        // before the flags it releases
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned prev = atomicAdd(pd.done, 1u);
            if (prev == gridDim.x - 1) {
                *pd.done = 0;
                __threadfence_system();
                for (int r = 0; r < pd.world; ++r) {
                    unsigned *flags = reinterpret_cast<unsigned *>(pd.peers.buf[r] + 2LL * pd.world * pd.per);
                    unsigned *f = flags + (step & 1u) * pd.world + pd.rank;
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(step) : "memory");
                }
            }
        }
    }
}

static size_t table_smem_bytes(int B) { return 4 * (size_t)table_rows(B) * sizeof(int); }
static size_t decode_smem_bytes(int B) {
    return 1024 + (size_t)DEC_WARPS * DEC_STAGES * DEC_STAGE_BYTES + DEC_WARPS * DEC_STAGES * sizeof(uint64_t) +
           DEC_WARPS * DEC_RING * sizeof(RunEntry) + table_smem_bytes(B);
}

// Workspace layout: [0,256) status word and ticket counter; then the partial records, two per run,
// (1 + DEC_DYN_PER_WARP) * W runs at most.
// One partial record: [G][128] fp32 O, then m[G] and l[G], padded so records stay 16-byte aligned.
static int rec_floats_for(int G) { return G * NCKV_D + ((2 * G + 3) & ~3); }
static size_t ws_partial_bytes(int G) {
    const size_t runs = (size_t)(1 + DEC_DYN_PER_WARP) * sm_count() * DEC_CTAS_PER_SM * DEC_WARPS + 2;
    return 2 * runs * (size_t)rec_floats_for(G) * sizeof(float);
}


template <typename Kernel, typename... Args>
static cudaError_t launch_pdl(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

}  // namespace nckv

extern "C" {


size_t nckv_workspace_bytes(int B, int Hq, int Hkv, int D) {
    using namespace nckv;
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || D != NCKV_D || Hq % Hkv) return 0;
    return DEC_STATUS_BYTES + ws_partial_bytes(Hq / Hkv);
}

// Argument checks shared by the decode-attention entry points (nothing is enqueued here).
static int decode_check(const void *q, const void *k_cache, const void *v_cache, const int32_t *cache_seqlens,
                        const void *out, const float *out_f32, const void *workspace, int B, int Hq, int Hkv, int D,
                        int T_max, size_t workspace_bytes) {
    using namespace nckv;
    if (!q || !k_cache || !v_cache || !cache_seqlens || (!out && !out_f32) || !workspace) {
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
    if ((long long)B * Hkv * ((T_max + DEC_TILE - 1) / DEC_TILE) >= (1LL << 30)) {
        set_error("decode_attn: B*Hkv*T_max too large for 32-bit tile arithmetic");
        return NCKV_E_UNSUPPORTED;
    }
    const size_t need = nckv_workspace_bytes(B, Hq, Hkv, D);
    if (workspace_bytes < need) {
        set_error("decode_attn: workspace of %zu bytes given, %zu needed", workspace_bytes, need);
        return NCKV_E_CAPACITY;
    }
    return NCKV_OK;
}

static int decode_launch(const void *q, const void *k_cache, const void *v_cache, const int32_t *cache_seqlens,
                         void *out, float *out_f32, float *lse_out, int B, int Hq, int Hkv, int D, int T_max,
                         int64_t cache_batch_stride, int64_t cache_token_stride, int seqlen_offset, int window_left,
                         int kv_begin, int kv_end, nckv::KvSplit split, const nckv::PushDesc &push, void *workspace,
                         size_t workspace_bytes, void *stream, nckv::PagedDesc paged = nckv::PagedDesc{nullptr, 0, 0, 0}) {
    using namespace nckv;
    int rc0 = decode_check(q, k_cache, v_cache, cache_seqlens, out, out_f32, workspace, B, Hq, Hkv, D, T_max,
                           workspace_bytes);
    if (rc0 != NCKV_OK) return rc0;
    const int G = Hq / Hkv;
    // dense: the maps span (rows, T_max tokens); paged: (pages of the pool, page_tokens tokens)
    const int map_outer = paged.table ? paged.n_pages : B, map_tokens = paged.table ? paged.page_tokens : T_max;
    // Prefer the 5-D maps (one copy instruction per tile and tensor); if this driver does not accept
    // their stride order, use the 4-D maps (two per tile and tensor).  Decided once per process.
    // (A plain int shared by all host threads: concurrent first calls would both probe and store the
    // same answer.)
    static int map5_state = 0;  // 0 unknown, 1 usable, -1 refused
    CUtensorMap mk, mv;
    int rc = NCKV_E_CUDA;
    if (map5_state >= 0) {
        rc = make_kv_tensor_map_5d(&mk, k_cache, map_outer, map_tokens, Hkv, cache_batch_stride, cache_token_stride, DEC_TILE);
        if (rc == NCKV_OK)
            rc = make_kv_tensor_map_5d(&mv, v_cache, map_outer, map_tokens, Hkv, cache_batch_stride, cache_token_stride, DEC_TILE);
        if (rc == NCKV_E_ARG) return rc;
        if (map5_state == 0) map5_state = rc == NCKV_OK ? 1 : -1;
    }
    const bool map5 = rc == NCKV_OK;
    if (!map5 && paged.table) {
        set_error("decode_attn_paged: this driver does not accept the 5-D tensor maps the paged kernels use");
        return NCKV_E_UNSUPPORTED;
    }
    if (!map5) {
        rc = make_kv_tensor_map(&mk, k_cache, B, T_max, Hkv, cache_batch_stride, cache_token_stride, DEC_TILE);
        if (rc != NCKV_OK) return rc;
        rc = make_kv_tensor_map(&mv, v_cache, B, T_max, Hkv, cache_batch_stride, cache_token_stride, DEC_TILE);
        if (rc != NCKV_OK) return rc;
    }

    const int grid = sm_count() * DEC_CTAS_PER_SM;
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    DecodeParams p;
    p.q = static_cast<const __nv_bfloat16 *>(q);
    p.seqlens = cache_seqlens;
    p.out = static_cast<__nv_bfloat16 *>(out);
    p.out_f32 = out_f32;
    p.lse = lse_out;
    p.status = reinterpret_cast<int32_t *>(ws);
    p.run_counter = reinterpret_cast<int32_t *>(ws + 16);
    p.partials = reinterpret_cast<float *>(ws + DEC_STATUS_BYTES);
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.T_max = T_max;
    p.seqlen_offset = seqlen_offset;
    p.window_left = window_left;
    p.kv_begin = kv_begin;
    p.kv_end = kv_end;
    p.split = split;
    p.block_table = paged.table;
    p.page_tokens = paged.page_tokens;
    p.max_pages = paged.max_pages;
    p.n_pages = paged.n_pages;
    p.rec_floats = rec_floats_for(G);
    p.W = grid * DEC_WARPS;
    p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)D));

    const size_t smem = decode_smem_bytes(B), smem_max = decode_smem_bytes(DEC_MAX_B);
    static bool attr_set[64] = {false};  // per device; setting the attribute twice from racing threads is harmless
    int dev = 0;
    NCKV_CUDA_CHECK(cudaGetDevice(&dev));
    const bool ghi = G > 8;
    if (dev < 64 && !attr_set[dev]) {
        NCKV_CUDA_CHECK(cudaFuncSetAttribute(decode_attn_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
        NCKV_CUDA_CHECK(cudaFuncSetAttribute(decode_attn_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
        NCKV_CUDA_CHECK(cudaFuncSetAttribute(decode_attn_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
        NCKV_CUDA_CHECK(cudaFuncSetAttribute(decode_attn_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
        NCKV_CUDA_CHECK(cudaFuncSetAttribute(decode_attn_kernel<true, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
        NCKV_CUDA_CHECK(cudaFuncSetAttribute(decode_attn_kernel<false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
        attr_set[dev] = true;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Both launches allow programmatic overlap with their predecessor in the stream: each kernel
    // runs its set-up early and waits (griddepcontrol.wait) before it touches dependent data.
    const dim3 g3(grid), b3(DEC_WARPS * 32);
    if (paged.table && ghi) NCKV_CUDA_CHECK(launch_pdl(decode_attn_kernel<true, true, true>, g3, b3, smem, s, true, mk, mv, p));
    else if (paged.table) NCKV_CUDA_CHECK(launch_pdl(decode_attn_kernel<false, true, true>, g3, b3, smem, s, true, mk, mv, p));
    else if (ghi && map5) NCKV_CUDA_CHECK(launch_pdl(decode_attn_kernel<true, true>, g3, b3, smem, s, true, mk, mv, p));
    else if (ghi) NCKV_CUDA_CHECK(launch_pdl(decode_attn_kernel<true, false>, g3, b3, smem, s, true, mk, mv, p));
    else if (map5) NCKV_CUDA_CHECK(launch_pdl(decode_attn_kernel<false, true>, g3, b3, smem, s, true, mk, mv, p));
    else NCKV_CUDA_CHECK(launch_pdl(decode_attn_kernel<false, false>, g3, b3, smem, s, true, mk, mv, p));
    const int items = B * Hq;
    PushDesc pd = push;
    pd.done = reinterpret_cast<unsigned *>(ws + 32);
    // Few long (row, kv head) pairs: their tiles are spread over many runs each (about 4 runs per slice
    // of the W a pair spans), so a block merges one item; otherwise a warp does.
    const size_t merge_smem = table_smem_bytes(B) + MERGE_WARPS * (NCKV_D + 4) * sizeof(float);
    if ((long long)B * Hkv * 4 <= p.W) {
        const int merge_grid = items < 8 * sm_count() ? items : 8 * sm_count();
        NCKV_CUDA_CHECK(launch_pdl(decode_merge_kernel<MERGE_WARPS>, dim3(merge_grid), dim3(MERGE_WARPS * 32), merge_smem, s, true, p, pd));
    } else {
        int merge_grid = (items + MERGE_WARPS - 1) / MERGE_WARPS;
        if (merge_grid > 4 * sm_count()) merge_grid = 4 * sm_count();
        NCKV_CUDA_CHECK(launch_pdl(decode_merge_kernel<1>, dim3(merge_grid), dim3(MERGE_WARPS * 32), merge_smem, s, true, p, pd));
    }
    return NCKV_OK;
}

int nckv_decode_attn(const void *q, const void *k_cache, const void *v_cache,
                     const int32_t *cache_seqlens, void *out, float *out_f32, float *lse_out,
                     int B, int Hq, int Hkv, int D, int T_max, int64_t cache_batch_stride,
                     int64_t cache_token_stride, int seqlen_offset, int window_left,
                     int kv_begin, int kv_end, void *workspace, size_t workspace_bytes,
                     void *stream) {
    if (!out) {
        nckv::set_error("decode_attn: null pointer argument");
        return NCKV_E_ARG;
    }
    nckv::PushDesc none = {};
    return decode_launch(q, k_cache, v_cache, cache_seqlens, out, out_f32, lse_out, B, Hq, Hkv, D, T_max,
                         cache_batch_stride, cache_token_stride, seqlen_offset, window_left, kv_begin, kv_end,
                         nckv::KvSplit{0, 0, 0}, none, workspace, workspace_bytes, stream);
}

int nckv_decode_attn_paged(const void *q, const void *k_pool, const void *v_pool, const int32_t *block_table,
                           const int32_t *cache_seqlens, void *out, float *out_f32, float *lse_out, int B, int Hq,
                           int Hkv, int D, int page_tokens, int max_pages, int n_pages, int64_t page_stride,
                           int64_t token_stride, int seqlen_offset, int window_left, void *workspace,
                           size_t workspace_bytes, void *stream) {
    using namespace nckv;
    if (!out || !block_table) {
        set_error("decode_attn_paged: null pointer argument");
        return NCKV_E_ARG;
    }
    if (page_tokens <= 0 || (page_tokens % DEC_TILE) != 0 || max_pages <= 0 || n_pages <= 0) {
        set_error("decode_attn_paged: page_tokens=%d must be a positive multiple of %d, max_pages=%d and n_pages=%d positive",
                  page_tokens, DEC_TILE, max_pages, n_pages);
        return NCKV_E_ARG;
    }
    if ((long long)page_tokens * max_pages > 0x3fffffffLL) {
        set_error("decode_attn_paged: page_tokens * max_pages too large");
        return NCKV_E_UNSUPPORTED;
    }
    PushDesc none = {};
    return decode_launch(q, k_pool, v_pool, cache_seqlens, out, out_f32, lse_out, B, Hq, Hkv, D, page_tokens * max_pages,
                         page_stride, token_stride, seqlen_offset, window_left, 0, 0, KvSplit{0, 0, 0}, none, workspace,
                         workspace_bytes, stream, PagedDesc{block_table, page_tokens, max_pages, n_pages});
}

int nckv_paged_tile_tokens(void) { return nckv::DEC_TILE; }

int nckv_decode_attn_split(const void *q, const void *k_cache, const void *v_cache, const int32_t *cache_seqlens,
                           float *part_out, float *part_lse, int B, int Hq, int Hkv, int D, int T_local,
                           int64_t cache_batch_stride, int64_t cache_token_stride, int seqlen_offset, int world,
                           int rank, int block, void *const *peer_bufs, const uint32_t *step_counter,
                           void *workspace, size_t workspace_bytes, void *stream) {
    using namespace nckv;
    if (!part_out || !part_lse) {
        set_error("decode_attn_split: part_out and part_lse are required");
        return NCKV_E_ARG;
    }
    if (world <= 0 || world > NCKV_MAX_PEERS || rank < 0 || rank >= world || block <= 0) {
        set_error("decode_attn_split: bad split (world=%d rank=%d block=%d)", world, rank, block);
        return NCKV_E_ARG;
    }
    PushDesc pd = {};
    if (peer_bufs) {
        if (!step_counter) {
            set_error("decode_attn_split: step_counter is required with peer_bufs");
            return NCKV_E_ARG;
        }
        for (int i = 0; i < world; ++i) {
            pd.peers.buf[i] = static_cast<float *>(peer_bufs[i]);
            if (!pd.peers.buf[i] || ((uintptr_t)pd.peers.buf[i] & 15)) {
                set_error("decode_attn_split: peer buffer %d is null or misaligned", i);
                return NCKV_E_ARG;
            }
        }
        pd.step_counter = step_counter;
        pd.world = world;
        pd.rank = rank;
        pd.rows = B * Hq;
        pd.per = p2p_per_floats(B * Hq);
    }
    return decode_launch(q, k_cache, v_cache, cache_seqlens, nullptr, part_out, part_lse, B, Hq, Hkv, D, T_local,
                         cache_batch_stride, cache_token_stride, seqlen_offset, -1, 0, 0, KvSplit{world, rank, block},
                         pd, workspace, workspace_bytes, stream);
}

// ---- decode attention for callers that must not allocate ----------------------------------------
// Scratch lives in this file-scope device array instead of a caller-provided workspace.  Every GPU
// that loads the library carries it until the process exits.
#define NCKV_STATIC_SCRATCH_BYTES (14u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[NCKV_STATIC_SCRATCH_BYTES];

extern "C" int nckv_decode_key_ranges(const int32_t *cache_seqlens, int B, int T_max, int seqlen_offset,
                                      int window_left, int kv_begin, int kv_end, int split_world, int split_rank,
                                      int split_block, int32_t *key_begin, int32_t *key_end, int32_t *status,
                                      void *stream) {
    using namespace nckv;
    if (!cache_seqlens || !key_begin || !key_end || !status) {
        set_error("decode_key_ranges: null pointer argument");
        return NCKV_E_ARG;
    }
    if (B <= 0 || B > DEC_MAX_B || T_max <= 0) {
        set_error("decode_key_ranges: B=%d must be in 1..%d and T_max=%d positive", B, DEC_MAX_B, T_max);
        return NCKV_E_ARG;
    }
    if (split_block < 0 || (split_block > 0 && (split_world <= 0 || split_rank < 0 || split_rank >= split_world))) {
        set_error("decode_key_ranges: bad split (world=%d rank=%d block=%d)", split_world, split_rank, split_block);
        return NCKV_E_ARG;
    }
    DecodeParams p = {};
    p.split = KvSplit{split_world, split_rank, split_block};
    p.seqlens = cache_seqlens;
    p.status = status;
    p.B = B;
    p.T_max = T_max;
    p.seqlen_offset = seqlen_offset;
    p.window_left = window_left;
    p.kv_begin = kv_begin;
    p.kv_end = kv_end;
    decode_key_ranges_kernel<<<1, 128, table_smem_bytes(B), static_cast<cudaStream_t>(stream)>>>(p, key_begin, key_end);
    NCKV_CUDA_CHECK(cudaGetLastError());
    return NCKV_OK;
}

int nckv_decode_attn_static(const void *q, const void *k_cache, const void *v_cache,
                            const int32_t *cache_seqlens, void *out, float *out_f32, float *lse_out,
                            int B, int Hq, int Hkv, int D, int T_max, int64_t cache_batch_stride,
                            int64_t cache_token_stride, int seqlen_offset, int window_left,
                            int kv_begin, int kv_end, void **status_word, void *stream) {
    using namespace nckv;
    if (!out) {
        set_error("decode_attn_static: null pointer argument");
        return NCKV_E_ARG;
    }
    // In host code `g_static_scratch` is only a handle; the address kernels can use has to be
    // asked for, once per device, with that device current.  (Racing first calls from two host
    // threads would both store the same address.)
    static void *dev_ptr[64] = {nullptr};
    int dev = 0;
    NCKV_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_error("decode_attn_static: device index %d out of range", dev);
        return NCKV_E_UNSUPPORTED;
    }
    if (dev_ptr[dev] == nullptr) {
        void *ptr = nullptr;
        NCKV_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_static_scratch));
        dev_ptr[dev] = ptr;
    }
    const size_t need = nckv_workspace_bytes(B, Hq, Hkv, D);
    if (need == 0 || need > (size_t)NCKV_STATIC_SCRATCH_BYTES) {
        set_error("decode_attn_static: this shape needs %zu bytes of scratch, the built-in array holds %u "
                  "(group size Hq/Hkv up to 4 fits); use nckv_decode_attn with a workspace instead",
                  need, (unsigned)NCKV_STATIC_SCRATCH_BYTES);
        return need == 0 ? NCKV_E_UNSUPPORTED : NCKV_E_CAPACITY;
    }
    unsigned char *base = static_cast<unsigned char *>(dev_ptr[dev]);
    if (status_word) *status_word = base;
    // reject bad arguments before anything touches the shared array
    const int chk = decode_check(q, k_cache, v_cache, cache_seqlens, out, out_f32, base, B, Hq, Hkv, D, T_max,
                                 NCKV_STATIC_SCRATCH_BYTES);
    if (chk != NCKV_OK) return chk;
    // The array keeps whatever the previous call left.  The ticket counter must start at zero (it
    // returns to zero by itself unless a call was cut short); the partial records need no clearing,
    // every record that is read was written by the same call.
    NCKV_CUDA_CHECK(cudaMemsetAsync(base + 16, 0, sizeof(int32_t), static_cast<cudaStream_t>(stream)));
    return nckv_decode_attn(q, k_cache, v_cache, cache_seqlens, out, out_f32, lse_out, B, Hq, Hkv, D, T_max,
                            cache_batch_stride, cache_token_stride, seqlen_offset, window_left, kv_begin, kv_end,
                            base, NCKV_STATIC_SCRATCH_BYTES, stream);
}

}  // extern "C"
