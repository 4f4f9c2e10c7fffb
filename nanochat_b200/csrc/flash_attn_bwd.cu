// Backward of flash_attn_func (causal, optional sliding window, GQA) on the 5th-generation tensor cores.
//
//   delta[b, h, t] = sum_c dO * O                                       (attn_bwd_delta_kernel)
//   P = exp(S / sqrt(D) - lse),  dP = dO V^T,  dS = P o (dP - delta) / sqrt(D)
//   dV = P^T dO,  dK = dS^T Q                                          (attn_bwd_dkdv_kernel: one CTA per 128 keys)
//   dQ = dS K                                                           (attn_bwd_dq_kernel:   one CTA per 128 queries)
//
// Scores and probabilities are recomputed from q, k and the forward's log-sum-exp; nothing is accumulated
// with atomics, so the gradients are the same bits on every run.  Both kernels follow the forward kernel's
// forms: operands arrive by TMA into 128-byte-swizzled shared memory, tcgen05.mma accumulates in tensor memory,
// one thread issues the products and another the copies, eight warps (two threads per accumulator row) do the
// elementwise work between the two groups of products and write P / dS back to tensor memory as bf16 over the
// scores they came from, where the second group of products reads them as its A operand.  A CTA owns 128 rows
// (two tiles, loaded once) and walks the rows of the other side 64 at a step ("unit") through a ring of five units.
//
//   dK/dV kernel   the CTA owns K_j, V_j (128 keys) and walks the queries that see them, for every q head of the kv
//                  head.  Per unit: S^T = K_j Q_u^T and dP^T = V_j dO_u^T (accumulator rows = keys, 64 columns each),
//                  elementwise over a key's row (lse and delta of the unit's queries come from shared memory),
//                  dV += P^T dO_u and dK += dS^T Q_u.  Tensor memory: S^T and dP^T of two units (2 x 128 columns), dV,
//                  dK (128 columns each); the score products run one unit ahead of the elementwise threads.
//   dQ kernel      the CTA owns Q_i, dO_i (128 queries of one q head) and walks the keys it sees.  Per unit:
//                  S = Q_i K_u^T and dP = dO_i V_u^T (accumulator rows = queries, lse and delta are per thread),
//                  dQ += dS K_u.  Tensor memory: S and dP of three units (3 x 128 columns) and dQ; the score
//                  products run two units ahead.
// Running ahead matters because a group of products is only known to be complete some 900 cycles after its last
// instruction was issued; with the scores of the next unit(s) already under way that latency is not on the
// elementwise threads' path.  What then bounds both kernels is the time of the thread that issues the products
// (issue runs at the tensor pipe's pace), which is why the copies have a thread of their own and the loops keep
// counters instead of dividing.  Every barrier wait is bounded; a wait that runs out sets NCKV_ST_TIMEOUT in the
// status word, the CTA stops issuing work, frees its tensor memory and returns.
//
// Replaces: the backward of F.scaled_dot_product_attention / flash_attn_func as reached from
// flash_attention.py:107-128 during training (gpt.py:108).
#include <math.h>

#include <type_traits>

#include "nckv_common.cuh"
#include "tc05.cuh"

namespace nckv {

constexpr int BT = 128;                        // keys per dK/dV CTA, queries per dQ CTA, and the walked block
constexpr int BT_TILE_BYTES = BT * NCKV_D * 2;  // 32 KB: two 64-channel halves of [128][128 B]
constexpr int BT_HALF = BT_TILE_BYTES / 2;
constexpr int BT_EW_THREADS = 256;             // elementwise threads: two per accumulator row, 64 columns each
constexpr int BT_TMEM_COLS = 512;
constexpr unsigned long long BT_WAIT_LIMIT = NCKV_WAIT_LIMIT_NS;

struct BwdParams {
    const float *lse;    // (B, Hq, T) natural log-sum-exp of the forward
    const float *delta;  // (B, Hq, T)
    __nv_bfloat16 *dq, *dk, *dv;
    int32_t *status;
    int B, T, Hq, Hkv, n_blocks;
    int window_left;
    float scale, scale_log2;
};

// delta[b, h, t] = sum_c dO[b, t, h, c] * O[b, t, h, c]: half a warp per row, 16 bytes of each tensor per lane
__global__ void __launch_bounds__(256) attn_bwd_delta_kernel(const __nv_bfloat16 *out, const __nv_bfloat16 *dout,
                                                             float *delta, int B, int T, int Hq) {
    const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;  // (b, t, h) flattened
    const int j = threadIdx.x & 15;
    const bool live = row < (long long)B * T * Hq;
    float acc = 0.f;
    if (live) {
        const uint4 o = __ldg(reinterpret_cast<const uint4 *>(out + row * NCKV_D) + j);
        const uint4 g = __ldg(reinterpret_cast<const uint4 *>(dout + row * NCKV_D) + j);
        const __nv_bfloat162 *o2 = reinterpret_cast<const __nv_bfloat162 *>(&o);
        const __nv_bfloat162 *g2 = reinterpret_cast<const __nv_bfloat162 *>(&g);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 a = __bfloat1622float2(o2[i]), c = __bfloat1622float2(g2[i]);
            acc += a.x * c.x + a.y * c.y;
        }
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (live && j == 0) {
        const int h = (int)(row % Hq);
        const long long bt = row / Hq;
        const int t = (int)(bt % T), b = (int)(bt / T);
        delta[((long long)b * Hq + h) * T + t] = acc;
    }
}

// ---- pieces shared by the two kernels -------------------------------------------------------------------
__device__ __forceinline__ void bt_load_tile(uint8_t *dst, const CUtensorMap *map, uint64_t *bar, int head, int tok0, int b) {
    tma_load_4d(dst, map, bar, 0, head, tok0, b);
    tma_load_4d(dst + BT_HALF, map, bar, 64, head, tok0, b);
}
// 64 fp32 accumulator columns starting at `taddr` -> 64 bf16 at `dst` (32-byte aligned).
__device__ __forceinline__ void bt_store_half_row(uint32_t taddr, __nv_bfloat16 *dst, bool live) {
    float c[64];
    tmem_ld64(taddr, c);
    if (live) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t w[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) w[e] = pack_bf16x2(c[16 * i + 2 * e], c[16 * i + 2 * e + 1]);
            st_global_v8(reinterpret_cast<uint4 *>(dst) + i * 2, w);
        }
    }
}

// ---- walked rows come 64 at a step ("unit"): queries in the dK/dV kernel, keys in the dQ kernel ---------------
constexpr int BU = 64;                          // walked rows per unit
constexpr int BU_TILE_BYTES = BU * NCKV_D * 2;  // 16 KB: two 64-channel halves of [64][128 B]
constexpr int BU_HALF = BU_TILE_BYTES / 2;
constexpr int BU_RING = 5;                      // units (two tiles each) in shared memory
constexpr int BU_BUFS = 3;                      // dQ kernel: units whose S and dP are in tensor memory (score products two units ahead)

struct BuShared {  // behind the operand tiles of the dQ kernel
    // bar_walk[u % 5] (phase u / 5) "the unit's K and V tiles have landed"; bar_s[u % 3] (phase u / 3) "its score products
    // are complete"; bar_p[u % 3] "its dS is in tensor memory"; bar_d[u & 1] (phase u / 2) "its gradient product is complete"
    uint64_t bar_own, bar_walk[BU_RING], bar_s[BU_BUFS], bar_p[BU_BUFS], bar_d[2];
    uint32_t tmem_slot;
    int abort_flag;
};
constexpr int BU_SMEM_BYTES = 2 * BT_TILE_BYTES + BU_RING * 2 * BU_TILE_BYTES + (int)sizeof(BuShared);

// D = A B^T, 128 x 64 x 128: A an own tile (128 rows), B a unit tile (64 rows), both K-major in shared memory.
__device__ __forceinline__ void bu_mma_ss(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b) {
    constexpr uint32_t IDESC = umma_idesc(BT, BU, 0, 0);
#pragma unroll
    for (int kk = 0; kk < NCKV_D / 16; ++kk) {
        const uint64_t off_a = (uint64_t)(((kk >> 2) * BT_HALF + (kk & 3) * 32) >> 4);
        const uint64_t off_b = (uint64_t)(((kk >> 2) * BU_HALF + (kk & 3) * 32) >> 4);
        umma_bf16(d_tmem, desc_a + off_a, desc_b + off_b, IDESC, kk > 0 ? 1u : 0u);
    }
}
// D (+)= A B, 128 x 128 x 64, with A (128 rows x 64 bf16) in tensor memory and B a unit tile used in place as an
// MN-major operand (contraction over the unit's 64 rows, 16 per instruction).  A sits where the elementwise threads
// left it: the bf16 of score columns [0, 32) over columns [0, 16) of the unit's fp32 scores, those of score columns
// [32, 64) over columns [32, 48) (each thread overwrites only scores it has read itself).
__device__ __forceinline__ void bu_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t desc_b_mn, bool accumulate) {
    constexpr uint32_t IDESC = umma_idesc(BT, NCKV_D, 0, 1);
#pragma unroll
    for (int ks = 0; ks < BU / 16; ++ks)
        umma_bf16_a_tmem(d_tmem, a_tmem + (uint32_t)((ks >> 1) * 32 + (ks & 1) * 8), desc_b_mn + (uint64_t)((ks * 16 * 128) >> 4),
                         IDESC, (accumulate || ks > 0) ? 1u : 0u);
}

constexpr int BU_THREADS = BT_EW_THREADS + 64;  // + a warp whose lane 0 issues the products + a warp whose lane 0 issues the copies

struct BvShared {  // behind the operand tiles of the dK/dV kernel
    // bar_walk[u % 5] (phase u / 5) "the unit's Q and dO tiles have landed"; bar_s[u & 1] (phase u / 2) "its score
    // products are complete"; bar_p[u & 1] "its P^T and dS^T are in tensor memory"; bar_d[u & 1] "its gradient products
    // are complete"
    uint64_t bar_own, bar_walk[BU_RING], bar_s[2], bar_p[2], bar_d[2];
    uint32_t tmem_slot;
    int abort_flag;
    // the walked queries' values, one per accumulator column: -lse * log2(e) and delta / sqrt(D)
    alignas(16) float neg_lse2[2][BU];
    alignas(16) float delta_s[2][BU];
};
constexpr int BV_SMEM_BYTES = 2 * BT_TILE_BYTES + BU_RING * 2 * BU_TILE_BYTES + (int)sizeof(BvShared);

// grid: (key blocks x Hkv x B), heaviest key blocks (most queries to walk) first
__global__ void __launch_bounds__(BU_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                     const BwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0) {  // uniform; checked rather than assumed
        if (threadIdx.x == 0) atomicOr(p.status, (int)NCKV_ST_TIMEOUT);
        return;
    }
    uint8_t *sK = smem, *sV = smem + BT_TILE_BYTES;
    uint8_t *ring = smem + 2 * BT_TILE_BYTES;  // [5][Q unit, dO unit]
    BvShared &sh = *reinterpret_cast<BvShared *>(ring + BU_RING * 2 * BU_TILE_BYTES);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int pairs = p.B * p.Hkv;
    const int jb = blockIdx.x / pairs;  // key blocks in ascending order: the first ones walk the most queries
    const int hkv = (blockIdx.x % pairs) % p.Hkv, b = (blockIdx.x % pairs) / p.Hkv;
    const int k0 = jb * BT;
    const int rep = p.Hq / p.Hkv;
    // query units (64 rows) that see a key of this block: causal from the diagonal on, up to the window's reach
    const int u_lo = 2 * jb;
    const int u_last = (p.T + BU - 1) / BU - 1;
    const int u_hi = p.window_left >= 0 ? min(u_last, (k0 + BT - 1 + p.window_left) / BU) : u_last;
    const int per_head = u_hi - u_lo + 1;
    const int n_units = per_head * rep;  // >= 1

    if (tid == 0) {
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
        prefetch_tensormap(&tmap_do);
        mbar_init(&sh.bar_own, 1);
        for (int i = 0; i < BU_RING; ++i) mbar_init(&sh.bar_walk[i], 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh.bar_s[i], 1);
            mbar_init(&sh.bar_p[i], BT_EW_THREADS / 32);
            mbar_init(&sh.bar_d[i], 1);
        }
        sh.abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&sh.tmem_slot, BT_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh.tmem_slot;
    // unit u: S^T at columns 128 (u & 1) + [0, 64), dP^T at + [64, 128); dV at [256, 384), dK at [384, 512)
    const uint32_t tmem_dv = tmem_base + 256, tmem_dk = tmem_base + 384;
    auto timed_out = [&]() {
        sh.abort_flag = 1;
        atomicOr(p.status, (int)NCKV_ST_TIMEOUT);
    };

    if (warp == BT_EW_THREADS / 32 + 1) {
        // =============== one thread issues the copies ================================================
        if ((tid & 31) == 0) {
            mbar_arrive_expect_tx(&sh.bar_own, 2 * BT_TILE_BYTES);
            bt_load_tile(sK, &tmap_k, &sh.bar_own, hkv, k0, b);
            bt_load_tile(sV, &tmap_v, &sh.bar_own, hkv, k0, b);
            bool ok = true;
            for (int u = 0; u < n_units && ok; ++u) {
                // the ring slot of unit u held unit u - 5: free once that unit's gradient products have completed
                if (u >= BU_RING) {
                    const int w = u - BU_RING;
                    ok = mbar_wait_bounded(&sh.bar_d[w & 1], (uint32_t)(w >> 1) & 1u, BT_WAIT_LIMIT);
                    if (!ok) break;
                }
                const int hq = hkv * rep + u / per_head, q0 = (u_lo + u % per_head) * BU;
                uint8_t *dst = ring + (u % BU_RING) * 2 * BU_TILE_BYTES;
                uint64_t *bar = &sh.bar_walk[u % BU_RING];
                mbar_arrive_expect_tx(bar, 2 * BU_TILE_BYTES);
                tma_load_4d(dst, &tmap_q, bar, 0, hq, q0, b);
                tma_load_4d(dst + BU_HALF, &tmap_q, bar, 64, hq, q0, b);
                tma_load_4d(dst + BU_TILE_BYTES, &tmap_do, bar, 0, hq, q0, b);
                tma_load_4d(dst + BU_TILE_BYTES + BU_HALF, &tmap_do, bar, 64, hq, q0, b);
            }
            if (!ok) timed_out();
        }
        __syncwarp();
    } else if (warp == BT_EW_THREADS / 32) {
        // =============== one thread issues the products ==============================================
        if ((tid & 31) == 0) {
            const uint64_t desc_k = smem_desc_sw128(smem_u32(sK), 16, 1024);
            const uint64_t desc_v = smem_desc_sw128(smem_u32(sV), 16, 1024);
            const uint32_t ring_addr = smem_u32(ring);
            // S^T = K Q^T, dP^T = V dO^T (rows = keys) into score buffer `buf` from ring slot `slot`
            auto scores = [&](int slot, uint32_t slot_parity, int buf) -> bool {
                if (!mbar_wait_bounded(&sh.bar_walk[slot], slot_parity, BT_WAIT_LIMIT)) return false;
                tc_fence_after();
                const uint32_t qa = ring_addr + (uint32_t)slot * 2 * BU_TILE_BYTES, da = qa + BU_TILE_BYTES;
                const uint32_t ts = tmem_base + (uint32_t)buf * 128;
                bu_mma_ss(ts, desc_k, smem_desc_sw128(qa, 16, 1024));
                bu_mma_ss(ts + 64, desc_v, smem_desc_sw128(da, 16, 1024));
                umma_commit(&sh.bar_s[buf]);
                return true;
            };
            bool ok = mbar_wait_bounded(&sh.bar_own, 0, BT_WAIT_LIMIT);
            // The score products run one unit ahead of the elementwise threads (tensor memory has room for two units'
            // scores beside dV and dK).  Counters instead of divisions: this thread's time per unit bounds the kernel.
            int s_slot = 0;
            uint32_t s_slot_par = 0;
            if (ok) {
                ok = scores(0, 0, 0);
                s_slot = 1;
            }
            int g_slot = 0;
            for (int u = 0; u < n_units && ok; ++u) {
                // buffer (u + 1) & 1 held unit u - 1, whose P^T / dS^T the gradient products issued in the last round
                // have read (products of one thread execute in order)
                if (u + 1 < n_units) {
                    ok = scores(s_slot, s_slot_par, (u + 1) & 1);
                    if (++s_slot == BU_RING) { s_slot = 0; s_slot_par ^= 1u; }
                }
                if (!ok) break;
                ok = mbar_wait_bounded(&sh.bar_p[u & 1], (uint32_t)(u >> 1) & 1u, BT_WAIT_LIMIT);
                if (!ok) break;
                tc_fence_after();
                // dV += P^T dO, dK += dS^T Q with the unit's tiles in place as MN-major operands (contraction over its queries)
                const uint32_t qa = ring_addr + (uint32_t)g_slot * 2 * BU_TILE_BYTES, da = qa + BU_TILE_BYTES;
                const uint32_t ts = tmem_base + (uint32_t)(u & 1) * 128;
                bu_mma_ts(tmem_dv, ts, smem_desc_sw128(da, BU_HALF, 1024), u > 0);
                bu_mma_ts(tmem_dk, ts + 64, smem_desc_sw128(qa, BU_HALF, 1024), u > 0);
                umma_commit(&sh.bar_d[u & 1]);
                if (++g_slot == BU_RING) g_slot = 0;
            }
            if (!ok) timed_out();
        }
        __syncwarp();
    } else {
        // =============== elementwise threads: two per key of the block ===============================
        const int kr = tid & (BT - 1);  // accumulator row == TMEM lane
        const int half = tid >> 7;      // which 32 of a unit's 64 query columns (and, at the end, dV or dK)
        const int kp = k0 + kr;         // the key's position
        const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
        bool aborted = false;
        auto warp_wait = [&](uint64_t *bar, uint32_t parity) -> bool {
            int ok = 1;
            if ((tid & 31) == 0) ok = mbar_wait_bounded(bar, parity, BT_WAIT_LIMIT) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            __syncwarp();
            return ok != 0;
        };
        const float2 scale_log2_2 = make_float2(p.scale_log2, p.scale_log2), scale_2 = make_float2(p.scale, p.scale);
        const float2 zero_2 = make_float2(0.f, 0.f);
        // threads 0-63 fetch -lse * log2(e), threads 64-127 delta / sqrt(D), of one of a unit's queries for everybody,
        // one unit ahead so that the load is not on the path
        int head = 0, in_head = 0;  // of the unit whose values are fetched next: u / per_head, u % per_head
        auto fetch = [&]() -> float {
            float mine = 0.f;
            if (tid < 2 * BU && head < rep) {
                const int hq = hkv * rep + head, tq = (u_lo + in_head) * BU + (tid & (BU - 1));
                mine = tid < BU ? -INFINITY : 0.f;  // a query past the end: P = 2^-inf = 0
                if (tq < p.T) {
                    const long long o = ((long long)b * p.Hq + hq) * p.T + tq;
                    if (tid < BU) {
                        const float l = p.lse[o];
                        mine = l == -INFINITY ? -INFINITY : -l * 1.4426950408889634f;
                    } else {
                        mine = p.delta[o] * p.scale;
                    }
                }
            }
            if (++in_head == per_head) { in_head = 0; ++head; }
            return mine;
        };
        float mine = fetch();
        int cur_in_head = 0;  // u % per_head of the current unit
        for (int u = 0; u < n_units; ++u) {
            const int q0 = (u_lo + cur_in_head) * BU;
            if (++cur_in_head == per_head) cur_in_head = 0;
            const int buf = u & 1;
            const float mine_next = fetch();  // unit u + 1 (nothing past the last unit)
            // (all eight warps take the same decision here: they meet at a named barrier right below)
            if (!warp_wait(&sh.bar_s[buf], (uint32_t)(u >> 1) & 1u)) {
                timed_out();
                aborted = true;
                break;
            }
            tc_fence_after();
            if (tid < BU) sh.neg_lse2[buf][tid] = mine;
            else if (tid < 2 * BU) sh.delta_s[buf][tid - BU] = mine;
            asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight elementwise warps
            // only units on the diagonal or at the window's edge need masking: this key is seen by the unit's
            // queries [c_lo, c_hi)
            const bool edge = (q0 < k0 + BT - 1) || (p.window_left >= 0 && q0 + BU - 1 - k0 > p.window_left);
            const int c_lo = kp - q0;
            const int c_hi = p.window_left >= 0 ? kp + p.window_left - q0 + 1 : BU;
            const int col0 = half * 32;
            const uint32_t t_s = tmem_base + (uint32_t)buf * 128 + lane_sel + col0;
            const float *nls = &sh.neg_lse2[buf][col0], *dls = &sh.delta_s[buf][col0];
            // two copies of the loop: the masked one only runs for the few units that need it
            auto chunk = [&](auto masked) {
                constexpr bool MASKED = decltype(masked)::value;
                float s[32], d[32];
                tmem_ld32x2(t_s, s, t_s + 64, d);
                uint32_t pw[16], dw[16];
#pragma unroll
                for (int c = 0; c < 32; c += 4) {
                    const float4 nl = *reinterpret_cast<const float4 *>(nls + c);
                    const float4 dl = *reinterpret_cast<const float4 *>(dls + c);
                    // P = 2^(s * scale * log2(e) - lse * log2(e));  dS = P * (dP * scale - delta * scale)
                    const float2 x01 = ffma2(make_float2(s[c], s[c + 1]), scale_log2_2, make_float2(nl.x, nl.y));
                    const float2 x23 = ffma2(make_float2(s[c + 2], s[c + 3]), scale_log2_2, make_float2(nl.z, nl.w));
                    const float2 t01 = ffma2(make_float2(d[c], d[c + 1]), scale_2, make_float2(-dl.x, -dl.y));
                    const float2 t23 = ffma2(make_float2(d[c + 2], d[c + 3]), scale_2, make_float2(-dl.z, -dl.w));
                    float2 p01 = make_float2(ex2_approx(x01.x), ex2_approx(x01.y));
                    float2 p23 = make_float2(ex2_approx(x23.x), ex2_approx(x23.y));
                    if (MASKED) {
                        const int col = col0 + c;
                        if (!(col >= c_lo && col < c_hi)) p01.x = 0.f;
                        if (!(col + 1 >= c_lo && col + 1 < c_hi)) p01.y = 0.f;
                        if (!(col + 2 >= c_lo && col + 2 < c_hi)) p23.x = 0.f;
                        if (!(col + 3 >= c_lo && col + 3 < c_hi)) p23.y = 0.f;
                    }
                    const float2 ds01 = ffma2(p01, t01, zero_2), ds23 = ffma2(p23, t23, zero_2);
                    pw[c / 2] = pack_bf16x2(p01.x, p01.y);
                    pw[c / 2 + 1] = pack_bf16x2(p23.x, p23.y);
                    dw[c / 2] = pack_bf16x2(ds01.x, ds01.y);
                    dw[c / 2 + 1] = pack_bf16x2(ds23.x, ds23.y);
                }
                // bf16 over the front of this thread's own fp32 scores, all of which it has read by now
                tmem_st_words(t_s, pw);
                tmem_st_words(t_s + 64, dw);
            };
            if (edge) chunk(std::true_type{});
            else chunk(std::false_type{});
            tc_fence_before();
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(&sh.bar_p[buf]);
            mine = mine_next;
        }
        if (!aborted) {
            if (warp_wait(&sh.bar_d[(n_units - 1) & 1], (uint32_t)((n_units - 1) >> 1) & 1u)) {
                tc_fence_after();
                const bool live = kp < p.T;
                const long long o = (((long long)b * p.T + (live ? kp : 0)) * p.Hkv + hkv) * NCKV_D;
                // the first 128 threads store dV, the others dK
                const uint32_t acc = (half == 0 ? tmem_dv : tmem_dk) + lane_sel;
                __nv_bfloat16 *dst = (half == 0 ? p.dv : p.dk) + o;
                bt_store_half_row(acc, dst, live);
                bt_store_half_row(acc + 64, dst + 64, live);
            } else {
                timed_out();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, BT_TMEM_COLS);
}

// grid: (query blocks x Hq x B), heaviest query blocks (most keys to walk) first
__global__ void __launch_bounds__(BU_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                   const BwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0) {  // uniform; checked rather than assumed
        if (threadIdx.x == 0) atomicOr(p.status, (int)NCKV_ST_TIMEOUT);
        return;
    }
    uint8_t *sQ = smem, *sdO = smem + BT_TILE_BYTES;
    uint8_t *ring = smem + 2 * BT_TILE_BYTES;  // [5][K unit, V unit]
    BuShared &sh = *reinterpret_cast<BuShared *>(ring + BU_RING * 2 * BU_TILE_BYTES);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int pairs = p.B * p.Hq;
    const int ib = p.n_blocks - 1 - blockIdx.x / pairs;  // the last query blocks walk the most keys: first
    const int hq = (blockIdx.x % pairs) % p.Hq, b = (blockIdx.x % pairs) / p.Hq;
    const int hkv = hq / (p.Hq / p.Hkv);
    const int q0 = ib * BT;
    // key units a query of this block sees: from the window's reach up to the end of the diagonal block
    const int u_lo = p.window_left >= 0 ? max(0, (q0 - p.window_left) / BU) : 0;
    const int u_hi = min((p.T + BU - 1) / BU - 1, 2 * ib + 1);
    const int n_units = u_hi - u_lo + 1;  // >= 1

    if (tid == 0) {
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
        prefetch_tensormap(&tmap_do);
        mbar_init(&sh.bar_own, 1);
        for (int i = 0; i < BU_RING; ++i) mbar_init(&sh.bar_walk[i], 1);
        for (int i = 0; i < BU_BUFS; ++i) {
            mbar_init(&sh.bar_s[i], 1);
            mbar_init(&sh.bar_p[i], BT_EW_THREADS / 32);
        }
        mbar_init(&sh.bar_d[0], 1);
        mbar_init(&sh.bar_d[1], 1);
        sh.abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&sh.tmem_slot, BT_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh.tmem_slot;
    // unit u: S at columns 128 (u % 3) + [0, 64), dP at + [64, 128); dQ at [384, 512)
    const uint32_t tmem_dq = tmem_base + 384;
    auto timed_out = [&]() {
        sh.abort_flag = 1;
        atomicOr(p.status, (int)NCKV_ST_TIMEOUT);
    };

    if (warp == BT_EW_THREADS / 32 + 1) {
        // =============== one thread issues the copies ================================================
        if ((tid & 31) == 0) {
            mbar_arrive_expect_tx(&sh.bar_own, 2 * BT_TILE_BYTES);
            bt_load_tile(sQ, &tmap_q, &sh.bar_own, hq, q0, b);
            bt_load_tile(sdO, &tmap_do, &sh.bar_own, hq, q0, b);
            bool ok = true;
            for (int u = 0; u < n_units && ok; ++u) {
                // the ring slot of unit u held unit u - 5: free once that unit's gradient product has completed
                if (u >= BU_RING) {
                    const int w = u - BU_RING;
                    ok = mbar_wait_bounded(&sh.bar_d[w & 1], (uint32_t)(w >> 1) & 1u, BT_WAIT_LIMIT);
                    if (!ok) break;
                }
                uint8_t *dst = ring + (u % BU_RING) * 2 * BU_TILE_BYTES;
                uint64_t *bar = &sh.bar_walk[u % BU_RING];
                mbar_arrive_expect_tx(bar, 2 * BU_TILE_BYTES);
                tma_load_4d(dst, &tmap_k, bar, 0, hkv, (u_lo + u) * BU, b);
                tma_load_4d(dst + BU_HALF, &tmap_k, bar, 64, hkv, (u_lo + u) * BU, b);
                tma_load_4d(dst + BU_TILE_BYTES, &tmap_v, bar, 0, hkv, (u_lo + u) * BU, b);
                tma_load_4d(dst + BU_TILE_BYTES + BU_HALF, &tmap_v, bar, 64, hkv, (u_lo + u) * BU, b);
            }
            if (!ok) timed_out();
        }
        __syncwarp();
    } else if (warp == BT_EW_THREADS / 32) {
        // =============== one thread issues the products ==============================================
        if ((tid & 31) == 0) {
            const uint64_t desc_q = smem_desc_sw128(smem_u32(sQ), 16, 1024);
            const uint64_t desc_do = smem_desc_sw128(smem_u32(sdO), 16, 1024);
            const uint32_t ring_addr = smem_u32(ring);
            // S = Q K^T, dP = dO V^T (rows = queries) into score buffer `buf` from ring slot `slot` (phase parities given)
            auto scores = [&](int slot, uint32_t slot_parity, int buf) -> bool {
                if (!mbar_wait_bounded(&sh.bar_walk[slot], slot_parity, BT_WAIT_LIMIT)) return false;
                tc_fence_after();
                const uint32_t ka = ring_addr + (uint32_t)slot * 2 * BU_TILE_BYTES, va = ka + BU_TILE_BYTES;
                const uint32_t ts = tmem_base + (uint32_t)buf * 128;
                bu_mma_ss(ts, desc_q, smem_desc_sw128(ka, 16, 1024));
                bu_mma_ss(ts + 64, desc_do, smem_desc_sw128(va, 16, 1024));
                umma_commit(&sh.bar_s[buf]);
                return true;
            };
            bool ok = mbar_wait_bounded(&sh.bar_own, 0, BT_WAIT_LIMIT);
            // the score products run two units ahead of the elementwise threads: their completion is known to the
            // threads some 900 cycles after the last one has been issued.  (Counters instead of divisions: this
            // thread's time per unit is what bounds the kernel.)
            int s_slot = 0, s_buf = 0;          // ring slot and score buffer of the next unit to get its score products
            uint32_t s_slot_par = 0;
            for (int u = 0; u < BU_BUFS - 1 && u < n_units && ok; ++u) {
                ok = scores(s_slot, s_slot_par, s_buf);
                if (++s_slot == BU_RING) { s_slot = 0; s_slot_par ^= 1u; }
                if (++s_buf == BU_BUFS) s_buf = 0;
            }
            int g_slot = 0, g_buf = 0;          // the same for the next unit to get its gradient product
            uint32_t g_buf_par = 0;
            for (int u = 0; u < n_units && ok; ++u) {
                // buffer (u + 2) % 3 held unit u - 1, whose dS the gradient product issued in the last round has read
                // (products of one thread execute in order)
                if (u + BU_BUFS - 1 < n_units) {
                    ok = scores(s_slot, s_slot_par, s_buf);
                    if (++s_slot == BU_RING) { s_slot = 0; s_slot_par ^= 1u; }
                    if (++s_buf == BU_BUFS) s_buf = 0;
                }
                if (!ok) break;
                ok = mbar_wait_bounded(&sh.bar_p[g_buf], g_buf_par, BT_WAIT_LIMIT);
                if (!ok) break;
                tc_fence_after();
                // dQ += dS K with the unit's K tile in place as an MN-major operand (contraction over its keys)
                bu_mma_ts(tmem_dq, tmem_base + (uint32_t)g_buf * 128,
                          smem_desc_sw128(ring_addr + (uint32_t)g_slot * 2 * BU_TILE_BYTES, BU_HALF, 1024), u > 0);
                umma_commit(&sh.bar_d[u & 1]);
                if (++g_slot == BU_RING) g_slot = 0;
                if (++g_buf == BU_BUFS) { g_buf = 0; g_buf_par ^= 1u; }
            }
            if (!ok) timed_out();
        }
        __syncwarp();
    } else {
        // =============== elementwise threads: two per query of the block =============================
        const int qr = tid & (BT - 1);  // accumulator row == TMEM lane
        const int half = tid >> 7;      // which 32 of a unit's 64 key columns (and, at the end, which 64 channels)
        const int qp = q0 + qr;         // the query's position
        const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
        bool aborted = false;
        auto warp_wait = [&](uint64_t *bar, uint32_t parity) -> bool {
            int ok = 1;
            if ((tid & 31) == 0) ok = mbar_wait_bounded(bar, parity, BT_WAIT_LIMIT) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            __syncwarp();
            return ok != 0;
        };
        float neg_lse2 = -INFINITY, delta_s = 0.f;  // a query past the end: P = 2^-inf = 0
        if (qp < p.T) {
            const long long o = ((long long)b * p.Hq + hq) * p.T + qp;
            const float l = p.lse[o];
            neg_lse2 = l == -INFINITY ? -INFINITY : -l * 1.4426950408889634f;
            delta_s = p.delta[o] * p.scale;
        }
        const float2 scale_log2_2 = make_float2(p.scale_log2, p.scale_log2), scale_2 = make_float2(p.scale, p.scale);
        const float2 neg_lse2_2 = make_float2(neg_lse2, neg_lse2), neg_delta_2 = make_float2(-delta_s, -delta_s);
        const float2 zero_2 = make_float2(0.f, 0.f);
        for (int u = 0; u < n_units; ++u) {
            const int k0 = (u_lo + u) * BU, buf = u % BU_BUFS;
            if (!warp_wait(&sh.bar_s[buf], (uint32_t)(u / BU_BUFS) & 1u)) {
                timed_out();
                aborted = true;
                break;
            }
            tc_fence_after();
            // only units on the diagonal or at the window's edge need masking: this query sees the unit's keys [c_lo, c_hi)
            const bool edge = (k0 + BU - 1 > q0) || (p.window_left >= 0 && q0 + BT - 1 - k0 > p.window_left);
            const int c_hi = qp - k0 + 1;
            const int c_lo = p.window_left >= 0 ? qp - p.window_left - k0 : 0;
            const int col0 = half * 32;
            const uint32_t t_s = tmem_base + (uint32_t)buf * 128 + lane_sel + col0;
            // two copies of the loop: the masked one only runs for the few units that need it
            auto chunk = [&](auto masked) {
                constexpr bool MASKED = decltype(masked)::value;
                float s[32], d[32];
                tmem_ld32x2(t_s, s, t_s + 64, d);
                uint32_t dw[16];
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    // P = 2^(s * scale * log2(e) - lse * log2(e));  dS = P * (dP * scale - delta * scale)
                    const float2 x = ffma2(make_float2(s[c], s[c + 1]), scale_log2_2, neg_lse2_2);
                    const float2 t = ffma2(make_float2(d[c], d[c + 1]), scale_2, neg_delta_2);
                    float2 pe = make_float2(ex2_approx(x.x), ex2_approx(x.y));
                    if (MASKED) {
                        const int col = col0 + c;
                        if (!(col >= c_lo && col < c_hi)) pe.x = 0.f;
                        if (!(col + 1 >= c_lo && col + 1 < c_hi)) pe.y = 0.f;
                    }
                    const float2 ds = ffma2(pe, t, zero_2);
                    dw[c / 2] = pack_bf16x2(ds.x, ds.y);
                }
                tmem_st_words(t_s, dw);  // over the front of this thread's own fp32 scores, all of which it has read by now
            };
            if (edge) chunk(std::true_type{});
            else chunk(std::false_type{});
            tc_fence_before();
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(&sh.bar_p[buf]);
        }
        if (!aborted) {
            if (warp_wait(&sh.bar_d[(n_units - 1) & 1], (uint32_t)((n_units - 1) >> 1) & 1u)) {
                tc_fence_after();
                const bool live = qp < p.T;
                bt_store_half_row(tmem_dq + lane_sel + half * 64,
                                  p.dq + (((long long)b * p.T + (live ? qp : 0)) * p.Hq + hq) * NCKV_D + half * 64, live);
            } else {
                timed_out();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, BT_TMEM_COLS);
}

}  // namespace nckv

extern "C" size_t nckv_flash_attn_bwd_workspace_bytes(int B, int T, int Hq) {
    const size_t delta_bytes = (size_t)B * (size_t)T * (size_t)Hq * sizeof(float);
    return (delta_bytes + 255) / 256 * 256 + 256;  // delta, then the device status word (NCKV_ST_* bits, 0 = clean)
}

extern "C" int nckv_flash_attn_bwd(const void *q, const void *k, const void *v, const void *out, const void *dout,
                                   const float *lse, void *dq, void *dk, void *dv, void *workspace, int B, int T,
                                   int Hq, int Hkv, int D, int window_left, void *stream) {
    using namespace nckv;
    if (!q || !k || !v || !out || !dout || !lse || !dq || !dk || !dv || !workspace) {
        set_error("flash_attn_bwd: null pointer argument");
        return NCKV_E_ARG;
    }
    if (B <= 0 || T <= 0 || Hq <= 0 || Hkv <= 0) {
        set_error("flash_attn_bwd: non-positive size (B=%d T=%d Hq=%d Hkv=%d)", B, T, Hq, Hkv);
        return NCKV_E_ARG;
    }
    if (D != NCKV_D) {
        set_error("flash_attn_bwd: head_dim %d unsupported (kernels are built for 128)", D);
        return NCKV_E_UNSUPPORTED;
    }
    if (Hq % Hkv != 0) {
        set_error("flash_attn_bwd: Hq=%d must be a multiple of Hkv=%d", Hq, Hkv);
        return NCKV_E_UNSUPPORTED;
    }
    const int n_blocks = (T + BT - 1) / BT;
    if ((long long)n_blocks * Hq * B > 0x7fffffffLL) {
        set_error("flash_attn_bwd: B=%d x Hq=%d x %d blocks exceed the grid limit", B, Hq, n_blocks);
        return NCKV_E_UNSUPPORTED;
    }
    if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out | (uintptr_t)dout | (uintptr_t)dq | (uintptr_t)dk |
          (uintptr_t)dv | (uintptr_t)workspace) & 31) != 0) {
        set_error("flash_attn_bwd: tensors must be 32-byte aligned");
        return NCKV_E_ARG;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t delta_bytes = (size_t)B * T * Hq * sizeof(float);
    BwdParams p;
    p.lse = lse;
    p.delta = static_cast<const float *>(workspace);
    p.status = reinterpret_cast<int32_t *>(static_cast<uint8_t *>(workspace) + (delta_bytes + 255) / 256 * 256);
    NCKV_CUDA_CHECK(cudaMemsetAsync(p.status, 0, sizeof(int32_t), st));
    p.dq = static_cast<__nv_bfloat16 *>(dq);
    p.dk = static_cast<__nv_bfloat16 *>(dk);
    p.dv = static_cast<__nv_bfloat16 *>(dv);
    p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.n_blocks = n_blocks;
    p.window_left = window_left;
    p.scale = (float)(1.0 / sqrt((double)D));
    p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)D));

    // every tensor is an own operand (boxes of 128 rows) in one kernel and a walked one (boxes of 64 rows) in the other
    CUtensorMap mq[2], mk[2], mv[2], mdo[2];
    int rc = NCKV_OK;
    for (int i = 0; i < 2 && rc == NCKV_OK; ++i) {
        const int box = i == 0 ? BT : BU;
        rc = make_kv_tensor_map(&mq[i], q, B, T, Hq, (int64_t)T * Hq * D, (int64_t)Hq * D, box);
        if (rc == NCKV_OK) rc = make_kv_tensor_map(&mdo[i], dout, B, T, Hq, (int64_t)T * Hq * D, (int64_t)Hq * D, box);
        if (rc == NCKV_OK) rc = make_kv_tensor_map(&mk[i], k, B, T, Hkv, (int64_t)T * Hkv * D, (int64_t)Hkv * D, box);
        if (rc == NCKV_OK) rc = make_kv_tensor_map(&mv[i], v, B, T, Hkv, (int64_t)T * Hkv * D, (int64_t)Hkv * D, box);
    }
    if (rc != NCKV_OK) return rc;

    const long long rows = (long long)B * T * Hq;
    attn_bwd_delta_kernel<<<(unsigned)((rows + 15) / 16), 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(out),
                                                                       static_cast<const __nv_bfloat16 *>(dout),
                                                                       static_cast<float *>(workspace), B, T, Hq);
    NCKV_CUDA_CHECK(cudaGetLastError());

    static bool attr_set[64] = {false};  // per device; setting the attribute twice from racing threads is harmless
    int dev = 0;
    NCKV_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        NCKV_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BV_SMEM_BYTES));
        NCKV_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BU_SMEM_BYTES));
        attr_set[dev] = true;
    }
    attn_bwd_dkdv_kernel<<<(unsigned)(n_blocks * Hkv * B), BU_THREADS, BV_SMEM_BYTES, st>>>(mq[1], mk[0], mv[0], mdo[1], p);
    NCKV_CUDA_CHECK(cudaGetLastError());
    attn_bwd_dq_kernel<<<(unsigned)(n_blocks * Hq * B), BU_THREADS, BU_SMEM_BYTES, st>>>(mq[0], mk[1], mv[1], mdo[0], p);
    NCKV_CUDA_CHECK(cudaGetLastError());
    return NCKV_OK;
}
