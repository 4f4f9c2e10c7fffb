// Backward of flash_attn_func (training): dq, dk, dv of causal / sliding-window attention over plain
// (B, T, H, D) tensors, from q, k, v, the forward output, its gradient and the forward's log-sum-exp.
//
//   P  = exp(scale * Q K^T - lse)            (recomputed per tile, never stored)
//   dV = P^T dO
//   dP = dO V^T,   delta = rowsum(dO * O),   dS = P * (dP - delta)
//   dQ = scale * dS K,    dK = scale * dS^T Q
//
// Three kernels.  `delta` is one warp per (row, token, head).  The dK/dV kernel gives a CTA one tile
// of 64 keys of one (row, kv head) and walks the query tiles (of every q head of the group) that see
// them; the dQ kernel gives a CTA one tile of 64 queries of one (row, q head) and walks its key
// tiles.  Scores are recomputed in both (7 matrix products per tile pair instead of 5) so that no
// gradient needs atomics: results do not depend on scheduling.  The products run on the warp-level
// tensor-core path (ldmatrix + mma.sync.m16n8k16 bf16, fp32 accumulation) with operands staged in shared
// memory by cp.async; P and dS are formed in registers from the score accumulators.  The kernels are bound by
// shared-memory operand fetches, so a warp owns 2 x 2 blocks of 16 x 16 of each gradient (every fragment it loads
// feeds two products) and two CTAs of 8 warps share an SM.  This is a first,
// correct version: it makes no claim on the tcgen05 roofline.
//
// Replaces: autograd through F.scaled_dot_product_attention as reached from flash_attn_func
// (flash_attention.py:107-128, caller gpt.py:108) when training.
#include <math.h>

#include "nckv_common.cuh"

namespace nckv {

constexpr int BW_T = 64;             // queries and keys per tile
constexpr int BW_THREADS = 256;      // 8 warps; two CTAs per SM overlap each other's barrier-separated phases
constexpr int BW_LD = NCKV_D + 8;    // bf16 row stride of the 64 x 128 operand tiles (272 B: ldmatrix without bank conflicts)
constexpr int BW_LDS = BW_T + 8;     // bf16 row stride of the 64 x 64 P and dS tiles (144 B)

struct BwdParams {
    const __nv_bfloat16 *q, *k, *v, *dout;
    const float *lse, *delta;
    __nv_bfloat16 *dq, *dk, *dv;
    int B, T, Hq, Hkv;
    int window_left;
    float scale, scale_log2;
};

// The tiles a CTA keeps for its whole life (`own`) and the tiles it walks (`walk`, refilled with cp.async every
// iteration; 89 KB in all, so that two CTAs share an SM and one computes while the other waits for its copies).
// dK/dV kernel: own = K, V; walk = Q, dO and their row statistics.  dQ kernel: own = Q, dO and the statistics; walk = K, V.
struct BwdSmem {
    __nv_bfloat16 own[2][BW_T * BW_LD];
    __nv_bfloat16 walk[2][BW_T * BW_LD];  // [tile]; after the loop: staging of a 64 x 128 fp32 result
    __nv_bfloat16 p[BW_T * BW_LDS];
    __nv_bfloat16 ds[BW_T * BW_LDS];
    float lse[BW_T];    // natural-log log-sum-exp of the rows
    float delta[BW_T];
};
static_assert(sizeof(__nv_bfloat16) * 2 * BW_T * BW_LD >= sizeof(float) * BW_T * NCKV_D, "the result staging area");

// ---- 16 x 16 x 16 products on the warp-level tensor-core path: ldmatrix + mma.sync.m16n8k16 ----------------
struct FragA { uint32_t r[4]; };   // A, 16 (m) x 16 (k)
struct FragB { uint32_t r[4]; };   // B, 16 (k) x 16 (n): r[0], r[1] for n 0..7, r[2], r[3] for n 8..15
struct Acc { float c[8]; };        // 16 x 16 fp32: c[0..3] columns 0..7, c[4..7] columns 8..15
// element e of Acc sits at row (lane / 4) + 8 * ((e >> 1) & 1), column 8 * (e >> 2) + 2 * (lane % 4) + (e & 1)

__device__ __forceinline__ void load_a_mk(FragA &f, const __nv_bfloat16 *base, int ld, int lane) {  // A(m,k) at base[m ld + k]
    const __nv_bfloat16 *ptr = base + ((lane & 7) + ((lane >> 3) & 1) * 8) * ld + (lane >> 4) * 8;
    ldmatrix_x4(f.r[0], f.r[1], f.r[2], f.r[3], smem_u32(ptr));
}
__device__ __forceinline__ void load_a_km(FragA &f, const __nv_bfloat16 *base, int ld, int lane) {  // A(m,k) at base[k ld + m]
    const int i = lane >> 3, j = lane & 7;
    const __nv_bfloat16 *ptr = base + ((i >> 1) * 8 + j) * ld + (i & 1) * 8;
    ldmatrix_x4_trans(f.r[0], f.r[1], f.r[2], f.r[3], smem_u32(ptr));
}
__device__ __forceinline__ void load_b_nk(FragB &f, const __nv_bfloat16 *base, int ld, int lane) {  // B(k,n) at base[n ld + k]
    const int i = lane >> 3, j = lane & 7;
    const __nv_bfloat16 *ptr = base + ((i >> 1) * 8 + j) * ld + (i & 1) * 8;
    ldmatrix_x4(f.r[0], f.r[1], f.r[2], f.r[3], smem_u32(ptr));
}
__device__ __forceinline__ void load_b_kn(FragB &f, const __nv_bfloat16 *base, int ld, int lane) {  // B(k,n) at base[k ld + n]
    const int i = lane >> 3, j = lane & 7;
    const __nv_bfloat16 *ptr = base + ((i & 1) * 8 + j) * ld + (i >> 1) * 8;
    ldmatrix_x4_trans(f.r[0], f.r[1], f.r[2], f.r[3], smem_u32(ptr));
}
__device__ __forceinline__ void mma16(Acc &d, const FragA &a, const FragB &b) {
    mma_bf16_16816(d.c[0], d.c[1], d.c[2], d.c[3], a.r[0], a.r[1], a.r[2], a.r[3], b.r[0], b.r[1]);
    mma_bf16_16816(d.c[4], d.c[5], d.c[6], d.c[7], a.r[0], a.r[1], a.r[2], a.r[3], b.r[2], b.r[3]);
}
__device__ __forceinline__ void zero(Acc &d) {
#pragma unroll
    for (int e = 0; e < 8; ++e) d.c[e] = 0.f;
}
// fp32 accumulator block (rows r0.., columns c0..) into a row-major fp32 array
__device__ __forceinline__ void store_acc(float *dst, int ld, int r0, int c0, const Acc &d, int lane) {
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
        const int row = r0 + (lane >> 2) + 8 * ((e >> 1) & 1), col = c0 + 8 * (e >> 2) + 2 * (lane & 3);
        *reinterpret_cast<float2 *>(dst + row * ld + col) = make_float2(d.c[e], d.c[e + 1]);
    }
}

// Asynchronous copies (cp.async): `bytes` of the source are copied, the rest of the 16 or 4 bytes is zero-filled.
__device__ __forceinline__ void cp_async_16(void *dst, const void *src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_4(void *dst, const void *src, int bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// 64 rows x 256 bytes of a (B, T, H, D) tensor into a padded shared-memory tile, asynchronously; rows at or
// beyond T are zero-filled (the source address is clamped to a valid row, no byte of it is read).
__device__ __forceinline__ void load_tile(__nv_bfloat16 *dst, const __nv_bfloat16 *src, int b, int t0, int h, int T,
                                          int H) {
    for (int i = threadIdx.x; i < BW_T * (NCKV_D / 8); i += BW_THREADS) {
        const int r = i / (NCKV_D / 8), c = i % (NCKV_D / 8);
        const int t = t0 + r;
        const int tc = t < T ? t : T - 1;
        cp_async_16(dst + r * BW_LD + c * 8, src + (((long long)b * T + tc) * H + h) * NCKV_D + c * 8, t < T ? 16 : 0);
    }
}

// One warp's 16 x 32 block of S = Q K^T and of dP = dO V^T (the Q / dO fragments feed two key blocks each), turned
// in registers into P and dS (bf16, written to shared memory for the products that follow).
// Queries q0 + 16 r .., keys k0 + 32 c2 ..
__device__ __forceinline__ void scores_to_p_ds(BwdSmem &sm, const BwdParams &p, const __nv_bfloat16 *tq,
                                               const __nv_bfloat16 *tdo, const __nv_bfloat16 *tk, const __nv_bfloat16 *tv,
                                               const float *lse, const float *delta, int q0, int k0, int warp, int lane) {
    const int r = warp >> 1, c2 = warp & 1;
    Acc acc_s[2], acc_p[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        zero(acc_s[j]);
        zero(acc_p[j]);
    }
#pragma unroll
    for (int kk = 0; kk < NCKV_D / 16; ++kk) {
        FragA a_q, a_do;
        load_a_mk(a_q, tq + r * 16 * BW_LD + kk * 16, BW_LD, lane);
        load_a_mk(a_do, tdo + r * 16 * BW_LD + kk * 16, BW_LD, lane);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            FragB b_k, b_v;  // B(k = channel, n = key) at tile[key][channel]
            load_b_nk(b_k, tk + (c2 * 2 + j) * 16 * BW_LD + kk * 16, BW_LD, lane);
            load_b_nk(b_v, tv + (c2 * 2 + j) * 16 * BW_LD + kk * 16, BW_LD, lane);
            mma16(acc_s[j], a_q, b_k);
            mma16(acc_p[j], a_do, b_v);
        }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {  // the thread's two rows
        const int row = r * 16 + (lane >> 2) + 8 * h;
        const int tq_ = q0 + row;
        const float lse2 = lse[row] * 1.4426950408889634f, dl = delta[row];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int nb = 0; nb < 2; ++nb) {
                const int col = (c2 * 2 + j) * 16 + 8 * nb + 2 * (lane & 3);
                float pr[2], ds[2];
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const int e = nb * 4 + h * 2 + x;
                    const int tk_ = k0 + col + x;
                    const bool visible = tq_ < p.T && tk_ <= tq_ && (p.window_left < 0 || tq_ - tk_ <= p.window_left);
                    // a visible score implies a finite log-sum-exp (the row has at least this key)
                    pr[x] = visible ? exp2f(acc_s[j].c[e] * p.scale_log2 - lse2) : 0.f;
                    ds[x] = visible ? pr[x] * (acc_p[j].c[e] - dl) * p.scale : 0.f;
                }
                *reinterpret_cast<uint32_t *>(sm.p + row * BW_LDS + col) = pack_bf16x2(pr[0], pr[1]);
                *reinterpret_cast<uint32_t *>(sm.ds + row * BW_LDS + col) = pack_bf16x2(ds[0], ds[1]);
            }
        }
    }
}

__device__ __forceinline__ void load_row_stats(float *lse, float *delta, const BwdParams &p, int b, int hq, int q0) {
    for (int r = threadIdx.x; r < BW_T; r += BW_THREADS) {
        const int t = q0 + r;
        const long long o = ((long long)b * p.Hq + hq) * p.T + (t < p.T ? t : p.T - 1);
        cp_async_4(lse + r, p.lse + o, t < p.T ? 4 : 0);
        cp_async_4(delta + r, p.delta + o, t < p.T ? 4 : 0);
    }
}

// fp32 64 x 128 result in the staging area -> bf16 rows of a (B, T, H, D) tensor
__device__ __forceinline__ void store_result(const float *stage, __nv_bfloat16 *dst, int b, int t0, int h, int T,
                                             int H) {
    for (int i = threadIdx.x; i < BW_T * (NCKV_D / 8); i += BW_THREADS) {
        const int r = i / (NCKV_D / 8), c = i % (NCKV_D / 8);
        const int t = t0 + r;
        if (t >= T) continue;
        const float *src = stage + r * NCKV_D + c * 8;
        uint4 val;
        val.x = pack_bf16x2(src[0], src[1]);
        val.y = pack_bf16x2(src[2], src[3]);
        val.z = pack_bf16x2(src[4], src[5]);
        val.w = pack_bf16x2(src[6], src[7]);
        *reinterpret_cast<uint4 *>(dst + (((long long)b * T + t) * H + h) * NCKV_D + c * 8) = val;
    }
}

// delta[b, h, t] = sum_c dO[b, t, h, c] * O[b, t, h, c]
__global__ void __launch_bounds__(256) attn_bwd_delta_kernel(const __nv_bfloat16 *out, const __nv_bfloat16 *dout,
                                                             float *delta, int B, int T, int Hq) {
    const long long row = (long long)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);  // (b, t, h) flattened
    if (row >= (long long)B * T * Hq) return;
    const int lane = threadIdx.x & 31;
    const uint2 o = *reinterpret_cast<const uint2 *>(out + row * NCKV_D + lane * 4);
    const uint2 g = *reinterpret_cast<const uint2 *>(dout + row * NCKV_D + lane * 4);
    const __nv_bfloat162 *o2 = reinterpret_cast<const __nv_bfloat162 *>(&o);
    const __nv_bfloat162 *g2 = reinterpret_cast<const __nv_bfloat162 *>(&g);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float2 a = __bfloat1622float2(o2[i]), c = __bfloat1622float2(g2[i]);
        acc += a.x * c.x + a.y * c.y;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) {
        const int h = (int)(row % Hq);
        const long long bt = row / Hq;
        const int t = (int)(bt % T), b = (int)(bt / T);
        delta[((long long)b * Hq + h) * T + t] = acc;
    }
}

// One CTA: 64 keys of one (row, kv head).  grid = (key tiles, Hkv, B)
__global__ void __launch_bounds__(BW_THREADS, 2) attn_bwd_dkdv_kernel(const BwdParams p) {
    extern __shared__ __align__(128) uint8_t bw_smem[];
    BwdSmem &sm = *reinterpret_cast<BwdSmem *>(bw_smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k0 = blockIdx.x * BW_T, hkv = blockIdx.y, b = blockIdx.z;
    const int rep = p.Hq / p.Hkv;

    __nv_bfloat16 *sk = sm.own[0], *sv = sm.own[1];
    __nv_bfloat16 *sq = sm.walk[0], *sdo = sm.walk[1];
    load_tile(sk, p.k, b, k0, hkv, p.T, p.Hkv);
    load_tile(sv, p.v, b, k0, hkv, p.T, p.Hkv);

    // output: 4 (key blocks) x 8 (channel blocks) of 16 x 16; a warp owns key blocks rb, rb + 1 x channel blocks cb, cb + 1
    const int cb = (warp & 3) * 2, rb = (warp >> 2) * 2;
    Acc acc_dk[2][2], acc_dv[2][2];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            zero(acc_dk[r][c]);
            zero(acc_dv[r][c]);
        }
    // query tiles that see any of these keys: positions k0 .. (last key + window), for every q head of the group
    const int last_key = min(k0 + BW_T, p.T) - 1;
    const int q_hi = p.window_left >= 0 ? min(p.T - 1, last_key + p.window_left) : p.T - 1;
    const int per_head = (q_hi - k0) / BW_T + 1;  // causal: queries at or after the tile's first key
    const int n_iter = rep * per_head;
    for (int it = 0; it < n_iter; ++it) {
        const int hq = hkv * rep + it / per_head, q0 = k0 + (it % per_head) * BW_T;
        __syncthreads();  // the previous iteration's products have read q, dout, p and ds
        load_tile(sq, p.q, b, q0, hq, p.T, p.Hq);
        load_tile(sdo, p.dout, b, q0, hq, p.T, p.Hq);
        load_row_stats(sm.lse, sm.delta, p, b, hq, q0);
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
        scores_to_p_ds(sm, p, sq, sdo, sk, sv, sm.lse, sm.delta, q0, k0, warp, lane);
        __syncthreads();
#pragma unroll
        for (int qq = 0; qq < BW_T / 16; ++qq) {
            FragB b_do[2], b_q[2];  // B(k = query, n = channel) at tile[query][channel]
            FragA a_p[2], a_ds[2];  // A(m = key, k = query) at tile[query][key]
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                load_b_kn(b_do[c], sdo + qq * 16 * BW_LD + (cb + c) * 16, BW_LD, lane);
                load_b_kn(b_q[c], sq + qq * 16 * BW_LD + (cb + c) * 16, BW_LD, lane);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                load_a_km(a_p[r], sm.p + qq * 16 * BW_LDS + (rb + r) * 16, BW_LDS, lane);
                load_a_km(a_ds[r], sm.ds + qq * 16 * BW_LDS + (rb + r) * 16, BW_LDS, lane);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    mma16(acc_dv[r][c], a_p[r], b_do[c]);
                    mma16(acc_dk[r][c], a_ds[r], b_q[c]);
                }
        }
    }
    cp_async_wait<0>();
    __syncthreads();
    float *stage = reinterpret_cast<float *>(&sm.walk[0][0]);
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int c = 0; c < 2; ++c) store_acc(stage, NCKV_D, (rb + r) * 16, (cb + c) * 16, acc_dk[r][c], lane);
    __syncthreads();
    store_result(stage, p.dk, b, k0, hkv, p.T, p.Hkv);
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int c = 0; c < 2; ++c) store_acc(stage, NCKV_D, (rb + r) * 16, (cb + c) * 16, acc_dv[r][c], lane);
    __syncthreads();
    store_result(stage, p.dv, b, k0, hkv, p.T, p.Hkv);
}

// One CTA: 64 queries of one (row, q head).  grid = (query tiles, Hq, B)
__global__ void __launch_bounds__(BW_THREADS, 2) attn_bwd_dq_kernel(const BwdParams p) {
    extern __shared__ __align__(128) uint8_t bw_smem[];
    BwdSmem &sm = *reinterpret_cast<BwdSmem *>(bw_smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // longest tiles first: the last query tile sees the most keys
    const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * BW_T, hq = blockIdx.y, b = blockIdx.z;
    const int hkv = hq / (p.Hq / p.Hkv);

    __nv_bfloat16 *sq = sm.own[0], *sdo = sm.own[1];
    __nv_bfloat16 *sk = sm.walk[0], *sv = sm.walk[1];
    load_tile(sq, p.q, b, q0, hq, p.T, p.Hq);
    load_tile(sdo, p.dout, b, q0, hq, p.T, p.Hq);
    load_row_stats(sm.lse, sm.delta, p, b, hq, q0);

    // output: 4 (query blocks) x 8 (channel blocks); a warp owns query blocks rb, rb + 1 x channel blocks cb, cb + 1
    const int cb = (warp & 3) * 2, rb = (warp >> 2) * 2;
    Acc acc_dq[2][2];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int c = 0; c < 2; ++c) zero(acc_dq[r][c]);

    const int last_q = min(q0 + BW_T, p.T) - 1;
    int k_lo = p.window_left >= 0 ? max(0, q0 - p.window_left) : 0;
    k_lo -= k_lo % BW_T;
    for (int k0 = k_lo; k0 <= last_q; k0 += BW_T) {
        __syncthreads();  // the previous iteration's product has read k and ds
        load_tile(sk, p.k, b, k0, hkv, p.T, p.Hkv);
        load_tile(sv, p.v, b, k0, hkv, p.T, p.Hkv);
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
        scores_to_p_ds(sm, p, sq, sdo, sk, sv, sm.lse, sm.delta, q0, k0, warp, lane);
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BW_T / 16; ++kk) {
            FragB b_k[2];   // B(k = key, n = channel) at tile[key][channel]
            FragA a_ds[2];  // A(m = query, k = key) at tile[query][key]
#pragma unroll
            for (int c = 0; c < 2; ++c) load_b_kn(b_k[c], sk + kk * 16 * BW_LD + (cb + c) * 16, BW_LD, lane);
#pragma unroll
            for (int r = 0; r < 2; ++r) load_a_mk(a_ds[r], sm.ds + (rb + r) * 16 * BW_LDS + kk * 16, BW_LDS, lane);
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int c = 0; c < 2; ++c) mma16(acc_dq[r][c], a_ds[r], b_k[c]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();
    float *stage = reinterpret_cast<float *>(&sm.walk[0][0]);
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int c = 0; c < 2; ++c) store_acc(stage, NCKV_D, (rb + r) * 16, (cb + c) * 16, acc_dq[r][c], lane);
    __syncthreads();
    store_result(stage, p.dq, b, q0, hq, p.T, p.Hq);
}

}  // namespace nckv

extern "C" size_t nckv_flash_attn_bwd_workspace_bytes(int B, int T, int Hq) {
    return (size_t)B * (size_t)T * (size_t)Hq * sizeof(float);
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
    const int n_tiles = (T + BW_T - 1) / BW_T;
    if (Hq > 65535 || B > 65535) {
        set_error("flash_attn_bwd: B=%d or Hq=%d exceeds the grid limit 65535", B, Hq);
        return NCKV_E_UNSUPPORTED;
    }
    if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out | (uintptr_t)dout | (uintptr_t)dq | (uintptr_t)dk |
          (uintptr_t)dv) & 15) != 0) {
        set_error("flash_attn_bwd: tensors must be 16-byte aligned");
        return NCKV_E_ARG;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    BwdParams p;
    p.q = static_cast<const __nv_bfloat16 *>(q);
    p.k = static_cast<const __nv_bfloat16 *>(k);
    p.v = static_cast<const __nv_bfloat16 *>(v);
    p.dout = static_cast<const __nv_bfloat16 *>(dout);
    p.lse = lse;
    p.delta = static_cast<const float *>(workspace);
    p.dq = static_cast<__nv_bfloat16 *>(dq);
    p.dk = static_cast<__nv_bfloat16 *>(dk);
    p.dv = static_cast<__nv_bfloat16 *>(dv);
    p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
    p.window_left = window_left;
    p.scale = (float)(1.0 / sqrt((double)D));
    p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)D));

    const long long rows = (long long)B * T * Hq;
    attn_bwd_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(out), p.dout,
                                                                       static_cast<float *>(workspace), B, T, Hq);
    NCKV_CUDA_CHECK(cudaGetLastError());

    const size_t smem = sizeof(BwdSmem);
    static bool attr_set[64] = {false};
    int dev = 0;
    NCKV_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        NCKV_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        NCKV_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev] = true;
    }
    attn_bwd_dkdv_kernel<<<dim3((unsigned)n_tiles, (unsigned)Hkv, (unsigned)B), BW_THREADS, smem, st>>>(p);
    NCKV_CUDA_CHECK(cudaGetLastError());
    attn_bwd_dq_kernel<<<dim3((unsigned)n_tiles, (unsigned)Hq, (unsigned)B), BW_THREADS, smem, st>>>(p);
    NCKV_CUDA_CHECK(cudaGetLastError());
    return NCKV_OK;
}
