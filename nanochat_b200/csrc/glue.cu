// Decode-time elementwise glue of the transformer trunk, fused per layer and bit-exact against the
// eager bf16 op sequence it replaces (every eager op computes in fp32 and rounds its result to bf16;
// the kernels round at the same points).
//
//   glue_row_kernel   one row (one token's residual vector, C channels) per CTA:
//                       a = x                      or  bf16(x + add)                  block residual (gpt.py:148-150)
//                       y = bf16(bf16(rl * a) + bf16(xl * x0))                        lambda mix     (gpt.py:457)
//                        or bf16(a - bf16(bl * xb))                                   backout        (gpt.py:466-467)
//                        or a
//                       n = bf16(y * rsqrt(mean_fp32(y^2) + eps))                     norm           (gpt.py:42-43)
//                     The fp32 sum of squares follows the order of torch's vectorised row kernel: a
//                     block of 32 x 4 threads, thread t accumulates the 4-element vectors t, t + 128,
//                     ... sequentially (fused multiply-add), then a shuffle-down tree inside each warp
//                     (offsets 16, 8, 4, 2, 1), then warps (0 += 2, 1 += 3), then 0 += 1.
//   relu_sq_kernel    bf16(max(h, 0)^2)                                               MLP            (gpt.py:136)
//   ve_gate_kernel    bf16(v + bf16(bf16(3 * bf16(sigmoid(g))) * ve))                 value residual (gpt.py:92-95)
#include "nckv_common.cuh"

namespace nckv {

constexpr int GLUE_THREADS = 128;  // 32 x 4, the block shape whose reduction order is reproduced
constexpr int GLUE_MAX_VEC = 16;   // vectors of 4 channels per thread: C <= 8192

struct GlueRowParams {
    const uint2 *x, *add, *x0, *xb;
    uint2 *out_sum, *out_x, *out_norm;
    float rl, xl, bl, eps;
    int C, mode;  // mode 0: y = a, 1: lambda mix, 2: backout
};

__device__ __forceinline__ void unpack4(const uint2 &v, float (&f)[4]) {
    f[0] = bf16lo(v.x); f[1] = bf16hi(v.x);
    f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
}
__device__ __forceinline__ uint2 pack4(const float (&f)[4]) {
    uint2 v;
    v.x = pack_bf16x2(f[0], f[1]);
    v.y = pack_bf16x2(f[2], f[3]);
    return v;
}

__global__ void __launch_bounds__(GLUE_THREADS) glue_row_kernel(const GlueRowParams p) {
    __shared__ float s_buf[4];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int n_vec = p.C >> 2;
    const long long base = (long long)blockIdx.x * n_vec;
    float y[GLUE_MAX_VEC][4];
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < GLUE_MAX_VEC; ++k) {
        const int i = t + k * GLUE_THREADS;
        if (i < n_vec) {
            float a[4];
            unpack4(p.x[base + i], a);
            if (p.add) {
                float b[4];
                unpack4(p.add[base + i], b);
#pragma unroll
                for (int e = 0; e < 4; ++e) a[e] = round_bf16(__fadd_rn(a[e], b[e]));
                if (p.out_sum) p.out_sum[base + i] = pack4(a);
            }
            if (p.mode == 1) {
                float z[4];
                unpack4(p.x0[base + i], z);
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    a[e] = round_bf16(__fadd_rn(round_bf16(__fmul_rn(p.rl, a[e])), round_bf16(__fmul_rn(p.xl, z[e]))));
            } else if (p.mode == 2) {
                float z[4];
                unpack4(p.xb[base + i], z);
#pragma unroll
                for (int e = 0; e < 4; ++e) a[e] = round_bf16(__fsub_rn(a[e], round_bf16(__fmul_rn(p.bl, z[e]))));
            }
            if (p.out_x) p.out_x[base + i] = pack4(a);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                y[k][e] = a[e];
                acc = __fmaf_rn(a[e], a[e], acc);
            }
        }
    }
    if (!p.out_norm) return;  // uniform over the grid
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, off));
    if (lane == 0 && warp >= 2) s_buf[warp - 2] = acc;
    __syncthreads();
    if (lane == 0 && warp < 2) acc = __fadd_rn(acc, s_buf[warp]);
    __syncthreads();
    if (lane == 0 && warp == 1) s_buf[0] = acc;
    __syncthreads();
    if (t == 0) s_buf[1] = __fadd_rn(acc, s_buf[0]);
    __syncthreads();
    const float rstd = rsqrtf(__fadd_rn(__fdiv_rn(s_buf[1], (float)p.C), p.eps));
#pragma unroll
    for (int k = 0; k < GLUE_MAX_VEC; ++k) {
        const int i = t + k * GLUE_THREADS;
        if (i < n_vec) {
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = __fmul_rn(y[k][e], rstd);  // pack4 rounds to bf16
            p.out_norm[base + i] = pack4(o);
        }
    }
}

__global__ void __launch_bounds__(256) relu_sq_kernel(const uint4 *__restrict__ h, uint4 *__restrict__ out, long long n_vec) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (long long)gridDim.x * blockDim.x) {
        const uint4 v = h[i];
        uint4 o;
        const uint32_t in[4] = {v.x, v.y, v.z, v.w};
        uint32_t res[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float a = fmaxf(bf16lo(in[e]), 0.f), b = fmaxf(bf16hi(in[e]), 0.f);
            res[e] = pack_bf16x2(__fmul_rn(a, a), __fmul_rn(b, b));
        }
        o.x = res[0]; o.y = res[1]; o.z = res[2]; o.w = res[3];
        out[i] = o;
    }
}

// v, ve, v_out: (rows, Hkv, 128) bf16, v with its own row stride (it may be a column slice of a projection
// output); g: (rows, Hkv) bf16 (output of the gate's linear layer)
__global__ void __launch_bounds__(256) ve_gate_kernel(const uint4 *__restrict__ v, const __nv_bfloat16 *__restrict__ g,
                                                      const uint4 *__restrict__ ve, uint4 *__restrict__ v_out,
                                                      long long n_vec, int row_vecs, long long v_row_stride) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (long long)gridDim.x * blockDim.x) {
        const float lin = __bfloat162float(g[i >> 4]);  // 16 vectors of 8 channels per head
        const float sig = round_bf16(__fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-lin))));
        const float gate = round_bf16(__fmul_rn(3.0f, sig));
        const long long row = i / row_vecs;
        const uint4 a = v[row * v_row_stride + (i - row * row_vecs)], b = ve[i];
        const uint32_t av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
        uint32_t res[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float lo = __fadd_rn(bf16lo(av[e]), round_bf16(__fmul_rn(gate, bf16lo(bv[e]))));
            const float hi = __fadd_rn(bf16hi(av[e]), round_bf16(__fmul_rn(gate, bf16hi(bv[e]))));
            res[e] = pack_bf16x2(lo, hi);
        }
        uint4 o;
        o.x = res[0]; o.y = res[1]; o.z = res[2]; o.w = res[3];
        v_out[i] = o;
    }
}

}  // namespace nckv

extern "C" {

int nckv_glue_mix_norm(const void *x, const void *add, const void *x0, const void *x_backout, void *out_sum,
                       void *out_x, void *out_norm, int rows, int C, int mode, float resid_lambda, float x0_lambda,
                       float backout_lambda, float eps, void *stream) {
    using namespace nckv;
    if (!x || rows <= 0 || (!out_x && !out_norm && !out_sum)) {
        set_error("glue_mix_norm: null pointer or non-positive row count");
        return NCKV_E_ARG;
    }
    if (C <= 0 || (C % 4) != 0 || C > 4 * GLUE_THREADS * GLUE_MAX_VEC) {
        set_error("glue_mix_norm: C=%d must be a multiple of 4 and at most %d", C, 4 * GLUE_THREADS * GLUE_MAX_VEC);
        return NCKV_E_UNSUPPORTED;
    }
    if (mode < 0 || mode > 2 || (mode == 1 && !x0) || (mode == 2 && !x_backout) || (out_sum && !add)) {
        set_error("glue_mix_norm: mode %d lacks its operand (1 needs x0, 2 needs x_backout; out_sum needs add)", mode);
        return NCKV_E_ARG;
    }
    const uintptr_t a = (uintptr_t)x | (uintptr_t)add | (uintptr_t)x0 | (uintptr_t)x_backout | (uintptr_t)out_sum |
                        (uintptr_t)out_x | (uintptr_t)out_norm;
    if ((a & 7) || ((C * 2) & 7)) {
        set_error("glue_mix_norm: rows must be 8-byte aligned");
        return NCKV_E_ARG;
    }
    GlueRowParams p;
    p.x = static_cast<const uint2 *>(x);
    p.add = static_cast<const uint2 *>(add);
    p.x0 = static_cast<const uint2 *>(x0);
    p.xb = static_cast<const uint2 *>(x_backout);
    p.out_sum = static_cast<uint2 *>(out_sum);
    p.out_x = static_cast<uint2 *>(out_x);
    p.out_norm = static_cast<uint2 *>(out_norm);
    p.rl = resid_lambda; p.xl = x0_lambda; p.bl = backout_lambda; p.eps = eps;
    p.C = C; p.mode = mode;
    glue_row_kernel<<<rows, GLUE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(p);
    NCKV_CUDA_CHECK(cudaGetLastError());
    return NCKV_OK;
}

int nckv_glue_relu_sq(const void *h, void *out, int64_t n, void *stream) {
    using namespace nckv;
    if (!h || !out || n <= 0 || (n % 8) != 0 || (((uintptr_t)h | (uintptr_t)out) & 15)) {
        set_error("glue_relu_sq: null/misaligned pointer or element count %lld not a positive multiple of 8", (long long)n);
        return NCKV_E_ARG;
    }
    const long long n_vec = n / 8;
    long long blocks = (n_vec + 255) / 256;
    const long long cap = (long long)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    relu_sq_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4 *>(h), static_cast<uint4 *>(out), n_vec);
    NCKV_CUDA_CHECK(cudaGetLastError());
    return NCKV_OK;
}

int nckv_glue_ve_gate(const void *v, int64_t v_row_stride, const void *gate_lin, const void *ve, void *v_out, int rows,
                      int Hkv, int D, void *stream) {
    using namespace nckv;
    if (!v || !gate_lin || !ve || !v_out || rows <= 0 || Hkv <= 0) {
        set_error("glue_ve_gate: null pointer or non-positive size");
        return NCKV_E_ARG;
    }
    if (D != NCKV_D) {
        set_error("glue_ve_gate: head_dim %d unsupported (kernels are built for 128)", D);
        return NCKV_E_UNSUPPORTED;
    }
    if (v_row_stride == 0) v_row_stride = (int64_t)Hkv * D;
    if (v_row_stride % 8 || v_row_stride < (int64_t)Hkv * D) {
        set_error("glue_ve_gate: v_row_stride must be a multiple of 8 elements and span a row's heads");
        return NCKV_E_ARG;
    }
    if (((uintptr_t)v | (uintptr_t)ve | (uintptr_t)v_out) & 15) {
        set_error("glue_ve_gate: tensors must be 16-byte aligned");
        return NCKV_E_ARG;
    }
    const long long n_vec = (long long)rows * Hkv * (NCKV_D / 8);
    long long blocks = (n_vec + 255) / 256;
    const long long cap = (long long)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    ve_gate_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4 *>(v), static_cast<const __nv_bfloat16 *>(gate_lin), static_cast<const uint4 *>(ve),
        static_cast<uint4 *>(v_out), n_vec, Hkv * (NCKV_D / 8), (long long)(v_row_stride / 8));
    NCKV_CUDA_CHECK(cudaGetLastError());
    return NCKV_OK;
}

}  // extern "C"
