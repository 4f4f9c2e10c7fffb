// Exchange step of the sequence-split long-context path over NVLink peer memory, without NCCL.
//
// Every rank owns one symmetric buffer (same size on every GPU, peer-mapped into every process):
//     data  [2][world][per] fp32   slot (parity, r) receives rank r's partial for a step of that parity
//     flags [2][world]      u32    flag (parity, r) = number of the step whose data slot (parity, r) holds
// per = rows*D normalised partial output + rows log-sum-exp values (padded to 4 floats).
//
//   (decode_merge_kernel)    in the fused form (nckv_decode_attn_split with peer buffers) the kernel that
//                            merges the split partials stores each finished row straight into every
//                            peer's slot and its last block releases the flags; no separate push.
//   p2p_push_kernel          CTA p of rank r copies r's partial into peer p's slot (step&1, r) with
//                            plain 16-byte stores through the peer mapping, fences at system scope
//                            and then releases the flag with the step number (read from a device
//                            word, so the exchange can be replayed from a CUDA graph).
//   p2p_wait_combine_kernel  waits (bounded, wall clock) until all `world` flags of its parity show the
//                            step, then merges the partials with a log-sum-exp, reading the local
//                            buffer with L1-bypassing loads.
// Two parities suffice: a rank can only push step s+2 after it has combined step s+1, which needed every
// peer's step-s+1 push, which each peer issues after its own combine of step s (stream order).
// The reference has no counterpart: it never splits keys.
#include <math.h>

#include "nckv_common.cuh"

namespace nckv {

__global__ void __launch_bounds__(1024) p2p_push_kernel(const float4 *__restrict__ send, long long per,
                                                        const __grid_constant__ PeerPtrs peers, int world, int rank,
                                                        const unsigned *step_counter) {
    pdl_wait_prior_grids();
    pdl_launch_dependents();
    // The step number lives on the device (so the whole exchange can sit in a CUDA graph).  This
    // kernel only reads it; the wait/combine kernel that follows advances it when its last block ends.
    const unsigned step = *step_counter + 1u;
    const unsigned parity = step & 1u;
    const int peer = blockIdx.x;  // one CTA per destination
    const long long n_vec = per / 4;
    float4 *dst = reinterpret_cast<float4 *>(peers.buf[peer] + ((long long)parity * world + rank) * per);
    for (long long i = threadIdx.x; i < n_vec; i += blockDim.x) dst[i] = send[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned *flags = reinterpret_cast<unsigned *>(peers.buf[peer] + 2LL * world * per);
        unsigned *f = flags + parity * world + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(step) : "memory");
    }
}

__global__ void __launch_bounds__(256) p2p_wait_combine_kernel(const float *__restrict__ local, long long per, int world,
                                                               int rows, unsigned *step_counter,
                                                               __nv_bfloat16 *__restrict__ out,
                                                               float *__restrict__ lse_out, int32_t *status,
                                                               unsigned long long limit_ns) {
    __shared__ int s_ok;
    // No grid-dependency wait yet: the flags are the synchronisation.  This grid may be resident while
    // the kernels of its own step are still running (they release their dependents early); the step
    // counter is stable by then, since those kernels only started after the previous step's
    // wait/combine grid (the only writer of the counter) had completed.  The local rank's flag is set by
    // the last block of its own push, so passing the poll implies the local partial is in place too.
    // Whatever follows in the stream may be scheduled now: a libnckv append (and the attention kernel
    // behind it) then runs its own prologue, and loads the first key tiles of the next step, while this
    // grid waits for the peers.  Nothing a dependent reads before its own grid-dependency wait is
    // written here.
    pdl_launch_dependents();
    const unsigned step = *step_counter + 1u;  // the step whose partials are awaited
    const unsigned parity = step & 1u;
    unsigned *done = step_counter + 1;         // blocks of this grid that have finished
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < world) {
        const unsigned *f = reinterpret_cast<const unsigned *>(local + 2LL * world * per) + parity * world + threadIdx.x;
        const unsigned long long t0 = global_timer_ns();
        bool ok = false;
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if (v == step) { ok = true; break; }
            if (global_timer_ns() - t0 > limit_ns) break;
            __nanosleep(100);
        }
        if (!ok) s_ok = 0;
    }
    __syncthreads();
    pdl_wait_prior_grids();  // `out` may still be read by an earlier kernel; nothing is written before this
    const int lane = threadIdx.x & 31;
    const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (!s_ok) {  // a peer never delivered: report, write nothing, keep the context usable
        if (threadIdx.x == 0) atomicOr(status, (int)NCKV_ST_TIMEOUT);
    } else if (row < rows) {
        const float *data = local + (long long)parity * world * per;
        float M = -INFINITY;
        for (int i = 0; i < world; ++i) M = fmaxf(M, __ldcg(data + i * per + (long long)rows * NCKV_D + row));
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.f;
        if (M > -INFINITY) {
            for (int i = 0; i < world; ++i) {
                const float w = expf(__ldcg(data + i * per + (long long)rows * NCKV_D + row) - M);
                if (w == 0.f) continue;
                const float4 v = __ldcg(reinterpret_cast<const float4 *>(data + i * per + row * NCKV_D) + lane);
                L += w;
                acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
            }
            const float inv = 1.f / L;
            acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
        }
        uint2 packed;
        packed.x = pack_bf16x2(acc.x, acc.y);
        packed.y = pack_bf16x2(acc.z, acc.w);
        reinterpret_cast<uint2 *>(out + row * NCKV_D)[lane] = packed;
        if (lse_out && lane == 0) lse_out[row] = M > -INFINITY ? M + logf(L) : -INFINITY;
    }
    // the last block to finish advances the step (every block has read the old value by then)
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(done, 1u);
        if (prev == gridDim.x - 1) {
            *done = 0;
            *step_counter = step;
        }
    }
}

}  // namespace nckv

extern "C" {

size_t nckv_p2p_buffer_bytes(int world, int rows, int D) {
    if (world <= 0 || world > NCKV_MAX_PEERS || rows <= 0 || D != NCKV_D) return 0;
    return (size_t)(2LL * world * nckv::p2p_per_floats(rows)) * 4 + (size_t)2 * world * 4 + 256;
}

int nckv_p2p_push(const float *send, int rows, int D, void *const *peer_bufs, int world, int rank,
                  const uint32_t *step_counter, void *stream) {
    using namespace nckv;
    if (!send || !peer_bufs || !step_counter || rows <= 0 || world <= 0 || world > NCKV_MAX_PEERS || rank < 0 ||
        rank >= world) {
        set_error("p2p_push: bad argument (rows=%d world=%d rank=%d)", rows, world, rank);
        return NCKV_E_ARG;
    }
    if (D != NCKV_D) {
        set_error("p2p_push: head_dim %d unsupported (kernels are built for 128)", D);
        return NCKV_E_UNSUPPORTED;
    }
    PeerPtrs pp;
    for (int i = 0; i < NCKV_MAX_PEERS; ++i) pp.buf[i] = i < world ? static_cast<float *>(peer_bufs[i]) : nullptr;
    for (int i = 0; i < world; ++i) {
        if (!pp.buf[i] || ((uintptr_t)pp.buf[i] & 15)) {
            set_error("p2p_push: peer buffer %d is null or misaligned", i);
            return NCKV_E_ARG;
        }
    }
    if ((uintptr_t)send & 15) {
        set_error("p2p_push: send buffer must be 16-byte aligned");
        return NCKV_E_ARG;
    }
    // programmatic dependent launch: the grid may be scheduled while its predecessor (the merge of
    // the partial results) is still running; the kernel waits for it before it reads anything
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)world);
    cfg.blockDim = dim3(1024);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NCKV_CUDA_CHECK(cudaLaunchKernelEx(&cfg, p2p_push_kernel, reinterpret_cast<const float4 *>(send), p2p_per_floats(rows), pp,
                                       world, rank, static_cast<const unsigned *>(step_counter)));
    return NCKV_OK;
}

int nckv_p2p_wait_combine(const void *local_buf, int world, int rows, int D, uint32_t *step_counter, void *out,
                          float *lse_out, int32_t *status, uint64_t limit_ns, void *stream) {
    using namespace nckv;
    if (!local_buf || !out || !status || !step_counter || rows <= 0 || world <= 0 || world > NCKV_MAX_PEERS) {
        set_error("p2p_wait_combine: bad argument (rows=%d world=%d)", rows, world);
        return NCKV_E_ARG;
    }
    if (D != NCKV_D) {
        set_error("p2p_wait_combine: head_dim %d unsupported (kernels are built for 128)", D);
        return NCKV_E_UNSUPPORTED;
    }
    if (limit_ns == 0) limit_ns = NCKV_WAIT_LIMIT_NS;
    const int threads = 256;
    const long long blocks = ((long long)rows * 32 + threads - 1) / threads;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(threads);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NCKV_CUDA_CHECK(cudaLaunchKernelEx(&cfg, p2p_wait_combine_kernel, static_cast<const float *>(local_buf), p2p_per_floats(rows),
                                       world, rows, static_cast<unsigned *>(step_counter), static_cast<__nv_bfloat16 *>(out),
                                       lse_out, status, (unsigned long long)limit_ns));
    return NCKV_OK;
}

}  // extern "C"
