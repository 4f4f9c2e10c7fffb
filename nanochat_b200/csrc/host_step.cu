// One decode step for a caller whose new-token activations live in host memory (nckv_decode_step_host):
// H2D copy of q|k|v (one pinned block), fused append, decode attention, D2H copy of the output.  The copies
// are made by a copy kernel through the device alias of the pinned blocks when they have one, by the copy
// engine otherwise.
//
// The operations of a step depend only on the call's arguments, and a decode loop repeats the same
// arguments every step.  So the sequence is captured once per distinct argument list into a CUDA graph on
// a stream the library owns, ending in a one-thread kernel that writes a running count into a pinned host
// word; later calls replay the graph (one launch instead of five) and return when the host sees the count
// arrive, which takes less than waking up from a stream synchronise.  The host wait is bounded: after
// a spin limit it falls back to synchronising the stream.  A call whose arguments cannot be captured
// (or that does not fit the small plan table) runs the same operations directly on the caller's stream.
#include <mutex>
#include <string.h>

#include "nckv_common.cuh"

namespace nckv {

// The three small kernels of a step are launched with programmatic dependent launch like the library's other
// kernels: each lets its successor be scheduled at once and waits for its predecessors before touching data.
template <typename Kernel, typename... Args>
static cudaError_t launch_dependent(Kernel kernel, int grid, int block, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)block);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

__global__ void host_flag_kernel(unsigned long long *counter, volatile unsigned long long *flag) {
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const unsigned long long v = *counter + 1;
    *counter = v;
    __threadfence_system();  // the result stores of the kernels before this one are ordered before the flag
    *flag = v;
}

// 16-byte copy between a pinned host block (through its device alias) and device memory.  Inside a graph a
// copy of a few hundred KB issued by the SMs starts sooner than a copy-engine node.
__global__ void __launch_bounds__(256) host_block_copy_kernel(uint4 *dst, const uint4 *src, long long n16) {
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x)
        dst[i] = src[i];
}

static void *device_alias(const void *host) {
    void *alias = nullptr;
    if (cudaHostGetDevicePointer(&alias, const_cast<void *>(host), 0) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return alias;
}

static cudaError_t copy_block(void *dst, const void *src, size_t bytes, cudaStream_t s) {
    const long long n16 = (long long)(bytes / 16);
    const int grid = (int)((n16 + 255) / 256 < 4 * sm_count() ? (n16 + 255) / 256 : 4 * sm_count());
    return launch_dependent(host_block_copy_kernel, grid, 256, s, static_cast<uint4 *>(dst), static_cast<const uint4 *>(src),
                            n16);
}

struct StepArgs {
    const void *qkv_host;
    void *qkv_dev, *q_rot_dev, *out_dev, *out_host, *k_cache, *v_cache;
    const int32_t *cache_seqlens;
    const void *cos, *sin;
    int B, Hq, Hkv, D, T_max;
    int64_t cache_batch_stride, cache_token_stride;
    int rope_len;
    float qk_scale, eps;
    int window_left;
    void *workspace;
    size_t workspace_bytes;
    int device;
};

// The operations of one step on stream s, without any wait on the host.
static int enqueue_step(const StepArgs &a, cudaStream_t s) {
    const size_t nq = (size_t)a.B * a.Hq * a.D, nk = (size_t)a.B * a.Hkv * a.D;
    const __nv_bfloat16 *base = static_cast<const __nv_bfloat16 *>(a.qkv_dev);
    if (a.qkv_dev) {
        const void *alias = device_alias(a.qkv_host);
        const size_t bytes = (nq + 2 * nk) * 2;
        if (alias && bytes % 16 == 0 && (((uintptr_t)alias | (uintptr_t)a.qkv_dev) & 15) == 0) {
            NCKV_CUDA_CHECK(copy_block(a.qkv_dev, alias, bytes, s));
        } else {
            NCKV_CUDA_CHECK(cudaMemcpyAsync(a.qkv_dev, a.qkv_host, bytes, cudaMemcpyHostToDevice, s));
        }
    } else {  // mapped mode: the append kernel reads the host block through its device alias
        void *alias = nullptr;
        if (cudaHostGetDevicePointer(&alias, const_cast<void *>(a.qkv_host), 0) != cudaSuccess || !alias) {
            (void)cudaGetLastError();
            set_error("decode_step_host: qkv_host is not page-locked memory the device can address");
            return NCKV_E_ARG;
        }
        base = static_cast<const __nv_bfloat16 *>(alias);
    }
    void *out_target = a.out_dev;
    if (!a.out_dev) {  // mapped mode: the attention kernels store into the host block
        if (cudaHostGetDevicePointer(&out_target, a.out_host, 0) != cudaSuccess || !out_target) {
            (void)cudaGetLastError();
            set_error("decode_step_host: out_host is not page-locked memory the device can address");
            return NCKV_E_ARG;
        }
    }
    int rc = nckv_append_rope_norm(base, base + nq, base + nq + nk, a.q_rot_dev, a.k_cache, a.v_cache, a.cache_seqlens,
                                   a.cos, a.sin, a.B, 1, a.Hq, a.Hkv, a.D, a.T_max, a.cache_batch_stride,
                                   a.cache_token_stride, a.rope_len, a.qk_scale, a.eps,
                                   static_cast<int32_t *>(a.workspace), s);
    if (rc != NCKV_OK) return rc;
    rc = nckv_decode_attn(a.q_rot_dev, a.k_cache, a.v_cache, a.cache_seqlens, out_target, nullptr, nullptr, a.B, a.Hq,
                          a.Hkv, a.D, a.T_max, a.cache_batch_stride, a.cache_token_stride, 1, a.window_left, 0, 0,
                          a.workspace, a.workspace_bytes, s);
    if (rc != NCKV_OK) return rc;
    if (a.out_dev) {
        void *alias = device_alias(a.out_host);
        if (alias && (nq * 2) % 16 == 0 && (((uintptr_t)alias | (uintptr_t)a.out_dev) & 15) == 0) {
            NCKV_CUDA_CHECK(copy_block(alias, a.out_dev, nq * 2, s));
        } else {
            NCKV_CUDA_CHECK(cudaMemcpyAsync(a.out_host, a.out_dev, nq * 2, cudaMemcpyDeviceToHost, s));
        }
    }
    return NCKV_OK;
}

struct StepPlan {
    bool live = false;
    StepArgs args;
    cudaGraphExec_t exec = nullptr;
    cudaStream_t stream = nullptr;
    cudaEvent_t after_caller = nullptr;
    unsigned long long *flag_host = nullptr;   // pinned, device-addressable
    unsigned long long *counter_dev = nullptr;
    unsigned long long expected = 0;
    unsigned long long last_use = 0;
};

constexpr int STEP_PLANS = 64;  // one per (layer, cache) a caller cycles through; least recently used entry replaced
static std::mutex g_step_mutex;  // guards the table and serialises the steps that go through it
static StepPlan g_step_plans[STEP_PLANS];
static unsigned long long g_step_tick = 0;
static int g_step_misses = 0;  // plans built since the last replay: a caller that never repeats an argument list
                               // would pay a capture per call, so beyond a table's worth it gets the direct path

static void release_plan(StepPlan &pl) {
    if (pl.exec) cudaGraphExecDestroy(pl.exec);
    if (pl.stream) cudaStreamDestroy(pl.stream);
    if (pl.after_caller) cudaEventDestroy(pl.after_caller);
    if (pl.flag_host) cudaFreeHost(pl.flag_host);
    if (pl.counter_dev) cudaFree(pl.counter_dev);
    (void)cudaGetLastError();
    pl = StepPlan();
}

// Captures the step into a graph.  Returns false (plan released, error state cleared) when that is not possible.
static bool build_plan(StepPlan &pl, const StepArgs &a) {
    pl = StepPlan();
    pl.args = a;
    bool ok = cudaStreamCreateWithFlags(&pl.stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&pl.after_caller, cudaEventDisableTiming) == cudaSuccess &&
              cudaHostAlloc(reinterpret_cast<void **>(&pl.flag_host), sizeof(unsigned long long), cudaHostAllocMapped) ==
                  cudaSuccess &&
              cudaMalloc(reinterpret_cast<void **>(&pl.counter_dev), sizeof(unsigned long long)) == cudaSuccess &&
              cudaMemset(pl.counter_dev, 0, sizeof(unsigned long long)) == cudaSuccess;
    void *flag_alias = nullptr;
    if (ok) {
        *pl.flag_host = 0;
        ok = cudaHostGetDevicePointer(&flag_alias, pl.flag_host, 0) == cudaSuccess && flag_alias;
    }
    cudaGraph_t graph = nullptr;
    if (ok) ok = cudaStreamBeginCapture(pl.stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
    if (ok) {
        const int rc = enqueue_step(a, pl.stream);
        if (rc == NCKV_OK)
            (void)launch_dependent(host_flag_kernel, 1, 1, pl.stream, pl.counter_dev,
                                   static_cast<volatile unsigned long long *>(flag_alias));
        const bool ended = cudaStreamEndCapture(pl.stream, &graph) == cudaSuccess && graph;
        ok = rc == NCKV_OK && ended && cudaGraphInstantiate(&pl.exec, graph, 0) == cudaSuccess;
    }
    if (graph) cudaGraphDestroy(graph);
    if (!ok) {
        (void)cudaGetLastError();
        release_plan(pl);
        return false;
    }
    pl.live = true;
    return true;
}

}  // namespace nckv

extern "C" int nckv_decode_step_host(const void *qkv_host, void *qkv_dev, void *q_rot_dev, void *out_dev, void *out_host,
                                     void *k_cache, void *v_cache, const int32_t *cache_seqlens, const void *cos,
                                     const void *sin, int B, int Hq, int Hkv, int D, int T_max,
                                     int64_t cache_batch_stride, int64_t cache_token_stride, int rope_len, float qk_scale,
                                     float eps, int window_left, void *workspace, size_t workspace_bytes, void *stream) {
    using namespace nckv;
    if (!qkv_host || !q_rot_dev || !out_host || !workspace) {
        set_error("decode_step_host: null pointer argument");
        return NCKV_E_ARG;
    }
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || D != NCKV_D) {
        set_error("decode_step_host: bad shape (B=%d Hq=%d Hkv=%d D=%d)", B, Hq, Hkv, D);
        return D != NCKV_D ? NCKV_E_UNSUPPORTED : NCKV_E_ARG;
    }
    cudaStream_t caller = static_cast<cudaStream_t>(stream);
    StepArgs a;
    memset(&a, 0, sizeof(a));  // padding bytes too: plans are compared with memcmp
    a.qkv_host = qkv_host; a.qkv_dev = qkv_dev; a.q_rot_dev = q_rot_dev; a.out_dev = out_dev; a.out_host = out_host;
    a.k_cache = k_cache; a.v_cache = v_cache; a.cache_seqlens = cache_seqlens; a.cos = cos; a.sin = sin;
    a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.T_max = T_max;
    a.cache_batch_stride = cache_batch_stride; a.cache_token_stride = cache_token_stride;
    a.rope_len = rope_len; a.qk_scale = qk_scale; a.eps = eps; a.window_left = window_left;
    a.workspace = workspace; a.workspace_bytes = workspace_bytes;
    NCKV_CUDA_CHECK(cudaGetDevice(&a.device));

    {
        std::lock_guard<std::mutex> lock(g_step_mutex);
        StepPlan *pl = nullptr, *victim = &g_step_plans[0];
        for (StepPlan &c : g_step_plans) {
            if (c.live && memcmp(&c.args, &a, sizeof(a)) == 0) pl = &c;
            if (!c.live || (victim->live && c.last_use < victim->last_use)) victim = &c;
        }
        if (pl) {
            g_step_misses = 0;
        } else if (g_step_misses < STEP_PLANS) {
            ++g_step_misses;
            if (victim->live) release_plan(*victim);
            if (build_plan(*victim, a)) pl = victim;
        }
        if (pl) {
            pl->last_use = ++g_step_tick;
            // what the caller has enqueued so far (cache_seqlens updates, for instance) comes first
            NCKV_CUDA_CHECK(cudaEventRecord(pl->after_caller, caller));
            NCKV_CUDA_CHECK(cudaStreamWaitEvent(pl->stream, pl->after_caller, 0));
            NCKV_CUDA_CHECK(cudaGraphLaunch(pl->exec, pl->stream));
            const unsigned long long want = ++pl->expected;
            volatile unsigned long long *flag = pl->flag_host;
            bool seen = false;
            for (long spin = 0; spin < 20000000L; ++spin) {  // some tens of milliseconds at most
                if (*flag >= want) {
                    seen = true;
                    break;
                }
            }
            if (!seen) NCKV_CUDA_CHECK(cudaStreamSynchronize(pl->stream));
            return NCKV_OK;
        }
    }
    // no plan: the same operations on the caller's stream
    const int rc = enqueue_step(a, caller);
    if (rc != NCKV_OK) return rc;
    NCKV_CUDA_CHECK(cudaStreamSynchronize(caller));
    return NCKV_OK;
}
