/*
 * nckv.h — C ABI of libnckv.so, the B200 (sm_100a) KV-cache decode path for nanochat.
 *
 * Every entry point takes raw device pointers, sizes, element strides and a CUDA
 * stream (passed as void*, i.e. a cudaStream_t).  There are no torch types here;
 * the Python package binds these symbols with ctypes.
 *
 * Conventions
 *   - dtype: all tensors are bf16 unless a parameter says otherwise; head_dim D must be 128.
 *   - return value: 0 = launched; < 0 = rejected on the host (NCKV_E_*), nothing ran.
 *     Device-side guards (capacity overflow, a bounded wait that ran out) never trap:
 *     they skip the access and OR a bit into the int32 status word at the start of the
 *     workspace / at `status`; read it with nckv_read_status().
 *   - nothing here allocates device memory except where stated.
 *   - layouts follow the reference: new q/k/v are (B, T_new, H, D) contiguous; one
 *     layer's cache is a (B, T_max, Hkv, D) view with element strides
 *     (cache_batch_stride, cache_token_stride, D, 1); cache_seqlens is int32 (B,).
 *
 * Reference symbols are cited as file:line inside the nanochat source tree.
 */
#ifndef NCKV_H
#define NCKV_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define NCKV_API __attribute__((visibility("default")))
#else
#define NCKV_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* host-side rejection codes */
#define NCKV_OK 0
#define NCKV_E_ARG (-1)         /* null pointer, non-positive size, misaligned pointer */
#define NCKV_E_UNSUPPORTED (-2) /* head_dim != 128, group size > 16, batch too large ... */
#define NCKV_E_CAPACITY (-3)    /* host-known capacity overflow (T_new > T_max, workspace too small) */
#define NCKV_E_CUDA (-4)        /* a CUDA runtime/driver call failed; see nckv_last_error() */

/* device status bits (OR-ed into the status word) */
#define NCKV_ST_OVERFLOW 1u   /* cache_seqlens[b] + T_new > T_max, or position >= rope_len: row skipped */
#define NCKV_ST_TIMEOUT 2u    /* a bounded wait on a shared-memory barrier ran out */
#define NCKV_ST_BAD_SEQLEN 4u /* negative cache_seqlens[b] */
#define NCKV_ST_BAD_PAGE 8u   /* a block-table entry outside the page pool: the tile was read as zeros / the row not written */

/* Library version and the SM architecture the kernels were compiled for ("sm_100a"). */
NCKV_API int nckv_version(void);
NCKV_API const char *nckv_arch(void);
/* Text of the last host-side error on this thread (empty string if none). */
NCKV_API const char *nckv_last_error(void);

/*
 * Bytes of scratch nckv_decode_attn / nckv_prefill_attn need for a problem of this shape
 * on the current device.  The first 256 bytes hold the status word; the rest holds split
 * partials and arrival counters.  The buffer must be zero-filled once after allocation
 * (the kernels leave the counters at zero when they finish) and must not be shared by
 * launches that overlap in time.
 */
NCKV_API size_t nckv_workspace_bytes(int B, int Hq, int Hkv, int D);

/* Synchronising read (stream-ordered copy + stream sync) of a status word; returns the
 * word (>= 0) or NCKV_E_CUDA.  If `clear` is non-zero the word is reset to 0. */
NCKV_API int nckv_read_status(void *status_word, int clear, void *stream);

/*
 * Fused RoPE + QK-norm + scale + KV append.
 * Replaces apply_rotary_emb (gpt.py:57-63), norm (gpt.py:42-43), the 1.2 scale
 * (gpt.py:101-102) and the cache slice-assign of flash_attn_with_kvcache
 * (flash_attention.py:160-162), per row:  position p = cache_seqlens[b] + t,
 *   q_out[b,t,h,:]        = bf16(1.2 * rmsnorm(rope(q_in[b,t,h,:], cos[p], sin[p])))
 *   k_cache[b,p,h,:]      = same transform of k_in[b,t,h,:]
 *   v_cache[b,p,h,:]      = v_in[b,t,h,:]
 * with a bf16 rounding after every reference op so the bytes equal the eager bf16 path.
 * cos/sin are the reference's own bf16 tables, (rope_len, D/2) contiguous.
 * q_in may be NULL (then q_out is ignored) and q_out may alias q_in.
 * cache_seqlens is not modified.
 */
NCKV_API int nckv_append_rope_norm(const void *q_in, const void *k_in, const void *v_in, void *q_out,
                          void *k_cache, void *v_cache, const int32_t *cache_seqlens,
                          const void *cos, const void *sin, int B, int T_new, int Hq, int Hkv,
                          int D, int T_max, int64_t cache_batch_stride,
                          int64_t cache_token_stride, int rope_len, float qk_scale, float eps,
                          int32_t *status, void *stream);

/*
 * nckv_append_rope_norm with q_in, k_in and v_in given as strided rows: token t of row b starts
 * (b T_new + t) * stride elements into the tensor, its heads packed behind each other.  Lets q, k and v be
 * column slices of the output of one [c_q; c_k; c_v] projection.  Strides are multiples of 8 elements;
 * 0 means packed.  q_out is always packed (B, T_new, Hq, D).
 */
NCKV_API int nckv_append_rope_norm_strided(const void *q_in, const void *k_in, const void *v_in, int64_t q_token_stride,
                                  int64_t k_token_stride, int64_t v_token_stride, void *q_out, void *k_cache,
                                  void *v_cache, const int32_t *cache_seqlens, const void *cos, const void *sin, int B,
                                  int T_new, int Hq, int Hkv, int D, int T_max, int64_t cache_batch_stride,
                                  int64_t cache_token_stride, int rope_len, float qk_scale, float eps, int32_t *status,
                                  void *stream);

/*
 * Same as nckv_append_rope_norm for a sequence-split cache (no counterpart in the reference):
 * `positions[b]` is the sequence position of row b's first new token (drives RoPE, as
 * cache_seqlens does above) while `write_slots[b]` is the index in THIS shard's cache where its
 * k/v go, or -1 if another shard owns that position (q_out is still produced).
 */
NCKV_API int nckv_append_rope_norm_at(const void *q_in, const void *k_in, const void *v_in, void *q_out,
                             void *k_cache, void *v_cache, const int32_t *positions, const int32_t *write_slots,
                             const void *cos, const void *sin, int B, int T_new, int Hq, int Hkv,
                             int D, int T_max, int64_t cache_batch_stride, int64_t cache_token_stride,
                             int rope_len, float qk_scale, float eps, int32_t *status, void *stream);

/*
 * Introspection of kernel (b)'s work list: writes, for every row, the half-open range of key
 * positions [key_begin[b], key_end[b]) the decode kernel would read for these arguments, computed on
 * the device by the same routine the attention kernels call.  Restates the visible-key rule of
 * flash_attention.py:83-88 (keys [max(0, L - w), L] of a row whose new token sits at position L),
 * intersected with [kv_begin, kv_end) when that range is not empty.  With split_block > 0 the
 * lengths are global and the ranges are local indices into shard split_rank's block-cyclic part (as
 * nckv_decode_attn_split reads them).  Out-of-range lengths are clamped and flagged in *status like
 * the attention entry points do.  Used by the parity tests.
 */
NCKV_API int nckv_decode_key_ranges(const int32_t *cache_seqlens, int B, int T_max, int seqlen_offset,
                                    int window_left, int kv_begin, int kv_end, int split_world, int split_rank,
                                    int split_block, int32_t *key_begin, int32_t *key_end, int32_t *status,
                                    void *stream);

/*
 * Bookkeeping of the sequence-split long-context path (no counterpart in the reference): key
 * positions are owned block-cyclically, position p by shard (p / block) % world at local index
 * (p / (block*world)) * block + p % block.  From the global cache_seqlens (lengths before the new
 * tokens) computes, for shard `rank`: local_len_after[b] = keys of row b this shard holds once the
 * T_new new tokens are in, and write_slot[b] = local index for the new token, or -1 if it is not ours.
 * The *_split entry points below apply the same rule inside their kernels; this one exposes it (to
 * the parity tests, and to callers that lay out their own caches).  Its kernel does not release its
 * dependents early, so a libnckv kernel launched behind it sees the finished arrays.
 */
NCKV_API int nckv_kv_split_plan(const int32_t *cache_seqlens, int B, int T_new, int world, int rank, int block,
                       int32_t *local_len_after, int32_t *write_slot, void *stream);

/*
 * nckv_append_rope_norm for shard `rank` of a block-cyclic sequence split (no counterpart in the
 * reference): cache_seqlens are the GLOBAL lengths (they drive RoPE), the caches are this shard's
 * compact part (capacity T_local), and k/v of row b are stored only if this shard owns position
 * cache_seqlens[b], at the local index nckv_kv_split_plan would report.  q_out is always produced.
 * T_new must be 1.
 */
NCKV_API int nckv_append_rope_norm_split(const void *q_in, const void *k_in, const void *v_in, void *q_out,
                                void *k_cache, void *v_cache, const int32_t *cache_seqlens, const void *cos,
                                const void *sin, int B, int T_new, int Hq, int Hkv, int D, int T_local,
                                int64_t cache_batch_stride, int64_t cache_token_stride, int rope_len,
                                float qk_scale, float eps, int world, int rank, int block, int32_t *status,
                                void *stream);

/*
 * Plain append (k already rotated/normalised by the caller): the cache write of
 * flash_attn_with_kvcache (flash_attention.py:160-162) with per-row positions.
 */
NCKV_API int nckv_append(const void *k_in, const void *v_in, void *k_cache, void *v_cache,
                const int32_t *cache_seqlens, int B, int T_new, int Hkv, int D, int T_max,
                int64_t cache_batch_stride, int64_t cache_token_stride, int32_t *status,
                void *stream);

/*
 * One whole decode step of a layer for host-resident activations: the KV branch of
 * CausalSelfAttention.forward (gpt.py:97-121) for T == 1, including the copies the reference's
 * callers do around it (engine.py:279: ids to the device; the result read back on the host).
 * qkv_host: pinned host block [q (B,Hq,D) | k (B,Hkv,D) | v (B,Hkv,D)] bf16; qkv_dev: device block of
 * the same size; q_rot_dev, out_dev: device (B,Hq,D) bf16 scratch/result; out_host: pinned host
 * (B,Hq,D) bf16.  Performs H2D, nckv_append_rope_norm, nckv_decode_attn, D2H and waits for them; on
 * return out_host holds the attention output.  cache_seqlens is not advanced.  The operations are
 * ordered after everything already enqueued on `stream`.  They are captured once per distinct argument
 * list (a table of 64, least recently used entry replaced; a caller that never repeats an argument list gets the operations directly on its stream) into a CUDA graph on a stream of the
 * library's own and replayed by later calls; the wait is a bounded spin on a pinned word the graph's last
 * node writes, with a stream synchronise as its fallback.  Calls are serialised by a mutex.
 * Mapped mode: with qkv_dev == NULL the append kernel reads the pinned host block itself (over
 * PCIe, through the device alias of the host pointer) and no H2D copy is enqueued; with
 * out_dev == NULL the attention kernels store the result straight into out_host and no D2H copy
 * is enqueued.  Both blocks must then be page-locked memory the device can address
 * (cudaHostAlloc / cudaHostRegister); anything else is rejected with NCKV_E_ARG.
 */
NCKV_API int nckv_decode_step_host(const void *qkv_host, void *qkv_dev, void *q_rot_dev, void *out_dev, void *out_host,
                          void *k_cache, void *v_cache, const int32_t *cache_seqlens, const void *cos,
                          const void *sin, int B, int Hq, int Hkv, int D, int T_max, int64_t cache_batch_stride,
                          int64_t cache_token_stride, int rope_len, float qk_scale, float eps, int window_left,
                          void *workspace, size_t workspace_bytes, void *stream);

/*
 * Split-KV decode attention, one query token per row (T_new == 1).
 * Replaces the Tq == 1 branch of _sdpa_attention (flash_attention.py:83-89) as reached
 * from flash_attn_with_kvcache (flash_attention.py:165-177), with per-row lengths:
 *   n_b   = cache_seqlens[b] + seqlen_offset          (keys present, incl. the new one)
 *   keys  = [max(0, n_b - 1 - window_left), n_b)      (window_left < 0: from 0)
 *           intersected with [kv_begin, kv_end) when kv_end > kv_begin (a cross-GPU shard)
 *   out[b,h,:] = softmax(q[b,h,:] . K[keys, h / (Hq/Hkv), :] / sqrt(D)) V[keys, ...]
 * q is (B, Hq, D) contiguous, out is (B, Hq, D) bf16.  When lse_out != NULL it receives
 * the natural-log sum-exp per (b, h) as fp32 (-inf for an empty key range, out = 0), and
 * when out_f32 != NULL the normalised output is also written there as fp32 (for the
 * cross-GPU combine).  workspace: see nckv_workspace_bytes().
 * Ordering: the kernels start while the kernel launched before them in the stream may still be
 * running (programmatic dependent launch) and read cache_seqlens and all but the last
 * max(seqlen_offset, 1) visible positions of every row before they wait for it.  This only matters
 * behind a kernel that releases its dependents before it has finished, which among ordinary
 * kernels only libnckv's own appends do: an append directly in front of this call must not have
 * written older positions than those (a decode step appends exactly that one position) and must
 * not be what produces cache_seqlens.  A kernel that never releases early (every torch or library
 * kernel, nckv_kv_split_plan) has completed before these kernels read anything.
 */
NCKV_API int nckv_decode_attn(const void *q, const void *k_cache, const void *v_cache,
                     const int32_t *cache_seqlens, void *out, float *out_f32, float *lse_out,
                     int B, int Hq, int Hkv, int D, int T_max, int64_t cache_batch_stride,
                     int64_t cache_token_stride, int seqlen_offset, int window_left,
                     int kv_begin, int kv_end, void *workspace, size_t workspace_bytes,
                     void *stream);

/*
 * nckv_decode_attn over shard `rank` of a block-cyclic sequence split (no counterpart in the
 * reference, which never splits the keys): cache_seqlens are the GLOBAL lengths, the caches are this
 * shard's compact part (capacity T_local), and the keys read of row b are the local indices
 * [0, owned_below(cache_seqlens[b] + seqlen_offset)) (full causal; windows need global indices, use
 * kv_begin/kv_end of nckv_decode_attn for those).  part_out (B, Hq, D) fp32 receives the normalised
 * partial output and part_lse (B, Hq) fp32 its natural-log sum-exp (-inf and zeros for a shard
 * without keys of a row).
 * With peer_bufs != NULL (world pointers: every rank's exchange buffer as mapped into this process,
 * see nckv_p2p_buffer_bytes) the kernel that merges the split partials also stores the packed
 * partial into this rank's slot of every peer's buffer and releases the step's flag there, which
 * replaces a separate nckv_p2p_push; follow it with nckv_p2p_wait_combine.  Plain peer stores only.
 */
NCKV_API int nckv_decode_attn_split(const void *q, const void *k_cache, const void *v_cache,
                           const int32_t *cache_seqlens, float *part_out, float *part_lse, int B, int Hq,
                           int Hkv, int D, int T_local, int64_t cache_batch_stride, int64_t cache_token_stride,
                           int seqlen_offset, int world, int rank, int block, void *const *peer_bufs,
                           const uint32_t *step_counter, void *workspace, size_t workspace_bytes, void *stream);

/*
 * Decode attention without any allocation (no counterpart in the reference; same computation and
 * arguments as nckv_decode_attn, minus the workspace).
 *
 * For callers that cannot obtain device memory at the point of the call: a serving loop that has
 * handed all of its memory to the KV cache up front, a host thread that may not enter the torch
 * allocator, a plugin boundary that forbids cudaMalloc.  The split partials and the ticket
 * counter live in a 14 MiB device array built into the library (held on every GPU that loads it,
 * until the process exits), so the call performs no cudaMalloc / cudaFree and calls no allocating
 * routine.  Limits and rules:
 *   - shapes whose nckv_workspace_bytes() exceeds 14 MiB are rejected with NCKV_E_CAPACITY
 *     (group sizes Hq/Hkv up to 4 fit, any B up to the per-launch row limit);
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress), which
 *     is also when the CUDA runtime may first set the array up on that device (modules load
 *     lazily).  Make that first call at start-up: before the process gives its free memory away,
 *     and outside any stream capture;
 *   - all calls on a device share the one array: two calls whose kernels can overlap on the GPU
 *     (different streams, no ordering between them) race on it.  Serialise them;
 *   - if status_word != NULL it receives the device address of the status word, to be read with
 *     nckv_read_status().
 */
NCKV_API int nckv_decode_attn_static(const void *q, const void *k_cache, const void *v_cache,
                            const int32_t *cache_seqlens, void *out, float *out_f32, float *lse_out,
                            int B, int Hq, int Hkv, int D, int T_max, int64_t cache_batch_stride,
                            int64_t cache_token_stride, int seqlen_offset, int window_left,
                            int kv_begin, int kv_end, void **status_word, void *stream);

/*
 * Log-sum-exp combine of n_parts partial attention results (the exchange step of the
 * sequence-split long-context path; no counterpart in the reference, which never splits
 * the keys): parts_o holds n_parts blocks of (rows, D) fp32 normalised partial outputs,
 * part_stride_o elements apart (>= rows*D, multiple of 4); parts_lse holds n_parts blocks of
 * (rows,) fp32, part_stride_lse elements apart (>= rows), so the two may be views of one
 * gathered buffer; out is (rows, D) bf16, lse_out (optional) is (rows,) fp32.
 *   lse = log sum_i exp(lse_i),  out = sum_i exp(lse_i - lse) * o_i ; parts with -inf drop out.
 */
NCKV_API int nckv_lse_combine(const float *parts_o, const float *parts_lse, int n_parts, int rows, int D,
                     int64_t part_stride_o, int64_t part_stride_lse, void *out, float *lse_out, void *stream);

/*
 * The same exchange over NVLink peer memory instead of a collective library (no counterpart in
 * the reference).  Every rank owns a symmetric buffer of nckv_p2p_buffer_bytes() bytes, zeroed once
 * and mapped into every peer (peer_bufs[r] = rank r's buffer as seen from this process).  The step
 * number (1, 2, 3, ... in lock step on all ranks) lives in two device words `step_counter[2]`
 * (zeroed once; the wait/combine kernel advances it), so the exchange can be replayed from a CUDA
 * graph.  Per step:
 * nckv_p2p_push copies this rank's packed partial
 * ([rows*D normalised output | rows lse, padded to 4 floats] fp32) into its slot of every peer's
 * buffer and releases a flag there; nckv_p2p_wait_combine waits until the local buffer has all
 * `world` flags of that step (at most limit_ns of wall time, 0 = default; on timeout it sets
 * NCKV_ST_TIMEOUT in *status, writes nothing and returns), then merges like nckv_lse_combine.
 */
NCKV_API size_t nckv_p2p_buffer_bytes(int world, int rows, int D);
NCKV_API int nckv_p2p_push(const float *send, int rows, int D, void *const *peer_bufs, int world, int rank,
                  const uint32_t *step_counter, void *stream);
NCKV_API int nckv_p2p_wait_combine(const void *local_buf, int world, int rows, int D, uint32_t *step_counter,
                          void *out, float *lse_out, int32_t *status, uint64_t limit_ns, void *stream);

/*
 * Prefill broadcast: KVCache.prefill (engine.py:123-137).  Copies the first p tokens of a
 * batch-1 cache (L, 1, T_src, Hkv, D) into every row of (L, B, T_dst, Hkv, D) for K and V
 * and, when dst_seqlens != NULL, sets dst_seqlens[b] = p.  The source is read once.
 */
NCKV_API int nckv_prefill_broadcast(const void *src_k, const void *src_v, void *dst_k, void *dst_v,
                           int32_t *dst_seqlens, int L, int B, int p, int Hkv, int D, int T_src,
                           int T_dst, void *stream);

/*
 * Paged KV storage (the "next" format after the dense (L, B, T_max, H, D) tensors of engine.py:98-100;
 * no counterpart in the reference).  One layer's K or V is a pool of pages (n_pages, page_tokens, Hkv,
 * D) with element strides (page_stride, token_stride, D, 1); block_table is int32 (B, max_pages): token t
 * of row b lives in page block_table[b][t / page_tokens] at index t % page_tokens.  page_tokens must be a
 * multiple of nckv_paged_tile_tokens() so that a tile of keys never straddles two pages.  Rows may
 * share pages they only read (a common prompt).  A table entry outside [0, n_pages) met by a kernel
 * sets NCKV_ST_BAD_PAGE and is skipped (read as zeros / not written).
 *   nckv_append_rope_norm_paged   nckv_append_rope_norm with the k/v rows written through the table
 *   nckv_decode_attn_paged        nckv_decode_attn (all of its semantics except kv_begin/kv_end) reading
 *                                 through the table
 *   nckv_paged_fill               KVCache.prefill (engine.py:123-137) into pages: n_jobs jobs of three
 *                                 int32 (page, first source token, tokens) copy runs of the batch-1 source
 *                                 cache (L, 1, T_src, Hkv, D) into pages of the pools (L, n_pages,
 *                                 page_tokens, Hkv, D), K and V in one launch.  With the full prompt pages
 *                                 shared between the rows this writes each of them once instead of B times.
 */
NCKV_API int nckv_paged_tile_tokens(void);
NCKV_API int nckv_append_rope_norm_paged(const void *q_in, const void *k_in, const void *v_in, void *q_out, void *k_pool,
                                void *v_pool, const int32_t *block_table, const int32_t *cache_seqlens,
                                const void *cos, const void *sin, int B, int T_new, int Hq, int Hkv, int D,
                                int page_tokens, int max_pages, int n_pages, int64_t page_stride, int64_t token_stride,
                                int rope_len, float qk_scale, float eps, int32_t *status, void *stream);
NCKV_API int nckv_decode_attn_paged(const void *q, const void *k_pool, const void *v_pool, const int32_t *block_table,
                           const int32_t *cache_seqlens, void *out, float *out_f32, float *lse_out, int B, int Hq,
                           int Hkv, int D, int page_tokens, int max_pages, int n_pages, int64_t page_stride,
                           int64_t token_stride, int seqlen_offset, int window_left, void *workspace,
                           size_t workspace_bytes, void *stream);
NCKV_API int nckv_paged_fill(const void *src_k, const void *src_v, void *k_pool, void *v_pool, const int32_t *jobs,
                    int n_jobs, int L, int Hkv, int D, int T_src, int page_tokens, int n_pages, void *stream);

/*
 * Dense (T_new >= 1) causal attention over a cache or plain k/v, tcgen05/TMEM tiles.
 * Replaces the full-causal and explicit-mask branches of _sdpa_attention
 * (flash_attention.py:79-80, 92-102) as reached from flash_attn_with_kvcache
 * (flash_attention.py:165-177) and flash_attn_func (flash_attention.py:107-128).
 * Query t of row b sits at absolute position p = cache_seqlens[b] + t (cache_seqlens may
 * be NULL = all zero) and sees keys j with j <= p and (window_left < 0 or p - j <= window_left).
 * q and out are (B, T_new, Hq, D) contiguous; k/v are (B, T_k, Hkv, D) views with the
 * given element strides, T_k being the capacity of the view.
 */
NCKV_API int nckv_prefill_attn(const void *q, const void *k, const void *v, const int32_t *cache_seqlens,
                      void *out, int B, int T_new, int Hq, int Hkv, int D, int T_k,
                      int64_t kv_batch_stride, int64_t kv_token_stride, int window_left,
                      int32_t *status, void *stream);

/*
 * flash_attn_func for training (flash_attention.py:107-128, caller gpt.py:108): causal attention with a
 * left window over plain (B, T, H, D) bf16 tensors, forward with the log-sum-exp kept, and backward.
 * Replaces F.scaled_dot_product_attention and the autograd graph behind it on this path.
 *   nckv_flash_attn_fwd   out (B, T, Hq, D) and lse (B, Hq, T) fp32, the natural log of each row's sum of
 *                         exponentials of the scaled scores.  Same kernel as nckv_prefill_attn; `status` is
 *                         the first word of a zero-initialised workspace as there.
 *   nckv_flash_attn_bwd   dq (B, T, Hq, D), dk and dv (B, T, Hkv, D) from q, k, v, out, dout and lse.
 *                         `workspace` holds nckv_flash_attn_bwd_workspace_bytes(B, T, Hq) bytes of scratch:
 *                         rowsum(dout * out), and in its last 256 bytes the call's device status word (an int32
 *                         of NCKV_ST_* bits, cleared by the call, 0 = no guard fired).  All pointers 32-byte
 *                         aligned.  No atomics are used: the gradients are the same bits on every run.
 */
NCKV_API int nckv_flash_attn_fwd(const void *q, const void *k, const void *v, void *out, float *lse, int B, int T,
                        int Hq, int Hkv, int D, int window_left, int32_t *status, void *stream);
NCKV_API size_t nckv_flash_attn_bwd_workspace_bytes(int B, int T, int Hq);
NCKV_API int nckv_flash_attn_bwd(const void *q, const void *k, const void *v, const void *out, const void *dout,
                        const float *lse, void *dq, void *dk, void *dv, void *workspace, int B, int T, int Hq,
                        int Hkv, int D, int window_left, void *stream);

/*
 * Decode-time glue of the transformer trunk around the KV branch: the elementwise ops between the
 * matrix products of GPT.forward / Block.forward for one new token per row, fused per layer.  Each
 * kernel rounds to bf16 exactly where the eager op sequence does, so results are bit-identical to it.
 *
 * nckv_glue_mix_norm, one launch for (rows, C) bf16 row vectors:
 *     a = x                          or, with add != NULL,  a = bf16(x + add)      residual add, gpt.py:148-150
 *     mode 0:  y = a
 *     mode 1:  y = bf16(bf16(resid_lambda * a) + bf16(x0_lambda * x0))             gpt.py:457
 *     mode 2:  y = bf16(a - bf16(backout_lambda * x_backout))                      gpt.py:466-467
 *     out_norm = bf16(y * rsqrt(mean(y^2) + eps))   (norm, gpt.py:42-43)           gpt.py:149-150, 468
 * out_sum (optional, needs add) receives a, out_x (optional) receives y, out_norm (optional) the
 * normalised row; the fp32 sum of squares is accumulated in the order of torch's row kernel.
 * nckv_glue_relu_sq: out = bf16(max(h, 0)^2) over n elements (n % 8 == 0), MLP.forward gpt.py:136.
 * nckv_glue_ve_gate: v_out = bf16(v + bf16(bf16(3 * bf16(sigmoid(gate_lin))) * ve)) with v, ve (rows, Hkv, D)
 * and gate_lin (rows, Hkv) the output of the gate's linear layer: the value residual of gpt.py:92-95.  v may have
 * its own row stride in elements (v_row_stride, 0 = packed): a column slice of a projection output.
 */
NCKV_API int nckv_glue_mix_norm(const void *x, const void *add, const void *x0, const void *x_backout, void *out_sum,
                       void *out_x, void *out_norm, int rows, int C, int mode, float resid_lambda, float x0_lambda,
                       float backout_lambda, float eps, void *stream);
NCKV_API int nckv_glue_relu_sq(const void *h, void *out, int64_t n, void *stream);
NCKV_API int nckv_glue_ve_gate(const void *v, int64_t v_row_stride, const void *gate_lin, const void *ve, void *v_out, int rows, int Hkv, int D,
                      void *stream);

#ifdef __cplusplus
}
#endif
#endif /* NCKV_H */
