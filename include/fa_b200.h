/*
 * C-ABI of the B200 (sm_100a) FlashAttention library  --  libfa_b200.so
 *
 * Every entry point is `extern "C"`, takes plain device pointers, sizes and
 * element strides, launches on the caller's stream, never allocates, never
 * synchronises and never reads device memory on the host.  Return value:
 * FA_OK or an fa_status error; fa_last_error() gives the message of the last
 * failure on the calling thread.  There is no CPU fallback behind any of them.
 *
 * The entry points stand in for the pybind functions of the reference's two
 * extension modules (paths inside the reference project):
 *   v2  csrc/ascend910/flash_attn_npu/flash_api.cpp:1330-1338
 *         fwd :639, varlen_fwd :848, fwd_kvcache :356, bwd :1279, varlen_bwd :1092
 *   v3  csrc/ascend910/flash_attn_npu_3/flash_api.cpp:829-835
 *         fwd :60, bwd :573, get_scheduler_metadata :506
 * Outputs and workspaces are allocated by the caller (the reference allocates
 * them as at::Tensor inside those functions, e.g. flash_api.cpp:443, :567).
 */
#ifndef FA_B200_H
#define FA_B200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    FA_OK = 0,
    FA_ERR_NULL = 1,        /* required pointer is null                      */
    FA_ERR_BAD_DTYPE = 2,   /* dtype is not f16 / bf16                       */
    FA_ERR_BAD_SHAPE = 3,   /* sizes out of range or inconsistent            */
    FA_ERR_MISALIGNED = 4,  /* pointer or stride not a multiple of 16 bytes  */
    FA_ERR_UNSUPPORTED = 5, /* feature the reference rejects as well         */
    FA_ERR_WORKSPACE = 6,   /* workspace missing or too small                */
    FA_ERR_CUDA = 7         /* a CUDA runtime call failed                    */
} fa_status;

typedef enum { FA_F16 = 0, FA_BF16 = 1 } fa_dtype;

/* A (batch, seq, head, dim) view; strides in ELEMENTS, dim stride is 1.
 * Packed "TND" tensors: batch stride unused, row index = cu_seqlens[b] + i.
 * Paged caches: batch = block, seq = row inside the page. */
typedef struct {
    void*   ptr;
    int64_t stride_b;
    int64_t stride_s;
    int64_t stride_h;
} fa_tensor;

/* ------------------------------------------------------------------------
 * Forward.  One parameter block serves the three forward entry points.
 *   fa_fwd          dense (B,S,H,D)                  mha_fwd         flash_api.cpp:639
 *   fa_varlen_fwd   packed (T,H,D) + cu_seqlens      mha_varlen_fwd  flash_api.cpp:848
 *   fa_fwd_kvcache  dense or paged KV cache, in-place append of k_new/v_new,
 *                   rotary, split-KV                 mha_fwd_kvcache flash_api.cpp:356
 *                   (v3: mha_fwd csrc/ascend910/flash_attn_npu_3/flash_api.cpp:60)
 * Window sizes are the caller's raw values; -1 = unbounded.  `causal` forces
 * window_right = 0.  The mask is aligned to the bottom-right corner.
 * Rows without any visible key give O = 0 and LSE = +inf.
 * ---------------------------------------------------------------------- */
typedef struct {
    fa_tensor q, k, v, o;
    float*    lse;                 /* fp32 */
    int64_t   lse_stride_b, lse_stride_h, lse_stride_s;

    const int32_t* cu_seqlens_q;   /* (b+1) or null                                   */
    const int32_t* cu_seqlens_k;   /* (b+1) or null                                   */
    const int32_t* seqused_k;      /* (b) keys in use per sequence (cache_seqlens)    */
    const int32_t* block_table;    /* (b, block_table_stride) or null = not paged      */
    int64_t        block_table_stride;
    int32_t        page_size;
    const int32_t* cache_batch_idx;/* (b) or null; dense cache only                    */
    const float*   alibi_slopes;   /* (hq) or (b,hq) fp32, or null                     */
    int64_t        alibi_stride_b; /* 0 when slopes are shared by the batch            */

    int32_t b, sq, sk;             /* sq/sk: max lengths for varlen / cache            */
    int32_t total_q;               /* rows of a packed q tensor (cu_seqlens_q != null) */
    int32_t total_k;               /* rows of a packed k/v tensor (cu_seqlens_k != null) */
    int32_t hq, hkv, d, dv;
    float   scale, softcap;
    int32_t causal, window_left, window_right;
    int32_t dtype;                 /* fa_dtype                                         */

    /* new tokens appended in place at positions seqused_k[b] .. +s_new-1 (kvcache)   */
    fa_tensor k_new, v_new;
    int32_t   s_new;
    const void* rotary_cos;        /* (seqlen_ro, rotary_dim/2), q's dtype, or null    */
    const void* rotary_sin;
    int32_t   rotary_dim, rotary_interleaved, seqlen_ro;

    /* split-KV.  num_splits: 0 = heuristic, 1 = none, n = exactly n.               */
    int32_t num_splits;
    /* Restrict every sequence to keys [kv_begin, kv_end) (kv_end <= 0: no limit)
     * and, if partials_only != 0, leave fp32 partial (O, LSE) in o_partial /
     * lse_partial instead of combining: the cross-GPU KV-sharded decode.           */
    int32_t kv_begin, kv_end, partials_only;
    float*  o_partial;             /* (splits, rows, dv) fp32, rows = b*sq*hq          */
    float*  lse_partial;           /* (splits, rows) fp32                              */
    void*   workspace;             /* >= fa_fwd_workspace_bytes()                      */
    size_t  workspace_bytes;
    const void* sched_meta;        /* blob from fa_scheduler_metadata, or null.  The
                                    * split-KV decode kernels take every sequence's keys
                                    * per split from it; a blob built for another batch
                                    * size, split count or for other lengths is ignored
                                    * on the device (the host's uniform plan runs).     */
    int64_t kv_entries;            /* cache calls: how many pages (paged cache) or cache
                                    * entries (dense cache) lie behind k.ptr / v.ptr, i.e. the
                                    * first dimension of the cache tensors; 0 = not known.
                                    * The tile copies (TMA) of the cache are bounded by it;
                                    * without it cache calls run on the kernels that use
                                    * plain guarded loads (slower, same results).          */
    void*   stream;                /* cudaStream_t                                     */
} fa_fwd_params;

int    fa_fwd(const fa_fwd_params* p);
int    fa_varlen_fwd(const fa_fwd_params* p);
int    fa_fwd_kvcache(const fa_fwd_params* p);
/* The same call for hosts that cannot provide scratch memory (a sealed memory pool, a plugin that
 * must not allocate inside a step).  No counterpart in the reference, which allocates its workspace
 * inside the op.  `workspace` / `workspace_bytes` are ignored; scratch comes from a 64 MiB pool built
 * into the library (fa_static_scratch_bytes()), present on every GPU that loads it.  Calls needing
 * more are refused with FA_ERR_WORKSPACE.  Allocates nothing.  The first call on a device resolves
 * the pool's address and should happen before any stream capture.  All calls share the pool:
 * calls that overlap on the GPU race; keep them ordered on one stream. */
int    fa_fwd_kvcache_static(const fa_fwd_params* p);
size_t fa_static_scratch_bytes(void);
size_t fa_fwd_workspace_bytes(const fa_fwd_params* p);
/* Number of KV splits the library will use for these parameters (>= 1). */
int    fa_fwd_num_splits(const fa_fwd_params* p);

/* ------------------------------------------------------------------------
 * Backward.   fa_bwd: mha_bwd flash_api.cpp:1279 (launch_fag_general,
 * fag_general_host.cpp:18);  fa_varlen_bwd: mha_varlen_bwd flash_api.cpp:1092;
 * v3 mha_bwd csrc/ascend910/flash_attn_npu_3/flash_api.cpp:573.
 * dq/dk/dv are written in the input dtype.  deterministic != 0 selects a fixed
 * accumulation order for dQ.  alibi_slopes (as in fa_fwd_params) adds the same
 * bias -slope * |i + sk - sq - j| to the recomputed scores; the reference's
 * backward takes the argument and ignores it, the slopes get no gradient.
 * ---------------------------------------------------------------------- */
typedef struct {
    fa_tensor dout, q, k, v, o, dq, dk, dv;
    const float* lse;
    int64_t lse_stride_b, lse_stride_h, lse_stride_s;
    const int32_t* cu_seqlens_q;
    const int32_t* cu_seqlens_k;
    int32_t b, sq, sk;             /* max lengths when packed                          */
    int32_t total_q, total_k;      /* rows of packed q / k tensors                     */
    int32_t hq, hkv, d, dv_dim;
    float   scale, softcap;
    int32_t causal, window_left, window_right;
    int32_t dtype;
    int32_t deterministic;
    void*   workspace;             /* >= fa_bwd_workspace_bytes()                      */
    size_t  workspace_bytes;
    void*   stream;
    const float* alibi_slopes;     /* (hq) or (b,hq) fp32, or null                     */
    int64_t      alibi_stride_b;   /* 0 when slopes are shared by the batch            */
} fa_bwd_params;

int    fa_bwd(const fa_bwd_params* p);
int    fa_varlen_bwd(const fa_bwd_params* p);
size_t fa_bwd_workspace_bytes(const fa_bwd_params* p);

/* ------------------------------------------------------------------------
 * LSE-weighted combine of split partials: CombineScale.hpp:76-357; v3 Python
 * flash_attn_combine (flash_attn_npu_3/flash_attn_npu_interface.py:961).
 * o_partial (nsplit, rows, dv) fp32 already normalised, lse_partial (nsplit, rows).
 * ---------------------------------------------------------------------- */
typedef struct {
    const float* o_partial;
    const float* lse_partial;
    int64_t o_split_stride, o_row_stride;    /* elements */
    int64_t lse_split_stride;
    void*   o;                               /* (rows, dv) in out_dtype, row stride o_stride */
    int64_t o_stride;
    float*  lse;                             /* (rows) or null */
    int32_t nsplit, rows, dv;
    int32_t out_dtype;                       /* fa_dtype, or 2 = fp32 */
    void*   stream;
} fa_combine_params;

int fa_combine(const fa_combine_params* p);

/* ------------------------------------------------------------------------
 * KV-sharded decode over the GPUs of one box: exchange of the partial (O, LSE)
 * fused with their combine.  No counterpart in the reference (single device;
 * the combine itself is CombineScale.hpp:76-357).  Every rank owns an exchange
 * buffer which the other ranks map through CUDA IPC; fa_fwd_kvcache /
 * fa_mla_decode with partials_only leave the rank's partials in a slot of it;
 * fa_peer_combine then signals the peers, waits (bounded) for their signals and
 * combines all ranks' partials with loads over NVLink, without a library
 * collective.  All ranks make the same sequence of calls with epoch = 1, 2, ...
 * and alternate between two slots (slot = epoch & 1).  A rank may combine only
 * a range of the rows (slot_offset / lse_offset advanced to the first row, rows
 * = the count; rows = 0 is allowed and still signals): when every rank needs
 * the result of its own sequences only, the bytes crossing NVLink drop by the
 * number of ranks.  If `status` comes back non-zero the contents of `o` are
 * undefined and the exchange must be rebuilt before its next use.
 * ---------------------------------------------------------------------- */
#define FA_MAX_PEERS 16
#define FA_PEER_HANDLE_BYTES 64
/* cudaMalloc + clear + export; `handle` is sent to the other processes */
int fa_peer_buffer_create(size_t bytes, void** ptr, unsigned char handle[FA_PEER_HANDLE_BYTES]);
/* maps another process's buffer into this one (peer access is enabled as needed) */
int fa_peer_buffer_open(const unsigned char handle[FA_PEER_HANDLE_BYTES], void** ptr);
int fa_peer_buffer_close(void* ptr);     /* of fa_peer_buffer_open   */
int fa_peer_buffer_destroy(void* ptr);   /* of fa_peer_buffer_create */

typedef struct {
    int32_t  rank, world;
    void*    peers[FA_MAX_PEERS];   /* buffer of every rank as mapped here; peers[rank] = own */
    size_t   slot_offset;           /* bytes from a buffer's start to this call's (rows, dv) fp32 partial O */
    size_t   lse_offset;            /* ... to its (rows) fp32 partial LSE                      */
    size_t   flag_offset;           /* ... to its `world` uint32 flags (zero before epoch 1)   */
    uint32_t epoch;                 /* call counter, the same on all ranks                     */
    uint32_t timeout_ms;            /* limit of the wait for the peers' signals; 0 = 1000      */
    int64_t  rows;
    int32_t  dv;                    /* multiple of 4                                           */
    int32_t  out_dtype;             /* fa_dtype, or 2 = fp32                                   */
    void*    o;                     /* (rows, dv) in out_dtype, row stride o_stride            */
    int64_t  o_stride;
    float*   lse;                   /* (rows) or null                                          */
    int32_t* status;                /* device int, stays 0 on success; 1 + r if rank r's signal
                                     * did not arrive in time (o is then undefined: blocks that
                                     * saw the signal in time may have written their rows)     */
    void*    stream;
} fa_peer_combine_params;

int fa_peer_combine(const fa_peer_combine_params* p);

/* Pitched copy on a stream (cudaMemcpy2DAsync, direction from the pointers): moves a group of heads of a
 * (batch, seqlen, heads, headdim) tensor between pinned host memory and the device without a staging copy.
 * No counterpart in the reference (its operands are created on the device). */
int fa_copy_2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                     size_t rows, void* stream);

/* ------------------------------------------------------------------------
 * int8 latent (MLA) paged decode.  No counterpart in the reference (it has no
 * quantised path).  K_j = [scale_j * latent_j (512) | rope_j (64)], V_j = the
 * dequantised latent; one shared KV head, seqlen_q = 1.
 * ---------------------------------------------------------------------- */
typedef struct {
    const void*   q_nope;       /* (b, hq, 512) bf16, row stride q_nope_stride_b / _h */
    const void*   q_rope;       /* (b, hq, 64) bf16                                   */
    int64_t q_nope_stride_b, q_nope_stride_h, q_rope_stride_b, q_rope_stride_h;
    const int8_t* latent;       /* (blocks, page, 512) int8, contiguous               */
    const float*  scales;       /* (blocks, page) fp32                                */
    const void*   rope;         /* (blocks, page, 64) bf16                            */
    const int32_t* block_table; int64_t block_table_stride; int32_t page_size;
    const int32_t* cache_seqlens;
    void*   o;                  /* (b, hq, 512) bf16; o_stride_b / _h                 */
    int64_t o_stride_b, o_stride_h;
    float*  lse;                /* (b, hq) fp32 or null                               */
    int32_t b, hq;
    float   scale;
    int32_t num_splits;         /* 0 = heuristic                                      */
    int32_t kv_begin, kv_end, partials_only;
    float*  o_partial;          /* (splits, b*hq, 512) fp32                           */
    float*  lse_partial;        /* (splits, b*hq) fp32                                */
    void*   workspace; size_t workspace_bytes;
    void*   stream;
} fa_mla_params;

int    fa_mla_decode(const fa_mla_params* p);
size_t fa_mla_workspace_bytes(const fa_mla_params* p);
int    fa_mla_num_splits(const fa_mla_params* p);

/* ------------------------------------------------------------------------
 * Device-side schedule for the kvcache forward: get_scheduler_metadata
 * csrc/ascend910/flash_attn_npu_3/flash_api.cpp:506-571 (ComputeFAMetadata,
 * fa_metadata.aicpu:32-151); the forward that takes its tiling from the blob
 * instead of planning on the host is flash_api.cpp:248-267 there.  Fills `meta`
 * (int32, fa_scheduler_metadata_ints(b) = 8 + 8 b entries) on the stream from
 * the device-resident lengths, without a host sync:
 *   [0] magic  [1] b  [2] split count of the launch grid  [3] 64-key blocks per
 *   split of the host plan  [4] longest sequence  [5] total blocks  [6] active
 *   (sequence, split) pairs  [7] 0; then per sequence: length, blocks, active
 *   splits, keys per active split (the sequence's keys spread evenly), prefix of
 *   active splits, 0, 0, 0.
 * `sk` must be the capacity the forward call will pass (page-table width x page
 * size, or the rows of a dense cache), since the grid is planned from it.
 * ---------------------------------------------------------------------- */
typedef struct {
    const int32_t* seqused_k;   /* (b) */
    const int32_t* cu_seqlens_q;/* (b+1) or null */
    int32_t b, sq, sk, hq, hkv, d, dv, page_size, s_new, causal, window_left, window_right;
    int32_t num_splits;
    int32_t* meta;
    void*   stream;
} fa_sched_params;

int    fa_scheduler_metadata(const fa_sched_params* p);
size_t fa_scheduler_metadata_ints(int32_t b);

/* host-only helpers */
const char* fa_last_error(void);
const char* fa_version(void);
/* Name of the kernel family the last forward / backward call on this thread used
 * ("sm100_tcgen05", "generic_mma", "decode_splitkv", ...); for tests and benchmarks. */
const char* fa_last_kernel(void);
/* Force the kernel family, process-wide: 0 = automatic, 1 = generic tensor-core kernels only. */
void        fa_set_kernel_policy(int policy);

/* Process-wide switches for tests and benchmarks (plain atomics: flipping one while another thread is inside a
 * call changes which kernel that call's NEXT launch takes, never its results).  Debug keys: 2 = error code left by a
 * timed-out wait in a tcgen05 / TMA kernel (get; synchronises the device), 3 = clear that code (set), 4 = 0 makes
 * the decode kernel load cache tiles with 16-byte cp.async copies instead of TMA (set), 7 = 0 makes the tcgen05
 * backward recompute S and dP in its dQ kernel instead of reading the dS tiles the dK/dV kernel leaves in the
 * workspace (set). */
void        fa_debug_set(int key, int value);
int         fa_debug_get(int key);

/* Per-kernel timing for benchmarks: lend `count` cudaEvent_t handles (created with timing
 * enabled) to the calling thread.  The next forward / backward call records events[0] before
 * its first launch and one more event after every kernel it launches, on the call's stream;
 * fa_kernel_events_used() tells how many were recorded.  Pass (NULL, 0) to stop. */
void        fa_set_kernel_events(void** events, int count);
int         fa_kernel_events_used(void);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H */
