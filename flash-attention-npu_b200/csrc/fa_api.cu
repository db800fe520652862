// C-ABI entry points of libfa_b200.so: argument validation, launch planning, dispatch.
// Nothing here allocates, synchronises or reads device memory.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include "fa_internal.h"

namespace fa {

static thread_local char g_err[512] = "";
static thread_local const char* g_kernel = "";
static std::atomic<int> g_policy{0};          // process-wide test switch (fa_set_kernel_policy)
// optional per-kernel timing: the caller lends CUDA events, one is recorded after every launch
static thread_local cudaEvent_t* g_events = nullptr;
static thread_local int g_nevents = 0, g_event_idx = 0;

bool kernel_events_active() { return g_events != nullptr; }
void mark_kernel(cudaStream_t st) {
    if (g_events && g_event_idx < g_nevents) cudaEventRecord(g_events[g_event_idx++], st);
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
void note_kernel(const char* name) { g_kernel = name; }
int cuda_ok(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return FA_OK;
    return fail(FA_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

int sm_count() {
    static int cached[16] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev < 16 && cached[dev]) return cached[dev];
    int n = 148;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (dev < 16) cached[dev] = n;
    return n;
}

static inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int check_tensor(const char* name, const fa_tensor& t, bool need) {
    if (!t.ptr) return need ? fail(FA_ERR_NULL, "%s is null", name) : FA_OK;
    if (!aligned16(t.ptr)) return fail(FA_ERR_MISALIGNED, "%s must be 16-byte aligned", name);
    if ((t.stride_b % 8) || (t.stride_s % 8) || (t.stride_h % 8))
        return fail(FA_ERR_MISALIGNED, "%s strides must be multiples of 8 elements (16 bytes)", name);
    return FA_OK;
}

static int check_common(const fa_fwd_params& p) {
    if (p.dtype != FA_F16 && p.dtype != FA_BF16) return fail(FA_ERR_BAD_DTYPE, "only fp16 and bf16 are supported");
    if (p.b < 0 || p.sq < 0 || p.sk < 0 || p.hq <= 0 || p.hkv <= 0) return fail(FA_ERR_BAD_SHAPE, "negative or zero size");
    if (p.hq % p.hkv) return fail(FA_ERR_BAD_SHAPE, "number of heads in q must be divisible by the number of heads in k/v");
    if (p.d <= 0 || p.d > 256 || p.dv <= 0 || p.dv > 256) return fail(FA_ERR_BAD_SHAPE, "head dimension must be in [1, 256]");
    if ((p.d % 8) || (p.dv % 8)) return fail(FA_ERR_BAD_SHAPE, "head dimension must be a multiple of 8 (pad it)");
    if (int e = check_tensor("q", p.q, true)) return e;
    if (int e = check_tensor("k", p.k, true)) return e;
    if (int e = check_tensor("v", p.v, true)) return e;
    if (!p.partials_only) { if (int e = check_tensor("out", p.o, true)) return e; }
    if (p.partials_only && (!p.o_partial || !p.lse_partial)) return fail(FA_ERR_NULL, "partials_only needs o_partial and lse_partial");
    return FA_OK;
}

void plan_forward(const fa_fwd_params& p, FwdPlan& plan) {
    memset(&plan, 0, sizeof(plan));
    const int G = p.hq / p.hkv;
    const bool cache_like = p.seqused_k || p.block_table;
    plan.pack_gqa = (G > 1 && p.sq <= 32) ? 1 : 0;
    const int rows = plan.pack_gqa ? p.sq * G : p.sq;
    const int mblocks = (rows + kGenericBM - 1) / kGenericBM;
    const int nblocks = (p.sk + kGenericBN - 1) / kGenericBN;
    int nsplit = 1;
    plan.use_decode = fwd_decode_supported(p) ? 1 : 0;
    // A cache call that the tcgen05 forward takes is split over the keys (two-tile kernel, head dim <= 128) until
    // about two waves of CTAs exist, with at least 512 keys a split for short chunks and 2048 for prefill chunks of
    // 64 or more rows a head; the split is by the cache capacity (the lengths are not known here), so one long sequence
    // among short ones does not set the call's time either.
    plan.use_sm100 = (g_policy == 0 && cache_like && !p.partials_only && fwd_sm100_supported(p) && (p.d <= 128 || p.num_splits <= 1)) ? 1 : 0;
    if (p.num_splits > 1) nsplit = p.num_splits;
    else if (plan.use_sm100 && (p.num_splits == 1 || p.d > 128)) nsplit = 1;
    else if (plan.use_sm100) {
        const long ctas = fwd_sm100_ctas(p);
        long n = (2L * sm_count() + ctas - 1) / ctas;
        const int min_keys = p.sq >= 64 ? 2048 : 512;
        const long cap = (p.sk + min_keys - 1) / min_keys;
        if (n > cap) n = cap;
        nsplit = (int)(n < 1 ? 1 : n);
    } else if (p.num_splits == 0 && plan.use_decode && nblocks > 1) {
        // decode kernel: the unit of parallelism is a warp per (sequence, KV head, split); aim at about
        // 1024 keys per split, at least four waves of warps, and never fewer than 256 keys per split
        // (with 17-64 stacked rows a whole CTA streams one KV head: four waves of CTAs)
        const long base = (long)p.hkv * (p.b > 0 ? p.b : 1);
        const long target = (p.sq * G > 16 ? 4L : 16L) * sm_count();
        const long by_occ = (target + base - 1) / base;
        const long by_bal = (p.sk + 1023) / 1024;
        const long cap = (p.sk + 255) / 256;
        long n = by_occ > by_bal ? by_occ : by_bal;
        if (n > cap) n = cap;
        nsplit = (int)(n < 1 ? 1 : n);
    } else if (p.num_splits == 0 && cache_like && nblocks > 1 && p.sq <= 64) {
        const long base = (long)mblocks * (plan.pack_gqa ? p.hkv : p.hq) * (p.b > 0 ? p.b : 1);
        const long target = 4L * sm_count();
        long by_occ = base >= target ? 1 : (target + base - 1) / base;
        long by_bal = nblocks >= 64 ? (nblocks + 31) / 32 : 1;
        nsplit = (int)(by_occ > by_bal ? by_occ : by_bal);
    }
    if (nsplit > nblocks) nsplit = nblocks;
    if (nsplit > 256) nsplit = 256;
    if (nsplit < 1) nsplit = 1;
    plan.blocks_per_split = nblocks > 0 ? (nblocks + nsplit - 1) / nsplit : 1;
    if (plan.use_sm100) plan.blocks_per_split += plan.blocks_per_split & 1;      // whole 128-key tiles a split
    plan.nsplit = nblocks > 0 ? (nblocks + plan.blocks_per_split - 1) / plan.blocks_per_split : 1;
    plan.rotate_q = (p.rotary_cos && p.rotary_sin) ? 1 : 0;
    const size_t rows_all = (size_t)(p.cu_seqlens_q ? p.total_q : (int64_t)p.b * p.sq) * p.hq;
    plan.q_rot_bytes = plan.rotate_q ? align256((size_t)p.b * p.sq * p.hq * p.d * 2) : 0;
    if (plan.nsplit > 1) {
        plan.o_part_bytes = align256((size_t)plan.nsplit * rows_all * p.dv * sizeof(float));
        plan.lse_part_bytes = align256((size_t)plan.nsplit * rows_all * sizeof(float));
    }
}

// Window normalisation of the reference's forward host code (flash_api.cpp:684-704, :936-956, :483-505), `sk` being
// the (longest) key length the host knows: a side that reaches sk is unbounded; under a sliding window an unbounded
// RIGHT side then becomes sk keys past the diagonal, which for seqlen_q > seqlen_k + 1 is a real bound (rows whose
// diagonal lies more than sk keys before the first key see nothing).  The reference does the same to the left
// side, where it never changes the mask.
static void normalize_windows_like_forward(int sk, int causal, int32_t& wl, int32_t& wr) {
    if (sk <= 0) return;
    if (wl >= sk) wl = -1;
    if (wr >= sk) wr = -1;
    if (causal) return;                                   // the kernels force window_right = 0
    const bool is_causal = wl < 0 && wr == 0;
    const bool is_local = (wl >= 0 || wr >= 0) && !is_causal;
    if (is_local && wr < 0) wr = sk;
}

static int run_forward(const fa_fwd_params& pin, bool allow_fast) {
    fa_fwd_params p = pin;
    if (p.b == 0 || p.hq == 0) return FA_OK;
    if ((p.cu_seqlens_q ? p.total_q : p.sq) == 0) return FA_OK;
    normalize_windows_like_forward(p.sk, p.causal, p.window_left, p.window_right);
    FwdPlan plan;
    plan_forward(p, plan);
    mark_kernel(reinterpret_cast<cudaStream_t>(p.stream));
    const size_t need = plan.q_rot_bytes + plan.o_part_bytes + plan.lse_part_bytes;
    if (need > 0 && (!p.workspace || p.workspace_bytes < need))
        return fail(FA_ERR_WORKSPACE, "workspace of %zu bytes required, %zu given", need, p.workspace_bytes);
    char* ws = reinterpret_cast<char*>(p.workspace);
    void* q_rot = plan.rotate_q ? ws : nullptr;
    float* o_part = plan.nsplit > 1 ? reinterpret_cast<float*>(ws + plan.q_rot_bytes) : nullptr;
    float* lse_part = plan.nsplit > 1 ? reinterpret_cast<float*>(ws + plan.q_rot_bytes + plan.o_part_bytes) : nullptr;

    // in-place append (and rotary) first; the attention kernels then see the updated cache
    if (p.s_new > 0 || plan.rotate_q) {
        const int by_pos = (p.causal || p.window_left >= 0 || p.window_right >= 0) ? 1 : 0;
        if (int e = launch_append_rotary(p, q_rot, by_pos)) return e;
        if (plan.rotate_q) {
            p.q.ptr = q_rot;
            p.q.stride_h = p.d;
            p.q.stride_s = (int64_t)p.hq * p.d;
            p.q.stride_b = (int64_t)p.sq * p.hq * p.d;
        }
    }
    const bool cache_call = p.seqused_k || p.block_table;
    if (allow_fast && g_policy == 0 && !p.partials_only && fwd_sm100_supported(p) &&
        (plan.nsplit == 1 || (cache_call && plan.use_sm100 && p.d <= 128))) {
        if (int e = launch_fwd_sm100(p, plan.nsplit, plan.blocks_per_split * kGenericBN, o_part, lse_part)) return e;
        return plan.nsplit > 1 ? launch_fwd_combine(p, plan.nsplit, o_part, lse_part, 0) : FA_OK;
    }

    if (p.partials_only && plan.nsplit == 1) { o_part = p.o_partial; lse_part = p.lse_partial; }
    int e = (g_policy == 0 && plan.use_decode) ? launch_fwd_decode(p, plan, o_part, lse_part)
                                                : launch_fwd_generic(p, plan, o_part, lse_part);
    if (e) return e;
    if (plan.nsplit > 1) return launch_fwd_combine(p, plan.nsplit, o_part, lse_part, p.partials_only);
    return FA_OK;
}

}  // namespace fa

using namespace fa;

extern "C" {

int fa_fwd(const fa_fwd_params* p) {
    if (!p) return fail(FA_ERR_NULL, "params is null");
    if (int e = check_common(*p)) return e;
    if (p->cu_seqlens_q || p->cu_seqlens_k || p->block_table || p->seqused_k)
        return fail(FA_ERR_UNSUPPORTED, "fa_fwd takes dense tensors; use fa_varlen_fwd / fa_fwd_kvcache");
    fa_fwd_params q = *p;
    q.num_splits = 1; q.s_new = 0; q.rotary_cos = q.rotary_sin = nullptr; q.kv_begin = 0; q.kv_end = 0; q.partials_only = 0;
    return run_forward(q, true);
}

int fa_varlen_fwd(const fa_fwd_params* p) {
    if (!p) return fail(FA_ERR_NULL, "params is null");
    if (int e = check_common(*p)) return e;
    if (!p->cu_seqlens_q) return fail(FA_ERR_NULL, "cu_seqlens_q is null");
    if (!p->cu_seqlens_k && !p->block_table) return fail(FA_ERR_NULL, "cu_seqlens_k is null");
    if (p->block_table && !p->seqused_k && !p->cu_seqlens_k) return fail(FA_ERR_NULL, "paged varlen needs seqused_k or cu_seqlens_k");
    fa_fwd_params q = *p;
    q.s_new = 0; q.rotary_cos = q.rotary_sin = nullptr;
    if (!q.block_table) q.num_splits = 1;
    return run_forward(q, true);
}

int fa_fwd_kvcache(const fa_fwd_params* p) {
    if (!p) return fail(FA_ERR_NULL, "params is null");
    if (int e = check_common(*p)) return e;
    if (p->block_table && p->page_size <= 0) return fail(FA_ERR_BAD_SHAPE, "page_size must be positive");
    if (p->block_table && p->cache_batch_idx) return fail(FA_ERR_UNSUPPORTED, "cache_batch_idx is not used with a paged cache");
    if (p->s_new > 0) {
        if (!p->seqused_k) return fail(FA_ERR_NULL, "appending k/v needs cache_seqlens");
        if (int e = check_tensor("k_new", p->k_new, true)) return e;
        if (int e = check_tensor("v_new", p->v_new, true)) return e;
    }
    if ((p->rotary_cos != nullptr) != (p->rotary_sin != nullptr)) return fail(FA_ERR_NULL, "rotary_cos and rotary_sin go together");
    if (p->rotary_cos) {
        if (!p->seqused_k) return fail(FA_ERR_NULL, "rotary needs cache_seqlens");
        if (p->cu_seqlens_q) return fail(FA_ERR_UNSUPPORTED, "rotary with packed q is not supported");
        if (p->rotary_dim <= 0 || p->rotary_dim > p->d || (p->rotary_dim % 2)) return fail(FA_ERR_BAD_SHAPE, "rotary_dim must be even and <= headdim");
        if (p->seqlen_ro <= 0) return fail(FA_ERR_BAD_SHAPE, "seqlen_ro must be positive");
    }
    return run_forward(*p, true);
}

size_t fa_fwd_workspace_bytes(const fa_fwd_params* p) {
    if (!p || p->hkv <= 0 || p->hq <= 0) return 0;
    FwdPlan plan;
    plan_forward(*p, plan);
    return plan.q_rot_bytes + plan.o_part_bytes + plan.lse_part_bytes;
}

int fa_fwd_num_splits(const fa_fwd_params* p) {
    if (!p || p->hkv <= 0 || p->hq <= 0) return 1;
    FwdPlan plan;
    plan_forward(*p, plan);
    return plan.nsplit;
}

static int check_bwd(const fa_bwd_params& p) {
    if (p.dtype != FA_F16 && p.dtype != FA_BF16) return fail(FA_ERR_BAD_DTYPE, "only fp16 and bf16 are supported");
    if (p.b < 0 || p.sq < 0 || p.sk < 0 || p.hq <= 0 || p.hkv <= 0) return fail(FA_ERR_BAD_SHAPE, "negative or zero size");
    if (p.hq % p.hkv) return fail(FA_ERR_BAD_SHAPE, "number of heads in q must be divisible by the number of heads in k/v");
    if (p.d <= 0 || p.d > 256 || p.dv_dim <= 0 || p.dv_dim > 256 || (p.d % 8) || (p.dv_dim % 8))
        return fail(FA_ERR_BAD_SHAPE, "head dimension must be a multiple of 8 in [8, 256]");
    const char* names[8] = {"dout", "q", "k", "v", "out", "dq", "dk", "dv"};
    const fa_tensor* ts[8] = {&p.dout, &p.q, &p.k, &p.v, &p.o, &p.dq, &p.dk, &p.dv};
    for (int i = 0; i < 8; ++i) if (int e = check_tensor(names[i], *ts[i], true)) return e;
    if (!p.lse) return fail(FA_ERR_NULL, "softmax_lse is null");
    return FA_OK;
}

static int run_backward(const fa_bwd_params& pin) {
    fa_bwd_params p = pin;
    if (p.b == 0) return FA_OK;
    // The forward's rule first, because for seqlen_q > seqlen_k it changes the mask and the saved LSE was computed
    // under that mask; then the rule of
    // the reference's backward host code (fag_general_host.cpp:81-92, flash_api.cpp:1155-1162), which never
    // changes the mask.
    normalize_windows_like_forward(p.sk, p.causal, p.window_left, p.window_right);
    if (p.window_left >= p.sk - 1) p.window_left = -1;
    if (p.window_right >= p.sq - 1) p.window_right = -1;
    mark_kernel(reinterpret_cast<cudaStream_t>(p.stream));
    const bool fast = g_policy == 0 && bwd_sm100_supported(p);
    const size_t need = fast ? bwd_sm100_workspace(p) : bwd_generic_workspace(p);
    if (!p.workspace || p.workspace_bytes < need)
        return fail(FA_ERR_WORKSPACE, "workspace of %zu bytes required, %zu given", need, p.workspace_bytes);
    return fast ? launch_bwd_sm100(p) : launch_bwd_generic(p);
}

int fa_bwd(const fa_bwd_params* p) {
    if (!p) return fail(FA_ERR_NULL, "params is null");
    if (int e = check_bwd(*p)) return e;
    if (p->cu_seqlens_q || p->cu_seqlens_k) return fail(FA_ERR_UNSUPPORTED, "fa_bwd takes dense tensors; use fa_varlen_bwd");
    return run_backward(*p);
}

int fa_varlen_bwd(const fa_bwd_params* p) {
    if (!p) return fail(FA_ERR_NULL, "params is null");
    if (int e = check_bwd(*p)) return e;
    if (!p->cu_seqlens_q || !p->cu_seqlens_k) return fail(FA_ERR_NULL, "cu_seqlens_q / cu_seqlens_k is null");
    return run_backward(*p);
}

size_t fa_bwd_workspace_bytes(const fa_bwd_params* p) {
    if (!p || p->hq <= 0) return 0;
    const size_t a = bwd_generic_workspace(*p), b = bwd_sm100_workspace(*p);
    return a > b ? a : b;
}

int fa_combine(const fa_combine_params* c) {
    if (!c) return fail(FA_ERR_NULL, "params is null");
    if (!c->o_partial || !c->lse_partial || !c->o) return fail(FA_ERR_NULL, "null pointer");
    if (c->nsplit <= 0 || c->rows < 0 || c->dv <= 0) return fail(FA_ERR_BAD_SHAPE, "bad sizes");
    if (c->out_dtype < 0 || c->out_dtype > 2) return fail(FA_ERR_BAD_DTYPE, "out_dtype must be f16, bf16 or fp32");
    return fa::combine_flat(*c);
}

int fa_peer_combine(const fa_peer_combine_params* c) {
    if (!c) return fail(FA_ERR_NULL, "params is null");
    if (c->out_dtype < 0 || c->out_dtype > 2) return fail(FA_ERR_BAD_DTYPE, "out_dtype must be f16, bf16 or fp32");
    return fa::peer_combine(*c);
}
int fa_peer_buffer_create(size_t bytes, void** ptr, unsigned char* handle) { return fa::peer_buffer_create(bytes, ptr, handle); }
int fa_peer_buffer_open(const unsigned char* handle, void** ptr) { return fa::peer_buffer_open(handle, ptr); }
int fa_peer_buffer_close(void* ptr) { return ptr ? fa::cuda_ok(cudaIpcCloseMemHandle(ptr), "peer buffer close") : FA_OK; }
int fa_peer_buffer_destroy(void* ptr) { return ptr ? fa::cuda_ok(cudaFree(ptr), "peer buffer free") : FA_OK; }

int fa_copy_2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows,
                     void* stream) {
    if (!dst || !src) return fail(FA_ERR_NULL, "null pointer");
    if (width_bytes == 0 || rows == 0) return FA_OK;
    if (width_bytes > dst_pitch || width_bytes > src_pitch) return fail(FA_ERR_BAD_SHAPE, "row wider than its pitch");
    return fa::cuda_ok(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDefault,
                                         reinterpret_cast<cudaStream_t>(stream)), "pitched copy");
}

const char* fa_last_error(void) { return g_err; }
const char* fa_version(void) { return "fa_b200 0.1.0 (sm_100a)"; }
const char* fa_last_kernel(void) { return g_kernel; }
void fa_debug_set(int key, int value) {
    if (key == 3) { fa::sm100_error_flag(true); fa::decode_error_flag(true); }
    if (key == 4) fa::decode_set_use_tma(value);
    if (key == 7) fa::bwd_sm100_set_ds_spill(value);
}
int fa_debug_get(int key) {
    if (key != 2) return 0;
    const int a = fa::sm100_error_flag(false);
    return a ? a : fa::decode_error_flag(false);
}
void fa_set_kernel_events(void** events, int count) {
    g_events = reinterpret_cast<cudaEvent_t*>(events);
    g_nevents = events ? count : 0;
    g_event_idx = 0;
}
int fa_kernel_events_used(void) { return g_event_idx; }
void fa_set_kernel_policy(int policy) { g_policy = policy; }
}  // extern "C"
namespace fa { int kernel_policy() { return g_policy; } }
extern "C" {

}  // extern "C"
