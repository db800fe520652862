// fa_fwd_kvcache_static: the KV-cache forward for callers that cannot hand over scratch memory.
//
// Some hosts of this library may not allocate device memory at the moment they call attention:
// a serving loop whose memory pool is sealed once the model is loaded, a plugin running inside
// another runtime's step function where cudaMalloc would synchronise the device or is simply
// forbidden, a real-time path that must not touch the allocator.  fa_fwd_kvcache needs scratch for
// its split-KV partial results (and for the rotated queries when rotary tables are given) and
// expects the caller to provide it.  This variant brings its own: a fixed pool that lives in the
// library image on every GPU that loads it, for as long as the process lives.
//
// Limits and rules
//   * The pool holds kStaticScratchBytes (64 MiB).  A call whose scratch need
//     (fa_fwd_workspace_bytes) is larger is refused with FA_ERR_WORKSPACE and a message that names
//     both numbers; nothing is launched.
//   * The first call on each device looks up the pool's device address (cudaGetSymbolAddress, with
//     that device current) and remembers it.  Make that first call outside any stream capture.
//   * No call here allocates or frees: no cudaMalloc / cudaFree, no allocating library routine.
//   * All calls on a device share the one pool, and it keeps whatever the previous call left in it.
//     Nothing in it has to start at zero: every partial-result slot and every rotated query row a
//     call reads is written by that same call first.  Two calls that overlap on the GPU (different
//     streams, or graphs replayed concurrently) would race on the pool: keep them on one stream or
//     otherwise ordered.
#include <cuda_runtime.h>
#include "fa_internal.h"

namespace {

constexpr size_t kStaticScratchBytes = 64u << 20;
constexpr int kMaxDevices = 64;

// The pool itself.  In host code this name is only a handle for the symbol, never a device
// address: the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

void* g_pool_addr[kMaxDevices] = {};

int pool_for_current_device(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return fa::fail(FA_ERR_CUDA, "fa_fwd_kvcache_static: cannot identify the current device");
    if (!g_pool_addr[dev]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr)
            return fa::fail(FA_ERR_CUDA, "fa_fwd_kvcache_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_pool_addr[dev] = ptr;
    }
    *out = g_pool_addr[dev];
    return FA_OK;
}

}  // namespace

extern "C" {

size_t fa_static_scratch_bytes(void) { return kStaticScratchBytes; }

int fa_fwd_kvcache_static(const fa_fwd_params* p) {
    if (!p) return fa::fail(FA_ERR_NULL, "params is null");
    const size_t need = fa_fwd_workspace_bytes(p);
    if (need > kStaticScratchBytes)
        return fa::fail(FA_ERR_WORKSPACE,
                        "fa_fwd_kvcache_static: this call needs %zu bytes of scratch but the built-in pool holds %zu; "
                        "lower num_splits or the batch, or use fa_fwd_kvcache with your own workspace",
                        need, kStaticScratchBytes);
    fa_fwd_params q = *p;
    q.workspace = nullptr;
    q.workspace_bytes = 0;
    if (need > 0) {
        void* pool = nullptr;
        if (int e = pool_for_current_device(&pool)) return e;
        q.workspace = pool;
        q.workspace_bytes = kStaticScratchBytes;
    }
    return fa_fwd_kvcache(&q);
}

}  // extern "C"
