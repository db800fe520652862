// KV-sharded decode across the GPUs of one box: exchange of the fp32 partial (O, LSE) fused with their combine.
//
// Every rank owns one exchange buffer that all other ranks have mapped through CUDA IPC.  The decode kernels of a call
// leave this rank's partials in a slot of its own buffer; one kernel per rank then
//   1. tells every peer "my partials of call `epoch` are in place" with one 4-byte store into the peer's flag array,
//   2. waits, with a time limit, until the flags of all peers have arrived in its own buffer,
//   3. reads every rank's partials with loads over NVLink and writes the LSE-weighted sum.
// No library collective and no staging copy: the gathered partials never exist in local memory.  Two slots are used in
// turn; a rank can only reach call n+2 after every peer has signalled call n+1, which a peer does after its combine
// of call n has finished, so a slot is never overwritten while a peer still reads it.
//
// The reference has no multi-device decode; the combine follows CombineScale.hpp:76-357 like combine_kernel.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <string.h>
#include "fa_internal.h"

namespace fa {
namespace {

constexpr int kPeerWarps = 4;

struct PeerArgs {
    const float* o_part[FA_MAX_PEERS];      // slot of every rank: (rows, dv) fp32
    const float* lse_part[FA_MAX_PEERS];    // (rows) fp32
    unsigned*    flags[FA_MAX_PEERS];       // flag array (world entries) of this slot in every rank's buffer
    int rank, world;
    unsigned epoch;
    int64_t rows;
    int dv;
    int64_t o_stride;
    void* o;
    float* lse;
    int* status;
    unsigned long long timeout_ns;
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// partials of a peer are read around the L1 (the slot is reused two calls later)
__device__ __forceinline__ float4 ld_peer_v4(const float* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ld_peer_f32(const float* p) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

template <typename OutT> __device__ __forceinline__ void put(OutT* d, float v);
template <> __device__ __forceinline__ void put<float>(float* d, float v) { *d = v; }
template <> __device__ __forceinline__ void put<__half>(__half* d, float v) { *d = __float2half_rn(v); }
template <> __device__ __forceinline__ void put<__nv_bfloat16>(__nv_bfloat16* d, float v) { *d = __float2bfloat16_rn(v); }

template <typename OutT>
__global__ void __launch_bounds__(kPeerWarps * 32) peer_combine_kernel(const PeerArgs a) {
    __shared__ int s_fail;
    __shared__ float s_w[kPeerWarps][FA_MAX_PEERS];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) s_fail = 0;
    // 1. signal: the partials were written by earlier kernels of this stream, so they are complete; the first block
    //    publishes that to every rank (its own flag included, so that the wait below has one form).
    if (blockIdx.x == 0 && threadIdx.x < a.world) {
        __threadfence_system();
        st_release_sys(a.flags[threadIdx.x] + a.rank, a.epoch);
    }
    __syncthreads();
    // 2. wait for every rank's flag in the local buffer, with a time limit
    if (threadIdx.x < a.world) {
        const unsigned* f = a.flags[a.rank] + threadIdx.x;
        const unsigned long long t0 = global_ns();
        bool ok = false;
        while (true) {
            if ((int)(ld_acquire_sys(f) - a.epoch) >= 0) { ok = true; break; }
            if (global_ns() - t0 > a.timeout_ns) break;
            __nanosleep(64);
        }
        if (!ok) {
            atomicExch(a.status, 1 + (int)threadIdx.x);       // 1 + the rank whose signal did not arrive
            s_fail = 1;
        }
    }
    __syncthreads();
    if (s_fail) return;
    // 3. combine, one warp per row
    const int64_t row = (int64_t)blockIdx.x * kPeerWarps + wid;
    if (row >= a.rows) return;
    float ls = lane < a.world ? ld_peer_f32(a.lse_part[lane] + row) : -INFINITY;
    float m = ls;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    const float ms = m == -INFINITY ? 0.f : m;
    float tot = lane < a.world ? expf(ls - ms) : 0.f;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, d);
    const float l = tot > 0.f ? ms + logf(tot) : -INFINITY;
    if (lane < FA_MAX_PEERS) s_w[wid][lane] = (lane < a.world && ls != -INFINITY) ? expf(ls - l) : 0.f;   // no key seen: weight 0
    __syncwarp();
    OutT* orow = reinterpret_cast<OutT*>(a.o) + row * a.o_stride;
    for (int c = lane * 4; c < a.dv; c += 128) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r0 = 0; r0 < a.world; r0 += 4) {
            float4 v[4];
            float w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int r = r0 + u;
                w[u] = r < a.world ? s_w[wid][r] : 0.f;
                v[u] = w[u] != 0.f ? ld_peer_v4(a.o_part[r] + row * a.dv + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                acc.x += w[u] * v[u].x; acc.y += w[u] * v[u].y; acc.z += w[u] * v[u].z; acc.w += w[u] * v[u].w;
            }
        }
        put<OutT>(orow + c, acc.x);
        put<OutT>(orow + c + 1, acc.y);
        put<OutT>(orow + c + 2, acc.z);
        put<OutT>(orow + c + 3, acc.w);
    }
    if (a.lse != nullptr && lane == 0) a.lse[row] = l;
}

}  // namespace

int peer_combine(const fa_peer_combine_params& c) {
    cudaStream_t st = reinterpret_cast<cudaStream_t>(c.stream);
    if (c.world < 1 || c.world > FA_MAX_PEERS || c.rank < 0 || c.rank >= c.world)
        return fail(FA_ERR_BAD_SHAPE, "peer combine: rank %d of %d (at most %d ranks)", c.rank, c.world, FA_MAX_PEERS);
    if (c.dv <= 0 || c.dv % 4 != 0) return fail(FA_ERR_BAD_SHAPE, "peer combine: dv must be a multiple of 4");
    if (c.rows < 0 || c.status == nullptr || (c.o == nullptr && c.rows > 0)) return fail(FA_ERR_BAD_SHAPE, "peer combine: null argument");
    if (c.slot_offset % 16 != 0 || c.lse_offset % 16 != 0 || c.flag_offset % 16 != 0)
        return fail(FA_ERR_BAD_SHAPE, "peer combine: offsets must be multiples of 16 bytes");
    // a rank without rows of its own still signals and waits: the other ranks count on its flag
    PeerArgs a{};
    for (int r = 0; r < c.world; ++r) {
        if (c.peers[r] == nullptr) return fail(FA_ERR_BAD_SHAPE, "peer combine: buffer of rank %d is not mapped", r);
        char* base = reinterpret_cast<char*>(c.peers[r]);
        a.o_part[r] = reinterpret_cast<const float*>(base + c.slot_offset);
        a.lse_part[r] = reinterpret_cast<const float*>(base + c.lse_offset);
        a.flags[r] = reinterpret_cast<unsigned*>(base + c.flag_offset);
    }
    a.rank = c.rank; a.world = c.world; a.epoch = c.epoch; a.rows = c.rows; a.dv = c.dv;
    a.o_stride = c.o_stride; a.o = c.o; a.lse = c.lse; a.status = c.status;
    a.timeout_ns = (unsigned long long)(c.timeout_ms ? c.timeout_ms : 1000u) * 1000000ull;
    dim3 grid((unsigned)((c.rows + kPeerWarps - 1) / kPeerWarps > 0 ? (c.rows + kPeerWarps - 1) / kPeerWarps : 1));
    if (c.out_dtype == FA_F16) peer_combine_kernel<__half><<<grid, kPeerWarps * 32, 0, st>>>(a);
    else if (c.out_dtype == FA_BF16) peer_combine_kernel<__nv_bfloat16><<<grid, kPeerWarps * 32, 0, st>>>(a);
    else peer_combine_kernel<float><<<grid, kPeerWarps * 32, 0, st>>>(a);
    note_kernel("peer_combine");
    mark_kernel(st);
    return cuda_ok(cudaGetLastError(), "peer combine launch");
}

int peer_buffer_create(size_t bytes, void** ptr, unsigned char* handle) {
    if (ptr == nullptr || handle == nullptr || bytes == 0) return fail(FA_ERR_BAD_SHAPE, "peer buffer: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == FA_PEER_HANDLE_BYTES, "handle size");
    void* p = nullptr;
    int rc = cuda_ok(cudaMalloc(&p, bytes), "peer buffer allocation");
    if (rc != FA_OK) return rc;
    rc = cuda_ok(cudaMemset(p, 0, bytes), "peer buffer clear");
    cudaIpcMemHandle_t h;
    if (rc == FA_OK) rc = cuda_ok(cudaIpcGetMemHandle(&h, p), "peer buffer export");
    if (rc != FA_OK) { cudaFree(p); return rc; }
    memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return FA_OK;
}

int peer_buffer_open(const unsigned char* handle, void** ptr) {
    if (ptr == nullptr || handle == nullptr) return fail(FA_ERR_BAD_SHAPE, "peer buffer: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    return cuda_ok(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess), "peer buffer open");
}

}  // namespace fa
