// Host-side internals shared by the translation units of libfa_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include "../../include/fa_b200.h"

namespace fa {

// error reporting (thread-local message, see fa_api.cu)
int fail(int code, const char* fmt, ...);
void note_kernel(const char* name);
int cuda_ok(cudaError_t e, const char* what);
// records the next lent timing event (if any) on the stream; call after every kernel launch
void mark_kernel(cudaStream_t st);

// Resolved launch plan of one forward call.
struct FwdPlan {
    int pack_gqa;        // rows of one KV head's query group are stacked into the M dimension
    int nsplit;          // KV splits (>= 1)
    int blocks_per_split;// KV blocks (of kGenericBN keys) per split
    int rotate_q;        // q is rotated into the workspace first
    size_t q_rot_bytes, o_part_bytes, lse_part_bytes;
    int use_sm100;       // tcgen05 kernel eligible
    int use_decode;      // warp-per-split decode kernel eligible
};

// scheduler-metadata blob (sched_meta.cu): header, then kSchedSeqInts entries per sequence
constexpr int kSchedMagic = 0x46413130;
constexpr int kSchedHeaderInts = 8;
constexpr int kSchedSeqInts = 8;

constexpr int kGenericBM = 64;
constexpr int kGenericBN = 64;

int  sm_count();
void plan_forward(const fa_fwd_params& p, FwdPlan& plan);

// kernels' host launchers (each returns an fa_status)
int launch_fwd_generic(const fa_fwd_params& p, const FwdPlan& plan, float* o_part, float* lse_part);
int launch_fwd_decode(const fa_fwd_params& p, const FwdPlan& plan, float* o_part, float* lse_part);
bool fwd_decode_supported(const fa_fwd_params& p);
void decode_set_use_tma(int v);
int decode_error_flag(bool clear);
// nsplit > 1 (two-tile kernel, cache calls): fp32 partials into o_part / lse_part, keys_per_split a multiple of 128
int launch_fwd_sm100(const fa_fwd_params& p, int nsplit = 1, int keys_per_split = 0, float* o_part = nullptr, float* lse_part = nullptr);
bool fwd_sm100_supported(const fa_fwd_params& p);
long fwd_sm100_ctas(const fa_fwd_params& p);         // CTAs of one key split of the call
// reads (and optionally clears) the code a timed-out wait left behind; synchronises
int sm100_error_flag(bool clear);
int launch_append_rotary(const fa_fwd_params& p, void* q_rot, int rotate_q_by_pos);
int launch_fwd_combine(const fa_fwd_params& p, int nsplit, const float* o_part, const float* lse_part,
                       int to_partial);
int combine_flat(const fa_combine_params& c);
int combine_flat_keep(const fa_combine_params& c);
// exchange of partials over peer memory fused with the combine (peer_combine.cu)
int peer_combine(const fa_peer_combine_params& c);
int peer_buffer_create(size_t bytes, void** ptr, unsigned char* handle);
int peer_buffer_open(const unsigned char* handle, void** ptr);
int launch_bwd_generic(const fa_bwd_params& p);
// 0 = automatic kernel choice, 1 = generic kernels only (fa_set_kernel_policy)
int kernel_policy();
// int8 latent decode on tcgen05 over a pair of CTAs that split the score dimensions (mla_sm100_pair.cu)
bool mla_pair_supported(const fa_mla_params& p);
int launch_mla_pair(const fa_mla_params& p, int nsplit, int tokens_per_split, float* o_part, float* lse_part,
                    int final_direct, cudaStream_t st);
int mla_pair_error_flag(bool clear);
int launch_bwd_sm100(const fa_bwd_params& p);
// 1 (default): dense calls hand dS^T tiles from the dK/dV kernel to a one-GEMM dQ kernel (fa_debug_set key 7)
void bwd_sm100_set_ds_spill(int v);
// true while the caller has lent per-kernel timing events to this thread
bool kernel_events_active();
bool bwd_sm100_supported(const fa_bwd_params& p);
size_t bwd_generic_workspace(const fa_bwd_params& p);
size_t bwd_sm100_workspace(const fa_bwd_params& p);

}  // namespace fa
