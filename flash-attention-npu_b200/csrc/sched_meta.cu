// Device-side schedule for the KV-cache forward (get_scheduler_metadata,
// csrc/ascend910/flash_attn_npu_3/flash_api.cpp:506-571; ComputeFAMetadata,
// fa_metadata.aicpu:32-151): one CTA reads the device-resident lengths and writes the split
// plan, so the host never synchronises to learn them.
//
// Layout of the int32 blob (fa_scheduler_metadata_ints(b) = 8 + 8 b entries):
//   [0] magic 0x46413130  [1] b  [2] split count of the launch grid  [3] KV blocks (64 keys) per split of the host plan
//   [4] longest sequence  [5] total KV blocks  [6] total active (sequence, split) pairs  [7] 0
//   then per sequence 8 entries: length (after append), KV blocks, active splits, keys per active split,
//   prefix of active splits, 0, 0, 0.
// The host plans the grid from the cache capacity (the only length it knows); a sequence of `len` keys uses
// act = ceil(len / keys per host split) of the grid's splits, and the blob spreads its keys EVENLY over those
// (keys per active split = ceil(len / act) rounded up to 64), where the host plan alone would leave the last split
// of every sequence partly empty.  The decode kernels take the per-sequence figure from the blob (decode_splitkv.cu).
#include "fa_internal.h"

namespace fa {

__global__ void sched_meta_kernel(const fa_sched_params p, int nsplit, int bps) {
    __shared__ int s_max, s_blocks, s_active;
    if (threadIdx.x == 0) { s_max = 0; s_blocks = 0; s_active = 0; }
    __syncthreads();
    for (int b = threadIdx.x; b < p.b; b += blockDim.x) {
        const long long cap = (long long)p.sk + p.s_new;
        const int len = (int)max(0LL, min((long long)p.seqused_k[b] + p.s_new, cap));
        const int nb = (len + kGenericBN - 1) / kGenericBN;
        const int act = min(nsplit, (nb + bps - 1) / bps);
        const int per = act > 0 ? ((len + act - 1) / act + kGenericBN - 1) / kGenericBN * kGenericBN : 0;
        int* m = p.meta + kSchedHeaderInts + kSchedSeqInts * b;
        m[0] = len; m[1] = nb; m[2] = act; m[3] = per; m[5] = 0; m[6] = 0; m[7] = 0;
        atomicMax(&s_max, len);
        atomicAdd(&s_blocks, nb);
        atomicAdd(&s_active, act);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int b = 0; b < p.b; ++b) {
            int* m = p.meta + kSchedHeaderInts + kSchedSeqInts * b;
            m[4] = run;
            run += m[2];
        }
        p.meta[0] = kSchedMagic; p.meta[1] = p.b; p.meta[2] = nsplit; p.meta[3] = bps;
        p.meta[4] = s_max; p.meta[5] = s_blocks; p.meta[6] = s_active; p.meta[7] = 0;
    }
}

}  // namespace fa

extern "C" {

size_t fa_scheduler_metadata_ints(int32_t b) { return fa::kSchedHeaderInts + fa::kSchedSeqInts * (size_t)(b > 0 ? b : 0); }

int fa_scheduler_metadata(const fa_sched_params* p) {
    using namespace fa;
    if (!p || !p->seqused_k || !p->meta) return fail(FA_ERR_NULL, "null pointer");
    if (p->b <= 0 || p->hq <= 0 || p->hkv <= 0 || p->hq % p->hkv) return fail(FA_ERR_BAD_SHAPE, "bad sizes");
    fa_fwd_params f = {};
    f.seqused_k = p->seqused_k; f.b = p->b; f.sq = p->sq; f.sk = p->sk + p->s_new; f.hq = p->hq; f.hkv = p->hkv;
    f.d = p->d; f.dv = p->dv; f.num_splits = p->num_splits; f.page_size = p->page_size;
    FwdPlan plan;
    plan_forward(f, plan);
    sched_meta_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(p->stream)>>>(*p, plan.nsplit, plan.blocks_per_split);
    return cuda_ok(cudaGetLastError(), "sched_meta launch");
}

}
