"""ctypes view of libfa_b200.so (include/fa_b200.h) plus the few torch helpers the
extension modules share.  torch is used for device memory and streams only; every
computation happens in the CUDA library.  If the library cannot be loaded the
import fails: there is no other code path."""
import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# FA_B200_LIB points the loader at another build of the same library (a debug or tuning build)
LIB_PATH = os.environ.get("FA_B200_LIB") or os.path.join(_HERE, "lib", "libfa_b200.so")


class FaTensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_s", C.c_int64), ("stride_h", C.c_int64)]


class FwdParams(C.Structure):
    _fields_ = [
        ("q", FaTensor), ("k", FaTensor), ("v", FaTensor), ("o", FaTensor),
        ("lse", C.c_void_p), ("lse_stride_b", C.c_int64), ("lse_stride_h", C.c_int64), ("lse_stride_s", C.c_int64),
        ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_k", C.c_void_p), ("seqused_k", C.c_void_p),
        ("block_table", C.c_void_p), ("block_table_stride", C.c_int64), ("page_size", C.c_int32),
        ("cache_batch_idx", C.c_void_p), ("alibi_slopes", C.c_void_p), ("alibi_stride_b", C.c_int64),
        ("b", C.c_int32), ("sq", C.c_int32), ("sk", C.c_int32), ("total_q", C.c_int32), ("total_k", C.c_int32),
        ("hq", C.c_int32), ("hkv", C.c_int32), ("d", C.c_int32), ("dv", C.c_int32),
        ("scale", C.c_float), ("softcap", C.c_float),
        ("causal", C.c_int32), ("window_left", C.c_int32), ("window_right", C.c_int32), ("dtype", C.c_int32),
        ("k_new", FaTensor), ("v_new", FaTensor), ("s_new", C.c_int32),
        ("rotary_cos", C.c_void_p), ("rotary_sin", C.c_void_p),
        ("rotary_dim", C.c_int32), ("rotary_interleaved", C.c_int32), ("seqlen_ro", C.c_int32),
        ("num_splits", C.c_int32), ("kv_begin", C.c_int32), ("kv_end", C.c_int32), ("partials_only", C.c_int32),
        ("o_partial", C.c_void_p), ("lse_partial", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("sched_meta", C.c_void_p), ("kv_entries", C.c_int64), ("stream", C.c_void_p),
    ]


class BwdParams(C.Structure):
    _fields_ = [
        ("dout", FaTensor), ("q", FaTensor), ("k", FaTensor), ("v", FaTensor), ("o", FaTensor),
        ("dq", FaTensor), ("dk", FaTensor), ("dv", FaTensor),
        ("lse", C.c_void_p), ("lse_stride_b", C.c_int64), ("lse_stride_h", C.c_int64), ("lse_stride_s", C.c_int64),
        ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_k", C.c_void_p),
        ("b", C.c_int32), ("sq", C.c_int32), ("sk", C.c_int32), ("total_q", C.c_int32), ("total_k", C.c_int32),
        ("hq", C.c_int32), ("hkv", C.c_int32), ("d", C.c_int32), ("dv_dim", C.c_int32),
        ("scale", C.c_float), ("softcap", C.c_float),
        ("causal", C.c_int32), ("window_left", C.c_int32), ("window_right", C.c_int32),
        ("dtype", C.c_int32), ("deterministic", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
        ("alibi_slopes", C.c_void_p), ("alibi_stride_b", C.c_int64),
    ]


class CombineParams(C.Structure):
    _fields_ = [
        ("o_partial", C.c_void_p), ("lse_partial", C.c_void_p),
        ("o_split_stride", C.c_int64), ("o_row_stride", C.c_int64), ("lse_split_stride", C.c_int64),
        ("o", C.c_void_p), ("o_stride", C.c_int64), ("lse", C.c_void_p),
        ("nsplit", C.c_int32), ("rows", C.c_int32), ("dv", C.c_int32), ("out_dtype", C.c_int32),
        ("stream", C.c_void_p),
    ]


MAX_PEERS = 16
PEER_HANDLE_BYTES = 64


class PeerCombineParams(C.Structure):
    _fields_ = [
        ("rank", C.c_int32), ("world", C.c_int32),
        ("peers", C.c_void_p * MAX_PEERS),
        ("slot_offset", C.c_size_t), ("lse_offset", C.c_size_t), ("flag_offset", C.c_size_t),
        ("epoch", C.c_uint32), ("timeout_ms", C.c_uint32),
        ("rows", C.c_int64), ("dv", C.c_int32), ("out_dtype", C.c_int32),
        ("o", C.c_void_p), ("o_stride", C.c_int64), ("lse", C.c_void_p), ("status", C.c_void_p),
        ("stream", C.c_void_p),
    ]


class MlaParams(C.Structure):
    _fields_ = [
        ("q_nope", C.c_void_p), ("q_rope", C.c_void_p),
        ("q_nope_stride_b", C.c_int64), ("q_nope_stride_h", C.c_int64),
        ("q_rope_stride_b", C.c_int64), ("q_rope_stride_h", C.c_int64),
        ("latent", C.c_void_p), ("scales", C.c_void_p), ("rope", C.c_void_p),
        ("block_table", C.c_void_p), ("block_table_stride", C.c_int64), ("page_size", C.c_int32),
        ("cache_seqlens", C.c_void_p),
        ("o", C.c_void_p), ("o_stride_b", C.c_int64), ("o_stride_h", C.c_int64), ("lse", C.c_void_p),
        ("b", C.c_int32), ("hq", C.c_int32), ("scale", C.c_float), ("num_splits", C.c_int32),
        ("kv_begin", C.c_int32), ("kv_end", C.c_int32), ("partials_only", C.c_int32),
        ("o_partial", C.c_void_p), ("lse_partial", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
    ]


class SchedParams(C.Structure):
    _fields_ = [
        ("seqused_k", C.c_void_p), ("cu_seqlens_q", C.c_void_p),
        ("b", C.c_int32), ("sq", C.c_int32), ("sk", C.c_int32), ("hq", C.c_int32), ("hkv", C.c_int32),
        ("d", C.c_int32), ("dv", C.c_int32), ("page_size", C.c_int32), ("s_new", C.c_int32),
        ("causal", C.c_int32), ("window_left", C.c_int32), ("window_right", C.c_int32), ("num_splits", C.c_int32),
        ("meta", C.c_void_p), ("stream", C.c_void_p),
    ]


EXPORTS = {
    "fa_fwd": (C.c_int, [C.POINTER(FwdParams)]),
    "fa_varlen_fwd": (C.c_int, [C.POINTER(FwdParams)]),
    "fa_fwd_kvcache": (C.c_int, [C.POINTER(FwdParams)]),
    "fa_fwd_kvcache_static": (C.c_int, [C.POINTER(FwdParams)]),
    "fa_static_scratch_bytes": (C.c_size_t, []),
    "fa_fwd_workspace_bytes": (C.c_size_t, [C.POINTER(FwdParams)]),
    "fa_fwd_num_splits": (C.c_int, [C.POINTER(FwdParams)]),
    "fa_bwd": (C.c_int, [C.POINTER(BwdParams)]),
    "fa_varlen_bwd": (C.c_int, [C.POINTER(BwdParams)]),
    "fa_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(BwdParams)]),
    "fa_combine": (C.c_int, [C.POINTER(CombineParams)]),
    "fa_mla_decode": (C.c_int, [C.POINTER(MlaParams)]),
    "fa_peer_combine": (C.c_int, [C.POINTER(PeerCombineParams)]),
    "fa_copy_2d_async": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p]),
    "fa_peer_buffer_create": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]),
    "fa_peer_buffer_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "fa_peer_buffer_close": (C.c_int, [C.c_void_p]),
    "fa_peer_buffer_destroy": (C.c_int, [C.c_void_p]),
    "fa_mla_workspace_bytes": (C.c_size_t, [C.POINTER(MlaParams)]),
    "fa_mla_num_splits": (C.c_int, [C.POINTER(MlaParams)]),
    "fa_scheduler_metadata": (C.c_int, [C.POINTER(SchedParams)]),
    "fa_scheduler_metadata_ints": (C.c_size_t, [C.c_int32]),
    "fa_last_error": (C.c_char_p, []),
    "fa_version": (C.c_char_p, []),
    "fa_last_kernel": (C.c_char_p, []),
    "fa_set_kernel_policy": (None, [C.c_int]),
    "fa_debug_set": (None, [C.c_int, C.c_int]),
    "fa_debug_get": (C.c_int, [C.c_int]),
    "fa_set_kernel_events": (None, [C.POINTER(C.c_void_p), C.c_int]),
    "fa_kernel_events_used": (C.c_int, []),
}


def load_library(path=LIB_PATH):
    if not os.path.exists(path):
        raise ImportError(
            f"{path} not found: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(there is no fallback implementation)")
    lib = C.CDLL(path)
    for name, (res, args) in EXPORTS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = load_library()

DTYPES = {torch.float16: 0, torch.bfloat16: 1}


def check(status):
    if status != 0:
        raise RuntimeError(lib.fa_last_error().decode())


def last_kernel():
    return lib.fa_last_kernel().decode()


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_ptr(device):
    return torch.cuda.current_stream(device).cuda_stream


def tensor4(t, packed=False):
    """(B,S,H,D) view -> FaTensor; packed (T,H,D) uses the seq and head strides only."""
    if t is None:
        return FaTensor(None, 0, 0, 0)
    if t.stride(-1) != 1:
        raise RuntimeError("last dimension must be contiguous")
    if packed:
        return FaTensor(t.data_ptr(), 0, t.stride(0), t.stride(1))
    return FaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("expected CUDA tensors: this library has no CPU implementation")


def workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)
