"""ctypes binding of librew_b200.so (the C ABI declared in include/rew_b200.h).

The library is CUDA-only.  Importing this module never falls back to a CPU
implementation: if the shared object is missing it raises, and every compute
entry point fails with the library's own message when no B200 is present.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "librew_b200.so")

OK = 0
BOOL, I8, I16, I32, I64, U8 = 0, 1, 2, 3, 4, 5
F16, BF16, F32, F64 = 9, 10, 11, 12


class RewB200Error(RuntimeError):
    """Raised for every non-zero status; carries rewb200_last_error()."""


class Config(C.Structure):
    _fields_ = [
        ("vocab", C.c_int32), ("d_model", C.c_int32), ("n_layers", C.c_int32), ("n_heads", C.c_int32),
        ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("ffn", C.c_int32), ("max_seq", C.c_int32),
        ("theta", C.c_double), ("eps", C.c_float), ("norm_kind", C.c_int32), ("mask_kind", C.c_int32),
        ("n_routed", C.c_int32), ("n_shared", C.c_int32), ("top_k", C.c_int32), ("moe_ffn", C.c_int32),
        ("first_dense", C.c_int32), ("dtype", C.c_int32), ("tp_rank", C.c_int32), ("tp_size", C.c_int32),
        ("ep_rank", C.c_int32), ("ep_size", C.c_int32), ("weight_quant", C.c_int32),
    ]


_lib = None

P = C.c_void_p
PP = C.POINTER(C.c_void_p)
I64P = C.POINTER(C.c_int64)
I32P = C.POINTER(C.c_int32)
F32P = C.POINTER(C.c_float)

# name -> (restype, argtypes); exactly the declarations of include/rew_b200.h
SIGNATURES = {
    "rewb200_init": (C.c_int, [I32P, C.c_int]),
    "rewb200_shutdown": (C.c_int, []),
    "rewb200_last_error": (C.c_char_p, []),
    "rewb200_sync": (C.c_int, [C.c_int, C.c_int]),
    "rewb200_set_option": (C.c_int, [C.c_int, C.c_char_p, C.c_char_p]),
    "rewb200_launch_count": (C.c_int64, [C.c_int]),
    "rewb200_buffer_from_host": (C.c_int, [C.c_int, P, C.c_int, I64P, C.c_int, PP]),
    "rewb200_buffer_alloc": (C.c_int, [C.c_int, C.c_int, I64P, C.c_int, PP]),
    "rewb200_buffer_to_host": (C.c_int, [P, P, C.c_size_t]),
    "rewb200_buffer_info": (C.c_int, [P, I32P, I64P, I32P]),
    "rewb200_buffer_device_ptr": (C.c_void_p, [P]),
    "rewb200_buffer_release": (None, [P]),
    "rewb200_dispatch": (C.c_int, [C.c_char_p, PP, C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_char_p), C.c_int, PP, I32P]),
    "rewb200_linear": (C.c_int, [P, P, P, PP]),
    "rewb200_rmsnorm": (C.c_int, [P, P, C.c_float, PP]),
    "rewb200_layernorm": (C.c_int, [P, P, P, C.c_float, PP]),
    "rewb200_rope_tables": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_double, PP, PP]),
    "rewb200_rope": (C.c_int, [P, P, P, C.c_int64, PP]),
    "rewb200_gqa_attention": (C.c_int, [P, P, P, C.c_int, C.c_int, PP]),
    "rewb200_gqa_attention_timed": (C.c_int, [P, P, P, C.c_int, C.c_int, C.c_int, F32P, PP]),
    "rewb200_swiglu_ffn": (C.c_int, [P, P, P, P, P, P, P, PP]),
    "rewb200_embed_gather": (C.c_int, [P, P, PP]),
    "rewb200_moe_route": (C.c_int, [P, P, P, C.c_int, PP, PP]),
    "rewb200_linear_noalloc": (C.c_int, [C.c_int, P, P, P, P, C.c_int64, C.c_int64, C.c_int64]),
    "rewb200_model_create": (C.c_int, [C.c_int, C.POINTER(Config), PP]),
    "rewb200_model_free": (None, [P]),
    "rewb200_model_tensor_count": (C.c_int64, [P]),
    "rewb200_model_set_tensor": (C.c_int, [P, C.c_int64, F32P, C.c_int64]),
    "rewb200_model_tensor_layout": (C.c_int, [P, C.c_int64, I32P, I64P, I64P, I64P, I32P]),
    "rewb200_model_set_tensor_shard": (C.c_int, [P, C.c_int64, F32P, I64P, I64P, C.c_int]),
    "rewb200_model_init_random": (C.c_int, [P, C.c_uint64, C.c_float]),
    "rewb200_model_finalize": (C.c_int, [P]),
    "rewb200_model_weight_bytes": (C.c_int64, [P]),
    "rewb200_session_create": (C.c_int, [P, C.c_int, C.c_int, PP]),
    "rewb200_session_free": (None, [P]),
    "rewb200_session_reset": (C.c_int, [P]),
    "rewb200_session_forward": (C.c_int, [P, I32P, C.c_int, I32P, F32P]),
    "rewb200_session_decode": (C.c_int, [P, C.c_int, I32P, F32P]),
    "rewb200_generate": (C.c_int, [P, I32P, C.c_int, C.c_int, C.c_int, I32P, F32P]),
    "rewb200_nf4_pack": (C.c_int, [P, PP]),
    "rewb200_nf4_free": (None, [P]),
    "rewb200_nf4_info": (C.c_int, [P, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "rewb200_nf4_unpack": (C.c_int, [P, C.POINTER(C.c_uint8), F32P]),
    "rewb200_nf4_dequantize": (C.c_int, [P, PP]),
    "rewb200_qlora_linear": (C.c_int, [P, P, P, P, P, C.c_float, PP]),
    "rewb200_session_create_paged": (C.c_int, [P, C.c_int, C.c_int, C.c_int, PP]),
    "rewb200_session_free_blocks": (C.c_int, [P]),
    "rewb200_lane_length": (C.c_int, [P, C.c_int]),
    "rewb200_lane_admit": (C.c_int, [P, C.c_int, I32P, C.c_int, C.c_uint64, I32P]),
    "rewb200_lanes_step": (C.c_int, [P, C.c_int, I32P]),
    "rewb200_lane_release": (C.c_int, [P, C.c_int]),
    "rewb200_session_set_sampling": (C.c_int, [P, C.c_float, C.c_int, C.c_float, C.c_float, C.c_float, C.c_int,
                                               C.POINTER(C.c_uint64)]),
    "rewb200_session_clear_sampling": (C.c_int, [P]),
    "rewb200_session_logprobs": (C.c_int, [P, C.c_int, F32P]),
    "rewb200_session_last_ms": (C.c_int, [P, F32P, F32P]),
    "rewb200_session_graph_kernels": (C.c_int, [P]),
    "rewb200_session_routing": (C.c_int, [P, C.c_int, I32P, C.c_int64]),
    "rewb200_session_trace_step": (C.c_int, [P, F32P, C.c_int]),
    "rewb200_session_profile_linears": (C.c_int, [P, C.c_int, F32P, I64P, I32P]),
    "rewb200_model_forward_all": (C.c_int, [P, I32P, C.c_int, C.c_int64, C.c_int, F32P]),
    "rewb200_comm_unique_id": (C.c_int, [P]),
    "rewb200_comm_init": (C.c_int, [C.c_int, P, C.c_int, C.c_int]),
    "rewb200_comm_allreduce_f32": (C.c_int, [C.c_int, P, C.c_int64]),
    "rewb200_comm_alltoall": (C.c_int, [C.c_int, P, P, C.c_int64]),
    "rewb200_generate_stop": (C.c_int, [P, I32P, C.c_int, C.c_int, C.c_int, I32P, C.c_int, I32P, F32P]),
    "rewb200_kv_create": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, PP]),
    "rewb200_kv_free": (None, [P]),
    "rewb200_kv_length": (C.c_int, [P]),
    "rewb200_kv_reset": (C.c_int, [P]),
    "rewb200_qkv_rope_kvappend": (C.c_int, [P, P, P, P, P, P, P, P, P, P, PP]),
    "rewb200_gqa_attention_cached": (C.c_int, [P, P, C.c_int, C.c_int, PP]),
    "rewb200_experts_create": (C.c_int, [C.c_int, C.c_int, P, P, P, P, P, P, PP]),
    "rewb200_experts_free": (None, [P]),
    "rewb200_moe_experts": (C.c_int, [P, P, P, P, PP]),
    "rewb200_sampler_create": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float,
                                         C.c_float, C.c_int, C.POINTER(C.c_uint64), PP]),
    "rewb200_sampler_free": (None, [P]),
    "rewb200_sampler_observe": (C.c_int, [P, I32P, C.c_int]),
    "rewb200_lmhead_sample": (C.c_int, [P, P, P, P, I32P, F32P]),
    "rewb200_comm_peer_alloc": (C.c_int, [C.c_int, C.c_int64, C.c_int64, P]),
    "rewb200_comm_peer_attach": (C.c_int, [C.c_int, P]),
    "rewb200_comm_destroy": (C.c_int, [C.c_int]),
}


def lib():
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RewB200Error(
                "librew_b200.so is missing (%s); build it with `python -m rew_b200.build`. "
                "There is no CPU fallback." % LIB_PATH)
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(status):
    if status != OK:
        raise RewB200Error(lib().rewb200_last_error().decode("utf-8", "replace"))


_initialised = False


def init(device=None):
    """rewb200_init for this process's GPU (LOCAL_RANK or 0)."""
    global _initialised
    if _initialised:
        return
    if device is None:
        device = int(os.environ.get("LOCAL_RANK", "0"))
    arr = (C.c_int32 * 1)(device)
    check(lib().rewb200_init(arr, 1))
    _initialised = True
