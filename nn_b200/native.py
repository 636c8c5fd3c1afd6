"""ctypes binding of libns_b200.so -- the Python twin of the reference's P/Invoke class
(src/NeuralSharp/Backends/Cuda/CudaDriver.cs:63-179): one declaration per exported function and a
``check`` that turns a non-zero return code into an exception carrying ``ns_last_error()``.

There is no fallback: if the library is missing, or no CUDA device is usable, calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libns_b200.so")

NS_F32, NS_BF16, NS_I8, NS_I32 = 0, 1, 2, 3
EPI_NONE, EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESIDUAL = 0, 1, 2, 3
SPLIT_NONE, SPLIT_COLUMN, SPLIT_ROW = 0, 1, 2

u64, i64, i32, u32, f32, vp, cp = C.c_uint64, C.c_int64, C.c_int, C.c_uint32, C.c_float, C.c_void_p, C.c_char_p
P = C.POINTER

# name -> argument types (every function returns int unless listed in _SPECIAL)
SIGNATURES = {
    "ns_device_count": [P(i32)],
    "ns_device_open": [i32, P(vp)],
    "ns_device_open_on_stream": [i32, u64, P(vp)],
    "ns_device_close": [vp],
    "ns_device_info": [vp, C.c_char_p, P(i32), P(u64), P(u64)],
    "ns_device_stream": [vp, P(u64)],
    "ns_stream_sync": [vp],
    "ns_device_status": [vp, P(i32)],
    "ns_device_tune": [vp, i32, i32],
    "ns_debug_tail_times": [vp, u64],
    "ns_alloc": [vp, u64, i32, P(u64)],
    "ns_free": [vp, u64],
    "ns_h2d": [vp, u64, vp, u64],
    "ns_d2h": [vp, vp, u64, u64],
    "ns_h2d_async": [vp, u64, vp, u64],
    "ns_d2h_async": [vp, vp, u64, u64],
    "ns_d2d_async": [vp, u64, u64, u64],
    "ns_d2d_2d_async": [vp, u64, u64, u64, u64, u64, u64],
    "ns_memset32_async": [vp, u64, u32, u64],
    "ns_host_alloc": [u64, P(vp)],
    "ns_host_free": [vp],
    "ns_ipc_handle": [vp, u64, vp],
    "ns_ipc_open": [vp, vp, P(u64)],
    "ns_ipc_close": [vp, u64],
    "ns_capture_begin": [vp],
    "ns_capture_end": [vp, P(vp)],
    "ns_capture_abort": [vp],
    "ns_graph_launch": [vp, vp],
    "ns_graph_destroy": [vp],
    "ns_event_create": [vp, P(u64)],
    "ns_event_record": [vp, u64],
    "ns_event_elapsed_ms": [vp, u64, u64, P(f32)],
    "ns_event_destroy": [vp, u64],
    "ns_stream_wait_event": [vp, u64],
    "ns_quantize_rows_i8": [vp, u64, i32, i64, i32, u64, u64],
    "ns_qmatmul_i8": [vp, u64, u64, u64, u64, u64, u64, i32, i32, i32, i32, i32, i32, u64, u64],
    "ns_qmatmul_i8_static": [vp, u64, u64, u64, u64, u64, u64, i32, i32, i32, i32, i32, i32, u64],
    "ns_bench_i8_mainloop": [vp, u64, u64, i32, i32, i32],
    "ns_matmul_bf16": [vp, u64, u64, u64, i32, i32, i32, i32, i32, u64, u64, i32, i32, i32],
    "ns_layernorm": [vp, u64, i32, u64, u64, i64, i32, f32, i32, u64, u64],
    "ns_embed_pos": [vp, u64, u64, u64, i32, u64, i32, i32, i32, i32, i32, i32, u64],
    "ns_argmax_i32": [vp, u64, i32, i32, i64, u64],
    "ns_add_i32": [vp, u64, C.c_int32],
    "ns_convert": [vp, u64, i32, u64, i32, i64],
    "ns_fill_normal": [vp, u64, i32, i64, u32, f32, f32],
    "ns_fill_ids": [vp, u64, i64, u32, u32],
    "ns_kv_cache_create": [vp, i32, i32, i32, i32, P(vp)],
    "ns_kv_cache_create_in": [vp, i32, i32, i32, i32, u64, u64, P(vp)],
    "ns_kv_cache_destroy": [vp],
    "ns_kv_scatter_heads": [vp, vp, u64, i32, i32, i32, i32, P(u64), P(u64), i32, i32, i32, u64, i32, i32, u64, u64],
    "ns_kv_cache_pools": [vp, P(u64), P(u64), P(u64)],
    "ns_kv_append": [vp, vp, u64, u64, i64, u64, i32, u64, i32, i32],
    "ns_attention_decode": [vp, vp, u64, i64, u64, i64, u64, i32, u64, i32, i32, f32],
    "ns_attention_prefill": [vp, u64, u64, u64, u64, i32, i32, i32, i32, P(i64), P(i64), P(i64), P(i64), f32, i32],
    "ns_linear_create": [vp, i32, i32, i32, P(f32), P(f32), i32, i32, i32, i32, P(vp)],
    "ns_linear_destroy": [vp],
    "ns_linear_info": [vp, P(i32), P(i32), P(i32), P(u64), P(u64), P(u64)],
    "ns_linear_forward": [vp, vp, u64, u64, i32, i32, u64, i32, i32, u64],
    "ns_linear_forward_host": [vp, vp, vp, i32, i32, vp, i32],
    "ns_linear_forward_partial": [vp, vp, u64, i32, P(u64), P(i32)],
    "ns_finish_norm_quant": [vp, u64, i32, vp, u64, u64, i64, u64, u64, u64, f32, u64, u64],
    "ns_finish_gelu_quant": [vp, u64, i32, vp, u64, i64, u64, u64],
    "ns_finish_kv_append": [vp, u64, i32, vp, u64, i32, i32, u64, vp, u64, i32, u64],
    "ns_linear_forward_norm_quant": [vp, vp, u64, u64, u64, i64, u64, u64, u64, f32, u64, u64],
    "ns_linear_forward_gelu_quant": [vp, vp, u64, u64, i64, u64, u64],
    "ns_linear_forward_kv_append": [vp, vp, u64, u64, i32, i32, u64, vp, u64, i32, u64],
    "ns_linear_forward_tp_norm_quant": [vp, vp, vp, i32, u64, u64, u64, i64, u64, u64, u64, f32, u64, u64],
    "ns_attention_decode_quant": [vp, vp, u64, i64, u64, i64, u64, i32, u64, i32, i32, f32, u64, u64],
    "ns_bias_residual": [vp, u64, u64, u64, i32, i64, i32, i32, u64],
    "ns_argmax_partial": [vp, u64, i32, i32, i64, i32, u64, u64],
    "ns_argmax_merge": [vp, u64, u64, i32, i32, u64],
    "ns_comm_unique_id": [vp],
    "ns_comm_init_rank": [vp, vp, i32, i32, P(vp)],
    "ns_comm_info": [vp, P(i32), P(i32), P(i32)],
    "ns_allreduce": [vp, vp, u64, i64, i32],
    "ns_allgather": [vp, vp, u64, u64, i64, i32],
    "ns_comm_async_error": [vp, P(i32)],
    "ns_comm_abort": [vp],
    "ns_comm_destroy": [vp],
    "ns_peer_group_create": [vp, i32, i32, u64, P(vp)],
    "ns_peer_group_handle": [vp, vp],
    "ns_peer_group_connect": [vp, vp],
    "ns_peer_group_slot": [vp, i32, P(u64)],
    "ns_tp_reduce_norm_quant": [vp, vp, i32, u64, u64, i64, i32, u64, u64, u64, f32, u64, u64],
    "ns_peer_group_destroy": [vp],
    "ns_f32_batched_matmul": [vp, u64, u64, u64, i32, i32, i32, i32, i32, i32, f32],
    "ns_f32_scale_mask_softmax": [vp, u64, u64, u64, i32, i32, i32, f32],
    "ns_f32_layernorm_fused": [vp, u64, u64, u64, u64, i32, i32, f32],
    "ns_f32_bias_gelu": [vp, u64, u64, u64, i64, i32],
    "ns_f32_add_row_vector": [vp, u64, u64, u64, i32, i32],
    "ns_f32_add": [vp, u64, u64, u64, i64],
    "ns_f32_affine": [vp, u64, u64, i64, f32, f32],
    "ns_f32_add_broadcast_scalar": [vp, u64, u64, i64, f32],
    "ns_f32_decoder_mask": [vp, u64, u64, i32, i32],
    "ns_f32_key_value_write": [vp, u64, u64, u64, i32, i32, i32, i32],
    "ns_f32_gather": [vp, u64, u64, u64, i32, i32, i32],
    "ns_f32_argmax": [vp, u64, u64, i32, i32],
    "ns_f32_argmax_strided": [vp, u64, u64, i32, i32, i64, i64],
    "ns_f32_permute": [vp, u64, u64, P(i32), P(i32), i32, i32],
    "ns_f32_copy2d": [vp, u64, i64, i32, u64, i64, i32, i32, i32, i32],
    "ns_f32_sample_rows": [vp, u64, u64, u64, u64, i32, i32, i32, i32, f32, i32, f32, f32, u32],
    "ns_f32_penalize_rows": [vp, u64, u64, u64, u64, i32, i32, i32, i32, i32, i32, f32, f32, f32],
    "ns_f32_history_push": [vp, u64, u64, u64, i32, i32],
}

_SPECIAL = {
    "ns_last_error": (C.c_char_p, []),
    "ns_error_name": (C.c_char_p, [i32]),
    "ns_version": (i32, []),
}


class NsError(RuntimeError):
    """A libns_b200 call returned a non-zero code."""

    def __init__(self, call: str, code: int, text: str):
        super().__init__(f"{call} failed: {text} [{code}]")
        self.call, self.code, self.text = call, code, text


_lib = None


def load() -> C.CDLL:
    """Loads the library (once).  Raises FileNotFoundError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "or `make -C nn_b200/csrc`; there is no CPU fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in _SPECIAL.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = i32, args
    _lib = lib
    return lib


def exported_names() -> list[str]:
    return sorted(list(SIGNATURES) + list(_SPECIAL))


def check(call: str, code: int) -> None:
    if code != 0:
        text = load().ns_last_error().decode("utf-8", "replace")
        raise NsError(call, code, text)


def call(name: str, *args) -> None:
    check(name, getattr(load(), name)(*args))
