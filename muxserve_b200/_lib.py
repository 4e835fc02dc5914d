"""ctypes binding of ``libmuxb200.so`` — the C ABI declared in ``include/muxb200.h``.

There is no fallback: if the library is missing or does not export a symbol
the import of the op modules fails with a clear error.  Build it with
``python -m muxserve_b200.build``.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libmuxb200.so"

MUX_DTYPE_F16 = 0
MUX_DTYPE_BF16 = 1

MUX_DEV_BAD_BLOCK_ID = 1
MUX_DEV_WAIT_TIMEOUT = 2
MUX_DEV_BAD_CONTEXT = 4
MUX_DEV_BAD_SLOT = 8
MUX_DEV_BAD_HEAD_MAPPING = 16
MUX_DEV_INTERNAL = 32
MUX_DEV_BAD_GROUP = 64

MUX_ATTN_EARLY_KV = 1
MUX_OPROJ_EARLY_W = 1

MUX_TP_AUTO, MUX_TP_ONE_SHOT, MUX_TP_TWO_SHOT = 0, 1, 2

ABI_VERSION = 16


class CacheWriteArgs(C.Structure):
    _fields_ = [
        ("k", C.c_void_p), ("v", C.c_void_p),
        ("k_token_stride", C.c_int64), ("k_head_stride", C.c_int64),
        ("v_token_stride", C.c_int64), ("v_head_stride", C.c_int64),
        ("key_cache", C.c_void_p), ("value_cache", C.c_void_p),
        ("num_blocks", C.c_int64),
        ("slot_mapping", C.c_void_p),
        ("slot_token_stride", C.c_int64), ("slot_head_stride", C.c_int64),
        ("num_tokens", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_size", C.c_int32), ("block_size", C.c_int32),
        ("dtype", C.c_int32), ("reserved", C.c_int32),
    ]


class AttnArgs(C.Structure):
    _fields_ = [
        ("out", C.c_void_p), ("q", C.c_void_p),
        ("q_seq_stride", C.c_int64), ("q_head_stride", C.c_int64),
        ("out_seq_stride", C.c_int64), ("out_head_stride", C.c_int64),
        ("key_cache", C.c_void_p), ("value_cache", C.c_void_p),
        ("num_blocks", C.c_int64),
        ("head_mapping", C.c_void_p),
        ("block_tables", C.c_void_p),
        ("bt_seq_stride", C.c_int64), ("bt_head_stride", C.c_int64),
        ("context_lens", C.c_void_p),
        ("seq_rows", C.c_void_p),
        ("scale", C.c_float),
        ("num_seqs", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_size", C.c_int32), ("block_size", C.c_int32), ("max_context_len", C.c_int32),
        ("dtype", C.c_int32), ("partition_size", C.c_int32), ("num_stages", C.c_int32),
        ("flags", C.c_int32), ("num_units", C.c_int32), ("units", C.c_void_p),
    ]


class AttnMixedArgs(C.Structure):
    _fields_ = [
        ("out", C.c_void_p), ("q", C.c_void_p),
        ("q_row_stride", C.c_int64), ("out_row_stride", C.c_int64),
        ("key_cache", C.c_void_p), ("value_cache", C.c_void_p),
        ("num_blocks", C.c_int64),
        ("block_tables", C.c_void_p), ("bt_item_stride", C.c_int64),
        ("item_context_len", C.c_void_p), ("item_q_row", C.c_void_p),
        ("item_group", C.c_void_p), ("item_scale", C.c_void_p),
        ("num_items", C.c_int32), ("max_group", C.c_int32),
        ("head_size", C.c_int32), ("block_size", C.c_int32), ("max_context_len", C.c_int32),
        ("dtype", C.c_int32), ("partition_size", C.c_int32), ("num_stages", C.c_int32),
        ("flags", C.c_int32), ("num_units", C.c_int32), ("units", C.c_void_p),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("attn", AttnArgs), ("k", C.c_void_p), ("v", C.c_void_p),
        ("k_seq_stride", C.c_int64), ("k_head_stride", C.c_int64),
        ("v_seq_stride", C.c_int64), ("v_head_stride", C.c_int64),
        ("cos_sin_cache", C.c_void_p), ("max_position", C.c_int64),
        ("new_tokens", C.c_int32), ("reserved", C.c_int32),
    ]


class DecodeMixedArgs(C.Structure):
    _fields_ = [
        ("attn", AttnMixedArgs), ("k", C.c_void_p), ("v", C.c_void_p),
        ("k_row_stride", C.c_int64), ("v_row_stride", C.c_int64),
        ("cos_sin_cache", C.c_void_p), ("max_position", C.c_int64),
        ("new_tokens", C.c_int32), ("reserved", C.c_int32),
    ]


class RotaryArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p),
        ("q_token_stride", C.c_int64), ("q_head_stride", C.c_int64),
        ("k_token_stride", C.c_int64), ("k_head_stride", C.c_int64),
        ("positions", C.c_void_p), ("cos_sin_cache", C.c_void_p), ("max_position", C.c_int64),
        ("num_tokens", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_size", C.c_int32),
        ("dtype", C.c_int32), ("reserved", C.c_int32),
    ]


class PrefillArgs(C.Structure):
    _fields_ = [
        ("out", C.c_void_p), ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("out_seq_stride", C.c_int64), ("out_head_stride", C.c_int64),
        ("q_seq_stride", C.c_int64), ("q_head_stride", C.c_int64),
        ("k_seq_stride", C.c_int64), ("k_head_stride", C.c_int64),
        ("v_seq_stride", C.c_int64), ("v_head_stride", C.c_int64),
        ("cu_seqlens", C.c_void_p), ("scale", C.c_float),
        ("num_seqs", C.c_int32), ("total_tokens", C.c_int32), ("max_prompt_len", C.c_int32),
        ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_size", C.c_int32),
        ("dtype", C.c_int32), ("block_size", C.c_int32),
        ("key_cache", C.c_void_p), ("value_cache", C.c_void_p), ("slot_mapping", C.c_void_p),
        ("slot_token_stride", C.c_int64), ("slot_head_stride", C.c_int64), ("num_blocks", C.c_int64),
        ("block_tables", C.c_void_p), ("bt_seq_stride", C.c_int64), ("bt_head_stride", C.c_int64),
        ("max_blocks_per_seq", C.c_int32), ("num_units", C.c_int32), ("units", C.c_void_p),
    ]


class TpComm(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("buffers", C.c_void_p * 8), ("buffer_bytes", C.c_int64)]


class OprojArgs(C.Structure):
    _fields_ = [("a", C.c_void_p), ("a_row_stride", C.c_int64), ("w", C.c_void_p), ("w_row_stride", C.c_int64),
                ("out", C.c_void_p), ("out_row_stride", C.c_int64), ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
                ("dtype", C.c_int32), ("algo", C.c_int32), ("flags", C.c_int32)]


class MixedModel(C.Structure):
    _fields_ = [("scheduler", C.c_void_p), ("request_ids", C.POINTER(C.c_int32)), ("num_requests", C.c_int32),
                ("num_q_heads", C.c_int32), ("scale", C.c_float)]


class MixedSpan(C.Structure):
    _fields_ = [("model", C.c_int32), ("first_item", C.c_int32), ("num_items", C.c_int32), ("first_row", C.c_int32),
                ("num_rows", C.c_int32), ("num_layers", C.c_int32)]


_I32P = C.POINTER(C.c_int32)
_I64P = C.POINTER(C.c_int64)

# name -> (restype, argtypes); every symbol include/muxb200.h declares
SIGNATURES = {
    "mux_strerror": (C.c_char_p, [C.c_int]),
    "mux_last_cuda_error": (C.c_int, []),
    "mux_abi_version": (C.c_int, []),
    "mux_reshape_and_cache": (C.c_int, [C.POINTER(CacheWriteArgs), C.c_void_p]),
    "mux_paged_attention_workspace_size": (C.c_size_t, [C.POINTER(AttnArgs)]),
    "mux_paged_attention": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "mux_paged_attention_static_scratch": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "mux_paged_attention_mixed_workspace_size": (C.c_size_t, [C.POINTER(AttnMixedArgs)]),
    "mux_paged_attention_mixed": (C.c_int, [C.POINTER(AttnMixedArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "mux_decode_attention": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "mux_decode_attention_mixed": (C.c_int, [C.POINTER(DecodeMixedArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "mux_rotary_embedding": (C.c_int, [C.POINTER(RotaryArgs), C.c_void_p]),
    "mux_prefill_attention": (C.c_int, [C.POINTER(PrefillArgs), C.c_void_p]),
    "mux_block_table_append": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                                         C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "mux_tp_allreduce_buffer_size": (C.c_size_t, [C.c_int32, C.c_size_t]),
    "mux_tp_buffer_create": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "mux_tp_buffer_destroy": (C.c_int, [C.c_void_p]),
    "mux_tp_buffer_export": (C.c_int, [C.c_void_p, C.c_char_p]),
    "mux_tp_buffer_import": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "mux_tp_buffer_release": (C.c_int, [C.c_void_p]),
    "mux_tp_allreduce": (C.c_int, [C.POINTER(TpComm), C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                   C.c_int32, C.c_void_p]),
    "mux_tp_allreduce_emulated": (C.c_int, [C.c_int32, C.POINTER(C.c_void_p), C.c_int64, C.POINTER(C.c_void_p),
                                            C.POINTER(C.c_void_p), C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                                            C.c_void_p]),
    "mux_tp_oproj_allreduce": (C.c_int, [C.POINTER(TpComm), C.POINTER(OprojArgs), C.c_void_p]),
    "mux_tp_oproj_allreduce_emulated": (C.c_int, [C.c_int32, C.POINTER(C.c_void_p), C.c_int64, C.POINTER(OprojArgs),
                                                  C.c_void_p, C.c_void_p]),
    "mux_selftest_wait_timeout": (C.c_int, [C.c_void_p]),
    "mux_device_status": (C.c_int, [C.c_void_p]),
    "mux_kv_storage_create": (C.c_void_p, [C.c_int32]),
    "mux_kv_storage_destroy": (None, [C.c_void_p]),
    "mux_kv_storage_allocate": (C.c_int, [C.c_void_p, C.c_int32, _I32P]),
    "mux_kv_storage_allocate_batch": (C.c_int, [C.c_void_p, _I32P, C.c_int32, C.c_int32, C.c_int32,
                                                _I32P, C.c_int64, _I64P]),
    "mux_kv_storage_free_batch": (C.c_int64, [C.c_void_p, _I32P, C.c_int32]),
    "mux_kv_storage_new_blocks_allocated": (C.c_int32, [C.c_void_p]),
    "mux_kv_storage_num_blocks_allocated": (C.c_int32, [C.c_void_p]),
    "mux_kv_storage_num_free": (C.c_int64, [C.c_void_p]),
    "mux_kv_storage_free_list": (C.c_int, [C.c_void_p, _I32P, C.c_int64]),
    "mux_kv_storage_check": (C.c_int, [C.c_void_p]),
    "mux_batch_scheduler_create": (C.c_void_p, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "mux_batch_scheduler_destroy": (None, [C.c_void_p]),
    "mux_batch_scheduler_add_request": (C.c_int, [C.c_void_p, _I32P, C.c_int32, C.c_int32, C.c_int32]),
    "mux_batch_scheduler_try_batch": (C.c_int, [C.c_void_p, _I32P, C.c_int32, _I32P, C.c_int32, _I32P]),
    "mux_batch_scheduler_get_batch_info": (C.c_int, [C.c_void_p, _I32P, C.c_int32, _I32P, C.c_int64,
                                                     _I32P, C.c_int32, _I32P]),
    "mux_batch_scheduler_get_batch": (C.c_int, [C.c_void_p, _I32P, C.c_int32, _I32P, C.c_int64,
                                                _I32P, _I32P, C.c_int32, _I32P, C.c_int32,
                                                _I32P, C.c_int64, _I64P, C.c_int64]),
    "mux_batch_scheduler_get_batch_decode_layered": (C.c_int, [C.c_void_p, _I32P, C.c_int32, _I32P, C.c_int64,
                                                               _I32P, _I32P, C.c_int32, _I32P, C.c_int32,
                                                               _I32P, C.c_int64, _I64P, C.c_int64]),
    "mux_batch_scheduler_get_batch_mixed": (C.c_int, [C.POINTER(MixedModel), C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                                      _I32P, _I32P, _I32P, C.POINTER(C.c_float), _I32P, C.c_int64,
                                                      C.POINTER(MixedSpan), _I32P]),
    "mux_batch_scheduler_release_requests": (C.c_int, [C.c_void_p, _I32P, C.c_int32]),
    "mux_batch_scheduler_preempt_requests": (C.c_int32, [C.c_void_p, _I32P, C.c_int32]),
    "mux_batch_scheduler_prompt_info": (C.c_int32, [C.c_void_p, _I32P, C.c_int32]),
    "mux_batch_scheduler_batch_reqs": (C.c_int32, [C.c_void_p, _I32P, C.c_int32]),
    "mux_batch_scheduler_request_state": (C.c_int, [C.c_void_p, C.c_int32, _I32P]),
}

_lib = None


class MuxError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().mux_strerror(status).decode()
        if status == -9:
            msg += f" [cudaError {lib().mux_last_cuda_error()}]"
        super().__init__(f"{where}: {msg} (status {status})")


def lib() -> C.CDLL:
    """Loads the shared library once and types every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build the CUDA extension with `python -m muxserve_b200.build` "
            "(there is no CPU fallback for these ops)")
    handle = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(handle, name)
        except AttributeError as exc:
            raise ImportError(f"{LIB_PATH} does not export {name}; rebuild it") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    if handle.mux_abi_version() != ABI_VERSION:
        raise ImportError(f"{LIB_PATH} has ABI {handle.mux_abi_version()}, bindings expect {ABI_VERSION}; rebuild it")
    _lib = handle
    return handle


def check(status: int, where: str) -> int:
    if status < 0:
        raise MuxError(status, where)
    return status


def i32p(arr):
    """Pointer to the data of a C-contiguous int32 numpy array."""
    return arr.ctypes.data_as(_I32P)


def i64p(arr):
    return arr.ctypes.data_as(_I64P)
