"""ctypes declarations for libloom_b200.so (the C ABI in include/loom_b200.h).

Nothing here computes: every call goes into the CUDA library.  Loading fails loudly when the
library has not been built; there is no CPU fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, c_char, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t,
                    c_uint8, c_uint16, c_uint32, c_uint64, c_void_p)

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("LOOM_B200_LIBRARY", os.path.join(HERE, "libloom_b200.so"))

HEAD_DIM = 128
PAGE_SIZE = 16
PARTIAL_STATE_WIDTH = 130
APPEND_MAX_TOKENS = 64

F32, F16, BF16, I32, U8 = 0, 1, 2, 3, 4
ACCESS_READ, ACCESS_WRITE, ACCESS_READ_WRITE = 0, 1, 2


class ErrorInfo(ctypes.Structure):
    _fields_ = [("status", c_int32), ("name", c_char * 48), ("operand", c_char * 32),
                ("a", c_int64), ("b", c_int64), ("c", c_int64), ("d", c_int64),
                ("message", c_char * 256)]


class PagedSpec(ctypes.Structure):
    _fields_ = [("batch_size", c_size_t), ("max_num_pages", c_size_t),
                ("num_query_heads", c_size_t), ("num_kv_heads", c_size_t),
                ("softmax_scale", c_float)]


class AppendTokensSpec(ctypes.Structure):
    _fields_ = [("paged", PagedSpec), ("tokens", c_size_t), ("max_tokens", c_size_t)]


class RopePosIdsSpec(ctypes.Structure):
    _fields_ = [("tokens", c_size_t), ("query_heads", c_size_t), ("key_heads", c_size_t),
                ("head_dim", c_size_t), ("rotary_dim", c_size_t), ("rope_scale", c_float),
                ("rope_theta", c_float)]


class Handle(ctypes.Structure):
    _fields_ = [("set_id", c_uint64), ("slot", c_uint32), ("dtype", c_uint8),
                ("access", c_uint8), ("reserved", c_uint16)]


class DecodeOptions(ctypes.Structure):
    _fields_ = [("partitions", c_uint32), ("heads_per_cta", c_uint32), ("balanced", c_uint32),
                ("balanced_ctas", c_uint32), ("indices_capacity", c_uint32),
                ("wait_limit_us", c_uint32), ("test_skip_page", c_uint32),
                ("cluster", c_uint32), ("merge_in_kernel", c_uint32), ("max_stages", c_uint32),
                ("producer_warps", c_uint32), ("reserved", c_uint32)]


class AppendOptions(ctypes.Structure):
    _fields_ = [("indices_capacity", c_uint32), ("one_command", c_uint32),
                ("reserved", c_uint32 * 2)]


class DecodePlanInfo(ctypes.Structure):
    _fields_ = [("algorithm", c_int32), ("partitions", c_uint32), ("heads_per_cta", c_uint32),
                ("q_tiles", c_uint32), ("q_blocks", c_uint32), ("pages_per_stage", c_uint32),
                ("stages", c_uint32), ("grid", c_uint32), ("block", c_uint32),
                ("shared_bytes", c_uint32), ("merge_grid", c_uint32), ("merge_block", c_uint32),
                ("commands", c_uint32), ("workspace_numel", c_size_t),
                ("workspace_bytes", c_size_t), ("merged_in_kernel", c_uint32), ("reserved", c_uint32)]


class DecodeArgs(ctypes.Structure):
    _fields_ = [(name, Handle) for name in
                ("query", "key_pages", "value_pages", "page_indptr", "page_indices",
                 "last_page_len", "output", "lse", "workspace")]


class GatherLayout(ctypes.Structure):
    _fields_ = [("total_requests", c_size_t), ("gathered_query_heads", c_size_t),
                ("head_offset", c_size_t), ("defer_wait", c_uint32), ("reserved", c_uint32)]


class DecodeGatherArgs(ctypes.Structure):
    _fields_ = [("decode", DecodeArgs), ("dest_rows", Handle)]


class OutputGatherArgs(ctypes.Structure):
    _fields_ = [("local", Handle), ("gathered", Handle)]


class AppendArgs(ctypes.Structure):
    _fields_ = [(name, Handle) for name in
                ("query", "key", "value", "batch_indices", "positions", "page_indptr",
                 "page_indices", "last_page_len", "query_output", "key_pages", "value_pages",
                 "workspace")]


class StateMergeArgs(ctypes.Structure):
    _fields_ = [("states", Handle), ("output", Handle), ("lse", Handle)]


class RopePosIdsArgs(ctypes.Structure):
    _fields_ = [(name, Handle) for name in
                ("query", "key", "position_ids", "query_output", "key_output")]


class AppendPlanInfo(ctypes.Structure):
    _fields_ = [("explicit_tokens", c_int32), ("tokens", c_uint32), ("grid", c_uint32),
                ("block", c_uint32), ("shared_bytes", c_uint32), ("commands", c_uint32),
                ("workspace_numel", c_size_t)]


class PrefillSpec(ctypes.Structure):
    _fields_ = [("batch_size", c_size_t), ("nnz_qo", c_size_t), ("max_num_pages", c_size_t),
                ("num_query_heads", c_size_t), ("num_kv_heads", c_size_t),
                ("softmax_scale", c_float)]


class PrefillOptions(ctypes.Structure):
    _fields_ = [("q_tiles", c_uint32), ("indices_capacity", c_uint32), ("algorithm", c_uint32),
                ("partitions", c_uint32), ("wait_limit_us", c_uint32),
                ("test_lost_copy", c_uint32), ("reserved", c_uint32 * 2)]


class PrefillPlanInfo(ctypes.Structure):
    _fields_ = [("algorithm", c_int32), ("q_tiles", c_uint32), ("pages_per_stage", c_uint32),
                ("stages", c_uint32), ("rows_per_cta", c_uint32), ("tiles", c_uint32),
                ("grid", c_uint32), ("block", c_uint32), ("shared_bytes", c_uint32),
                ("commands", c_uint32), ("partitions", c_uint32), ("merge_grid", c_uint32),
                ("merge_block", c_uint32), ("min_chunk_blocks", c_uint32),
                ("workspace_numel", c_size_t)]


class PrefillArgs(ctypes.Structure):
    _fields_ = [(name, Handle) for name in
                ("query", "key_pages", "value_pages", "qo_indptr", "page_indptr", "page_indices",
                 "last_page_len", "output", "lse", "workspace")]


RECORD_FN = ctypes.CFUNCTYPE(c_int32, c_void_p, c_void_p)

_I32P = POINTER(c_int32)

# name -> (restype, argtypes); every symbol include/loom_b200.h declares
SIGNATURES = {
    "lb_status_name": (c_char_p, [c_int32]),
    "lb_last_error": (None, [POINTER(ErrorInfo)]),
    "lb_build_info": (c_char_p, []),
    "lb_paged_spec_new": (c_int32, [c_size_t] * 6 + [POINTER(PagedSpec)]),
    "lb_paged_spec_query_numel": (c_size_t, [POINTER(PagedSpec)]),
    "lb_paged_spec_kv_pages_numel": (c_size_t, [POINTER(PagedSpec)]),
    "lb_paged_spec_lse_numel": (c_size_t, [POINTER(PagedSpec)]),
    "lb_paged_spec_gqa_group_size": (c_size_t, [POINTER(PagedSpec)]),
    "lb_paged_spec_kv_head_for_query_head": (c_int64, [POINTER(PagedSpec), c_size_t]),
    "lb_paged_spec_validate_page_table": (c_int32, [POINTER(PagedSpec), _I32P, c_size_t, _I32P,
                                                    c_size_t, _I32P, c_size_t]),
    "lb_page_table_request_kv_len": (c_int, [POINTER(PagedSpec), _I32P, _I32P, c_size_t,
                                             POINTER(c_size_t)]),
    "lb_page_table_physical_page_for_token": (c_int, [POINTER(PagedSpec), _I32P, _I32P, _I32P,
                                                      c_size_t, c_size_t, POINTER(c_size_t),
                                                      POINTER(c_size_t)]),
    "lb_append_spec_validate_page_table": (c_int32, [POINTER(PagedSpec), _I32P, c_size_t, _I32P,
                                                     c_size_t, _I32P, c_size_t]),
    "lb_append_tokens_spec_new": (c_int32, [c_size_t] * 7 + [POINTER(AppendTokensSpec)]),
    "lb_append_tokens_spec_new_extended": (c_int32, [c_size_t] * 7 + [POINTER(AppendTokensSpec)]),
    "lb_append_extended_max_tokens": (c_size_t, []),
    "lb_append_tokens_spec_validate_metadata": (
        c_int32, [POINTER(AppendTokensSpec), _I32P, c_size_t, _I32P, c_size_t, _I32P, c_size_t,
                  _I32P, c_size_t, _I32P, c_size_t, POINTER(c_int64)]),
    "lb_split_partition_range": (c_int, [c_size_t, c_size_t, c_size_t, POINTER(c_size_t),
                                         POINTER(c_size_t)]),
    "lb_paged_split_workspace_numel": (c_int32, [POINTER(PagedSpec), c_size_t,
                                                 POINTER(c_size_t)]),
    "lb_paged_split_state_offset": (c_int64, [POINTER(PagedSpec), c_size_t, c_size_t, c_size_t,
                                              c_size_t]),
    "lb_handle_read": (Handle, [Handle]),
    "lb_handle_write": (Handle, [Handle]),
    "lb_queue_create": (c_int32, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "lb_queue_destroy": (None, [c_void_p]),
    "lb_queue_stream": (c_void_p, [c_void_p]),
    "lb_queue_max_commands": (c_size_t, [c_void_p]),
    "lb_queue_is_poisoned": (c_int, [c_void_p]),
    "lb_queue_bindings": (c_int32, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "lb_queue_begin": (c_int32, [c_void_p, c_void_p, POINTER(c_void_p)]),
    "lb_bindings_len": (c_size_t, [c_void_p]),
    "lb_bindings_capacity": (c_size_t, [c_void_p]),
    "lb_bindings_destroy": (None, [c_void_p]),
    "lb_bind_read": (c_int32, [c_void_p, c_int, c_void_p, c_size_t, POINTER(Handle)]),
    "lb_bind_read_write": (c_int32, [c_void_p, c_int, c_void_p, c_size_t, POINTER(Handle)]),
    "lb_take_read_write": (c_int32, [c_void_p, Handle, POINTER(c_void_p), POINTER(c_size_t)]),
    "lb_scope_finish": (c_int32, [c_void_p, POINTER(c_void_p)]),
    "lb_scope_abandon": (None, [c_void_p]),
    "lb_scope_submitted": (c_size_t, [c_void_p]),
    "lb_completion_is_complete": (c_int32, [c_void_p, POINTER(c_int)]),
    "lb_completion_submitted": (c_size_t, [c_void_p]),
    "lb_completion_wait": (c_int32, [c_void_p, POINTER(c_void_p)]),
    "lb_completion_abandon": (None, [c_void_p]),
    "lb_decode_provider_load": (c_int32, [c_int, POINTER(c_void_p)]),
    "lb_decode_provider_destroy": (None, [c_void_p]),
    "lb_decode_provider_device_status": (c_int32, [c_void_p, POINTER(c_int32)]),
    "lb_paged_decode_plan_create": (c_int32, [c_void_p, POINTER(PagedSpec),
                                              POINTER(DecodeOptions), POINTER(c_void_p)]),
    "lb_paged_decode_plan_destroy": (None, [c_void_p]),
    "lb_paged_decode_plan_info_get": (c_int32, [c_void_p, POINTER(PagedSpec),
                                                POINTER(DecodePlanInfo)]),
    "lb_paged_decode_enqueue": (c_int32, [c_void_p, c_void_p, POINTER(DecodeArgs)]),
    "lb_paged_decode_choose": (c_int32, [POINTER(PagedSpec), c_uint32, POINTER(DecodeOptions),
                                         POINTER(DecodePlanInfo)]),
    "lb_paged_decode_split_noalloc_max_states": (c_size_t, []),
    "lb_paged_decode_split_noalloc": (c_int32, [POINTER(PagedSpec), c_uint32, c_void_p, c_void_p,
                                                c_void_p, c_void_p, _I32P, _I32P, c_size_t, _I32P,
                                                c_void_p, c_void_p]),
    "lb_paged_decode_split_noalloc_status": (c_int32, [c_int, POINTER(c_int32)]),
    "lb_peer_group_unique_id": (c_int32, [POINTER(ctypes.c_uint8)]),
    "lb_peer_group_create": (c_int32, [c_int, c_int, c_int, POINTER(ctypes.c_uint8),
                                       POINTER(c_void_p)]),
    "lb_peer_group_destroy": (None, [c_void_p]),
    "lb_peer_group_rank": (c_int, [c_void_p]),
    "lb_peer_group_world": (c_int, [c_void_p]),
    "lb_peer_buffer_create": (c_int32, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "lb_peer_buffer_destroy": (None, [c_void_p]),
    "lb_peer_buffer_local": (c_void_p, [c_void_p]),
    "lb_peer_buffer_bytes": (c_size_t, [c_void_p]),
    "lb_output_gather_plan_create": (c_int32, [c_void_p, c_int, POINTER(c_size_t), c_size_t,
                                               POINTER(c_void_p)]),
    "lb_output_gather_plan_destroy": (None, [c_void_p]),
    "lb_output_gather_enqueue": (c_int32, [c_void_p, c_void_p, POINTER(OutputGatherArgs)]),
    "lb_paged_decode_enqueue_gathered": (c_int32, [c_void_p, c_void_p, POINTER(DecodeGatherArgs),
                                                   POINTER(GatherLayout), c_void_p, c_void_p,
                                                   c_void_p]),
    "lb_rope_provider_load": (c_int32, [c_int, POINTER(c_void_p)]),
    "lb_rope_provider_destroy": (None, [c_void_p]),
    "lb_rope_provider_device_status": (c_int32, [c_void_p, POINTER(c_int32)]),
    "lb_rope_append_plan_create": (c_int32, [c_void_p, POINTER(PagedSpec), POINTER(c_void_p)]),
    "lb_rope_append_tokens_plan_create": (c_int32, [c_void_p, POINTER(AppendTokensSpec),
                                                    POINTER(c_void_p)]),
    "lb_rope_append_plan_create_with": (c_int32, [c_void_p, POINTER(PagedSpec),
                                                  POINTER(AppendOptions), POINTER(c_void_p)]),
    "lb_rope_append_tokens_plan_create_with": (c_int32, [c_void_p, POINTER(AppendTokensSpec),
                                                         POINTER(AppendOptions),
                                                         POINTER(c_void_p)]),
    "lb_rope_append_plan_destroy": (None, [c_void_p]),
    "lb_rope_append_plan_info_get": (c_int32, [c_void_p, POINTER(AppendPlanInfo)]),
    "lb_rope_append_enqueue": (c_int32, [c_void_p, c_void_p, POINTER(AppendArgs)]),
    "lb_state_merge_plan_create": (c_int32, [c_void_p, c_size_t, c_size_t, POINTER(c_void_p)]),
    "lb_state_merge_plan_destroy": (None, [c_void_p]),
    "lb_state_merge_enqueue": (c_int32, [c_void_p, c_void_p, POINTER(StateMergeArgs)]),
    "lb_rope_pos_ids_spec_new": (c_int32, [c_size_t] * 5 + [c_float, c_float,
                                                            POINTER(RopePosIdsSpec)]),
    "lb_rope_pos_ids_spec_query_numel": (c_size_t, [POINTER(RopePosIdsSpec)]),
    "lb_rope_pos_ids_spec_key_numel": (c_size_t, [POINTER(RopePosIdsSpec)]),
    "lb_rope_pos_ids_plan_create": (c_int32, [c_void_p, POINTER(RopePosIdsSpec),
                                              POINTER(c_void_p)]),
    "lb_rope_pos_ids_plan_destroy": (None, [c_void_p]),
    "lb_rope_pos_ids_enqueue": (c_int32, [c_void_p, c_void_p, POINTER(RopePosIdsArgs)]),
    "lb_prefill_spec_new": (c_int32, [c_size_t] * 7 + [POINTER(PrefillSpec)]),
    "lb_prefill_spec_query_numel": (c_size_t, [POINTER(PrefillSpec)]),
    "lb_prefill_spec_kv_pages_numel": (c_size_t, [POINTER(PrefillSpec)]),
    "lb_prefill_spec_lse_numel": (c_size_t, [POINTER(PrefillSpec)]),
    "lb_prefill_spec_validate_metadata": (c_int32, [POINTER(PrefillSpec), _I32P, c_size_t, _I32P,
                                                    c_size_t, _I32P, c_size_t, _I32P, c_size_t]),
    "lb_prefill_metadata_causal_kv_end": (c_int, [POINTER(PrefillSpec), _I32P, _I32P, _I32P,
                                                  c_size_t, c_size_t, POINTER(c_size_t)]),
    "lb_prefill_provider_load": (c_int32, [c_int, POINTER(c_void_p)]),
    "lb_prefill_provider_destroy": (None, [c_void_p]),
    "lb_prefill_provider_device_status": (c_int32, [c_void_p, POINTER(c_int32)]),
    "lb_paged_prefill_plan_create": (c_int32, [c_void_p, POINTER(PrefillSpec),
                                               POINTER(PrefillOptions), POINTER(c_void_p)]),
    "lb_paged_prefill_plan_destroy": (None, [c_void_p]),
    "lb_paged_prefill_plan_info_get": (c_int32, [c_void_p, POINTER(PrefillSpec),
                                                 POINTER(PrefillPlanInfo)]),
    "lb_paged_prefill_enqueue": (c_int32, [c_void_p, c_void_p, POINTER(PrefillArgs)]),
    "lb_paged_prefill_choose": (c_int32, [POINTER(PrefillSpec), c_uint32, POINTER(PrefillOptions),
                                          POINTER(PrefillPlanInfo)]),
    "lb_graph_queue_create": (c_int32, [c_int, c_size_t, POINTER(c_void_p)]),
    "lb_graph_queue_destroy": (None, [c_void_p]),
    "lb_graph_queue_bindings": (c_int32, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "lb_graph_capture": (c_int32, [c_void_p, c_void_p, RECORD_FN, c_void_p, POINTER(c_void_p)]),
    "lb_captured_graph_commands": (c_size_t, [c_void_p]),
    "lb_captured_graph_instantiate": (c_int32, [c_void_p, POINTER(c_void_p)]),
    "lb_captured_graph_destroy": (None, [c_void_p]),
    "lb_graph_exec_commands": (c_size_t, [c_void_p]),
    "lb_graph_exec_launches": (c_uint64, [c_void_p]),
    "lb_graph_exec_launch": (c_int32, [c_void_p, POINTER(c_void_p)]),
    "lb_graph_exec_measure_launch_ms": (c_int32, [c_void_p, POINTER(c_float)]),
    "lb_graph_exec_into_bindings": (c_int32, [c_void_p, POINTER(c_void_p)]),
    "lb_graph_exec_destroy": (None, [c_void_p]),
    "lb_graph_completion_launch_index": (c_uint64, [c_void_p]),
    "lb_graph_completion_is_complete": (c_int32, [c_void_p, POINTER(c_int)]),
    "lb_graph_completion_wait": (c_int32, [c_void_p]),
    "lb_graph_completion_abandon": (None, [c_void_p]),
    "lb_test_use_fake_driver": (None, [c_int, c_int]),
    "lb_test_fake_fail": (None, [c_char_p, c_int, c_int]),
    "lb_test_launch_count": (c_uint64, []),
    "lb_test_noalloc_is_set_up": (c_int, [c_int]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Loads the CUDA library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m loom_kernels_b200.build` "
                "(nvcc, sm_100a). There is no CPU fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib
