"""ctypes declarations for libforja_cuda.so (see include/forja_cuda.h)."""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build


class FjTensor(C.Structure):
    _fields_ = [("buffer", C.c_uint64), ("dtype", C.c_uint32), ("rank", C.c_uint32), ("offset", C.c_uint64),
                ("shape", C.c_uint32 * 8), ("strides", C.c_uint64 * 8)]


class FjDispatch(C.Structure):
    _fields_ = [("op", C.c_uint32), ("n_inputs", C.c_uint32), ("n_outputs", C.c_uint32), ("u0", C.c_uint32), ("u1", C.c_uint32),
                ("u2", C.c_uint32), ("u3", C.c_uint32), ("f0", C.c_float), ("program", C.c_uint64),
                ("inputs", C.POINTER(FjTensor)), ("outputs", C.POINTER(FjTensor))]


class FjDeviceError(C.Structure):
    _fields_ = [("submission", C.c_uint64), ("dispatch", C.c_uint32), ("op", C.c_uint32), ("flag", C.c_uint32),
                ("value", C.c_uint32), ("code", C.c_int64)]


class FjDeviceInfo(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("sm_count", C.c_uint32), ("cc_major", C.c_uint32), ("cc_minor", C.c_uint32),
                ("total_memory", C.c_uint64), ("l2_bytes", C.c_uint64), ("max_smem_per_block", C.c_uint32)]


class FjDispatchProfile(C.Structure):
    _fields_ = [("op", C.c_uint32), ("kernels", C.c_uint32), ("ns", C.c_uint64), ("read_bytes", C.c_uint64), ("write_bytes", C.c_uint64), ("flops", C.c_uint64)]


class FjKvCheckpoint(C.Structure):
    _fields_ = [("pool", C.c_uint64), ("lane_epoch", C.c_uint64), ("logical_len", C.c_uint64)] + \
               [(n, C.c_uint32) for n in ("lane", "active", "has_tail", "index", "page", "immutable", "retained", "reserved")]


class FjGraphBinding(C.Structure):
    _fields_ = [("dispatch", C.c_uint32), ("field", C.c_uint32), ("param", C.c_uint32), ("scale", C.c_uint32), ("offset", C.c_uint64)]


class FjWeightTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_uint32), ("rank", C.c_uint32), ("shape", C.c_uint32 * 8), ("byte_offset", C.c_uint64),
                ("byte_len", C.c_uint64), ("dtype_aligned", C.c_uint32)]


class FjPackView(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("lanes", C.c_uint32), ("logical_lengths", C.c_uint64), ("query_starts", C.c_uint64),
                ("absolute_positions", C.c_uint64), ("activity", C.c_uint64), ("cu_seqlens", C.c_uint64), ("positions", C.c_uint64),
                ("slot_mapping", C.c_uint64), ("row_lane", C.c_uint64)]


class FjDenseConfig(C.Structure):
    _fields_ = [("dtype", C.c_uint32), ("layers", C.c_uint32), ("hidden", C.c_uint32), ("q_heads", C.c_uint32), ("kv_heads", C.c_uint32),
                ("head_dim", C.c_uint32), ("intermediate", C.c_uint32), ("vocab", C.c_uint32), ("qk_norm", C.c_uint32),
                ("eps", C.c_float), ("theta", C.c_float), ("max_rows", C.c_uint32)]


class FjDenseLayerWeights(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("input_norm", "wq", "wk", "wv", "q_norm", "k_norm", "wo", "post_norm", "w_gate", "w_up", "w_down")]


class FjQuantWeight(C.Structure):
    _fields_ = [("packed", C.c_uint64), ("scales", C.c_uint64), ("biases", C.c_uint64)]


class FjMoeConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("layers", "hidden", "q_heads", "kv_heads", "head_dim", "experts", "top_k", "expert_intermediate", "vocab",
                                          "group_size", "router_bits")] + [("eps", C.c_float), ("theta", C.c_float), ("max_rows", C.c_uint32), ("grouped_min_routes", C.c_uint32), ("stream_rows_per_expert", C.c_uint32), ("ep_return_bf16", C.c_uint32), ("ep_chunks", C.c_uint32)]


class FjMoeLayerWeights(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("input_norm", "q_norm", "k_norm", "post_norm")] + \
               [(n, FjQuantWeight) for n in ("qkv", "o", "router", "gate", "up", "down")]


SCHED_RESERVE_FN = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_uint64, C.c_uint64)

# Every symbol include/forja_cuda.h declares; the loader test checks that the library exports them all.
EXPORTS = [
    "fj_backend_create", "fj_backend_destroy", "fj_device_info", "fj_set_memory_limit", "fj_memory_usage", "fj_alloc",
    "fj_import_readonly", "fj_release", "fj_write", "fj_read", "fj_read_strided", "fj_buffer_device_ptr", "fj_program_prepare",
    "fj_program_info", "fj_program_classify", "fj_tensor_byte_span", "fj_submit", "fj_graph_prepare", "fj_graph_replay", "fj_graph_destroy", "fj_sub_wait", "fj_sub_gpu_time_ns", "fj_sub_completion_serial", "fj_sub_error",
    "fj_sub_kernel_launches", "fj_sub_profile", "fj_sub_destroy", "fj_synchronize", "fj_kernel_launch_count", "fj_timer_create",
    "fj_timer_record", "fj_timer_elapsed_ns", "fj_kvpool_create", "fj_kvpool_destroy", "fj_kvpool_reserve", "fj_kvpool_release",
    "fj_kvpool_read_table", "fj_kvpool_read_generations", "fj_kvpool_read_free", "fj_kvpool_read_refcounts", "fj_kvpool_fork", "fj_kvpool_cow_tail", "fj_kvpool_rewind_private", "fj_kvpool_checkpoint", "fj_kvpool_rollback", "fj_kvpool_checkpoint_drop", "fj_dense_copy_page", "fj_kvpool_tables_buffer",
    "fj_kvpool_generations_buffer", "fj_pack_step", "fj_dense_model_create", "fj_dense_model_destroy", "fj_dense_step",
    "fj_dense_step_stats", "fj_dense_graph_replay", "fj_dense_graph_stats", "fj_dense_kv_pages", "fj_dense_fill_kv", "fj_dense_profile_attention", "fj_dense_attention_time",
    "fj_paged_decode_attention_static", "fj_sched_create", "fj_sched_destroy", "fj_sched_set_prompt_chunk_multiple", "fj_sched_enqueue",
    "fj_sched_reconcile_active", "fj_sched_complete", "fj_sched_retry_admission", "fj_sched_admit", "fj_sched_admit_pages",
    "fj_sched_decode_bucket", "fj_sched_ready_prompt", "fj_sched_prompt_batch", "fj_sched_waiting", "fj_sched_active",
    "fj_safetensors_open", "fj_safetensors_open_all", "fj_safetensors_close", "fj_safetensors_tensor_count", "fj_safetensors_shard_name",
    "fj_safetensors_file_len", "fj_safetensors_data_start", "fj_safetensors_tensor", "fj_safetensors_find", "fj_weights_last_error",
    "fj_safetensors_import", "fj_safetensors_view", "fj_safetensors_quant_views",
    "fj_prompt_chunk_work", "fj_prompt_chunk_merged_work", "fj_reservations_fit", "fj_prefill_plan",
    "fj_ep_load", "fj_ep_unique_id", "fj_ep_create", "fj_ep_destroy", "fj_ep_all_to_all", "fj_ep_set_timeout", "fj_ep_poll_selftest", "fj_moe_ep_export", "fj_moe_ep_connect", "fj_moe_ep_direct", "fj_moe_ep_disconnect", "fj_moe_ep_wait_polls", "fj_moe_ep_return_mode", "fj_moe_ep_received", "fj_moe_uniform_routing",
    "fj_ep_wait_selftest", "fj_moe_model_create", "fj_moe_model_destroy",
    "fj_moe_step", "fj_moe_step_stats", "fj_fill_random", "fj_tcgen05_wait_giveups", "fj_moe_capture_routes", "fj_moe_read_routes", "fj_moe_phase_timing", "fj_moe_read_phase_ms",
]

_lib = None


def library_path() -> str:
    return _build.OUTPUT


def load():
    """Loads the in-tree library, building it first when sources are newer. Raises when it cannot
    be built or loaded: there is no fallback implementation."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.OUTPUT
    if _build.needs_build():
        if os.environ.get("FORJA_B200_NO_BUILD"):
            if not os.path.exists(path):
                raise RuntimeError(f"{path} is missing and FORJA_B200_NO_BUILD is set")
        else:
            _build.build()
    # Kernels are loaded when the context is created, not at their first launch: a first launch that has to load its module
    # synchronises the whole device, and with two streams of one GPU in flight (two micro-batches of an expert-parallel model)
    # that load would wait for the other stream's bounded wait on a peer, which in turn waits for this rank. The setting only
    # takes effect if CUDA has not been initialised in this process yet.
    os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
    lib = C.CDLL(path)
    for name in EXPORTS:
        getattr(lib, name)
    lib.fj_sub_completion_serial.restype = C.c_uint64
    lib.fj_kernel_launch_count.restype = C.c_uint64
    lib.fj_sub_kernel_launches.restype = C.c_uint32
    lib.fj_kvpool_tables_buffer.restype = C.c_uint64
    lib.fj_kvpool_generations_buffer.restype = C.c_uint64
    lib.fj_backend_destroy.restype = None
    lib.fj_sub_destroy.restype = None
    lib.fj_kvpool_destroy.restype = None
    lib.fj_graph_destroy.restype = None
    lib.fj_graph_destroy.argtypes = [C.c_void_p]
    lib.fj_dense_model_destroy.restype = None
    for name in ("fj_backend_destroy", "fj_sub_destroy", "fj_kvpool_destroy", "fj_dense_model_destroy", "fj_sub_completion_serial",
                 "fj_kernel_launch_count", "fj_sub_kernel_launches", "fj_kvpool_tables_buffer", "fj_kvpool_generations_buffer"):
        getattr(lib, name).argtypes = [C.c_void_p]
    P, U32, U64, I32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32
    argtypes = {
        "fj_backend_create": [I32, U64, P], "fj_device_info": [P, P], "fj_set_memory_limit": [P, U64], "fj_memory_usage": [P, P, P],
        "fj_alloc": [P, U64, P], "fj_import_readonly": [P, P, U64, P], "fj_release": [P, U64], "fj_write": [P, U64, U64, P, U64],
        "fj_read": [P, U64, U64, P, U64], "fj_read_strided": [P, P, P], "fj_buffer_device_ptr": [P, U64, P, P],
        "fj_program_prepare": [P, U32, P, U32, P, U32, P], "fj_program_info": [P, U64, P, P], "fj_program_classify": [U32, P, U32, P, U32, P, P], "fj_tensor_byte_span": [P, P, P], "fj_submit": [P, P, U32, U32, P], "fj_graph_prepare": [P, P, U32, P, U32, U32, P], "fj_graph_replay": [P, P, U32, U32, P],
        "fj_sub_wait": [P, U64], "fj_sub_gpu_time_ns": [P, P], "fj_sub_error": [P, P], "fj_sub_profile": [P, P, U32, P],
        "fj_synchronize": [P], "fj_timer_create": [P, P], "fj_timer_record": [P, U64], "fj_timer_elapsed_ns": [P, U64, U64, P],
        "fj_kvpool_create": [P, U32, U32, U32, U32, P], "fj_kvpool_reserve": [P, P, P, U32, P], "fj_kvpool_release": [P, P, U32],
        "fj_kvpool_read_table": [P, U32, P], "fj_kvpool_read_generations": [P, P], "fj_kvpool_read_free": [P, P, U32, P],
        "fj_kvpool_read_refcounts": [P, P], "fj_kvpool_fork": [P, U32, U64, U32, U64, U64], "fj_kvpool_cow_tail": [P, U32, U64, P], "fj_kvpool_rewind_private": [P, U32, U64, U64], "fj_kvpool_checkpoint": [P, U32, U64, P], "fj_kvpool_rollback": [P, U32, P, P], "fj_kvpool_checkpoint_drop": [P, P], "fj_dense_copy_page": [P, U32, U32, U32],
        "fj_pack_step": [P, P, P, U32, P], "fj_dense_model_create": [P, P, U64, U64, P, P, P], "fj_dense_step": [P, P, P, U64],
        "fj_dense_step_stats": [P, P, P], "fj_dense_graph_replay": [P, U32], "fj_dense_graph_stats": [P, P, P, P], "fj_dense_kv_pages": [P, U32, U32, U32, U32, P, U32], "fj_dense_fill_kv": [P, U64], "fj_dense_profile_attention": [P, U32],
        "fj_dense_attention_time": [P, P, P],
        "fj_paged_decode_attention_static": [P, P, P, P, P, P, P, P, U32, U32, U32, U32, U32, U32, C.c_float, P],
    }
    for name, types in argtypes.items():
        fn = getattr(lib, name)
        fn.argtypes = types
        fn.restype = C.c_int32
    # host scheduler: (argtypes, restype)
    sched = {
        "fj_sched_create": ([P, U32, U64, U64, U32, U32, P], I32), "fj_sched_destroy": ([P], None),
        "fj_sched_set_prompt_chunk_multiple": ([P, U32], None), "fj_sched_enqueue": ([P, U64, U64], None),
        "fj_sched_reconcile_active": ([P, U64], None), "fj_sched_complete": ([P, U64], None),
        "fj_sched_retry_admission": ([P, U64, U64], None), "fj_sched_admit": ([P, SCHED_RESERVE_FN, P, P, U64], U64),
        "fj_sched_admit_pages": ([P, U32, P, P, U64], U64), "fj_sched_decode_bucket": ([P, P, U64], C.c_int64),
        "fj_sched_ready_prompt": ([P, U64, U32], None), "fj_sched_prompt_batch": ([P, I32, P, P, U64], U64),
        "fj_sched_waiting": ([P], U64), "fj_sched_active": ([P], U64),
        "fj_safetensors_open": ([C.c_char_p, P], I32), "fj_safetensors_open_all": ([C.c_char_p, P, U32, P], I32), "fj_safetensors_close": ([P], None),
        "fj_safetensors_tensor_count": ([P], U32), "fj_safetensors_shard_name": ([P], C.c_char_p), "fj_safetensors_file_len": ([P], U64),
        "fj_safetensors_data_start": ([P], U64), "fj_safetensors_tensor": ([P, U32, P], I32), "fj_safetensors_find": ([P, C.c_char_p, P], I32),
        "fj_weights_last_error": ([], C.c_char_p), "fj_safetensors_import": ([P, P, P], I32), "fj_safetensors_view": ([P, C.c_char_p, U64, P], I32),
        "fj_safetensors_quant_views": ([P, C.c_char_p, U64, U32, U32, P, P, P], I32),
        "fj_prompt_chunk_work": ([U32, U32, U32], U32), "fj_prompt_chunk_merged_work": ([U32, U32, U32], U32),
        "fj_reservations_fit": ([U32, U32, P, U64], I32), "fj_prefill_plan": ([U32, U32, U32, P, U64], U64),
        "fj_ep_load": ([C.c_char_p], I32), "fj_ep_unique_id": ([P], I32), "fj_ep_create": ([P, P, U32, U32, P], I32), "fj_ep_destroy": ([P], None),
        "fj_ep_all_to_all": ([P, U64, U64, U64], I32), "fj_ep_set_timeout": ([P, U64], I32), "fj_ep_poll_selftest": ([U64, U64, U64, P], I32), "fj_moe_ep_export": ([P, P], I32), "fj_moe_ep_connect": ([P, P], I32), "fj_moe_ep_direct": ([P, U32], I32),
        "fj_moe_ep_disconnect": ([P], I32), "fj_moe_ep_wait_polls": ([P, U32], I32), "fj_moe_ep_return_mode": ([P, U32], I32), "fj_moe_ep_received": ([P, P, U32], I32), "fj_moe_uniform_routing": ([P, U32], I32), "fj_ep_wait_selftest": ([P, U32], I32), "fj_moe_model_create": ([P, P, P, U64, P, P, P, P, P], I32),
        "fj_moe_model_destroy": ([P], None), "fj_moe_step": ([P, P, P, U64], I32), "fj_moe_step_stats": ([P, P, P], I32),
        "fj_fill_random": ([P, U64, U64, U64, U32, U64, C.c_float, C.c_float], I32), "fj_tcgen05_wait_giveups": ([P, P], I32), "fj_moe_capture_routes": ([P, U32], I32), "fj_moe_read_routes": ([P, U32, U32, P, P], I32), "fj_moe_phase_timing": ([P, U32], I32), "fj_moe_read_phase_ms": ([P, P], I32),
    }
    for name, (types, restype) in sched.items():
        fn = getattr(lib, name)
        fn.argtypes = types
        fn.restype = restype
    _lib = lib
    return lib
