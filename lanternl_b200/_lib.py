"""ctypes binding of luaTL.so: the same C ABI the LuaJIT shim binds with ffi.cdef.

Nothing here computes.  Loading fails loudly when the shared library is missing; every
status other than 0 raises LuaTLError with the library's message (the equivalent of the
reference's ck(), ai/gpu/luaTL.lua:240-246).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "luaTL.so")

F32, F16, BF16 = 0, 1, 2
STATUS_NAME = {0: "OK", -1: "NULL_POINTER", -2: "SHAPE", -3: "DTYPE", -4: "CUDA", -5: "OUT_OF_MEMORY",
               -6: "BAD_ARGUMENT", -7: "CAPACITY", -8: "UNSUPPORTED"}


class LuaTLError(RuntimeError):
    def __init__(self, ctx, status, msg):
        self.status = status
        super().__init__(f"luaTL[{ctx}]: {msg or 'unspecified backend error'} ({STATUS_NAME.get(status, status)})")


class Tensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("nelem", C.c_uint64), ("nbytes", C.c_uint64),
                ("rows", C.c_int32), ("cols", C.c_int32), ("dtype", C.c_int32), ("owns", C.c_int32),
                ("pool", C.c_void_p), ("device", C.c_int32), ("flags", C.c_int32)]


class Op(C.Structure):
    _fields_ = ([("op", C.c_int32), ("dtype", C.c_int32), ("act", C.c_int32), ("pre", C.c_int32)]
                + [(f"i{k}", C.c_int32) for k in range(8)]
                + [(f"f{k}", C.c_float) for k in range(8)]
                + [(f"s{k}", C.c_int64) for k in range(9)]
                + [("n", C.c_uint64)]
                + [(f"p{k}", C.c_void_p) for k in range(8)])


class Prog(C.Structure):
    _fields_ = [("ops", C.POINTER(Op)), ("count", C.c_int32), ("capacity", C.c_int32),
                ("flags", C.c_int32), ("status", C.c_int32), ("stream", C.c_void_p),
                ("ev_start", C.c_void_p), ("ev_stop", C.c_void_p), ("graph", C.c_void_p),
                ("graph_exec", C.c_void_p), ("last_ms", C.c_double), ("total_runs", C.c_uint64),
                ("total_ops", C.c_uint64), ("owns_stream", C.c_int32), ("timing", C.c_int32),
                ("captured", C.c_int32), ("capturing", C.c_int32)]


class PoolStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("bytes_reserved", "bytes_in_use", "peak_in_use", "block_count",
                                          "free_block_count", "n_alloc", "n_free", "n_cuda_malloc",
                                          "n_cuda_free", "n_cache_hit", "n_cache_miss", "n_trim")]


class DevInfo(C.Structure):
    _fields_ = ([(n, C.c_int32) for n in (
        "device", "major", "minor", "mp_count", "warp_size", "max_threads_per_block", "max_threads_per_mp",
        "max_blocks_per_mp", "regs_per_block", "regs_per_mp", "clock_khz", "memory_clock_khz",
        "memory_bus_width", "l2_cache_size", "concurrent_kernels", "async_engines", "unified_addressing",
        "cooperative_launch", "has_tensor_cores", "has_fp16", "has_bf16", "ecc_enabled", "integrated",
        "cores_per_mp")]
        + [(n, C.c_uint64) for n in ("shared_mem_per_block", "shared_mem_per_mp", "total_global_mem",
                                     "free_global_mem")]
        + [(n, C.c_double) for n in ("peak_mem_bandwidth_gbs", "peak_fp32_gflops", "peak_fp16_gflops")]
        + [("name", C.c_char * 256)])


class Plan(C.Structure):
    _fields_ = ([(n, C.c_int32) for n in ("tm", "tn", "tk", "block_x", "block_y", "grid_x", "grid_y", "shmem_bytes",
                                          "kernel_id", "unroll", "use_tensor_core", "from_cache")]
                + [("measured_ms", C.c_double)])


class Arena(C.Structure):
    _fields_ = [("base", C.c_void_p), ("capacity", C.c_uint64), ("offset", C.c_uint64), ("peak", C.c_uint64),
                ("alignment", C.c_uint64), ("pool", C.c_void_p)]


class Cmd(C.Structure):
    _fields_ = ([("op", C.c_int32), ("dtype", C.c_int32), ("act", C.c_int32), ("flags", C.c_int32)]
                + [(f"i{k}", C.c_int32) for k in range(4)]
                + [(f"f{k}", C.c_float) for k in range(6)]
                + [("n", C.c_uint64)]
                + [(f"p{k}", C.c_void_p) for k in range(6)])


class Pipeline(C.Structure):
    _fields_ = [("cmds", C.POINTER(Cmd)), ("count", C.c_int32), ("capacity", C.c_int32), ("flags", C.c_int32),
                ("status", C.c_int32), ("stream", C.c_void_p), ("ev_start", C.c_void_p), ("ev_stop", C.c_void_p),
                ("last_ms", C.c_double), ("total_runs", C.c_uint64), ("total_ops", C.c_uint64),
                ("owns_stream", C.c_int32), ("timing", C.c_int32)]


class LmConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("vocab", "dim", "layers", "heads", "ffn", "max_seq", "batch",
                                         "decode_batch", "tie", "dtype", "use_rope", "rope_interleaved",
                                         "causal", "kv_splits")] + [("eps", C.c_float), ("rope_base", C.c_float)]


class LmResult(C.Structure):
    _fields_ = [("loss", C.c_float), ("grad_norm", C.c_float), ("correct", C.c_int32),
                ("valid", C.c_int32), ("finite", C.c_int32), ("step_ms", C.c_float)]


class LmTrainArgs(C.Structure):
    _fields_ = [("optimizer", C.c_int32), ("step", C.c_int32), ("lr", C.c_float), ("weight_decay", C.c_float),
                ("clip_norm", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("adam_eps", C.c_float),
                ("valid_global", C.c_int32), ("no_update", C.c_int32), ("accumulate", C.c_int32),
                ("skip_allreduce", C.c_int32)]


_vp, _i, _f, _u64, _i64, _ll = C.c_void_p, C.c_int, C.c_float, C.c_uint64, C.c_int64, C.c_longlong
_cp = C.c_char_p

# name -> (restype, argtypes).  int-returning entries are status-checked by call().
SIGNATURES = {
    "luaTL_version": (_cp, []), "luaTL_train_version": (_cp, []), "luaTL_set_verbose": (None, [_i]),
    "luaTL_init": (_i, [_i]), "luaTL_shutdown": (None, []), "luaTL_shutdown_safe": (None, []),
    "luaTL_finalize": (None, []), "luaTL_epoch": (_u64, []), "luaTL_device_name": (_cp, []),
    "luaTL_get_last_error": (_cp, []), "luaTL_has_error": (_i, []), "luaTL_clear_error": (None, []),
    "luaTL_sync": (_i, []), "luaTL_get_devinfo": (_i, [_i, C.POINTER(DevInfo)]),
    "luaTL_mem_info": (_i, [C.POINTER(_u64), C.POINTER(_u64)]),
    "luaTL_stream_create": (_vp, [_i]), "luaTL_stream_destroy": (None, [_vp]), "luaTL_stream_sync": (_i, [_vp]),
    "luaTL_host_alloc_pinned": (_vp, [_u64]), "luaTL_host_free_pinned": (None, [_vp]),
    "luaTL_pool_create": (_vp, [_i]), "luaTL_pool_destroy": (None, [_vp]),
    "luaTL_arena_create": (C.POINTER(Arena), [_vp, _u64]), "luaTL_arena_destroy": (None, [C.POINTER(Arena)]),
    "luaTL_arena_alloc": (_vp, [C.POINTER(Arena), _u64]), "luaTL_arena_reset": (None, [C.POINTER(Arena)]),
    "luaTL_gpu_malloc": (_vp, [_u64]), "luaTL_gpu_free": (None, [_vp]),
    "luaTL_to_gpu": (_i, [_vp, _vp, _u64]), "luaTL_to_cpu": (_i, [_vp, _vp, _u64]),
    "luaTL_plan_gemm": (_i, [_i, _i, _i, _i, _i, C.POINTER(Plan)]), "luaTL_set_tile_override": (None, [_i]),
    "luaTL_tune_reset": (None, []), "luaTL_autotune_benchmark": (_i, [_i, _i, _i, _i, _i, C.POINTER(Plan)]),
    "luaTL_bcast_add": (_i, [_vp, _vp, _vp, _i, _i, _f, _i]), "luaTL_transpose": (_i, [_vp, _vp, _i, _i, _i]),
    "luaTL_rms_rowscale": (_i, [_vp, _vp, _i, _i, _f, _i]),
    "luaTL_reduce_cols": (_i, [_vp, _vp, _i, _i, _ll, _f, _f, _i]),
    "luaTL_gather_rows": (_i, [_vp, _vp, _vp, _i, _i, _i, _i]),
    "luaTL_row_rms": (_i, [_vp, _vp, _i, _i, _ll, _ll, _f, _i]),
    "matmul_cuda": (_i, [_vp, _vp, _vp, _i, _i, _i]),
    "fused_rmsnorm_matmul_cuda": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f]),
    "fused_gelu_matmul_cuda": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i]),
    "fused_silu_matmul_cuda": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i]),
    "fused_matmul_gelu_cuda": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i]),
    "add_cuda": (_i, [_vp, _vp, _vp, _u64]), "add_inplace_cuda": (_i, [_vp, _vp, _u64, _f]),
    "rmsnorm_cuda": (_i, [_vp, _vp, _vp, _i, _i, _f]), "rmsnorm_inplace_cuda": (_i, [_vp, _vp, _i, _i, _f]),
    "softmax_cuda": (_i, [_vp, _vp, _i, _i]),
    "fused_add_bias_softmax_cuda": (_i, [_vp, _vp, _vp, _i, _i, _f, _i]),
    "luaTL_pipeline_create": (C.POINTER(Pipeline), [_i, _i]), "luaTL_pipeline_destroy": (None, [C.POINTER(Pipeline)]),
    "luaTL_pipeline_reset": (None, [C.POINTER(Pipeline)]),
    "luaTL_pipeline_push": (_i, [C.POINTER(Pipeline), C.POINTER(Cmd)]),
    "luaTL_pipeline_run": (_i, [C.POINTER(Pipeline)]), "luaTL_pipeline_wait": (_i, [C.POINTER(Pipeline)]),
    "luaTL_default_pool": (_vp, []), "luaTL_tensor_alloc": (_vp, [_vp, _u64]),
    "luaTL_tensor_free": (None, [_vp, _vp]), "luaTL_pool_trim": (None, [_vp]),
    "luaTL_pool_get_stats": (_i, [_vp, C.POINTER(PoolStats)]), "luaTL_pool_owns": (_i, [_vp, _vp]),
    "luaTL_tensor_init": (_i, [C.POINTER(Tensor), _i, _i, _i, _vp]),
    "luaTL_tensor_wrap": (_i, [C.POINTER(Tensor), _vp, _i, _i, _i]),
    "luaTL_tensor_release": (None, [C.POINTER(Tensor)]),
    "luaTL_tensor_release_safe": (None, [C.POINTER(Tensor)]),
    "luaTL_tensor_view": (_i, [C.POINTER(Tensor), C.POINTER(Tensor), _i, _i, _i]),
    "luaTL_tensor_zero": (_i, [C.POINTER(Tensor)]),
    "luaTL_tensor_upload": (_i, [C.POINTER(Tensor), _vp, _u64]),
    "luaTL_tensor_download": (_i, [C.POINTER(Tensor), _vp, _u64]),
    "luaTL_tensor_copy": (_i, [C.POINTER(Tensor), C.POINTER(Tensor)]),
    "luaTL_tensor_cast": (_i, [C.POINTER(Tensor), C.POINTER(Tensor)]),
    "luaTL_gpu_copy": (_i, [_vp, _vp, _u64]), "luaTL_gpu_zero": (_i, [_vp, _u64]),
    "luaTL_upload_i32": (_i, [_vp, _vp, _u64]), "luaTL_download_i32": (_i, [_vp, _vp, _u64]),
    "luaTL_download_f32": (_i, [_vp, _vp, _u64]),
    "luaTL_gemm_ex": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i] + [_ll] * 9 + [_i, _f, _f, _f, _i, _i]),
    "luaTL_gemm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _f, _i, _i]),
    "luaTL_rmsnorm": (_i, [_vp, _vp, _vp, _i, _i, _f, _i]),
    "luaTL_rmsnorm_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i]),
    "luaTL_rmsnorm_bwd_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i]),
    "luaTL_softmax": (_i, [_vp, _vp, _vp, _i, _i, _f, _i, _i, _i]),
    "luaTL_softmax_ex": (_i, [_vp, _vp, _vp, _i, _i, _f, _i, _i, _i, _i]),
    "luaTL_softmax_bwd": (_i, [_vp, _vp, _vp, _i, _i, _f, _i, _i, _i, _i]),
    "luaTL_swiglu_fwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i]),
    "luaTL_swiglu_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i]),
    "luaTL_rope": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _i]),
    "luaTL_embed_fwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _i]),
    "luaTL_embed_bwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _f, _i]),
    "luaTL_cross_entropy": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _i]),
    "luaTL_l2_accum": (_i, [_vp, _u64, _vp, _i]),
    "luaTL_clip_by_nsq": (_i, [_vp, _u64, _vp, _f, _i]),
    "luaTL_sum_f32": (_i, [_vp, _u64, _vp, _f]),
    "luaTL_argmax_rows": (_i, [_vp, _vp, _i, _i, _i]),
    "luaTL_elementwise": (_i, [_vp, _vp, _vp, _u64, _i, _i, _f, _f]),
    "luaTL_adamw": (_i, [_vp, _vp, _vp, _vp, _vp, _u64, _i, _f, _f, _f, _f, _f, _i, _f]),
    "luaTL_sgd": (_i, [_vp, _vp, _u64, _f, _f, _vp, _f]),
    "luaTL_gemm_bf16_tc": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i]),
    "luaTL_attention_fwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _i]),
    "luaTL_attention_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _i]),
    "luaTL_gemm_bf16_tc_xty": (_i, [_vp, _vp, _vp, _i, _i, _i, _i]),
    "luaTL_gemm_bf16_rows": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i]),
    "luaTL_gemm_bf16_resid": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i]),
    "luaTL_gemm_bf16_rowscale": (_i, [_vp, _vp, _vp, _vp, _i, _f, _i, _i, _i, _i, _i, _i]),
    "luaTL_set_deferred": (None, [_i]), "luaTL_timer_start": (_i, []), "luaTL_timer_stop": (_i, [C.POINTER(C.c_float)]),
    "luaTL_rmsnorm_bwd_residual": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f]),
    "luaTL_sample_rows": (_i, [_vp, _i, _i, _f, _i, _f, _u64, _vp, _vp]),
    "luaTL_lm_set_sampling": (_i, [_vp, _f, _i, _f, _u64, _i]),
    "luaTL_gemm_bf16_tc_time": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, C.POINTER(C.c_float)]),
    "luaTL_prog_create": (C.POINTER(Prog), [_i, _i]), "luaTL_prog_destroy": (None, [C.POINTER(Prog)]),
    "luaTL_prog_reset": (None, [C.POINTER(Prog)]), "luaTL_prog_push": (_i, [C.POINTER(Prog), C.POINTER(Op)]),
    "luaTL_prog_run": (_i, [C.POINTER(Prog)]), "luaTL_prog_capture": (_i, [C.POINTER(Prog)]),
    "luaTL_prog_replay": (_i, [C.POINTER(Prog)]), "luaTL_prog_wait": (_i, [C.POINTER(Prog)]),
    "luaTL_prog_graph_free": (None, [C.POINTER(Prog)]),
    "luaTL_lm_create": (_vp, [C.POINTER(LmConfig)]), "luaTL_lm_destroy": (None, [_vp]),
    "luaTL_lm_nparams": (_i64, [_vp]), "luaTL_lm_ntensors": (_i, [_vp]),
    "luaTL_lm_tensor_info": (_i, [_vp, _i, _cp, C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                  C.POINTER(_i64), C.POINTER(C.c_int32)]),
    "luaTL_lm_write_params": (_i, [_vp, _i64, _i64, _vp]), "luaTL_lm_read_params": (_i, [_vp, _i64, _i64, _vp]),
    "luaTL_lm_read_grads": (_i, [_vp, _i64, _i64, _vp]),
    "luaTL_lm_params_device": (_vp, [_vp]), "luaTL_lm_grads_device": (_vp, [_vp]),
    "luaTL_lm_train_step": (_i, [_vp, _vp, _vp, C.POINTER(LmTrainArgs), C.POINTER(LmResult)]),
    "luaTL_lm_train_step_dev": (_i, [_vp, _vp, _vp, C.POINTER(LmTrainArgs), C.POINTER(LmResult)]),
    "luaTL_lm_set_tf32": (_i, [_vp, _i]), "luaTL_gemm_tf32_tc": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i]),
    "luaTL_lm_set_graph": (_i, [_vp, _i]), "luaTL_lm_graph_ready": (_i, [_vp]),
    "luaTL_lm_eval_step": (_i, [_vp, _vp, _vp, C.POINTER(LmResult)]),
    "luaTL_lm_forward": (_i, [_vp, _vp, _i, _i, _vp, _i]),
    "luaTL_lm_state_reset": (_i, [_vp]), "luaTL_lm_slot_reset": (_i, [_vp, _i]), "luaTL_lm_step": (_i, [_vp, _i, C.c_int32, _vp]),
    "luaTL_lm_state_len": (_i, [_vp, _i]),
    "luaTL_lm_generate": (_i, [_vp, _vp, _i, _i, _i, _vp, C.POINTER(LmResult)]),
    "luaTL_lm_generate_dev": (_i, [_vp, _vp, _i, _i, _i, _vp, C.POINTER(LmResult)]),
    "luaTL_lm_time_decode_attn": (_i, [_vp, _i, _i, _i, C.POINTER(_f)]),
    "luaTL_lm_last_timing": (_i, [_vp, C.POINTER(_f), C.POINTER(_f), C.POINTER(_i64)]),
    "luaTL_lm_time_decode_launches": (_i, [_vp, _i, _i, _i, C.POINTER(_f), _i]),
    "luaTL_comm_unique_id": (_i, [_cp]), "luaTL_comm_init": (_i, [_cp, _i, _i]),
    "luaTL_comm_world": (_i, []), "luaTL_comm_allreduce_f32": (_i, [_vp, _u64]),
    "luaTL_comm_destroy": (None, []), "luaTL_comm_set_timeout": (None, [_i]),
    "luaTL_comm_selftest_wait": (_i, [_cp, _i, _i, _i, C.POINTER(C.c_int)]),
}

# int-returning functions whose value is not a status
_NOT_STATUS = {"luaTL_init", "luaTL_has_error", "luaTL_pool_owns", "luaTL_lm_ntensors", "luaTL_lm_state_len", "luaTL_lm_graph_ready",
               "luaTL_comm_world"}

_lib = None


def load():
    """The CDLL with argtypes set.  Raises if luaTL.so has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise ImportError(f"{SO_PATH} is missing: build it with `python -m lanternl_b200.build` "
                              "(this backend has no CPU fallback)")
        L = C.CDLL(SO_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)          # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error():
    L = load()
    msg = L.luaTL_get_last_error().decode("utf-8", "replace")
    L.luaTL_clear_error()
    return msg


def call(name, *args):
    """Call an int-status entry point; raise LuaTLError on a non-zero status."""
    rc = getattr(load(), name)(*args)
    if name not in _NOT_STATUS and rc != 0:
        raise LuaTLError(name.replace("luaTL_", ""), rc, last_error())
    return rc


_device = None


def init(device=0):
    """luaTL_init: bind the device; returns the device count.  Raises when there is no GPU."""
    global _device
    n = load().luaTL_init(device)
    if n <= 0:
        raise LuaTLError("init", -4, last_error())
    _device = device
    return n


def ensure_init():
    if _device is None:
        init(int(os.environ.get("LOCAL_RANK", "0")))
