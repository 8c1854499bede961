"""ctypes binding of libbpdq.so -- the same argtypes tables the reference's callers write
for its libraries (bench/verify_quant_gpu.py:27-42, bench/bench_gpu_sweep.py:11-20,
bench/bench_dequant_gpu_h2h.py:5-13, inference/llamatov_gpu_llama.py:15-31), plus the
additive status-returning entry points.

There is no fallback: if the shared library is missing or cannot be loaded this module
raises, and every compute call launches a CUDA kernel.
"""
import ctypes as C
import os

from . import _build

_LIB = None

vp, i32, sz, f32 = C.c_void_p, C.c_int, C.c_size_t, C.c_float

# name -> (restype, argtypes).  Kept in one table so tests can check that the library exports
# every symbol the header declares.
SIGNATURES = {
    # library state
    "bpdq_set_stream": (None, [vp]),
    "bpdq_get_stream": (vp, []),
    "bpdq_last_status": (i32, []),
    "bpdq_device_error_word": (i32, []),
    "bpdq_clear_status": (None, []),
    "bpdq_set_tuning": (None, [i32, i32, i32, i32, i32]),
    "bpdq_sm_count": (i32, []),
    "bpdq_set_dequant_tuning": (None, [i32, i32]),
    # memory (size_t)
    "bpdq_alloc": (vp, [sz]),
    "bpdq_free": (None, [vp]),
    "bpdq_h2d": (None, [vp, vp, sz]),
    "bpdq_d2h": (None, [vp, vp, sz]),
    "bpdq_d2d": (None, [vp, vp, sz]),
    "bpdq_h2d_async": (i32, [vp, vp, sz, vp]),
    "bpdq_d2h_async": (i32, [vp, vp, sz, vp]),
    "bpdq_host_alloc": (vp, [sz]),
    "bpdq_host_free": (None, [vp]),
    "bpdq_sync": (None, []),
    "bpdq_stream_sync": (i32, [vp]),
    # events, memset, streams, graphs
    "bpdq_event_create": (vp, []),
    "bpdq_event_destroy": (None, [vp]),
    "bpdq_event_record": (i32, [vp, vp]),
    "bpdq_event_elapsed_ms": (f32, [vp, vp]),
    "bpdq_memset_async": (i32, [vp, i32, sz, vp]),
    "bpdq_stream_create": (vp, []),
    "bpdq_stream_wait_event": (i32, [vp, vp]),
    "bpdq_stream_destroy": (None, [vp]),
    "bpdq_graph_begin": (i32, [vp]),
    "bpdq_graph_end": (vp, [vp]),
    "bpdq_graph_launch": (i32, [vp, vp]),
    "bpdq_graph_destroy": (None, [vp]),
    "bpdq_set_device": (i32, [i32]),
    "bpdq_mem_info": (i32, [vp, vp]),
    "bpdq_l2_bytes": (i32, []),
    # reference memory helpers
    **{f"{p}_alloc": (vp, [i32]) for p in ("qgpu", "sgpu", "gpu")},
    **{f"{p}_free": (None, [vp]) for p in ("qgpu", "sgpu", "gpu")},
    **{f"{p}_h2d": (None, [vp, vp, i32]) for p in ("qgpu", "sgpu")},
    **{f"{p}_d2h": (None, [vp, vp, i32]) for p in ("qgpu", "sgpu")},
    **{f"{p}_sync": (None, []) for p in ("qgpu", "sgpu", "gpu")},
    "galloc": (vp, [i32]), "gfree": (None, [vp]), "gh2d": (None, [vp, vp, i32]),
    "gd2h": (None, [vp, vp, i32]), "gsync": (None, []),
    "gpu_copy_h2d": (None, [vp, vp, i32]), "gpu_copy_d2h": (None, [vp, vp, i32]),
    "gpu_copy_d2d": (None, [vp, vp, i32]),
    # Q4_K dequant
    "bpd_dequant_q4k_gpu": (None, [vp, vp, i32]),
    "bpd_dequant_q4k_gpu_st": (i32, [vp, vp, sz, i32, vp]),
    "run_llamacpp": (None, [vp, vp, i32]),
    "run_bpd": (None, [vp, vp, i32]),
    **{n: (None, [vp, vp, i32]) for n in (
        "dequant_v1_256", "dequant_v1_128", "dequant_v1_64", "dequant_v1_32",
        "dequant_ilp2", "dequant_multi2", "dequant_multi4", "dequant_multi8")},
    # Q4_K x Q8_K
    "bpd_quant_q8_K_cuda": (i32, [vp, vp, sz, vp]),
    "bpd_qmatmul_q4k_q8k_cuda": (i32, [vp, vp, vp, i32, i32, vp]),
    "bpd_qmatmul_q4k_q8k_multi_cuda": (i32, [i32, vp, vp, vp, vp, i32, vp]),
    "bpd_qmatmul_q4k_q8k_batch_cuda": (i32, [i32, vp, vp]),
    "bpd_qmatmul_q4k_q8k_batch_ready_cuda": (i32, [i32, vp, vp, sz, vp]),
    # decode glue: record producers and products over records
    "bpdq_records_bytes": (sz, [i32]),
    "bpd_quant_q8k_records_cuda": (i32, [vp, vp, i32, vp]),
    "bpd_rmsnorm_q8k_records_cuda": (i32, [vp, vp, vp, i32, i32, f32, vp]),
    "bpd_swiglu_q8k_records_cuda": (i32, [vp, vp, vp, i32, vp]),
    "bpd_qmatmul_q4k_records_cuda": (i32, [i32, vp, vp, C.c_uint, vp]),
    "bpd_qmatmul_q4k_fused_cuda": (i32, [i32, vp, i32, vp, vp, f32, C.c_uint, vp]),
    "bpd_rmsnorm_llama_cuda": (i32, [vp, vp, vp, i32, i32, f32, vp]),
    "bpd_rope_norm_freqs_cuda": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, f32, vp]),
    "bpd_kv_cache_write_f16_cuda": (i32, [vp, vp, vp, i32, i32, i32, i32, vp]),
    "bpd_kv_cache_write_cuda": (i32, [vp, vp, vp, i32, i32, i32, i32, vp]),
    "bpd_gqa_attn_cuda": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32, i32, vp]),
    "bpd_swiglu_fuse_cuda": (i32, [vp, vp, vp, i32, vp]),
    "bpd_argmax_dim_cuda": (i32, [vp, vp, i32, i32, i32, vp]),
    "bpd_llama_block_cuda": (i32, [vp, vp, vp, vp, i32, i32, vp, vp, vp, vp, vp, vp, vp]),
    "bpd_llama_forward_cuda": (i32, [vp, i32, vp, vp, vp, i32, vp, vp, vp, vp, vp]),
    "bpdq_ipc_export": (i32, [vp, vp]),
    "bpdq_ipc_import": (vp, [vp]),
    "bpdq_ipc_close": (i32, [vp]),
    "bpdq_set_peer_outputs": (i32, [vp, sz, i32, vp]),
    "bpdq_peer_signal": (i32, [vp, i32, C.c_uint, vp]),
    "bpdq_peer_wait": (i32, [vp, i32, C.c_uint, vp]),
    "bpdq_peer_signal_wait": (i32, [vp, vp, i32, C.c_uint, vp]),
    "bpd_llama_forward_tiles_cuda": (i32, [vp, i32, vp, vp, vp, vp, i32, vp, vp, vp, vp, vp]),
    "bpdq_gemv_stream_create": (vp, [i32, vp, vp, sz]),
    "bpdq_gemv_stream_run": (i32, [vp, vp]),
    "bpdq_gemv_stream_run_ready": (i32, [vp, vp]),
    "bpdq_gemv_stream_launches": (i32, [vp]),
    "bpdq_gemv_stream_q8_0_workspace_bytes": (sz, [i32, vp]),
    "bpdq_gemv_stream_create_q8_0": (vp, [i32, vp, vp, sz]),
    "bpdq_gemv_stream_destroy": (None, [vp]),
    "bpdq_chain_create": (vp, [i32, vp]),
    "bpdq_chain_run": (i32, [vp, vp]),
    "bpdq_chain_destroy": (None, [vp]),
    "bpd_qmatmul_q4k_q8k_batch_ws_cuda": (i32, [i32, vp, vp, sz, vp]),
    "bpdq_batch_workspace_bytes": (sz, [i32, vp]),
    "bpd_qmatmul_q4k_q8k_batch_static_cuda": (i32, [i32, vp, vp]),
    "bpdq_batch_static_capacity": (sz, []),
    "bpd_qmm_q4k_q8k_cuda": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp]),
    "bpdq_qmm_q4k_q8k_workspace_bytes": (sz, [i32, i32, i32]),
    "bpd_qmm_q4k_q8k_ws_cuda": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, sz, vp]),
    "bpd_qmm_q4k_q8k_mma_ints_cuda": (i32, [vp, vp, vp, vp, i32, i32, i32, vp]),
    "bpd_qmm_q4k_q8k_tc5_ints_cuda": (i32, [vp, vp, vp, vp, i32, i32, i32, vp]),
    "bpd_q4k_rg16_bytes": (sz, [i32, i32]),
    "bpd_repack_q4k_rg16_cuda": (i32, [vp, vp, i32, i32, vp]),
    "bpd_unrepack_q4k_rg16_cuda": (i32, [vp, vp, i32, i32, vp]),
    "bpd_qmm_q4k_q8k_rg16_cuda": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "bpdq_qmm_q4k_q8k_rg16_workspace_bytes": (sz, [i32, i32]),
    "bpd_qmm_q4k_q8k_rg16_ws_cuda": (i32, [vp, vp, vp, i32, i32, i32, vp, sz, vp]),
    "bpd_qmm_q4k_q8k_rg16_ints_cuda": (i32, [vp, vp, vp, vp, i32, i32, i32, vp]),
    "bpdq_gemm_rg16_stream_workspace_bytes": (sz, [i32, vp, i32]),
    "bpdq_gemm_rg16_stream_create": (vp, [i32, vp, i32, vp, sz]),
    "bpdq_gemm_rg16_stream_run": (i32, [vp, vp]),
    "bpdq_gemm_rg16_stream_launches": (i32, [vp]),
    "bpdq_gemm_rg16_stream_destroy": (None, [vp]),
    "bpd_qmm_q4k_q8k_mma_cuda": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "bpd_qmm_q4k_q8k_tc5_cuda": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "gpu_vecmat_q4k": (None, [vp, vp, vp, i32, i32]),
    # fp32 decode operators
    "gpu_vecmat": (None, [vp, vp, vp, i32, i32]),
    "gpu_rms_norm": (None, [vp, vp, vp, i32, i32, f32]),
    "gpu_add": (None, [vp, vp, vp, i32]),
    "gpu_mul": (None, [vp, vp, vp, i32]),
    "gpu_silu": (None, [vp, vp, i32]),
    "gpu_matmul": (None, [vp, vp, vp, i32, i32, i32]),
    "gpu_matmul_opt": (None, [vp, vp, vp, i32, i32, i32]),
    # Q4_K x fp32
    "bpd_qmatmul_q4k_gpu": (None, [vp, vp, vp, i32, i32]),
    "bpd_qmatmul_q4k_gpu_st": (i32, [vp, vp, vp, i32, i32, vp]),
    "bpd_qmm_q4k_cuda": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    # Q8_0
    "bpd_dequant_q8_0_cuda": (i32, [vp, vp, sz, vp]),
    "bpd_quant_q8_0_cuda": (i32, [vp, vp, sz, vp]),
    "bpd_q8_0_block_dots_cuda": (i32, [vp, vp, vp, sz, vp]),
    "bpd_qmatmul_q8_0_cuda": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "bpd_embed_lookup_q8_0_cuda": (i32, [vp, vp, vp, i32, i32, vp]),
    "bpd_embed_lookup_q8_0_vocab_cuda": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "bpd_qmatmul_q8_0_llamafile_cuda": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "bpd_qmatmul_q8_0_dispatch_cuda": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    **{f"bpd_gemm_q8_0_{rm}_{rn}_cuda": (i32, [vp, vp, i32, i32, i32, vp, i32, vp]) for rm in (1, 2, 4) for rn in (1, 2, 4)},
    "bpdq_qmatmul_q8_0_tiles_workspace_bytes": (sz, [i32, i32, i32]),
    "bpd_qmatmul_q8_0_tiles_ws_cuda": (i32, [vp, vp, vp, i32, i32, i32, vp, sz, vp]),
    "bpdq_llama_forward_workspace_bytes": (sz, [vp, i32]),
    "bpd_llama_forward_ws_cuda": (i32, [vp, i32, vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, sz, vp]),
    "bpd_q8_0_tiles_bytes": (sz, [i32, i32]),
    "bpd_repack_q8_0_tiles_cuda": (i32, [vp, vp, i32, i32, vp]),
    "bpd_unrepack_q8_0_tiles_cuda": (i32, [vp, vp, i32, i32, vp]),
    "bpd_qmatmul_q8_0_tiles_cuda": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "gpu_vecmat_q8_0": (None, [vp, vp, vp, i32, i32]),
    "gpu_matmul_q4k": (None, [vp, vp, vp, i32, i32, i32]),
}


def lib_path():
    return _build.LIB


def load(build_if_missing=True):
    """Returns the bound library; raises if it cannot be built or loaded."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not os.path.exists(path):
        if not build_if_missing:
            raise FileNotFoundError(f"{path} is missing: run bpd_substrate_b200._build.build()")
        _build.build()
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


class GemvDesc(C.Structure):
    """bpdq_gemv_desc: one product of a batched launch."""
    _fields_ = [("W", vp), ("x", vp), ("out", vp), ("M", i32), ("K", i32)]


class ChainPhase(C.Structure):
    """bpdq_chain_phase: one phase of a persistent decode chain."""
    _fields_ = [("n", i32), ("prologue", i32), ("a", vp), ("b", vp), ("eps", f32), ("accumulate_mask", C.c_uint),
                ("prod", GemvDesc * 3)]


class LlamaConfig(C.Structure):
    """bpd_llama_config (bench/bpd_cpu.c:5537-5553 of the reference)."""
    _fields_ = [(n, i32) for n in ("n_layers", "n_heads", "n_kv_heads", "head_dim", "embed_dim", "ffn_dim", "vocab_size",
                                   "max_seq_len")] + [("rms_eps", f32), ("rope_base", f32), ("rope_dim", i32),
                                                      ("kv_cache_f16", i32)]


class LlamaLayerWeights(C.Structure):
    """bpd_llama_layer_weights: nine pointers in the reference's order."""
    _fields_ = [(n, vp) for n in ("attn_norm_w", "w_q", "w_k", "w_v", "w_o", "ffn_norm_w", "w_gate", "w_up", "w_down")]


class LlamaWeights(C.Structure):
    """bpd_llama_weights; `layers` points to a host array of LlamaLayerWeights."""
    _fields_ = [("token_embd", vp), ("layers", C.POINTER(LlamaLayerWeights)), ("output_norm_w", vp), ("output_w", vp),
                ("rope_freqs", vp)]


class BpdqError(RuntimeError):
    pass


def check(status, what=""):
    if status != 0:
        raise BpdqError(f"{what or 'libbpdq call'} failed with status {status}")
    return status
