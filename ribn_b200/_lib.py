"""ctypes binding of ``libribn_b200.so`` — exactly the symbols declared in
``include/ribn_b200.h``.  There is no fallback: a missing library raises."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))

F32, F16, Q8_0, Q4_K, Q6_K = 0, 1, 8, 12, 14
OK, PENDING, REJECTED, DEFERRED, SELECTED, ERROR = 0, 1, 2, 3, 4, -1
ROW_READY, ROW_DEFERRED, ROW_REJECTED = 0, 1, 2
INJECT_ALLOC_REFUSAL, INJECT_ERROR_WORD, INJECT_BAD_ROW = 1, 2, 3
PREFILL, DECODE = 0, 1
SCHEME_Q8_0, SCHEME_Q4_K_M = 0, 1
FLAG_KEEP_LOGITS, FLAG_REFERENCE_KERNELS, FLAG_NO_GRAPH, FLAG_NO_TCGEN05, FLAG_KV_ON_DEMAND = 1, 2, 4, 8, 16
FLAG_OPERAND_CACHE = 32


class Config(C.Structure):
    _fields_ = [
        ("layers", C.c_int32), ("hidden", C.c_int32), ("q_heads", C.c_int32), ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("ffn", C.c_int32), ("vocab", C.c_int32),
        ("rope_base", C.c_float), ("rms_eps", C.c_float),
        ("context_tokens", C.c_int32), ("max_sequences", C.c_int32), ("max_batch_tokens", C.c_int32),
        ("kv_pages", C.c_int32), ("device", C.c_int32), ("flags", C.c_int32),
        ("tp_size", C.c_int32), ("tp_rank", C.c_int32),
    ]


class Limits(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "context_tokens", "max_sequences", "max_batch_tokens", "max_decode_tokens", "kv_page_tokens",
        "kv_pages_total", "kv_pages_free")]


class BatchItemC(C.Structure):
    _fields_ = [("sequence", C.c_uint64), ("kind", C.c_uint32), ("prefix", C.c_uint32),
                ("token_budget", C.c_uint32), ("output_budget", C.c_uint32)]


class SamplingC(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_uint32), ("reserved", C.c_uint32),
                ("seed", C.c_uint64)]


class PreparedRowC(C.Structure):
    _fields_ = [("state", C.c_uint32), ("token_budget", C.c_uint32), ("output_budget", C.c_uint32),
                ("reserved", C.c_uint32)]


class NcclId(C.Structure):
    _fields_ = [("bytes", C.c_char * 128)]


class CompletionC(C.Structure):
    _fields_ = [("sequence", C.c_uint64), ("prefix", C.c_uint32), ("n_tokens", C.c_uint32),
                ("token", C.c_uint32), ("reserved", C.c_uint32)]


_P = C.c_void_p
# name -> (restype, argtypes); one entry per declaration in include/ribn_b200.h
SIGNATURES = {
    "ribn_b200_create": (C.c_int, [C.POINTER(Config), C.POINTER(_P), C.c_char_p, C.c_size_t]),
    "ribn_b200_destroy": (C.c_int, [_P]),
    "ribn_b200_load_tensor": (C.c_int, [_P, C.c_char_p, C.c_int32, C.c_int64, C.c_int64, _P, C.c_size_t]),
    "ribn_b200_init_synthetic": (C.c_int, [_P, C.c_uint64, C.c_int32]),
    "ribn_b200_read_tensor": (C.c_int, [_P, C.c_char_p, C.POINTER(C.c_int32), C.POINTER(C.c_int64),
                                        C.POINTER(C.c_int64), _P, C.c_size_t, C.POINTER(C.c_size_t)]),
    "ribn_b200_finalize": (C.c_int, [_P]),
    "ribn_b200_info": (C.c_int, [_P, C.POINTER(Limits)]),
    "ribn_b200_admit": (C.c_int, [_P, C.c_uint64, C.c_uint64, _P, C.c_uint32, C.c_uint32, C.POINTER(SamplingC), _P,
                                  C.c_uint32]),
    "ribn_b200_prepare": (C.c_int, [_P, C.POINTER(BatchItemC), C.c_uint32]),
    "ribn_b200_prepare_rows": (C.c_int, [_P, C.POINTER(BatchItemC), C.c_uint32, C.POINTER(PreparedRowC)]),
    "ribn_b200_tp_unique_id": (C.c_int, [C.c_char_p, C.POINTER(NcclId), C.c_char_p, C.c_size_t]),
    "ribn_b200_tp_init": (C.c_int, [_P, C.c_char_p, C.POINTER(NcclId)]),
    "ribn_b200_tp_time_allreduce": (C.c_int, [_P, C.c_uint32, C.c_uint32, C.POINTER(C.c_float)]),
    "ribn_b200_tp_shard": (C.c_int, [C.POINTER(Config), C.c_char_p, C.c_int64, C.c_int64, C.POINTER(C.c_int64),
                                     C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "ribn_b200_debug_inject": (C.c_int, [_P, C.c_int32, C.c_int32]),
    "ribn_b200_debug_wait_expiry": (C.c_int, [_P, C.c_uint32]),
    "ribn_b200_debug_unpack": (C.c_int, [C.c_int32, C.c_int32, _P, C.c_int64, C.c_int64, _P]),
    "ribn_b200_op_embedding": (C.c_int, [C.c_int32, C.c_int32, _P, C.c_int32, C.c_int32, _P, C.c_int32, _P]),
    "ribn_b200_op_qk_norm_rope_append": (C.c_int, [C.c_int32, _P, _P, _P, _P, _P, _P, _P, C.c_int32, C.c_int32,
                                                   C.c_int32, C.c_int32, C.c_float, C.c_float, _P, _P, C.c_int32]),
    "ribn_b200_op_attention_decode": (C.c_int, [C.c_int32, _P, _P, _P, _P, _P, C.c_float, C.c_float, _P, _P, C.c_int32,
                                                _P, C.c_int32, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P]),
    "ribn_b200_abandon_preparation": (C.c_int, [_P]),
    "ribn_b200_submit": (C.c_int, [_P, C.POINTER(BatchItemC), C.c_uint32, C.POINTER(C.c_uint64)]),
    "ribn_b200_poll": (C.c_int, [_P, C.c_uint64, C.POINTER(CompletionC), C.c_uint32, C.POINTER(C.c_uint32)]),
    "ribn_b200_release": (C.c_int, [_P, C.c_uint64]),
    "ribn_b200_synchronize": (C.c_int, [_P]),
    "ribn_b200_last_error": (C.c_size_t, [_P, C.c_char_p, C.c_size_t]),
    "ribn_b200_op_last_error": (C.c_size_t, [C.c_char_p, C.c_size_t]),
    "ribn_b200_copy_logits": (C.c_int, [_P, C.c_uint32, _P, C.c_size_t]),
    "ribn_b200_copy_kv": (C.c_int, [_P, C.c_uint64, C.c_int32, C.c_int32, C.c_uint32, _P]),
    "ribn_b200_debug_set_context": (C.c_int, [_P, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint64]),
    "ribn_b200_last_step_stats": (C.c_int, [_P, C.POINTER(C.c_float), C.POINTER(C.c_uint32)]),
    "ribn_b200_step_bytes": (C.c_int, [_P, C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "ribn_b200_time_projection": (C.c_int, [_P, C.c_int32, C.c_uint32, C.POINTER(C.c_float), C.POINTER(C.c_uint64)]),
    "ribn_b200_op_dequantize": (C.c_int, [C.c_int32, C.c_int32, _P, C.c_int64, C.c_int64, _P]),
    "ribn_b200_op_gemv": (C.c_int, [C.c_int32, C.c_int32, _P, C.c_int64, C.c_int64, _P, C.c_int32, _P, C.c_int32]),
    "ribn_b200_op_rms_norm": (C.c_int, [C.c_int32, _P, _P, C.c_int32, C.c_int32, C.c_float, _P]),
    "ribn_b200_op_silu_mul": (C.c_int, [C.c_int32, _P, _P, C.c_int64, _P]),
    "ribn_b200_op_gdn_step": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P, _P, _P, _P, _P,
                                        _P, _P, C.c_float, C.c_float, _P, _P, _P, _P, _P]),
    "ribn_b200_op_attention_gate": (C.c_int, [C.c_int32, _P, _P, C.c_int64, C.c_int32, C.c_int32, _P]),
    "ribn_b200_op_argmax": (C.c_int, [C.c_int32, _P, C.c_int32, C.c_int64, _P]),
    "ribn_b200_op_rope_neox": (C.c_int, [C.c_int32, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float]),
    "ribn_b200_op_f32_to_f16": (C.c_int, [C.c_int32, _P, C.c_int64, _P]),
    "ribn_b200_op_attention": (C.c_int, [C.c_int32, _P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                         C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, C.c_int32]),
    "ribn_b200_op_batch_metadata": (C.c_int, [C.c_int32, _P, _P, _P, C.c_int32, _P, C.c_int32, C.c_int32, _P, _P,
                                              _P, _P]),
    "ribn_b200_attention_noalloc": (C.c_int, [C.c_int32, _P, _P, _P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32,
                                              C.c_int32, C.c_int32, C.c_int32, _P, C.c_char_p, C.c_size_t]),
    "ribn_b200_debug_repack": (C.c_int, [C.c_int32, _P, C.c_int64, C.c_int64, _P, C.c_size_t,
                                         C.POINTER(C.c_size_t)]),
    "ribn_b200_build_info": (C.c_char_p, []),
}

GEMMA_MAX_LAYERS = 64


class GemmaConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "layers", "hidden", "heads", "kv_heads", "head_dim", "global_head_dim", "ffn", "vocab", "ple", "ple_vocab",
        "window", "context", "kv_shared")] + \
        [(n, C.c_float) for n in ("eps", "softcap", "theta_local", "theta_global")] + \
        [("full", C.c_int32 * GEMMA_MAX_LAYERS)] + \
        [(n, C.c_int32) for n in ("max_sequences", "max_batch_tokens", "device", "flags")]


class GemmaRow(C.Structure):
    _fields_ = [("sequence", C.c_uint64), ("tokens", C.POINTER(C.c_uint32)), ("n_tokens", C.c_uint32),
                ("want_output", C.c_uint32)]


_U32P, _U64P = C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)
# one entry per declaration in include/ribn_b200_gemma.h
SIGNATURES.update({
    "ribn_b200_gemma_create": (C.c_int, [C.POINTER(GemmaConfig), C.POINTER(_P), C.c_char_p, C.c_size_t]),
    "ribn_b200_gemma_destroy": (C.c_int, [_P]),
    "ribn_b200_gemma_last_error": (C.c_char_p, [_P]),
    "ribn_b200_gemma_load_tensor": (C.c_int, [_P, C.c_char_p, _P, C.c_size_t]),
    "ribn_b200_gemma_init_synthetic": (C.c_int, [_P, C.c_uint64]),
    "ribn_b200_gemma_read_tensor": (C.c_int, [_P, C.c_char_p, _P, C.c_size_t, C.POINTER(C.c_size_t)]),
    "ribn_b200_gemma_finalize": (C.c_int, [_P]),
    "ribn_b200_gemma_open": (C.c_int, [_P, _U64P]),
    "ribn_b200_gemma_advance_prefill": (C.c_int, [_P, C.c_uint64, _P, C.c_uint32]),
    "ribn_b200_gemma_prefill": (C.c_int, [_P, C.c_uint64, _P, C.c_uint32, _P, _U32P]),
    "ribn_b200_gemma_decode": (C.c_int, [_P, C.c_uint64, C.c_uint32, _P, _U32P]),
    "ribn_b200_gemma_position": (C.c_int, [_P, C.c_uint64, _U32P]),
    "ribn_b200_gemma_close": (C.c_int, [_P, C.c_uint64]),
    "ribn_b200_gemma_step": (C.c_int, [_P, C.POINTER(GemmaRow), C.c_uint32, _P, _P]),
    "ribn_b200_gemma_synchronize": (C.c_int, [_P]),
    "ribn_b200_gemma_last_step_stats": (C.c_int, [_P, C.POINTER(C.c_float), _U32P]),
})

# ---- include/ribn_b200_engine.h ---------------------------------------------------------------------------
_INFO_FN = C.CFUNCTYPE(C.c_int, _P, C.POINTER(Limits))
_ADMIT_FN = C.CFUNCTYPE(C.c_int, _P, C.c_uint64, C.c_uint64, _U32P, C.c_uint32, C.c_uint32, C.POINTER(SamplingC), _U32P, C.c_uint32)
_PREPARE_FN = C.CFUNCTYPE(C.c_int, _P, C.POINTER(BatchItemC), C.c_uint32, C.POINTER(PreparedRowC))
_ABANDON_FN = C.CFUNCTYPE(C.c_int, _P)
_SUBMIT_FN = C.CFUNCTYPE(C.c_int, _P, C.POINTER(BatchItemC), C.c_uint32, _U64P)
_POLL_FN = C.CFUNCTYPE(C.c_int, _P, C.c_uint64, C.POINTER(CompletionC), C.c_uint32, _U32P)
_RELEASE_FN = C.CFUNCTYPE(C.c_int, _P, C.c_uint64)
_LAST_ERROR_FN = C.CFUNCTYPE(C.c_size_t, _P, C.POINTER(C.c_char), C.c_size_t)


class ExecutorTable(C.Structure):
    _fields_ = [("self", _P), ("info", _INFO_FN), ("admit", _ADMIT_FN), ("prepare_rows", _PREPARE_FN),
                ("abandon_preparation", _ABANDON_FN), ("submit", _SUBMIT_FN), ("poll", _POLL_FN),
                ("release", _RELEASE_FN), ("last_error", _LAST_ERROR_FN)]


class EngineConfigC(C.Structure):
    _fields_ = [("max_active_requests", C.c_uint32), ("max_queued_requests", C.c_uint32)]


class SchedulePolicyC(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("max_batch_tokens", "prefill_chunk_tokens", "decode_tokens", "max_decode_only_steps")]


class RequestStatusC(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("state", "finish", "prompt_tokens", "prefix", "generated", "output_tokens")] + \
        [(n, C.c_uint64) for n in ("enqueue_ns", "first_token_ns", "last_token_ns")]


class EngineCountersC(C.Structure):
    _fields_ = [("steps", C.c_uint64), ("decode_only_steps", C.c_uint32), ("waiting", C.c_uint32), ("prefill", C.c_uint32),
                ("decode", C.c_uint32), ("parked", C.c_uint32), ("in_flight_rows", C.c_uint32), ("resource_epoch", C.c_uint64),
                ("faulted", C.c_uint32), ("reserved", C.c_uint32)]


# one entry per declaration in include/ribn_b200_engine.h
SIGNATURES.update({
    "ribn_b200_engine_create": (C.c_int, [C.POINTER(ExecutorTable), C.POINTER(EngineConfigC), C.POINTER(SchedulePolicyC),
                                          C.POINTER(_P), C.c_char_p, C.c_size_t]),
    "ribn_b200_engine_create_for": (C.c_int, [_P, C.POINTER(EngineConfigC), C.POINTER(SchedulePolicyC), C.POINTER(_P),
                                              C.c_char_p, C.c_size_t]),
    "ribn_b200_engine_destroy": (C.c_int, [_P]),
    "ribn_b200_engine_enqueue": (C.c_int, [_P, _P, C.c_uint32, C.c_uint32, _P, C.c_uint32, C.c_float, _U64P]),
    "ribn_b200_engine_step": (C.c_int, [_P, C.POINTER(C.c_int32)]),
    "ribn_b200_engine_idle": (C.c_int, [_P]),
    "ribn_b200_engine_status": (C.c_int, [_P, C.c_uint64, C.POINTER(RequestStatusC)]),
    "ribn_b200_engine_output": (C.c_int, [_P, C.c_uint64, _P, C.c_uint32, _U32P]),
    "ribn_b200_engine_token_times": (C.c_int, [_P, C.c_uint64, _P, C.c_uint32, _U32P]),
    "ribn_b200_engine_finish_reason": (C.c_size_t, [_P, C.c_uint64, C.c_char_p, C.c_size_t]),
    "ribn_b200_engine_counters": (C.c_int, [_P, C.POINTER(EngineCountersC)]),
    "ribn_b200_engine_last_error": (C.c_size_t, [_P, C.c_char_p, C.c_size_t]),
})

_LIB = None


def library_path() -> str:
    return os.path.join(HERE, "libribn_b200.so")


def lib() -> C.CDLL:
    """Load the CUDA library.  Raises if it has not been built: the product
    path has no CPU implementation to fall back to."""
    global _LIB
    if _LIB is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m ribn_b200.build` (needs nvcc); "
                "ribn_b200 has no CPU fallback")
        handle = C.CDLL(path)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = restype
            fn.argtypes = argtypes
        _LIB = handle
    return _LIB
