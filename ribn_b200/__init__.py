"""ribn_b200 — B200-native batched decode / chunked-prefill executor behind
ribn's ``GenerationExecutor`` protocol.

The product is the CUDA shared library ``libribn_b200.so`` (C ABI declared in
``include/ribn_b200.h``).  This package is the thin host-side mirror of the
reference's executor interface used by the tests and the benchmark; it never
computes anything on the CPU and fails loudly when the library is missing.
"""
from ._lib import (  # noqa: F401
    F32, F16, Q8_0, Q4_K, Q6_K, OK, PENDING, REJECTED, DEFERRED, SELECTED, ERROR, PREFILL, DECODE,
    SCHEME_Q8_0, SCHEME_Q4_K_M, FLAG_KEEP_LOGITS, FLAG_REFERENCE_KERNELS, FLAG_NO_GRAPH, FLAG_NO_TCGEN05,
    FLAG_KV_ON_DEMAND, FLAG_OPERAND_CACHE, INJECT_ALLOC_REFUSAL, INJECT_ERROR_WORD, INJECT_BAD_ROW,
    Config, lib, library_path,
)
from .executor import (  # noqa: F401
    Admission, BatchItem, ExecutionError, ExecutorInfo, GenerationLimits, PreparedRow, QwenB200, Sampling,
    StepCompletion, StepKind, nccl_library_path, tp_shard, tp_unique_id,
)
from .engine import Engine, EngineConfig, SchedulePolicy, TokenRequest  # noqa: F401
from .native_engine import NativeEngine  # noqa: F401
from . import gemma  # noqa: F401
from . import gguf  # noqa: F401
from .gemma import GemmaB200, GemmaExecutor, GemmaSequence  # noqa: F401
from . import ops  # noqa: F401

QWEN3_0_6B = dict(layers=28, hidden=1024, q_heads=16, kv_heads=8, head_dim=128, ffn=3072, vocab=151936,
                  rope_base=1.0e6, rms_eps=1.0e-6)
QWEN3_8B = dict(layers=36, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, ffn=12288, vocab=151936,
                rope_base=1.0e6, rms_eps=1.0e-6)
QWEN3_32B = dict(layers=64, hidden=5120, q_heads=64, kv_heads=8, head_dim=128, ffn=25600, vocab=151936,
                 rope_base=1.0e6, rms_eps=1.0e-6)

# Reduced Gemma-4-architecture decoder: five sliding-window (512) layers, then one full-attention layer.
GEMMA4_REDUCED = dict(layers=6, hidden=1152, heads=4, kv_heads=1, head_dim=256, global_head_dim=256, ffn=6912,
                      vocab=32768, ple=256, ple_vocab=32768, window=512, context=512, kv_shared=0, eps=1.0e-6,
                      softcap=30.0, theta_local=1.0e4, theta_global=1.0e6,
                      layer_types=["sliding"] * 5 + ["full"])
