"""cogito_b200: a Blackwell-native (B200, sm_100a) deep-learning framework with the capabilities of
cogito-ml/cogito.  Sub-packages: ``nn`` (modules), ``ops`` (kernel-backed autograd functions), ``optim``,
``models``, ``parallel`` (data / tensor / pipeline / 3-D), ``quant``, ``serve``, ``jit``, ``io``, ``data``,
``utils``.  The names a training or serving script needs are also reachable from the top level; they are
imported on first use, so ``import cogito_b200`` stays cheap and loads no native library.

The ``cg_*`` C API of the reference lives in ``lib/libcogito.so`` (headers in ``include/``, ctypes binding in
``bindings/cogito.py``) and versions itself through ``COGITO_VERSION_*`` in ``include/cogito.h``.
"""
from __future__ import annotations

import importlib

__version__ = "1.0.0"

_SUBPACKAGES = ("nn", "ops", "optim", "models", "parallel", "quant", "serve", "jit", "io", "data", "utils", "train", "cli", "build")

_NAMES = {
    # models
    "GPT2": "models.gpt2", "GPT2Config": "models.gpt2", "Llama": "models.llama", "LlamaConfig": "models.llama",
    "MLPClassifier": "models.mlp", "XorNet": "models.mlp", "ConvClassifier": "models.cnn",
    # training
    "Trainer": "train", "FusedAdam": "optim.fused", "FusedSGD": "optim.fused", "GradScaler": "optim.fused",
    # parallel training
    "init_parallel": "parallel.groups", "ParallelContext": "parallel.groups", "DataParallel": "parallel.data_parallel",
    "DPFusedAdam": "parallel.data_parallel", "build_tp_gpt2": "parallel.tensor_parallel", "Trainer3D": "parallel.llama_parallel",
    # quantisation and serving
    "quantize_int4": "quant.int4", "dequantize_int4": "quant.int4", "Int4Linear": "quant.int4",
    "PagedKVCacheInt4": "serve.kv_cache", "LlamaInt4Engine": "serve.engine", "SpeculativeDecoder": "serve.engine",
    # checkpoints, profiling, failure detection, JIT
    "save_model": "io.checkpoint", "load_model": "io.checkpoint", "save_training_state": "io.checkpoint",
    "load_training_state": "io.checkpoint", "Profiler": "utils.profiler", "instrument": "utils.profiler",
    "Heartbeat": "utils.failure", "RankFailure": "utils.failure", "run_with_restarts": "utils.failure",
    "checkpoint": "utils.recompute", "fuse": "jit.fuse", "manual_seed": "utils.rng",
}

__all__ = ["__version__", *_SUBPACKAGES, *_NAMES]


def __getattr__(name: str):
    if name in _NAMES:
        value = getattr(importlib.import_module(f"{__name__}.{_NAMES[name]}"), name)
    elif name in _SUBPACKAGES:
        value = importlib.import_module(f"{__name__}.{name}")
    else:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    globals()[name] = value
    return value


def __dir__():
    return sorted(set(globals()) | set(__all__))
