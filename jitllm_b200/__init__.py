"""B200-native (sm_100a) CUDA implementation of jitLLM's Llama decode / prefill hot path behind a
C ABI (include/jitllm_b200.h), with a Python mirror of the reference's host interfaces."""
from .api import (  # noqa: F401
    B200BatchExecutor,
    B200InvocationBoundary,
    B200Model,
    BatchSlots,
    Configuration,
    Device,
    DeviceTimeoutError,
    GGMLType,
    IllegalStateError,
    InsufficientDeviceMemoryError,
    KvStorage,
    KvStorageRequest,
    Sampler,
    TensorRole,
    UNMAPPED,
    argmax,
    load_model,
    precomputeFreqsCis,
    quantize,
    random_blocks,
    synth_model_tensors,
    synth_tensor,
)
from .tensor_parallel import TensorParallel, local_shape, shard_tensor, torch_broadcast  # noqa: F401,E402
from .gguf import GgufFile, load_model_gguf, write_gguf  # noqa: F401,E402
