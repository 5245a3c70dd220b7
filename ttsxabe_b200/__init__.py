"""B200-native attention hot path of llmtie-rs behind its device-handle API.

`Gpu` mirrors `llmtie_cuda::Gpu` for attention, RoPE and the KV cache;
`KvCache` carries the model crates' cache growth policy; `ShardedDecode`
spreads one long context over several GPUs. Everything computes through
libllmtie_b200.so; there is no CPU path.
"""
from .gpu import (  # noqa: F401
    CacheOverrun,
    CudaError,
    DecodeScratch,
    DeviceTimeout,
    DriverError,
    Exchange,
    Gpu,
    InvalidArgument,
    Misaligned,
    MissingKernel,
    NoDevice,
    OddCacheCapacity,
    OddHeadDim,
    RaggedBlock,
    SliceOverrun,
    UnsupportedAttention,
    decode_cut,
    decode_plan,
)
from .cache import KvCache, Prefix, shared_prefix, want_capacity  # noqa: F401
