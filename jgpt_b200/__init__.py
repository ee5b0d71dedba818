"""jgpt_b200: B200-native KV-cache decode path for JGPT behind a C ABI.

The product is ``lib/libjgpt_b200.so`` (hand-written CUDA for sm_100a, declared in
``include/jgpt_b200.h``).  This package is the thin host-side mirror of the reference's Java
classes on that path (``KvCacheGpu`` and the attention ops of ``TensorOps``), written over
ctypes because no JDK is available where it is tested; a JNI / FFM binding maps one to one.
"""
from .binding import JgptError, PoolExhausted, load  # noqa: F401
from .runtime import Context, DeviceBuffer  # noqa: F401
from .kv_cache import KvPool, KvCacheGpu  # noqa: F401
from .model import GPTModel  # noqa: F401
from .scheduler import ContinuousBatcher, TokenGather, pack_pairs, shard_requests, unpack_pairs  # noqa: F401
