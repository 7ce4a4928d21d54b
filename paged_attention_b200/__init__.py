"""B200-native paged split-KV flash-decoding engine.

`paged_attention_b200.decode` mirrors the reference's `decode::` C++ interface
(KVDtype, DecodeParams, DecodePlan, DevicePlan, make_plan, paged_decode,
PagedKVCache) over the C ABI of libpd_b200.so (include/pd_b200.h).
"""
from .decode import *  # noqa: F401,F403
from .decode import __all__  # noqa: F401
