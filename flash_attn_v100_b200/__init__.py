"""B200-native attention operators behind the `flash_attn_v100` operator API."""
from .ops import *  # noqa: F401,F403
from .ops import (REFERENCE_EXPORTS, check_async_errors, check_prefill_errors, set_decode_tuning,  # noqa: F401
                  set_prefill_impl, rope_append_paged_fp16)
from .kv_cache import PagedKVCache  # noqa: F401

__all__ = list(REFERENCE_EXPORTS) + ["check_async_errors", "check_prefill_errors", "set_decode_tuning", "set_prefill_impl",
                                     "rope_append_paged_fp16", "PagedKVCache"]
