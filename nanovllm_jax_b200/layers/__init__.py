from .attention import (PALLAS_AVAILABLE, Attention, KVCache, paged_attention, paged_prefill_attention,
                        store_kv_to_cache, variable_length_attention_prefill)

__all__ = ["Attention", "KVCache", "store_kv_to_cache", "variable_length_attention_prefill", "paged_attention",
           "paged_prefill_attention", "PALLAS_AVAILABLE"]
