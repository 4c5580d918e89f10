from .context import AttentionContext, create_decode_context, create_prefill_context

__all__ = ["AttentionContext", "create_decode_context", "create_prefill_context"]
