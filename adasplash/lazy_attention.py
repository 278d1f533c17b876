from flash_lazy_attention_b200.layers import LazyAttention, LazyAttentionLayer  # noqa: F401
