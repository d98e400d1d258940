"""lm_head_topk: the caller of dense_reader's top-k records (an LM head that returns token ids, not logits)."""
