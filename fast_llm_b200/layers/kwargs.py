"""Names of the per-micro-batch entries passed to every layer through `kwargs` (the model input contract).

Parity: `fast_llm/layers/block/config.py` BlockKwargs, `fast_llm/layers/attention/config.py` AttentionKwargs,
`fast_llm/layers/language_model/config.py` LanguageModelKwargs.
"""


class BlockKwargs:
    token_ids = "token_ids"
    position_ids = "position_ids"  # [tokens] position of each token inside its document
    document_index = "document_index"  # [tokens] index of the document each token belongs to
    cu_seqlens_q = "cu_seqlens_q"
    cu_seqlens_k = "cu_seqlens_k"
    max_seqlen_q = "max_seqlen_q"
    max_seqlen_k = "max_seqlen_k"
    num_tokens = "num_tokens"
    sequence_first = "sequence_first"
    grad_output = "grad_output"
    iteration = "iteration"
    phase = "phase"
    hidden_states = "hidden_states"
    output_hidden_states = "output_hidden_states"
    past_key_values = "past_key_values"
    presents = "presents"
    key_value_rows = "key_value_rows"  # generation: cached and new keys / values are both [rows * n, width]; joined row by row
    micro_sequence_index = "micro_sequence_index"
    sequence_k_offset = "sequence_k_offset"


class LanguageModelKwargs(BlockKwargs):
    labels = "labels"
    loss_mask = "loss_mask"
    num_labels = "num_labels"
    chosen_spans = "chosen_spans"
    rejected_spans = "rejected_spans"
    advantages = "advantages"
    old_log_probabilities = "old_log_probabilities"
    embedding_map = "embedding_map"
    position_embedding_ids = "position_embedding_ids"
    reference_logits = "reference_logits"
    mask_inputs = "mask_inputs"
