"""Forward-only execution of a staged model (reference models for distillation / preference losses, evaluation,
generation).  Parity: `fast_llm/engine/inference/runner.py:13-71`."""

import torch

from fast_llm_b200.data.document import LanguageModelBatch, LanguageModelDocument
from fast_llm_b200.engine.multi_stage.config import StageMode
from fast_llm_b200.parallel.topology import PhaseType


class KeyValueCache:
    """Generation cache of an attention-only decoder.  Per attention layer, in layer order: the rotated keys and values of
    every row's positions so far, `[rows * length, width]` with the rows one after another (a row's left padding included:
    it is a document of its own, as in the packed forward pass).  Parity: the `past_key_values` / `presents` lists of
    `fast_llm/models/gpt/huggingface.py:158-199`."""

    def __init__(self, pads: list[int]):
        self.pads = list(pads)  # left padding of every row
        self.layers: list[torch.Tensor] = []
        self.length = 0  # positions held per row
        self.on_reorder = None  # called with the row index before a reorder (tensor-parallel workers follow it)

    @property
    def rows(self) -> int:
        return len(self.pads)

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.length

    def reorder_cache(self, beam_idx: torch.Tensor) -> None:
        """The name `transformers` beam search calls."""
        if self.on_reorder is not None:
            self.on_reorder(beam_idx)
        self.reorder(beam_idx)

    def reorder(self, index: torch.Tensor) -> None:
        """Beam search: row i continues from row index[i]."""
        order = index.tolist()
        self.layers = [kv.view(self.rows, self.length, -1).index_select(0, index.to(kv.device)).reshape(len(order) * self.length, -1)
                       for kv in self.layers]
        self.pads = [self.pads[i] for i in order]


class InferenceRunner:
    def __init__(self, model):
        self._model = model
        self._is_setup = False

    @property
    def model(self):
        return self._model

    def setup(self, distributed=None, pretrained_config=None) -> None:
        if not self._model.is_setup:
            self._model.setup(distributed, mode=StageMode.inference)
        self._distributed = self._model.distributed
        self._is_setup = True

    def load(self, pretrained_config) -> None:
        if pretrained_config.pretrained.path is not None:
            self._model.load_checkpoint(pretrained_config.pretrained)
        else:
            self._model.initialize_weights()

    @torch.no_grad()
    def forward_kwargs(self, tokens: torch.Tensor, kwargs: dict, iteration: int = 0) -> dict:
        """Run every stage on one prepared micro-sequence; results (logits, hidden states) land in `kwargs`."""
        assert self._is_setup
        kwargs["training"] = False
        output = tokens
        for stage in self._model.stages_on_device.values():
            stage.restore_parameters()
            output, _ = stage.forward(output, kwargs)
        return kwargs

    @torch.no_grad()
    def forward_tokens(self, tokens: torch.Tensor, document_lengths: list[int] | None = None, output_hidden_states=None):
        """Logits [tokens, vocab] for a flat token stream (one document unless lengths are given).  With
        `output_hidden_states` (a list of layer names, possibly empty) returns `(logits, {name: hidden})`."""
        n = len(tokens)
        lengths = document_lengths or [n]
        batch = LanguageModelBatch(tokens=torch.cat([tokens.cpu().long(), torch.full((1,), -100, dtype=torch.long)]),
                                   document_lengths=lengths[:-1] + [lengths[-1] + 1])
        (inp,) = batch.get_model_inputs(micro_batch_size=n, predicted_tokens=1)
        kwargs = inp.to_kwargs(self._distributed.device)
        kwargs.pop("labels", None)
        kwargs["return_logits"] = True
        if output_hidden_states:
            kwargs["output_hidden_states"] = set(output_hidden_states)
            kwargs["hidden_states"] = {}
        for layer in self._model.base_model.get_layers():
            layer.preprocess(kwargs)
        self.forward_kwargs(kwargs["token_ids"], kwargs)
        if output_hidden_states is not None:
            return kwargs["logits"], kwargs.get("hidden_states", {})
        return kwargs["logits"]

    def supports_key_value_cache(self) -> bool:
        """True when every mixer of the decoder is attention on this rank's own sequence (recurrent mixers keep no state
        between calls, sequence-data parallelism splits the keys)."""
        from fast_llm_b200.layers.attention import Attention
        from fast_llm_b200.layers.block import DecoderBlock

        blocks = [layer.unwrap() for layer in self._model.base_model.get_layers() if isinstance(layer.unwrap(), DecoderBlock)]
        return bool(blocks) and all(type(block.mixer) is Attention and block.mixer._sdp_dim.size == 1 for block in blocks)

    @torch.no_grad()
    def forward_rows(self, tokens: torch.Tensor, cache: KeyValueCache, output_hidden_states=None):
        """`tokens` [rows, n]: the next n positions of every row of `cache` (the whole left-padded prompt when the cache is
        empty).  Returns logits [rows * n, vocab] (and the hidden states asked for) and extends the cache."""
        from fast_llm_b200.layers.kwargs import LanguageModelKwargs

        rows, new = tokens.shape
        assert rows == cache.rows
        held = cache.length
        cu_q, cu_k, positions, documents = [0], [0], [], []
        for pad in cache.pads:
            pad_queries = pad if held == 0 else 0  # the padding is only ever seen by itself, in the first pass
            if pad:
                cu_q.append(cu_q[-1] + pad_queries)
                cu_k.append(cu_k[-1] + pad)
                positions.append(torch.arange(pad_queries))
                documents += [len(cu_q) - 2] * pad_queries
            queries, seen = new - pad_queries, max(held - pad, 0)  # `seen`: real positions of this row in the cache
            cu_q.append(cu_q[-1] + queries)
            cu_k.append(cu_k[-1] + seen + queries)
            positions.append(torch.arange(seen, seen + queries))
            documents += [len(cu_q) - 2] * queries
        lengths_q = [b - a for a, b in zip(cu_q, cu_q[1:])]
        lengths_k = [b - a for a, b in zip(cu_k, cu_k[1:])]
        device = self._distributed.device
        kwargs = {
            LanguageModelKwargs.token_ids: tokens.reshape(-1).to(device),
            LanguageModelKwargs.position_ids: torch.cat(positions).to(device=device, dtype=torch.int32),
            LanguageModelKwargs.document_index: torch.tensor(documents, dtype=torch.int32, device=device),
            LanguageModelKwargs.cu_seqlens_q: torch.tensor(cu_q, dtype=torch.int32, device=device),
            LanguageModelKwargs.cu_seqlens_k: torch.tensor(cu_k, dtype=torch.int32, device=device),
            LanguageModelKwargs.max_seqlen_q: max(lengths_q), LanguageModelKwargs.max_seqlen_k: max(lengths_k),
            LanguageModelKwargs.num_tokens: rows * new, LanguageModelKwargs.micro_sequence_index: 0,
            LanguageModelKwargs.sequence_k_offset: rows * (held + new), "max_position": held + new,
            LanguageModelKwargs.key_value_rows: rows, LanguageModelKwargs.presents: [], "return_logits": True,
        }
        if cache.layers:
            kwargs[LanguageModelKwargs.past_key_values] = list(cache.layers)
        if output_hidden_states:
            kwargs["output_hidden_states"] = set(output_hidden_states)
            kwargs["hidden_states"] = {}
        for layer in self._model.base_model.get_layers():
            layer.preprocess(kwargs)
        self.forward_kwargs(kwargs[LanguageModelKwargs.token_ids], kwargs)
        cache.layers = [kv.detach() for kv in kwargs[LanguageModelKwargs.presents]]
        cache.length = held + new
        return kwargs["logits"], kwargs.get("hidden_states", {})
