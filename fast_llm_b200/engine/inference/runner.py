"""Forward-only execution of a staged model (reference models for distillation / preference losses, evaluation,
generation).  Parity: `fast_llm/engine/inference/runner.py:13-71`."""

import torch

from fast_llm_b200.data.document import LanguageModelBatch, LanguageModelDocument
from fast_llm_b200.engine.multi_stage.config import StageMode
from fast_llm_b200.parallel.topology import PhaseType


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
