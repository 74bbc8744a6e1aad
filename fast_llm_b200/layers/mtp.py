"""Multi-token prediction: extra heads that predict tokens further ahead from the trunk's second-to-last hidden state.

The trunk's last block hands over `stack(input, output)`.  Head 1 scores `output` against the next token; every extra
prediction distance d owns one more decoder block (same config as the trunk's last) applied to the shared `input`, and
a head (sharing the output weights) scored against the token d positions ahead.  All of it forms ONE layer of the model's
layer list, so the heads always live on the same pipeline stage and their losses add up in one backward.
Parity: `fast_llm/layers/language_model/multi_token_prediction.py:18-108`, `head.py:150-171`.
"""

import torch

from fast_llm_b200.engine.base_model import Layer


class MultiTokenPredictionStage(Layer):
    layer_count = 1000.0  # like the head: closes the last stage

    def __init__(self, head, extra: list[tuple[Layer, Layer]], distributed_config):
        super().__init__(head._config, distributed_config)
        self.head = head
        self._extra = extra
        for index, (block, extra_head) in enumerate(extra):
            setattr(self, f"block_{index}", block)
            setattr(self, f"head_{index}", extra_head)
        self.module_name = "multi_token_prediction"

    def set_names(self, prefix: str = "") -> None:
        pass  # the owning model names the wrapped layers

    def setup(self, distributed) -> None:
        self._distributed = distributed
        self._is_setup = True
        for layer in (self.head, *(l for pair in self._extra for l in pair)):
            if not layer._is_setup:
                layer.setup(distributed)

    def forward(self, input_: torch.Tensor, kwargs: dict, losses: dict | None = None, metrics: dict | None = None) -> torch.Tensor:
        if input_.dim() == 3 and input_.shape[0] == 2:
            shared, output = input_[0], input_[1]
        else:  # a trunk that does not expose its last block's input: every head reads the trunk output
            shared = output = input_
        total = self.head.forward(output, kwargs, losses, metrics)
        if kwargs.get("return_logits", False) or not torch.is_tensor(total) or total.dim() > 0:
            return total  # inference: logits of the next-token head
        for block, head in self._extra:
            hidden = block.forward(shared, kwargs, losses, metrics)
            total = total + head.forward(hidden, kwargs, losses, metrics)
        return total

    def get_compute_usage(self, input_meta, kwargs, config=None) -> int:
        return sum(layer.get_compute_usage(input_meta, kwargs, config) for layer in (self.head, *(l for pair in self._extra for l in pair)))
