"""Multimodal model: vision encoder layers, then the GPT layers; image embeddings are added at their token positions.

Per micro-batch the vision layers read their own kwargs namespace: normalised patches, (row, column) coordinates for the
2-D rotary embedding and `cu_seqlens` with one entry per image, so patches attend only within their image.  The language
model's embedding layer receives the adapter output and the `embedding_map` (patch index -> token index).
Parity: `fast_llm/models/multimodal/model.py:18-90`, `fast_llm/layers/vision/vision_encoder.py:81-135`,
`fast_llm/data/document/patch.py:31-177`.
"""

import torch

from fast_llm_b200.layers.kwargs import BlockKwargs, LanguageModelKwargs
from fast_llm_b200.layers.vision import VisionKwargs
from fast_llm_b200.models.gpt.model import GPTBaseModel, GPTModel

VISION_NAMESPACE = "vision_encoder"


class MultiModalBaseModel(GPTBaseModel):
    def __init__(self, config, distributed_config):
        super().__init__(config, distributed_config)
        self._vision_layers = config.vision_encoder.get_layers(distributed_config, self._hidden_dim, lr_scale=config.lr_scale,
                                                               peft=None, namespace=VISION_NAMESPACE)
        for i, layer in enumerate(self._vision_layers):
            setattr(self, f"vision_{i}", layer)

    def set_names(self, prefix: str = "") -> None:
        super().set_names(prefix)  # the vision layers are named by their config when they are built

    def get_layers(self):
        return [*self._vision_layers, *super().get_layers()]

    def _sequence_split(self) -> int:
        """Ranks the patch sequence is split over between vision layers (sequence-tensor parallelism)."""
        dc = self._distributed_config
        return dc.tensor_parallel if dc.sequence_tensor_parallel else 1

    def get_activation_shape(self, layer_index: int, kwargs: dict):
        """Between vision layers the activation is `[patches, vision width]`; the adapter hands `[patches, hidden]` to the
        embedding layer; from there on the default `[tokens, hidden]`."""
        vision_layers = len(self._vision_layers)
        if not 0 < layer_index <= vision_layers:
            return None
        patches = kwargs[VISION_NAMESPACE][BlockKwargs.num_tokens] // self._sequence_split()
        width = self._config.vision_encoder.hidden_size if layer_index < vision_layers else self._hidden_dim.size
        return (patches, width)

    def preprocess_batch(self, model_inputs, *, phase, iteration, metrics=None, device=None):
        device = device or (self._distributed.device if self._distributed is not None else "cpu")
        normalization = self._config.vision_encoder.normalization
        compute_dtype = self._distributed_config.compute_dtype.torch
        for model_input in model_inputs:
            extras = model_input.extras
            patches = extras.pop("image_patches", None)
            token_positions = extras.pop("image_patch_positions", None)
            coordinates = extras.pop("patch_positions", None)
            if patches is None:
                shape = self._vision_layers[0].unwrap().get_preprocessing_config()["patch_shape"]
                patches = torch.zeros((0, *shape))
                token_positions = torch.zeros(0, dtype=torch.int64)
            if coordinates is None:
                coordinates = torch.zeros(len(patches), 2, dtype=torch.int64)
            # keep the patches whose token lies in this rank's slice of the micro-sequence
            begin = model_input.sequence_k_end - len(model_input.tokens)
            keep = (token_positions >= begin) & (token_positions < model_input.sequence_k_end)
            patches, coordinates, token_positions = patches[keep], coordinates[keep], token_positions[keep] - begin
            # one attention segment per image: a patch at (0, 0) opens a new image
            starts = ((coordinates[:, 0] == 0) & (coordinates[:, 1] == 0)).nonzero().flatten().tolist()
            if len(patches) and (not starts or starts[0] != 0):
                starts = [0, *starts]
            bounds = [*starts, len(patches)]
            lengths = [b - a for a, b in zip(bounds[:-1], bounds[1:])]
            real_patches = len(patches)
            padding = -real_patches % self._sequence_split()
            if padding:
                # sequence parallelism splits the patch sequence evenly over the tensor ranks: blank patches that form an
                # image of their own (nothing attends to them, no token takes their output) fill it up
                patches = torch.cat([patches, patches.new_zeros((padding, *patches.shape[1:]))])
                coordinates = torch.cat([coordinates, coordinates.new_zeros((padding, 2))])
                lengths.append(padding)
            cu = torch.tensor([0, *torch.tensor(lengths, dtype=torch.int64).cumsum(0).tolist()] if lengths else [0, 0], dtype=torch.int32)
            extras[VISION_NAMESPACE] = {
                VisionKwargs.patches: normalization.normalize(patches).to(compute_dtype),
                VisionKwargs.patch_positions: coordinates,
                BlockKwargs.cu_seqlens_q: cu, BlockKwargs.cu_seqlens_k: cu,
                BlockKwargs.max_seqlen_q: max(lengths, default=0), BlockKwargs.max_seqlen_k: max(lengths, default=0),
                BlockKwargs.num_tokens: len(patches), "training": phase.is_training,
            }
            extras[LanguageModelKwargs.embedding_map] = (torch.arange(real_patches), token_positions.to(torch.int64))
        out = super().preprocess_batch(model_inputs, phase=phase, iteration=iteration, metrics=metrics, device=device)
        for _, kwargs in out:
            vision = kwargs[VISION_NAMESPACE]
            for key, value in list(vision.items()):
                if torch.is_tensor(value):
                    vision[key] = value.to(device, non_blocking=True)
            kwargs[LanguageModelKwargs.embedding_map] = tuple(t.to(device, non_blocking=True) for t in kwargs[LanguageModelKwargs.embedding_map])
        return out


class MultiModalModel(GPTModel):
    from fast_llm_b200.models.multimodal.config import MultiModalModelConfig as config_class  # noqa: E402

    base_model_class = MultiModalBaseModel
