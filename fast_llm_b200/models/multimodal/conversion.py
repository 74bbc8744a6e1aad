"""External checkpoint formats of the multimodal model (filled in by the llava converter)."""

MULTIMODAL_CHECKPOINT_FORMATS: tuple = ()
