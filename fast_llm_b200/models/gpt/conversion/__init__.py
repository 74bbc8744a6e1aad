"""Hugging Face checkpoint formats of the GPT model family."""

from fast_llm_b200.models.gpt.conversion.apriel2 import Apriel2TextCheckpointFormat
from fast_llm_b200.models.gpt.conversion.formats import GPT_CHECKPOINT_FORMATS as _BASE_FORMATS
from fast_llm_b200.models.gpt.conversion.gemma4 import Gemma4CheckpointFormat

GPT_CHECKPOINT_FORMATS = _BASE_FORMATS + (Apriel2TextCheckpointFormat, Gemma4CheckpointFormat)
