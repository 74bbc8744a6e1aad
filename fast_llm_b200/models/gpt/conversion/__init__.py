"""Hugging Face checkpoint formats of the GPT model family."""

try:
    from fast_llm_b200.models.gpt.conversion.formats import GPT_CHECKPOINT_FORMATS  # noqa: F401
except ImportError:  # formats module not built yet
    GPT_CHECKPOINT_FORMATS = ()
