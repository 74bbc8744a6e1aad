"""Importing this module registers every model family, trainer and dataset type with its registry
(parity: `fast_llm/models/auto.py`, `fast_llm/data/auto.py`)."""

from fast_llm_b200.data import config as _data_config  # noqa: F401
from fast_llm_b200.layers import attention as _attention, block as _block, mlp as _mlp  # noqa: F401
from fast_llm_b200.models.gpt import config as _gpt_config  # noqa: F401
from fast_llm_b200.models.gpt import conversion as _gpt_conversion  # noqa: F401  (Hugging Face format names resolve from a fresh process)
from fast_llm_b200.models.gpt import trainer as _gpt_trainer  # noqa: F401

for _optional in ("fast_llm_b200.layers.moe", "fast_llm_b200.layers.ssm", "fast_llm_b200.layers.stochastic_mixer",
                  "fast_llm_b200.data.memmap", "fast_llm_b200.models.multimodal.config", "fast_llm_b200.models.multimodal.conversion",
                  "fast_llm_b200.engine.checkpoint.convert", "fast_llm_b200.engine.evaluation.evaluators",
                  "fast_llm_b200.data.preparation.config"):
    try:
        __import__(_optional)
    except ModuleNotFoundError as e:
        if e.name != _optional and not _optional.startswith(e.name or "\0"):
            raise
