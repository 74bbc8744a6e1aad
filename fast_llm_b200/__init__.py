"""B200-native LLM pre-training framework with the capabilities and user contract of Fast-LLM."""

__version__ = "0.4.0"
