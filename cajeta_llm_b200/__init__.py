"""A B200-native inference engine for Qwen2-MoE, built from parts.

Importing the package registers the built-in parts and architectures.  The public
entry points are :class:`cajeta_llm_b200.engine.llm_engine.LlmEngine` (load, submit,
generate), ``python -m cajeta_llm_b200`` (command line) and ``bin/trace_run``.
"""
from . import parts  # noqa: F401  (registers the built-in parts)
from .models import qwen2_moe  # noqa: F401  (registers the architecture)

__version__ = "0.1.0"
