"""B200-native (sm_100a) implementation of the LLM decode hot path of kcvlex/my-nn-engine.

The compute lives in ``libmynn_b200.so`` (hand-written CUDA behind a C ABI, see include/mynn_b200.h); this
package is the host side that mirrors the engine's operator and LLM-session interface for that path.
There is no CPU fallback: the operators raise if the library or a CUDA device is missing.
"""
from . import ffi  # noqa: F401
from .session import GenerateOptions, LlmSession, PromptTooLong  # noqa: F401

__all__ = ["ffi", "LlmSession", "GenerateOptions", "PromptTooLong"]
