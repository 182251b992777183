"""kairyu_b200: a small single-GPU inference engine for dense decoder models on
NVIDIA B200 (sm_100a), with hand-written CUDA kernels."""

from kairyu_b200.config.engine_config import EngineConfig
from kairyu_b200.entrypoints.outputs import CompletionOutput, RequestOutput
from kairyu_b200.entrypoints.prompt import TextPrompt, TokensPrompt
from kairyu_b200.sampling.params import SamplingParams

__version__ = "0.1.0"


def __getattr__(name: str):
    if name == "LLM":  # imported lazily: it pulls in torch and the engine
        from kairyu_b200.entrypoints.llm import LLM

        return LLM
    raise AttributeError(name)


__all__ = [
    "CompletionOutput", "EngineConfig", "LLM", "RequestOutput", "SamplingParams", "TextPrompt", "TokensPrompt",
]
