"""llm_b200: a single-GPU inference engine for the dense Llama decoder on B200 (sm_100a).

    from llm_b200 import LLM
    llm = LLM("/path/to/model_folder", dtype="bfloat16")
    out = llm.generate([[1, 2, 3]], max_new_tokens=16)
"""
from .config import EngineOptions, LlamaConfig, load_config, register_architecture

__all__ = ["EngineOptions", "LLM", "LlamaConfig", "load_config", "register_architecture", "Engine", "StepEntry"]


def __getattr__(name):
    if name == "LLM":
        from .engine.llm import LLM
        return LLM
    if name in ("Engine", "StepEntry"):
        from .engine import engine as _e
        return getattr(_e, name)
    raise AttributeError(name)
