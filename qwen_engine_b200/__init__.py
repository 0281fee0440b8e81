"""A small, whole, single-GPU inference engine for the Qwen3 dense decoder on
NVIDIA B200 (sm_100a): everything between a request's tokens and its next token.

    from qwen_engine_b200 import LLM, SamplingParams
    llm = LLM(model="/path/to/model_folder", dtype="bfloat16")
    outs = llm.generate([[1, 2, 3]], SamplingParams(max_new_tokens=8))
"""
__version__ = "0.1.0"

_LAZY = {
    "LLM": ("qwen_engine_b200.engine.llm", "LLM"),
    "LLMEngine": ("qwen_engine_b200.engine.llm", "LLMEngine"),
    "RequestOutput": ("qwen_engine_b200.engine.llm", "RequestOutput"),
    "SamplingParams": ("qwen_engine_b200.sampling.params", "SamplingParams"),
    "EngineConfig": ("qwen_engine_b200.config", "EngineConfig"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        module, attr = _LAZY[name]
        return getattr(importlib.import_module(module), attr)
    raise AttributeError(name)
