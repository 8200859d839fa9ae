"""Import shim: the framework's sources live in the directory ``1cat-vllm_b200/``
(not a valid Python identifier), and are imported under the name ``onecat_vllm``.

Public surface mirrors the reference's top-level package
(reference: vllm/__init__.py:23-46): ``LLM``, ``SamplingParams``, ``RequestOutput``,
``CompletionOutput``, ``EngineArgs``, ``AsyncLLM``.
"""
import os as _os

_SRC = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "1cat-vllm_b200")
__path__.insert(0, _SRC)  # submodules resolve inside 1cat-vllm_b200/

__version__ = "0.1.0"

_LAZY = {
    "LLM": "onecat_vllm.entrypoints.llm",
    "SamplingParams": "onecat_vllm.sampling_params",
    "RequestOutput": "onecat_vllm.outputs",
    "CompletionOutput": "onecat_vllm.outputs",
    "EngineArgs": "onecat_vllm.config",
    "AsyncEngineArgs": "onecat_vllm.config",
    "VllmConfig": "onecat_vllm.config",
    "LLMEngine": "onecat_vllm.engine.llm_engine",
    "AsyncLLM": "onecat_vllm.engine.async_llm",
    "TokensPrompt": "onecat_vllm.inputs",
    "TextPrompt": "onecat_vllm.inputs",
    "PoolingParams": "onecat_vllm.sampling_params",
}


def __getattr__(name):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module 'onecat_vllm' has no attribute {name!r}")
    import importlib

    return getattr(importlib.import_module(mod), name)


__all__ = list(_LAZY)
