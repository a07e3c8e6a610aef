"""oxidize-b200: a Blackwell-native LLM inference engine.  The public names are loaded on first use, so that importing
the package (for its build script, say) does not import torch."""

_PUBLIC = {"Llama": ".api", "LLM": ".engine.llm", "EngineConfig": ".engine.llm", "SamplingParams": ".engine.sampler"}
__all__ = sorted(_PUBLIC)


def __getattr__(name):
    if name in _PUBLIC:
        import importlib

        return getattr(importlib.import_module(_PUBLIC[name], __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
