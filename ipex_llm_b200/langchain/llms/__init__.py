from .transformersllm import TransformersLLM, TransformersPipelineLLM  # noqa: F401

__all__ = ["TransformersLLM", "TransformersPipelineLLM"]
