from .bigdlllm import BigdlNativeLLM, BloomLLM, ChatGLMLLM, GptneoxLLM, LlamaLLM, StarcoderLLM  # noqa: F401
from .transformersllm import TransformersLLM, TransformersPipelineLLM  # noqa: F401

__all__ = ["BigdlNativeLLM", "LlamaLLM", "BloomLLM", "GptneoxLLM", "StarcoderLLM", "ChatGLMLLM", "TransformersLLM",
           "TransformersPipelineLLM"]

# name -> class, as LangChain's loaders look wrappers up (reference langchain/llms/__init__.py:40-48)
type_to_cls_dict = {"BigdlNativeLLM": BigdlNativeLLM, "LlamaLLM": LlamaLLM, "BloomLLM": BloomLLM,
                    "GptneoxLLM": GptneoxLLM, "StarcoderLLM": StarcoderLLM, "ChatGLMLLM": ChatGLMLLM,
                    "TransformersPipelineLLM": TransformersPipelineLLM, "TransformersLLM": TransformersLLM}
