from .ipexllm import IpexLLM  # noqa: F401

BigdlLLM = IpexLLM
__all__ = ["IpexLLM", "BigdlLLM"]
