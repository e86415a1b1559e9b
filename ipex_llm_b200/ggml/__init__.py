"""Legacy native-model API surface (reference: python/llm/src/ipex_llm/ggml/): qtype table and llama-cpp-python
style model classes, here thin fronts over the transformers-style API."""
from ..quant.qtypes import ggml_tensor_qtype  # noqa: F401
