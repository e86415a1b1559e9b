"""Reference module path ``ipex_llm.transformers.low_bit_linear`` (python/llm/src/ipex_llm/transformers/
low_bit_linear.py: ``FP4Params`` :312-459, ``LowBitLinear`` :573-715, ``FP16Linear`` / ``BF16Linear`` :718-908,
``MatMulLowBit`` :500-570, the ``ggml_*`` wrappers :104-259).  The implementations live in ``ops.linear`` and
``quant.params``; every public name of both is available here."""
from ..ops import linear as _linear
from ..quant import params as _params
from ..quant.qtypes import *  # noqa: F401,F403
from ..quant.qtypes import ggml_tensor_qtype  # noqa: F401

globals().update({k: v for k, v in vars(_params).items() if not k.startswith("_")})
globals().update({k: v for k, v in vars(_linear).items() if not k.startswith("_")})
