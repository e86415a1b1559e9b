"""Reference module path ``ipex_llm.transformers.utils`` (imatrix reader and per-layer qtype policy,
python/llm/src/ipex_llm/transformers/utils.py:186-400; ``get_xpu_device_name`` :183)."""
import torch

from ..quant import policy as _policy
from ..utils.common import invalidInputError  # noqa: F401

globals().update({k: v for k, v in vars(_policy).items() if not k.startswith("_")})


def get_xpu_device_name(device=None) -> str:
    """The reference keys kernel choices on the Intel device family ("arc", "pvc", "mtl" ...); here there is one
    family.  Returns "b200" on a CUDA device, "cpu" otherwise."""
    if device is not None and torch.device(device).type == "cuda" or device is None and torch.cuda.is_available():
        return "b200"
    return "cpu"
