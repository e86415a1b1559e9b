"""Reference import path ``ipex_llm.transformers.models.sd`` (python/llm/src/ipex_llm/transformers/models/sd.py):
the Stable-Diffusion attention processor and VAE precision fix live in ``ipex_llm_b200.models.sd``."""
from ...models.sd import AttnProcessor2_0, is_diffusion_pipeline, optimize_pipeline, upcast_vae  # noqa: F401
