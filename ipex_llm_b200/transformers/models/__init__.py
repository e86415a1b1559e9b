"""Reference package path ``ipex_llm.transformers.models`` (per-family forward files of the reference,
python/llm/src/ipex_llm/transformers/models/).  The family registry and forwards live in ``ipex_llm_b200.models``."""
