"""Reference module path ``ipex_llm.transformers.patches``: small monkey patches of third-party loaders the
reference applies on import (``get_class_from_dynamic_module`` caching for remote-code models).  Nothing needs
patching with the installed transformers; the functions are kept as no-ops."""


def patch_flash_attn_import(filename: str) -> None:
    return None


def patch_sdpa_available() -> bool:
    return True
