"""``bigdl`` — legacy top-level name of the reference project (``bigdl.llm`` became ``ipex_llm``;
python/llm/src/ipex_llm/__init__.py:38-47 keeps the old name importable).  ``bigdl.llm`` resolves to this package's
implementation as well."""
