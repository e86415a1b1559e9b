"""LangChain integration (reference: python/llm/src/ipex_llm/langchain/).  The classes subclass LangChain's base
classes when ``langchain_core`` is installed and otherwise stand alone with the same methods (``invoke``,
``__call__``, ``embed_documents``, ``embed_query``)."""
