from .transformersembeddings import TransformersEmbeddings  # noqa: F401

__all__ = ["TransformersEmbeddings"]
