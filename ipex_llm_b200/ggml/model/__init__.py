from .generic import Bloom, ChatGLM, GenericModel, Gptneox, Llama, Starcoder  # noqa: F401
