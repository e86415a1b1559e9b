"""Reference module path ``ipex_llm.vllm.cpu.entrypoints.openai.api_server``."""
from ....entrypoints.openai.api_server import main, make_parser  # noqa: F401

if __name__ == "__main__":
    main()
