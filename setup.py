"""Packaging of ipex_llm_b200 (with the ``ipex_llm`` and ``bigdl`` import aliases).  The native libraries are built
in-tree for sm_100a by ``python __graft_entry__.py`` (or ``python -m ipex_llm_b200.native.build``) and shipped as
package data; the reference's setup.py downloads prebuilt binaries instead (python/llm/setup.py:92-325)."""
from setuptools import find_packages, setup

setup(
    name="ipex_llm_b200",
    version="0.1.0",
    description="Blackwell-native low-bit LLM library with the API surface of ipex-llm",
    packages=find_packages(include=["ipex_llm_b200*", "ipex_llm*", "bigdl*"]),
    package_data={"ipex_llm_b200": ["native/*.so", "native/cuda/*.cu", "native/cuda/*.cuh", "native/cuda/*.h",
                                    "native/cuda/common/*.cuh", "native/host/*.cpp", "native/host/*.h", "native/tools/*.cpp", "native/bin/*"]},
    python_requires=">=3.10",
    install_requires=["torch", "transformers", "numpy"],
    extras_require={"serving": ["fastapi", "uvicorn", "pydantic"], "all": ["sentencepiece", "pyyaml", "safetensors"]},
    entry_points={"console_scripts": [
        "llm-cli=ipex_llm_b200.cli.llm_cli:main",
        "llm-chat=ipex_llm_b200.cli.llm_cli:chat_main",
        "llm-convert=ipex_llm_b200.convert_model:main",
        "ipex-llm-init=ipex_llm_b200.cli.ipex_llm_init:main",
        "ipex-quantize=ipex_llm_b200.cli.llm_cli:quantize_main",
    ]},
)
