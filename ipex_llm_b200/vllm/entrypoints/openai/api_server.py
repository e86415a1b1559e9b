"""OpenAI-compatible vLLM server with low-bit weights:
``python -m ipex_llm.vllm.entrypoints.openai.api_server --model <path> --load-in-low-bit sym_int4 [vLLM flags]``.

Counterpart of python/llm/src/ipex_llm/vllm/xpu/entrypoints/openai/api_server.py (a copy of vLLM's server whose engine
is built with ``load_in_low_bit``).  vLLM's own server is used as it is: this entry point adds the one flag to vLLM's
argument parser, installs the loader patches for that format (keeping the engine core in this process so that they
apply), and hands over to ``vllm.entrypoints.openai.api_server.run_server``.
"""
from __future__ import annotations

import asyncio


def make_parser():
    from vllm.entrypoints.openai.cli_args import make_arg_parser
    try:
        from vllm.utils.argparse_utils import FlexibleArgumentParser
    except ImportError:                                    # older layout
        from vllm.utils import FlexibleArgumentParser
    parser = make_arg_parser(FlexibleArgumentParser(description="vLLM OpenAI-compatible server with low-bit weights"))
    parser.add_argument("--load-in-low-bit", type=str, default="sym_int4",
                        help="weight format the workers pack the model to after loading (sym_int4, fp8, nf4, ...)")
    return parser


def main(argv=None):
    args = make_parser().parse_args(argv)
    from ...engine import _convert
    _convert(args.load_in_low_bit)
    from vllm.entrypoints.openai.api_server import run_server
    return asyncio.run(run_server(args))


if __name__ == "__main__":
    main()
