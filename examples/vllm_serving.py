"""vLLM with low-bit weights: offline generation through ``IPEXLLMClass`` or the OpenAI-compatible server.
Reference: python/llm/example/GPU/vLLM-Serving/offline_inference.py and
python/llm/src/ipex_llm/vllm/xpu/entrypoints/openai/api_server.py

    python examples/vllm_serving.py --model <hf dir> --low-bit sym_int4 --prompt "Hello"
    python -m ipex_llm.vllm.entrypoints.openai.api_server --model <hf dir> --load-in-low-bit fp8 --port 8000
"""
import argparse

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--low-bit", default="sym_int4")
    ap.add_argument("--prompt", action="append", default=None)
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--max-tokens", type=int, default=64)
    a = ap.parse_args()
    from vllm import SamplingParams

    from ipex_llm.vllm.engine import IPEXLLMClass
    llm = IPEXLLMClass(model=a.model, load_in_low_bit=a.low_bit, tensor_parallel_size=a.tensor_parallel_size,
                       dtype="float16", enforce_eager=True)
    for out in llm.generate(a.prompt or ["What is AI?"], SamplingParams(temperature=0.0, max_tokens=a.max_tokens)):
        print(repr(out.prompt), "->", repr(out.outputs[0].text))
