"""python examples/serving.py --repo-id-or-model-path <dir> --low-bit sym_int4 --port 8000
then:  curl http://localhost:8000/v1/chat/completions -H 'Content-Type: application/json' \
            -d '{"model": "m", "messages": [{"role": "user", "content": "Hello"}], "max_tokens": 64, "stream": true}'"""
from ipex_llm_b200.serving.api_server import main

if __name__ == "__main__":
    main()
