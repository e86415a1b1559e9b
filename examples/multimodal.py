"""Vision-language chat with a low-bit model (Qwen2-VL, Qwen2.5-VL, GLM-4V, InternVL, Llama-3.2-Vision, ...): the
vision tower and the language model are both converted.  Reference: python/llm/example/GPU/HuggingFace/Multimodal

    python examples/multimodal.py --model <hf dir> --image photo.jpg --prompt "Describe the picture."
"""
import argparse

import torch

from ipex_llm import optimize_model

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--image", required=True)
    ap.add_argument("--prompt", default="Describe the picture.")
    ap.add_argument("--low-bit", default="sym_int4")
    ap.add_argument("--n-predict", type=int, default=64)
    a = ap.parse_args()
    from PIL import Image
    from transformers import AutoModelForImageTextToText, AutoProcessor
    processor = AutoProcessor.from_pretrained(a.model)
    model = AutoModelForImageTextToText.from_pretrained(a.model, dtype=torch.float16)
    model = optimize_model(model, low_bit=a.low_bit)
    if torch.cuda.is_available():
        model = model.to("cuda")
    messages = [{"role": "user", "content": [{"type": "image"}, {"type": "text", "text": a.prompt}]}]
    text = processor.apply_chat_template(messages, add_generation_prompt=True)
    inputs = processor(text=text, images=Image.open(a.image), return_tensors="pt").to(next(model.parameters()).device)
    out = model.generate(**inputs, max_new_tokens=a.n_predict, do_sample=False)
    print(processor.batch_decode(out[:, inputs["input_ids"].shape[1]:], skip_special_tokens=True)[0])
