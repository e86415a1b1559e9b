"""Stable Diffusion / SDXL with the UNet's attention on the package's kernels (and, with --low-bit, packed UNet
linears).  Reference: python/llm/example/GPU/HuggingFace/Multimodal/StableDiffusion/sdxl.py

    python examples/stable_diffusion.py --model stabilityai/stable-diffusion-xl-base-1.0 --prompt "An astronaut"

Needs the ``diffusers`` package (not part of this repository's requirements).
"""
import argparse

import torch

from ipex_llm import optimize_model

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompt", default="An astronaut in the forest, detailed, 8k")
    ap.add_argument("--low-bit", default=None)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--out", default="image.png")
    a = ap.parse_args()
    from diffusers import DiffusionPipeline
    pipe = DiffusionPipeline.from_pretrained(a.model, torch_dtype=torch.float16, use_safetensors=True)
    pipe = optimize_model(pipe, low_bit=a.low_bit)
    pipe.to("cuda")
    pipe(prompt=a.prompt, num_inference_steps=a.steps).images[0].save(a.out)
