"""LISA (layer-wise importance sampled AdamW): every ``interval_steps`` optimizer steps a fresh random subset of
``n_layers`` decoder blocks is unfrozen and all others are frozen.

Counterpart of python/llm/src/ipex_llm/transformers/lisa.py:23-81 (``DynamicLayerActivationCallback``).  The decoder
stack is found structurally (the longest ``nn.ModuleList`` of the model) instead of through a class-name table, so
any decoder-only architecture works; only floating-point parameters are toggled (packed low-bit weights stay frozen).
"""
from __future__ import annotations

import random

from torch import nn

from ..train.trainer import TrainerCallback
from ..utils.common import invalidInputError


def find_decoder_layers(model) -> nn.ModuleList:
    best = None
    for m in model.modules():
        if isinstance(m, nn.ModuleList) and len(m) > 0 and (best is None or len(m) > len(best)):
            best = m
    invalidInputError(best is not None, f"Model {type(model).__name__} has no layer stack: not supported.")
    return best


class DynamicLayerActivationCallback(TrainerCallback):
    def __init__(self, n_layers: int, interval_steps: int, model, seed: int = 0):
        self.n_layers = n_layers
        self.interval_steps = interval_steps
        self.model = model
        self.layers = find_decoder_layers(model)
        self.total_layers = len(self.layers)
        invalidInputError(0 < n_layers <= self.total_layers, "n_layers must be in [1, number of decoder layers]")
        self.active_layers_indices = []
        self._rng = random.Random(seed)

    @staticmethod
    def _trainable(p):
        return p.is_floating_point() and not hasattr(p, "qtype")

    def freeze_all_layers(self):
        for layer in self.layers:
            for p in layer.parameters():
                p.requires_grad = False

    def on_step_begin(self, args, state, control, **kwargs):
        if state.global_step % self.interval_steps == 0:
            self.switch_active_layers()

    def switch_active_layers(self):
        self.freeze_all_layers()
        self.active_layers_indices = sorted(self._rng.sample(range(self.total_layers), self.n_layers))
        print(f"Activating layers at indices: {self.active_layers_indices} for the next steps.", flush=True)
        for idx in self.active_layers_indices:
            for p in self.layers[idx].parameters():
                if self._trainable(p):
                    p.requires_grad = True
