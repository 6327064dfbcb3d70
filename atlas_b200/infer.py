"""Mirror of the reference's atlas-infer crate: InferEngine (crates/atlas-infer/src/engine.rs:132-218),
StigmergicHook (src/hook.rs:31-33) and PheromoneDeposit (engine.rs:34-43).

Without a hook generate() is the model's own generate_with_sampling and returns no deposits.  With a
hook the reference falls back to its CPU model (engine.rs:144-162); here the GPU path is kept: the
layer outputs of every forward are copied to pinned host memory behind the step and the hook runs on
the host while the next forward executes on the device."""
from dataclasses import dataclass
from typing import List, Optional

import numpy as np

from . import _ffi
from ._ffi import check
from .model import OlmoModel, SamplingConfig


class StigmergicHook:
    """on_layer(layer_idx, hidden) -> Optional[float]; hidden is a read-only float32 view of d_model values."""

    def on_layer(self, layer_idx: int, hidden: np.ndarray) -> Optional[float]:
        return None


@dataclass
class PheromoneDeposit:
    token_id: int
    total_delta: float
    layers_fired: int


class InferEngine:
    def __init__(self, model: OlmoModel):
        self.model = model
        self.hook = None
        self._cb = None

    def with_hook(self, hook):
        self.set_hook(hook)
        return self

    def has_hook(self):
        return self.hook is not None

    def set_hook(self, hook):
        """Replace or clear (None) the hook at run time."""
        self.hook = hook
        self._cb = self.model.set_layer_hook(None if hook is None else hook.on_layer)

    def generate(self, prompt, max_new, cfg: SamplingConfig, seed=None):
        toks = self.model.generate_with_sampling(prompt, max_new, cfg, seed=seed)
        if self.hook is None:
            return toks, []
        return toks, [PheromoneDeposit(t, d, f) for t, d, f in self.model.deposits()]

    def generate_streaming(self, prompt, max_new, cfg: SamplingConfig, on_token, seed=None):
        """engine.rs:171-217 — on_token(token, deposit or None) -> keep going?; returns the number of tokens seen.
        Without a hook the tokens are handed over while the generation runs and a false return ends it;
        with a hook the reference generates first and then walks the tokens, and so does this."""
        count = 0
        if self.hook is None:
            def each(tok):
                nonlocal count
                count += 1
                return on_token(tok, None)
            self.model.generate_streaming(prompt, max_new, cfg, each, seed=seed)
            return count
        toks, deps = self.generate(prompt, max_new, cfg, seed=seed)
        for tok, dep in zip(toks, deps):
            count += 1
            if not on_token(tok, dep):
                break
        return count

    def reset(self):
        self.model.reset()
