"""Mirror of InferEngine (crates/atlas-infer/src/engine.rs:132-218) for the hook-less path:
generate() returns (tokens, deposits) with deposits empty, exactly what the reference returns
when no StigmergicHook is attached; a hook makes the reference fall back to its CPU model,
which this library does not contain."""
from ._ffi import AtlasError
from .model import OlmoModel, SamplingConfig


class InferEngine:
    def __init__(self, model: OlmoModel):
        self.model = model
        self.hook = None

    def has_hook(self):
        return self.hook is not None

    def set_hook(self, hook):
        if hook is not None:
            raise AtlasError("hooks run on the reference's CPU path; the GPU path has none")
        self.hook = None

    def generate(self, prompt, max_new, cfg: SamplingConfig):
        return self.model.generate_with_sampling(prompt, max_new, cfg), []

    def generate_streaming(self, prompt, max_new, cfg: SamplingConfig, on_token):
        count = 0
        for tok in self.model.generate_with_sampling(prompt, max_new, cfg):
            count += 1
            if not on_token(tok, None):
                break
        return count

    def reset(self):
        self.model.reset()
