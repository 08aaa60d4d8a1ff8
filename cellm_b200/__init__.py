"""cellm_b200: an LFM2 inference engine for one B200 GPU, in the manner of
jeffasante/cellm: model folder in, tokens out, over a paged cache.

    from cellm_b200 import Engine, SamplingParams
    eng = Engine("model_dir", dtype="bfloat16", total_blocks=4096)
    out = eng.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_new_tokens=16))
"""
from . import parts as _parts    # noqa: F401  registers the built-in parts
from . import models as _models  # noqa: F401  registers the architectures
from .config import EngineConfig, Lfm2Config
from .engine import Engine
from .sampling import SamplingParams
from .weights import write_random_model

__version__ = "0.1.0"
__all__ = ["Engine", "EngineConfig", "SamplingParams", "Lfm2Config", "write_random_model", "generate"]


def generate(model: str, prompts, params: SamplingParams | None = None, **engine_options):
    """One-call form: loads `model`, generates for the prompts (lists of token ids)."""
    return Engine(model, **engine_options).generate(prompts, params)
