"""cellm_b200: an LFM2 inference engine for one B200 GPU, in the manner of
jeffasante/cellm: model folder in, tokens out, over a paged cache."""
from . import parts as _parts    # noqa: F401  registers the built-in parts
from . import models as _models  # noqa: F401  registers the architectures

__version__ = "0.1.0"
