"""Importing this package registers every architecture the engine knows."""
from . import lfm2  # noqa: F401
from .decoder import DecoderModel

__all__ = ["DecoderModel", "load_model"]


def load_model(folder: str, dtype, device="cuda:0"):
    """(typed config, plan, DecoderModel) for a folder with config.json and
    model.safetensors; the architecture is chosen by config.json."""
    import torch
    from .. import parts  # noqa: F401  (registers the built-in parts)
    from ..config import load_config, parse_dtype
    from ..weights import load_weights
    dtype = parse_dtype(dtype)
    if not torch.cuda.is_available():
        raise RuntimeError("cellm_b200 runs on a CUDA GPU only; none is visible")
    cfg, plan = load_config(folder)
    tensors = load_weights(folder, plan, dtype, device)
    return cfg, plan, DecoderModel(plan, tensors, dtype, device)
