"""janus_b200: a small Llama inference library for one B200 (sm_100a).

    model = janus_b200.load(model_dir, dtype="bfloat16", max_tokens=8192)
    tokens, stats = model.generate([[1, 2, 3]], max_tokens=16)
"""
from .api import Model, load, load_random

__version__ = "0.1.0"
__all__ = ["Model", "load", "load_random", "__version__"]
