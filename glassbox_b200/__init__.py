"""glassbox_b200: a small, whole inference engine for one B200, for the Llama-family decoder
that Glassbox runs (SmolLM2): typed configuration and an architecture registry (``config``, ``models``),
safetensors weights (``weights``), layers put together from parts (``parts``), a paged cache manager
(``cache``), one step function, a scheduler and trace replay (``engine``), sampling, and hand-written CUDA
kernels for sm_100a (``csrc``, called through ``kernels``)."""
from . import models  # noqa: F401  (registers the architectures)
from . import parts  # noqa: F401   (registers the parts)
from .config import ConfigError, load_config, parse_config, register_architecture
from .weights import WeightsError, write_random_model



def load(model_dir, dtype="bfloat16", **kwargs):
    """Load a model folder for generation; see ``glassbox_b200.api.LLM``."""
    from .api import load as _load
    return _load(model_dir, dtype, **kwargs)


__version__ = "0.1.0"
__all__ = ["ConfigError", "WeightsError", "load", "load_config", "parse_config", "register_architecture",
           "write_random_model"]
