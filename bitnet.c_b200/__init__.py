"""bitnet.c_b200: a small B200-native library for Llama-style dense decoders.

Entry points: ``load_model`` (a folder with config.json and model.safetensors),
``write_random_model`` (a seeded model folder from a configuration), ``Model.step`` (one step
of a batch of sequences from the cache) and ``generate`` (the generation loop).
"""
__version__ = "0.1.0"

from .config import ConfigError, LlamaConfig, known_architectures  # noqa: E402,F401
from .weights import WeightsError, write_random_model  # noqa: E402,F401
from .cache import Cache, CacheError, CacheFull  # noqa: E402,F401
from .engine import Completion, Diagnostics, Model, SeqStep, StepError  # noqa: E402,F401
from .engine import generate_with_model as generate  # noqa: E402,F401
from .sampling import SamplingParams  # noqa: E402,F401


def load_model(model_dir: str, dtype: str = "bfloat16", device: str = "cuda:0", max_seq: int = 0) -> "Model":
    """Load the model in ``model_dir``; its class is chosen by config.json's ``architectures``.

    ``dtype='float32'`` runs everything in true single precision (float32 weights, cache and
    products; no reduced-precision matrix mode).  ``max_seq`` caps the context like the
    reference's ``--maxseq``.
    """
    import torch
    # float32 products are true float32 everywhere (also for a float32 tensor in a bfloat16 model)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    return Model.from_dir(model_dir, dtype=dtype, device=device, max_seq=max_seq)


def load_plugins(modules) -> None:
    """Import the named Python modules.  A module may register parts (``parts.register_mixer`` and
    the like) or a whole architecture (``config.register_architecture``) of its own, which
    ``load_model`` then finds by config.json's ``architectures`` like the ones that ship; this is
    what the command line's and ``bin/trace_run``'s ``--plugin`` do."""
    import importlib
    for name in modules or ():
        try:
            importlib.import_module(name)
        except ImportError as e:
            raise ConfigError(f"plugin module '{name}' cannot be imported: {e}") from None
