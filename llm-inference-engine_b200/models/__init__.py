"""Model registry: config.json names an architecture, the registry names the class that reads that configuration and its checkpoint and
builds the engine that serves it.

    model = load_model(model_dir, dtype="bfloat16", device="cuda:0", max_tokens=4096, max_seqs=4)

Every entry builds on the package's engines: the Llama-2 family on the fused decoder (weights.build_decoder), layer-list designs on the
hybrid decoder (hybrid.HybridDecoder)."""
import importlib
import json
import os

_REGISTRY = {}


def register(*names):
    def deco(cls):
        for n in names:
            _REGISTRY[n.lower()] = cls
        return cls
    return deco


def architectures():
    _populate()
    return sorted(_REGISTRY)


def _populate():
    for sub in ("vasolix", "zefenex", "fedovik", "silonex", "llama"):
        importlib.import_module(f"{__name__}.{sub}")


def architecture_of(config):
    name = config.get("architecture") or (config.get("architectures") or [None])[0] or config.get("model_type")
    if not name:
        raise ValueError("config.json names no architecture")
    return name


def load_model(model_dir, dtype="bfloat16", device="cuda:0", **limits):
    """Reads model_dir/config.json, picks the class by its architecture and lets it load model_dir's checkpoint."""
    _populate()
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    name = architecture_of(config)
    cls = _REGISTRY.get(name.lower())
    if cls is None:
        raise ValueError(f"architecture {name!r} is not served; known: {architectures()}")
    return cls.from_pretrained(model_dir, config, dtype=dtype, device=device, **limits)
