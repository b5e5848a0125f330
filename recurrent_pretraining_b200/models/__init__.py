"""Model families: depth-recurrent LM (training), GPT baseline, HF-compatible inference model."""
from . import variants  # noqa: F401  (registers the research block / MLP variants by name)
from .recurrent import GPT, RecurrentGPT  # noqa: F401


def build_model(config, **kwargs):
    if config.architecture_class_name == "RecurrentGPT":
        return RecurrentGPT(config, **kwargs)
    if config.architecture_class_name == "GPT":
        return GPT(config, **kwargs)
    raise ValueError(f"Invalid architecture {config.architecture_class_name} provided.")
