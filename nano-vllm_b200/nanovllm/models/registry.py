"""Model registry: the architecture named by a checkpoint's config.json -> (configuration reader, model class).

Two kinds of config.json are understood: Hugging Face ones (``architectures: [...]``, read through ``AutoConfig``) and
self-describing ones with a single ``architecture`` key, whose reader lives next to the model."""
from __future__ import annotations

import json
import os


def _qwen3():
    from .qwen3 import Qwen3ForCausalLM
    return Qwen3ForCausalLM


def _tafopel():
    from .tafopel import TafopelForCausalLM
    return TafopelForCausalLM


def _tafopel_config(raw: dict):
    from .tafopel import TafopelConfig
    return TafopelConfig(raw)


def _tipetar():
    from .tipetar import TipetarForCausalLM
    return TipetarForCausalLM


def _tipetar_config(raw: dict):
    from .tipetar import TipetarConfig
    return TipetarConfig(raw)


def _musavik():
    from .musavik import MusavikForCausalLM
    return MusavikForCausalLM


def _musavik_config(raw: dict):
    from .musavik import MusavikConfig
    return MusavikConfig(raw)


def _fegolorn():
    from .fegolorn import FegolornForCausalLM
    return FegolornForCausalLM


def _fegolorn_config(raw: dict):
    from .fegolorn import FegolornConfig
    return FegolornConfig(raw)


MODELS = {"Qwen3ForCausalLM": _qwen3, "Qwen2ForCausalLM": _qwen3, "Tafopel": _tafopel, "Tipetar": _tipetar, "Musavik": _musavik, "Fegolorn": _fegolorn}
CONFIG_READERS = {"Tafopel": _tafopel_config, "Tipetar": _tipetar_config, "Musavik": _musavik_config, "Fegolorn": _fegolorn_config}


def architecture_of(hf_config) -> str:
    names = getattr(hf_config, "architectures", None) or []
    for n in names:
        if n in MODELS:
            return n
    return "Qwen3ForCausalLM"          # configurations built by hand (tests, synthetic presets) carry no name


def model_class(hf_config):
    return MODELS[architecture_of(hf_config)]()


def read_config(model_dir: str):
    """The model configuration of a checkpoint directory."""
    path = os.path.join(model_dir, "config.json")
    if os.path.isfile(path):
        with open(path) as f:
            raw = json.load(f)
        arch = raw.get("architecture")
        if arch is not None:
            if arch not in CONFIG_READERS:
                raise ValueError(f"unknown architecture {arch!r} in {path}")
            return CONFIG_READERS[arch](raw)
    from transformers import AutoConfig
    return AutoConfig.from_pretrained(model_dir)
