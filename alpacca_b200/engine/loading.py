"""From a model folder (or a configuration and a seed) to a model with weights."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config import ModelConfig, config_from_dict, get_architecture, load_config
from ..parts.base import BuildOptions
from ..weights import FolderSource, RandomSource, write_safetensors
from .model import DecoderModel

DTYPE_BY_NAME = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
                 "fp32": torch.float32, "f32": torch.float32}


DEFAULT_MAX_POSITIONS = 4096   # for a configuration that sets no limit (alpacca/model.py:211 has the same default)


def resolve_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype} is not supported (bfloat16 or float32)")
        return dtype
    try:
        return DTYPE_BY_NAME[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"dtype {dtype!r} is not supported (bfloat16 or float32)") from None


def build_model(config: ModelConfig | dict, dtype=torch.bfloat16, device="cuda",
                max_positions: int | None = None) -> DecoderModel:
    """The model of `config`'s architecture, without weights."""
    if isinstance(config, dict):
        config = config_from_dict(config)
    arch = get_architecture(config.architecture)
    limit = config.max_positions or DEFAULT_MAX_POSITIONS
    opts = BuildOptions(dtype=resolve_dtype(dtype), device=device,
                        max_positions=min(int(max_positions), limit) if max_positions else limit)
    return DecoderModel(arch.build(config, opts), opts, config)


def load_model_dir(model_dir, dtype=torch.bfloat16, device="cuda", max_positions: int | None = None) -> DecoderModel:
    """config.json chooses the model class; model.safetensors is read by tensor name."""
    config = load_config(model_dir)
    model = build_model(config, dtype, device, max_positions)
    source = FolderSource(model_dir)
    try:
        model.load_weights(source, where=str(model_dir))
    finally:
        source.close()
    return model


def random_model(config: ModelConfig | dict, seed: int, dtype=torch.bfloat16, device="cuda",
                 max_positions: int | None = None, std: float = 0.02) -> DecoderModel:
    """A model whose weights are drawn on the device from `seed` (no folder is written)."""
    model = build_model(config, dtype, device, max_positions)
    gen_device = "cuda" if torch.device(device).type == "cuda" else "cpu"
    model.load_weights(RandomSource(model.param_specs(), seed, resolve_dtype(dtype), std, device=gen_device),
                       where="random weights")
    return model


def write_random_model_dir(model_dir, config: ModelConfig | dict, seed: int, dtype=torch.bfloat16,
                           std: float = 0.02) -> Path:
    """Random-weights mode: writes config.json and model.safetensors for `config` from `seed`.

    Tensor names and shapes are the ones the architecture's parts declare; the
    values of a tensor depend on (seed, its name) only.
    """
    if isinstance(config, dict):
        config = config_from_dict(config)
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    model = build_model(config, dtype, device="cpu")
    source = RandomSource(model.param_specs(), seed, resolve_dtype(dtype), std, device="cpu")
    out = config.to_dict()
    out["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}[resolve_dtype(dtype)]
    (model_dir / "config.json").write_text(json.dumps(out, indent=1))
    entries = [(name, dt, shape, (lambda n=name: source.get(n))) for name, (dt, shape) in source.table().items()]
    write_safetensors(model_dir / "model.safetensors", entries, metadata={"format": "pt", "seed": seed})
    return model_dir
