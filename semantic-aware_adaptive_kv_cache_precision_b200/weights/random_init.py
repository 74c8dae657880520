"""Random weights from a configuration and a seed.

`write_random_model` writes a model folder (config.json, model.safetensors) that
loads like any checkpoint. Every tensor has its own generator, keyed by the seed
and the tensor's name, so a tensor's values do not depend on which other tensors
the model has. Matrices and biases are N(0, std) with std the configuration's
`initializer_range`; norm weights are 1 + N(0, std). The reference has no such
mode (it only loads real checkpoints, `src/microinfer/engine.py:927-974`).

`random_arena` fills the device allocation directly with the device's generator,
for models too large to write to disk first (benchmarks).
"""

from __future__ import annotations

import json
import zlib
from pathlib import Path

import numpy as np
import torch

from .decl import TensorDecl
from .loader import WeightArena
from .safetensors_io import write_safetensors

_TORCH = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def random_tensor(decl: TensorDecl, seed: int, std: float, dtype: torch.dtype) -> torch.Tensor:
    rng = np.random.default_rng([int(seed), zlib.crc32(decl.name.encode())])
    shape = tuple(int(s) for s in decl.shape)
    if decl.integer:
        return torch.from_numpy(rng.integers(0, 2 ** 15, size=shape, dtype=np.int32))
    if decl.init == "zeros":
        values = np.zeros(shape, dtype=np.float32)
    else:
        values = rng.standard_normal(shape, dtype=np.float32) * np.float32(std)
        if decl.init == "ones_normal":
            values += np.float32(1.0)
    return torch.from_numpy(values).to(dtype)


def write_random_model(folder, config, seed: int, dtype: str | None = None) -> Path:
    """Write `folder/config.json` and `folder/model.safetensors` for `config` (a
    configuration object of a registered architecture, or its dict)."""
    from ..config import config_from_dict
    from ..engine.model import DecoderModel
    if isinstance(config, dict):
        config = config_from_dict(config)
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    spec = config.model_spec()
    stored = _TORCH[dtype or spec.stored_dtype]
    decls = DecoderModel.tensor_decls_of(spec)

    class _Maker:
        def __init__(self, decl):
            self.decl, self.shape = decl, tuple(decl.shape)
            self.dtype = torch.int32 if decl.integer else stored

        def __call__(self):
            return random_tensor(self.decl, seed, spec.init_std, self.dtype)

    raw = config.to_dict()
    raw["torch_dtype"] = dtype or spec.stored_dtype
    (folder / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", {d.name: _Maker(d) for d in decls},
                      metadata={"format": "pt", "seed": seed})
    return folder


def random_arena(decls: list[TensorDecl], seed: int, std: float, mode: str, device,
                 stored: str = "bfloat16") -> WeightArena:
    """A weight arena filled on the device; same distributions as the written mode
    but the device's own random stream."""
    from .loader import device_dtype
    code = {"bfloat16": "BF16", "float16": "F16", "float32": "F32"}[stored]
    stored_dtype = _TORCH[stored]
    dtypes = {d.name: device_dtype("I32" if d.integer else code, mode) for d in decls}
    arena = WeightArena(decls, dtypes, device)
    gen = torch.Generator(device=device)
    for d in decls:
        gen.manual_seed((int(seed) << 32) ^ zlib.crc32(d.name.encode()))
        view = arena.view(d.name)
        if d.integer:
            view.copy_(torch.randint(0, 2 ** 15, view.shape, generator=gen, device=device,
                                     dtype=torch.int32))
        elif d.init == "zeros":
            view.zero_()
        else:
            chunk = 1 << 26
            flat = view.reshape(-1)
            for begin in range(0, flat.numel(), chunk):
                part = flat[begin:begin + chunk]
                noise = torch.randn(part.shape, generator=gen, device=device,
                                    dtype=torch.float32) * std
                if d.init == "ones_normal":
                    noise += 1.0
                part.copy_(noise.to(stored_dtype))     # the value a checkpoint would store
    return arena
