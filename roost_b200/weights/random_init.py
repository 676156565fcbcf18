"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a configuration and a seed.

Every tensor has its own generator seeded from the model seed and a hash of the tensor's name, so the values
do not depend on the order tensors are written in, nor on which other tensors exist (the property of the
reference's seeded tiny weights, src/Starlings.Roost.Models.Tiny/TinyWeights.cs:22-32). Matrices and the
embedding are N(0, std); norm weights are 1, or 1 + N(0, norm_std). Values are drawn in float32 and rounded
to the config's ``torch_dtype``.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from ..config.reader import ConfigReader
from .. import registry
from .loader import expected_tensors
from .safetensors_io import write_safetensors

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _tensor_seed(seed: int, name: str) -> int:
    h = int.from_bytes(hashlib.sha256(name.encode()).digest()[:8], "little")
    return (seed ^ h) & ((1 << 63) - 1)


def random_tensors(config: dict, seed: int, std: float = 0.02, norm_std: float = 0.0) -> dict[str, torch.Tensor]:
    from ..engine.model import parameter_declarations
    reader = ConfigReader(config, "config")
    arch = registry.resolve(reader)
    cfg = arch.read_config(reader)
    spec = arch.to_spec(cfg, None)
    decls = parameter_declarations(spec)
    shapes = expected_tensors(decls, spec.weight_names)
    roles = {}
    for scope, params in decls.items():
        for local, decl in params.items():
            for n in spec.weight_names[scope][local]:
                roles[n] = decl.role
    dtype = _DTYPES[spec.stored_dtype]
    out = {}
    for name, shape in shapes.items():
        g = torch.Generator().manual_seed(_tensor_seed(seed, name))
        if roles[name] == "vector":
            t = torch.ones(shape, dtype=torch.float32)
            if norm_std > 0:
                t += torch.randn(shape, generator=g, dtype=torch.float32) * norm_std
        else:
            t = torch.randn(shape, generator=g, dtype=torch.float32) * std
        out[name] = t.to(dtype)
    return out


def write_random_model(model_dir, config: dict, seed: int, std: float = 0.02, norm_std: float = 0.0) -> Path:
    """Writes ``config`` as config.json and seeded random weights as model.safetensors; returns the folder."""
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(config, seed, std, norm_std)
    (model_dir / "config.json").write_text(json.dumps(config, indent=2) + "\n")
    write_safetensors(model_dir / "model.safetensors", tensors, metadata={"format": "pt", "seed": seed})
    return model_dir


def random_parameters(spec, seed: int, device, dtype: torch.dtype, std: float = 0.02, norm_std: float = 0.0) -> dict:
    """scope -> local name -> tensor, drawn on ``device`` in ``dtype`` without a file: the random-weights mode of
    benchmarks, where a model of many gigabytes is made where it will live. Seeded per parameter like
    ``random_tensors`` (the values differ from the file-writing mode, which draws on the host)."""
    from ..engine.model import parameter_declarations
    out: dict = {}
    for scope, params in parameter_declarations(spec).items():
        out[scope] = {}
        for local, decl in params.items():
            g = torch.Generator(device=device).manual_seed(_tensor_seed(seed, f"{scope}.{local}"))
            if decl.role == "vector":
                t = torch.ones(decl.shape, dtype=torch.float32, device=device)
                if norm_std > 0:
                    t += torch.randn(decl.shape, generator=g, dtype=torch.float32, device=device) * norm_std
                out[scope][local] = t.to(dtype)
            else:
                t = torch.empty(decl.shape, dtype=dtype, device=device)
                rows = max(1, (1 << 26) // max(1, t[0].numel()))  # draw in slabs: no float32 copy of a whole matrix
                for r0 in range(0, decl.shape[0], rows):
                    part = t[r0 : r0 + rows]
                    part.copy_(torch.randn(part.shape, generator=g, dtype=torch.float32, device=device) * std)
                out[scope][local] = t
    return out
