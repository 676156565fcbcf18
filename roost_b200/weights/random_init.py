"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a configuration and a seed.

Every tensor has its own generator seeded from the model seed and a hash of the tensor's name, so the values
do not depend on the order tensors are written in, nor on which other tensors exist (the property of the
reference's seeded tiny weights, src/Starlings.Roost.Models.Tiny/TinyWeights.cs:22-32). Matrices and the
embedding are N(0, std); norm weights are 1, or 1 + N(0, norm_std). Values are drawn in float32 and rounded
to the config's ``torch_dtype``.

A second mode, ``reference``, draws every tensor exactly as the reference's own generator does for a model of the same
sizes (``reference_tensors``): with the reference's seed and its roost-tiny sizes the folder holds the very weights the
reference's tests run, so its pinned greedy tokens can be asked of this engine.
"""
from __future__ import annotations

import hashlib
import json
import math
from pathlib import Path

import numpy as np
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


REFERENCE_TINY_SEED = 0x524F4F53540001   # the seed of the reference's dense tiny model (src/Starlings.Roost.Models.Tiny/TinyConfig.cs:63-66)
_U64 = (1 << 64) - 1


def reference_slot_values(model_seed: int, slot: str, shape: tuple) -> np.ndarray:
    """The values of one weight slot as the reference's generator draws them, in float64 before rounding to the stored
    dtype (src/Starlings.Roost.Models.Tiny/TinyWeights.cs:45-78,155-162): the generator's state starts at the model seed
    xor the 64-bit FNV-1a hash of the slot name's characters; draw i is SplitMix64 of state + (i + 1) * 0x9E3779B97F4A7C15;
    u = (draw >> 11) * 2^-53; the value is 1 + (2u - 1) * 0.1 for a slot whose name ends in "norm", (2u - 1) for "embed",
    (2u - 1) * 1.5 / sqrt(last dimension) for every other slot."""
    h = 0xCBF29CE484222325
    for ch in slot:
        h = ((h ^ ord(ch)) * 0x100000001B3) & _U64
    state = np.uint64((model_seed ^ h) & _U64)
    count = int(np.prod(shape))
    with np.errstate(over="ignore"):     # arithmetic modulo 2^64 is the generator's definition
        z = state + np.arange(1, count + 1, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z ^= z >> np.uint64(31)
    u = (z >> np.uint64(11)).astype(np.float64) * 2.0 ** -53
    if slot.endswith("norm"):
        offset, amplitude = 1.0, 0.1
    elif slot == "embed":
        offset, amplitude = 0.0, 1.0
    else:
        offset, amplitude = 0.0, 1.5 / math.sqrt(shape[-1])
    return (offset + (2.0 * u - 1.0) * amplitude).reshape(shape)


def reference_tensors(config: dict, model_seed: int = REFERENCE_TINY_SEED) -> dict[str, torch.Tensor]:
    """Checkpoint tensors drawn by the reference's generator, slot by slot under the reference's slot names, each rounded
    to float32 and then to the config's ``torch_dtype`` as the reference rounds (TinyWeights.cs:86-91); a slot that
    spans several checkpoint tensors (gate_up) is cut into them by rows."""
    reader = ConfigReader(config, "config")
    arch = registry.resolve(reader)
    if arch.reference_slots is None:
        raise ValueError(f"the reference defines no model of architecture {arch.name}: its generator's slot names are not known")
    cfg = arch.read_config(reader)
    dtype = _DTYPES[arch.to_spec(cfg, None).stored_dtype]
    out = {}
    for slot, shape, names in arch.reference_slots(cfg):
        t = torch.from_numpy(reference_slot_values(model_seed, slot, shape).astype(np.float32)).to(dtype)
        rows = shape[0] // len(names)
        for i, n in enumerate(names):
            out[n] = t[i * rows : (i + 1) * rows].clone() if len(names) > 1 else t
    return out


def write_random_model(model_dir, config: dict, seed: int, std: float = 0.02, norm_std: float = 0.0, mode: str = "normal") -> Path:
    """Writes ``config`` as config.json and seeded random weights as model.safetensors; returns the folder. ``mode``
    "normal": N(0, std) matrices; "reference": the reference's generator with ``seed`` as its model seed."""
    if mode not in ("normal", "reference"):
        raise ValueError(f"random-weights mode '{mode}' is neither normal nor reference")
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(config, seed, std, norm_std) if mode == "normal" else reference_tensors(config, seed)
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
