"""Weights from safetensors by tensor name.

A model declares, per scope and part-local parameter, the shape it wants and the checkpoint tensors that make
it up (several names = rows concatenated in order, the reference's "a+b" source,
src/Starlings.Roost.Models.Tiny/RoostTiny.cs:35). Every name is checked before any tensor is read: missing
tensors, unexpected tensors and wrong shapes are reported together in one ``WeightError``
(the reference fails per tensor, src/Starlings.Roost.Worker/Weights/ModelWeightLoader.cs:190-215).

Stored dtypes are kept: bfloat16 stays bfloat16, a tensor stored in 32-bit stays 32-bit, float16 is widened to
float32, integer tables become int32. What a part then does with its parameter (matrices go to the compute
dtype, vectors stay as stored; the 32-bit path widens everything) is decided by ``ParamDecl.role``.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=(), index_faults=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.index_faults = list(index_faults)   # disagreements between a shard index and its shards


def checkpoint_index(model_dir) -> dict | None:
    """The ``weight_map`` (tensor name -> shard file name) of model.safetensors.index.json, or None when the folder holds
    a single model.safetensors. The reference's loader reads one file (src/Starlings.Roost.Worker/Weights/
    ModelWeightLoader.cs:198-221); checkpoints of the sizes this engine serves come in shards with this index beside
    them."""
    model_dir = Path(model_dir)
    if (model_dir / "model.safetensors").exists():
        return None
    index = model_dir / "model.safetensors.index.json"
    if not index.exists():
        raise WeightError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json is present")
    try:
        weight_map = json.loads(index.read_text())["weight_map"]
    except (json.JSONDecodeError, KeyError, TypeError) as e:
        raise WeightError(f"{index}: not a shard index (no readable 'weight_map': {e})") from None
    if not isinstance(weight_map, dict) or not all(isinstance(k, str) and isinstance(v, str) for k, v in weight_map.items()):
        raise WeightError(f"{index}: 'weight_map' must map tensor names to shard file names")
    return weight_map


def checkpoint_files(model_dir) -> list[Path]:
    """model.safetensors, or the shards named by model.safetensors.index.json."""
    model_dir = Path(model_dir)
    weight_map = checkpoint_index(model_dir)
    if weight_map is None:
        return [model_dir / "model.safetensors"]
    return [model_dir / n for n in sorted(set(weight_map.values()))]


def checkpoint_has(model_dir, name: str) -> bool:
    weight_map = checkpoint_index(model_dir)
    if weight_map is not None:
        return name in weight_map      # the index says what the checkpoint holds
    with SafetensorsFile(Path(model_dir) / "model.safetensors") as st:
        return name in st.entries


def expected_tensors(decls: dict, names: dict) -> dict[str, tuple]:
    """Checkpoint tensor name -> shape, from the parts' declarations and the architecture's name map."""
    out = {}
    for scope, params in decls.items():
        for local, decl in params.items():
            try:
                srcs = names[scope][local]
            except KeyError:
                raise WeightError(f"the architecture names no checkpoint tensor for parameter '{local}' of '{scope}'") from None
            if len(srcs) == 1:
                out[srcs[0]] = tuple(decl.shape)
            else:
                if decl.row_splits is None or len(decl.row_splits) != len(srcs):
                    raise WeightError(f"parameter '{local}' of '{scope}' is made of {len(srcs)} tensors but declares row splits {decl.row_splits}")
                for s, rows in zip(srcs, decl.row_splits):
                    out[s] = (rows, *decl.shape[1:])
    return out


def _stored(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32):
        return t
    if t.dtype in (torch.float16, torch.float64):
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.int32, torch.bool):
        return t.to(torch.int32)
    raise WeightError(f"a tensor of dtype {t.dtype} cannot be kept")


def load_checkpoint(model_dir, decls: dict, names: dict, allow_unexpected=()) -> dict[str, dict[str, torch.Tensor]]:
    """scope -> local name -> tensor on the host, concatenated as declared."""
    weight_map = checkpoint_index(model_dir)
    files = checkpoint_files(model_dir)
    opened = []
    try:
        try:
            opened = [SafetensorsFile(f) for f in files]
        except SafetensorsError as e:
            raise WeightError(str(e)) from None
        where = {}
        index_faults = []
        if weight_map is None:
            for n in opened[0].names():
                where[n] = opened[0]
        else:
            # the index is what the checkpoint says it holds: a tensor is read from the shard the index names, a tensor
            # a shard holds without the index naming it does not exist for the model, and both disagreements are told
            by_name = {st.path.name: st for st in opened}
            for n, shard in weight_map.items():
                if n in by_name[shard].entries:
                    where[n] = by_name[shard]
                else:
                    index_faults.append(f"{n} is named for {shard}, which does not hold it")
            for st in opened:
                for n in st.names():
                    if weight_map.get(n) != st.path.name:
                        index_faults.append(f"{n} lies in {st.path.name} but the index " +
                                            (f"names {weight_map[n]} for it" if n in weight_map else "does not name it"))
        want = expected_tensors(decls, names)
        missing = [n for n in want if n not in where]
        unexpected = [n for n in where if n not in want and n not in allow_unexpected]
        wrong = [(n, tuple(where[n].entries[n].shape), shape) for n, shape in want.items()
                 if n in where and tuple(where[n].entries[n].shape) != shape]
        if missing or unexpected or wrong or index_faults:
            lines = [f"{Path(model_dir)}: the checkpoint does not match the model"]
            if index_faults:
                lines.append(f"  shard index ({len(index_faults)}): " + "; ".join(index_faults))
            if missing:
                lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
            if unexpected:
                lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
            if wrong:
                lines.append(f"  wrong shape ({len(wrong)}): " + ", ".join(f"{n} is {list(g)}, expected {list(w)}" for n, g, w in wrong))
            raise WeightError("\n".join(lines), missing, unexpected, wrong, index_faults)
        out: dict[str, dict[str, torch.Tensor]] = {}
        for scope, params in decls.items():
            out[scope] = {}
            for local in params:
                parts = [_stored(where[n].tensor(n)) for n in names[scope][local]]
                out[scope][local] = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
        return out
    finally:
        for st in opened:
            st.close()
