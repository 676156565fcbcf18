"""A model: blocks built from a ``ModelSpec``, run in the order of its schedule.

The forward pass of one step is: the embedding part; every schedule entry's block over the step's tokens with
that entry's cache; the final norm of the selected rows (the last residual sum fused into it); the head part, which
gives 32-bit logits (src/Starlings.Roost.Models.Tiny/RoostTiny.cs:39-56). Logits are float32 whatever
the activation dtype is, as the reference's LmHead (src/Starlings.Roost.Ops/CpuOps.cs:465-495).
"""
from __future__ import annotations

from pathlib import Path

import torch

from ..config.reader import ConfigReader
from ..config.spec import ModelSpec
from ..parts.base import BLOCKS, EMBEDDINGS, HEADS, NORMS, ParamDecl, Runtime
from ..parts.linear import Linear
from .. import registry
from ..weights import loader as weight_loader


def parameter_declarations(spec: ModelSpec) -> dict[str, dict[str, ParamDecl]]:
    """scope -> local parameter -> declaration, from the part classes alone (no device needed)."""
    decls: dict[str, dict[str, ParamDecl]] = {"embed": EMBEDDINGS.get(spec.embedding.kind).parameters(spec.embedding)}
    for i, b in enumerate(spec.blocks):
        block_cls = BLOCKS.get(b.kind)
        for part_name, (reg, part_spec) in block_cls.sub_specs(b).items():
            params = reg.get(part_spec.kind).parameters(part_spec)
            if params:
                decls[f"blocks.{i}.{part_name}"] = params
    decls["final_norm"] = NORMS.get(spec.final_norm.kind).parameters(spec.final_norm)
    if not spec.tie_embeddings:
        decls["lm_head"] = HEADS.get(spec.head.kind).parameters(spec.head)
    return decls


class Model:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.blocks = [BLOCKS.build(b, runtime) for b in spec.blocks]
        self.final_norm = NORMS.build(spec.final_norm, runtime)
        self.embedding = EMBEDDINGS.build(spec.embedding, runtime)
        self.head = HEADS.build(spec.head, runtime)
        # what each run keeps between steps (None: nothing, or another run's cache)
        self.cache_needs = []
        for n, e in enumerate(spec.schedule):
            need = self.blocks[e.block].mixer.cache_need()
            if e.reads_cache_of is not None:
                owner = self.blocks[spec.schedule[e.reads_cache_of].block].mixer.cache_need()
                if need != owner:
                    raise ValueError(f"schedule entry {n} reads the cache of entry {e.reads_cache_of}, whose geometry differs "
                                     f"({owner} against {need})")
                need = None
            self.cache_needs.append(need)

    # ------------------------------------------------------------------ weights
    def _place(self, t: torch.Tensor, decl: ParamDecl) -> torch.Tensor:
        if t.dtype == torch.int32:
            return t.to(self.rt.device)
        if self.rt.full_precision:
            return t.to(device=self.rt.device, dtype=torch.float32)
        if decl.role == "matrix":
            return t.to(device=self.rt.device, dtype=self.rt.dtype)
        return t.to(self.rt.device)  # vectors keep their stored dtype: 32-bit stays 32-bit

    def load(self, params: dict[str, dict[str, torch.Tensor]]) -> None:
        decls = parameter_declarations(self.spec)
        placed = {scope: {k: self._place(v, decls[scope][k]) for k, v in p.items()} for scope, p in params.items()}
        self.embedding.load(placed["embed"])
        for i, block in enumerate(self.blocks):
            for name, part in block.sub_parts().items():
                part.load(placed.get(f"blocks.{i}.{name}", {}))
        self.final_norm.load(placed["final_norm"])
        if self.spec.tie_embeddings:
            shared = self.embedding.tied_weight()
            if shared is None:
                raise ValueError(f"the model ties its head to its embedding, but an embedding of kind '{self.spec.embedding.kind}' has no matrix to share")
            self.head.load({"weight": shared})
        else:
            self.head.load(placed["lm_head"])

    def parts(self):
        """Every part of the model, for questions asked of all of them."""
        yield self.embedding
        yield self.head
        for b in self.blocks:
            yield b
            yield from b.sub_parts().values()

    def weight_bytes(self) -> int:
        seen, total = set(), 0

        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        for part in [self.embedding, self.head] + [p for b in self.blocks for p in b.sub_parts().values()]:
            for v in vars(part).values():
                if isinstance(v, torch.Tensor):
                    add(v)
                elif isinstance(v, Linear):
                    add(v.weight)
                elif hasattr(v, "weight") and isinstance(getattr(v, "weight"), torch.Tensor):
                    add(v.weight)
        add(self.final_norm.weight)
        return total

    # ------------------------------------------------------------------ the step's forward pass
    def forward(self, batch, storage) -> torch.Tensor:
        """Logits [selected, vocab] in float32 for ``batch.selected`` (an empty tensor when nothing is wanted)."""
        k = self.rt.kernels
        h = self.embedding(batch.ids, batch)
        residual = None
        for n, e in enumerate(self.spec.schedule):
            owner = n if e.reads_cache_of is None else e.reads_cache_of
            h, residual = self.blocks[e.block](h, residual, batch, storage.view(owner), write_cache=e.reads_cache_of is None)
        if batch.num_selected == 0:
            return torch.empty((0, self.spec.vocab), dtype=torch.float32, device=self.rt.device)
        if residual is None:
            final = self.final_norm(h, rows=batch.selected)
        else:
            final, _ = self.final_norm.add_norm(h, residual, rows=batch.selected)
        return self.head(final, batch)


def read_model_config(model_dir):
    """(architecture entry, typed configuration, reader) of a model folder."""
    reader = ConfigReader.from_path(Path(model_dir))
    arch = registry.resolve(reader)
    return arch, arch.read_config(reader), reader


def load_model(model_dir, dtype: torch.dtype, device="cuda", kernels=None) -> Model:
    """Builds the model config.json names and loads model.safetensors into it."""
    from ..kernels import library
    arch, cfg, _ = read_model_config(model_dir)
    tied = getattr(cfg, "tie_word_embeddings", None)
    if tied is None:
        tied = not weight_loader.checkpoint_has(model_dir, "lm_head.weight")
    spec = arch.to_spec(cfg, tied)
    runtime = Runtime(dtype, device, kernels if kernels is not None else library.load())
    model = Model(spec, runtime)
    decls = parameter_declarations(spec)
    allow = ("lm_head.weight",) if spec.tie_embeddings else ()
    params = weight_loader.load_checkpoint(model_dir, decls, spec.weight_names, allow_unexpected=allow)
    model.load(params)
    model.config = cfg
    return model
