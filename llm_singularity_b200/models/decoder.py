"""The generic decoder: embedding -> blocks in the spec's run order -> head.

Nothing here is specific to one architecture.  ``ModelSpec.blocks`` gives the
parts of each block, ``ModelSpec.order`` the sequence of calls (a block may be
called twice, and a call may read the cache another call wrote), and
``ModelSpec.tensor_names`` the checkpoint names of every parameter.  The
reference's counterpart is ``LlamaModel::forward_impl``
(models/llama/llama_model.cpp:298-726), which hard-wires one block shape and runs
prompts and decode tokens in separate passes; here one pass serves any mix.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..config.specs import ModelSpec
from ..parts import BLOCKS
from ..parts.base import ParamSpec, Part, Runtime
from ..parts.embedding import Embedding, LMHead


class DecoderModel:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.embedding = Embedding(spec.embedding, rt)
        self.blocks: List[Part] = [BLOCKS.build(b, rt) for b in spec.blocks]
        self.head = LMHead(spec.head, rt)
        for call in spec.order:
            if not 0 <= call.block < len(self.blocks):
                raise ValueError(f"run order names block {call.block}, model has {len(self.blocks)}")

    # --------------------------------------------------------------- parameters
    def _owners(self) -> Dict[str, Part]:
        owners: Dict[str, Part] = {}

        def walk(path: str, part: Part):
            owners[path] = part
            for name, child in part.children().items():
                walk(f"{path}.{name}", child)

        walk("embedding", self.embedding)
        walk("head", self.head)
        for i, b in enumerate(self.blocks):
            walk(f"blocks.{i}", b)
        return owners

    def expected_tensors(self) -> Dict[str, Tuple[str, str, ParamSpec]]:
        """checkpoint name -> (owner path, local name, ParamSpec); checks the spec's map."""
        owners = self._owners()
        declared = {(path, local): ps for path, part in owners.items()
                    for local, ps in type(part).params(part.spec).items()}
        out: Dict[str, Tuple[str, str, ParamSpec]] = {}
        for ckpt_name, (path, local) in self.spec.tensor_names:
            if (path, local) not in declared:
                raise ValueError(f"spec maps '{ckpt_name}' to {path}.{local}, which no part declares")
            out[ckpt_name] = (path, local, declared.pop((path, local)))
        if declared:
            missing = ", ".join(f"{p}.{l}" for p, l in sorted(declared))
            raise ValueError(f"spec gives no checkpoint name for: {missing}")
        return out

    def load_tensors(self, tensors: Dict[str, torch.Tensor]) -> None:
        """``tensors``: checkpoint name -> CPU tensor, already checked against
        ``expected_tensors``.  Matrices and tables go to the compute dtype, vectors
        to 32-bit, integer tables to int32."""
        owners = self._owners()
        per_owner: Dict[str, Dict[str, torch.Tensor]] = {p: {} for p in owners}
        for ckpt_name, (path, local, ps) in self.expected_tensors().items():
            t = tensors[ckpt_name]
            if ps.role in ("matrix", "table"):
                dt = self.rt.dtype
            elif ps.role == "int_table":
                dt = torch.int32
            else:
                dt = torch.float32
            per_owner[path][local] = t.to(device=self.rt.device, dtype=dt)
        for path, part in owners.items():
            if per_owner[path] or type(part).params(part.spec):
                part.load(per_owner[path])
        if self.spec.head.tied:
            self.head.tie(self.embedding)

    # -------------------------------------------------------------------- cache
    def cache_specs(self) -> List[object]:
        """What each cache id of the run order must hold (from the mixer that writes it)."""
        specs: List[object] = [None] * self.spec.num_caches
        for call in self.spec.order:
            cs = self.blocks[call.block].mixer.cache_spec()
            if call.writes_cache or specs[call.cache] is None:
                if specs[call.cache] is not None and specs[call.cache] != cs and call.writes_cache:
                    raise ValueError(f"cache {call.cache} is written by mixers with different needs")
                specs[call.cache] = cs
        return specs

    def required_kernels(self) -> List[str]:
        names = []
        for part in self._owners().values():
            for k in getattr(part, "kernels", ()):
                if k not in names:
                    names.append(k)
        if self.rt.dtype == torch.bfloat16 and "gemm" in names:
            names += ["gemm_tc", "gemm_small", "gemm_stream"]    # bfloat16 products run on the tensor cores
        return names

    # ------------------------------------------------------------------ forward
    def forward(self, ctx, caches) -> torch.Tensor:
        """Run this step's tokens through every layer call; logits ``[wanted, vocab]``."""
        residual = self.embedding.forward(ctx.token_ids)
        pending = None
        for call in self.spec.order:
            pending = self.blocks[call.block].forward(
                residual, pending, ctx, caches.view(call.cache, ctx), call.writes_cache)
        if ctx.n_wanted == 0:
            return torch.empty(0, self.spec.head.vocab_size, dtype=torch.float32,
                               device=self.rt.device)
        return self.head.forward(residual, pending, ctx.want_rows)
