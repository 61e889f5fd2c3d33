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
    @staticmethod
    def _own_tensors(block: Part, view) -> Dict[tuple, torch.Tensor]:
        """(path, attribute) -> tensor, for every tensor a block's parts hold and its cache view."""
        out: Dict[tuple, torch.Tensor] = {}

        def walk(path: str, part: Part):
            for name, val in vars(part).items():
                if isinstance(val, torch.Tensor):
                    out[(path, name)] = val
            for cname, child in part.children().items():
                walk(f"{path}.{cname}", child)

        walk("block", block)
        if view is not None:
            for name, val in vars(view).items():
                if isinstance(val, torch.Tensor):
                    out[("cache", name)] = val
        return out

    def _replay_key(self, call, view):
        """What two layer calls must have in common for one's recorded launches to serve the other
        (None: this call cannot be recorded or replayed)."""
        block = self.blocks[call.block]
        parts = [block]
        k = 0
        while k < len(parts):
            parts.extend(parts[k].children().values())
            k += 1
        if not all(p.replayable for p in parts):
            return None
        shapes = tuple((key, tuple(t.shape), t.dtype) for key, t in sorted(self._own_tensors(block, view).items()))
        return (self.spec.blocks[call.block], call.writes_cache, type(view).__name__,
                getattr(view, "group", None), getattr(view, "window", None), shapes)

    def forward(self, ctx, caches) -> torch.Tensor:
        """Run this step's tokens through every layer call; logits ``[wanted, vocab]``.

        A layer call whose parts are all ``replayable`` is recorded launch by launch the first
        time its kind comes up in a step (from the second layer on: the first has no delta coming
        in), and the calls of the same kind after it repeat those launches with their own weights
        and cache pages; the delta between layers alternates between the recorded call's input
        and output buffers.

        In a step of a few rows (``ops.folds_norm``) a block that can is told which norm its output
        meets first, the next block's, and may fold it into its last product; such steps are not
        recorded."""
        ops = self.rt.ops
        residual = self.embedding.forward(ctx.token_ids)
        fold = getattr(ops, "folds_norm", None)
        fold = fold is not None and fold(residual.shape[0], self.rt.dtype)
        replay = getattr(ops, "LAYER_REPLAY", False) and hasattr(ops, "LayerRecording") and not fold
        pending = None
        rec = rec_key = None
        order = self.spec.order
        memo = self.__dict__.setdefault("_replay_memo", {})     # per layer call: its key and addresses
        for i, call in enumerate(order):
            block, view = self.blocks[call.block], caches.view(call.cache, ctx)
            if replay and i not in memo:
                key = self._replay_key(call, view)
                memo[i] = (key, None if key is None else
                           {name: t.data_ptr() for name, t in self._own_tensors(block, view).items()})
            key = memo[i][0] if replay and pending is not None else None
            if key is not None and rec is not None and key == rec_key:
                own = dict(memo[i][1])
                own["delta in"], own["delta out"] = pending.data_ptr(), rec_bufs[pending is rec_bufs[0]].data_ptr()
                rec.replay(own)
                pending = rec_bufs[pending is rec_bufs[0]]
                continue
            worth = key is not None and i + 1 < len(order) and rec_key != key
            if worth:
                with ops.LayerRecording() as rec:
                    out = block.forward(residual, pending, ctx, view, call.writes_cache)
                roles = {t.data_ptr(): name for name, t in self._own_tensors(block, view).items()}
                if pending.data_ptr() in roles or out.data_ptr() in roles or pending.data_ptr() == out.data_ptr():
                    rec = rec_key = None                         # (cannot tell the buffers apart)
                else:
                    roles[pending.data_ptr()], roles[out.data_ptr()] = "delta in", "delta out"
                    rec.bind(roles)
                    rec_key, rec_bufs = key, (pending, out)
                pending = out
                continue
            next_norm = None
            if fold and block.folds_next and i + 1 < len(order):
                first = getattr(self.blocks[order[i + 1].block], "first_norm", None)
                next_norm = first() if first is not None else None
            if next_norm is not None:
                pending = block.forward(residual, pending, ctx, view, call.writes_cache, next_norm=next_norm)
            else:
                pending = block.forward(residual, pending, ctx, view, call.writes_cache)
        if ctx.n_wanted == 0:
            return torch.empty(0, self.spec.head.vocab_size, dtype=torch.float32,
                               device=self.rt.device)
        return self.head.forward(residual, pending, ctx.want_rows)
