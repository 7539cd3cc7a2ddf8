"""A causal language model assembled from a ``ModelPlan``.

Owns the parts and the map from checkpoint tensor names to the parts' local
names.  ``forward`` runs the plan's schedule over the tokens of one step and
returns float32 logits at the wanted rows (final norm and head run on those rows
only; the reference norms every row first, src/inference.cu:68-69).
"""
from __future__ import annotations

from typing import Callable, Mapping

import torch

from ..config.plan import ModelPlan
from .base import FixedStateSpec, PagedKVSpec, Part, WeightSpec, build_part


class CausalLM:
    def __init__(self, plan: ModelPlan):
        self.plan = plan
        self.embedding = build_part("embedding", plan.embedding)
        self.final_norm = build_part("norm", plan.final_norm)
        self.head = build_part("head", plan.head)
        self.blocks = []
        self._named: list[tuple[str, Part]] = [
            (plan.names["embedding"], self.embedding),
            (plan.names["final_norm"], self.final_norm),
            (plan.names["head"], self.head),
        ]
        for lp in plan.layers:
            parts = {
                "mixer": build_part("mixer", lp.mixer),
                "ffn": build_part("ffn", lp.ffn),
                "mixer_norm": build_part("norm", lp.mixer_norm),
                "ffn_norm": build_part("norm", lp.ffn_norm),
            }
            self.blocks.append(build_part("block", lp.block, **parts))
            for role, part in parts.items():
                self._named.append((lp.names[role], part))

    # ---- weights -------------------------------------------------------------------------
    def expected_tensors(self) -> dict[str, WeightSpec]:
        """Checkpoint name -> shape and initialisation class of every tensor the model needs."""
        out: dict[str, WeightSpec] = {}
        for prefix, part in self._named:
            for local, spec in part.weight_specs().items():
                out[prefix + local] = spec
        return out

    def duplicate_tensors(self) -> dict[str, str]:
        """Checkpoint names the model does not need but a folder may still hold, each with the
        name of the tensor it repeats: a tied head's own table beside the embedding's (some
        published checkpoints with tied embeddings store the table twice).  The reference never
        reads a head of its own (src/model.cpp:120-121)."""
        if getattr(self.head, "tied", False):
            return {self.plan.names["head"] + "weight": self.plan.names["embedding"] + "weight"}
        return {}

    def load_weights(self, fetch: Callable[[str], torch.Tensor], ops) -> None:
        """``fetch(name)`` returns the checkpoint tensor on the device, dtype as stored."""
        for prefix, part in self._named:
            names = part.weight_specs()
            part.load_weights({local: fetch(prefix + local) for local in names}, ops)
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding)

    def step_lists(self) -> list:
        """The host-built lists that the model's parts ask of every step, each name once."""
        found: dict = {}
        for _, part in self._named:
            for sl in part.step_lists():
                found.setdefault(sl.name, sl)
        return list(found.values())

    # ---- cache ---------------------------------------------------------------------------
    def cache_specs(self) -> list[PagedKVSpec | FixedStateSpec | None]:
        """What each cache slot of the schedule holds (from the mixer that writes it)."""
        specs: list = [None] * self.plan.num_cache_slots
        for entry in self.plan.schedule:
            spec = self.blocks[entry.layer].mixer.cache_spec()
            if entry.writes_cache:
                specs[entry.cache_slot] = spec
            elif specs[entry.cache_slot] != spec:
                raise ValueError(
                    f"layer {entry.layer} reads cache slot {entry.cache_slot} holding "
                    f"{specs[entry.cache_slot]}, but needs {spec}")
        return specs

    # ---- forward -------------------------------------------------------------------------
    def forward(self, ops, step, cache_views: Mapping[tuple[int, bool], object]) -> torch.Tensor:
        step.scratch.clear()           # what kernels derived from the step in an earlier pass is stale
        x = torch.empty((step.num_tokens, self.plan.hidden_size), dtype=torch.float32,
                        device=step.token_ids.device)
        self.embedding.forward(ops, step.token_ids, x)
        for entry in self.plan.schedule:
            cache = cache_views[(entry.cache_slot, entry.writes_cache)]
            self.blocks[entry.layer].forward(ops, x, step, cache)
        ops.flush()                        # nothing a part asked for may still be held back
        if step.num_logit_rows == 0:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=x.device)
        h = self.final_norm.forward_rows(ops, x, step.logit_rows, step.act_dtype)
        return self.head.forward(ops, h)
