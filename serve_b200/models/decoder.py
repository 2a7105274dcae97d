"""A decoder built from a ``ModelSpec``: embedding, scheduled layers, final norm, head.

It owns the parts and runs them in the order the schedule gives; it knows no
architecture. The forward pass handles whatever tokens the step brings (flat
[T]), reads and writes the cache through the views it is handed, and returns
float32 logits for the requested rows only (the reference projects the last
row of each prompt, serve/model.py:230-231, or every decode row, 226-227).
"""
from __future__ import annotations

from typing import Dict, List, Optional

from ..config.spec import ModelSpec
from ..parts.base import CacheNeed, TensorDecl, build_part


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime):
        spec.validate()
        self.spec = spec
        self.rt = runtime
        self.embedding = build_part("embedding", spec.embedding, runtime)
        self.blocks = [build_part("block", ls.block, runtime, parts=ls.parts) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.head = build_part("head", spec.head, runtime)
        self.schedule = list(spec.schedule)
        self._layer_runs = None     # runs of scheduled layers that one kernel can take whole (found at the first step)

    # ---- weights -------------------------------------------------------
    def all_parts(self):
        parts = [self.embedding]
        for b in self.blocks:
            parts.extend(b.parts())
        parts.extend([self.final_norm, self.head])
        return parts

    def tensor_decls(self) -> Dict[str, TensorDecl]:
        decls: Dict[str, TensorDecl] = {}
        for part in self.all_parts():
            for d in part.tensor_decls():
                if d.name in decls and decls[d.name].shape != d.shape:
                    raise ValueError(f"tensor {d.name} declared with shapes {decls[d.name].shape} and {d.shape}")
                decls.setdefault(d.name, d)
        return decls

    def ignorable_tensors(self) -> List[str]:
        names: List[str] = []
        for part in self.all_parts():
            names.extend(part.ignorable_tensors())
        return names

    def load(self, tensors) -> None:
        for part in self.all_parts():
            part.load(tensors)

    # ---- cache ---------------------------------------------------------
    def cache_needs(self) -> List[Optional[CacheNeed]]:
        """One entry per schedule entry that owns a cache (None: that execution needs none)."""
        needs: List[Optional[CacheNeed]] = []
        for e in self.schedule:
            if e.cache_of is not None:
                needs.append(None)
            else:
                needs.append(self.blocks[e.layer].cache_need())
        return needs

    # ---- forward -------------------------------------------------------
    def _find_layer_runs(self, cache_views):
        """{first schedule entry: (entry after the last, plan)} for runs of layers that the kernels can run as one launch
        in a decoding step. The blocks describe themselves; the kernels object decides what it takes."""
        runs = {}
        planner = getattr(self.rt.kernels, "plan_layer_run", None)
        if planner is None:
            return runs
        descs = []
        for i, e in enumerate(self.schedule):
            describe = getattr(self.blocks[e.layer], "fused_description", None)
            descs.append(describe(cache_views[i]) if describe is not None and cache_views[i] is not None else None)
        i = 0
        while i < len(descs):
            if descs[i] is None:
                i += 1
                continue
            j = i
            while j < len(descs) and descs[j] is not None:
                j += 1
            # the longest prefix of descs[i:j] the kernels take as one run
            n, plan = planner(descs[i:j])
            if n > 0:
                runs[i] = (i + n, plan)
                i += n
            else:
                i += 1
        return runs

    def forward(self, ctx, cache_views):
        """ctx: StepContext. cache_views[i]: CacheView of schedule entry i (or None)."""
        x = self.embedding.forward(ctx.tokens, ctx)
        pending = None
        runs = self._layer_runs
        if runs is None and getattr(self.rt.kernels, "use_layer_runs", False):
            runs = self._layer_runs = self._find_layer_runs(cache_views)      # (made only once somebody asks for them)
        i, n = 0, len(self.schedule)
        while i < n:
            run = runs.get(i) if runs else None
            if run is not None and self.rt.kernels.layer_run_takes(run[1], ctx):
                x, pending = self.rt.kernels.layer_run(run[1], x, pending, ctx)
                i = run[0]
                continue
            x, pending = self.blocks[self.schedule[i].layer].forward(x, pending, ctx, cache_views[i])
            i += 1
        if ctx.logit_rows.shape[0] == 0:
            return None
        h = self.final_norm.forward_rows(x, pending, ctx.logit_rows, ctx)
        return self.head.forward(h, ctx)
