"""The generic decoder: embedding, layers in the order the description gives, final norm, head.

It is assembled from a :class:`ModelSpec` through the part registries and knows no architecture.  One
``forward`` serves every kind of step: it runs the rows it is given against the cache views and returns
float32 logits for the wanted rows only (the reference computes the head for the last row or for all
rows: src/qwen_model.cpp:1421-1486, 1358-1371).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import CacheManager, CacheNeed
from ..weights.loader import TensorSpec, load_tensors
from .base import BuildContext, make_part
from .context import CacheView, ResidualStream, StepContext
from .spec import ModelSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec, compute_dtype: torch.dtype = torch.float32, options: Optional[dict] = None):
        spec.validate()
        self.spec = spec
        self.compute_dtype = compute_dtype
        self.build = BuildContext(compute_dtype, options)
        from . import block as _block  # noqa: F401  (registers the arrangements)
        from .base import ARRANGEMENTS
        self.embedding = make_part("embedding", spec.embedding, self.build)
        self.layers = []
        for layer in spec.layers:
            if layer.arrangement not in ARRANGEMENTS:
                raise KeyError(f"no block arrangement {layer.arrangement!r} is registered")
            self.layers.append(ARRANGEMENTS[layer.arrangement](layer, self.build))
        self.final_norm = make_part("norm", spec.final_norm, self.build)
        self.head = make_part("head", spec.head, self.build)
        self.device = None

    # ---- weights ---------------------------------------------------------------------------------
    def _all_parts(self):
        yield self.embedding
        for layer in self.layers:
            yield from layer.parts()
        yield self.final_norm
        yield self.head

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for p in self._all_parts():
            for name, spec in p.tensor_specs().items():
                if name in out and out[name] != spec:
                    raise ValueError(f"two parts read {name!r} with different shapes or roles")
                out[name] = spec
        return out

    def ignored_tensors(self):
        names = set()
        for p in self._all_parts():
            names.update(p.ignored_tensors())
        return names

    def load(self, model_dir: str, device) -> None:
        tensors = load_tensors(model_dir, self.tensor_specs(), self.compute_dtype, device, self.ignored_tensors())
        self.bind(tensors, device)

    def bind(self, tensors: Dict[str, torch.Tensor], device) -> None:
        self.device = torch.device(device)
        for p in self._all_parts():
            p.bind(tensors, device)

    def required_libraries(self):
        libs = set()
        for p in self._all_parts():
            libs.update(p.required_libraries())
        return tuple(sorted(libs))

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for p in self._all_parts():
            for v in vars(p).values():
                ts = [v] if isinstance(v, torch.Tensor) else ([v.weight] if hasattr(v, "weight") and
                                                              isinstance(getattr(v, "weight"), torch.Tensor) else [])
                for t in ts:
                    key = t.untyped_storage().data_ptr()
                    if key not in seen:
                        seen.add(key)
                        total += t.untyped_storage().nbytes()
        return total

    # ---- cache -----------------------------------------------------------------------------------
    def cache_needs(self) -> List[CacheNeed]:
        """One need per entry of the run order (an entry that borrows a cache needs nothing itself)."""
        needs = []
        for call in self.spec.schedule:
            if call.cache_from is not None:
                needs.append(CacheNeed())
            else:
                needs.append(self.layers[call.layer].mixer.cache_need())
        return needs

    def cache_views(self, manager: CacheManager) -> List[CacheView]:
        views: List[CacheView] = []
        for i, call in enumerate(self.spec.schedule):
            owner = i if call.cache_from is None else call.cache_from
            need = manager.needs[owner]
            if need.kind == "pages":
                g = manager.groups[manager.entry_group[owner]]
                slot = g.entry_slot(owner)
                views.append(CacheView("pages", g.index, g.pool[0, slot, 0], g.pool[0, slot, 1], g.pool.stride(0),
                                       manager.page_size, num_pages=g.pool.shape[0], writable=(owner == i)))
            elif need.kind == "state":
                views.append(CacheView("state", state=manager.state[owner], writable=(owner == i)))
            else:
                views.append(CacheView("none"))
        return views

    # ---- step ------------------------------------------------------------------------------------
    def forward(self, ctx: StepContext, views: List[CacheView], want_rows: Optional[torch.Tensor],
                n_want: int) -> Optional[torch.Tensor]:
        """Run the rows of ``ctx``.  ``want_rows`` (int32, device) are the rows whose logits are returned
        as float32 [n_want, vocab]; with ``n_want`` 0 the head is skipped and None is returned."""
        stream = ResidualStream(self.embedding.forward(ctx))
        for call, view in zip(self.spec.schedule, views):
            self.layers[call.layer].forward(stream, ctx, view)
        if n_want == 0:
            return None
        xn = self.final_norm.forward(stream, ctx, rows=want_rows, n_rows=n_want)
        return self.head.forward(xn, ctx, n_want)
