"""Several mixers side by side: all read the same input, and their outputs are added with one constant each,

    out = sum over parts of scale_part * part(h).

``parts`` lists them: each entry gives a registered mixer's ``kind``, its ``params``, where its tensors lie under this
mixer's prefix (``under``: "left", say) and its ``scale``.  Each part keeps what it would keep alone: the cache manager
is asked for a ``CompositeNeed`` of the parts' needs and hands back a tuple in the parts' order, a paged part's cache
group takes that part's wish for attention work items, and a recurrent part its own slot.  The sum is formed in float32
and rounded once.
"""

from __future__ import annotations

from ..kernels import ops
from .base import MIXERS, CompositeNeed, Mixer, make, register_mixer
from .spec import PartSpec


class ParallelMixers(Mixer):
    def __init__(self, spec, rt, position_encodings=None):
        super().__init__(spec, rt)
        entries = spec.params["parts"]
        if len(entries) < 2:
            raise ValueError("mixers side by side are two or more")
        self.parts, self.scales = [], []
        for e in entries:
            under = e.get("under", "")
            prefix = ".".join(x for x in (spec.prefix, under) if x)
            self.parts.append(make(MIXERS, "mixer", PartSpec(e["kind"], dict(e.get("params", {})), prefix), rt,
                                   position_encodings=position_encodings))
            self.scales.append(float(e.get("scale", 1.0)))

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", False) for p in self.parts)

    def tensors(self):
        return [t for p in self.parts for t in p.tensors()]

    def bind(self, tensors):
        for p in self.parts:
            p.bind(tensors)

    def cache_need(self):
        return CompositeNeed(tuple(p.cache_need() for p in self.parts))

    def forward(self, x, step, cache, writes_cache=True):
        outs = [p.forward(x, step, c, writes_cache) for p, c in zip(self.parts, cache)]
        acc = ops.scaled_sum2(outs[0], outs[1], self.scales[0], self.scales[1])
        for o, s in zip(outs[2:], self.scales[2:]):
            ops.scaled_sum2(acc, o, 1.0, s)
        if self.rt.trace is not None:
            self.rt.record(self._name("out"), acc)
        return acc


register_mixer("parallel_mixers", ParallelMixers)
