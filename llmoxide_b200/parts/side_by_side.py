"""Two mixers side by side as one mixer: both read the same input, and the
result is left_scale * left(x) + right_scale * right(x).

The two are parts of the mixer registry themselves (parameters ``left`` and
``right`` are their ``PartSpec``s), so any pair can stand side by side as long
as they do not want the same kind of cache: the layer call's cache entry
gives its keys and values to the one that asks for them and its per-sequence
state to the one that asks for that.  The block's position encoding goes to
the side(s) named by ``position_to`` ("left", "right" or "both").  The two
results are not added here: they are handed on as a ``WeightedSum``, which the
norm kernel that adds them to the residual stream sums with their weights.
"""

from __future__ import annotations

from ..errors import Unsupported
from .norm import WeightedSum
from .registry import MIXERS, lookup, register_mixer


@register_mixer("side_by_side")
class SideBySide:
    def __init__(self, spec, position, weights: dict, rt):
        to = spec.get("position_to", "left")
        self.left = lookup(MIXERS, "mixer", spec["left"].kind)(
            spec["left"], position if to in ("left", "both") else None, weights, rt)
        self.right = lookup(MIXERS, "mixer", spec["right"].kind)(
            spec["right"], position if to in ("right", "both") else None, weights, rt)
        self.left_scale, self.right_scale = float(spec.get("left_scale", 1.0)), float(spec.get("right_scale", 1.0))
        (kl, sl), (kr, sr) = self.left.cache_need(), self.right.cache_need()
        if (kl is not None and kr is not None) or (sl is not None and sr is not None):
            raise Unsupported("two mixers side by side that both want keys and values, or both want state")
        self._need = (kl if kl is not None else kr, sl if sl is not None else sr)
        # output biases: this mixer's own is the weighted sum of its sides', which then leave theirs to it
        self.out_bias, self.defer_out_bias = None, False
        for part, w in ((self.left, self.left_scale), (self.right, self.right_scale)):
            b = getattr(part, "out_bias", None)
            if b is not None:
                part.defer_out_bias = True
                self.out_bias = b * w if self.out_bias is None else self.out_bias + b * w
        if self.out_bias is not None:
            self.out_bias = self.out_bias.contiguous()

    def cache_need(self):
        return self._need

    def libraries(self) -> set:
        libs = self.left.libraries() | self.right.libraries()
        return libs | ({"post_norm"} if self.out_bias is not None else set())

    @property
    def graph_safe(self) -> bool:
        return getattr(self.left, "graph_safe", True) and getattr(self.right, "graph_safe", True)

    def forward(self, x, ctx, view, writes_cache=True):
        a = self.left.forward(x, ctx, view, writes_cache)
        b = self.right.forward(x, ctx, view, writes_cache)
        if self.out_bias is not None and not self.defer_out_bias:
            from .. import kernels
            kernels.add_bias(a if a.dim() == 2 else a[0], self.out_bias / self.left_scale)
        return WeightedSum([(a, self.left_scale), (b, self.right_scale)])
