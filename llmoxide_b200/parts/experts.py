"""Routed experts as a feed-forward: every token uses ``top`` of ``n_experts``
small gated layers, down(act(gate x) * (up x)), weighted by the router.

Router logits z = W_r x are float32 (the router's matrix is kept in float32;
x may be the compute dtype's rounding), plus the tensor ``router_bias`` when
there is one.  ``score``: s = sigmoid(z), or a softmax over z, or
"softmax_top": the ``top`` largest z win and their weights are the softmax
over those z alone; or "table": there is no router, the integer tensor ``table`` [vocab, top] names every token
id's experts, and each counts ``table_weight``.  With ``n_groups`` > 1 the expert indices are cut into
``n_groups`` contiguous blocks of equal length; every block is ranked by the
sum of its ``group_score_top`` highest s, and a token's choice is restricted
to the ``keep_groups`` top-ranked blocks.  The ``top`` highest s among the
eligible experts are taken; their weights are those s, over (their sum +
``normalize_eps``) when ``normalize``, times ``scale``.  With a tensor
``correction`` (one number per expert) the choice goes by s + correction while
the weights stay s.  The last ``n_identity`` of the router's outputs are
identity experts: they have no tensors and their output is the input itself
(times the weight).  ``activation`` names the experts' gated activation
(``kernels.gate_act_args``; "clamped_swish" takes ``act_slope``, ``act_limit``,
``act_up_shift``).  A shared expert (``shared_size``; tensors ``shared_gate``,
``shared_up``, ``shared_down``, ``shared_sg`` [1, d]; its limit ``shared_limit``)
runs for every token and is added times sigmoid(shared_sg . x), or as it is
when there is no ``shared_sg``.

The step's (token, choice) pairs are ordered by expert on the device and the
two products run grouped over that order (csrc/moe.cu), so nothing is read
back to the host and a decode step stays inside a CUDA graph.  The result is
handed on as one float32 partial per choice (and one for the shared expert),
[top (+1), T, d], which the norm that adds it to the residual stream sums in
order.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..errors import ConfigError, Unsupported
from .registry import register_feed_forward


@register_feed_forward("none")
class NoFeedForward:
    """A layer without a feed-forward."""

    def __init__(self, spec, weights: dict, rt):
        pass

    def libraries(self) -> set:
        return set()

    def forward(self, x, ctx, residual=None):
        return None


@register_feed_forward("routed_experts")
class RoutedExperts:
    def __init__(self, spec, weights: dict, rt):
        name = spec.get("activation", "silu")
        if name not in kernels.GATE_ACTS:
            raise Unsupported(f"routed_experts activation {name!r}: built are {sorted(kernels.GATE_ACTS)}")
        act = lambda limit: name if name != "clamped_swish" else (
            name, float(spec.get("act_slope", 1.0)), float(limit), float(spec.get("act_up_shift", 0.0)))
        self.activation = act(spec.get("act_limit", 0.0))
        self.rt = rt
        self.E, self.top, self.F = spec["n_experts"], spec["top"], spec["intermediate_size"]
        self.n_identity = int(spec.get("n_identity") or 0)
        self.E_all = self.E + self.n_identity         # what the router chooses among
        self.n_groups, self.keep_groups = spec.get("n_groups", 1), spec.get("keep_groups", 1)
        self.group_top = spec.get("group_score_top", 2)
        self.score = spec.get("score", "sigmoid")
        self.normalize, self.norm_eps = bool(spec.get("normalize", True)), float(spec.get("normalize_eps", 0.0))
        self.scale = float(spec.get("scale", 1.0))
        if self.E_all % self.n_groups or self.top > self.E_all // self.n_groups * self.keep_groups:
            raise ConfigError(f"{self.E_all} experts in {self.n_groups} groups, {self.keep_groups} kept, top {self.top}")
        if self.E_all > 1024 or self.top > 16:
            raise Unsupported(f"{self.E_all} experts / top {self.top}: the routing kernel takes up to 1024 / 16")
        t = spec.tensors
        self.table = None
        if self.score == "table":
            if self.n_identity or self.n_groups != 1 or "router" in t or spec.get("shared_size"):
                raise Unsupported("routing by a table is built for plain experts without groups or a shared expert")
            self.table = weights.pop(t["table"].name).to(torch.int32).contiguous()
            self.table_weight = float(spec.get("table_weight", 1.0 / self.top))
            if self.table.dim() != 2 or self.table.shape[1] != self.top:
                raise ConfigError(f"the routing table has shape {tuple(self.table.shape)}, expected [vocab, {self.top}]")
        # the router decides in float32 whatever the compute dtype
        self.router = None if self.table is not None else weights.pop(t["router"].name).to(torch.float32).contiguous()
        self.correction = (weights.pop(t["correction"].name).to(torch.float32).contiguous()
                           if "correction" in t else None)
        self.router_bias = (weights.pop(t["router_bias"].name).to(torch.float32).contiguous()
                            if "router_bias" in t else None)
        self.shared, self.shared_gated = None, "shared_sg" in t
        if spec.get("shared_size"):
            if self.shared_gated:
                # the shared expert's gate reads the same rows as the router: its vector is one more row of that matrix
                self.router = torch.cat([self.router, weights.pop(t["shared_sg"].name).to(torch.float32).reshape(1, -1)],
                                        dim=0).contiguous()
            # the shared expert itself is a gated feed-forward of this package, with the experts' activation
            from ..config.spec import PartSpec
            from .feed_forward import GatedMLP
            self.shared = GatedMLP(PartSpec("gated_mlp", dict(
                hidden_size=spec["hidden_size"], intermediate_size=int(spec["shared_size"]),
                activation=act(spec.get("shared_limit", spec.get("act_limit", 0.0)))),
                dict(gate=t["shared_gate"], up=t["shared_up"], down=t["shared_down"])), weights, rt)
        dt = rt.act_dtype
        gate_up = [torch.cat([weights.pop(t[f"gate{e}"].name), weights.pop(t[f"up{e}"].name)], dim=0).to(dt)
                   for e in range(self.E)]
        self.gate_up = torch.stack(gate_up).contiguous()             # [E, 2F, d]: gate rows, then up rows
        del gate_up
        self.down = torch.stack([weights.pop(t[f"down{e}"].name).to(dt) for e in range(self.E)]).contiguous()  # [E, d, F]

        # bfloat16 with sizes the TMA takes: the grouped products run on tcgen05 (csrc/moe_tc.cu)
        self.tensor_cores = bool(rt.tensor_cores and dt == torch.bfloat16 and self.gate_up.shape[2] % 8 == 0
                                 and self.F % 8 == 0 and kernels.moe_tc_gated_supports(self.activation))

    def libraries(self) -> set:
        libs = {"moe", "elementwise"} | ({"moe_tc"} if self.tensor_cores else set())
        if self.shared:
            libs |= self.shared.libraries()
        return libs

    def tile_rows(self, n_pairs: int) -> int:
        """Rows per tile of the grouped products: narrow tiles when an expert gets few rows (a decode step streams
        the weights), wide ones for prompts."""
        per_expert = n_pairs / self.E
        return 16 if per_expert <= 16 else 64 if per_expert <= 96 else 128

    def forward(self, x, ctx, residual=None):
        T, dev = x.shape[0], x.device
        P = T * self.top
        ids = torch.empty((T, self.top), dtype=torch.int32, device=dev)
        pair_w = torch.empty((T, self.top), dtype=torch.float32, device=dev)
        shared_z = torch.empty((T, 1), dtype=torch.float32, device=dev) if self.shared and self.shared_gated else None
        if self.table is not None:
            kernels.moe_table_route(ctx.tokens, self.table, self.E, self.table_weight, ids, pair_w)
        else:
            kernels.moe_router(x, self.router, ids, pair_w, self.n_groups, self.keep_groups, self.group_top, self.score,
                               self.normalize, self.norm_eps, self.scale, bias=self.correction, extra_out=shared_z,
                               logit_bias=self.router_bias)
        probe = getattr(ctx, "probe", None)
        if probe:
            probe("router_ids", ids), probe("router_weights", pair_w)
        perm = torch.empty((P,), dtype=torch.int32, device=dev)
        fast = self.tensor_cores and x.dtype == torch.bfloat16 and kernels.moe_tc_supports(x, self.gate_up)
        rows = self.tile_rows(P) if fast else kernels.MOE_TILE
        tiles = torch.empty((kernels.moe_max_tiles(P, self.E_all, rows), 3), dtype=torch.int32, device=dev)
        act = torch.empty((P, self.F), dtype=self.rt.act_dtype, device=dev)
        d = self.down.shape[1]
        y = torch.empty((self.top + (1 if self.shared else 0), T, d), dtype=torch.float32, device=dev)
        if fast:
            dest = torch.empty((P,), dtype=torch.int32, device=dev)
            sorted_w = torch.empty((P,), dtype=torch.float32, device=dev)
            kernels.moe_sort(ids, self.E_all, perm, tiles, rows, pair_w, dest, sorted_w, n_tiled=self.E)
            xs = torch.empty((P, x.shape[1]), dtype=torch.bfloat16, device=dev)
            kernels.moe_gather_rows(x, perm, self.top, xs)
            kernels.moe_grouped_tc(xs, self.gate_up, act, tiles, rows, dest, sorted_w, gated=True,
                                   activation=self.activation)
            kernels.moe_grouped_tc(act, self.down, y, tiles, rows, dest, sorted_w, gated=False)
        else:
            kernels.moe_sort(ids, self.E_all, perm, tiles, rows, n_tiled=self.E)
            kernels.moe_grouped(x, self.gate_up, act, perm, tiles, pair_w, self.top, T, gated=True,
                                activation=self.activation)
            kernels.moe_grouped(act, self.down, y, perm, tiles, pair_w, self.top, T, gated=False)
        if self.n_identity or self.shared:
            # an identity expert's output is the token's own row times the weight; the shared expert's result is
            # weighted by its gate: both join y in one launch
            shared = self.shared.forward(x, ctx) if self.shared else None
            kernels.moe_extras(x, ids, pair_w, y, self.E, shared, shared_z[:, 0] if shared_z is not None else None)
        return y
