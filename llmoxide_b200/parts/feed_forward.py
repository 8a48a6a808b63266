"""Gated feed-forward: down(act(gate x) * (up x)), act = SiLU x/(1+exp(-x))
(crates/model/src/qwen35/cpu.rs:386-395, crates/model/src/ops.rs:176-178).
Gate and up are one matrix product over the rows [gate; up].  ``activation``
may also be "relu", "gelu_tanh" (0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3)))), or
("clamped_swish", slope, limit, shift):
min(g, limit) * sigmoid(slope * min(g, limit)) * (clamp(u, -limit, limit) + shift).
Tensors ``gate_bias``, ``up_bias``, ``down_bias``: biases of the three projections (gate and up: added where the
activation reads the product, which is the tensor-core product's own epilogue where that applies the activation;
down: offered as ``out_bias`` to an arrangement that adds it in its norm kernel, else added here)."""

from __future__ import annotations

import torch

from .. import kernels
from ..errors import Unsupported
from .row_scaled import RowScaled
from .linear import Linear
from .registry import register_feed_forward


import os

# Above this many tokens the gate/up product applies the activation in its epilogue (no split of its
# reduction); at or below it the reduction is split and the activation sums the partials.  Measured at
# Qwen3-8B layer sizes the fused form is as fast or faster at every batch size, so it is the default.
FUSE_MIN_TOKENS = int(os.environ.get("LLMX_FUSE_MIN_TOKENS", "0"))


@register_feed_forward("gated_mlp")
class GatedMLP:
    def __init__(self, spec, weights: dict, rt):
        self.activation = spec.get("activation", "silu")
        if isinstance(self.activation, list):
            self.activation = tuple(self.activation)
        name = self.activation if isinstance(self.activation, str) else self.activation[0]
        if name not in kernels.GATE_ACTS:
            raise Unsupported(f"gated_mlp activation {name!r}: built are {sorted(kernels.GATE_ACTS)}")
        self.rt, self.F = rt, spec["intermediate_size"]
        t = spec.tensors
        wg, wu = weights.pop(t["gate"].name), weights.pop(t["up"].name)
        if wg.dtype != wu.dtype:
            wg, wu = wg.float(), wu.float()
        # One matrix for gate and up.  Where the width allows, rows go in blocks of 16 gate rows each
        # followed by the 16 up rows of the same features: a warp of the matrix product's epilogue (32 rows of
        # a tile) then holds both halves of 16 features, and the activation is one shuffle away.  Otherwise
        # gate rows, then up rows.
        self.block = 16 if self.F % 16 == 0 else 0
        if self.block:
            k = wg.shape[1]
            fused = torch.stack([wg.view(-1, 16, k), wu.view(-1, 16, k)], dim=1).reshape(2 * self.F, k)
        else:
            fused = torch.cat([wg, wu], dim=0)
        del wg, wu
        self.gate_up = Linear(fused, rt)
        del fused
        self.gu_bias = self.gu_bias_tc = None
        if "gate_bias" in t:
            bg, bu = (weights.pop(t[r].name).to(torch.float32) for r in ("gate_bias", "up_bias"))
            # in the order of the fused matrix's rows
            self.gu_bias = (torch.stack([bg.view(-1, 16), bu.view(-1, 16)], dim=1).reshape(-1) if self.block
                            else torch.cat([bg, bu])).contiguous()
            if self.block and self.gate_up._tc is not None:
                # for the tensor-core product's epilogue: whole row tiles of a CTA pair
                pad = -self.gu_bias.numel() % kernels.TC_BIAS_PAD
                self.gu_bias_tc = torch.cat([self.gu_bias, self.gu_bias.new_zeros(pad)]).contiguous()
        self.down = Linear(weights.pop(t["down"].name), rt,
                           bias=weights.pop(t["down_bias"].name) if "down_bias" in t else None)
        self.out_bias, self.defer_out_bias = self.down.bias, False

    def libraries(self) -> set:
        return {"elementwise"} | self.gate_up.libraries() | self.down.libraries()

    @property
    def takes_row_scales(self) -> bool:
        """The gate|up product can apply a norm's row scales in its epilogue, ahead of the activation."""
        return (self.gate_up._tc is not None and kernels.gemm_tc_gated_supports(self.activation)
                and self.gu_bias is None)

    adds_to_residual = True      # forward() takes ``residual`` and may return None: "already added"

    def forward(self, x, ctx, residual=None):
        tc = self.gate_up._tc
        scaled = isinstance(x, RowScaled)
        n_tokens = x.shape[0]
        if tc is not None and (self.gu_bias is None or self.gu_bias_tc is not None) and x.dtype == torch.bfloat16 and (
                n_tokens > FUSE_MIN_TOKENS) and (scaled or kernels.gemm_tc_supports(x, tc.weight)) and (
                kernels.gemm_tc_gated_supports(self.activation)):
            # the activation (and the biases of gate and up) are the epilogue of the gate/up product
            act = tc.gated(x, self.rt.act_dtype, self.block, self.activation, bias=self.gu_bias_tc)
        else:
            assert not scaled
            gu = self.gate_up(x, splits_ok=True)
            act = torch.empty((n_tokens, self.F), dtype=self.rt.act_dtype, device=x.device)
            kernels.silu_gate(gu, act, self.block, self.activation, bias=self.gu_bias)
        if self.out_bias is None and residual is not None and self.down.add_into(act, residual):
            return None
        return self.down(act, splits_ok=True, add_bias=not self.defer_out_bias)
