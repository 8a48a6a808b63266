"""The matrix memory of an mLSTM layer as a mixer: linear attention whose decay
and input weight are gates computed from the layer's input, kept stable by a
running maximum, with a normaliser.

    q, k: [heads, D], v: [heads, Dv], gate: [heads * Dv], i, f: [heads]   one fused projection of the layer's input
    q <- q * q_scale
    i_t = cap tanh((i + b_i) / cap),  f_t = logsigmoid(cap tanh((f + b_f) / cap))       per head; ``gate_cap``
    m_t = max(f_t + m_(t-1), i_t)                                         m starts at ``m_start`` (0)
    S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T     S, n start at zero
    n_t = exp(f_t + m_(t-1) - m_t) n_(t-1) + exp(i_t - m_t) k_t
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + den_eps)
    o <- o / sqrt(mean(o^2) + eps) per head, times a gain over all heads' columns
    y = W_o (o * sigmoid(gate))

Per sequence and head the state is S [D, Dv], n [D] and m, float32, in the
cache's state area: n rides as one more column of S (the column of a value
that is 1 for every token), m behind them.  The gates, the state, every
multiply-add of the recurrence, the normaliser and the norm are float32
whatever the compute dtype; the fused projection leaves float32 rows, so the
gates are never rounded to 16 bits.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache import StateNeed
from ..errors import ConfigError, Unsupported
from .linear import Linear
from .registry import register_mixer


@register_mixer("mlstm")
class MLSTM:
    def __init__(self, spec, position, weights: dict, rt):
        self.rt = rt
        self.H, self.D, self.Dv = spec["n_heads"], spec["head_dim"], spec["v_head_dim"]
        if self.D > 256:
            raise Unsupported(f"head_dim {self.D}: the recurrence kernel takes sizes up to 256")
        self.eps = float(spec["eps"])
        self.cap = float(spec.get("gate_cap") or 0.0)
        self.q_scale = float(spec.get("q_scale", self.D ** -0.5))
        self.den_eps = float(spec.get("den_eps", 1e-6))
        self.m_start = float(spec.get("m_start", 0.0))
        if self.m_start != 0.0:
            raise ConfigError("a running maximum that does not start at 0 is not built (the state area starts at zero)")
        t = spec.tensors
        ws = [weights.pop(t[r].name) for r in ("q", "k", "v", "g", "i", "f")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        # one matrix product for q, k, v, the output gate and the two gates of the recurrence: rows in that order
        self.proj = Linear(torch.cat(ws, dim=0), rt)
        del ws
        self.bias_i = weights.pop(t["i_bias"].name).to(torch.float32).contiguous() if "i_bias" in t else None
        self.bias_f = weights.pop(t["f_bias"].name).to(torch.float32).contiguous() if "f_bias" in t else None
        self.o = Linear(weights.pop(t["o"].name), rt)
        self.gain = weights.pop(t["norm"].name).to(torch.float32).contiguous() if "norm" in t else None
        HD, HDv = self.H * self.D, self.H * self.Dv
        self.q_off, self.k_off, self.v_off, self.g_off = 0, HD, 2 * HD, 2 * HD + HDv
        self.i_off, self.f_off = 2 * HD + 2 * HDv, 2 * HD + 2 * HDv + self.H
        # a head's state: S with n as its last column [D, Dv + 1], then m; padded to whole 16 bytes
        self.m_off = self.D * (self.Dv + 1)
        self.head_floats = (self.m_off + 1 + 3) // 4 * 4

    def cache_need(self):
        return None, StateNeed((self.H, self.head_floats))

    def libraries(self) -> set:
        return {"linear_attention"} | self.proj.libraries() | self.o.libraries()

    adds_to_residual = True      # forward() takes ``residual`` and may return None: "already added"

    def forward(self, x, ctx, view, writes_cache=True, residual=None):
        if not writes_cache:
            raise Unsupported("a recurrent state has one writer: the layer that owns it")
        T, H, Dv = x.shape[0], self.H, self.Dv
        proj = self.proj(x, out_dtype=torch.float32, splits_ok=True)
        gates = torch.empty((T, H, 4), dtype=torch.float32, device=x.device)
        kernels.gate_scan(proj, self.i_off, self.f_off, self.bias_i, self.bias_f, self.cap, gates, view.state, self.m_off,
                          ctx.seq_start, ctx.seq_slot, H)
        o = torch.empty((T, H * (Dv + 1)), dtype=torch.float32, device=x.device)
        kernels.decay_scan(proj, o, view.state, ctx.seq_start, ctx.token_pos, ctx.seq_slot, None, None, None, 0, "none",
                           1.0, H, self.D, Dv, self.q_off, self.k_off, self.v_off, max_new=ctx.max_new, gates=gates,
                           q_scale=self.q_scale, ones_column=True)
        y = torch.empty((T, H * Dv), dtype=self.rt.act_dtype, device=x.device)
        kernels.gated_norm(o, proj, self.g_off, self.gain, self.eps, "sigmoid", True, y, H, Dv, gates=gates,
                           den_eps=self.den_eps)
        if residual is not None and self.o.add_into(y, residual):
            return None
        return self.o(y, splits_ok=True)
