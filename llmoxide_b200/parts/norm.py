"""RMSNorm with a plain multiplicative gain: x / sqrt(mean(x^2) + eps) * g
(crates/model/src/ops.rs:40-59), fused with the residual add that precedes it.

Several copies of the residual stream (h [S,T,d], "hyper-connections").  The
norm of a sublayer then reads u = sum_s read[s] h_s, and what the sublayer
returns joins the copies as h_r <- sum_s mix[s,r] h_s + mult * out[r] * y.  The
three weights ride with the norm (tensors ``hc_in`` [S], ``hc_out`` [S],
``hc_mix`` [S,S] indexed [from, to]; ``residual_mult`` is the parameter
``mult``); without them the norm reads the plain sum and the result is added
to every copy times ``mult``.  As with one stream, the update is applied by
the next norm's kernel: ``owed(y)`` wraps a sublayer's result into the
``StreamUpdate`` that the next ``add_forward`` (or ``add``) takes as ``delta``.

``layer_norm`` is the norm with the mean taken off and no bias,
(x - mean) / sqrt(mean((x - mean)^2) + eps) * g.  Either norm can also stand
BEHIND a sublayer ("sandwich" blocks, h += norm_b(f(norm_a(h)))): ``owed(y)``
then wraps the sublayer's result into a ``PostNormed``, and the next norm's
kernel norms it, adds it to the stream and norms the stream in one pass.  Two
mixers side by side hand over a ``WeightedSum`` of their results."""

from __future__ import annotations

import torch

from .. import kernels
from .row_scaled import RowScaled
from .registry import register_norm


class StreamUpdate:
    """What a sublayer owes the copies of the residual stream: h_r <- sum_s mix[s,r] h_s + write[r] * delta."""

    __slots__ = ("delta", "mix", "write")

    def __init__(self, delta, mix, write):
        self.delta, self.mix, self.write = delta, mix, write


class WeightedSum:
    """Several results that join the stream as sum_g weight_g * delta_g (each delta [T,d] or partials [S,T,d])."""

    __slots__ = ("terms",)

    def __init__(self, terms):
        self.terms = list(terms)          # [(delta, weight)], at most two


class PostNormed:
    """What a sublayer owes the residual stream when its result is normed first:
    h += norm((sum_g weight_g * delta_g + bias) * sigmoid(z + zb)) * gain, the gate (z, zb) optional."""

    __slots__ = ("terms", "bias", "gain", "center", "eps", "gate")

    def __init__(self, terms, bias, gain, center, eps, gate=None):
        self.terms, self.bias, self.gain, self.center, self.eps, self.gate = terms, bias, gain, center, eps, gate


def _terms(delta):
    return delta.terms if isinstance(delta, WeightedSum) else [(delta, 1.0)]


def _owed_normed(norm, delta, bias, center: bool, gate=None):
    if delta is None:
        return None
    return PostNormed(_terms(delta), bias, norm.gain, center, norm.eps, gate)


def _general_add_norm(h, delta, gain, center: bool, eps: float, out, rows, write_h: bool):
    """h += delta in any of its forms (a tensor, partials, a weighted sum, a normed result); out = norm(h) * gain."""
    gate = None
    if delta is None:
        terms, bias, post_gain, post_center, post_eps = [], None, None, False, 0.0
    elif isinstance(delta, PostNormed):
        terms, bias, post_gain, post_center, post_eps = delta.terms, delta.bias, delta.gain, delta.center, delta.eps
        gate = delta.gate
    else:
        terms, bias, post_gain, post_center, post_eps = _terms(delta), None, None, False, 0.0
    kernels.post_norm_add_norm(h, terms, bias, post_gain, post_center, post_eps, gain, center, eps, out, rows=rows,
                               write_h=write_h, gate=gate)


@register_norm("layer_norm")
class LayerNorm:
    """(x - mean) / sqrt(variance + eps) * gain, the variance the mean of the squared deviations; no bias."""

    center = True

    def __init__(self, spec, weights: dict, rt):
        self.size, self.eps, self.rt = spec["size"], float(spec["eps"]), rt
        self.gain = weights[spec.tensors["gain"].name].to(torch.float32).contiguous()

    def libraries(self) -> set:
        return {"post_norm"}

    def owed(self, delta, bias=None, gate=None):
        """The sublayer's result ``delta`` (None: nothing), to be normed by this norm before it joins the stream;
        ``gate`` = (z, zb): times sigmoid(z + zb) first."""
        return _owed_normed(self, delta, bias, self.center, gate)

    def add(self, h, delta) -> None:
        if delta is not None:
            _general_add_norm(h, delta, None, False, 0.0, None, None, True)

    def add_forward(self, h, delta, rows=None, write_h=True, out_dtype=None, row_scales_ok=False):
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype or self.rt.act_dtype, device=h.device)
        _general_add_norm(h, delta, self.gain, self.center, self.eps, out, rows, write_h)
        return out


@register_norm("rms_norm")
class RMSNorm:
    def __init__(self, spec, weights: dict, rt):
        self.size, self.eps, self.rt = spec["size"], float(spec["eps"]), rt
        self.gain = weights[spec.tensors["gain"].name].to(torch.float32).contiguous()
        self.mult = float(spec.get("residual_mult", 1.0))
        self.read = self.mix = self.write = None
        if "hc_mix" in spec.tensors:
            t = spec.tensors
            self.read = weights.pop(t["hc_in"].name).to(torch.float32).contiguous()
            self.mix = weights.pop(t["hc_mix"].name).to(torch.float32).contiguous()
            self.write = (weights.pop(t["hc_out"].name).to(torch.float32) * self.mult).contiguous()
        self._plain: dict = {}

    def libraries(self) -> set:
        return {"elementwise", "stream_mix", "post_norm"}

    def owed(self, delta, n_streams: int = 0, bias=None, gate=None):
        """The update by which a sublayer's result ``delta`` (None: nothing) joins ``n_streams`` copies; without
        ``n_streams``: the result normed by this norm before it joins the one stream (a norm behind a sublayer),
        with ``gate`` = (z, zb) times sigmoid(z + zb) first."""
        if delta is None:
            return None
        if not n_streams:
            return _owed_normed(self, delta, bias, False, gate)
        if self.mix is None:        # no connection weights: every copy keeps itself and gets mult * delta
            if n_streams not in self._plain:
                self._plain[n_streams] = (torch.eye(n_streams, dtype=torch.float32, device=self.gain.device).contiguous(),
                                          torch.full((n_streams,), self.mult, dtype=torch.float32, device=self.gain.device))
            return StreamUpdate(delta, *self._plain[n_streams])
        return StreamUpdate(delta, self.mix, self.write)

    def _streams(self, h, delta, out, rows, write_h):
        if delta is None:
            d, mix, write = None, None, None
        elif isinstance(delta, StreamUpdate):
            d, mix, write = delta.delta, delta.mix, delta.write
        else:
            upd = RMSNorm.owed(self, delta, h.shape[0]) if self.mix is None else None
            if upd is None:
                raise ValueError("a result that joins several copies of the residual stream comes as a StreamUpdate")
            d, mix, write = upd.delta, upd.mix, upd.write
        kernels.stream_mix_norm(h, d, mix, write, self.read if out is not None else None, self.gain, self.eps, out,
                                rows=rows, write_h=write_h)

    ROW_SCALE_MAX_TOKENS = 64      # what the products' epilogues take

    def add(self, h, delta) -> None:
        """h += delta (``delta`` [T,d] or split partials [S,T,d], added in order); nothing is normed."""
        if isinstance(delta, (PostNormed, WeightedSum)):
            kernels._library("post_norm")
            return _general_add_norm(h, delta, None, False, 0.0, None, None, True)
        if h.dim() == 2 and isinstance(delta, StreamUpdate):
            h = h.unsqueeze(0)       # one copy, with connection weights of its own
        if h.dim() == 3:
            if delta is not None:
                self._streams(h, delta, None, None, True)
            return
        kernels.add_rms_norm(h, delta, self.gain, self.eps, None)

    def add_forward(self, h, delta, rows=None, write_h=True, out_dtype=None, row_scales_ok=False):
        """With ``row_scales_ok`` the caller's next products apply the norm's scale themselves; for a step of
        few tokens the result is then ``RowScaled`` (the norm in two halves, see ``parts.row_scaled``)."""
        if isinstance(delta, (PostNormed, WeightedSum)):
            n = h.shape[0] if rows is None else rows.numel()
            out = torch.empty((n, self.size), dtype=out_dtype or self.rt.act_dtype, device=h.device)
            _general_add_norm(h, delta, self.gain, False, self.eps, out, rows, write_h)
            return out
        if h.dim() == 2 and isinstance(delta, StreamUpdate):
            h = h.unsqueeze(0)       # one copy, with connection weights of its own
        if h.dim() == 3:
            n = h.shape[1] if rows is None else rows.numel()
            out = torch.empty((n, self.size), dtype=out_dtype or self.rt.act_dtype, device=h.device)
            self._streams(h, delta, out, rows, write_h)
            return out
        if (row_scales_ok and rows is None and write_h and out_dtype in (None, torch.bfloat16)
                and self.rt.act_dtype == torch.bfloat16 and h.shape[0] <= self.ROW_SCALE_MAX_TOKENS
                and self.size % 4 == 0):
            T = h.shape[0]
            parts = (self.size + kernels.ADD_SLICE - 1) // kernels.ADD_SLICE
            x = torch.empty((T, self.size), dtype=torch.bfloat16, device=h.device)
            sumsq = torch.empty((parts, max(T, 8)), dtype=torch.float32, device=h.device)
            kernels.add_gain_sumsq(h, delta, self.gain, x, sumsq)
            return RowScaled(x, sumsq, parts, self.eps, self.size)
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype or self.rt.act_dtype, device=h.device)
        kernels.add_rms_norm(h, delta, self.gain, self.eps, out, rows=rows, write_h=write_h)
        return out
