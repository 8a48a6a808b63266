"""Arrangements: how one layer's norms, mixer and feed-forward are wired
around the residual stream.  ``pre_norm`` is the reference's block
(crates/model/src/qwen35/cpu.rs:141-146,374-400):
h += mixer(norm(h)); h += feed_forward(norm(h)).

The residual stream stays float32.  Each residual add is fused into the norm
that follows it, so a block hands its last delta on as ``pending`` instead of
adding it itself.  ``parallel`` is the block with one norm whose output both
sublayers read: h += mixer(norm(h)) + feed_forward(norm(h)).  A mixer or feed-forward with ``adds_to_residual`` is given the
stream (``residual=h``) and may add its result there itself, in the kernel of its
last product; it then returns None, and the norm that follows has nothing to add.
``sandwich`` norms a sublayer's result as well as its input: h += norm_b(mixer(norm_a(h))), then the same around
the feed-forward; the norm behind a sublayer, the residual add and the norm before the next sublayer are one kernel.
Two options of ``sandwich`` (``BlockSpec.params`` and ``BlockSpec.tensors``): ``mixer_conv_taps`` n > 0, the mixer
reads u + conv(u) instead of the normed stream u, conv a causal convolution over time on every channel (tensor
``mixer_conv`` [width, n]; the last n - 1 rows of u of a sequence are its state, kept in the cache entry's state area);
``result_gate`` "sigmoid", every sublayer's result is multiplied by sigmoid(W u + b) before the norm behind it (tensors
``mixer_gate`` / ``mixer_gate_bias``, ``feed_forward_gate`` / ``feed_forward_gate_bias``; u is the normed stream, before
the convolution); the product W u is one more matrix product, sigmoid and multiplication happen in the norm kernel.
A part whose last product has a bias offers it as ``out_bias``; an arrangement that can add it in its own norm
kernel sets the part's ``defer_out_bias``, and the part then leaves the bias to it."""

from __future__ import annotations

import torch

from .. import kernels
from ..cache import StateNeed
from ..errors import Unsupported
from .linear import Linear
from .registry import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, lookup, register_arrangement)


def build_part(table, family, spec, *args):
    return lookup(table, family, spec.kind)(spec, *args)


@register_arrangement("pre_norm")
class PreNormBlock:
    def __init__(self, spec, weights: dict, rt):
        position = None
        if spec.position is not None:
            position = rt_shared_position(spec.position, weights, rt)
        self.mixer_norm = build_part(NORMS, "norm", spec.norms["mixer"], weights, rt)
        self.ff_norm = build_part(NORMS, "norm", spec.norms["feed_forward"], weights, rt)
        self.mixer = lookup(MIXERS, "mixer", spec.mixer.kind)(spec.mixer, position, weights, rt)
        self.feed_forward = build_part(FEED_FORWARDS, "feed-forward", spec.feed_forward, weights, rt)

    def cache_need(self):
        return self.mixer.cache_need()

    def libraries(self) -> set:
        libs = set()
        for part in (self.mixer_norm, self.ff_norm, self.mixer, self.feed_forward):
            libs |= getattr(part, "libraries", set)()
        return libs

    def forward(self, h, pending, ctx, view, writes_cache=True):
        probe = getattr(ctx, "probe", None)
        x = _norm(self.mixer_norm, h, pending, self.mixer, plain=probe is not None)
        if probe:
            probe("resid_in", h), probe("attn_norm", x)      # names after crates/model/src/qwen35/cpu.rs:136-401
        if probe is None and getattr(self.mixer, "adds_to_residual", False):
            a = self.mixer.forward(x, ctx, view, writes_cache, residual=h)
        else:
            a = self.mixer.forward(x, ctx, view, writes_cache)
        if probe:
            probe("attn_output", _summed(a))
        x = _norm(self.ff_norm, h, a, self.feed_forward, plain=probe is not None)
        if probe:
            probe("attn_residual", h), probe("attn_post_norm", x)
        if probe is None and getattr(self.feed_forward, "adds_to_residual", False):
            out = self.feed_forward.forward(x, ctx, residual=h)
        else:
            out = self.feed_forward.forward(x, ctx)
        if probe:
            probe("ffn_out", _summed(out))
        return out


def _summed(delta):
    """A delta as one tensor: split partials [S,T,d] are added in order."""
    from .norm import WeightedSum
    if isinstance(delta, WeightedSum):
        return sum(w * _summed(t).float() for t, w in delta.terms)
    if delta.dim() == 2:
        return delta
    out = torch.empty(delta.shape[1:], dtype=torch.float32, device=delta.device)
    kernels.sum_splits(delta, out)
    return out


def _norm(norm, h, delta, consumer, plain=False):
    """h += delta; x = norm(h).  Where both sides can, the norm is done in two halves: the norm part leaves the
    scale to the consumer's first products (``takes_row_scales`` on the consumer, ``row_scales_ok`` on the norm);
    not when the step's intermediates are asked for (``plain``), which wants the normalised rows themselves."""
    if not plain and getattr(consumer, "takes_row_scales", False) and getattr(norm, "ROW_SCALE_MAX_TOKENS", 0):
        return norm.add_forward(h, delta, row_scales_ok=True)
    return norm.add_forward(h, delta)


def rt_shared_position(spec, weights, rt):
    """Layers with the same position encoding share one object (and its tables)."""
    key = ("position", spec.kind, tuple(sorted((k, repr(v)) for k, v in spec.params.items())))
    if key not in rt.shared:
        rt.shared[key] = build_part(POSITIONS, "position encoding", spec, weights, rt)
    return rt.shared[key]


def build_block(spec, weights: dict, rt):
    return lookup(ARRANGEMENTS, "block arrangement", spec.arrangement)(spec, weights, rt)


@register_arrangement("parallel")
class ParallelBlock:
    """A single norm feeds mixer and feed-forward: x = norm(h); h += mixer(x) + feed_forward(x).  The mixer's
    result joins the float32 stream at once (nothing else reads the stream before the next layer's norm, and the
    feed-forward reads x); the feed-forward's is handed on as the pending delta, which the next norm adds."""

    def __init__(self, spec, weights: dict, rt):
        position = None
        if spec.position is not None:
            position = rt_shared_position(spec.position, weights, rt)
        self.norm = build_part(NORMS, "norm", spec.norms["shared"], weights, rt)
        self.mixer = lookup(MIXERS, "mixer", spec.mixer.kind)(spec.mixer, position, weights, rt)
        self.feed_forward = build_part(FEED_FORWARDS, "feed-forward", spec.feed_forward, weights, rt)

    def cache_need(self):
        return self.mixer.cache_need()

    def libraries(self) -> set:
        libs = set()
        for part in (self.norm, self.mixer, self.feed_forward):
            libs |= getattr(part, "libraries", set)()
        return libs

    def forward(self, h, pending, ctx, view, writes_cache=True):
        probe = getattr(ctx, "probe", None)
        x = self.norm.add_forward(h, pending)
        if probe:
            probe("resid_in", h), probe("attn_norm", x)
        if probe is None and getattr(self.mixer, "adds_to_residual", False):
            a = self.mixer.forward(x, ctx, view, writes_cache, residual=h)
        else:
            a = self.mixer.forward(x, ctx, view, writes_cache)
        if probe:
            probe("attn_output", _summed(a))
        out = self.feed_forward.forward(x, ctx)
        if probe and out is not None:
            probe("ffn_out", _summed(out))
        if a is not None:
            if out is None:
                return a
            self.norm.add(h, a)
        return out


@register_arrangement("hyper_connections")
class HyperConnectionBlock:
    """Pre-norm sublayers over ``streams`` copies of the residual stream (h [S,T,d], float32).  Sublayer q reads
    u = sum_s in_q[s] h_s through its norm; its result y joins the copies as
    h_r <- sum_s mix_q[s,r] h_s + residual_mult * out_q[r] * y, every copy from the old ones.  The weights ride
    with the sublayer's norm (``parts.norm``); the update is owed to the next norm, whose kernel applies it while it
    reads the copies, so a layer is two norm kernels beside its mixer and feed-forward as in ``pre_norm``.  With one
    copy and no connection weights this is h += residual_mult * sublayer(norm(h))."""

    def __init__(self, spec, weights: dict, rt):
        position = None
        if spec.position is not None:
            position = rt_shared_position(spec.position, weights, rt)
        self.streams = int(spec.params.get("streams", 1))
        mult = float(spec.params.get("residual_mult", 1.0))
        self.mixer_norm = build_part(NORMS, "norm", _with_mult(spec.norms["mixer"], mult), weights, rt)
        self.mixer = lookup(MIXERS, "mixer", spec.mixer.kind)(spec.mixer, position, weights, rt)
        self.feed_forward = build_part(FEED_FORWARDS, "feed-forward", spec.feed_forward, weights, rt)
        self.ff_norm = None
        if "feed_forward" in spec.norms:
            self.ff_norm = build_part(NORMS, "norm", _with_mult(spec.norms["feed_forward"], mult), weights, rt)

    def cache_need(self):
        return self.mixer.cache_need()

    def libraries(self) -> set:
        libs = set()
        for part in (self.mixer_norm, self.ff_norm, self.mixer, self.feed_forward):
            if part is not None:
                libs |= getattr(part, "libraries", set)()
        return libs

    def forward(self, h, pending, ctx, view, writes_cache=True):
        if h.dim() == 2:
            h = h.unsqueeze(0)
        S = h.shape[0]
        probe = getattr(ctx, "probe", None)
        if probe:
            self.mixer_norm.add(h, pending)
            pending = None
            probe("resid_in", h.sum(0))
        x = self.mixer_norm.add_forward(h, pending)
        a = self.mixer.forward(x, ctx, view, writes_cache)
        if probe:
            probe("attn_norm", x), probe("attn_output", _summed(a))
        pending = self.mixer_norm.owed(a, S)
        if self.ff_norm is None:
            return pending
        x = self.ff_norm.add_forward(h, pending)
        out = self.feed_forward.forward(x, ctx)
        if probe:
            probe("attn_post_norm", x)
            if out is not None:
                probe("ffn_out", _summed(out))
        return self.ff_norm.owed(out, S)


def _with_mult(norm_spec, mult: float):
    """The norm's description with the factor on its sublayer's result."""
    from ..config.spec import PartSpec
    return PartSpec(norm_spec.kind, dict(norm_spec.params, residual_mult=mult), norm_spec.tensors)


@register_arrangement("sandwich")
class SandwichBlock:
    """A norm before and a norm behind each sublayer: h += post(mixer(pre(h))), then h += post(feed_forward(pre(h)))
    (norms ``mixer``, ``mixer_post``, ``feed_forward``, ``feed_forward_post``; a layer without a feed-forward has the
    first two).  The normed result is owed to the next norm before a sublayer, whose kernel norms it, adds it to the
    float32 stream and norms the stream in one pass over the row; the sublayers' output biases ride along."""

    def __init__(self, spec, weights: dict, rt):
        position = None
        if spec.position is not None:
            position = rt_shared_position(spec.position, weights, rt)
        self.mixer_norm = build_part(NORMS, "norm", spec.norms["mixer"], weights, rt)
        self.mixer_post = build_part(NORMS, "norm", spec.norms["mixer_post"], weights, rt)
        self.mixer = lookup(MIXERS, "mixer", spec.mixer.kind)(spec.mixer, position, weights, rt)
        self.feed_forward = build_part(FEED_FORWARDS, "feed-forward", spec.feed_forward, weights, rt)
        self.ff_norm = self.ff_post = None
        if "feed_forward" in spec.norms:
            self.ff_norm = build_part(NORMS, "norm", spec.norms["feed_forward"], weights, rt)
            self.ff_post = build_part(NORMS, "norm", spec.norms["feed_forward_post"], weights, rt)
        for part in (self.mixer, self.feed_forward):
            if getattr(part, "out_bias", None) is not None:
                part.defer_out_bias = True           # added by the norm kernel behind the part
        self.width = spec.norms["mixer"]["size"]
        self.taps = int(spec.params.get("mixer_conv_taps") or 0)
        self.conv_w = None
        if self.taps:
            if self.taps > kernels.CONV_MAX_TAPS:
                raise Unsupported(f"{self.taps} taps: the convolution kernels take up to {kernels.CONV_MAX_TAPS}")
            # [channels, taps] -> tap-major [taps, channels]: neighbouring threads read neighbouring channels of a tap
            self.conv_w = weights.pop(spec.tensors["mixer_conv"].name).to(torch.float32).t().contiguous()
        gate = spec.params.get("result_gate")
        if gate not in (None, "sigmoid"):
            raise Unsupported(f"result_gate {gate!r}: 'sigmoid' or none")
        self.mixer_gate = self.ff_gate = None
        if gate:
            t = spec.tensors
            self.mixer_gate = Linear(weights.pop(t["mixer_gate"].name), rt, bias=weights.pop(t["mixer_gate_bias"].name))
            if self.ff_norm is not None:
                self.ff_gate = Linear(weights.pop(t["feed_forward_gate"].name), rt,
                                      bias=weights.pop(t["feed_forward_gate_bias"].name))

    def cache_need(self):
        kv, state = self.mixer.cache_need()
        if self.taps > 1:
            if state is not None:
                raise Unsupported("a convolution before a mixer that keeps state of its own is not built")
            state = StateNeed((self.taps - 1, self.width))
        return kv, state

    def libraries(self) -> set:
        libs = {"short_conv"} if self.taps else set()
        for part in (self.mixer_norm, self.mixer_post, self.ff_norm, self.ff_post, self.mixer, self.feed_forward,
                     self.mixer_gate, self.ff_gate):
            if part is not None:
                libs |= getattr(part, "libraries", set)()
        return libs

    def _convolved(self, x, ctx, view):
        """u + conv(u), and the state moved on by the step's rows."""
        out = torch.empty_like(x)
        inline = bool(ctx.is_decode and self.taps > 1)
        kernels.residual_conv(x, view.state, self.conv_w, self.taps, out, ctx, inline_state=inline)
        if self.taps > 1 and not inline:
            kernels.conv_state_update(x, view.state, self.taps, ctx)
        return out

    def forward(self, h, pending, ctx, view, writes_cache=True):
        probe = getattr(ctx, "probe", None)
        if probe:
            self.mixer_norm.add(h, pending)
            pending = None
            probe("resid_in", h)
        x = self.mixer_norm.add_forward(h, pending)
        # the gate's logits come from the normed stream itself; its bias, the sigmoid and the multiplication are
        # the norm kernel's
        gate = None
        if self.mixer_gate is not None:
            gate = (self.mixer_gate(x, out_dtype=torch.float32, splits_ok=True, add_bias=False), self.mixer_gate.bias)
        u = self._convolved(x, ctx, view) if self.taps else x
        a = self.mixer.forward(u, ctx, view, writes_cache)
        if probe:
            probe("attn_norm", x), probe("attn_output", _summed(a))
        pending = self.mixer_post.owed(a, bias=getattr(self.mixer, "out_bias", None), gate=gate)
        if self.ff_norm is None:
            return pending
        x = self.ff_norm.add_forward(h, pending)
        gate = None
        if self.ff_gate is not None:
            gate = (self.ff_gate(x, out_dtype=torch.float32, splits_ok=True, add_bias=False), self.ff_gate.bias)
        out = self.feed_forward.forward(x, ctx)
        if probe:
            probe("attn_residual", h), probe("attn_post_norm", x)
            if out is not None:
                probe("ffn_out", _summed(out))
        return self.ff_post.owed(out, bias=getattr(self.feed_forward, "out_bias", None), gate=gate)
