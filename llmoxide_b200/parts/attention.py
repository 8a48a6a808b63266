"""Grouped-query attention as a mixer: fused q/k/v projection, optional
per-head RMSNorm of q and k, rotation, cache write, attention over the cache
(all keys or a window of them), output projection.

Formulas in the reference's order (crates/model/src/qwen35/cpu.rs:283-368):
q = Wq x, k = Wk x, v = Wv x; per head q <- rope(rms(q) * q_norm), k likewise,
v untouched; k and v of the whole step are stored before any score is taken;
query head hq reads kv head hq // (H/G); scores are scaled by ``scale``; the
query at position p sees keys first..p, first = 0 or p-(w-1) under a window
(crates/model/src/cache.rs:31-37).

Beyond the reference's layer: values may have a size of their own
(``v_head_dim``); under a window the first ``keep_first`` keys of a sequence
may stay visible (from position p, key j is visible iff j <= p and either
p - j < window or j < keep_first); a layer without key/value projections of its own
(``own_kv`` false) only makes queries and reads the cache entry of the call
that owns it, which then keeps what the widest of its readers can see
(``cache_window``, ``cache_keep_first``).

Three more options, each a parameter.  ``conv_taps`` n > 0: a short causal
convolution over time on every channel of q, k and v, directly after the
projection (tensors ``q_conv``, ``k_conv``, ``v_conv`` [channels, n], no bias:
y_p = sum_j w[:, j] u_(p - n + 1 + j), zeros before the sequence's start); the
last n - 1 projected rows of a sequence are per-sequence state.  ``sink`` s > 0:
the softmax's denominator has s added, w_j = exp(s_j) / (s + sum_j exp(s_j)) (a
sink of score 0 that has no value).  ``v_mix``: "source" leaves this call's
values (after the convolution) for later calls of the step under the name
``v_mix_key``; "mix" replaces its values by (1 - l) v + l v_source with the
learned scalar l (tensor ``v_mix``) before they are cached.

``chunk`` n > 0: positions are cut into chunks of n, counted from position 0 of
the sequence, and a query sees the keys j <= p of its own chunk only
(floor(j / n) = floor(p / n)); the cache entry keeps what a window of n would.
``pool`` n > 1, beside a window: every block of n positions that lies wholly before the window (block b =
positions b*n .. b*n+n-1, seen from p once b*n+n-1 <= p - window) is seen as one key and one value, the means of the
block's keys and values as the cache holds them (after norm and rotation), in the same softmax as the window's keys.
The cache entry then owns a second store of one row per block (``KVNeed.pool``), written when a step brings a
block's last position; positions that have left the window and whose block is not complete are not seen.  A position
encoding that pairs neighbouring dimensions is met by reordering the rows of the q and k projections once
(``parts.position.halves_order``).
Tensors ``q_bias``, ``k_bias``, ``v_bias``, ``o_bias``: biases of the four
projections (q, k, v: added where the projected row is read, before norm and
rotation; o: offered as ``out_bias`` to an arrangement that adds it in its
norm kernel, else added here).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache import KVNeed, StateNeed
from ..errors import Unsupported
from .linear import Linear
from .position import halves_order
from .registry import register_mixer


@register_mixer("gqa_attention")
class GQAttention:
    def __init__(self, spec, position, weights: dict, rt):
        self.rt = rt
        self.H, self.G, self.D = spec["n_heads"], spec["n_kv_heads"], spec["head_dim"]
        self.scale = float(spec["scale"])
        self.Dv = spec.get("v_head_dim") or self.D
        self.window = spec.get("window")
        self.keep_first = int(spec.get("keep_first") or 0) if self.window else 0
        self.chunk = int(spec.get("chunk") or 0)
        if self.chunk and (self.window or not bool(spec.get("own_kv", True))):
            raise Unsupported("a chunked mask is built for a layer with its own keys and values and no window")
        # what the cache entry holds: this layer's own mask unless the description names a wider one
        self.cache_window = spec.get("cache_window", self.window) if "cache_window" in spec.params else self.window
        if self.chunk:
            self.cache_window = self.chunk           # nothing before the last `chunk` positions is seen again
        self.pool = int(spec.get("pool") or 0)
        if self.pool == 1:
            self.pool = 0                            # blocks of one position: every earlier key, as it is
            self.window = self.cache_window = None
        if self.pool:
            if not self.window or self.keep_first or self.chunk or not bool(spec.get("own_kv", True)):
                raise Unsupported("pooled blocks are built for a layer with its own keys and values under a plain window")
            # a block's mean is taken from the cache when its last position arrives
            self.cache_window = max(int(self.cache_window or 0), self.pool)
        self.cache_keep_first = int(spec.get("cache_keep_first", self.keep_first) or 0) if self.cache_window else 0
        self.own_kv = bool(spec.get("own_kv", True))
        self.eps = float(spec.get("qk_norm_eps") or 0.0)
        if self.H % self.G:
            raise Unsupported(f"{self.H} heads are not a multiple of {self.G} kv heads")
        # the shape the tiled kernels are written for; every other one goes to the general kernel
        self.plain = self.Dv == self.D and self.D % 16 == 0
        if max(self.D, self.Dv) > 256:
            raise Unsupported(f"head sizes {self.D}/{self.Dv}: the attention kernels take sizes up to 256")
        t = spec.tensors
        if self.own_kv:
            wq, wk, wv = (weights.pop(t[r].name) for r in ("q", "k", "v"))
            if not (wq.dtype == wk.dtype == wv.dtype):
                wq, wk, wv = wq.float(), wk.float(), wv.float()
            wq, wk = halves_order(position, wq, self.H, self.D), halves_order(position, wk, self.G, self.D)
            # One matrix product for q, k and v: rows of q, then k, then v.
            wqkv = torch.cat([wq, wk, wv], dim=0)
            del wq, wk, wv
            self.qkv = Linear(wqkv, rt)
            self.q_only = Linear(wqkv[: self.H * self.D], rt)
        else:
            self.qkv = None
            self.q_only = Linear(halves_order(position, weights.pop(t["q"].name), self.H, self.D), rt)
        self.o = Linear(weights.pop(t["o"].name), rt, bias=weights.pop(t["o_bias"].name) if "o_bias" in t else None)
        self.out_bias, self.defer_out_bias = self.o.bias, False
        self.qkv_bias = None
        if "q_bias" in t:
            if not self.own_kv:
                raise Unsupported("projection biases are built for a layer with its own keys and values")
            bq, bk, bv = (weights.pop(t[r].name).to(torch.float32) for r in ("q_bias", "k_bias", "v_bias"))
            bq = halves_order(position, bq.unsqueeze(1), self.H, self.D).squeeze(1)
            bk = halves_order(position, bk.unsqueeze(1), self.G, self.D).squeeze(1)
            self.qkv_bias = torch.cat([bq, bk, bv]).contiguous()
        self.q_gain = self.k_gain = None
        if "q_norm" in t:
            self.q_gain = weights.pop(t["q_norm"].name).to(torch.float32).contiguous()
            self.k_gain = weights.pop(t["k_norm"].name).to(torch.float32).contiguous()
        self.position = position
        if getattr(position, "pairing", "halves") == "neighbours" and ("q_norm" in t or spec.get("conv_taps")):
            raise Unsupported("a rotation of neighbouring pairs beside a q/k norm or a short convolution is not built")
        self.taps = int(spec.get("conv_taps") or 0)
        self.sink = float(spec.get("sink") or 0.0)
        self.v_mix, self.v_mix_key = spec.get("v_mix"), spec.get("v_mix_key", "v_mix")
        if self.v_mix not in (None, "source", "mix"):
            raise Unsupported(f"v_mix {self.v_mix!r}: 'source' or 'mix'")
        self.conv_w = self.v_lambda = None
        if self.qkv_bias is not None and (self.taps or self.v_mix):
            raise Unsupported("projection biases beside a short convolution or mixed values are not built")
        if self.taps:
            if not self.own_kv or self.q_gain is not None:
                raise Unsupported("the short convolution is built for a layer with its own keys and values and no q/k norm")
            # [channels of q | k | v, taps] -> tap-major [taps, channels]: a warp reads neighbouring channels of a tap
            self.conv_w = torch.cat([weights.pop(t[r].name).to(torch.float32) for r in ("q_conv", "k_conv", "v_conv")],
                                    dim=0).t().contiguous()
        if self.v_mix == "mix":
            self.v_lambda = weights.pop(t["v_mix"].name).to(torch.float32).reshape(1).contiguous()
        # the projection's rows go through the convolution kernel (which also rotates, mixes and writes the cache)
        self.staged = bool(self.taps or self.v_mix)
        self.channels = (self.H + self.G) * self.D + self.G * self.Dv

    def cache_need(self):
        state = StateNeed((self.taps - 1, self.channels)) if self.taps > 1 else None
        return KVNeed(self.G, self.D, self.cache_window, v_head_dim=None if self.Dv == self.D else self.Dv,
                      keep_first=self.cache_keep_first, pool=self.pool), state

    @property
    def takes_row_scales(self) -> bool:
        """Its first products (q|k|v) can apply a norm's row scales in their epilogue."""
        return (self.qkv is None or self.qkv.takes_row_scales) and self.q_only.takes_row_scales

    def libraries(self) -> set:
        libs = {"elementwise"} | self.q_only.libraries() | self.o.libraries()
        if self.staged:
            libs.add("short_conv")
        if self.pool:
            libs.add("attention")           # the blocks' means are made there
        if not self.plain:
            return libs | {"attention"}
        if self.rt.dtype == "bfloat16" and self.rt.tensor_cores:
            tc = self.D == 128 and not self.pool      # (pooled blocks: the mma.sync kernel, at both head sizes)
            libs |= {"attention_decode",
                     "attention_prefill_tc" if tc else "attention_prefill" if self.D in (64, 128) else "attention"}
        else:
            libs.add("attention")
        return libs

    adds_to_residual = True      # forward() takes ``residual`` and may return None: "already added"

    def forward(self, x, ctx, view, writes_cache=True, residual=None):
        H, G, D, Dv = self.H, self.G, self.D, self.Dv
        T = x.shape[0]
        dev = x.device
        tables = self.position.rotary_tables() if self.position is not None else None
        cos, sin, n_rot = tables if tables is not None else (None, None, 0)
        block_table = ctx.block_tables[view.group]
        if writes_cache and not self.own_kv:
            raise Unsupported("a layer without key/value projections cannot write a cache entry")
        if self.staged:
            if not writes_cache:
                raise Unsupported("a layer with a short convolution or mixed values owns its cache entry")
            qkv = self.qkv(x, splits_ok=True)
            q = torch.empty((T, H * D), dtype=self.rt.act_dtype, device=dev)
            v_first, mode = None, 0
            if self.v_mix == "source":
                v_first = ctx.carry[self.v_mix_key] = torch.empty((T, G * Dv), dtype=torch.float32, device=dev)
                mode = 1
            elif self.v_mix == "mix":
                v_first, mode = ctx.carry[self.v_mix_key], 2
            # a step of single tokens moves the convolution's state on inside the same kernel
            inline = bool(ctx.is_decode and self.taps > 1)
            kernels.conv_rope_cache(qkv, view.state, self.conv_w, self.taps, q, view.k, view.v, block_table, ctx, cos, sin,
                                    n_rot, v_first, self.v_lambda, mode, H, G, D, Dv, inline_state=inline)
            if not inline:
                kernels.conv_state_update(qkv, view.state, self.taps, ctx)
        elif not writes_cache and self.q_gain is None and n_rot == 0 and self.qkv_bias is None:
            # A call that reads another call's cache entry makes only queries; nothing is done to them.
            q = self.q_only(x, out_dtype=self.rt.act_dtype)
        else:
            if writes_cache:
                qkv = self.qkv(x, splits_ok=True)
            elif self.qkv_bias is not None:
                raise Unsupported("a layer with projection biases owns its cache entry")
            else:
                q_part = self.q_only(x)
                qkv = torch.empty((T, (H + G) * D + G * Dv), dtype=q_part.dtype, device=dev)
                qkv[:, : H * D] = q_part
            q = torch.empty((T, H * D), dtype=self.rt.act_dtype, device=dev)
            kernels.qk_norm_rope_cache(qkv, q, view.k, view.v, block_table, ctx.token_seq, ctx.token_pos,
                                       self.q_gain, self.k_gain, self.eps, cos, sin, n_rot, H, G, D, writes_cache,
                                       v_head_dim=Dv, bias=self.qkv_bias)
        if self.pool and writes_cache:
            kernels.pool_blocks(view.k, view.v, block_table, view.pool_k, view.pool_v, ctx.block_tables[view.pool_group],
                                ctx.seq_start, ctx.seq_past, ctx.n_seqs, T, G, D, Dv, self.pool)
        out = torch.empty((T, H * Dv), dtype=self.rt.act_dtype, device=dev)
        self.attend(q, out, view, block_table, ctx)
        if self.out_bias is None and residual is not None and self.o.add_into(out, residual):
            return None
        return self.o(out, splits_ok=True, add_bias=not self.defer_out_bias)

    def attend(self, q, out, view, block_table, ctx):
        """bfloat16: the split-key kernel when every sequence brings one token;
        for prompts the tcgen05 kernel at head size 128 and the mma.sync tiled
        kernel at head size 64; the general kernel otherwise (values of another
        size than the keys among them) and always in float32.  All of them take
        a window that keeps its first keys, and a chunked mask."""
        H, G, D = self.H, self.G, self.D
        fast = (self.plain and q.dtype == torch.bfloat16 and view.k.dtype == torch.bfloat16
                and self.rt.tensor_cores and self.scale > 0)       # (the tiled kernels take the maximum before the scale)
        pooled = dict(pool=self.pool, pool_k=view.pool_k, pool_v=view.pool_v,
                      pool_table=ctx.block_tables[view.pool_group]) if self.pool else {}
        if fast and ctx.is_decode:
            kernels.attention_decode(q, out, view.k, view.v, block_table, ctx.seq_past, H, G, D, self.window,
                                     self.scale, keep_first=self.keep_first, sink=self.sink, chunk=self.chunk, **pooled)
        elif fast and D == 128 and not self.pool:
            kernels.attention_prefill_tc(q, out, view.k, view.v, block_table, ctx.seq_start, ctx.seq_past,
                                         ctx.n_seqs, ctx.max_new, H, G, D, self.window, self.scale,
                                         keep_first=self.keep_first, sink=self.sink, chunk=self.chunk)
        elif fast and kernels.attention_prefill_supports(q, view.k, D):
            kernels.attention_prefill(q, out, view.k, view.v, block_table, ctx.seq_start, ctx.seq_past,
                                      ctx.n_seqs, ctx.max_new, H, G, D, self.window, self.scale,
                                      keep_first=self.keep_first, sink=self.sink, chunk=self.chunk, **pooled)
        else:
            kernels.attention_paged(q, out, view.k, view.v, block_table, ctx.token_seq, ctx.token_pos,
                                    H, G, D, self.window, self.scale, v_head_dim=self.Dv, keep_first=self.keep_first,
                                    sink=self.sink, chunk=self.chunk, **pooled)
