"""Attention whose queries, keys and values come through low-rank latents.

For the mixer's input x (one row per token), H heads, per head D unrotated and
R rotated query/key dimensions and values of size Dv:

    cq = rms(W_dq x) * g_q                     the query latent (rank ``q_rank``)
    q  = W_uq cq                               per head [D unrotated | R rotated]
    [c_raw | kr] = W_dkv x                     ``kv_rank`` + R rows
    c  = rms(c_raw) * g_kv                     the key/value latent
    k_h = [W_uk c (head h, D) | rot(kr)]       kr is one rotated part that all heads share
    v_h = W_uv c (head h, Dv)
    s   = (q_plain . k_plain + rot(q_rot) . rot(kr)) * scale, softmax over the window's keys
    out = W_o concat_h( sigmoid(W_g x)_h * sum_j w_j v_j )      (``out_gate`` "sigmoid"; None: no gate)

rms is x / sqrt(mean(x^2) + eps) in float32.  The rotation is the position
part's (any table of ``rot_dim`` dimensions: scaled frequencies, an amplitude).

What is cached.  The latent c and the rotated part kr are all that later
tokens need, and a cache of those alone is the smallest there is; this part
caches every head's assembled key [rot(kr) | k_plain] and value instead, H
heads of R + D and Dv, because the design it was built for attends under a
window: the cache holds at most the window's tokens per sequence whatever the
context's length, and assembled keys run on every attention kernel of this
package (tensor cores for prompts and decode at R + D = Dv in {64, 128})
without a product per cached token in every step.  Within a head the rotated
part is stored first, which no scalar product notices as queries are laid out
alike.

Products: W_dq, W_dkv and W_g read the same rows and are one fused product
(float32 out, so the norms and the gate see unrounded sums); W_uk and W_uv are
one product over c.  Two small kernels sit between them (``csrc/latent_attention.cu``):
the two latents' norms, and rotation + key assembly + cache write.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache import KVNeed
from ..errors import Unsupported
from .linear import Linear
from .position import halves_order
from .registry import register_mixer


@register_mixer("latent_attention")
class LatentAttention:
    def __init__(self, spec, position, weights: dict, rt):
        self.rt = rt
        self.H, self.D, self.R, self.Dv = spec["n_heads"], spec["head_dim"], spec["rot_dim"], spec["v_head_dim"]
        self.Rq, self.Rkv = spec["q_rank"], spec["kv_rank"]
        self.eps, self.scale = float(spec["eps"]), float(spec["scale"])
        self.window = spec.get("window")
        self.gate = spec.get("out_gate")
        if self.gate not in (None, "sigmoid"):
            raise Unsupported(f"out_gate {self.gate!r}: 'sigmoid' or none")
        if position is None or position.rotary_tables() is None or position.n_rot != self.R:
            raise Unsupported("latent attention rotates exactly its rot_dim dimensions: the position part must say so")
        self.position = position
        self.E = self.R + self.D                      # an assembled key, a query head
        if max(self.E, self.Dv) > 256:
            raise Unsupported(f"head sizes {self.E}/{self.Dv}: the attention kernels take sizes up to 256")
        H, D, R, Dv = self.H, self.D, self.R, self.Dv
        t = spec.tensors
        wdq, wdkv = weights.pop(t["dq"].name), weights.pop(t["dkv"].name)
        # the shared rotated part's rows in the order the kernels pair them
        wdkv = torch.cat([wdkv[: self.Rkv], halves_order(position, wdkv[self.Rkv :], 1, R)], dim=0)
        rows = [wdq, wdkv] + ([weights.pop(t["g"].name)] if self.gate else [])
        if len({w.dtype for w in rows}) > 1:
            rows = [w.float() for w in rows]
        self.down = Linear(torch.cat(rows, dim=0).contiguous(), rt)
        self.k_rot_off, self.gate_off = self.Rq + self.Rkv, self.Rq + self.Rkv + R
        # queries: every head's rows become [rotated (paired as the kernels pair) | unrotated]
        wuq = weights.pop(t["uq"].name)
        wuq = halves_order(position, wuq, H, D + R, first=D)
        index = torch.tensor([h * (D + R) + i for h in range(H) for i in list(range(D, D + R)) + list(range(D))],
                             device=wuq.device)
        self.uq = Linear(wuq.index_select(0, index).contiguous(), rt)
        wuk, wuv = weights.pop(t["uk"].name), weights.pop(t["uv"].name)
        if wuk.dtype != wuv.dtype:
            wuk, wuv = wuk.float(), wuv.float()
        self.ukv = Linear(torch.cat([wuk, wuv], dim=0).contiguous(), rt)
        self.q_gain = weights.pop(t["dq_norm"].name).to(torch.float32).contiguous()
        self.kv_gain = weights.pop(t["dkv_norm"].name).to(torch.float32).contiguous()
        self.o = Linear(weights.pop(t["o"].name), rt)
        self.out_bias, self.defer_out_bias = None, False
        # the shape the tiled kernels are written for
        self.plain = self.E == Dv and self.E % 16 == 0

    def cache_need(self):
        return KVNeed(self.H, self.E, self.window, v_head_dim=None if self.Dv == self.E else self.Dv), None

    def libraries(self) -> set:
        libs = {"latent_attention", "elementwise"} | self.down.libraries() | self.uq.libraries() | self.o.libraries()
        if self.plain and self.rt.dtype == "bfloat16" and self.rt.tensor_cores:
            libs |= {"attention_decode",
                     "attention_prefill_tc" if self.E == 128 else "attention_prefill" if self.E == 64 else "attention"}
        else:
            libs.add("attention")
        return libs

    def forward(self, x, ctx, view, writes_cache=True):
        if not writes_cache:
            raise Unsupported("a latent attention layer owns its cache entry")
        H, D, R, Dv, E = self.H, self.D, self.R, self.Dv, self.E
        T, dev, act = x.shape[0], x.device, self.rt.act_dtype
        down = self.down(x, out_dtype=torch.float32)                         # [T, Rq + Rkv + R (+ H)]
        cq = torch.empty((T, self.Rq), dtype=act, device=dev)
        c = torch.empty((T, self.Rkv), dtype=act, device=dev)
        kernels.latent_norms(down, self.q_gain, self.kv_gain, self.eps, cq, c, self.Rq, self.Rkv)
        q_up = self.uq(cq)
        kv_up = self.ukv(c)
        cos, sin, _ = self.position.rotary_tables()
        block_table = ctx.block_tables[view.group]
        q = torch.empty((T, H * E), dtype=act, device=dev)
        kernels.latent_rope_cache(q_up, kv_up, down, self.k_rot_off, q, view.k, view.v, block_table, ctx, cos, sin,
                                  H, D, R, Dv)
        gate = down[:, self.gate_off :] if self.gate else None               # the heads' gate logits, a view
        out = torch.empty((T, H * Dv), dtype=act, device=dev)
        self.attend(q, out, view, block_table, ctx, gate)
        return self.o(out, splits_ok=True)

    def attend(self, q, out, view, block_table, ctx, gate):
        """The general kernel applies the heads' gates itself; the tiled bfloat16 kernels (decode, and prompts at
        head sizes 64 and 128) are followed by the gate's own small kernel."""
        H, E = self.H, self.E
        fast = (self.plain and q.dtype == torch.bfloat16 and view.k.dtype == torch.bfloat16
                and self.rt.tensor_cores and self.scale > 0)
        if fast and ctx.is_decode:
            kernels.attention_decode(q, out, view.k, view.v, block_table, ctx.seq_past, H, H, E, self.window, self.scale)
        elif fast and E == 128:
            kernels.attention_prefill_tc(q, out, view.k, view.v, block_table, ctx.seq_start, ctx.seq_past,
                                         ctx.n_seqs, ctx.max_new, H, H, E, self.window, self.scale)
        elif fast and kernels.attention_prefill_supports(q, view.k, E):
            kernels.attention_prefill(q, out, view.k, view.v, block_table, ctx.seq_start, ctx.seq_past,
                                      ctx.n_seqs, ctx.max_new, H, H, E, self.window, self.scale)
        else:
            kernels.attention_paged(q, out, view.k, view.v, block_table, ctx.token_seq, ctx.token_pos,
                                    H, H, E, self.window, self.scale, v_head_dim=self.Dv, gate=gate)
            return
        if gate is not None:
            kernels.head_gate(out, gate, H, self.Dv)
