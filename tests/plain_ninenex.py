"""Plain, slow implementation of the Ninenex decoder, for tests only.

Written from the design's equations, one function per mechanism, recurrences
token by token, no cache, float64 on the CPU (so that it sits inside the
float32 rounding of any right implementation).  It shares no code with
``llmoxide_b200``: it has its own reader for the model folder and its own
handling of the configuration.

Notation: x [T, d] is the residual stream of one sequence, positions 0..T-1;
weights are stored [out, in] and applied as W x; ``w`` is the dict of tensors
and ``p`` a layer's prefix ("l3.").
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F = torch.float64


# --------------------------------------------------------------------------
# Model folder
# --------------------------------------------------------------------------

def read_safetensors(path) -> dict:
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = raw[8 + n + lo : 8 + n + hi]
        if info["dtype"] == "BF16":
            arr = (np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
        else:
            arr = np.frombuffer(buf, dtype={"F32": np.float32, "F16": np.float16, "I32": np.int32}[info["dtype"]])
        out[name] = torch.from_numpy(arr.reshape(info["shape"]).copy()).to(F)
    return out


def read_model(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# --------------------------------------------------------------------------
# Small functions
# --------------------------------------------------------------------------

def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x, gain, eps):
    """(x - mean) / sqrt(mean of squared deviations + eps) * gain; no bias."""
    mu = x.mean(-1, keepdim=True)
    dev = x - mu
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * gain


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def log_sigmoid(z):
    return -torch.nn.functional.softplus(-z)


def linear(x, w, name, bias=False):
    y = x @ w[name].T
    return y + w[name + ".b"] if bias else y


def rotate_half(x, positions, dims, base):
    """x [T, heads, D]: dimension i of the first ``dims`` is paired with i + dims/2 and the pair (u, v) is turned
    to (u cos a - v sin a, v cos a + u sin a), a = position * base^(-2i/dims); the other dimensions pass."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = positions.to(F)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# --------------------------------------------------------------------------
# Mixers
# --------------------------------------------------------------------------

def mlstm_recurrence(q, k, v, i_log, f_log):
    """q, k [T, H, D] (q already scaled), v [T, H, Dv], i_log and f_log [T, H]: the matrix memory with a
    running maximum that starts at 0.  Returns o [T, H, Dv]."""
    T, H, D = q.shape
    Dv = v.shape[-1]
    S = torch.zeros((H, D, Dv), dtype=F)
    n = torch.zeros((H, D), dtype=F)
    m = torch.zeros((H,), dtype=F)
    out = torch.zeros((T, H, Dv), dtype=F)
    for t in range(T):
        m_new = torch.maximum(f_log[t] + m, i_log[t])
        a = torch.exp(f_log[t] + m - m_new)
        b = torch.exp(i_log[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    return out


def mlstm_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, D, Dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = linear(h, w, p + "mix.q").view(T, H, D) * D ** -0.5
    k = linear(h, w, p + "mix.k").view(T, H, D)
    v = linear(h, w, p + "mix.v").view(T, H, Dv)
    i_log = cap * torch.tanh(linear(h, w, p + "mix.i", bias=True) / cap)
    f_log = log_sigmoid(cap * torch.tanh(linear(h, w, p + "mix.f", bias=True) / cap))
    o = mlstm_recurrence(q, k, v, i_log, f_log)
    o = unit_rms(o, eps).reshape(T, H * Dv) * w[p + "mix.norm"]
    o = o * torch.sigmoid(linear(h, w, p + "mix.g"))
    return linear(o, w, p + "mix.o")


def chunk_mask(T, size):
    """[T, T] bool: query i sees key j iff j <= i and both lie in the same chunk of ``size`` positions."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def softmax_attention(q, k, v, scale, visible):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; query head h uses key/value head h // (H/G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[-1]), dtype=F)
    for hq in range(H):
        g = hq // (H // G)
        s = (q[:, hq] @ k[:, g].T) * scale
        s = s.masked_fill(~visible, -math.inf)
        out[:, hq] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def chunked_attention(h, w, p, m):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, w, p + "q", bias=True).view(T, H, D)
    k = linear(h, w, p + "k", bias=True).view(T, G, D)
    v = linear(h, w, p + "v", bias=True).view(T, G, Dv)
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot:
        q = rotate_half(q, pos, rot["dims"], float(rot["base"]))
        k = rotate_half(k, pos, rot["dims"], float(rot["base"]))
    mask = m.get("mask")
    visible = chunk_mask(T, mask["size"]) if mask else chunk_mask(T, T)
    o = softmax_attention(q, k, v, float(m["scale"]), visible)
    return linear(o.reshape(T, H * Dv), w, p + "o", bias=True)


def decay_recurrence(q, k, v, decay):
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; S starts at zero."""
    T, H, D = q.shape
    Dv = v.shape[-1]
    S = torch.zeros((H, D, Dv), dtype=F)
    g = torch.tensor([float(x) for x in decay], dtype=F)
    out = torch.zeros((T, H, Dv), dtype=F)
    for t in range(T):
        S = g[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def retention(h, w, p, m, eps):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = linear(h, w, p + "q").view(T, H, D)
    k = linear(h, w, p + "k").view(T, H, D) * D ** -0.5
    v = linear(h, w, p + "v").view(T, H, Dv)
    o = unit_rms(decay_recurrence(q, k, v, m["decay"]), eps).reshape(T, H * Dv)
    return linear(o * silu(linear(h, w, p + "g")), w, p + "o")


def parallel_mixer(h, w, p, m, eps):
    left = chunked_attention(h, w, p + "mix.left.", m["left"])
    right = retention(h, w, p + "mix.right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# --------------------------------------------------------------------------
# Feed-forwards
# --------------------------------------------------------------------------

def dense_ff(h, w, p):
    g = gelu_tanh(linear(h, w, p + "gate", bias=True))
    return linear(g * linear(h, w, p + "up", bias=True), w, p + "down", bias=True)


def expert(h, w, p):
    return linear(silu(linear(h, w, p + "gate")) * linear(h, w, p + "up"), w, p + "down")


def route(z, top):
    """z [T, E] -> (indices [T, top], weights [T, top]): the largest logits, softmax over those only."""
    vals, idx = torch.sort(z, dim=-1, descending=True, stable=True)
    return idx[:, :top], torch.softmax(vals[:, :top], dim=-1)


def moe_ff(h, w, p, mlp, forced=None, logits_out=None):
    """``forced`` [T, top]: experts to use instead of the router's own choice (their weights are still the softmax
    over their logits); ``logits_out``: a list that receives the router's logits.  Both serve comparisons with a
    16-bit implementation, whose rounding may decide a near tie the other way."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = linear(h, w, p + "router", bias=True)
    idx, wt = route(z, top)
    if logits_out is not None:
        logits_out.append(z)
    if forced is not None:
        idx = torch.as_tensor(forced, dtype=torch.long)
        wt = torch.softmax(z.gather(1, idx), dim=-1)
    out = torch.zeros((h.shape[0], w[p + "e0.down"].shape[0]), dtype=F)
    for e in range(E):
        ye = expert(h, w, f"{p}e{e}.")
        for c in range(top):
            out += torch.where(idx[:, c : c + 1] == e, wt[:, c : c + 1] * ye, torch.zeros_like(ye))
    if mlp.get("shared") is not None:
        out = out + expert(h, w, p + "shared.")
    return out


# --------------------------------------------------------------------------
# Model
# --------------------------------------------------------------------------

def forward(cfg, w, tokens, layers_out=None, routing=None, router_logits_out=None):
    """Logits [T, vocab] of one sequence; ``layers_out``: a list that receives the residual stream after
    every layer run; ``routing``: {layer run: experts [T, top]} to use instead of the router's own choice;
    ``router_logits_out``: a dict that receives {layer run: router logits [T, experts]}."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        p = f"l{src}."
        hin = layer_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "mlstm":
            y = mlstm_mixer(hin, w, p, layer["mixer"], eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(hin, w, p, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm(y, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            hin = layer_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                y = dense_ff(hin, w, p + "mlp.")
            else:
                zs = []
                y = moe_ff(hin, w, p + "mlp.", mlp, forced=(routing or {}).get(i), logits_out=zs)
                if router_logits_out is not None:
                    router_logits_out[i] = zs[0]
            x = x + layer_norm(y, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], eps)
    return (x @ w["head"].T) * float(cfg["logit_scale"])
