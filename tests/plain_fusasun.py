"""Plain, slow implementation of the Fusasun decoder, for tests only.

Written from the design's equations, one function per mechanism, whole
sequences at once, no cache, float64 on the CPU (so that it sits inside the
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
YARN_AMPLITUDE_SLOPE = 0.1


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
            out[name] = torch.from_numpy(arr.reshape(info["shape"]).copy()).to(F)
        elif info["dtype"] in ("I32", "I64"):
            arr = np.frombuffer(buf, dtype={"I32": np.int32, "I64": np.int64}[info["dtype"]])
            out[name] = torch.from_numpy(arr.reshape(info["shape"]).astype(np.int64))
        else:
            arr = np.frombuffer(buf, dtype={"F32": np.float32, "F16": np.float16}[info["dtype"]])
            out[name] = torch.from_numpy(arr.reshape(info["shape"]).copy()).to(F)
    return out


def read_model(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# --------------------------------------------------------------------------
# Small functions
# --------------------------------------------------------------------------

def rms_norm(x, gain, eps):
    """x / sqrt(mean(x^2) + eps) * gain over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(h, taps_w):
    """h [T, C], taps_w [C, n]: out_t = sum_j taps_w[:, j] * h_(t - n + 1 + j), zeros before position 0."""
    T, n = h.shape[0], taps_w.shape[1]
    padded = torch.cat([torch.zeros((n - 1, h.shape[1]), dtype=h.dtype), h], dim=0)
    out = torch.zeros_like(h)
    for j in range(n):
        out = out + padded[j : j + T] * taps_w[:, j]
    return out


# --------------------------------------------------------------------------
# Rotation
# --------------------------------------------------------------------------

def plain_frequencies(dims, base):
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def wavelength_scaled_frequencies(dims, base, sc):
    """Short waves keep their frequency, long waves are slowed by ``factor``, and in between the two are blended
    by where original / wavelength lies between ``low`` and ``high``."""
    out = []
    for f in plain_frequencies(dims, base):
        wave = 2.0 * math.pi / f
        if wave < sc["original"] / sc["high"]:
            out.append(f)
        elif wave > sc["original"] / sc["low"]:
            out.append(f / sc["factor"])
        else:
            s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
            out.append((1.0 - s) * f / sc["factor"] + s * f)
    return out, 1.0


def ramp_scaled_frequencies(dims, base, sc):
    """A ramp over the pair index between the pair that turns ``fast`` times within ``original`` positions and the
    one that turns ``slow`` times; ramped pairs are slowed by ``factor``; cos and sin grow with ln(factor)."""
    turn = lambda t: dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turn(sc["fast"])), 0)
    hi = min(math.ceil(turn(sc["slow"])), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(dims, base)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / sc["factor"] * ramp + f * (1.0 - ramp))
    return out, YARN_AMPLITUDE_SLOPE * math.log(sc["factor"]) + 1.0


def rotation_of(rot, kind):
    """(frequencies per pair, amplitude) of a mixer's ``rot`` entry; ``kind`` picks the scaling rule's form."""
    dims, base, sc = rot["dims"], float(rot["base"]), rot.get("scaling")
    if not sc:
        return plain_frequencies(dims, base), 1.0
    return (wavelength_scaled_frequencies if kind == "wavelength" else ramp_scaled_frequencies)(dims, base, sc)


def rotate_neighbours(x, freqs, amplitude, first_position=0):
    """x [T, ..., n >= 2 * len(freqs)]: dims (2i, 2i+1) of every vector turn by position * freqs[i]; the rest pass."""
    T, n = x.shape[0], 2 * len(freqs)
    pos = torch.arange(first_position, first_position + T, dtype=F)
    angle = pos[:, None] * torch.tensor(freqs, dtype=F)[None, :]            # [T, n/2]
    shape = (T,) + (1,) * (x.dim() - 2) + (n // 2,)
    c, s = (torch.cos(angle) * amplitude).reshape(shape), (torch.sin(angle) * amplitude).reshape(shape)
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out = x.clone()
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


# --------------------------------------------------------------------------
# Masks and softmax attention
# --------------------------------------------------------------------------

def window_visible(i, j, size):
    return 0 <= i - j < size


def pooled_block_visible(i, b, size, pool):
    """Block b = positions b*pool .. b*pool + pool - 1 is seen from i once all of it lies before the window."""
    return b * pool + pool - 1 <= i - size


def attend_window_pooled(q, k, v, scale, size, pool=0):
    """q [T, D], k [T, D], v [T, Dv] of one head.  Query i sees the keys of its window and, with ``pool`` > 0, one
    mean key and mean value per block of ``pool`` positions that lies wholly before the window; one softmax."""
    T = q.shape[0]
    out = torch.zeros((T, v.shape[1]), dtype=F)
    n_blocks = T // pool if pool else 0
    if n_blocks:
        kb = k[: n_blocks * pool].reshape(n_blocks, pool, -1).mean(1)
        vb = v[: n_blocks * pool].reshape(n_blocks, pool, -1).mean(1)
    for i in range(T):
        js = [j for j in range(T) if window_visible(i, j, size)]
        keys, vals = [k[js]], [v[js]]
        bs = [b for b in range(n_blocks) if pooled_block_visible(i, b, size, pool)]
        if bs:
            keys.append(kb[bs]), vals.append(vb[bs])
        keys, vals = torch.cat(keys), torch.cat(vals)
        wgt = torch.softmax((keys @ q[i]) * scale, dim=0)
        out[i] = wgt @ vals
    return out


# --------------------------------------------------------------------------
# Mixers
# --------------------------------------------------------------------------

def round_like_cache(t, cache_dtype):
    """Keys and values as a cache of ``cache_dtype`` holds them (None: as computed)."""
    return t if cache_dtype is None else t.to(cache_dtype).to(F)


def attention_mixer(h, w, p, m, cache_dtype=None):
    """Grouped-query attention with a rotation of neighbouring pairs and a window with pooled blocks."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "mix.q"].T).reshape(T, H, D)
    k = (h @ w[p + "mix.k"].T).reshape(T, G, D)
    v = (h @ w[p + "mix.v"].T).reshape(T, G, Dv)
    rot = m.get("rot")
    if rot and rot["dims"]:
        freqs, amp = rotation_of(rot, "wavelength")
        q, k = rotate_neighbours(q, freqs, amp), rotate_neighbours(k, freqs, amp)
    k, v = round_like_cache(k, cache_dtype), round_like_cache(v, cache_dtype)
    mask = m["mask"]
    out = torch.zeros((T, H, Dv), dtype=F)
    for hq in range(H):
        g = hq // (H // G)
        out[:, hq] = attend_window_pooled(q[:, hq], k[:, g], v[:, g], m["scale"], mask["size"], mask.get("pool", 0))
    return out.reshape(T, H * Dv) @ w[p + "mix.o"].T


def latent_attention_mixer(h, w, p, m, eps, cache_dtype=None):
    """Queries and keys/values through low-rank latents; every head's key is an unrotated part made from the latent
    beside one rotated part that all heads share; a window; a gate per head on the output."""
    T = h.shape[0]
    H, D, R, Dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w[p + "mix.dq"].T, w[p + "mix.dq.norm"], eps)
    q = (cq @ w[p + "mix.uq"].T).reshape(T, H, D + R)
    down = h @ w[p + "mix.dkv"].T
    c = rms_norm(down[:, :rank], w[p + "mix.dkv.norm"], eps)
    k_rot = down[:, rank:]                                           # [T, R], one for all heads
    freqs, amp = rotation_of(m["rot"], "ramp")
    q = torch.cat([q[..., :D], rotate_neighbours(q[..., D:], freqs, amp)], dim=-1)
    k_rot = rotate_neighbours(k_rot, freqs, amp)
    k_plain = (c @ w[p + "mix.uk"].T).reshape(T, H, D)
    v = (c @ w[p + "mix.uv"].T).reshape(T, H, Dv)
    gate = torch.sigmoid(h @ w[p + "mix.g"].T)                        # [T, H]
    out = torch.zeros((T, H, Dv), dtype=F)
    for hq in range(H):
        keys = round_like_cache(torch.cat([k_plain[:, hq], k_rot], dim=-1), cache_dtype)
        out[:, hq] = attend_window_pooled(q[:, hq], keys, round_like_cache(v[:, hq], cache_dtype), m["scale"],
                                          m["mask"]["size"]) * gate[:, hq : hq + 1]
    return out.reshape(T, H * Dv) @ w[p + "mix.o"].T


# --------------------------------------------------------------------------
# Feed-forward
# --------------------------------------------------------------------------

def table_experts(h, tokens, w, p, mlp):
    """Every token id has its experts in a table; each chosen expert counts 1 / top."""
    top = mlp["router"]["top"]
    table = w[p + "mlp.table"]
    out = torch.zeros((h.shape[0], w[p + "mlp.e0.down"].shape[0]), dtype=F)
    for t, tok in enumerate(tokens):
        for e in table[tok].tolist():
            e = int(e)
            a = silu(w[f"{p}mlp.e{e}.gate"] @ h[t]) * (w[f"{p}mlp.e{e}.up"] @ h[t])
            out[t] += (w[f"{p}mlp.e{e}.down"] @ a) / top
    return out


# --------------------------------------------------------------------------
# The model
# --------------------------------------------------------------------------

def sublayer_gate(h, w, name):
    return torch.sigmoid(h @ w[name].T + w[name + ".b"])


def forward(cfg, w, tokens, cache_dtype=None, streams=None):
    """Logits [T, vocab] of one sequence; ``streams``, a list, receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        u = h + causal_conv(h, w[p + "canon1"])
        if layer["type"] == "attention":
            y = attention_mixer(u, w, p, layer["mixer"], cache_dtype)
        elif layer["type"] == "latent_attention":
            y = latent_attention_mixer(u, w, p, layer["mixer"], eps, cache_dtype)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y * sublayer_gate(h, w, p + "rg1"), w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            y = table_experts(h, tokens, w, p, layer["mlp"])
            x = x + rms_norm(y * sublayer_gate(h, w, p + "rg2"), w[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
