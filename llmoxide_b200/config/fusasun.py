"""Typed configuration of the Fusasun decoder and its description as a
``ModelSpec``.

config.json of this design is nested: ``vocab``, ``width``, ``norm.eps``,
``embedding.scale``, ``canon.taps`` and a list ``layers``; every layer names
its mixer (``type``: ``attention`` or ``latent_attention``) with the mixer's
sizes (``mixer``) and its feed-forward (``mlp``: ``kind`` ``moe``, or null for
none).  Tensors: ``embed``, ``l<i>.norm1`` / ``norm1b`` / ``norm2`` /
``norm2b``, ``l<i>.canon1``, ``l<i>.rg1`` (+ ``.b``), ``l<i>.rg2`` (+ ``.b``),
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.

A layer is a sandwich of RMS norms, x <- x + norm_b(gate * f(norm_a(x))) for
the mixer and then for the feed-forward, with two additions: the mixer reads
u + conv(u) where u is the normed stream and conv a causal convolution over
time on every channel (``canon1`` [width, taps]), and every sublayer's result
is multiplied by sigmoid(W u + b) (``rg1`` / ``rg2``) before the norm behind it.

Mixers.  ``attention``: grouped-query softmax attention, no biases, a rotation
of neighbouring pairs (2i, 2i+1) of the first ``rot.dims`` dimensions whose
frequencies are scaled by wavelength (``rot.scaling``: factor, low, high,
original), the score scale ``scale``, and a window of ``mask.size`` positions
beside which every block of ``mask.pool`` positions that lies wholly before
the window is seen as one mean key and mean value.  ``latent_attention``:
queries through a normed latent (dq, dq.norm, uq), keys and values through a
second normed latent (dkv, dkv.norm, uk, uv) beside one rotated key part of
``rot_dim`` dimensions that all heads share; the rotation's frequencies are
scaled by a ramp over the pairs (``rot.scaling``: factor, original, fast,
slow) with cos and sin times 0.1 ln(factor) + 1; a window of ``mask.size``
positions; a gate per head on the output (g); no biases.

Feed-forward ``moe``: ``router.experts`` experts e0.. (SiLU, no biases) of
which a token uses ``router.top``, named for its token id by the integer
``table`` [vocab, top]; each counts 1 / top.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field

from ..errors import ConfigError
from .spec import BlockSpec, LayerCall, ModelSpec, PartSpec, TensorSpec
from .tifapel import _need, _positive_int

_MIXERS = ("attention", "latent_attention")
# what the design fixes
RAMP_AMPLITUDE_SLOPE = 0.1      # cos and sin of a ramp-scaled rotation are multiplied by this * ln(factor) + 1
CONV_INIT = (0.0, 0.3)          # random convolution taps
BIAS_INIT = (0.0, 0.5)          # random gate biases


def _number(v, what: str) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"{what} must be a number, got {v!r}")
    return float(v)


@dataclass
class FusasunConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    taps: int
    layers: list                       # as in config.json: dicts with type / mixer / mlp
    max_positions: int = 1 << 20       # the design has no limit of its own; the cache's size is the limit
    torch_dtype: str = "bfloat16"
    extra: dict = field(default_factory=dict)
    generation: dict = field(default_factory=dict)

    # ---- reading -----------------------------------------------------------

    @classmethod
    def from_dict(cls, d: dict) -> "FusasunConfig":
        norm = _need(d, "norm", "the top level")
        known = {"architecture", "architectures", "vocab", "width", "norm", "embedding", "canon", "layers",
                 "max_positions", "torch_dtype"}
        cfg = cls(vocab=_need(d, "vocab", "the top level"), width=_need(d, "width", "the top level"),
                  eps=float(_need(norm, "eps", "norm")),
                  embedding_scale=_number(_need(_need(d, "embedding", "the top level"), "scale", "embedding"),
                                          "embedding.scale"),
                  taps=_need(_need(d, "canon", "the top level"), "taps", "canon"),
                  layers=copy.deepcopy(_need(d, "layers", "the top level")),
                  max_positions=int(d.get("max_positions") or (1 << 20)),
                  torch_dtype=d.get("torch_dtype") or "bfloat16",
                  extra={k: v for k, v in d.items() if k not in known})
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = dict(self.extra)
        d.update(architecture="Fusasun", vocab=self.vocab, width=self.width, norm={"eps": self.eps},
                 embedding={"scale": self.embedding_scale}, canon={"taps": self.taps},
                 layers=copy.deepcopy(self.layers), torch_dtype=self.torch_dtype)
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        return d

    # ---- checks ------------------------------------------------------------

    def validate(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.taps, "canon.taps")
        if not (self.eps > 0 and math.isfinite(self.eps)):
            raise ConfigError(f"norm.eps must be positive, got {self.eps!r}")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("'layers' must be a non-empty list")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"torch_dtype {self.torch_dtype!r}: supported are bfloat16 and float32")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}.type {kind!r}: this design has {', '.join(_MIXERS)}")
            m = _need(layer, "mixer", where)
            if kind == "attention":
                self._check_attention(m, where + ".mixer")
            else:
                self._check_latent(m, where + ".mixer")
            mlp = layer.get("mlp")
            if mlp is not None:
                self._check_mlp(mlp, where + ".mlp")

    @staticmethod
    def _check_rot(rot: dict, where: str, most: int, keys: tuple) -> None:
        dims = _positive_int(_need(rot, "dims", where), where + ".dims")
        if dims % 2 or dims > most:
            raise ConfigError(f"{where}.dims {dims} must be even and at most {most}")
        if not _number(_need(rot, "base", where), where + ".base") > 1:
            raise ConfigError(f"{where}.base must exceed one")
        sc = rot.get("scaling")
        if sc is not None:
            for key in keys:
                if not _number(_need(sc, key, where + ".scaling"), f"{where}.scaling.{key}") > 0:
                    raise ConfigError(f"{where}.scaling.{key} must be positive")

    @classmethod
    def _check_attention(cls, m: dict, where: str) -> None:
        for key in ("heads", "kv_heads", "dim", "vdim"):
            _positive_int(_need(m, key, where), f"{where}.{key}")
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")
        _number(_need(m, "scale", where), where + ".scale")
        mask = _need(m, "mask", where)
        _positive_int(_need(mask, "size", where + ".mask"), where + ".mask.size")
        if mask.get("pool") is not None:
            _positive_int(mask["pool"], where + ".mask.pool")
        rot = m.get("rot")
        if rot is not None and rot.get("dims") != 0:
            cls._check_rot(rot, where + ".rot", m["dim"], ("factor", "low", "high", "original"))
            sc = rot.get("scaling")
            if sc is not None and sc["high"] == sc["low"]:
                raise ConfigError(f"{where}.rot.scaling: 'high' and 'low' must differ")

    @classmethod
    def _check_latent(cls, m: dict, where: str) -> None:
        for key in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
            _positive_int(_need(m, key, where), f"{where}.{key}")
        _number(_need(m, "scale", where), where + ".scale")
        _positive_int(_need(_need(m, "mask", where), "size", where + ".mask"), where + ".mask.size")
        rot = _need(m, "rot", where)
        cls._check_rot(rot, where + ".rot", m["rot_dim"], ("factor", "original", "fast", "slow"))
        if rot["dims"] != m["rot_dim"]:
            raise ConfigError(f"{where}.rot.dims {rot['dims']} must equal rot_dim {m['rot_dim']}")

    def _check_mlp(self, mlp: dict, where: str) -> None:
        kind = _need(mlp, "kind", where)
        if kind != "moe":
            raise ConfigError(f"{where}.kind {kind!r}: 'moe' (or null for no feed-forward)")
        _positive_int(_need(_need(mlp, "expert", where), "ff", where + ".expert"), where + ".expert.ff")
        r = _need(mlp, "router", where)
        E = _positive_int(_need(r, "experts", where + ".router"), where + ".router.experts")
        top = _positive_int(_need(r, "top", where + ".router"), where + ".router.top")
        if top > E:
            raise ConfigError(f"{where}.router.top {top} exceeds the {E} experts")

    # ---- derived ----------------------------------------------------------------

    def n_params(self) -> int:
        return sum(math.prod(t.shape) for t in self.to_spec().tensors())

    def summary(self) -> str:
        kinds = "".join(layer["type"][0] for layer in self.layers)
        return (f"fusasun: {len(self.layers)} layers ({kinds}), width {self.width}, vocab {self.vocab}, "
                f"eps {self.eps:g}, {self.taps} taps, {self.n_params() / 1e6:.1f} M params, {self.torch_dtype}")

    # ---- description as parts ------------------------------------------------

    def _mixer(self, p: str, kind: str, m: dict):
        """(mixer, position) of one layer whose tensors start with ``p``."""
        d, eps = self.width, self.eps
        if kind == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            tensors = dict(q=TensorSpec(p + "mix.q", (H * D, d)), k=TensorSpec(p + "mix.k", (G * D, d)),
                           v=TensorSpec(p + "mix.v", (G * Dv, d)), o=TensorSpec(p + "mix.o", (d, H * Dv)))
            size, pool = m["mask"]["size"], int(m["mask"].get("pool") or 0)
            mixer = PartSpec("gqa_attention", dict(
                hidden_size=d, n_heads=H, n_kv_heads=G, head_dim=D, v_head_dim=Dv, scale=float(m["scale"]),
                window=size, pool=pool, qk_norm_eps=None, own_kv=True), tensors)
            position = None
            rot = m.get("rot")
            if rot and rot.get("dims"):
                sc = rot.get("scaling")
                position = PartSpec("rope_neox", dict(
                    n_rot=rot["dims"], base=float(rot["base"]), angles="float32", pairing="neighbours",
                    scaling=None if sc is None else dict(rule="wavelength", factor=float(sc["factor"]),
                                                         low=float(sc["low"]), high=float(sc["high"]),
                                                         original=float(sc["original"]))))
            return mixer, position
        H, D, R, Dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
        rq, rkv = m["q_rank"], m["kv_rank"]
        tensors = dict(dq=TensorSpec(p + "mix.dq", (rq, d)), dq_norm=TensorSpec(p + "mix.dq.norm", (rq,), "vector"),
                       uq=TensorSpec(p + "mix.uq", (H * (D + R), rq)), dkv=TensorSpec(p + "mix.dkv", (rkv + R, d)),
                       dkv_norm=TensorSpec(p + "mix.dkv.norm", (rkv,), "vector"),
                       uk=TensorSpec(p + "mix.uk", (H * D, rkv)), uv=TensorSpec(p + "mix.uv", (H * Dv, rkv)),
                       g=TensorSpec(p + "mix.g", (H, d)), o=TensorSpec(p + "mix.o", (d, H * Dv)))
        mixer = PartSpec("latent_attention", dict(
            hidden_size=d, n_heads=H, head_dim=D, rot_dim=R, v_head_dim=Dv, q_rank=rq, kv_rank=rkv, eps=eps,
            scale=float(m["scale"]), window=m["mask"]["size"], out_gate="sigmoid"), tensors)
        rot, sc = m["rot"], m["rot"].get("scaling")
        position = PartSpec("rope_neox", dict(
            n_rot=rot["dims"], base=float(rot["base"]), angles="float32", pairing="neighbours",
            scaling=None if sc is None else dict(rule="ramp", factor=float(sc["factor"]), original=float(sc["original"]),
                                                 fast=float(sc["fast"]), slow=float(sc["slow"]),
                                                 amplitude_slope=RAMP_AMPLITUDE_SLOPE)))
        return mixer, position

    def _feed_forward(self, p: str, mlp):
        d = self.width
        if mlp is None:
            return PartSpec("none", {}, {})
        r, F = mlp["router"], mlp["expert"]["ff"]
        E, top = r["experts"], r["top"]
        tensors = {"table": TensorSpec(p + "mlp.table", (self.vocab, top), "table", ("distinct_below", E))}
        for e in range(E):
            tensors[f"gate{e}"] = TensorSpec(f"{p}mlp.e{e}.gate", (F, d))
            tensors[f"up{e}"] = TensorSpec(f"{p}mlp.e{e}.up", (F, d))
            tensors[f"down{e}"] = TensorSpec(f"{p}mlp.e{e}.down", (d, F))
        return PartSpec("routed_experts", dict(hidden_size=d, intermediate_size=F, n_experts=E, top=top, score="table",
                                               table_weight=1.0 / top, n_groups=1, keep_groups=1, normalize=False,
                                               scale=1.0, activation="silu"), tensors)

    def to_spec(self) -> ModelSpec:
        d, eps = self.width, self.eps
        norm = lambda name: PartSpec("rms_norm", dict(size=d, eps=eps), dict(gain=TensorSpec(name, (d,), "vector")))
        blocks = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            mixer, position = self._mixer(p, layer["type"], layer["mixer"])
            mlp = layer.get("mlp")
            norms = dict(mixer=norm(p + "norm1"), mixer_post=norm(p + "norm1b"))
            own = dict(mixer_conv=TensorSpec(p + "canon1", (d, self.taps), "vector", CONV_INIT),
                       mixer_gate=TensorSpec(p + "rg1", (d, d)),
                       mixer_gate_bias=TensorSpec(p + "rg1.b", (d,), "vector", BIAS_INIT))
            if mlp is not None:
                norms.update(feed_forward=norm(p + "norm2"), feed_forward_post=norm(p + "norm2b"))
                own.update(feed_forward_gate=TensorSpec(p + "rg2", (d, d)),
                           feed_forward_gate_bias=TensorSpec(p + "rg2.b", (d,), "vector", BIAS_INIT))
            blocks.append(BlockSpec("sandwich", mixer, self._feed_forward(p, mlp), norms, position,
                                    params=dict(mixer_conv_taps=self.taps, result_gate="sigmoid"), tensors=own))
        return ModelSpec(
            architecture="Fusasun", hidden_size=d, vocab_size=self.vocab,
            embedding=PartSpec("gather", dict(scale=self.embedding_scale), dict(table=TensorSpec("embed", (self.vocab, d)))),
            blocks=tuple(blocks), schedule=tuple(LayerCall(layer=i, cache=i) for i in range(len(blocks))),
            final_norm=norm("final.norm"),
            head=PartSpec("linear", dict(softcap=None), dict(weight=TensorSpec("head", (self.vocab, d)))),
            max_positions=self.max_positions, stop_ids=(), storage_dtype=self.torch_dtype, default_sampling={},
        )
