"""Typed configuration of the Ninenex decoder and its description as a
``ModelSpec``.

config.json of this design is nested: ``vocab``, ``width``, ``norm.eps``,
``embedding.scale``, ``logit_scale`` and a list ``layers``; every layer names
its mixer (``type``: ``mlstm`` or ``parallel``) with the mixer's sizes
(``mixer``) and its feed-forward (``mlp``: ``kind`` ``dense`` or ``moe``, or
null for none).  A layer with ``weights_of: j`` has no tensors of its own: it
runs layer j's block on a cache entry of its own.  Every sublayer has a layer
norm (weight, no bias) before it and another behind it.  Tensors: ``embed``,
``l<i>.norm1`` / ``norm1b`` / ``norm2`` / ``norm2b``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``; a bias is its matrix's name + ``.b``.

Mixers.  ``mlstm``: the matrix memory of ``parts.mlstm`` (q scaled by
dim^-1/2, gates capped at ``gate_cap``, tensors q, k, v, g, o, norm, i, i.b,
f, f.b).  ``parallel``: under ``left`` a grouped-query softmax attention with
biases on all four projections, a rotation of the first ``rot.dims``
dimensions of q and k, the score scale ``scale`` and a chunked mask of
``mask.size`` positions; under ``right`` a retention layer (fixed decay per
head, k scaled by dim^-1/2, per-head unit norm, SiLU gate, no biases); the
result is left_scale * left + right_scale * right.

Feed-forwards.  ``dense``: down(gelu_tanh(gate x) * (up x)) with biases.
``moe``: ``router.experts`` experts e0.. (SiLU, no biases) of which a token
uses the ``router.top`` with the largest router logits (router matrix and
bias), weighted by the softmax over those logits only, plus a shared expert
(``shared``) that every token uses.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field

from ..errors import ConfigError
from .spec import BlockSpec, LayerCall, ModelSpec, PartSpec, TensorSpec
from .tifapel import _need, _positive_int

_MIXERS = ("mlstm", "parallel")
# what the design fixes
MLSTM_DEN_EPS = 1e-6        # added to the normaliser of the matrix memory
MLSTM_M_START = 0.0         # where the running maximum starts
BIAS_INIT = (0.0, 0.02)     # random biases


def _number(v, what: str) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"{what} must be a number, got {v!r}")
    return float(v)


@dataclass
class NinenexConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_scale: float
    layers: list                       # as in config.json: dicts with type / mixer / mlp (/ weights_of)
    max_positions: int = 1 << 20       # the design has no limit of its own; the cache's size is the limit
    torch_dtype: str = "bfloat16"
    extra: dict = field(default_factory=dict)
    generation: dict = field(default_factory=dict)

    # ---- reading -----------------------------------------------------------

    @classmethod
    def from_dict(cls, d: dict) -> "NinenexConfig":
        norm = _need(d, "norm", "the top level")
        known = {"architecture", "architectures", "vocab", "width", "norm", "embedding", "logit_scale", "layers",
                 "max_positions", "torch_dtype"}
        cfg = cls(vocab=_need(d, "vocab", "the top level"), width=_need(d, "width", "the top level"),
                  eps=float(_need(norm, "eps", "norm")),
                  embedding_scale=_number(_need(_need(d, "embedding", "the top level"), "scale", "embedding"),
                                          "embedding.scale"),
                  logit_scale=_number(_need(d, "logit_scale", "the top level"), "logit_scale"),
                  layers=copy.deepcopy(_need(d, "layers", "the top level")),
                  max_positions=int(d.get("max_positions") or (1 << 20)),
                  torch_dtype=d.get("torch_dtype") or "bfloat16",
                  extra={k: v for k, v in d.items() if k not in known})
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = dict(self.extra)
        d.update(architecture="Ninenex", vocab=self.vocab, width=self.width, norm={"eps": self.eps},
                 embedding={"scale": self.embedding_scale}, logit_scale=self.logit_scale,
                 layers=copy.deepcopy(self.layers), torch_dtype=self.torch_dtype)
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        return d

    # ---- checks ------------------------------------------------------------

    def validate(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
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
            if kind == "mlstm":
                self._check_mlstm(m, where + ".mixer")
            else:
                self._check_parallel(m, where + ".mixer")
            mlp = layer.get("mlp")
            if mlp is not None:
                self._check_mlp(mlp, where + ".mlp")
            if layer.get("weights_of") is not None:
                other = self.layers[self.source_of(i)]
                for key in ("type", "mixer", "mlp"):
                    if other.get(key) != layer.get(key):
                        raise ConfigError(f"{where}.weights_of {layer['weights_of']}: '{key}' differs from that layer's")

    def source_of(self, i: int) -> int:
        """The layer whose tensors layer i uses: itself, or where its ``weights_of`` leads (a layer that borrows may
        be named by another that borrows; the chain ends at a layer with tensors of its own)."""
        seen = {i}
        while self.layers[i].get("weights_of") is not None:
            src = self.layers[i]["weights_of"]
            if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < len(self.layers) or src in seen:
                raise ConfigError(f"layers[{i}].weights_of {src!r} must name another layer, and not in a circle")
            seen.add(src)
            i = src
        return i

    @staticmethod
    def _check_mlstm(m: dict, where: str) -> None:
        for key in ("heads", "dim", "vdim"):
            _positive_int(_need(m, key, where), f"{where}.{key}")
        if not _number(_need(m, "gate_cap", where), where + ".gate_cap") > 0:
            raise ConfigError(f"{where}.gate_cap must be positive")

    @staticmethod
    def _check_parallel(m: dict, where: str) -> None:
        left, right = _need(m, "left", where), _need(m, "right", where)
        _number(_need(m, "left_scale", where), where + ".left_scale")
        _number(_need(m, "right_scale", where), where + ".right_scale")
        lw, rw = where + ".left", where + ".right"
        for key in ("heads", "kv_heads", "dim", "vdim"):
            _positive_int(_need(left, key, lw), f"{lw}.{key}")
        if left["heads"] % left["kv_heads"]:
            raise ConfigError(f"{lw}: {left['heads']} heads are not a multiple of {left['kv_heads']} kv_heads")
        _number(_need(left, "scale", lw), lw + ".scale")
        mask = left.get("mask")
        if mask is not None:
            _positive_int(_need(mask, "size", lw + ".mask"), lw + ".mask.size")
        rot = left.get("rot")
        if rot is not None and _need(rot, "dims", lw + ".rot") != 0:
            dims = _positive_int(rot["dims"], lw + ".rot.dims")
            if dims % 2 or dims > left["dim"]:
                raise ConfigError(f"{lw}.rot.dims {dims} must be even and at most dim {left['dim']}")
            if not _number(_need(rot, "base", lw + ".rot"), lw + ".rot.base") > 0:
                raise ConfigError(f"{lw}.rot.base must be positive")
        for key in ("heads", "dim", "vdim"):
            _positive_int(_need(right, key, rw), f"{rw}.{key}")
        decay = _need(right, "decay", rw)
        if not isinstance(decay, list) or len(decay) != right["heads"]:
            raise ConfigError(f"{rw}.decay must list one decay per head ({right['heads']})")
        if any(isinstance(g, bool) or not isinstance(g, (int, float)) or not 0.0 <= g <= 1.0 for g in decay):
            raise ConfigError(f"{rw}.decay: every decay lies in [0, 1]")

    @staticmethod
    def _check_mlp(mlp: dict, where: str) -> None:
        kind = _need(mlp, "kind", where)
        if kind == "dense":
            _positive_int(_need(mlp, "ff", where), where + ".ff")
            return
        if kind != "moe":
            raise ConfigError(f"{where}.kind {kind!r}: 'dense' or 'moe' (or null for no feed-forward)")
        _positive_int(_need(_need(mlp, "expert", where), "ff", where + ".expert"), where + ".expert.ff")
        r = _need(mlp, "router", where)
        E = _positive_int(_need(r, "experts", where + ".router"), where + ".router.experts")
        top = _positive_int(_need(r, "top", where + ".router"), where + ".router.top")
        if top > E:
            raise ConfigError(f"{where}.router.top {top} exceeds the {E} experts")
        shared = mlp.get("shared")
        if shared is not None:
            _positive_int(_need(shared, "ff", where + ".shared"), where + ".shared.ff")

    # ---- derived ----------------------------------------------------------------

    def n_params(self) -> int:
        return sum(math.prod(t.shape) for t in self.to_spec().tensors())

    def summary(self) -> str:
        kinds = [layer["type"][0] + ("'" if layer.get("weights_of") is not None else "") for layer in self.layers]
        return (f"ninenex: {len(self.layers)} layers ({''.join(kinds)}), width {self.width}, vocab {self.vocab}, "
                f"eps {self.eps:g}, {self.n_params() / 1e6:.1f} M params, {self.torch_dtype}")

    # ---- description as parts ------------------------------------------------

    def _mixer(self, p: str, kind: str, m: dict):
        """(mixer, position) of one layer whose tensors start with ``p``."""
        d, eps = self.width, self.eps
        if kind == "mlstm":
            H, D, Dv = m["heads"], m["dim"], m["vdim"]
            tensors = dict(q=TensorSpec(p + "mix.q", (H * D, d)), k=TensorSpec(p + "mix.k", (H * D, d)),
                           v=TensorSpec(p + "mix.v", (H * Dv, d)), g=TensorSpec(p + "mix.g", (H * Dv, d)),
                           o=TensorSpec(p + "mix.o", (d, H * Dv)), norm=TensorSpec(p + "mix.norm", (H * Dv,), "vector"),
                           i=TensorSpec(p + "mix.i", (H, d)), i_bias=TensorSpec(p + "mix.i.b", (H,), "vector", (0.0, 1.0)),
                           f=TensorSpec(p + "mix.f", (H, d)), f_bias=TensorSpec(p + "mix.f.b", (H,), "vector", (3.0, 1.0)))
            return PartSpec("mlstm", dict(hidden_size=d, n_heads=H, head_dim=D, v_head_dim=Dv, eps=eps,
                                          gate_cap=float(m["gate_cap"]), q_scale=float(D) ** -0.5,
                                          den_eps=MLSTM_DEN_EPS, m_start=MLSTM_M_START), tensors), None
        left, right = m["left"], m["right"]
        H, G, D, Dv = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
        lp = p + "mix.left."
        bias = lambda name, n: TensorSpec(name, (n,), "vector", BIAS_INIT)
        lt = dict(q=TensorSpec(lp + "q", (H * D, d)), k=TensorSpec(lp + "k", (G * D, d)),
                  v=TensorSpec(lp + "v", (G * Dv, d)), o=TensorSpec(lp + "o", (d, H * Dv)),
                  q_bias=bias(lp + "q.b", H * D), k_bias=bias(lp + "k.b", G * D), v_bias=bias(lp + "v.b", G * Dv),
                  o_bias=bias(lp + "o.b", d))
        mask, rot = left.get("mask"), left.get("rot")
        attention = PartSpec("gqa_attention", dict(
            hidden_size=d, n_heads=H, n_kv_heads=G, head_dim=D, v_head_dim=Dv, scale=float(left["scale"]),
            window=None, chunk=mask["size"] if mask else 0, qk_norm_eps=None, own_kv=True), lt)
        position = None
        if rot and rot["dims"]:
            position = PartSpec("rope_neox", dict(n_rot=rot["dims"], base=float(rot["base"]), angles="float32"))
        Hr, Dr, Dvr = right["heads"], right["dim"], right["vdim"]
        rp = p + "mix.right."
        rt_ = dict(q=TensorSpec(rp + "q", (Hr * Dr, d)), k=TensorSpec(rp + "k", (Hr * Dr, d)),
                   v=TensorSpec(rp + "v", (Hr * Dvr, d)), g=TensorSpec(rp + "g", (Hr * Dvr, d)),
                   o=TensorSpec(rp + "o", (d, Hr * Dvr)))
        retention = PartSpec("decay_linear_attention", dict(
            hidden_size=d, n_heads=Hr, head_dim=Dr, v_head_dim=Dvr, decay=tuple(float(g) for g in right["decay"]),
            eps=eps, qkv_activation="none", k_scale=float(Dr) ** -0.5, out_norm="per_head", gate="silu"), rt_)
        tensors = {f"left.{k}": v for k, v in lt.items()}
        tensors.update({f"right.{k}": v for k, v in rt_.items()})
        return PartSpec("side_by_side", dict(left=attention, right=retention, left_scale=float(m["left_scale"]),
                                             right_scale=float(m["right_scale"]), position_to="left"), tensors), position

    def _feed_forward(self, p: str, mlp):
        d = self.width
        if mlp is None:
            return PartSpec("none", {}, {})
        bias = lambda name, n: TensorSpec(name, (n,), "vector", BIAS_INIT)
        if mlp["kind"] == "dense":
            F = mlp["ff"]
            return PartSpec("gated_mlp", dict(hidden_size=d, intermediate_size=F, activation="gelu_tanh"), dict(
                gate=TensorSpec(p + "mlp.gate", (F, d)), up=TensorSpec(p + "mlp.up", (F, d)),
                down=TensorSpec(p + "mlp.down", (d, F)), gate_bias=bias(p + "mlp.gate.b", F),
                up_bias=bias(p + "mlp.up.b", F), down_bias=bias(p + "mlp.down.b", d)))
        r, F = mlp["router"], mlp["expert"]["ff"]
        E = r["experts"]
        tensors = {"router": TensorSpec(p + "mlp.router", (E, d)),
                   "router_bias": TensorSpec(p + "mlp.router.b", (E,), "vector", BIAS_INIT)}
        for e in range(E):
            tensors[f"gate{e}"] = TensorSpec(f"{p}mlp.e{e}.gate", (F, d))
            tensors[f"up{e}"] = TensorSpec(f"{p}mlp.e{e}.up", (F, d))
            tensors[f"down{e}"] = TensorSpec(f"{p}mlp.e{e}.down", (d, F))
        params = dict(hidden_size=d, intermediate_size=F, n_experts=E, top=r["top"], score="softmax_top",
                      n_groups=1, keep_groups=1, normalize=False, scale=1.0, activation="silu")
        shared = mlp.get("shared")
        if shared is not None:
            Fs = shared["ff"]
            params["shared_size"] = Fs
            tensors.update(shared_gate=TensorSpec(p + "mlp.shared.gate", (Fs, d)),
                           shared_up=TensorSpec(p + "mlp.shared.up", (Fs, d)),
                           shared_down=TensorSpec(p + "mlp.shared.down", (d, Fs)))
        return PartSpec("routed_experts", params, tensors)

    def to_spec(self) -> ModelSpec:
        d, eps = self.width, self.eps
        norm = lambda name: PartSpec("layer_norm", dict(size=d, eps=eps), dict(gain=TensorSpec(name, (d,), "vector")))
        blocks, schedule, block_of = [], [], {}
        for i, layer in enumerate(self.layers):
            if layer.get("weights_of") is not None:
                continue
            p = f"l{i}."
            mixer, position = self._mixer(p, layer["type"], layer["mixer"])
            mlp = layer.get("mlp")
            norms = dict(mixer=norm(p + "norm1"), mixer_post=norm(p + "norm1b"))
            if mlp is not None:
                norms.update(feed_forward=norm(p + "norm2"), feed_forward_post=norm(p + "norm2b"))
            block_of[i] = len(blocks)
            blocks.append(BlockSpec("sandwich", mixer, self._feed_forward(p, mlp), norms, position))
        # a layer that borrows another's weights runs that layer's block on a cache entry of its own
        for i in range(len(self.layers)):
            schedule.append(LayerCall(layer=block_of[self.source_of(i)], cache=i))
        return ModelSpec(
            architecture="Ninenex", hidden_size=d, vocab_size=self.vocab,
            embedding=PartSpec("gather", dict(scale=self.embedding_scale), dict(table=TensorSpec("embed", (self.vocab, d)))),
            blocks=tuple(blocks), schedule=tuple(schedule), final_norm=norm("final.norm"),
            head=PartSpec("linear", dict(softcap=None, scale=self.logit_scale),
                          dict(weight=TensorSpec("head", (self.vocab, d)))),
            max_positions=self.max_positions, stop_ids=(), storage_dtype=self.torch_dtype, default_sampling={},
        )
