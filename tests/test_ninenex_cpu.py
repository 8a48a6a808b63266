"""CPU: the Ninenex configuration and its description as parts, and the plain implementation's own mechanisms
against closed forms."""

import copy
import math

import pytest
import torch

import plain_ninenex as plain
from ninenex_configs import ALL, NX_A, NX_B, NX_D

from llmoxide_b200.config import NinenexConfig, read_config
from llmoxide_b200.errors import ConfigError

F = torch.float64


def test_config_is_chosen_by_name_and_round_trips():
    for raw in ALL.values():
        cfg = read_config(copy.deepcopy(raw))
        assert isinstance(cfg, NinenexConfig)
        again = read_config(cfg.to_dict())
        assert again.to_dict() == cfg.to_dict()
        assert "ninenex" in cfg.summary()


def test_description_names_every_tensor_once_with_the_shapes_of_the_configuration():
    spec = read_config(copy.deepcopy(NX_A)).to_spec()
    names = [t.name for t in spec.tensors()]
    assert len(names) == len(set(names))
    shapes = {t.name: tuple(t.shape) for t in spec.tensors()}
    assert shapes["embed"] == (211, 96) and shapes["head"] == (211, 96) and shapes["final.norm"] == (96,)
    # the side-by-side layer: attention with biases on the left, retention without on the right
    assert shapes["l0.mix.left.q"] == (4 * 32, 96) and shapes["l0.mix.left.q.b"] == (128,)
    assert shapes["l0.mix.left.k"] == (2 * 32, 96) and shapes["l0.mix.left.v"] == (2 * 16, 96) and shapes["l0.mix.left.v.b"] == (32,)
    assert shapes["l0.mix.left.o"] == (96, 4 * 16) and shapes["l0.mix.left.o.b"] == (96,)
    assert shapes["l0.mix.right.q"] == (2 * 16, 96) and shapes["l0.mix.right.v"] == (2 * 24, 96) and shapes["l0.mix.right.o"] == (96, 48)
    assert "l0.mix.right.q.b" not in shapes and "l0.mix.right.norm" not in shapes
    assert shapes["l0.mlp.gate"] == (40, 96) and shapes["l0.mlp.gate.b"] == (40,) and shapes["l0.mlp.down.b"] == (96,)
    for n in ("norm1", "norm1b", "norm2", "norm2b"):
        assert shapes[f"l0.{n}"] == (96,)
    # the matrix memory: keys and values of different sizes, gates with biases
    assert shapes["l1.mix.q"] == (3 * 16, 96) and shapes["l1.mix.v"] == (3 * 24, 96) and shapes["l1.mix.g"] == (72, 96)
    assert shapes["l1.mix.norm"] == (72,) and shapes["l1.mix.i"] == (3, 96) and shapes["l1.mix.f.b"] == (3,)
    assert shapes["l1.mlp.router"] == (6, 96) and shapes["l1.mlp.router.b"] == (6,) and shapes["l1.mlp.e5.down"] == (96, 24)
    assert "l1.mlp.e6.gate" not in shapes and "l1.mlp.e0.gate.b" not in shapes and shapes["l1.mlp.shared.up"] == (40, 96)
    # a layer that borrows weights has no tensors; a layer without a feed-forward has no second pair of norms
    assert not any(n.startswith("l2.") for n in shapes)
    assert "l3.norm1b" in shapes and "l3.norm2" not in shapes and "l3.norm2b" not in shapes and "l3.mlp.gate" not in shapes
    # the borrowed layer runs block 0 again on a cache entry of its own
    assert [(c.layer, c.cache) for c in spec.schedule] == [(0, 0), (1, 1), (0, 2), (2, 3)]
    assert len(spec.blocks) == 3 and all(b.arrangement == "sandwich" for b in spec.blocks)
    mixer = spec.blocks[0].mixer
    assert mixer.kind == "side_by_side" and (mixer["left_scale"], mixer["right_scale"]) == (1.25, 0.6)
    left, right = mixer["left"], mixer["right"]
    assert (left["chunk"], left["scale"], left["v_head_dim"], left["n_kv_heads"]) == (20, 0.2, 16, 2)
    assert right["decay"] == (0.8, 0.995) and right["k_scale"] == 16 ** -0.5 and right["out_norm"] == "per_head"
    assert spec.blocks[0].position["n_rot"] == 16 and spec.blocks[0].position["base"] == 10000.0
    m = spec.blocks[1].mixer
    assert m.kind == "mlstm" and m["gate_cap"] == 10.0 and m["q_scale"] == 0.25 and m["den_eps"] == 1e-6
    ff = spec.blocks[1].feed_forward
    assert (ff["n_experts"], ff["top"], ff["score"], ff["shared_size"], ff["activation"]) == (6, 2, "softmax_top", 40, "silu")
    assert spec.blocks[0].feed_forward["activation"] == "gelu_tanh" and spec.blocks[2].feed_forward.kind == "none"
    assert spec.embedding["scale"] == 1.5 and spec.head["scale"] == 0.7
    # a layer without a mask or without rotation
    spec_b = read_config(copy.deepcopy(NX_B)).to_spec()
    assert spec_b.blocks[1].mixer["left"]["chunk"] == 64 and spec_b.blocks[1].position is None
    assert spec_b.blocks[2].mixer["left"]["chunk"] == 0 and spec_b.blocks[2].position["n_rot"] == 48
    assert "shared_size" not in spec_b.blocks[1].feed_forward.params


@pytest.mark.parametrize("change, word", [
    (lambda c: c["layers"][0].__setitem__("type", "retention"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 34), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("decay", [0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("decay", [0.5, 1.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("gate_cap", 0.0), "gate_cap"),
    (lambda c: c["layers"][1]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 7), "top"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "conv"), "kind"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 2), "weights_of"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 1), "differs"),
    (lambda c: (c["layers"][0].update(weights_of=2), c["layers"][2].update(weights_of=0)), "circle"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("left_scale", 1.0), "differs"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.pop("logit_scale"), "logit_scale"),
    (lambda c: c["embedding"].pop("scale"), "scale"),
])
def test_inconsistent_configurations_are_refused(change, word):
    raw = copy.deepcopy(NX_A)
    change(raw)
    with pytest.raises(ConfigError) as e:
        read_config(raw)
    assert word in str(e.value)


def test_borrowed_weights_through_a_chain_and_from_a_later_layer():
    """A layer may borrow from one that borrows, and from a layer further on: each runs the block of the layer the
    chain ends at, on a cache entry of its own.  A rotation of zero dimensions is no rotation."""
    raw = copy.deepcopy(NX_A)
    raw["layers"][3] = dict(copy.deepcopy(raw["layers"][2]), weights_of=2)      # 3 -> 2 -> 0
    spec = read_config(raw).to_spec()
    assert [c.layer for c in spec.schedule] == [0, 1, 0, 0] and [c.cache for c in spec.schedule] == [0, 1, 2, 3]
    raw = copy.deepcopy(NX_A)
    raw["layers"][0]["weights_of"] = 2                                            # the first layer borrows the third's
    raw["layers"][2].pop("weights_of")
    spec = read_config(raw).to_spec()
    assert [c.layer for c in spec.schedule] == [1, 0, 1, 2]
    assert {t.name.split(".")[0] for t in spec.tensors()} >= {"l1", "l2", "l3"}
    assert not any(t.name.startswith("l0.") for t in spec.tensors())
    raw = copy.deepcopy(NX_A)
    for i in (0, 2):
        raw["layers"][i]["mixer"]["left"]["rot"]["dims"] = 0
    assert read_config(raw).to_spec().blocks[0].position is None


# ---------------------------------------------------------------------------------------------------------
# the plain implementation against closed forms
# ---------------------------------------------------------------------------------------------------------

def test_layer_norm_centres_and_scales_and_unit_rms_does_not_centre():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=F)
    gain = torch.tensor([1.0, 2.0, 0.5, -1.0], dtype=F)
    dev = x - 3.0
    want = dev / math.sqrt(float((dev * dev).mean()) + 0.1) * gain           # variance 3.5: mean of squared deviations
    assert torch.allclose(plain.layer_norm(x, gain, 0.1), want, atol=1e-14)
    assert torch.allclose(plain.unit_rms(x, 0.1), x / math.sqrt(12.5 + 0.1), atol=1e-14)
    # a constant row: the deviations vanish, eps keeps the quotient finite
    assert torch.equal(plain.layer_norm(torch.full((1, 4), 7.0, dtype=F), gain, 1e-5), torch.zeros(1, 4, dtype=F))


def test_tanh_gelu_and_log_sigmoid():
    z = torch.tensor([-3.0, -0.5, 0.0, 0.7, 4.0], dtype=F)
    want = [0.5 * v * (1 + math.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3))) for v in z.tolist()]
    assert torch.allclose(plain.gelu_tanh(z), torch.tensor(want, dtype=F), atol=1e-15)
    assert abs(float(plain.gelu_tanh(torch.tensor(1.0, dtype=F))) - 0.8411919906082768) < 1e-12
    assert torch.allclose(plain.log_sigmoid(z), torch.log(1 / (1 + torch.exp(-z))), atol=1e-14)
    assert float(plain.log_sigmoid(torch.tensor(-800.0, dtype=F))) == -800.0       # no overflow far out


def test_rotation_pairs_dimension_i_with_i_plus_half_and_leaves_the_rest():
    T, H, D, dims, base = 5, 2, 10, 6, 100.0
    x = torch.randn(T, H, D, dtype=F, generator=torch.Generator().manual_seed(0))
    pos = torch.tensor([0, 1, 2, 50, 1000])
    y = plain.rotate_half(x, pos, dims, base)
    assert torch.equal(y[..., dims:], x[..., dims:]) and torch.allclose(y[0], x[0], atol=1e-15)
    for t, p in enumerate(pos.tolist()):
        for i in range(dims // 2):
            a = p * base ** (-2.0 * i / dims)
            u, v = x[t, :, i], x[t, :, i + dims // 2]
            assert torch.allclose(y[t, :, i], u * math.cos(a) - v * math.sin(a), atol=1e-12)
            assert torch.allclose(y[t, :, i + dims // 2], v * math.cos(a) + u * math.sin(a), atol=1e-12)
    # scores depend on the distance only
    q, k = x[:1].expand(T, H, D), x[1:2].expand(T, H, D)
    s1 = (plain.rotate_half(q, pos, dims, base)[3] * plain.rotate_half(k, pos, dims, base)[2]).sum(-1)
    s2 = (plain.rotate_half(q, pos + 17, dims, base)[3] * plain.rotate_half(k, pos + 17, dims, base)[2]).sum(-1)
    assert torch.allclose(s1, s2, atol=1e-10)


def test_chunk_mask_counts_chunks_from_position_zero():
    m = plain.chunk_mask(10, 4)
    for i in range(10):
        for j in range(10):
            assert bool(m[i, j]) == (j <= i and i // 4 == j // 4)
    assert m[3, 0] and not m[4, 3] and m[4, 4] and m[7, 4] and not m[8, 7]
    assert torch.equal(plain.chunk_mask(6, 6), torch.tril(torch.ones(6, 6, dtype=torch.bool)))
    assert torch.equal(plain.chunk_mask(5, 1), torch.eye(5, dtype=torch.bool))


def test_softmax_attention_uses_the_group_of_the_head_and_only_visible_keys():
    g = torch.Generator().manual_seed(1)
    T, H, G, D, Dv = 9, 4, 2, 6, 3
    q, k, v = torch.randn(T, H, D, dtype=F, generator=g), torch.randn(T, G, D, dtype=F, generator=g), torch.randn(T, G, Dv, dtype=F, generator=g)
    vis = plain.chunk_mask(T, 4)
    out = plain.softmax_attention(q, k, v, 0.3, vis)
    for i, hq in ((0, 0), (4, 3), (7, 1), (8, 2)):
        js = [j for j in range(T) if vis[i, j]]
        grp = hq // 2
        wts = torch.softmax(torch.stack([(q[i, hq] * k[j, grp]).sum() * 0.3 for j in js]), 0)
        assert torch.allclose(out[i, hq], sum(wt * v[j, grp] for wt, j in zip(wts, js)), atol=1e-12)
    assert torch.allclose(out[4], v[4].repeat_interleave(2, 0), atol=1e-14)        # first of a chunk: itself alone


def test_decay_recurrence_is_the_weighted_sum_over_the_past():
    g = torch.Generator().manual_seed(2)
    T, H, D, Dv, decay = 12, 2, 3, 4, [0.5, 1.0]
    q, k, v = torch.randn(T, H, D, dtype=F, generator=g), torch.randn(T, H, D, dtype=F, generator=g), torch.randn(T, H, Dv, dtype=F, generator=g)
    out = plain.decay_recurrence(q, k, v, decay)
    for h in range(H):
        for t in (0, 5, 11):
            want = sum(decay[h] ** (t - j) * (q[t, h] * k[j, h]).sum() * v[j, h] for j in range(t + 1))
            assert torch.allclose(out[t, h], want, atol=1e-12)


def test_matrix_memory_equals_its_unstabilised_form_and_starts_its_maximum_at_zero():
    """Without the running maximum: C_t = sigma(f~) C_(t-1) + exp(i) k v^T, o = C^T q / max(|n . q|, 1); the
    maximum only rescales numerator, normaliser and the 1 alike (the 1 becomes exp(-m)).  With m_0 = 0 and small
    gates the maximum stays 0 for a while, and then the two forms are the same numbers."""
    g = torch.Generator().manual_seed(3)
    T, H, D, Dv = 20, 2, 4, 3
    q, k, v = torch.randn(T, H, D, dtype=F, generator=g), torch.randn(T, H, D, dtype=F, generator=g), torch.randn(T, H, Dv, dtype=F, generator=g)
    i_log = torch.randn(T, H, dtype=F, generator=g) * 2
    f_log = plain.log_sigmoid(torch.randn(T, H, dtype=F, generator=g) * 3)
    out = plain.mlstm_recurrence(q, k, v, i_log, f_log)
    C, n = torch.zeros(H, D, Dv, dtype=F), torch.zeros(H, D, dtype=F)
    for t in range(T):
        C = torch.exp(f_log[t])[:, None, None] * C + torch.exp(i_log[t])[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = torch.exp(f_log[t])[:, None] * n + torch.exp(i_log[t])[:, None] * k[t]
        m = torch.zeros(H, dtype=F)
        for s in range(t + 1):
            m = torch.maximum(f_log[s] + m, i_log[s])
        num = torch.einsum("hdv,hd->hv", C, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.ones(H, dtype=F)) + 1e-6 * torch.exp(m)
        assert torch.allclose(out[t], num / den[:, None], atol=1e-11), t
    # all input gates far below zero: m stays at 0 (it does not start at minus infinity), so the first token's
    # output is exp(i) (k . q) v / (1 + 1e-6) and not v times the sign of k . q
    small = torch.full((T, H), -5.0, dtype=F)
    o = plain.mlstm_recurrence(q, k, v, small, f_log)
    want = math.exp(-5.0) * (q[0] * k[0]).sum(-1, keepdim=True) * v[0] / (1.0 + 1e-6)
    assert torch.allclose(o[0], want, atol=1e-14)


def test_gate_cap_bounds_both_gates():
    w = {"l0.mix.i": torch.tensor([[100.0]], dtype=F), "l0.mix.i.b": torch.tensor([3.0], dtype=F),
         "l0.mix.f": torch.tensor([[-100.0]], dtype=F), "l0.mix.f.b": torch.tensor([0.0], dtype=F)}
    h = torch.tensor([[1.0]], dtype=F)
    cap = 5.0
    i_log = cap * torch.tanh(plain.linear(h, w, "l0.mix.i", bias=True) / cap)
    f_log = plain.log_sigmoid(cap * torch.tanh(plain.linear(h, w, "l0.mix.f", bias=True) / cap))
    assert abs(float(i_log) - cap) < 1e-9 and abs(float(f_log) - (-cap - math.log1p(math.exp(-cap)))) < 1e-9


def test_routing_takes_the_largest_logits_and_softmaxes_them_alone():
    z = torch.tensor([[0.1, 2.0, -1.0, 1.5, 0.3], [5.0, 5.0, 1.0, 0.0, 4.0]], dtype=F)
    idx, wt = plain.route(z, 2)
    assert idx.tolist() == [[1, 3], [0, 1]]                 # ties: the lower index first
    assert torch.allclose(wt[0], torch.softmax(torch.tensor([2.0, 1.5], dtype=F), 0)) and torch.allclose(wt[1], torch.tensor([0.5, 0.5], dtype=F))
    idx, wt = plain.route(z, 5)                              # every expert chosen: the plain softmax
    assert torch.allclose(wt.gather(1, idx.argsort(1)), torch.softmax(z, -1), atol=1e-15)
    idx, wt = plain.route(z, 1)
    assert wt.tolist() == [[1.0], [1.0]]


def test_mixture_is_the_weighted_sum_of_the_chosen_experts_plus_the_shared_one():
    g = torch.Generator().manual_seed(4)
    d, Fe, E, T = 6, 5, 4, 7
    w = {"router": torch.randn(E, d, dtype=F, generator=g), "router.b": torch.randn(E, dtype=F, generator=g)}
    for name in [f"e{e}" for e in range(E)] + ["shared"]:
        w.update({f"{name}.gate": torch.randn(Fe, d, dtype=F, generator=g), f"{name}.up": torch.randn(Fe, d, dtype=F, generator=g),
                  f"{name}.down": torch.randn(d, Fe, dtype=F, generator=g)})
    h = torch.randn(T, d, dtype=F, generator=g)
    mlp = dict(router=dict(experts=E, top=2), shared=dict(ff=Fe))
    out = plain.moe_ff(h, w, "", mlp)
    for t in range(T):
        z = w["router"] @ h[t] + w["router.b"]
        best = sorted(range(E), key=lambda e: -float(z[e]))[:2]
        wt = torch.softmax(z[best], 0)
        want = sum(wt[c] * plain.expert(h[t : t + 1], w, f"e{e}.")[0] for c, e in enumerate(best))
        assert torch.allclose(out[t], want + plain.expert(h[t : t + 1], w, "shared.")[0], atol=1e-11)
    # the router's bias decides: a large bias on one expert makes every token choose it
    w["router.b"] = torch.tensor([0.0, 0.0, 50.0, 0.0], dtype=F)
    idx, _ = plain.route(plain.linear(h, w, "router", bias=True), 1)
    assert idx.flatten().tolist() == [2] * T


def test_a_layer_that_borrows_weights_has_a_state_of_its_own(tmp_path):
    """Whole model on the CPU: the layer that runs another's weights gives another result than that layer did
    (its input and its state are its own), and a model of one sequence is causal."""
    from ninenex_configs import make_folder

    folder = make_folder(tmp_path, "A", "float32")
    cfg, w = plain.read_model(folder)
    toks = [3, 50, 7, 7, 120, 9, 33, 2, 1, 0, 5, 5, 88, 100, 17, 4, 61, 62, 63, 64, 65, 66, 67]     # past one chunk of 20
    layers = []
    logits = plain.forward(cfg, w, toks, layers)
    assert logits.shape == (len(toks), 211) and len(layers) == 4 and torch.isfinite(logits).all()
    other = list(toks)
    other[-1] = 200
    assert torch.equal(plain.forward(cfg, w, other)[:-1], logits[:-1])
    # position 20 opens a chunk, but the recurrent sides still carry the past: changing token 0 moves its logits
    other = list(toks)
    other[0] = 4
    assert not torch.equal(plain.forward(cfg, w, other)[20], logits[20])


def test_sizes_that_coincide_in_one_configuration_differ_in_another():
    """The test configurations keep apart what a model may happen to make equal: key and value sizes, heads and
    key/value heads of the two sides, the widths of the dense, the expert and the shared feed-forward."""
    seen = set()
    for raw in (NX_A, NX_B, NX_D):
        for layer in raw["layers"]:
            m = layer["mixer"]
            if layer["type"] == "parallel":
                seen.add(("left d!=dv", m["left"]["dim"] != m["left"]["vdim"]))
                seen.add(("sides differ", m["left"]["heads"] != m["right"]["heads"]))
                seen.add(("kv<heads", m["left"]["kv_heads"] < m["left"]["heads"]))
                seen.add(("kv>1", m["left"]["kv_heads"] > 1))
            else:
                seen.add(("mlstm d!=dv", m["dim"] != m["vdim"]))
    for key in ("left d!=dv", "sides differ", "kv<heads", "kv>1", "mlstm d!=dv"):
        assert (key, True) in seen
