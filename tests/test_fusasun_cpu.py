"""CPU: the Fusasun configuration and its description as parts, the cache's store of one row per block, and the
plain implementation's own mechanisms against closed forms."""

import copy
import math

import pytest
import torch

import plain_fusasun as plain
from fusasun_configs import ALL, FS_A, FS_B, FS_D, make_folder

from llmoxide_b200.cache.allocator import PAGE, CacheAllocator
from llmoxide_b200.config import FusasunConfig, read_config
from llmoxide_b200.errors import CacheExhausted, ConfigError

F = torch.float64


def test_config_is_chosen_by_name_and_round_trips():
    for raw in ALL.values():
        cfg = read_config(copy.deepcopy(raw))
        assert isinstance(cfg, FusasunConfig)
        again = read_config(cfg.to_dict())
        assert again.to_dict() == cfg.to_dict()
        assert "fusasun" in cfg.summary()


def test_description_names_every_tensor_once_with_the_shapes_of_the_configuration():
    spec = read_config(copy.deepcopy(FS_A)).to_spec()
    names = [t.name for t in spec.tensors()]
    assert len(names) == len(set(names))
    shapes = {t.name: tuple(t.shape) for t in spec.tensors()}
    assert shapes["embed"] == (211, 96) and shapes["head"] == (211, 96) and shapes["final.norm"] == (96,)
    assert shapes["l0.mix.q"] == (4 * 32, 96) and shapes["l0.mix.k"] == (2 * 32, 96) and shapes["l0.mix.v"] == (2 * 16, 96)
    assert shapes["l0.mix.o"] == (96, 4 * 16) and "l0.mix.q.b" not in shapes
    assert shapes["l0.canon1"] == (96, 3) and shapes["l0.rg1"] == (96, 96) and shapes["l0.rg1.b"] == (96,)
    assert shapes["l0.rg2"] == (96, 96) and shapes["l0.mlp.table"] == (211, 2) and shapes["l0.mlp.e5.down"] == (96, 24)
    assert "l0.mlp.e6.gate" not in shapes and "l0.mlp.router" not in shapes
    assert shapes["l1.mix.dq"] == (40, 96) and shapes["l1.mix.dq.norm"] == (40,) and shapes["l1.mix.uq"] == (3 * 24, 40)
    assert shapes["l1.mix.dkv"] == (48 + 8, 96) and shapes["l1.mix.dkv.norm"] == (48,) and shapes["l1.mix.uk"] == (3 * 16, 48)
    assert shapes["l1.mix.uv"] == (3 * 24, 48) and shapes["l1.mix.g"] == (3, 96) and shapes["l1.mix.o"] == (96, 72)
    # a layer without a feed-forward has neither its norms nor its gate
    assert "l2.norm1b" in shapes and "l2.rg1" in shapes and "l2.canon1" in shapes
    assert not any(n in shapes for n in ("l2.norm2", "l2.norm2b", "l2.rg2", "l2.rg2.b", "l2.mlp.table"))
    assert [(c.layer, c.cache) for c in spec.schedule] == [(0, 0), (1, 1), (2, 2), (3, 3)]
    b0, b1 = spec.blocks[0], spec.blocks[1]
    assert b0.arrangement == "sandwich" and b0.params["mixer_conv_taps"] == 3 and b0.params["result_gate"] == "sigmoid"
    assert all(n.kind == "rms_norm" for n in b0.norms.values())
    m = b0.mixer
    assert m.kind == "gqa_attention" and (m["window"], m["pool"], m["scale"], m["v_head_dim"]) == (20, 4, 0.2, 16)
    assert b0.position["pairing"] == "neighbours" and b0.position["scaling"]["rule"] == "wavelength"
    assert b0.position["n_rot"] == 16 and b0.position["angles"] == "float32"
    assert b1.mixer.kind == "latent_attention" and (b1.mixer["rot_dim"], b1.mixer["kv_rank"], b1.mixer["window"]) == (8, 48, 33)
    assert b1.position["scaling"]["rule"] == "ramp" and b1.position["scaling"]["amplitude_slope"] == 0.1
    assert spec.blocks[2].position["scaling"] is None and spec.blocks[3].position["scaling"] is None
    ff = b0.feed_forward
    assert ff.kind == "routed_experts" and ff["score"] == "table" and ff["table_weight"] == 0.5 and ff["top"] == 2
    assert spec.blocks[2].feed_forward.kind == "none"
    assert spec.embedding["scale"] == 3.0


@pytest.mark.parametrize("path, value, text", [
    (("layers", 0, "type"), "mamba", "this design has"),
    (("layers", 0, "mixer", "kv_heads"), 3, "not a multiple"),
    (("layers", 0, "mixer", "mask"), None, "lacks 'mask'"),
    (("layers", 0, "mixer", "mask", "pool"), 0, "positive integer"),
    (("layers", 0, "mixer", "rot", "dims"), 15, "even"),
    (("layers", 0, "mixer", "rot", "dims"), 34, "at most"),
    (("layers", 0, "mixer", "rot", "scaling", "high"), 1.0, "must differ"),
    (("layers", 1, "mixer", "rot", "dims"), 6, "must equal rot_dim"),
    (("layers", 1, "mixer", "kv_rank"), None, "lacks 'kv_rank'"),
    (("layers", 1, "mixer", "rot", "scaling", "slow"), -1.0, "positive"),
    (("layers", 0, "mlp", "router", "top"), 7, "exceeds"),
    (("layers", 0, "mlp", "kind"), "dense", "'moe'"),
    (("canon", "taps"), 0, "positive integer"),
    (("embedding",), None, "lacks 'embedding'"),
    (("norm", "eps"), 0.0, "positive"),
])
def test_inconsistent_configurations_are_refused(path, value, text):
    raw = copy.deepcopy(FS_A)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=text):
        read_config(raw)


def test_random_table_rows_hold_different_experts(tmp_path):
    folder = make_folder(tmp_path, "A", "float32")
    cfg, w = plain.read_model(folder)
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("mlp") is None:
            continue
        table, r = w[f"l{i}.mlp.table"], layer["mlp"]["router"]
        assert table.shape == (cfg["vocab"], r["top"]) and table.dtype == torch.int64
        assert int(table.min()) >= 0 and int(table.max()) < r["experts"]
        assert all(len(set(row.tolist())) == r["top"] for row in table)
        assert len(set(table[:, 0].tolist())) == r["experts"]       # every expert is somebody's first


# ---------------------------------------------------------------------------------------------------------
# the cache's store of one row per block
# ---------------------------------------------------------------------------------------------------------

def test_a_group_of_one_row_per_block_holds_pages_for_complete_blocks_only():
    block = 8
    a = CacheAllocator(3, 10, [48, None], every=[None, (block, 4)])
    s = a.acquire()
    a.reserve(s, 70)
    a.commit(s, 70)
    # 70 positions: two pages of positions (the first not yet out of the window), 8 complete blocks: one page of rows
    assert len(a.page_row(s, 0)) == 2 and a.page_row(s, 1) == [0]
    n = PAGE * block - 70 - 1
    a.reserve(s, n)
    a.commit(s, n)
    assert len(a.page_row(s, 1)) == 1 and a.length(s) == PAGE * block - 1       # 63 blocks and seven positions
    a.reserve(s, 1)
    assert len(a.page_row(s, 1)) == 1                                           # the 64th block: still the first page
    a.commit(s, 1)
    a.reserve(s, block)
    assert len(a.page_row(s, 1)) == 2                                           # the 65th block opens a second page
    a.unreserve(s)
    assert len(a.page_row(s, 1)) == 1
    # the rows stay whatever the window gives back
    assert a.page_row(s, 0).count(-1) == (a.length(s) - 47) // PAGE and -1 not in a.page_row(s, 1)
    a.check_consistent()
    a.release(s)
    assert a.pages_held(0) == 0 and a.pages_held(1) == 0
    # its pool is its own: with one page of rows a sequence of 65 blocks does not fit, and nothing is taken
    a = CacheAllocator(3, 10, [48, None], every=[None, (block, 1)])
    s = a.acquire()
    with pytest.raises(CacheExhausted):
        a.reserve(s, (PAGE + 1) * block)
    assert a.pages_held(0) == 0 and a.pages_held(1) == 0
    a.reserve(s, PAGE * block)
    a.check_consistent()


def test_cache_gives_an_entry_with_pooled_blocks_a_second_store():
    from llmoxide_b200.cache import KVNeed

    need = KVNeed(2, 32, 48, v_head_dim=16, pool=8)
    assert need.pooled() == KVNeed(2, 32, None, v_head_dim=16, every=8) and need.pooled().pool == 0


# ---------------------------------------------------------------------------------------------------------
# the plain implementation against closed forms
# ---------------------------------------------------------------------------------------------------------

def test_plain_mask_of_window_and_pooled_blocks():
    size, pool = 5, 3
    # position 9 sees 5..9; block 0 (0..2) lies wholly before; block 1 (3..5) reaches into the window
    assert [j for j in range(12) if plain.window_visible(9, j, size)] == [5, 6, 7, 8, 9]
    assert [b for b in range(4) if plain.pooled_block_visible(9, b, size, pool)] == [0]
    # position 10 sees 6..10 and blocks 0 and 1 (its last position 5 = 10 - 5)
    assert [b for b in range(4) if plain.pooled_block_visible(10, b, size, pool)] == [0, 1]
    # positions 3 and 4 are seen from 9 by nobody: out of the window, block not complete before it
    q = torch.zeros(12, 2, dtype=F)
    k = torch.zeros(12, 2, dtype=F)
    v = torch.arange(12, dtype=F).reshape(12, 1).repeat(1, 2)
    out = plain.attend_window_pooled(q, k, v, 1.0, size, pool)
    # equal scores: the mean over the window's values and the blocks' mean values
    assert torch.allclose(out[9], torch.full((2,), (5 + 6 + 7 + 8 + 9 + 1.0) / 6, dtype=F))
    assert torch.allclose(out[10], torch.full((2,), (6 + 7 + 8 + 9 + 10 + 1.0 + 4.0) / 7, dtype=F))
    assert torch.allclose(out[4], torch.full((2,), 2.0, dtype=F))
    # blocks of one position: every earlier key, each as itself
    full = plain.attend_window_pooled(q, k, v, 1.0, size, 1)
    assert torch.allclose(full[9], torch.full((2,), 4.5, dtype=F))


def test_plain_convolution_and_rotation():
    h = torch.arange(1.0, 9.0, dtype=F).reshape(4, 2)
    w = torch.tensor([[0.5, 2.0, 1.0], [0.0, 1.0, -1.0]], dtype=F)
    y = plain.causal_conv(h, w)
    assert torch.allclose(y[0], torch.tensor([1.0, -2.0], dtype=F))                       # only the last tap meets a row
    assert torch.allclose(y[2], torch.tensor([0.5 * 1 + 2 * 3 + 5, 4.0 - 6.0], dtype=F))
    # neighbours (0, 1) turn by position * f_0, (2, 3) by position * f_1; the fifth dim passes
    x = torch.tensor([[1.0, 0.0, 0.0, 2.0, 7.0]], dtype=F).repeat(3, 1)
    r = plain.rotate_neighbours(x, [0.5, 0.25], 1.5)
    assert torch.allclose(r[2, :2], 1.5 * torch.tensor([math.cos(1.0), math.sin(1.0)], dtype=F))
    assert torch.allclose(r[2, 2:4], 1.5 * 2 * torch.tensor([-math.sin(0.5), math.cos(0.5)], dtype=F))
    assert float(r[2, 4]) == 7.0


def test_plain_frequency_rules():
    # wavelength rule: with base 10000 and 16 dims the wavelengths run from 6.3 to about 20 000 positions
    sc = dict(factor=8.0, low=1.0, high=4.0, original=64)
    freqs, amp = plain.wavelength_scaled_frequencies(16, 10000.0, sc)
    base = plain.plain_frequencies(16, 10000.0)
    assert amp == 1.0 and freqs[0] == base[0]                                   # 6.3 < 64 / 4: kept
    assert freqs[-1] == base[-1] / 8.0                                          # far longer than 64: slowed
    mid = [i for i, f in enumerate(base) if 16 <= 2 * math.pi / f <= 64]
    assert mid and all(base[i] / 8.0 < freqs[i] < base[i] for i in mid[1:])
    # ramp rule: pairs below the pair that turns `fast` times keep their frequency, those above `slow` are slowed
    sc = dict(factor=4.0, original=32, fast=16.0, slow=2.0)
    freqs, amp = plain.ramp_scaled_frequencies(8, 1000.0, sc)
    base = plain.plain_frequencies(8, 1000.0)
    assert amp == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert freqs[0] == base[0] and freqs[-1] == pytest.approx(base[-1] / 4.0)


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_position_part_makes_the_plain_frequencies(name):
    """The rotation tables the kernels read against cos and sin of position times the plain rule's frequency."""
    from llmoxide_b200.parts import Runtime
    from llmoxide_b200.parts.block import build_part
    from llmoxide_b200.parts.registry import POSITIONS

    spec = read_config(copy.deepcopy(ALL[name])).to_spec()
    rt = Runtime(dtype="float32", device=torch.device("cpu"), max_positions=300)
    for block, layer in zip(spec.blocks, ALL[name]["layers"]):
        if block.position is None:
            continue
        pos = build_part(POSITIONS, "position encoding", block.position, {}, rt)
        cos, sin, n_rot = pos.rotary_tables()
        freqs, amp = plain.rotation_of(layer["mixer"]["rot"], "wavelength" if layer["type"] == "attention" else "ramp")
        assert n_rot == layer["mixer"]["rot"]["dims"] and cos.shape == (300, n_rot // 2)
        angle = torch.arange(300, dtype=F)[:, None] * torch.tensor(freqs, dtype=F)[None, :]
        assert torch.allclose(cos.double(), torch.cos(angle) * amp, atol=2e-5)
        assert torch.allclose(sin.double(), torch.sin(angle) * amp, atol=2e-5)


def test_rows_reordered_for_neighbouring_pairs():
    from llmoxide_b200.parts.position import halves_order

    class P:
        pairing, n_rot = "neighbours", 4

    w = torch.arange(12.0).reshape(12, 1)              # two heads of six dims, rotation over dims 1..4 of each
    got = halves_order(P, w, 2, 6, first=1).flatten().tolist()
    assert got == [0, 1, 3, 2, 4, 5, 6, 7, 9, 8, 10, 11]
    P.pairing = "halves"
    assert halves_order(P, w, 2, 6, first=1) is w
