"""GPU: the Fusasun decoder's mechanisms one by one against the plain implementation (tests/plain_fusasun.py),
then whole models under every way of cutting the same requests into steps, and greedy generation through the
package's own entry point."""

import copy
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_fusasun as plain
import replay_util as ru
from fusasun_configs import ALL, make_folder
from tiny_configs import prompts

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F32_TOL, BF16_TOL = 2e-5, 3e-2
LENGTHS = {"A": [150, 1, 37, 64, 9, 201, 2], "B": [140, 70, 3, 65, 129], "C": [300, 40, 131, 17, 64], "D": [330, 12, 101, 55]}
F = torch.float64


def _rel(got, want):
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / max(np.abs(want).max(), 1e-30))


def _f32_exact(t):
    return t.to(torch.float32).to(torch.float64)


def _i32(x):
    return torch.tensor(np.asarray(x), dtype=torch.int32, device=DEV)


def _ctx(lens_past, counts, slots=None):
    """The step's index arrays for sequences that hold ``lens_past`` positions and bring ``counts`` tokens."""
    token_seq = [b for b, n in enumerate(counts) for _ in range(n)]
    token_pos = [lens_past[b] + k for b, n in enumerate(counts) for k in range(n)]
    starts = np.concatenate([[0], np.cumsum(counts)])
    return SimpleNamespace(token_seq=_i32(token_seq), token_pos=_i32(token_pos), seq_start=_i32(starts),
                           seq_past=_i32(lens_past), seq_slot=_i32(slots if slots is not None else range(len(counts))),
                           n_seqs=len(counts), n_tokens=int(sum(counts)), is_decode=all(n == 1 for n in counts))


# ---------------------------------------------------------------------------------------------------------
# the gate on a sublayer's result, inside the norm kernel
# ---------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("d, n_split, z_split", [(40, 1, 1), (96, 3, 2), (100, 1, 1), (1000, 2, 1), (2050, 1, 3)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gated_result_normed_added_and_normed_again(d, n_split, z_split, out_dtype):
    """v = h + rms(y * sigmoid(z + b)) * gain_b, out = rms(v) * gain, with y and z in split partials; gate logits
    large enough that a gate left out, or a bias left out, shows."""
    from llmoxide_b200 import kernels

    g = torch.Generator().manual_seed(d + n_split)
    T, eps_b, eps = 29, 1e-5, 1e-3
    h = _f32_exact(torch.randn(T, d, generator=g) + 1.0)
    y = _f32_exact(torch.randn(n_split, T, d, generator=g) * 2.0)
    z = _f32_exact(torch.randn(z_split, T, d, generator=g) * 3.0)
    zb = _f32_exact(torch.randn(d, generator=g) * 2.0)
    gain_b, gain = _f32_exact(torch.randn(d, generator=g)), _f32_exact(torch.randn(d, generator=g))
    for bias in (zb, None):
        gated = y.sum(0) * torch.sigmoid(z.sum(0) + (bias if bias is not None else 0.0))
        new_h = h + plain.rms_norm(gated, gain_b, eps_b)
        want = plain.rms_norm(new_h, gain, eps)
        hd = h.float().to(DEV).contiguous()
        out = torch.empty((T, d), dtype=out_dtype, device=DEV)
        kernels.post_norm_add_norm(hd, [(y.float().to(DEV).contiguous(), 1.0)], None, gain_b.float().to(DEV), False, eps_b,
                                   gain.float().to(DEV), False, eps, out,
                                   gate=(z.float().to(DEV).contiguous(), None if bias is None else bias.float().to(DEV)))
        assert _rel(hd.cpu().numpy(), new_h.numpy()) < 3e-6
        assert _rel(out.float().cpu().numpy(), want.numpy()) < (5e-6 if out_dtype == torch.float32 else 6e-3)
    # a bfloat16 result under a float32 gate, wanted rows only
    rows = [T - 1, 0, 5]
    yb = y[0].to(torch.bfloat16)
    gated = yb.to(F) * torch.sigmoid(z.sum(0) + zb)
    want = plain.rms_norm(h + plain.rms_norm(gated, gain_b, eps_b), gain, eps)[rows]
    hd = h.float().to(DEV).contiguous()
    out = torch.empty((3, d), dtype=torch.float32, device=DEV)
    kernels.post_norm_add_norm(hd, [(yb.to(DEV).contiguous(), 1.0)], None, gain_b.float().to(DEV), False, eps_b,
                               gain.float().to(DEV), False, eps, out, rows=_i32(rows), write_h=False,
                               gate=(z.float().to(DEV).contiguous(), zb.float().to(DEV)))
    assert torch.equal(hd.cpu(), h.float()) and _rel(out.cpu().numpy(), want.numpy()) < 5e-6
    kernels.check_status()


# ---------------------------------------------------------------------------------------------------------
# the convolution in front of the mixer
# ---------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("taps, C", [(1, 40), (2, 96), (3, 100), (5, 257), (16, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_input_convolution_with_its_state_under_every_cutting(taps, C, dtype):
    """Two sequences of unequal lengths through ``residual_conv`` (+ ``conv_state_update``), cut into steps in
    five ways; every cutting gives the plain convolution's rows, bit for bit the same as the whole prompt's; the
    state of a slot that nobody uses stays as it was."""
    from llmoxide_b200 import kernels

    g = torch.Generator().manual_seed(taps * 100 + C)
    lens = [23, 9]
    xs = [(torch.randn(n, C, generator=g)).to(dtype) for n in lens]
    w = _f32_exact(torch.randn(C, taps, generator=g))
    want = [x.to(F) + plain.causal_conv(x.to(F), w) for x in xs]
    w_dev = w.float().t().contiguous().to(DEV)
    cuttings = {"whole": [[23], [9]], "one by one": [[1] * 23, [1] * 9], "twos": [[2] * 11 + [1], [2] * 4 + [1]],
                "uneven": [[5, 1, 1, 16], [1, 8]], "late": [[20, 3], [2, 2, 2, 3]]}
    results = {}
    for what, cuts in cuttings.items():
        state = torch.zeros((4, max(taps - 1, 1), C), dtype=torch.float32, device=DEV) if taps > 1 else None
        if state is not None:
            state[3] = 7.0
        fed, outs = [0, 0], [[], []]
        for j in range(max(len(c) for c in cuts)):
            live = [i for i in range(2) if j < len(cuts[i])]
            counts = [cuts[i][j] for i in live]
            x = torch.cat([xs[i][fed[i] : fed[i] + cuts[i][j]] for i in live]).to(DEV).contiguous()
            ctx = _ctx([fed[i] for i in live], counts, slots=[2 * i for i in live])
            out = torch.empty_like(x)
            inline = ctx.is_decode and taps > 1
            kernels.residual_conv(x, state, w_dev, taps, out, ctx, inline_state=inline)
            if taps > 1 and not inline:
                kernels.conv_state_update(x, state, taps, ctx)
            at = 0
            for i, n in zip(live, counts):
                outs[i].append(out[at : at + n].cpu())
                at += n
                fed[i] += n
        results[what] = [torch.cat(o) for o in outs]
        for i in range(2):
            assert _rel(results[what][i].double().numpy(), want[i].numpy()) < (3e-6 if dtype == torch.float32 else 6e-3), what
            assert torch.equal(results[what][i], results["whole"][i]), (what, i)
        if state is not None:
            assert float(state[3].min()) == 7.0 and float(state[3].max()) == 7.0 and float(state[1].abs().max()) == 0.0
            for i in range(2):      # the state is the sequence's last taps - 1 rows
                last = xs[i][-(taps - 1):].float()
                assert torch.equal(state[2 * i][-last.shape[0]:].cpu(), last)
    kernels.check_status()


# ---------------------------------------------------------------------------------------------------------
# a window with pooled blocks
# ---------------------------------------------------------------------------------------------------------

def _store(n_rows_per_seq, G, D, Dv, dtype, seed):
    """An empty paged store for sequences of that many rows, pages dealt out in any order."""
    from llmoxide_b200 import kernels

    g = torch.Generator().manual_seed(seed)
    page = kernels.PAGE
    per = [max(1, (n + page - 1) // page) for n in n_rows_per_seq]
    order = torch.randperm(sum(per) + 2, generator=g).tolist()
    table = torch.full((len(per), max(per)), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(per):
        table[b, :n] = torch.tensor(order[at : at + n], dtype=torch.int32)
        at += n
    k = torch.zeros((sum(per) + 2, G, page, D), dtype=dtype, device=DEV)
    v = torch.zeros((sum(per) + 2, G, page, Dv), dtype=dtype, device=DEV)
    return table, k, v


def _fill(table, kc, vc, b, keys, vals):
    """keys [n, G, D], vals [n, G, Dv] of sequence b into its pages."""
    page = kc.shape[2]
    for j in range(keys.shape[0]):
        p = int(table[b, j // page])
        kc[p, :, j % page] = keys[j].to(kc.dtype).to(DEV)
        vc[p, :, j % page] = vals[j].to(vc.dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D, Dv, H, G, size, pool", [(16, 48, 6, 3, 36, 6), (32, 16, 4, 2, 20, 4), (64, 64, 8, 1, 130, 16),
                                                       (96, 32, 6, 2, 5, 8), (24, 24, 2, 2, 64, 64), (40, 8, 3, 1, 7, 3),
                                                       (128, 128, 4, 4, 70, 1)])
def test_one_key_stands_out_at_every_edge_of_window_and_blocks(D, Dv, H, G, size, pool, dtype):
    """The block store is filled by ``pool_blocks`` as tokens arrive (whole, and in steps that cut blocks apart), then
    every position attends; the general kernel against the plain attention.  Then one query whose scores single out
    one key: the window's first and last key, the position just outside it (seen only if its block is complete and
    wholly outside), a block's last and first position, a far block, a page border of the block store."""
    from llmoxide_b200 import kernels

    g = torch.Generator().manual_seed(D + size + pool)
    n = max(2 * size + 3 * pool + 70, 64 * pool + size + 5 if pool <= 3 else 0, 200)
    keys = torch.randn(n, G, D, generator=g) * 0.5
    # the blocks that are to stand out hold keys that nearly agree, so that their mean is as long as a single key
    p = n - 1
    last_block = (p - size + 1) // pool - 1                   # the last block that position p sees
    for b in {0, last_block // 2, last_block, 64 if n // pool > 64 else 0}:
        common = torch.randn(G, D, generator=g) * 0.5
        keys[b * pool : (b + 1) * pool] = common + 0.05 * keys[b * pool : (b + 1) * pool]
    keys = _f32_exact(keys).to(dtype).to(F)
    vals = _f32_exact(torch.randn(n, G, Dv, generator=g)).to(dtype).to(F)
    table, kc, vc = _store([n], G, D, Dv, dtype, 3)
    ptable_host, pk, pv = _store([n // pool], G, D, Dv, dtype, 4)
    # both tables have the width of the wider one
    width = max(table.shape[1], ptable_host.shape[1])
    pad = lambda t: torch.cat([t, torch.full((1, width - t.shape[1]), -1, dtype=torch.int32)], dim=1)
    table, ptable_host = pad(table), pad(ptable_host)
    _fill(table, kc, vc, 0, keys, vals)
    tab, ptab = table.to(DEV).contiguous(), ptable_host.to(DEV).contiguous()
    # blocks are made as their last position arrives: a first step of 2.5 blocks, then single tokens, then the rest
    first = 2 * pool + pool // 2
    cuts = [first] + [1] * (2 * pool) + [n - first - 2 * pool]
    at = 0
    for c in cuts:
        ctx = _ctx([at], [c])
        kernels.pool_blocks(kc, vc, tab, pk, pv, ptab, ctx.seq_start, ctx.seq_past, ctx.n_seqs, ctx.n_tokens, G, D, Dv, pool)
        at += c
    nb = n // pool
    kb = keys[: nb * pool].reshape(nb, pool, G, D).mean(1)
    vb = vals[: nb * pool].reshape(nb, pool, G, Dv).mean(1)
    page = kernels.PAGE
    got_k = torch.stack([pk[int(ptable_host[0, b // page]), :, b % page].cpu() for b in range(nb)]).double()
    assert _rel(got_k.numpy(), kb.numpy()) < (2e-6 if dtype == torch.float32 else 5e-3)
    # the stored means, as the attention reads them
    kb_c = got_k
    vb_c = torch.stack([pv[int(ptable_host[0, b // page]), :, b % page].cpu() for b in range(nb)]).double()

    def attend(q_rows, positions):
        q = q_rows.to(dtype).to(DEV).contiguous()
        out = torch.empty((q.shape[0], H * Dv), dtype=dtype, device=DEV)
        kernels.attention_paged(q, out, kc, vc, tab, _i32([0] * len(positions)), _i32(positions), H, G, D, size, 0.3,
                                v_head_dim=Dv, pool=pool, pool_k=pk, pool_v=pv, pool_table=ptab)
        return out.double().cpu().reshape(-1, H, Dv)

    def plain_row(q, p):
        """Query q [H, D] at position p over the window's keys and the stored block means."""
        out = torch.zeros((H, Dv), dtype=F)
        js = [j for j in range(p + 1) if plain.window_visible(p, j, size)]
        bs = [b for b in range(nb) if plain.pooled_block_visible(p, b, size, pool)]
        for h in range(H):
            gi = h // (H // G)
            kk = torch.cat([kb_c[bs, gi], keys[js, gi]]) if bs else keys[js, gi]
            vv = torch.cat([vb_c[bs, gi], vals[js, gi]]) if bs else vals[js, gi]
            out[h] = torch.softmax((kk @ q[h]) * 0.3, 0) @ vv
        return out

    tol = 5e-6 if dtype == torch.float32 else 1.5e-2
    # every position with a random query
    qs = _f32_exact(torch.randn(n, H, D, generator=g)).to(dtype).to(F)
    got = attend(qs.reshape(n, H * D), list(range(n)))
    for p in list(range(0, min(n, size + 3 * pool + 3))) + list(range(n - 3, n)):
        assert _rel(got[p].numpy(), plain_row(qs[p], p).numpy()) < tol, p
    # one key stands out: the query is a large multiple of that key (or of that block's mean)
    cases = {"window's first key": ("key", p - size + 1), "window's last key": ("key", p),
             "just outside the window": ("key", p - size), "last block seen": ("block", last_block),
             "first block": ("block", 0), "a block in the middle": ("block", last_block // 2)}
    if nb > page:
        cases["the block store's second page"] = ("block", page)
    for what, (kind, idx) in cases.items():
        if idx < 0:
            continue
        target = keys[idx] if kind == "key" else kb_c[idx]          # [G, D]
        q = torch.stack([target[h // (H // G)] / target[h // (H // G)].pow(2).sum() for h in range(H)]) * (300.0 / 0.3)
        q = q.to(dtype).to(F)
        got1 = attend(q.reshape(1, H * D), [p])[0]
        want1 = plain_row(q, p)
        assert _rel(got1.numpy(), want1.numpy()) < tol, what
        seen = kind == "block" or plain.window_visible(p, idx, size)
        hit = vals[idx] if kind == "key" else vb_c[idx]
        close = _rel(got1.numpy(), torch.stack([hit[h // (H // G)] for h in range(H)]).numpy()) < 0.05
        if what != "just outside the window":
            assert seen and close, what
        else:       # out of the window; its block is seen only as a mean, never as itself
            assert not close or pool == 1, what
    kernels.check_status()


def _pooled_case(lens, G, D, pool, seed):
    """Random bfloat16 keys and values for sequences of the given lengths, and their store of one row per block
    made by ``pool_blocks``; both block tables have one width."""
    from llmoxide_b200 import kernels

    g = torch.Generator().manual_seed(seed)
    table, kc, vc = _store(lens, G, D, D, torch.bfloat16, seed)
    ptable, pk, pv = _store([n // pool for n in lens], G, D, D, torch.bfloat16, seed + 1)
    width = max(table.shape[1], ptable.shape[1])
    pad = lambda t: torch.cat([t, torch.full((t.shape[0], width - t.shape[1]), -1, dtype=torch.int32)], dim=1)
    table, ptable = pad(table), pad(ptable)
    kc.copy_((torch.randn(kc.shape, generator=g) * 0.3).to(torch.bfloat16))
    vc.copy_(torch.randn(vc.shape, generator=g).to(torch.bfloat16))
    return table, kc, vc, ptable, pk, pv


def _make_blocks(table, kc, vc, ptable, pk, pv, lens, G, D, pool):
    from llmoxide_b200 import kernels

    ctx = _ctx([0] * len(lens), lens)
    kernels.pool_blocks(kc, vc, table.to(DEV), pk, pv, ptable.to(DEV), ctx.seq_start, ctx.seq_past, ctx.n_seqs,
                        ctx.n_tokens, G, D, D, pool)


@pytest.mark.parametrize("D, H, G", [(64, 8, 1), (128, 4, 2), (48, 3, 3), (96, 6, 1)])
@pytest.mark.parametrize("size, pool", [(36, 6), (5, 8), (64, 64), (130, 16), (7, 3), (33, 1)])
def test_decode_attention_with_pooled_blocks_equals_the_general_kernel(D, H, G, size, pool):
    """One token per sequence at lengths around the window's, the blocks' and the pages' edges.  The key just
    outside the window, the last block's last key or the first block's mean is made to stand out, so that a mask
    that is one key or one block off changes the result beyond any tolerance.  Every split gives the same answer."""
    from llmoxide_b200 import kernels

    lens = [1, 2, size, size + 1, size + pool - 1, size + pool, size + pool + 1, size + 2 * pool, 64, 65, 200, 399, 129,
            257, 64 * pool + size + 3 if pool <= 3 else 300]
    table, kc, vc, ptable, pk, pv = _pooled_case(lens, G, D, pool, seed=D + size + pool)
    B = len(lens)
    q = (torch.randn(B, H, D, generator=torch.Generator().manual_seed(1)) * 0.3).to(torch.bfloat16)
    page = kernels.PAGE
    for b, n in enumerate(lens):
        p = n - 1
        nb = max(0, (p - size + 1) // pool)
        j = [p - size, nb * pool - 1, (nb + 1) * pool - 1, 0][b % 4]
        if 0 <= j <= p:
            for g in range(G):
                kc[table[b, j // page], g, j % page] = (q[b, g * (H // G)].float() * 6.0 * (pool if b % 4 else 1)).to(torch.bfloat16)
    _make_blocks(table, kc, vc, ptable, pk, pv, lens, G, D, pool)
    past = _i32([n - 1 for n in lens])
    qd, td, ptd = q.view(B, H * D).to(DEV), table.to(DEV), ptable.to(DEV)
    want = torch.empty((B, H * D), dtype=torch.bfloat16, device=DEV)
    kernels.attention_paged(qd, want, kc, vc, td, _i32(np.arange(B)), past, H, G, D, size, 0.7, pool=pool, pool_k=pk,
                            pool_v=pv, pool_table=ptd)
    plain_window = torch.empty_like(want)
    kernels.attention_paged(qd, plain_window, kc, vc, td, _i32(np.arange(B)), past, H, G, D, size, 0.7)
    assert _rel(plain_window.float().cpu().numpy(), want.float().cpu().numpy()) > 0.1      # the blocks matter
    for n_chunks in (0, 1, 3, 8, 11):
        got = torch.empty_like(want)
        kernels.attention_decode(qd, got, kc, vc, td, past, H, G, D, size, 0.7, n_chunks=n_chunks, pool=pool, pool_k=pk,
                                 pool_v=pv, pool_table=ptd)
        assert _rel(got.float().cpu().numpy(), want.float().cpu().numpy()) < 1.5e-2, (n_chunks,)
    kernels.check_status()


@pytest.mark.parametrize("D, H, G", [(64, 8, 1), (128, 4, 2)])
@pytest.mark.parametrize("size, pool", [(36, 6), (5, 8), (64, 64), (130, 16), (7, 3), (33, 1), (200, 2)])
def test_prompt_attention_with_pooled_blocks_equals_the_general_kernel(D, H, G, size, pool):
    """Whole prompts and later portions (129 and 2 tokens after a cached prefix) in one launch: query tiles whose
    queries see different numbers of blocks, none at all, and more than a page of them."""
    from llmoxide_b200 import kernels

    lens = [1, 70, 200, 399, 257, 66, 64 * pool + size + 70 if pool <= 3 else 150]
    new = [1, 70, 200, 129, 2, 65, 100]          # the last `new` tokens of each are this step's
    table, kc, vc, ptable, pk, pv = _pooled_case(lens, G, D, pool, seed=3 * D + size + pool)
    T = sum(new)
    q = (torch.randn(T, H, D, generator=torch.Generator().manual_seed(2)) * 0.3).to(torch.bfloat16)
    start = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    tok_seq = np.concatenate([[b] * n for b, n in enumerate(new)]).astype(np.int32)
    tok_pos = np.concatenate([np.arange(L - n, L) for L, n in zip(lens, new)]).astype(np.int32)
    page = kernels.PAGE
    for b, L in enumerate(lens):                # keys that stand out for the sequence's last query and one in the middle
        for row, p in ((start[b + 1] - 1, L - 1), (start[b] + new[b] // 2, L - new[b] + new[b] // 2)):
            nb = max(0, (p - size + 1) // pool)
            j = [p - size, nb * pool - 1, (nb + 1) * pool - 1, 0][b % 4]
            if 0 <= j <= p:
                for g in range(G):
                    kc[table[b, j // page], g, j % page] = (q[row, g * (H // G)].float() * 6.0 * (pool if b % 4 else 1)).to(torch.bfloat16)
    _make_blocks(table, kc, vc, ptable, pk, pv, lens, G, D, pool)
    qd, td, ptd = q.view(T, H * D).to(DEV), table.to(DEV), ptable.to(DEV)
    want = torch.empty((T, H * D), dtype=torch.bfloat16, device=DEV)
    kernels.attention_paged(qd, want, kc, vc, td, _i32(tok_seq), _i32(tok_pos), H, G, D, size, 0.7, pool=pool, pool_k=pk,
                            pool_v=pv, pool_table=ptd)
    past = _i32([L - n for L, n in zip(lens, new)])
    got = torch.empty_like(want)
    kernels.attention_prefill(qd, got, kc, vc, td, _i32(start), past, len(lens), max(new), H, G, D, size, 0.7, pool=pool,
                              pool_k=pk, pool_v=pv, pool_table=ptd)
    assert _rel(got.float().cpu().numpy(), want.float().cpu().numpy()) < 1.5e-2
    kernels.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_output_gate_per_head(dtype):
    from llmoxide_b200 import kernels

    g = torch.Generator().manual_seed(5)
    T, H, Dv = 37, 5, 24
    out = torch.randn(T, H * Dv, generator=g).to(dtype)
    wide = (torch.randn(T, 11 + H, generator=g) * 3).float()            # the gates are the last columns of wider rows
    want = out.to(F).reshape(T, H, Dv) * torch.sigmoid(wide[:, 11:].to(F))[:, :, None]
    dev_out, dev_wide = out.to(DEV).contiguous(), wide.to(DEV)
    kernels.head_gate(dev_out, dev_wide[:, 11:], H, Dv)
    assert _rel(dev_out.double().cpu().numpy(), want.reshape(T, H * Dv).numpy()) < (2e-6 if dtype == torch.float32 else 5e-3)


# ---------------------------------------------------------------------------------------------------------
# experts named by a table
# ---------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d, Fe, E, top, T", [(72, 40, 6, 2, 33), (64, 16, 3, 3, 5), (96, 64, 8, 4, 300), (40, 8, 1, 1, 17),
                                               (128, 128, 12, 1, 700)])
def test_experts_named_by_a_table_against_the_plain_mixture(d, Fe, E, top, T, dtype):
    from llmoxide_b200.config.spec import PartSpec, TensorSpec
    from llmoxide_b200.parts import Runtime
    from llmoxide_b200.parts.block import build_part
    from llmoxide_b200.parts.registry import FEED_FORWARDS
    from llmoxide_b200 import kernels

    g = torch.Generator().manual_seed(d + E)
    vocab = 50
    rnd = lambda *s: _f32_exact(torch.randn(*s, generator=g) * 0.2).to(dtype).to(F)
    w = {}
    for e in range(E):
        w[f"p.mlp.e{e}.gate"], w[f"p.mlp.e{e}.up"], w[f"p.mlp.e{e}.down"] = rnd(Fe, d), rnd(Fe, d), rnd(d, Fe)
    table = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(vocab)])
    w["p.mlp.table"] = table
    tensors = {"table": TensorSpec("p.mlp.table", (vocab, top), "table")}
    for e in range(E):
        for r in ("gate", "up", "down"):
            tensors[f"{r}{e}"] = TensorSpec(f"p.mlp.e{e}.{r}", tuple(w[f"p.mlp.e{e}.{r}"].shape))
    spec = PartSpec("routed_experts", dict(hidden_size=d, intermediate_size=Fe, n_experts=E, top=top, score="table",
                                           table_weight=1.0 / top, n_groups=1, keep_groups=1, normalize=False, scale=1.0,
                                           activation="silu"), tensors)
    rt = Runtime(dtype="float32" if dtype == torch.float32 else "bfloat16", device=torch.device(DEV), max_positions=64)
    dev_w = {k: (v.to(torch.int32) if k.endswith("table") else v.to(dtype)).to(DEV) for k, v in w.items()}
    part = build_part(FEED_FORWARDS, "feed-forward", spec, dev_w, rt)
    tokens = torch.randint(0, vocab, (T,), generator=g)
    x = rnd(T, d) * 5
    y = part.forward(x.to(dtype).to(DEV).contiguous(), SimpleNamespace(tokens=_i32(tokens.numpy()), probe=None))
    got = y.sum(0).double().cpu()
    want = plain.table_experts(x, tokens.tolist(), w, "p.", dict(router=dict(top=top)))
    assert _rel(got.numpy(), want.numpy()) < (1e-5 if dtype == torch.float32 else 2e-2)
    kernels.check_status()


# ---------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("fusasun")
    return {(n, d): make_folder(base, n, d) for n in ALL for d in ("float32", "bfloat16")}


def _engine(folder, dtype, max_tokens=4096, **kw):
    from llmoxide_b200.engine.engine import Engine, LoadOptions

    return Engine.load(folder, LoadOptions(dtype=dtype, max_tokens=max_tokens, max_batch=8, **kw))


def _requests(name):
    toks = prompts(ALL[name]["vocab"], LENGTHS[name], seed=21)
    return {f"r{i}": t for i, t in enumerate(toks)}


def _expected(folder, reqs, cache_dtype=None):
    cfg, w = plain.read_model(folder)
    return {rid: plain.forward(cfg, w, toks, cache_dtype=cache_dtype).numpy() for rid, toks in reqs.items()}


def _rms_err(got, want):
    d = got - want
    w = want - want.mean(axis=1, keepdims=True)
    return (d - d.mean(axis=1, keepdims=True)).std(axis=1) / np.sqrt((w * w).mean())


def _compare(got, want, dtype, what):
    """float32: every logit of every position within rounding (largest difference against the largest logit).
    bfloat16: a position's error is the root mean square over the vocabulary of the difference (its mean taken
    off) against that of the logits; every position is held to the tolerance (the experts are named by a table, so
    no near tie of a router can change a token's path), the median to a third of it."""
    worst, n, over = 0.0, 0, 0
    errs = []
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid)
        e = (np.abs(got[rid] - want[rid]).max(axis=1) / np.abs(want[rid]).max() if dtype == "float32"
             else _rms_err(got[rid], want[rid]))
        errs.append(e)
        worst = max(worst, float(e.max()))
        n += len(e)
        over += int((e > (F32_TOL if dtype == "float32" else BF16_TOL)).sum())
    if dtype == "float32":
        assert over == 0, f"{what}: {over} of {n} positions differ from the plain implementation, worst {worst:.3e}"
    else:
        med = float(np.median(np.concatenate(errs)))
        assert over <= 0.02 * n and worst < 2 * BF16_TOL and med < 0.012, \
            f"{what}: {over} of {n} positions beyond {BF16_TOL}, worst {worst:.3e}, median {med:.3e}"
    return worst


def test_layer_by_layer_against_the_plain_stream(folders):
    """The residual stream after every layer, as the step's named intermediates report it."""
    for name in ALL:
        folder = folders[(name, "float32")]
        cfg, w = plain.read_model(folder)
        toks = prompts(ALL[name]["vocab"], [75], seed=4)[0]
        layers = []
        plain.forward(cfg, w, toks, streams=layers)
        eng = _engine(folder, "float32", max_tokens=512)
        got = {}
        eng.step([(eng.acquire(), toks)], [[0]], probe=lambda n, t: got.__setitem__(n, t.detach().float().cpu().numpy()))
        assert len(layers) == len(ALL[name]["layers"])
        for i, want in enumerate(layers):
            assert _rel(got[f"l_out-{i}"], want.numpy()) < 1e-5, (name, i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALL))
def test_every_cutting_matches_the_plain_implementation(folders, tmp_path, name, dtype):
    folder = folders[(name, dtype)]
    reqs = _requests(name)
    want = _expected(folder, reqs)
    vocab = ALL[name]["vocab"]
    eng = _engine(folder, dtype)
    results = {}
    # the same engine runs every trace: slots, pages, block rows and state rows are freed and used again
    for what, steps in (("whole", ru.trace_whole(reqs)),
                        ("last 48 one by one", ru.trace_tail_decode(reqs, 48)),
                        ("all but the first token one by one", ru.trace_tail_decode(reqs, 10 ** 6)),
                        ("unequal batches", ru.trace_batches(reqs, 4)),
                        ("unequal batches of 3, short prompts", ru.trace_batches(reqs, 3, 0.2)),
                        ("portions of 2", ru.trace_chunks({k: v for k, v in reqs.items() if len(v) <= 70}, 2, 3, tail=3)),
                        ("portions of 5", ru.trace_chunks(reqs, 5, 6, tail=4)),
                        ("portions of 48", ru.trace_chunks(reqs, 48, 3)),
                        ("portions of 64", ru.trace_chunks(reqs, 64, 4)),
                        ("portions of 100 beside single tokens", ru.trace_chunks(reqs, 100, 6, tail=40, mixed=True))):
        out = tmp_path / what.replace(" ", "_").replace(",", "")
        ru.run_in_process(eng, steps, out)
        for g in range(eng.cache.n_groups()):
            assert eng.cache.alloc.pages_held(g) == 0
        got = ru.collect(steps, out, vocab)
        worst = _compare(got, {rid: want[rid] for rid in got}, dtype, f"{name}/{dtype}/{what}")
        print(f"{name}/{dtype}/{what}: worst rel err {worst:.2e}")
        results[what] = got
    if dtype == "float32":      # how a prompt is cut changes the order of a few sums, nothing else
        for what, got in results.items():
            for rid in got:
                assert ru.rel_err(got[rid], results["whole"][rid]) < 6e-6, (what, rid)
    else:
        for what, got in results.items():
            e = np.concatenate([_rms_err(got[rid], results["whole"][rid]) for rid in got])
            assert (e > BF16_TOL).sum() <= 0.02 * len(e) and np.median(e) < 1.2e-2, \
                (what, int((e > BF16_TOL).sum()), float(np.median(e)), float(e.max()))
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_as_a_user_runs_it(folders, tmp_path, dtype):
    """``bin/trace_run`` as a subprocess on a Fusasun folder: unequal batches whose requests end at different
    steps, with ``--max-tokens`` the bare sum of the live requests' tokens."""
    folder = folders[("A", dtype)]
    reqs = _requests("A")
    steps = ru.trace_batches(reqs, 3, 0.6)
    ru.run_trace_run(folder, dtype, steps, tmp_path / "out", max_tokens=sum(len(t) for t in reqs.values()))
    got = ru.collect(steps, tmp_path / "out", ALL["A"]["vocab"])
    _compare(got, _expected(folder, reqs), dtype, f"trace_run/{dtype}")


def test_a_slot_used_again_starts_from_an_empty_state(folders):
    """One slot: a long request, then a short one in the same slot, then a part of the first; the later ones must
    see neither the earlier keys, nor the earlier blocks' means, nor the convolution's earlier rows."""
    folder = folders[("A", "float32")]
    eng = _engine(folder, "float32", max_tokens=512)
    cfg, w = plain.read_model(folder)
    long_req, short_req = prompts(ALL["A"]["vocab"], [200, 30], seed=5)
    for toks in (long_req, short_req, long_req[:90]):
        slot = eng.acquire()
        assert slot == 0
        got = eng.step([(slot, toks[:-2])], [list(range(len(toks) - 2))]).cpu().numpy()
        got = np.concatenate([got] + [eng.step([(slot, [t])], [[0]]).cpu().numpy() for t in toks[-2:]])
        eng.release(slot)
        assert ru.rel_err(got, plain.forward(cfg, w, toks).numpy()) < F32_TOL
    eng.cache.alloc.check_consistent()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_long_decoding_past_every_window_and_block_edge(folders, name, dtype):
    """A short prompt and 330 single-token steps: every window and many blocks' edges pass under decoded tokens,
    the block store grows row by row over a page border of the cache; decode steps replay a CUDA graph."""
    folder = folders[(name, dtype)]
    eng = _engine(folder, dtype, max_tokens=1024)
    cfg, w = plain.read_model(folder)
    toks = prompts(ALL[name]["vocab"], [340], seed=9)[0]
    want = plain.forward(cfg, w, toks).numpy()
    slot = eng.acquire()
    rows = [eng.step([(slot, toks[:10])], [list(range(10))]).cpu().numpy()]
    for t in toks[10:]:
        rows.append(eng.step([(slot, [t])], [[0]]).cpu().numpy())
    eng.release(slot)
    _compare({"r": np.concatenate(rows)}, {"r": want}, dtype, f"long decoding/{name}/{dtype}")
    eng.check_status()


def test_a_changed_token_moves_what_the_masks_let_it_reach(folders):
    """Whole model, float32: changing one token leaves every earlier position's logits bit for bit and moves the
    changed position's; model A's blocks carry it to the sequence's end, as in the plain implementation."""
    folder = folders[("A", "float32")]
    cfg, w = plain.read_model(folder)
    eng = _engine(folder, "float32", max_tokens=1024)
    toks = prompts(ALL["A"]["vocab"], [260], seed=12)[0]
    other = list(toks)
    other[100] = (toks[100] + 1) % ALL["A"]["vocab"]
    outs = []
    for seq in (toks, other):
        slot = eng.acquire()
        a = eng.step([(slot, seq[:150])], [list(range(150))]).cpu().numpy()
        b = [eng.step([(slot, [t])], [[0]]).cpu().numpy() for t in seq[150:]]
        eng.release(slot)
        outs.append(np.concatenate([a] + b))
        assert ru.rel_err(outs[-1], plain.forward(cfg, w, seq).numpy()) < F32_TOL
    moved = np.abs(outs[0] - outs[1]).max(axis=1) > 0
    assert not moved[:100].any() and moved[100] and moved[259]


@pytest.mark.parametrize("name, dtype", [("A", "float32"), ("C", "float32"), ("C", "bfloat16")])
def test_greedy_generation_through_the_session(folders, name, dtype):
    from llmoxide_b200 import LoadOptions, Request, Sampling, Session

    folder = folders[(name, dtype)]
    cfg, w = plain.read_model(folder)
    session = Session.load(folder, LoadOptions(dtype=dtype, max_tokens=2048, max_batch=4))
    reqs = prompts(ALL[name]["vocab"], [9, 1, 140, 40], seed=3)
    outs = session.generate([Request(p, 24, Sampling.greedy(), stop_ids=()) for p in reqs])
    for p, o in zip(reqs, outs):
        assert len(o.tokens) == 24
        ids = list(p)
        for tok in o.tokens:
            logits = plain.forward(cfg, w, ids)[-1].numpy()
            if dtype == "float32":
                assert logits.max() - logits[tok] <= 1e-5 * np.abs(logits).max(), (name, p[:4], o.tokens)
            else:       # bfloat16 may differ where the plain logits nearly tie
                assert logits.max() - logits[tok] <= 0.1 * np.abs(logits).max(), (name, p[:4], o.tokens)
            ids.append(tok)
    info = session.info()
    assert info["architecture"] == "Fusasun" and info["n_layers"] == len(ALL[name]["layers"])


def test_random_weights_on_the_device_equal_the_folder(folders):
    """``Engine.random`` makes the same model as the folder written from the same seed, the integer table too."""
    from llmoxide_b200 import Engine, LoadOptions, read_config

    folder = folders[("A", "float32")]
    toks = prompts(ALL["A"]["vocab"], [50], seed=1)[0]
    opts = dict(dtype="float32", max_tokens=256, max_batch=2)
    a = Engine.load(folder, LoadOptions(**opts))
    b = Engine.random(read_config(dict(copy.deepcopy(ALL["A"]), torch_dtype="float32")), 4321, LoadOptions(**opts))
    la = a.step([(a.acquire(), toks)], [[49]])
    lb = b.step([(b.acquire(), toks)], [[49]])
    assert torch.equal(la, lb)


def _drawn_config(rng):
    """A configuration whose every size is drawn: odd and even head sizes, ranks and widths that are no multiple of
    eight, windows and blocks from one position up, one to six taps, layers in any order, some without a
    feed-forward, rotations with and without scaling."""
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    width = int(pick(40, 48, 72, 100, 136, 176, 200))
    vocab = int(rng.integers(50, 400))
    layers = []
    for _ in range(int(rng.integers(2, 5))):
        E = int(rng.integers(1, 10))
        mlp = None if rng.random() < 0.2 else dict(kind="moe", expert=dict(ff=int(pick(8, 12, 20, 24, 40, 50))),
                                                   router=dict(experts=E, top=int(rng.integers(1, min(E, 4) + 1))))
        if rng.random() < 0.5:
            G = int(pick(1, 2, 3))
            H = G * int(pick(1, 2, 3))
            D = 2 * int(rng.integers(4, 40))
            rot = None
            if rng.random() < 0.85:
                dims = 2 * int(rng.integers(1, D // 2 + 1))
                sc = None if rng.random() < 0.3 else dict(factor=float(pick(2.0, 4.0, 8.0)), low=float(pick(0.5, 1.0)),
                                                          high=float(pick(2.0, 4.0)), original=int(pick(16, 64, 256)))
                rot = dict(dims=dims, base=float(pick(100.0, 10000.0, 500000.0)))
                if sc:
                    rot["scaling"] = sc
            mask = dict(size=int(rng.integers(1, 90)))
            if rng.random() < 0.85:
                mask["pool"] = int(pick(1, 2, 3, 5, 8, 13, 20, 64, 70))
            m = dict(heads=H, kv_heads=G, dim=D, vdim=int(rng.integers(3, 70)), scale=float(rng.uniform(0.05, 0.3)), mask=mask)
            if rot:
                m["rot"] = rot
            layers.append(dict(type="attention", mixer=m, mlp=mlp))
        else:
            R = 2 * int(rng.integers(1, 20))
            rot = dict(dims=R, base=float(pick(100.0, 10000.0, 500000.0)))
            if rng.random() < 0.7:
                rot["scaling"] = dict(factor=float(pick(2.0, 4.0, 16.0)), original=int(pick(16, 64, 512)),
                                      fast=float(pick(8.0, 32.0)), slow=float(pick(0.5, 1.0, 2.0)))
            layers.append(dict(type="latent_attention", mlp=mlp, mixer=dict(
                heads=int(rng.integers(1, 7)), dim=int(rng.integers(1, 60)), rot_dim=R, vdim=int(rng.integers(3, 70)),
                q_rank=int(rng.integers(5, 70)), kv_rank=int(rng.integers(5, 70)), scale=float(rng.uniform(0.05, 0.3)),
                mask=dict(size=int(rng.integers(1, 90))), rot=rot)))
    return dict(architecture="Fusasun", vocab=vocab, width=width, norm=dict(eps=float(pick(1e-5, 1e-6, 1e-3))),
                embedding=dict(scale=float(rng.uniform(0.5, 14.0))), canon=dict(taps=int(rng.integers(1, 7))), layers=layers)


@pytest.mark.parametrize("seed", range(16))
def test_drawn_configurations(tmp_path, seed):
    """Sixteen drawn configurations, each in both dtypes: whole prompts, the last 30 tokens one by one, and an
    unequal batch, against the plain implementation."""
    from llmoxide_b200.config import read_config
    from llmoxide_b200.weights import write_model_folder

    rng = np.random.default_rng(1000 + seed)
    raw = _drawn_config(rng)
    reqs = {f"r{i}": t for i, t in enumerate(prompts(raw["vocab"], [150, 37, 5, 70], seed=seed))}
    for dtype in ("float32", "bfloat16"):
        folder = write_model_folder(tmp_path / dtype, read_config(dict(raw, torch_dtype=dtype)), 99 + seed, dtype)
        want = _expected(folder, reqs)
        eng = _engine(folder, dtype, max_tokens=1024)
        for what, steps in (("whole", ru.trace_whole(reqs)), ("last 30 one by one", ru.trace_tail_decode(reqs, 30)),
                            ("an unequal batch", ru.trace_batches(reqs, 4, 0.4))):
            out = tmp_path / f"{dtype}_{what.replace(' ', '_')}"
            ru.run_in_process(eng, steps, out)
            got = ru.collect(steps, out, raw["vocab"])
            _compare(got, {rid: want[rid] for rid in got}, dtype, f"drawn {seed}/{dtype}/{what}: {raw}")
        eng.check_status()
