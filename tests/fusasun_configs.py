"""Small configurations of the Fusasun decoder for tests.  They differ from one another in every size and option:
head counts and key/value groups, key and value sizes that differ, windows shorter than, equal to and longer than a
cache page, pooled blocks shorter and longer than the window and of a single position, partial and full rotation
with and without scaled frequencies, one to five convolution taps, one to four experts per token, layers without a
feed-forward, widths that are no multiple of eight, and sizes that the tiled attention kernels take."""


def _moe(experts, top, ff):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def _attention(heads, kv_heads, dim, vdim, scale, size, pool, rot, mlp=None):
    mask = dict(size=size)
    if pool is not None:
        mask["pool"] = pool
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, mask=mask)
    if rot is not None:
        dims, base, scaling = rot
        m["rot"] = dict(dims=dims, base=base)
        if scaling is not None:
            factor, low, high, original = scaling
            m["rot"]["scaling"] = dict(factor=factor, low=low, high=high, original=original)
    return dict(type="attention", mixer=m, mlp=mlp)


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, size, base, scaling, mlp=None):
    rot = dict(dims=rot_dim, base=base)
    if scaling is not None:
        factor, original, fast, slow = scaling
        rot["scaling"] = dict(factor=factor, original=original, fast=fast, slow=slow)
    return dict(type="latent_attention", mlp=mlp,
                mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank,
                           scale=scale, mask=dict(size=size), rot=rot))


# An attention layer first; a window shorter than a page with blocks of four; two key/value groups; values narrower
# than keys; partial rotation with scaled frequencies; two experts per token; a layer without a feed-forward.
FS_A = dict(
    architecture="Fusasun", vocab=211, width=96, norm=dict(eps=1e-5), embedding=dict(scale=3.0), canon=dict(taps=3),
    layers=[
        _attention(4, 2, 32, 16, 0.2, 20, 4, (16, 10000.0, (8.0, 1.0, 4.0, 64)), mlp=_moe(6, 2, 24)),
        _latent(3, 16, 8, 24, 40, 48, 0.25, 33, 1000.0, (4.0, 32, 16.0, 2.0), mlp=_moe(5, 1, 40)),
        _attention(4, 2, 32, 16, 0.2, 7, 16, (32, 500.0, None), mlp=None),
        _latent(2, 24, 16, 8, 24, 20, 0.15, 5, 10000.0, None, mlp=_moe(6, 2, 24)),
    ])
# A width that is no multiple of eight (every product on the FMA units), one tap (no state), three key/value groups,
# values wider than keys, a window of exactly a page, blocks longer than the window, an attention layer without
# rotation, every expert used.
FS_B = dict(
    architecture="Fusasun", vocab=300, width=100, norm=dict(eps=1e-6), embedding=dict(scale=0.5), canon=dict(taps=1),
    layers=[
        _latent(5, 20, 12, 12, 36, 28, 0.3, 64, 50000.0, (2.0, 48, 8.0, 1.0), mlp=_moe(4, 4, 20)),
        _attention(6, 3, 16, 48, 0.25, 64, 70, None, mlp=_moe(3, 1, 36)),
        _attention(3, 3, 48, 40, 0.15, 10, 3, (48, 500000.0, (2.0, 2.0, 8.0, 100)), mlp=_moe(4, 4, 20)),
    ])
# The sizes the tiled kernels like (64 and 128), one kv head, a window longer than a page, blocks of a quarter page,
# assembled latent keys of 128 with values of 128, four taps.
FS_C = dict(
    architecture="Fusasun", vocab=512, width=256, norm=dict(eps=1e-6), embedding=dict(scale=1.0), canon=dict(taps=4),
    layers=[
        _latent(2, 96, 32, 128, 64, 128, 0.09, 130, 500000.0, (2.0, 128, 32.0, 1.0), mlp=_moe(8, 2, 128)),
        _attention(4, 1, 128, 128, 0.09, 130, 16, (128, 1000000.0, (4.0, 1.0, 4.0, 256)), mlp=_moe(8, 2, 128)),
        _attention(8, 4, 64, 64, 0.125, 44, 12, (32, 10000.0, None), mlp=_moe(8, 2, 128)),
        _latent(4, 32, 32, 64, 96, 64, 0.125, 40, 10000.0, None, mlp=None),
    ])
# Sizes that are no power of two, blocks of one position (every earlier key is seen), a window of two, a single
# expert, a single head, five taps, as many key/value heads as heads.
FS_D = dict(
    architecture="Fusasun", vocab=1000, width=184, norm=dict(eps=1e-4), embedding=dict(scale=7.5), canon=dict(taps=5),
    layers=[
        _attention(6, 2, 96, 32, 0.1, 2, 5, (32, 100.0, (16.0, 0.5, 2.0, 50)), mlp=_moe(1, 1, 72)),
        _latent(1, 40, 24, 72, 16, 200, 0.12, 300, 100000.0, (8.0, 200, 4.0, 0.5), mlp=_moe(20, 3, 72)),
        _attention(8, 8, 24, 24, 0.2, 50, 1, (24, 10000.0, None), mlp=_moe(20, 3, 72)),
        _attention(2, 1, 80, 48, 0.11, 100, None, (20, 2000.0, None), mlp=_moe(7, 2, 33)),
    ])
ALL = {"A": FS_A, "B": FS_B, "C": FS_C, "D": FS_D}


def make_folder(tmp_path, name: str, dtype: str, seed: int = 4321):
    from pathlib import Path

    from llmoxide_b200.config import read_config
    from llmoxide_b200.weights import write_model_folder

    cfg = dict(ALL[name], torch_dtype=dtype)
    folder = Path(tmp_path) / f"fusasun_{name}_{dtype}"
    if not (folder / "model.safetensors").exists():
        write_model_folder(folder, read_config(cfg), seed, dtype)
    return folder
