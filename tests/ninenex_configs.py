"""Small configurations of the Ninenex decoder for tests.  They differ from one another in every size and option:
head counts and key/value groups, key and value sizes that differ, chunks shorter than, equal to and longer than a
cache page, a layer without a mask, partial, full and no rotation, layers that borrow an earlier layer's weights,
dense and routed feed-forwards with and without a shared expert, a layer without a feed-forward, a width that is
no multiple of eight."""


def _dense(ff):
    return dict(kind="dense", ff=ff)


def _moe(experts, top, ff, shared=None):
    m = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    if shared:
        m["shared"] = dict(ff=shared)
    return m


def _mlstm(heads, dim, vdim, cap, mlp=None, weights_of=None):
    layer = dict(type="mlstm", mixer=dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap), mlp=mlp)
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def _parallel(left, right, scales, mlp=None, weights_of=None):
    heads, kv_heads, dim, vdim, scale, chunk, rot = left
    lm = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if chunk:
        lm["mask"] = dict(size=chunk)
    if rot:
        lm["rot"] = dict(dims=rot[0], base=rot[1])
    rh, rdim, rvdim, decay = right
    layer = dict(type="parallel", mlp=mlp,
                 mixer=dict(left=lm, right=dict(heads=rh, dim=rdim, vdim=rvdim, decay=decay),
                            left_scale=scales[0], right_scale=scales[1]))
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


# A chunk shorter than a page, two key/value groups, values narrower than keys, partial rotation; the attention
# layer comes first and is used twice; a layer without a feed-forward.
NX_A = dict(
    architecture="Ninenex", vocab=211, width=96, norm=dict(eps=1e-5), embedding=dict(scale=1.5), logit_scale=0.7,
    layers=[
        _parallel((4, 2, 32, 16, 0.2, 20, (16, 10000.0)), (2, 16, 24, [0.8, 0.995]), (1.25, 0.6), mlp=_dense(40)),
        _mlstm(3, 16, 24, 10.0, mlp=_moe(6, 2, 24, shared=40)),
        _parallel((4, 2, 32, 16, 0.2, 20, (16, 10000.0)), (2, 16, 24, [0.8, 0.995]), (1.25, 0.6), mlp=_dense(40),
                  weights_of=0),
        _mlstm(2, 24, 8, 4.0, mlp=None),
    ])
# A width that is no multiple of eight (every product on the FMA units), three key/value groups, values wider than
# keys, a chunk of exactly a page, a layer without a mask and without rotation, every expert used, no shared expert.
NX_B = dict(
    architecture="Ninenex", vocab=300, width=100, norm=dict(eps=1e-6), embedding=dict(scale=0.25), logit_scale=3.0,
    layers=[
        _mlstm(2, 20, 12, 30.0, mlp=_dense(36)),
        _parallel((6, 3, 16, 48, 0.25, 64, None), (3, 20, 12, [0.3, 0.97, 1.0]), (0.5, 2.0), mlp=_moe(4, 4, 20)),
        _mlstm(2, 20, 12, 30.0, mlp=_dense(36), weights_of=0),
        _parallel((3, 3, 48, 40, 0.15, None, (48, 500000.0)), (1, 8, 32, [0.9]), (1.0, 1.0), mlp=_moe(5, 1, 16, shared=8)),
        _mlstm(2, 20, 12, 30.0, mlp=_dense(36), weights_of=0),
    ])
# The sizes the tiled kernels like (multiples of 64 and 128), one kv head, a chunk longer than a page, an attention
# layer without a mask whose keys and values are alike (the tiled bfloat16 kernels), full rotation.
NX_C = dict(
    architecture="Ninenex", vocab=512, width=256, norm=dict(eps=1e-6), embedding=dict(scale=1.0), logit_scale=1.0,
    layers=[
        _mlstm(2, 128, 128, 15.0, mlp=_moe(8, 2, 128, shared=128)),
        _parallel((4, 1, 128, 128, 0.09, 130, (128, 1000000.0)), (2, 64, 128, [0.95, 0.999]), (0.9, 0.4), mlp=_dense(256)),
        _parallel((4, 2, 64, 64, 0.125, None, (32, 10000.0)), (2, 128, 64, [0.9, 0.99]), (0.7, 0.7), mlp=_moe(8, 2, 128, shared=128)),
        _mlstm(2, 128, 128, 15.0, mlp=_moe(8, 2, 128, shared=128), weights_of=0),
    ])
# Sizes that are no power of two, a chunk of two positions, one expert of which one is chosen, a single head.
NX_D = dict(
    architecture="Ninenex", vocab=1000, width=192, norm=dict(eps=1e-4), embedding=dict(scale=2.0), logit_scale=0.5,
    layers=[
        _mlstm(4, 48, 96, 8.0, mlp=_moe(1, 1, 72)),
        _parallel((6, 2, 96, 32, 0.1, 2, (32, 100.0)), (4, 48, 40, [0.5, 0.9, 0.99, 0.9995]), (0.3, 1.7), mlp=_moe(20, 3, 72, shared=24)),
        _mlstm(1, 200, 33, 12.0, mlp=_dense(80)),
        _parallel((6, 2, 96, 32, 0.1, 2, (32, 100.0)), (4, 48, 40, [0.5, 0.9, 0.99, 0.9995]), (0.3, 1.7), mlp=_moe(20, 3, 72, shared=24),
                  weights_of=1),
        _parallel((8, 8, 24, 24, 0.2, 300, (24, 10000.0)), (2, 32, 16, [0.99, 0.5]), (1.0, 0.5), mlp=_dense(64)),
    ])
ALL = {"A": NX_A, "B": NX_B, "C": NX_C, "D": NX_D}


def make_folder(tmp_path, name: str, dtype: str, seed: int = 4321):
    from pathlib import Path

    from llmoxide_b200.config import read_config
    from llmoxide_b200.weights import write_model_folder

    cfg = dict(ALL[name], torch_dtype=dtype)
    folder = Path(tmp_path) / f"ninenex_{name}_{dtype}"
    if not (folder / "model.safetensors").exists():
        write_model_folder(folder, read_config(cfg), seed, dtype)
    return folder
