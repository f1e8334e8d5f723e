"""Small Kivurax configurations for the tests, with weights made so that the routing is never a close call and the
recurrences remember long enough for a lost state to show."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def mlstm(heads, dim, vdim, cap):
    return dict(type="mlstm", mixer=dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap))


def delta(heads, kv_heads, dim, vdim, conv):
    return dict(type="delta", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv))


def rot(base, dims, scaling=None):
    out = dict(base=base, dims=dims)
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def side(heads, kv_heads, dim, scale, window, rotation, width, blocks, conv, left_scale, right_scale):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale, mask=dict(size=window), rot=rotation)
    return dict(type="parallel", mixer=dict(left=left, right=dict(width=width, blocks=blocks, conv=conv), left_scale=left_scale,
                                            right_scale=right_scale))


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


# Sizes that differ from one another everywhere: keys and values of different sizes in both matrix mixers, fewer query/key
# heads than value heads, fewer key heads than query heads under a short window, a rotation over part of a head with
# stretched frequencies and one over all of it without, two and three experts a token, a layer without a feed-forward,
# convolutions of two, three and five taps, gates in two, three and six parts.
KIVURAX_A = dict(architecture="Kivurax", vocab=211, width=96, norm=dict(eps=1e-5), residual_mult=0.7, layers=[
    layer(side(6, 3, 24, 0.23, 19, rot(5000.0, 16, (4.0, 64, 8.0, 2.0)), 72, 3, 3, 0.8, 1.3), moe(6, 2, 24)),
    layer(mlstm(3, 20, 12, 6.0), dense(56)),
    layer(delta(6, 2, 12, 20, 2), None),
    layer(delta(2, 2, 40, 8, 5), moe(5, 3, 16)),
    layer(mlstm(2, 8, 40, 15.0), moe(6, 2, 24)),
    layer(side(4, 4, 16, 0.31, 64, rot(300.0, 16), 48, 6, 2, 1.5, 0.4), dense(40)),
])
# One head and one part everywhere; every expert chosen; odd sizes (nothing a multiple of eight but the width); a
# convolution of one tap (no inputs kept); a window of one key (a token sees itself alone) and no rotation at all; a
# recurrent layer first and last.
KIVURAX_B = dict(architecture="Kivurax", vocab=157, width=72, norm=dict(eps=1e-6), residual_mult=1.0, layers=[
    layer(delta(1, 1, 10, 14, 1), moe(3, 3, 12)),
    layer(side(1, 1, 12, 0.4, 1, rot(100.0, 0), 20, 1, 1, 1.0, 1.0), dense(20)),
    layer(mlstm(1, 6, 10, 2.0), None),
    layer(side(5, 5, 6, 0.17, 7, rot(20000.0, 2), 35, 5, 4, 0.5, 2.0), moe(4, 1, 10)),
    layer(mlstm(5, 14, 6, 30.0), dense(18)),
])
# Sizes of the kind real models have in small: heads of 64 and 128 (the tensor-core attention kernels), keys of 64, 128
# and 256 entries in the matrix mixers, eight query heads per key head, many experts.
KIVURAX_C = dict(architecture="Kivurax", vocab=300, width=128, norm=dict(eps=1e-6), residual_mult=0.5, layers=[
    layer(mlstm(2, 128, 64, 15.0), dense(256)),
    layer(side(8, 1, 64, 0.125, 40, rot(1000000.0, 64, (8.0, 128, 32.0, 1.0)), 256, 8, 4, 1.0, 1.0), moe(16, 4, 32)),
    layer(delta(4, 2, 64, 32, 4), moe(12, 2, 32)),
    layer(side(4, 2, 128, 0.09, 100, rot(10000.0, 64), 128, 2, 4, 1.1, 0.7), dense(128)),
    layer(delta(2, 1, 256, 16, 3), moe(16, 4, 32)),
    layer(mlstm(4, 64, 128, 15.0), moe(12, 2, 32)),
])
# No attention at all (no pages are needed, only state slots), a layer list that ends without a feed-forward.
KIVURAX_D = dict(architecture="Kivurax", vocab=190, width=64, norm=dict(eps=1e-5), residual_mult=0.8, layers=[
    layer(delta(4, 1, 16, 24, 3), dense(48)),
    layer(mlstm(2, 32, 16, 8.0), moe(4, 2, 20)),
    layer(mlstm(4, 12, 20, 20.0), dense(32)),
    layer(delta(2, 2, 24, 32, 4), None),
])
# Nothing but side-by-side layers: heads of 32 and of 16 over one key head, a window shorter than a page and one that no
# request of the tests outgrows.
KIVURAX_E = dict(architecture="Kivurax", vocab=120, width=48, norm=dict(eps=1e-6), residual_mult=0.6, layers=[
    layer(side(3, 3, 32, 0.2, 9, rot(2000.0, 32, (3.0, 32, 16.0, 1.0)), 40, 4, 3, 0.9, 1.1), moe(5, 2, 16)),
    layer(side(4, 1, 16, 0.3, 500, rot(700.0, 8), 24, 3, 2, 1.4, 0.6), dense(36)),
])
CONFIGS = {"a": KIVURAX_A, "b": KIVURAX_B, "c": KIVURAX_C, "d": KIVURAX_D, "e": KIVURAX_E}


def _normal(shape, seed, std, mean=0.0):
    return mean + std * torch.randn(shape, generator=torch.Generator().manual_seed(seed))


def shape_weights(tensors: dict, config: dict) -> None:
    """Makes faults show.  Every routed layer gets columns of its own in the embedding: a token's row carries the marks 16,
    12, 9, ... in the columns of the experts id, id + 1, ... (mod the number of experts), as many as the layer chooses, and
    nothing in the layer's other columns; the router reads only its own columns (weight one quarter) and the norms of the
    sublayers' outputs have weight zero there, so the stream keeps the marks through all layers and the chosen experts'
    scores stand clear of the others'.  Decays are set so that the states remember a dozen tokens or more (a lost or
    mixed-up state shows), gate biases so that both gates move, and convolution taps are as large as the projections are
    small.  In place."""
    vocab, width = config["vocab"], config["width"]
    ids = torch.arange(vocab)
    embed = tensors["embed"].float()
    column = 0
    for index, entry in enumerate(config["layers"]):
        p = f"l{index}.mix."
        like = lambda name, value: value.to(tensors[name].dtype)       # noqa: E731
        if entry["type"] == "mlstm":
            heads = entry["mixer"]["heads"]
            tensors[p + "f.b"] = like(p + "f.b", _normal((heads,), 100 + index, 0.5, 3.0))
            tensors[p + "i.b"] = like(p + "i.b", _normal((heads,), 200 + index, 1.0))
            for name in ("i", "f"):
                tensors[p + name] = like(p + name, _normal(tuple(tensors[p + name].shape), 300 + index, 0.5))
        elif entry["type"] == "delta":
            heads = entry["mixer"]["heads"]
            tensors[p + "A_log"] = like(p + "A_log", _normal((heads,), 400 + index, 0.3, -1.5))
            tensors[p + "dt_bias"] = like(p + "dt_bias", _normal((heads,), 500 + index, 0.5))
            for name in ("q.conv", "k.conv", "v.conv"):
                tensors[p + name] = like(p + name, _normal(tuple(tensors[p + name].shape), 600 + index, 0.6))
            for name in ("a", "b"):
                tensors[p + name] = like(p + name, _normal(tuple(tensors[p + name].shape), 650 + index, 0.5))
        else:
            r = p + "right."
            channels = entry["mixer"]["right"]["width"]
            tensors[r + "lam"] = like(r + "lam", _normal((channels,), 700 + index, 0.4, -2.5))
            tensors[r + "conv"] = like(r + "conv", _normal(tuple(tensors[r + "conv"].shape), 800 + index, 0.6))
            for name in ("ra", "ri"):
                tensors[r + name] = like(r + name, _normal(tuple(tensors[r + name].shape), 850 + index, 0.4))
            for name in ("ra.b", "ri.b", "y.b", "x.b", "conv.b"):
                tensors[r + name] = like(r + name, _normal(tuple(tensors[r + name].shape), 900 + index, 0.3))
        mlp = entry["mlp"]
        if not mlp:
            continue
        if mlp["kind"] == "dense":
            for name in ("gate.b", "up.b", "down.b"):
                full = f"l{index}.mlp.{name}"
                tensors[full] = like(full, _normal(tuple(tensors[full].shape), 950 + index, 0.3))
            continue
        total, top = mlp["router"]["experts"], mlp["router"]["top"]
        embed[:, column:column + total] = 0
        for choice in range(top):
            embed[ids, column + (ids + choice) % total] = 16.0 * 0.75 ** choice
        name = f"l{index}.mlp.router"
        weight = torch.zeros(total, width)
        weight[:, column:column + total] = 0.25 * torch.eye(total)
        tensors[name] = weight.to(tensors[name].dtype)
        column += total
    if column > width:
        raise ValueError("the width is too small for the marks of all routed layers")
    for name in tensors:
        if name.endswith((".norm1", ".norm2")):
            tensors[name][:column] = 0.0
    tensors["embed"] = embed.to(tensors["embed"].dtype)


def make_folder(tmp_path, name: str, seed: int = 0, stored_dtype: str = "bfloat16", matrix_std: float = 0.08, config=None) -> Path:
    import miniserve_b200  # noqa: F401
    from miniserve_b200.weights import random_tensors
    from safetensors.torch import save_file

    folder = Path(tmp_path) / f"kivurax_{name}_{seed}_{stored_dtype}"
    if not folder.exists():
        folder.mkdir(parents=True)
        config = CONFIGS[name] if config is None else config
        tensors = random_tensors(config, seed, stored_dtype, matrix_std)
        shape_weights(tensors, config)
        (folder / "config.json").write_text(json.dumps(config, indent=1))
        save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
