"""Small Bafavik configurations for the tests, with weights made so that the states remember long enough for a lost state to
show and every vector of the design (shifts, layer scales, biases, the lambda vectors) moves its formula."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def rot(base, dims):
    return dict(base=base, dims=dims)


def softmax_left(heads, kv_heads, dim, vdim, scale, rotation, conv=None):
    out = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=rotation)
    if conv is not None:
        out["conv"] = conv
    return out


def pair(left, heads, dim, vdim, decay, left_scale, right_scale):
    return dict(type="parallel", mixer=dict(left=left, right=dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay)),
                                            left_scale=left_scale, right_scale=right_scale))


def pair_2(left, heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    right = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, decay_rank=decay_rank, gate_rank=gate_rank)
    return dict(type="parallel_2", mixer=dict(left=left, right=right))


def differential(heads, kv_heads, dim, vdim, scale, diff, chunk):
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, diff=diff,
                                             mask=dict(size=chunk)))


def layer(mix, ff):
    return dict(mix, mlp=None if ff is None else dict(kind="dense", ff=ff))


def model(vocab, width, eps, mult, logit_scale, embed_scale, bigram, loop, layers):
    embedding = dict(scale=embed_scale)
    if bigram is not None:
        embedding["bigram"] = dict(buckets=bigram[0], mul_prev=bigram[1], mul_cur=bigram[2])
    return dict(architecture="Bafavik", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult, logit_scale=logit_scale,
                embedding=embedding, loop=None if loop is None else dict(start=loop[0], stop=loop[1], times=loop[2]), layers=layers)


# Sizes that differ from one another everywhere: keys and values of different sizes in every mixer, fewer key heads than query
# heads, rotations over a part of a head and over all of it, chunks of 13 positions (no multiple of a page), two to four taps,
# a layer without feed-forward, a loop over the two middle layers that runs three times.
BAFAVIK_A = model(203, 96, 1e-5, 0.6, 0.7, 2.0, (97, 31, 5), (1, 3, 3), [
    layer(pair_2(softmax_left(4, 2, 16, 24, 0.3, rot(500.0, 8), conv=4), 4, 2, 12, 20, 2, 5, 7), 56),
    layer(pair(softmax_left(6, 3, 16, 8, 0.25, rot(10000.0, 16)), 3, 8, 16, (0.7, 0.95, 0.995), 0.7, 1.2), None),
    layer(differential(4, 2, 12, 20, 0.29, 0.3, 13), 40),
    layer(pair(softmax_left(2, 1, 24, 16, 0.2, rot(300.0, 12)), 2, 20, 12, (0.9, 0.99), 1.1, 0.9), 64),
])
# One head everywhere, one tap (no convolution inputs kept), no rotation and a rotation of one pair, a chunk of one position
# (a token sees itself alone) and one that no request of the tests outgrows, no loop, no token-pair table, constants of 1.
BAFAVIK_B = model(157, 72, 1e-6, 1.0, 1.0, 1.0, None, None, [
    layer(differential(1, 1, 10, 14, 0.4, 0.8, 1), 20),
    layer(pair_2(softmax_left(1, 1, 12, 6, 0.4, rot(100.0, 0), conv=1), 1, 1, 10, 14, 1, 1, 1), None),
    layer(pair(softmax_left(1, 1, 6, 10, 0.5, rot(20000.0, 2)), 1, 14, 6, (0.98,), 1.0, 1.0), 18),
    layer(differential(5, 5, 6, 6, 0.17, 0.5, 1000), 24),
])
# Sizes of the kind real models have in small: heads of 64 and 128 (the tensor-core attention kernels), keys of 64 to 128
# entries in the recurrences, eight query heads per key head, a loop that runs the first layers twice.
BAFAVIK_C = model(300, 128, 1e-6, 0.5, 0.6, 2.5, (509, 1000003, 7919), (0, 2, 2), [
    layer(pair(softmax_left(8, 1, 64, 64, 0.125, rot(1000000.0, 64)), 2, 128, 64, (0.9, 0.998), 1.0, 1.0), 256),
    layer(differential(4, 2, 32, 64, 0.18, 0.45, 50), 128),
    layer(pair_2(softmax_left(2, 1, 128, 64, 0.09, rot(10000.0, 64), conv=3), 4, 2, 64, 32, 4, 16, 8), 256),
    layer(pair(softmax_left(4, 2, 128, 128, 0.09, rot(10000.0, 32)), 4, 64, 128, (0.5, 0.8, 0.95, 0.99), 0.9, 1.1), 128),
])
# Widths that are no multiple of eight; head sizes that are odd or no multiple of four; a loop over the last layer alone.
BAFAVIK_D = model(120, 44, 1e-5, 0.8, 1.3, 0.5, (11, 3, 2), (1, 2, 4), [
    layer(pair_2(softmax_left(3, 3, 10, 7, 0.3, rot(2000.0, 6), conv=5), 3, 1, 9, 5, 3, 3, 2), 30),
    layer(differential(2, 1, 7, 9, 0.3, 0.2, 9), 18),
])
CONFIGS = {"a": BAFAVIK_A, "b": BAFAVIK_B, "c": BAFAVIK_C, "d": BAFAVIK_D}


def random_config(rng) -> dict:
    """A configuration drawn from ``rng`` (a ``random.Random``): one to five layers of any kind in any order, head counts,
    head sizes, taps, chunks, inner sizes of the two-step projections and a repeated run drawn independently of one another."""
    width = rng.choice([24, 40, 64, 72])

    def left(conv):
        kv = rng.choice([1, 2, 3])
        dim = rng.choice([4, 6, 8, 10, 16])
        dims = rng.choice([0, 2, dim // 2 * 2, dim // 4 * 2])
        return softmax_left(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([4, 8, 12]), rng.uniform(0.1, 0.5),
                            rot(rng.choice([100.0, 10000.0]), dims), conv=rng.choice([1, 2, 3, 4, 6]) if conv else None)

    layers = []
    for _ in range(rng.choice([1, 2, 3, 4, 5])):
        kind, ff = rng.choice(["parallel", "attention", "parallel_2"]), rng.choice([None, 16, 24, 50])
        if kind == "parallel":
            heads = rng.choice([1, 2, 3, 5])
            layers.append(layer(pair(left(False), heads, rng.choice([4, 6, 9, 16]), rng.choice([4, 8, 10]),
                                     [rng.uniform(0.5, 0.998) for _ in range(heads)], rng.uniform(0.3, 1.5), rng.uniform(0.3, 1.5)), ff))
        elif kind == "attention":
            kv = rng.choice([1, 2])
            layers.append(layer(differential(kv * rng.choice([1, 2, 3]), kv, rng.choice([4, 6, 16]), rng.choice([4, 5, 16]),
                                             rng.uniform(0.1, 0.5), rng.uniform(0.1, 0.9), rng.choice([1, 2, 5, 8, 16, 33, 500])), ff))
        else:
            kv = rng.choice([1, 2])
            layers.append(layer(pair_2(left(True), kv * rng.choice([1, 2, 3]), kv, rng.choice([4, 6, 9, 16]), rng.choice([8, 10]),
                                       rng.choice([1, 2, 4, 5]), rng.choice([1, 3, 8]), rng.choice([1, 2, 7])), ff))
    loop = None
    if rng.random() < 0.7:
        start = rng.randrange(0, len(layers))
        loop = (start, rng.randrange(start + 1, len(layers) + 1), rng.choice([1, 2, 3]))
    bigram = (rng.choice([5, 97, 1019]), rng.choice([1, 31, 99991]), rng.choice([1, 11, 5003])) if rng.random() < 0.8 else None
    return model(rng.choice([50, 131]), width, rng.choice([1e-5, 1e-6]), rng.uniform(0.3, 1.2), rng.uniform(0.3, 1.5),
                 rng.uniform(0.5, 3.0), bigram, loop, layers)


def _normal(shape, seed, std, mean=0.0):
    return mean + std * torch.randn(shape, generator=torch.Generator().manual_seed(seed))


def shape_weights(tensors: dict, config: dict) -> None:
    """Makes faults show: shifts spread over (0, 1), layer scales and norm weights away from their neutral values, biases and
    convolution taps as large as the projections' results, decays of the delta rule near one (a lost or mixed-up state shows
    dozens of tokens later), the vectors of lambda so that it is neither 0 nor ``diff``.  In place."""
    def put(name, value):
        tensors[name] = value.to(tensors[name].dtype)

    for index, entry in enumerate(config["layers"]):
        p, seed = f"l{index}.", 100 * index
        width = config["width"]
        put(p + "shift", torch.rand((width,), generator=torch.Generator().manual_seed(seed + 1)))
        for name in ("ls1", "ls2", "norm1", "norm2"):
            if p + name in tensors:
                put(p + name, _normal((width,), seed + 2 + len(name), 0.3, 1.0 if name.startswith("ls") else 0.0))
        m, mix = entry["mixer"], p + "mix."
        if entry["type"] == "attention":
            for k, name in enumerate(("lq1", "lk1", "lq2", "lk2")):
                put(mix + name, _normal((m["dim"],), seed + 10 + k, 0.35))
            for k, name in enumerate(("q.b", "k.b", "v.b")):
                put(mix + name, _normal(tuple(tensors[mix + name].shape), seed + 20 + k, 0.3))
            continue
        if entry["type"] == "parallel":
            for k, name in enumerate(("q.b", "k.b", "v.b", "o.b")):
                put(mix + "left." + name, _normal(tuple(tensors[mix + "left." + name].shape), seed + 30 + k, 0.3))
            continue
        r = mix + "right."
        for k, name in enumerate(("left.q.conv", "left.k.conv", "left.v.conv", "right.q.conv", "right.k.conv", "right.v.conv")):
            put(mix + name, _normal(tuple(tensors[mix + name].shape), seed + 40 + k, 0.6))
        put(r + "A_log", _normal((m["right"]["heads"],), seed + 50, 0.3, -2.5))
        put(r + "dt_bias", _normal(tuple(tensors[r + "dt_bias"].shape), seed + 51, 0.5))
        for k, name in enumerate(("a1", "a2", "g1", "g2", "b")):
            put(r + name, _normal(tuple(tensors[r + name].shape), seed + 60 + k, 0.5))
        for k, name in enumerate(("left.out", "right.out")):
            put(mix + name, _normal((width,), seed + 70 + k, 0.3, 1.0))
    put("final.norm", _normal((config["width"],), 7, 0.2))


def stored_config(config: dict) -> dict:
    """The configuration as a checkpoint's ``config.json`` spells it: without the inner sizes of the two-step projections,
    which the tensors' shapes give."""
    out = json.loads(json.dumps(config))
    for entry in out["layers"]:
        if entry["type"] == "parallel_2":
            entry["mixer"]["right"].pop("decay_rank")
            entry["mixer"]["right"].pop("gate_rank")
    return out


def make_folder(tmp_path, name: str, seed: int = 0, stored_dtype: str = "bfloat16", matrix_std: float = 0.08, config=None) -> Path:
    import miniserve_b200  # noqa: F401
    from miniserve_b200.weights import random_tensors
    from safetensors.torch import save_file

    folder = Path(tmp_path) / f"bafavik_{name}_{seed}_{stored_dtype}"
    if not folder.exists():
        folder.mkdir(parents=True)
        config = CONFIGS[name] if config is None else config
        tensors = random_tensors(config, seed, stored_dtype, matrix_std)
        shape_weights(tensors, config)
        (folder / "config.json").write_text(json.dumps(stored_config(config), indent=1))
        save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder


def load_folder(folder):
    from safetensors.torch import load_file

    config = json.loads((Path(folder) / "config.json").read_text())
    weights = {k: v.to(torch.float64) for k, v in load_file(str(Path(folder) / "model.safetensors")).items()}
    return config, weights
