"""Bafavik without a GPU: its configuration, what it declares, the plain implementation's own consistency, and the host-side
logic (parts, block, nested caches of mixers made of several, state slots, step function) on the CPU with plain PyTorch
functions standing in for the kernels, in every cutting, against the plain implementation."""

from __future__ import annotations

import copy
import json

import pytest
import torch

import bafavik_helpers as bh
import helpers
import plain_bafavik as plain
import plain_ops


def test_configuration_reads_every_size_and_round_trips():
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import BafavikConfig, resolve_architecture
    from miniserve_b200.parts import DecoderModel, PagedKVNeed, StateNeed

    for name, raw in bh.CONFIGS.items():
        architecture = resolve_architecture(raw)
        config = architecture.config_class.from_dict(raw)
        assert isinstance(config, BafavikConfig) and config.to_dict() == raw
        spec = architecture.build_spec(config)
        assert spec.output_name == "head" and spec.logit_scale == raw["logit_scale"] and spec.embedding_scale == raw["embedding"]["scale"]
        assert [run.layer for run in spec.order] == plain.layer_order(raw)
        assert len(spec.extra_embeddings) == (1 if "bigram" in raw["embedding"] else 0)
        model = DecoderModel(spec, torch.float32, "cpu")
        names = {s.name: s for s in model.param_specs()}
        width = raw["width"]
        shift_groups = set()
        for run, plan in zip(spec.order, model.run_caches):
            entry, p = raw["layers"][run.layer], f"l{run.layer}.mix."
            m = entry["mixer"]
            own, inner = plan                                  # the shifted input's state, then the mixer's own caches
            assert model.cache_groups[own.group].need == StateNeed((width,), torch.float32)
            shift_groups.add(own.group)
            if entry["type"] == "attention":
                need = model.cache_groups[inner.group].need
                assert need == PagedKVNeed(2 * m["kv_heads"], m["dim"], None, None if m["vdim"] == m["dim"] else m["vdim"], m["mask"]["size"],
                                           m["kv_heads"])          # both maps' key heads over ONE set of value heads
                assert names[p + "q"].shape == (m["heads"] * 2 * m["dim"], width) and names[p + "g"].shape == (m["heads"] * m["vdim"], width)
                assert names[p + "lk2"].shape == (m["dim"],) and names[p + "k.b"].shape == (m["kv_heads"] * 2 * m["dim"],)
            elif entry["type"] == "parallel":
                left, right = m["left"], m["right"]
                assert model.cache_groups[inner[0].group].need == PagedKVNeed(
                    left["kv_heads"], left["dim"], None, None if left["vdim"] == left["dim"] else left["vdim"])
                assert model.cache_groups[inner[1].group].need == StateNeed((right["heads"] * right["vdim"] * right["dim"],), torch.float32)
                assert names[p + "left.o.b"].shape == (width,) and names[p + "right.norm"].shape == (right["heads"] * right["vdim"],)
                assert p + "left.q.norm" not in names
            else:
                left, right = m["left"], m["right"]
                pages, conv_state = inner[0]
                channels = (left["heads"] + left["kv_heads"]) * left["dim"] + left["kv_heads"] * left["vdim"]
                assert model.cache_groups[conv_state.group].need == StateNeed(((left["conv"] - 1) * channels,), torch.float32)
                delta_channels = 2 * right["kv_heads"] * right["dim"] + right["heads"] * right["vdim"]
                assert model.cache_groups[inner[1].group].need == StateNeed(
                    ((right["conv"] - 1) * delta_channels + right["heads"] * right["vdim"] * right["dim"],), torch.float32)
                assert names[p + "left.g"].shape == (left["heads"] * left["vdim"], width)
                assert names[p + "right.a2"].shape == (right["heads"] * right["dim"], right["decay_rank"])
                assert names[p + "right.g1"].shape == (right["gate_rank"], width) and names[p + "right.dt_bias"].shape == (right["heads"] * right["dim"],)
                assert names[p + "left.out"].shape == (width,) and names[p + "right.norm"].shape == (right["vdim"],)
            assert (f"l{run.layer}.ls2" in names) == (entry["mlp"] is not None) == (f"l{run.layer}.norm2" in names)
        # every run of a layer, repeated or not, has a state of its own for its shifted input
        assert len(shift_groups) == 1 and model.cache_groups[shift_groups.pop()].n_slots == len(spec.order)
        if "bigram" in raw["embedding"]:
            assert names["bigram"].shape == (raw["embedding"]["bigram"]["buckets"] + 1, width)
            assert model.cache_groups[model.embedding_caches[0].group].need == StateNeed((1,), torch.int32)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][1].__setitem__("type", "hyena"), "not implemented"),
    (lambda c: c["layers"][1]["mixer"]["left"].__setitem__("heads", 7), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].__setitem__("dims", 26), "exceeds the head size"),
    (lambda c: c["layers"][1]["mixer"]["right"].__setitem__("decay", [0.5, 0.6]), "one finite number"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("kv_heads", 3), "multiple of"),
    (lambda c: c["layers"][2]["mixer"]["mask"].__setitem__("size", 0), "positive"),
    (lambda c: c["layers"][2]["mlp"].__setitem__("kind", "sparse"), "not implemented"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
    (lambda c: c.__delitem__("residual_mult"), "residual_mult"),
    (lambda c: c["embedding"].__delitem__("scale"), "scale"),
    (lambda c: c["norm"].__setitem__("eps", 0.0), "positive"),
])
def test_configuration_refuses_what_it_cannot_run(change, message):
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import resolve_architecture

    raw = copy.deepcopy(bh.BAFAVIK_A)
    change(raw)
    with pytest.raises(ValueError, match=message):
        resolve_architecture(raw).config_class.from_dict(raw)


def test_sizes_that_only_the_tensors_give(tmp_path):
    """A stored configuration does not name the inner sizes of the delta rule's two-step projections; the folder's tensor
    shapes give them, and without either the model cannot be described."""
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import load_model_config, resolve_architecture

    folder = bh.make_folder(tmp_path, "a", seed=1)
    stored = json.loads((folder / "config.json").read_text())
    assert "decay_rank" not in stored["layers"][0]["mixer"]["right"]
    architecture, config = load_model_config(folder)
    right = config.layers[0].mixer.right
    assert (right.decay_rank, right.gate_rank) == (5, 7)
    architecture.build_spec(config)
    with pytest.raises(ValueError, match="decay_rank"):
        architecture.build_spec(resolve_architecture(stored).config_class.from_dict(stored))


def test_plain_mechanisms_one_by_one():
    """The oracle against itself and on hand-made numbers: a prefix's outputs do not change when the sequence goes on; the
    recurrences remember; a differential row sees exactly its chunk; the shift and the token-pair rows look one token back."""
    torch.manual_seed(0)
    width, T, eps = 16, 40, 1e-5
    h = torch.randn(T, width, dtype=plain.F64)

    def tensors(shapes, scale=0.4):
        return {"x." + name: torch.randn(shape, dtype=plain.F64) * scale for name, shape in shapes.items()}

    d = dict(heads=4, kv_heads=2, dim=6, vdim=3, conv=3)
    wd = tensors({"q": (12, width), "q.conv": (12, 3), "k": (12, width), "k.conv": (12, 3), "v": (12, width), "v.conv": (12, 3), "b": (4, width),
                  "A_log": (4,), "norm": (3,), "a1": (2, width), "a2": (24, 2), "dt_bias": (24,), "g1": (3, width), "g2": (12, 3), "o": (width, 12)})
    wd["x.A_log"] -= 3.0
    li = dict(heads=2, dim=5, vdim=4, decay=[0.9, 0.99])
    wl = tensors({"q": (10, width), "k": (10, width), "v": (8, width), "g": (8, width), "o": (width, 8), "norm": (8,)})
    for run in (lambda x: plain.gated_delta_rule(x, wd, "x.", d, eps), lambda x: plain.lightning_attention(x, wl, "x.", li, eps)):
        whole = run(h)
        assert torch.allclose(run(h[:17]), whole[:17], atol=1e-12)
        changed = h.clone()
        changed[20] += 1.0
        assert torch.allclose(run(changed)[:20], whole[:20], atol=1e-12)
        assert not torch.allclose(run(changed)[33], whole[33], atol=1e-7)                 # the state remembers
    # a decay per key CHANNEL is not a decay per head: with the channels' decays replaced by their mean the outputs change
    a = dict(heads=4, kv_heads=2, dim=6, vdim=5, scale=0.4, diff=0.3, mask=dict(size=9))
    wa = tensors({"q": (48, width), "q.b": (48,), "k": (24, width), "k.b": (24,), "v": (10, width), "v.b": (10,), "g": (20, width), "o": (width, 20),
                  "lq1": (6,), "lk1": (6,), "lq2": (6,), "lk2": (6,)})
    whole = plain.differential_attention(h, wa, "x.", a, eps)
    changed = h.clone()
    changed[10] += 1.0                                       # position 10 lies in the chunk 9 .. 17
    after = plain.differential_attention(changed, wa, "x.", a, eps)
    assert torch.allclose(after[:10], whole[:10], atol=1e-12) and torch.allclose(after[18:], whole[18:], atol=1e-12)
    assert all(not torch.allclose(after[t], whole[t], atol=1e-7) for t in range(10, 18))
    # with lambda = 0 (diff 0, equal vectors) and one map, the layer is an ordinary attention, normed per head
    plain_rows = plain.softmax_attention(h[:, :12].reshape(T, 2, 6), h[:, :6].reshape(T, 1, 6), h[:, 6:11].reshape(T, 1, 5), 0.4, 9)
    assert torch.allclose(plain_rows[8, 0], plain.softmax_attention(h[:9, :12].reshape(9, 2, 6), h[:9, :6].reshape(9, 1, 6),
                                                                    h[:9, 6:11].reshape(9, 1, 5), 0.4, None)[8, 0])
    assert torch.allclose(plain_rows[9, 0], h[9, 6:11])      # the first token of a chunk sees itself alone
    # the shift: the first token moves towards zero, the others towards the token before as it was
    shift = torch.rand(width, dtype=plain.F64)
    shifted = plain.token_shift(h, shift)
    assert torch.allclose(shifted[0], h[0] * (1 - shift)) and torch.allclose(shifted[5], h[5] + (h[4] - h[5]) * shift)
    # the rotation: both layouts turn pairs by the same angles and leave the entries behind `dims` alone
    v = torch.randn(7, 2, 8, dtype=plain.F64)
    half, inter = plain.rotate(v, 4, 50.0, False), plain.rotate(v, 4, 50.0, True)
    assert torch.allclose(half[..., 4:], v[..., 4:]) and torch.allclose(inter[..., 4:], v[..., 4:]) and torch.allclose(half[0], v[0])
    angle = 3 * 50.0 ** (-2.0 / 4)
    assert torch.allclose(half[3, :, 1], v[3, :, 1] * torch.cos(torch.tensor(angle)) - v[3, :, 3] * torch.sin(torch.tensor(angle)))
    assert torch.allclose(inter[3, :, 2], v[3, :, 2] * torch.cos(torch.tensor(angle)) - v[3, :, 3] * torch.sin(torch.tensor(angle)))
    assert torch.allclose(v.pow(2).sum(-1), half.pow(2).sum(-1)) and torch.allclose(v.pow(2).sum(-1), inter.pow(2).sum(-1))
    # token pairs: the first token takes the table's last row, the others the hashed row
    config = dict(embedding=dict(scale=2.0, bigram=dict(buckets=7, mul_prev=3, mul_cur=5)))
    w = {"embed": torch.randn(20, 4, dtype=plain.F64), "bigram": torch.randn(8, 4, dtype=plain.F64)}
    x = plain.embed([4, 9, 9], w, config)
    assert torch.allclose(x[0], 2.0 * w["embed"][4] + w["bigram"][7])
    assert torch.allclose(x[1], 2.0 * w["embed"][9] + w["bigram"][(4 * 3 + 9 * 5) % 7])
    assert torch.allclose(x[2], 2.0 * w["embed"][9] + w["bigram"][(9 * 3 + 9 * 5) % 7])


@pytest.fixture
def cpu_runtime(monkeypatch, tmp_path):
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import EngineConfig
    from miniserve_b200.engine import runtime as runtime_module

    plain_ops.install(monkeypatch)
    monkeypatch.setattr(runtime_module, "require_device", lambda device: torch.device("cpu"))
    monkeypatch.setattr(runtime_module.kernels, "library", lambda: None)
    monkeypatch.setattr(torch.cuda, "set_device", lambda device: None)

    def build(name, num_pages, page_size, max_seqs=4):
        folder = bh.make_folder(tmp_path, name, seed=2)
        runtime = runtime_module.build_runtime(folder, EngineConfig(
            dtype="float32", kv_block_size=page_size, num_kv_blocks=num_pages, max_num_seqs=max_seqs,
            enable_prefix_cache=True, device="cpu", decode_execution="eager"))
        return folder, runtime
    return build


@pytest.mark.parametrize("name,page_size", [("a", 8), ("b", 4), ("d", 16)])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_cuttings_match_plain_on_cpu(cpu_runtime, name, page_size, cutting):
    from miniserve_b200.trace import TraceSession

    vocab = bh.CONFIGS[name]["vocab"]
    requests = {f"r{i}": helpers.random_tokens(vocab, n, seed=20 + i) for i, n in enumerate((1, 6, 17, 30, 41))}
    steps = {"whole": helpers.cut_whole, "tail": lambda r: helpers.cut_decode_tail(r, 9),
             "portions": helpers.cut_portions, "mixed": helpers.cut_mixed}[cutting](requests)
    pages = (helpers.max_live_tokens(steps, granule=page_size * 2) + page_size - 1) // page_size
    folder, runtime = cpu_runtime(name, pages, page_size)
    assert runtime.max_model_len == pages * page_size            # no position limit of the design's own: the pool's size
    assert runtime.manager.prefix is None                        # a model with per-request state shares no pages
    session, outputs = TraceSession(runtime), {}
    for record in steps:
        outputs[record["step"]] = session.run(record).double()
        runtime.manager.check_invariants()
    got = helpers.collect(steps, outputs)
    config, weights = bh.load_folder(folder)
    for rid, tokens in requests.items():
        expected = plain.forward(tokens, weights, config)
        assert sorted(got[rid]) == list(range(len(tokens)))
        for position, row in got[rid].items():
            assert torch.allclose(row, expected[position], atol=2e-4, rtol=2e-4), (rid, position)
    assert not runtime.manager.requests
    assert all(a.free_count == a.num_pages for a in runtime.manager.allocators)


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations_on_cpu(cpu_runtime, tmp_path, seed):
    """Layer kinds, orders, head counts, sizes, taps, chunks and repeated runs drawn at random, in a cutting and with a page
    size drawn with them."""
    import random

    from miniserve_b200.trace import TraceSession

    rng = random.Random(seed)
    config = bh.random_config(rng)
    bh.CONFIGS[f"random{seed}"] = config
    try:
        page_size = rng.choice([4, 8, 16])
        requests = {f"r{i}": helpers.random_tokens(config["vocab"], n, seed=20 + i) for i, n in enumerate((1, 6, 17, 30, 41))}
        cutting = rng.choice(["tail", "portions", "mixed"])
        steps = {"tail": lambda r: helpers.cut_decode_tail(r, 9), "portions": helpers.cut_portions, "mixed": helpers.cut_mixed}[cutting](requests)
        pages = (helpers.max_live_tokens(steps, granule=page_size * 2) + page_size - 1) // page_size
        folder, runtime = cpu_runtime(f"random{seed}", pages, page_size)
    finally:
        del bh.CONFIGS[f"random{seed}"]
    session, outputs = TraceSession(runtime), {}
    for record in steps:
        outputs[record["step"]] = session.run(record).double()
        runtime.manager.check_invariants()
    got = helpers.collect(steps, outputs)
    stored, weights = bh.load_folder(folder)
    for rid, tokens in requests.items():
        expected = plain.forward(tokens, weights, stored)
        for position, row in got[rid].items():
            assert torch.allclose(row, expected[position], atol=3e-4, rtol=3e-4), (seed, rid, position)


def test_pages_behind_a_chunk_are_given_back():
    """A paged group under a chunked mask keeps the pages of the chunk that the next token lies in and gives back those
    wholly before it."""
    import miniserve_b200  # noqa: F401
    from miniserve_b200.cache import CacheManager
    from miniserve_b200.cache.manager import RELEASED
    from miniserve_b200.parts import CacheGroup, PagedKVNeed

    need = PagedKVNeed(2, 8, None, None, 10)
    assert [need.first_needed(p) for p in (0, 9, 10, 25)] == [0, 0, 10, 20] and not need.keeps_all
    manager = CacheManager([CacheGroup(need, 1)], 4, 16, 2)
    manager.admit("r")
    for count, released in ((9, 0), (1, 2), (13, 5), (1, 5), (6, 7)):      # lengths 9, 10, 23, 24, 30: chunk starts 0, 10, 20, 20, 30
        manager.commit(manager.prepare([("r", count)]))
        table = manager.requests["r"].tables[0]
        assert [page == RELEASED for page in table] == [index < released for index in range(len(table))], (count, table)
        manager.check_invariants()
    manager.release("r")
    assert manager.allocators[0].free_count == 16
