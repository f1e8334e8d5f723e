"""Kivurax without a GPU: its configuration, what it declares, the plain implementation's own consistency, and the host-side
logic (parts, block, caches of a mixer made of two, state slots, step function) on the CPU with plain PyTorch functions
standing in for the kernels, in every cutting, against the plain implementation."""

from __future__ import annotations

import copy

import pytest
import torch

import helpers
import kivurax_helpers as kh
import plain_kivurax as plain
import plain_ops


def test_configuration_reads_every_size_and_round_trips():
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import KivuraxConfig, resolve_architecture
    from miniserve_b200.parts import DecoderModel, PagedKVNeed, StateNeed

    for name, raw in kh.CONFIGS.items():
        architecture = resolve_architecture(raw)
        config = architecture.config_class.from_dict(raw)
        assert isinstance(config, KivuraxConfig) and config.to_dict() == raw
        spec = architecture.build_spec(config)
        assert spec.output_name is None and spec.vocab_size == raw["vocab"]          # the output matrix is the embedding
        assert all(l.block.kind == "sandwich" and l.block.args["residual_scale"] == raw["residual_mult"] for l in spec.layers)
        assert all(l.mixer_norm.kind == "identity" and l.mixer_post_norm.kind == "rms" for l in spec.layers)
        model = DecoderModel(spec, torch.float32, "cpu")
        names = {s.name: s for s in model.param_specs()}
        for index, (entry, plan) in enumerate(zip(raw["layers"], model.run_caches)):
            m, mixer = entry["mixer"], model.blocks[index].mixer
            p = f"l{index}.mix."
            if entry["type"] == "mlstm":
                assert mixer.cache_need() == StateNeed((m["heads"] * (m["vdim"] + 1) * m["dim"] + m["heads"],), torch.float32)
                assert names[p + "v"].shape == (m["heads"] * m["vdim"], raw["width"]) and names[p + "i.b"].shape == (m["heads"],)
            elif entry["type"] == "delta":
                channels = 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"]
                assert mixer.cache_need() == StateNeed(((m["conv"] - 1) * channels + m["heads"] * m["vdim"] * m["dim"],), torch.float32)
                assert names[p + "k.conv"].shape == (m["kv_heads"] * m["dim"], m["conv"]) and names[p + "norm"].shape == (m["vdim"],)
            else:
                left, right = m["left"], m["right"]
                assert mixer.cache_need() == (PagedKVNeed(left["kv_heads"], left["dim"], left["mask"]["size"], None),
                                              StateNeed((right["conv"] * right["width"],), torch.float32))
                assert isinstance(plan, tuple) and len(plan) == 2 and plan[0].group != plan[1].group
                assert p + "left.v" not in names and names[p + "left.k.norm"].shape == (left["dim"],)
                assert names[p + "right.ra"].shape == (right["blocks"], right["width"] // right["blocks"], right["width"] // right["blocks"])
            assert (f"l{index}.norm2" in names) == (entry["mlp"] is not None)
            if entry["mlp"] and entry["mlp"]["kind"] == "moe":
                experts = entry["mlp"]["router"]["experts"]
                assert names[f"l{index}.mlp.router"].shape == (experts, raw["width"])
                assert f"l{index}.mlp.e{experts - 1}.gate" in names and f"l{index}.mlp.e{experts}.gate" not in names
            elif entry["mlp"]:
                assert names[f"l{index}.mlp.down.b"].shape == (raw["width"],)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][1].__setitem__("type", "hyena"), "not implemented"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("heads", 7), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("vdim", 16), "values are the keys"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 26), "exceeds the head size"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("blocks", 5), "does not divide"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_heads", 4), "multiple of"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("gate_cap", 0.0), "positive"),
    (lambda c: c["layers"][3]["mlp"]["router"].__setitem__("top", 6), "exceeds"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "sparse"), "not implemented"),
    (lambda c: c.__delitem__("residual_mult"), "residual_mult"),
    (lambda c: c["norm"].__setitem__("eps", 0.0), "positive"),
])
def test_configuration_refuses_what_it_cannot_run(change, message):
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import resolve_architecture

    raw = copy.deepcopy(kh.KIVURAX_A)
    change(raw)
    with pytest.raises(ValueError, match=message):
        resolve_architecture(raw).config_class.from_dict(raw)


def test_plain_recurrences_are_the_same_in_one_pass_and_in_two():
    """The oracle against itself: a prefix's outputs do not change when the sequence goes on, a change far back reaches the
    present through the state, and an attention row sees exactly its window."""
    torch.manual_seed(0)
    width, T = 16, 40
    h = torch.randn(T, width, dtype=plain.F64)

    def tensors(shapes, scale=0.4):
        return {"x." + name: torch.randn(shape, dtype=plain.F64) * scale for name, shape in shapes.items()}

    m = dict(heads=2, dim=6, vdim=5, gate_cap=7.0)
    w = tensors({"q": (12, width), "k": (12, width), "v": (10, width), "g": (10, width), "o": (width, 10), "norm": (10,), "i": (2, width),
                 "i.b": (2,), "f": (2, width), "f.b": (2,)})
    w["x.f.b"] += 3.0
    d = dict(heads=4, kv_heads=2, dim=6, vdim=3, conv=3)
    wd = tensors({"q": (12, width), "q.conv": (12, 3), "k": (12, width), "k.conv": (12, 3), "v": (12, width), "v.conv": (12, 3), "b": (4, width),
                  "A_log": (4,), "norm": (3,), "a": (4, width), "dt_bias": (4,), "g": (12, width), "o": (width, 12)})
    wd["x.A_log"] -= 2.0
    r = dict(width=12, blocks=3, conv=4)
    wr = tensors({"y": (12, width), "y.b": (12,), "x": (12, width), "x.b": (12,), "conv": (12, 4), "conv.b": (12,), "ra": (3, 4, 4), "ra.b": (3, 4),
                  "ri": (3, 4, 4), "ri.b": (3, 4), "lam": (12,), "o": (width, 12)})
    wr["x.lam"] -= 3.0
    for run in (lambda x: plain.mlstm(x, w, "x.", m, 1e-5), lambda x: plain.delta_rule(x, wd, "x.", d, 1e-5),
                lambda x: plain.gated_linear_recurrence(x, wr, "x.", r)):
        whole = run(h)
        assert torch.allclose(run(h[:17]), whole[:17], atol=1e-12)
        changed = h.clone()
        changed[20] += 1.0
        assert torch.allclose(run(changed)[:20], whole[:20], atol=1e-12)
        assert not torch.allclose(run(changed)[33], whole[33], atol=1e-7)                 # the state remembers
    a = dict(heads=4, kv_heads=2, dim=6, vdim=6, scale=0.4, mask=dict(size=9), rot=kh.rot(50.0, 4, (2.0, 16, 4.0, 1.0)))
    wa = tensors({"q": (24, width), "k": (12, width), "q.norm": (6,), "k.norm": (6,), "o": (width, 24)})
    whole = plain.window_attention(h, wa, "x.", a, 1e-5)
    changed = h.clone()
    changed[10] += 1.0
    after = plain.window_attention(changed, wa, "x.", a, 1e-5)
    assert torch.allclose(after[19:], whole[19:], atol=1e-12) and not torch.allclose(after[18], whole[18], atol=1e-7)
    assert torch.allclose(after[:10], whole[:10], atol=1e-12)


def test_plain_sink_and_weights_on_the_experts_input():
    """A lone key of score 0 shares the softmax with the sink (weight one half); an expert reads its weight times the input,
    which is not the weight times its output."""
    width = 8
    a = dict(heads=1, kv_heads=1, dim=4, vdim=4, scale=1.0, mask=dict(size=4), rot=kh.rot(10.0, 0))
    wa = {"x.q": torch.zeros(4, width, dtype=plain.F64), "x.k": torch.eye(4, width, dtype=plain.F64), "x.q.norm": torch.ones(4, dtype=plain.F64),
          "x.k.norm": torch.ones(4, dtype=plain.F64), "x.o": torch.eye(width, 4, dtype=plain.F64)}
    h = torch.zeros(1, width, dtype=plain.F64)
    h[0, :4] = torch.tensor([1.0, 2.0, 3.0, 4.0])
    out = plain.window_attention(h, wa, "x.", a, 1e-5)
    assert torch.allclose(out[0, :4], 0.5 * h[0, :4])              # the values are the keys as projected, not normed
    mlp = dict(kind="moe", expert=dict(ff=3), router=dict(experts=2, top=1))
    g = torch.Generator().manual_seed(1)
    w = {"f.router": torch.tensor([[2.0] + [0.0] * (width - 1), [0.0] * width], dtype=plain.F64)}
    for e in range(2):
        w[f"f.e{e}.gate"] = torch.randn(3, width, generator=g, dtype=plain.F64)
        w[f"f.e{e}.up"] = torch.randn(3, width, generator=g, dtype=plain.F64)
        w[f"f.e{e}.down"] = torch.randn(width, 3, generator=g, dtype=plain.F64)
    x = torch.randn(1, width, generator=g, dtype=plain.F64).abs()
    ids, weights, gap = plain.route(x, w, "f.", mlp)
    assert ids.tolist() == [[0]] and gap > 0 and 0.5 < float(weights[0, 0]) < 1.0
    scaled = weights[0, 0] * x[0]
    inside = (plain.silu(w["f.e0.gate"] @ scaled) * (w["f.e0.up"] @ scaled)) @ w["f.e0.down"].T
    outside = weights[0, 0] * ((plain.silu(w["f.e0.gate"] @ x[0]) * (w["f.e0.up"] @ x[0])) @ w["f.e0.down"].T)
    got = plain.mixture(x, w, "f.", mlp)[0]
    assert torch.allclose(got, inside) and not torch.allclose(got, outside, atol=1e-6)


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
        folder = kh.make_folder(tmp_path, name, seed=2)
        runtime = runtime_module.build_runtime(folder, EngineConfig(
            dtype="float32", kv_block_size=page_size, num_kv_blocks=num_pages, max_num_seqs=max_seqs,
            enable_prefix_cache=True, device="cpu", decode_execution="eager"))
        return folder, runtime
    return build


@pytest.mark.parametrize("name,page_size", [("a", 8), ("b", 4), ("d", 8), ("e", 16)])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_cuttings_match_plain_on_cpu(cpu_runtime, name, page_size, cutting):
    from miniserve_b200.trace import TraceSession

    vocab = kh.CONFIGS[name]["vocab"]
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
    config, weights = plain.load_folder(folder)
    for index, entry in enumerate(config["layers"]):
        if entry["mlp"] and entry["mlp"]["kind"] == "moe" and entry["mlp"]["router"]["top"] < entry["mlp"]["router"]["experts"]:
            assert plain.route(weights["embed"], weights, f"l{index}.mlp.", entry["mlp"])[2] > 0.02      # the marks decide
    for rid, tokens in requests.items():
        expected = plain.forward(tokens, weights, config)
        assert sorted(got[rid]) == list(range(len(tokens)))
        for position, row in got[rid].items():
            assert torch.allclose(row, expected[position], atol=2e-4, rtol=2e-4), (rid, position)
    assert not runtime.manager.requests
    assert all(a.free_count == a.num_pages for a in runtime.manager.allocators)
