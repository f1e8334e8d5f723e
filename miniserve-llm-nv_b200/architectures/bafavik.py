"""Bafavik: a decoder whose layers, in an order that ``config.json`` gives and with a run of them repeated (``loop``), carry
one of three mixers: softmax attention (biases, a half-split rotation, weightless norms of queries and keys) beside a linear
attention with a constant decay per head; differential attention under a chunked mask with a gate per entry; softmax attention
behind short convolutions (interleaved rotation, a gate per entry) beside the gated delta rule with a decay per key channel,
the two outputs normed and averaged.  Every mixer reads its input shifted towards the token before; what a sublayer adds is
multiplied by a constant and by a vector of the layer; the feed-forward is ``down(relu(up(x))^2)``.  Token embeddings are
scaled and receive a row of a hashed table of token pairs; logits are scaled.

Tensor names: ``embed``, ``bigram``, ``final.norm``, ``head`` and, for layer i, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1``,
``l<i>.ls2``, ``l<i>.shift``, ``l<i>.mlp.{up,down}`` and ``l<i>.mix.*`` as the mixers' parts declare them.
"""

from __future__ import annotations

from ..config.model_config import BafavikConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerRun, LayerSpec, ModelSpec, PartSpec

# The design gives positions no upper limit; this is the engine's own bound on a request's length (it sizes the block
# tables of captured decode steps), which `max_model_len` lowers.
NOMINAL_MAX_POSITIONS = 131072


def _rotation(m, interleaved: bool) -> PartSpec:
    if m.rot.dims == 0:
        return PartSpec("none")
    return PartSpec("rope", dict(head_dim=m.dim, theta=m.rot.base, rotary_dim=m.rot.dims, interleaved=interleaved,
                                 frequencies="float64"))


def _mixer(kind: str, m, width: int, eps: float, where: str) -> PartSpec:
    """The mixer of a layer; its tensor names start with ``mix.``."""
    if kind == "attention":
        return PartSpec("differential_attention", dict(
            hidden_size=width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, scale=m.scale,
            diff=m.diff, eps=eps, chunk=m.chunk, bias=True, output_gate=True, q_name="mix.q", k_name="mix.k", v_name="mix.v",
            o_name="mix.o", gate_name="mix.g", lq1_name="mix.lq1", lk1_name="mix.lk1", lq2_name="mix.lq2", lk2_name="mix.lk2"))
    left, right = m.left, m.right
    if kind == "parallel":
        attention = PartSpec("attention", dict(
            hidden_size=width, num_heads=left.heads, num_kv_heads=left.kv_heads, head_dim=left.dim, value_dim=left.vdim,
            qk_norm=True, qk_norm_weight=False, eps=eps, position=_rotation(left, False), scale=left.scale, bias=True,
            q_name="q", k_name="k", v_name="v", o_name="o"))
        linear = PartSpec("linear_attention", dict(
            hidden_size=width, heads=right.heads, head_dim=right.dim, value_dim=right.vdim, decay=right.decay, eps=eps))
        return PartSpec("side_by_side", dict(members=(("mix.left.", attention, m.left_scale), ("mix.right.", linear, m.right_scale))))
    if right.decay_rank is None or right.gate_rank is None:
        raise ValueError(f"{where}mixer.right: the inner sizes of the decay's and the gate's two-step projections come from "
                         "'decay_rank' and 'gate_rank' or from the shapes of the checkpoint's tensors; neither was given")
    attention = PartSpec("attention", dict(
        hidden_size=width, num_heads=left.heads, num_kv_heads=left.kv_heads, head_dim=left.dim, value_dim=left.vdim,
        qk_norm=False, eps=eps, position=_rotation(left, True), scale=left.scale, output_gate="entry", conv_taps=left.conv,
        q_name="q", k_name="k", v_name="v", o_name="o", gate_name="g"))
    delta = PartSpec("delta_rule", dict(
        hidden_size=width, heads=right.heads, kv_heads=right.kv_heads, head_dim=right.dim, value_dim=right.vdim, taps=right.conv,
        eps=eps, decay_per="channel", decay_rank=right.decay_rank, gate_rank=right.gate_rank, gate_activation="sigmoid"))
    return PartSpec("side_by_side", dict(members=(("mix.left.", attention, 0.5), ("mix.right.", delta, 0.5)),
                                         output_norms=("mix.left.out", "mix.right.out"), hidden_size=width, eps=eps))


def build_bafavik_spec(config: BafavikConfig) -> ModelSpec:
    width, eps = config.width, config.eps

    def stream_norm(name: str) -> PartSpec:
        return PartSpec("rms", dict(name=name, size=width, eps=eps, one_plus=True))

    layers, unused = [], []
    for index, layer in enumerate(config.layers):
        mixer = PartSpec("token_shift", dict(hidden_size=width, inner=_mixer(layer.type, layer.mixer, width, eps, f"layers[{index}]."),
                                             shift_name="shift"))
        feed_forward = None if layer.ff is None else PartSpec("mlp", dict(
            hidden_size=width, intermediate_size=layer.ff, activation="relu_square", up_name="mlp.up", down_name="mlp.down"))
        prefix = f"l{index}."
        layers.append(LayerSpec(
            prefix=prefix, mixer=mixer, feed_forward=feed_forward, mixer_norm=stream_norm("norm1"),
            feed_forward_norm=None if feed_forward is None else stream_norm("norm2"),
            block=PartSpec("scaled_pre_norm", dict(
                hidden_size=width, residual_scale=config.residual_mult, mixer_scale_name=prefix + "ls1",
                feed_forward_scale_name=None if feed_forward is None else prefix + "ls2"))))
        if feed_forward is None:
            unused += [prefix + "norm2", prefix + "ls2"]        # a checkpoint may carry them although nothing reads them
    n = len(layers)
    if config.loop is None:
        runs = list(range(n))
    else:
        start, stop, times = config.loop
        runs = list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))
    extra = ()
    if config.bigram is not None:
        extra = (PartSpec("token_pair", dict(name="bigram", hidden_size=width, buckets=config.bigram.buckets,
                                             mul_prev=config.bigram.mul_prev, mul_cur=config.bigram.mul_cur)),)
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=width, embedding_name="embed", layers=tuple(layers),
        order=tuple(LayerRun(index) for index in runs), final_norm=stream_norm("final.norm"), output_name="head",
        max_positions=NOMINAL_MAX_POSITIONS, nominal_max_positions=True, optional_names=tuple(unused),
        embedding_scale=config.embedding_scale, logit_scale=config.logit_scale, extra_embeddings=extra)


register_architecture("Bafavik", BafavikConfig, build_bafavik_spec)
