"""Kivurax: a decoder whose layers, in an order that ``config.json`` gives, carry one of three mixers (a matrix memory with
exponential gates; a windowed attention whose values are its keys beside a gated linear recurrence; the gated delta rule)
and a feed-forward that is a gated layer with biases or a mixture of gated experts with sigmoid scores that weight the
experts' inputs.  A sublayer reads the residual stream itself; only its output is normed, and what it adds is damped:
``x <- x + m * norm(sublayer(x))``.  The output matrix is the embedding table.

``config.json`` lists the layers one by one; tensor names are ``embed``, ``final.norm`` and, for layer i, ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.{q,k,v,g,o,norm,i,i.b,f,f.b}`` or ``l<i>.mix.left.{q,k,q.norm,k.norm,o}`` with
``l<i>.mix.right.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o}`` or
``l<i>.mix.{q,q.conv,k,k.conv,v,v.conv,b,a,A_log,dt_bias,g,norm,o}``, and ``l<i>.mlp.{gate,gate.b,up,up.b,down,down.b}`` or
``l<i>.mlp.{router,e<j>.gate,e<j>.up,e<j>.down}``.
"""

from __future__ import annotations

from ..config.model_config import KivuraxConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerRun, LayerSpec, ModelSpec, PartSpec

# The design gives positions no upper limit; this is the engine's own bound on a request's length (it sizes the block
# tables of captured decode steps), which `max_model_len` lowers.
NOMINAL_MAX_POSITIONS = 131072


def _mixer(kind: str, m, width: int, eps: float) -> PartSpec:
    """The mixer of a layer; its tensor names start with ``mix.``."""
    if kind == "mlstm":
        return PartSpec("matrix_memory", dict(
            hidden_size=width, heads=m.heads, head_dim=m.dim, value_dim=m.vdim, gate_cap=m.gate_cap, eps=eps,
            q_name="mix.q", k_name="mix.k", v_name="mix.v", g_name="mix.g", o_name="mix.o", norm_name="mix.norm",
            i_name="mix.i", i_bias_name="mix.i.b", f_name="mix.f", f_bias_name="mix.f.b"))
    if kind == "delta":
        return PartSpec("delta_rule", dict(
            hidden_size=width, heads=m.heads, kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, taps=m.conv, eps=eps,
            q_name="mix.q", k_name="mix.k", v_name="mix.v", b_name="mix.b", a_name="mix.a", a_log_name="mix.A_log",
            dt_bias_name="mix.dt_bias", g_name="mix.g", norm_name="mix.norm", o_name="mix.o"))
    left, right = m.left, m.right
    position = PartSpec("none") if left.rot.dims == 0 else PartSpec(
        "rope", dict(head_dim=left.dim, theta=left.rot.base, rotary_dim=left.rot.dims, interleaved=True,
                     scaling=left.rot.scaling_dict(), frequencies="float64"))
    attention = PartSpec("attention", dict(
        hidden_size=width, num_heads=left.heads, num_kv_heads=left.kv_heads, head_dim=left.dim, qk_norm=True, eps=eps,
        position=position, window=left.window, scale=left.scale, sink=True, values_from_keys=True,
        q_name="q", k_name="k", o_name="o", q_norm_name="q.norm", k_norm_name="k.norm"))
    recurrence = PartSpec("gated_linear_recurrence", dict(hidden_size=width, width=right.width, blocks=right.blocks, taps=right.conv))
    return PartSpec("side_by_side", dict(members=(("mix.left.", attention, m.left_scale), ("mix.right.", recurrence, m.right_scale))))


def build_kivurax_spec(config: KivuraxConfig) -> ModelSpec:
    width, eps = config.width, config.eps
    layers, order, unused = [], [], []
    for index, layer in enumerate(config.layers):
        mixer = _mixer(layer.type, layer.mixer, width, eps)
        feed_forward = None
        if layer.mlp is not None and layer.mlp.kind == "dense":
            feed_forward = PartSpec("gated_mlp", dict(
                hidden_size=width, intermediate_size=layer.mlp.ff, bias=True, gate_name="mlp.gate", up_name="mlp.up",
                down_name="mlp.down", gate_bias_name="mlp.gate.b", up_bias_name="mlp.up.b", down_bias_name="mlp.down.b"))
        elif layer.mlp is not None:
            feed_forward = PartSpec("routed_experts", dict(
                hidden_size=width, experts=layer.mlp.experts, top=layer.mlp.top, expert_size=layer.mlp.ff, router_bias=False,
                activation="silu_glu", scoring="sigmoid", weight_on="input", router_name="mlp.router",
                expert_name="mlp.e{index}."))
        through = PartSpec("identity", dict(size=width))
        layers.append(LayerSpec(
            prefix=f"l{index}.", mixer=mixer, feed_forward=feed_forward, mixer_norm=through,
            feed_forward_norm=None if feed_forward is None else through,
            block=PartSpec("sandwich", dict(residual_scale=config.residual_mult)),
            mixer_post_norm=PartSpec("rms", dict(name="norm1", size=width, eps=eps)),
            feed_forward_post_norm=None if feed_forward is None else PartSpec("rms", dict(name="norm2", size=width, eps=eps))))
        order.append(LayerRun(index))
        if feed_forward is None:
            unused.append(f"l{index}.norm2")        # a checkpoint may carry it although nothing reads it
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=width, embedding_name="embed", layers=tuple(layers), order=tuple(order),
        final_norm=PartSpec("rms", dict(name="final.norm", size=width, eps=eps)), output_name=None,
        max_positions=NOMINAL_MAX_POSITIONS, nominal_max_positions=True, optional_names=tuple(unused))


register_architecture("Kivurax", KivuraxConfig, build_kivurax_spec)
