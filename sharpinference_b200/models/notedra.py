"""The Notedra architecture, put together from parts, and its tensor names.

A decoder of *parallel* layers: one norm per layer (RMS norm whose weight is stored around zero and applied as
``1 + w``), whose output both the mixer and the feed-forward read; ``x += mixer(h) + ff(h)``.  Per layer
(``config.layers[i]``, every layer with sizes of its own):

* mixer ``mlstm``: the matrix-memory recurrence (:class:`MLSTMMixer`), gates capped by ``gate_cap``;
* mixer ``attention``: grouped-query attention with a sliding window of ``mask.size`` positions, interleaved-pair
  rotation of the first ``rot.dims`` elements of every head, the weightless RMS norm of q and k per head after the
  rotation, the score factor ``scale``, value heads of size ``vdim``;
* feed-forward: none, a dense network with biases, or a sigmoid-routed mixture of bias-free experts with a
  correction added to the scores for the choice only and weights ``router.scale * s`` that are not renormalised;
  the activation is the square of relu.

``config.loop`` runs layers ``start .. stop - 1`` ``times`` times with the same weights; every run has its own
cache or state (a schedule entry each), and before the first layer of pass ``t`` the stream becomes
``W_in [x ; x0] + step[t]`` with ``x0`` the embedding output (:class:`ReinjectInput`).  The output head is the
embedding table.

Tensor names (linear weights ``[out, in]``): ``embed``, ``final.norm``, ``loop.in [H, 2H]``, ``loop.step [times, H]``;
per layer ``l<i>.norm1``, ``l<i>.mix.{q,k,v,o}``, for mlstm also ``l<i>.mix.{g,norm,i,i.b,f,f.b}``;
``l<i>.mlp.{up,up.b,down,down.b}`` (dense) or ``l<i>.mlp.router``, ``l<i>.mlp.correction``,
``l<i>.mlp.e<j>.{up,down}`` (mixture).
"""
from __future__ import annotations

import torch

from ..config.notedra import NotedraConfig, NotedraLayer
from ..parts import (DenseMLP, GroupedLinear, L2Norm, Linear, MLSTMMixer, MoESigmoidTopK, PagedAttention, ParallelBlock,
                     ReinjectInput, RMSNorm, RotaryEncoding, fused_mlstm_columns, partial_rotary_inv_freq)
from ..registry import register_architecture
from ..weights.source import WeightSource
from .model import DecoderModel, ScheduleEntry


def _cat(tensors):
    if len({t.dtype for t in tensors}) > 1:      # one of them was stored in 32-bit: the fused product is 32-bit
        tensors = [t.to(torch.float32) for t in tensors]
    return torch.cat(tensors, dim=0).contiguous()


def _mlstm(c: NotedraConfig, layer: NotedraLayer, p: str, weights: WeightSource, act) -> MLSTMMixer:
    H, heads, d, dv = c.width, layer.heads, layer.dim, layer.vdim
    parts = [weights.matrix(p + "q", (heads * d, H)), weights.matrix(p + "k", (heads * d, H)),
             weights.matrix(p + "v", (heads * dv, H)), weights.matrix(p + "g", (heads * dv, H)),
             weights.matrix(p + "i", (heads, H)), weights.matrix(p + "f", (heads, H))]
    width = fused_mlstm_columns(heads, d, dv)[-1]
    rows = sum(t.shape[0] for t in parts)
    if width > rows:
        parts.append(torch.zeros((width - rows, H), dtype=parts[0].dtype, device=parts[0].device))
    return MLSTMMixer(proj=Linear(_cat(parts), p + "qkvgif"), out=Linear(weights.matrix(p + "o", (H, heads * dv)), p + "o"),
                      gate_bias_i=weights.vector(p + "i.b", (heads,), init="normal"),
                      gate_bias_f=weights.vector(p + "f.b", (heads,), init="normal"),
                      head_norm_weight=weights.vector(p + "norm", (heads * dv,)),
                      heads=heads, key_dim=d, value_dim=dv, gate_cap=layer.gate_cap, eps=c.eps, act_dtype=act)


def _attention(c: NotedraConfig, layer: NotedraLayer, p: str, weights: WeightSource, act) -> PagedAttention:
    H, nq, nkv, d, dv = c.width, layer.heads, layer.kv_heads, layer.dim, layer.vdim
    qkv = _cat([weights.matrix(p + "q", (nq * d, H)), weights.matrix(p + "k", (nkv * d, H)),
                weights.matrix(p + "v", (nkv * dv, H))])
    position = None
    if layer.rot_dims:
        inv_freq = partial_rotary_inv_freq(d, layer.rot_dims, layer.rot_base)
        position = RotaryEncoding(inv_freq if weights.device.type == "meta" else inv_freq.to(weights.device),
                                  "interleaved")
    return PagedAttention(qkv=Linear(qkv, p + "qkv"), out=Linear(weights.matrix(p + "o", (H, nq * dv)), p + "o"),
                          num_heads=nq, num_kv_heads=nkv, head_dim=d, value_dim=dv,
                          mask="window" if layer.window else "full", span=layer.window, position=position,
                          qk_norm=L2Norm(c.eps), softmax_scale=layer.scale, act_dtype=act)


def _feed_forward(c: NotedraConfig, layer: NotedraLayer, p: str, weights: WeightSource, act):
    m, H = layer.mlp, c.width
    if m is None:
        return None
    if m.kind == "dense":
        return DenseMLP(up=Linear(weights.matrix(p + "up", (m.ff, H)), p + "up",
                                  bias=weights.vector(p + "up.b", (m.ff,), init="normal")),
                        down=Linear(weights.matrix(p + "down", (H, m.ff)), p + "down",
                                    bias=weights.vector(p + "down.b", (H,), init="normal")),
                        activation="relu2", act_dtype=act)
    ups, downs = [], []
    for e in range(m.experts):                     # file order: e0.up, e0.down, e1.up, ...
        ups.append(weights.matrix(f"{p}e{e}.up", (m.ff, H)))
        downs.append(weights.matrix(f"{p}e{e}.down", (H, m.ff)))
    router = weights.vector(p + "router", (m.experts, H), init="normal")
    correction = weights.vector(p + "correction", (m.experts,), init="normal")
    return MoESigmoidTopK(router=router, correction=correction,
                          experts_up=GroupedLinear(torch.stack(ups).contiguous(), p + "experts.up"),
                          experts_down=GroupedLinear(torch.stack(downs).contiguous(), p + "experts.down"),
                          top_k=m.top, route_scale=m.route_scale, renormalize=False, activation="relu2",
                          act_dtype=act)


def build_notedra(config: NotedraConfig, weights: WeightSource) -> DecoderModel:
    c, act, H = config, weights.compute_dtype, config.width
    embedding = weights.matrix("embed", (c.vocab, H))
    stream_ops = []
    if c.loop_times:
        w_in = weights.matrix("loop.in", (H, 2 * H))
        steps = weights.vector("loop.step", (c.loop_times, H), init="normal")
        stream_ops = [ReinjectInput(proj=Linear(w_in, "loop.in", bias=steps[t].contiguous()), act_dtype=act)
                      for t in range(c.loop_times)]
    blocks = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        norm = RMSNorm(weights.vector(p + "norm1", (H,), init="zeros"), c.eps, unit_offset=True)
        mixer = (_mlstm if layer.type == "mlstm" else _attention)(c, layer, p + "mix.", weights, act)
        blocks.append(ParallelBlock(norm=norm, mixer=mixer, ffn=_feed_forward(c, layer, p + "mlp.", weights, act),
                                    act_dtype=act))
    final_norm = RMSNorm(weights.vector("final.norm", (H,), init="zeros"), c.eps, unit_offset=True)
    schedule = [ScheduleEntry(layer, before=(t if first else None)) for layer, t, first in c.layer_runs()]
    return DecoderModel(embedding=embedding, blocks=blocks, final_norm=final_norm, head=Linear(embedding, "head"),
                        act_dtype=act, schedule=schedule, config=c, stream_ops=stream_ops)


register_architecture("Notedra", NotedraConfig, build_notedra)
