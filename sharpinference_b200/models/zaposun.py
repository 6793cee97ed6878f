"""The Zaposun architecture, put together from parts, and its tensor names.

A decoder with several residual streams per token (:class:`HyperBlock`): every layer is pre-norm, a mixer and then
an optional dense feed-forward ``W_down (gelu_tanh(W_gate h) * (W_up h))``, each sublayer reading a weighted sum of
the streams through an RMS norm in groups and replacing all streams at once.  The mixer's input passes a token
shift.  The embedding adds a row of a hashed pair table chosen by the previous and the current token
(:class:`PairEmbedding`).  Per layer (``config.layers[i]``, every layer with sizes of its own):

* ``wkv``: :class:`WKVMixer`;
* ``parallel``: :class:`BranchPair` of chunked grouped-query attention (weighted RMS norm of q and k per head before a
  rotation of the head's leading elements, values rotated by their position and every head's sum turned back,
  a score factor from the configuration) and a :class:`SelectiveScanMixer`; half the sum of the two outputs, each
  first RMS-normed over the width.

The model's last norm reads the plain sum of the streams; the logits are ``head x * logit_scale``.

Tensor names (linear weights ``[out, in]``): ``embed``, ``bigram [buckets + 1, H]``, ``final.norm``, ``head``; per layer
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.shift``, ``l<i>.hc{1,2}.{in,out,mix}``, ``l<i>.mlp.{gate,up,down}``; for wkv
``l<i>.mix.mu.{r,k,v,g,w}``, ``l<i>.mix.{r,k,v,g,w1,w2,w0,u,norm,o}``; for parallel ``l<i>.mix.left.{q,k,v,q.norm,k.norm,o,out}``
and ``l<i>.mix.right.{in,conv,conv.b,x,dt,dt.b,A_log,D,o,out}``.
"""
from __future__ import annotations

import torch

from ..config.zaposun import ZaposunConfig, ZaposunLayer
from ..parts import (BranchPair, DenseSwiGLU, GroupRMSNorm, HyperBlock, Linear, PagedAttention, PairEmbedding, RMSNorm,
                     RotaryEncoding, SelectiveScanMixer, WKVMixer, leading_rotary_inv_freq)
from ..registry import register_architecture
from ..weights.source import WeightSource
from .model import DecoderModel
from .notedra import _cat


def _on(weights: WeightSource, t: torch.Tensor) -> torch.Tensor:
    return t if weights.device.type == "meta" else t.to(weights.device)


def _wkv(c: ZaposunConfig, layer: ZaposunLayer, p: str, weights: WeightSource, act) -> WKVMixer:
    H, heads, d = c.width, layer.heads, layer.dim
    hd = heads * d
    mu = torch.stack([weights.vector(f"{p}mu.{s}", (H,), init="normal") for s in "rkvgw"]).contiguous()
    lin = {s: weights.matrix(p + s, (hd, H)) for s in "kvg"}
    rank = layer.decay_rank or (weights.shape_of(p + "w1") or (0,))[0]
    if rank <= 0:
        raise ValueError(f"{p}w1: neither the configuration (decay_rank) nor a stored tensor gives the decay's inner size")
    w1 = weights.matrix(p + "w1", (rank, H))
    w2 = Linear(weights.matrix(p + "w2", (hd, rank)), p + "w2")
    w0 = weights.vector(p + "w0", (hd,), init="normal")
    u = weights.vector(p + "u", (heads, d), init="normal")
    norm = weights.vector(p + "norm", (hd,))
    out = Linear(weights.matrix(p + "o", (H, hd)), p + "o")
    lin["r"] = weights.matrix(p + "r", (hd, H))
    stacked = None
    if weights.device.type != "meta" and len({t.dtype for t in lin.values()}) == 1:
        stacked = torch.stack([lin[s] for s in "rkvg"]).contiguous()        # the four Linear below are views of it
        lin = {s: stacked[i] for i, s in enumerate("rkvg")}
    return WKVMixer(mu=mu, r=Linear(lin["r"], p + "r"), k=Linear(lin["k"], p + "k"), v=Linear(lin["v"], p + "v"),
                    g=Linear(lin["g"], p + "g"), w1=Linear(w1, p + "w1"), w2=w2, w0=w0, u=u.reshape(-1),
                    head_norm_weight=norm, out=out, heads=heads, head_dim=d, eps=c.eps, act_dtype=act,
                    rkvg_weight=stacked)


def _attention(c: ZaposunConfig, layer: ZaposunLayer, p: str, weights: WeightSource, act) -> PagedAttention:
    a, H = layer.left, c.width
    nq, nkv, d, dv = a.heads, a.kv_heads, a.dim, a.vdim
    q, k, v = (weights.matrix(p + "q", (nq * d, H)), weights.matrix(p + "k", (nkv * d, H)),
               weights.matrix(p + "v", (nkv * dv, H)))
    q_norm = RMSNorm(weights.vector(p + "q.norm", (d,)), c.eps)
    k_norm = RMSNorm(weights.vector(p + "k.norm", (d,)), c.eps)
    out = Linear(weights.matrix(p + "o", (H, nq * dv)), p + "o")
    position = (RotaryEncoding(_on(weights, leading_rotary_inv_freq(a.rot_dims, a.rot_base)), a.rot_layout, a.rot_dims)
                if a.rot_dims else None)
    value_position = RotaryEncoding(_on(weights, leading_rotary_inv_freq(dv, a.rot_base)), a.rot_layout, dv)
    return PagedAttention(qkv=Linear(_cat([q, k, v]), p + "qkv"), out=out, num_heads=nq, num_kv_heads=nkv, head_dim=d,
                          value_dim=dv, mask="chunk" if a.chunk else "full", span=a.chunk, position=position,
                          qk_norm=q_norm, k_norm=k_norm, qk_norm_first=True, softmax_scale=a.scale, act_dtype=act,
                          value_position=value_position)


def _scan(c: ZaposunConfig, layer: ZaposunLayer, p: str, weights: WeightSource, act) -> SelectiveScanMixer:
    s, H = layer.right, c.width
    return SelectiveScanMixer(
        in_proj=Linear(weights.matrix(p + "in", (2 * s.inner, H)), p + "in"),
        conv_weight=weights.vector(p + "conv", (s.inner, s.conv), init="normal"),
        conv_bias=weights.vector(p + "conv.b", (s.inner,), init="normal"),
        x_proj=Linear(weights.matrix(p + "x", (s.dt_rank + 2 * s.state, s.inner)), p + "x"),
        dt_proj=Linear(weights.matrix(p + "dt", (s.inner, s.dt_rank)), p + "dt"),
        dt_bias=weights.vector(p + "dt.b", (s.inner,), init="normal"),
        a_log=weights.vector(p + "A_log", (s.inner, s.state), init="normal"),
        d_skip=weights.vector(p + "D", (s.inner,)),
        out=Linear(weights.matrix(p + "o", (H, s.inner)), p + "o"),
        inner=s.inner, states=s.state, dt_rank=s.dt_rank, taps=s.conv, act_dtype=act)


def build_zaposun(config: ZaposunConfig, weights: WeightSource) -> DecoderModel:
    c, act, H, S = config, weights.compute_dtype, config.width, config.streams
    embedding = weights.matrix("embed", (c.vocab, H))
    pairs = weights.matrix("bigram", (c.buckets + 1, H))
    blocks = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        norm1_w = weights.vector(p + "norm1", (H,))
        norm2_w = weights.vector(p + "norm2", (H,))
        if layer.type == "wkv":
            mixer = _wkv(c, layer, p + "mix.", weights, act)
        else:
            left = _attention(c, layer, p + "mix.left.", weights, act)
            right = _scan(c, layer, p + "mix.right.", weights, act)
            mixer = BranchPair(left=left, right=right, left_weight=weights.vector(p + "mix.left.out", (H,)),
                               right_weight=weights.vector(p + "mix.right.out", (H,)), eps=c.eps, scale=0.5)
        ffn = None
        if layer.ff:
            gate_up = _cat([weights.matrix(p + "mlp.gate", (layer.ff, H)), weights.matrix(p + "mlp.up", (layer.ff, H))])
            ffn = DenseSwiGLU(gate_up=Linear(gate_up, p + "mlp.gate_up"),
                              down=Linear(weights.matrix(p + "mlp.down", (H, layer.ff)), p + "mlp.down"),
                              act_dtype=act, activation="gelu_tanh")
        hc = {}
        for q in (1, 2):
            hc[q] = (weights.vector(f"{p}hc{q}.in", (S,), init="normal"), weights.vector(f"{p}hc{q}.out", (S,), init="normal"),
                     weights.vector(f"{p}hc{q}.mix", (S, S), init="normal"))
        shift = weights.vector(p + "shift", (H,), init="normal")
        blocks.append(HyperBlock(
            streams=S, mixer_norm=GroupRMSNorm(norm1_w, c.eps, c.groups, S, inc=hc[1][0]), mixer=mixer,
            mixer_mix=hc[1][2], mixer_out=hc[1][1],
            ffn_norm=GroupRMSNorm(norm2_w, c.eps, c.groups, S, inc=hc[2][0]) if ffn is not None else None, ffn=ffn,
            ffn_mix=hc[2][2] if ffn is not None else None, ffn_out=hc[2][1] if ffn is not None else None,
            shift=shift, act_dtype=act))
    final_norm = GroupRMSNorm(weights.vector("final.norm", (H,)), c.eps, c.groups, S)
    head = Linear(weights.matrix("head", (c.vocab, H)), "head")
    embedder = PairEmbedding(embed=embedding, pairs=pairs, buckets=c.buckets, mul_prev=c.mul_prev, mul_cur=c.mul_cur,
                             streams=S)
    return DecoderModel(embedding=embedding, blocks=blocks, final_norm=final_norm, head=head, act_dtype=act, config=c,
                        embedder=embedder, logit_scale=c.logit_scale)


register_architecture("Zaposun", ZaposunConfig, build_zaposun)
