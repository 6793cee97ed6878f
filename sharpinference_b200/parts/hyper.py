"""Several residual streams per token (hyper-connections), the token shift before a mixer, and the embedding
with a hashed pair table.

``HyperBlock``: instead of one residual stream there are ``S`` copies ``x_1 .. x_S`` (all equal to the embedding
output at the start; stored side by side, ``[T, S * H]``).  A sublayer with coefficients ``in [S]``, ``mix [S, S]``
(indexed from, to) and ``out [S]`` reads ``u = sum_s in[s] x_s``, computes ``y = sublayer(norm(u))`` and then
replaces every stream at once: ``x_t <- sum_s mix[s, t] x_s + out[t] y``.  The block is pre-norm (mixer, then an
optional feed-forward, each with its own coefficients and norm); the replacement of the streams is not run as a
step of its own but inside the kernel of the norm that reads the streams next (``sharpi_hc_mix_norm``), the way
the other blocks fuse a residual add into the next norm: a block hands its last ``(y, mix, out)`` on as the
pending update.  At the end the model's norm reads the plain sum of the streams (:class:`GroupRMSNorm` with
``streams=S``).

The norm is an RMS norm in ``groups`` equal consecutive parts of the width, each divided by its own
``sqrt(mean(part^2) + eps)``, times a weight.

Token shift: what the mixer reads, ``h``, is replaced by ``h + (h' - h) * shift`` with ``h'`` the previous
token's ``h`` before the replacement (zeros before a sequence's first token).  The previous ``h`` is per-request
state of the block (``state_specs["shift"]``), so a prompt may be cut anywhere.

The reference keeps one residual stream and has no token shift (src/SharpInference.Engine/ForwardPass.cs:1557-1714).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Block, FeedForward, LayerSlot, Mixer, Norm, Part, StateSpec, StepContext, register_part


@register_part("norm", "group_rmsnorm")
class GroupRMSNorm(Norm):
    """RMS norm in ``groups`` consecutive parts over the sum (or a weighted sum, ``inc``) of ``streams`` residual
    streams.  ``apply`` takes as ``delta`` either None, a float32 update of a single stream, or the pending
    ``(y, mix, out)`` of a :class:`HyperBlock`, which is applied to the streams first."""

    def __init__(self, weight: torch.Tensor, eps: float, groups: int = 1, streams: int = 1,
                 inc: Optional[torch.Tensor] = None):
        if weight.numel() % groups != 0:
            raise ValueError(f"the width {weight.numel()} is no multiple of the {groups} norm groups")
        if not 1 <= streams <= ops.HC_MAX_STREAMS:
            raise ValueError(f"{streams} streams: the kernels take 1 to {ops.HC_MAX_STREAMS}")
        self.weight, self.eps, self.groups, self.streams, self.inc = weight, float(eps), int(groups), int(streams), inc
        self._one = None

    def apply(self, x, delta, *, rows=None, out_dtype=torch.bfloat16, want_fp32=False):
        if delta is not None and not isinstance(delta, tuple):
            if self.streams != 1:
                raise ValueError("a plain update needs a single stream")
            if self._one is None:
                self._one = torch.ones(1, dtype=torch.float32, device=x.device)
            delta = (delta, self._one, self._one)
        h = ops.hc_mix_norm(x, delta, self.inc, self.weight, streams=self.streams, groups=self.groups, eps=self.eps,
                            out_dtype=torch.float32 if want_fp32 else out_dtype, rows=rows)
        if want_fp32:
            return (h if out_dtype == torch.float32 else h.to(out_dtype)), h
        return h, None


@register_part("block", "hyper")
class HyperBlock(Block):
    graph_safe = True

    def __init__(self, *, streams: int, mixer_norm: GroupRMSNorm, mixer: Mixer, mixer_mix: torch.Tensor,
                 mixer_out: torch.Tensor, ffn_norm: Optional[GroupRMSNorm] = None, ffn: Optional[FeedForward] = None,
                 ffn_mix: Optional[torch.Tensor] = None, ffn_out: Optional[torch.Tensor] = None,
                 shift: Optional[torch.Tensor] = None, act_dtype: torch.dtype = torch.bfloat16):
        """``mixer_norm`` / ``ffn_norm`` carry the sublayers' ``in`` coefficients (``GroupRMSNorm(inc=...)``);
        ``*_mix [S, S]`` and ``*_out [S]`` are the coefficients of the replacement.  ``shift [H]``: the token
        shift of the mixer's input (None: no shift)."""
        for name, t, n in (("mixer mix", mixer_mix, streams * streams), ("mixer out", mixer_out, streams),
                           ("ffn mix", ffn_mix, streams * streams), ("ffn out", ffn_out, streams)):
            if t is not None and t.numel() != n:
                raise ValueError(f"{name} coefficients have {t.numel()} entries, expected {n}")
        if (ffn is None) != (ffn_norm is None) or (ffn is not None and (ffn_mix is None or ffn_out is None)):
            raise ValueError("a feed-forward needs its norm and its coefficients, and the other way round")
        self.streams, self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = streams, mixer_norm, mixer, ffn_norm, ffn
        self.mixer_mix, self.mixer_out, self.ffn_mix, self.ffn_out = mixer_mix, mixer_out, ffn_mix, ffn_out
        self.shift, self.act_dtype = shift, act_dtype
        self.state_specs = {"shift": StateSpec((shift.numel(),), torch.float32)} if shift is not None else None

    def forward(self, ctx: StepContext, slot: LayerSlot, x: torch.Tensor, pending):
        mixer_dtype = torch.float32 if getattr(self.mixer, "wants_fp32_input", False) else self.act_dtype
        if self.shift is not None:
            raw, _ = self.mixer_norm.apply(x, pending, rows=None, out_dtype=torch.float32)
            h = ops.token_shift(raw, self.shift, slot.states["shift"], row_request=ctx.row_request,
                                row_offsets=ctx.row_offsets, state_slots=ctx.state_slots, out_dtype=mixer_dtype)[0]
        else:
            h, _ = self.mixer_norm.apply(x, pending, rows=None, out_dtype=mixer_dtype)
        pending = (self.mixer.forward(ctx, slot, h), self.mixer_mix, self.mixer_out)
        if self.ffn is None:
            return x, pending
        h, h32 = self.ffn_norm.apply(x, pending, rows=None, out_dtype=self.act_dtype,
                                     want_fp32=self.ffn.wants_fp32_input)
        return x, (self.ffn.forward(ctx, h, h32), self.ffn_mix, self.ffn_out)

    def traced_stream(self, x: torch.Tensor, pending) -> torch.Tensor:
        """The sum of the streams with the pending update applied (tracing only; plain tensor code)."""
        T, S = x.shape[0], self.streams
        xs = x.view(T, S, -1)
        if pending is not None:
            y, mix, out = pending
            xs = torch.einsum("tsh,sr->trh", xs, mix.view(S, S)) + out.view(1, S, 1) * y.view(T, 1, -1)
        return xs.sum(dim=1)


class PairEmbedding(Part):
    """``embed[token] + pairs[(previous * mul_prev + token * mul_cur) mod buckets]``, row ``buckets`` of the pair
    table for a sequence's first token; the result is written to every one of ``streams`` residual streams.  The
    previous token of a request is model-level per-request state (``state_specs["prev_token"]``: the token plus
    one, so that a fresh slot's zero means "none")."""

    graph_safe = True

    def __init__(self, *, embed: torch.Tensor, pairs: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int,
                 streams: int = 1):
        if pairs.shape[0] != buckets + 1 or pairs.shape[1] != embed.shape[1]:
            raise ValueError(f"pair table is {tuple(pairs.shape)}, expected [{buckets + 1}, {embed.shape[1]}]")
        self.embed, self.pairs = embed, pairs
        self.buckets, self.mul_prev, self.mul_cur, self.streams = int(buckets), int(mul_prev), int(mul_cur), int(streams)
        self.state_specs = {"prev_token": StateSpec((), torch.int32)}

    def forward(self, ctx: StepContext) -> torch.Tensor:
        return ops.embed_pair(ctx.token_ids, self.embed, self.pairs, row_request=ctx.row_request,
                              row_offsets=ctx.row_offsets, state_slots=ctx.state_slots,
                              prev_state=ctx.model_states["prev_token"], streams=self.streams, buckets=self.buckets,
                              mul_prev=self.mul_prev, mul_cur=self.mul_cur)
