"""The WKV mixer: time mixing with a decay that depends on the token (RWKV family), state of fixed size per request.

With ``h`` the mixer's input and ``h'`` the previous token's (zeros before the first), each of r, k, v, g, w reads
its own mix ``h + (h' - h) * mu_s``.  ``r, k, v = W_r, W_k, W_v`` of their mixes (``heads`` x ``d``),
``gate = silu(W_g mix_g)``, and the decay ``w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))`` per head and key channel.
Per head:

    o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t          (the bonus u counts for the current token only)
    S_t = diag(w_t) S_{t-1} + k_t v_t^T

then every head's ``o`` is divided by its root mean square, the heads side by side are multiplied by a weight and
by the gate, and projected by ``W_o``.

The mixes, the decay with its two exponentials, the state and every product of the recurrence are float32; the
projections round their inputs to the activation dtype.  Two things are per-request state: the previous input
``h'`` (``state_specs["prev"]``) and ``S`` (``state_specs["S"]``, ``[heads, d, d]``, key channel first), both zero
at a sequence's start; a prompt may therefore arrive in portions of any size, and a row's result is the same
sequence of operations either way (``csrc/wkv.cu``).  The reference keeps per-sequence state of fixed size for
another recurrent layer (src/SharpInference.Engine/GdnStateCache.cs).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import LayerSlot, Mixer, StateSpec, StepContext, register_part
from .linear import Linear

_MIXES = ("r", "k", "v", "g", "w")


@register_part("mixer", "wkv")
class WKVMixer(Mixer):
    graph_safe = True
    cache_spec = None
    wants_fp32_input = True

    # Steps of up to this many rows compute r, k, v and g (four products of four different inputs) as one grouped
    # tensor-core product, the four inputs being the groups: one launch instead of four where a step is launch-bound.
    GROUPED_ROWS = 128

    def __init__(self, *, mu: torch.Tensor, r: Linear, k: Linear, v: Linear, g: Linear, w1: Linear, w2: Linear,
                 w0: torch.Tensor, u: torch.Tensor, head_norm_weight: torch.Tensor, out: Linear, heads: int,
                 head_dim: int, eps: float, act_dtype: torch.dtype = torch.bfloat16,
                 rkvg_weight: torch.Tensor = None):
        """``mu [5, H]``: the mixing vectors of r, k, v, g, w in this order.  ``rkvg_weight [4, heads * head_dim, H]``:
        the weights of r, k, v, g stacked (the four ``Linear`` may be views of it), for the grouped product of
        small steps; None: four products at every size."""
        hd = heads * head_dim
        H = r.in_features
        if head_dim > ops.WKV_MAX_HEAD_SIZE:
            raise ValueError(f"head size {head_dim} is beyond the {ops.WKV_MAX_HEAD_SIZE} the recurrence kernel takes")
        if mu.shape != (len(_MIXES), H):
            raise ValueError(f"mixing vectors are {tuple(mu.shape)}, expected [{len(_MIXES)}, {H}]")
        for name, lin in (("r", r), ("k", k), ("v", v), ("g", g), ("w2", w2)):
            if lin.out_features != hd:
                raise ValueError(f"projection {name} has {lin.out_features} rows, expected heads * head size = {hd}")
        if w1.out_features != w2.in_features or out.in_features != hd:
            raise ValueError("the decay's two projections or the output projection disagree on their inner size")
        for name, t in (("w0", w0), ("u", u), ("head norm weight", head_norm_weight)):
            if t.numel() != hd:
                raise ValueError(f"{name} has {t.numel()} entries, expected {hd}")
        self.mu, self.r, self.k, self.v, self.g, self.w1, self.w2, self.out = mu, r, k, v, g, w1, w2, out
        self.w0, self.u, self.head_norm_weight = w0, u, head_norm_weight
        self.heads, self.head_dim, self.eps, self.act_dtype = heads, head_dim, float(eps), act_dtype
        self.rkvg_weight = None
        if (rkvg_weight is not None and rkvg_weight.dtype == torch.bfloat16 and act_dtype == torch.bfloat16
                and H % 8 == 0 and tuple(rkvg_weight.shape) == (4, hd, H)):
            self.rkvg_weight = rkvg_weight
        self._group_offsets = {}
        self.state_specs = {"prev": StateSpec((H,), torch.float32),
                            "S": StateSpec((heads * head_dim * head_dim,), torch.float32)}

    def forward(self, ctx: StepContext, slot: LayerSlot, h: torch.Tensor) -> torch.Tensor:
        mixes = ops.token_shift(h, self.mu, slot.states["prev"], row_request=ctx.row_request,
                                row_offsets=ctx.row_offsets, state_slots=ctx.state_slots, out_dtype=self.act_dtype)
        T = h.shape[0]
        if self.rkvg_weight is not None and T <= self.GROUPED_ROWS:
            offsets = self._group_offsets.get(T)
            if offsets is None:                      # made on the device, once a step size (the first, eager step)
                if len(self._group_offsets) > 256:
                    self._group_offsets.clear()
                offsets = self._group_offsets[T] = torch.arange(5, dtype=torch.int32, device=h.device) * T
            r, k, v, g = ops.tc_grouped_gemm(mixes[:4].view(4 * T, -1), self.rkvg_weight, offsets,
                                             mode=ops.TC_MODE_STORE).view(4, T, -1).unbind(0)
        else:
            r, k, v, g = self.r(mixes[0]), self.k(mixes[1]), self.v(mixes[2]), self.g(mixes[3])
        wraw = self.w2(ops.tanh(self.w1(mixes[4]), self.act_dtype))
        o = ops.wkv_recurrence(r, k, v, wraw, self.w0, self.u, row_offsets=ctx.row_offsets,
                               state_slots=ctx.state_slots, state=slot.states["S"], heads=self.heads, d=self.head_dim)
        return self.out(ops.wkv_out(o, g, self.head_norm_weight, self.eps, self.heads, self.head_dim, self.act_dtype))
