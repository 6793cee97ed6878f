"""The selective state-space mixer (Mamba) and the mixer that runs two mixers side by side.

``SelectiveScanMixer``: ``W_in h = [x | z]`` (``inner`` channels each).  ``x`` passes a causal convolution per channel
(``taps`` inputs, the last weight column is the current token's, zeros before a sequence's start) with a bias, then
silu.  ``W_x x = [dt_in (dt_rank) | B (states) | C (states)]``; ``dt = softplus(W_dt dt_in + dt_bias)`` per channel;
``A = -exp(A_log)`` ``[inner, states]``.  Per channel c and state n:

    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n ;   y_c = sum_n S[c, n] C_n + D_c x_c

and the result is ``W_o (y * silu(z))``.  The convolution, step sizes, exponentials, state and sums are float32;
the projections round their inputs to the activation dtype.  Per-request state: ``S`` (``state_specs["S"]``) and
the convolution's last ``taps - 1`` inputs (``state_specs["conv"]``), both zero at a sequence's start
(``csrc/mamba.cu``).

``BranchPair``: two mixers that read the same input; the result is ``scale * (rms(left) * w_left + rms(right) *
w_right)``, each branch's output normed over the model width with a plain weight first.  The pair owns the cache
of whichever branch keeps keys and values and the state of both (names prefixed ``left.`` / ``right.``).
"""
from __future__ import annotations

from dataclasses import replace
from typing import Optional

import torch

from ..kernels import ops
from .base import LayerSlot, Mixer, StateSpec, StepContext, register_part
from .linear import Linear


@register_part("mixer", "selective_scan")
class SelectiveScanMixer(Mixer):
    graph_safe = True
    cache_spec = None

    def __init__(self, *, in_proj: Linear, conv_weight: torch.Tensor, conv_bias: Optional[torch.Tensor],
                 x_proj: Linear, dt_proj: Linear, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
                 out: Linear, inner: int, states: int, dt_rank: int, taps: int,
                 act_dtype: torch.dtype = torch.bfloat16):
        if in_proj.out_features != 2 * inner or x_proj.in_features != inner or out.in_features != inner:
            raise ValueError(f"the projections disagree with the inner size {inner}")
        if x_proj.out_features != dt_rank + 2 * states or dt_proj.in_features != dt_rank or dt_proj.out_features != inner:
            raise ValueError("the step-size projections disagree with dt_rank, the number of states or the inner size")
        if conv_weight.numel() != inner * taps or a_log.numel() != inner * states:
            raise ValueError("the convolution weight or A_log disagree with inner, taps or states")
        if states > ops.SCAN_MAX_STATES or taps < 1:
            raise ValueError(f"{states} states (at most {ops.SCAN_MAX_STATES}) or {taps} taps are not supported")
        self.in_proj, self.x_proj, self.dt_proj, self.out = in_proj, x_proj, dt_proj, out
        self.conv_weight, self.conv_bias, self.dt_bias, self.a_log, self.d_skip = conv_weight, conv_bias, dt_bias, a_log, d_skip
        self.inner, self.states, self.dt_rank, self.taps, self.act_dtype = inner, states, dt_rank, taps, act_dtype
        self.state_specs = {"S": StateSpec((inner * states,), torch.float32),
                            "conv": StateSpec((max(taps - 1, 1) * inner,), torch.float32)}

    def forward(self, ctx: StepContext, slot: LayerSlot, h: torch.Tensor) -> torch.Tensor:
        xz = self.in_proj(h)                                                     # [T, 2 inner] float32
        x32, xact = ops.causal_conv(xz, self.inner, self.conv_weight, self.conv_bias, slot.states["conv"],
                                    row_request=ctx.row_request, row_offsets=ctx.row_offsets,
                                    state_slots=ctx.state_slots, act_dtype=self.act_dtype, gate_col=self.inner)
        dbc = self.x_proj(xact)                                                  # [T, dt_rank + 2 states] float32
        dt = self.dt_proj(ops.slice_cols(dbc, 0, self.dt_rank, self.act_dtype))
        ops.bias_act(dt, self.dt_bias, ops.ACT_SOFTPLUS, torch.float32, out=dt)  # the step sizes, in place
        y = ops.selective_scan(x32, dt, dbc, self.dt_rank, self.dt_rank + self.states, self.a_log,
                               self.d_skip, xz, self.inner, row_offsets=ctx.row_offsets, state_slots=ctx.state_slots,
                               state=slot.states["S"], out_dtype=self.act_dtype)
        return self.out(y)


@register_part("mixer", "branch_pair")
class BranchPair(Mixer):
    def __init__(self, *, left: Mixer, right: Mixer, left_weight: torch.Tensor, right_weight: torch.Tensor, eps: float,
                 scale: float = 0.5):
        if left.cache_spec is not None and right.cache_spec is not None:
            raise ValueError("only one branch of a pair may keep keys and values")
        self.left, self.right, self.left_weight, self.right_weight = left, right, left_weight, right_weight
        self.eps, self.scale = float(eps), float(scale)
        self.cache_spec = left.cache_spec if left.cache_spec is not None else right.cache_spec
        self.state_spec = None
        self.state_specs = {}
        for prefix, m in (("left.", left), ("right.", right)):
            if m.state_spec is not None:
                self.state_specs[prefix + "state"] = m.state_spec
            for name, spec in (m.state_specs or {}).items():
                self.state_specs[prefix + name] = spec
        self.graph_safe = bool(getattr(left, "graph_safe", False) and getattr(right, "graph_safe", False))
        self.wants_fp32_input = False

    def step_planner(self, page_size: int):
        return self.left.step_planner(page_size) or self.right.step_planner(page_size)

    @staticmethod
    def _branch_slot(slot: LayerSlot, prefix: str, mixer: Mixer) -> LayerSlot:
        states = {name[len(prefix):]: t for name, t in slot.states.items() if name.startswith(prefix)}
        return replace(slot, states=states, state=states.get("state") if mixer.state_spec is not None else None)

    def forward(self, ctx: StepContext, slot: LayerSlot, h: torch.Tensor) -> torch.Tensor:
        a = self.left.forward(ctx, self._branch_slot(slot, "left.", self.left), h)
        b = self.right.forward(ctx, self._branch_slot(slot, "right.", self.right), h)
        return ops.norm_mean2(a, self.left_weight, b, self.right_weight, self.eps, self.scale)
