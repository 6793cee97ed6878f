"""The matrix-memory mixer (mLSTM of the xLSTM family): a recurrent layer with a state of fixed size per request.

Per head (``heads`` of them; key/query size ``d``, value size ``dv``), for the rows of a request in order:

    q_t = (Wq h_t) / sqrt(d),  k_t = Wk h_t,  v_t = Wv h_t
    i_t = cap tanh((wi . h_t + bi) / cap)                       log input gate
    f_t = logsigmoid(cap tanh((wf . h_t + bf) / cap))           log forget gate
    m_t = max(f_t + m_{t-1}, i_t)                               m starts at 0
    S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T
    n_t = exp(f_t + m_{t-1} - m_t) n_{t-1} + exp(i_t - m_t) k_t
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)

then every head's ``o_t`` is divided by its root mean square (``eps`` inside the root), the heads side by side are
multiplied by a weight and by ``sigmoid(Wg h_t)``, and projected by ``Wo``.  ``cap`` bounds the raw gates.

The projections q, k, v, g and the two gate rows are one fused product whose result stays float32; from there on
everything is float32: gates, exponentials, the state ``(S, n, m)`` and the products of the recurrence.  The state
lives in the cache manager's per-request slots (zeroed when a request is admitted) and is carried from step to
step, so a prompt may arrive in portions of any size and a decoded token is a portion of one row: a row's result
is the same sequence of operations either way.

The reference keeps per-sequence state of fixed size for another recurrent layer
(src/SharpInference.Engine/GdnStateCache.cs); the recurrence here is ``csrc/mlstm.cu``.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import LayerSlot, Mixer, StateSpec, StepContext, register_part
from .linear import Linear


def fused_mlstm_columns(heads: int, d: int, dv: int):
    """First column of q, k, v, g, i, f in the fused projection, and its width padded to a multiple of 8."""
    col_q = 0
    col_k = col_q + heads * d
    col_v = col_k + heads * d
    col_g = col_v + heads * dv
    col_i = col_g + heads * dv
    col_f = col_i + heads
    width = (col_f + heads + 7) // 8 * 8
    return col_q, col_k, col_v, col_g, col_i, col_f, width


@register_part("mixer", "mlstm")
class MLSTMMixer(Mixer):
    graph_safe = True        # reads the step through device tensors only
    cache_spec = None

    def __init__(self, *, proj: Linear, out: Linear, gate_bias_i: torch.Tensor, gate_bias_f: torch.Tensor,
                 head_norm_weight: torch.Tensor, heads: int, key_dim: int, value_dim: int, gate_cap: float,
                 eps: float, act_dtype: torch.dtype = torch.bfloat16):
        """``proj``: the fused projection, rows in the order of :func:`fused_mlstm_columns` (zero rows pad it)."""
        cols = fused_mlstm_columns(heads, key_dim, value_dim)
        if proj.out_features != cols[-1]:
            raise ValueError(f"fused mLSTM projection has {proj.out_features} rows, expected {cols[-1]}")
        if out.in_features != heads * value_dim:
            raise ValueError(f"output projection reads {out.in_features} columns, expected heads * value size = "
                             f"{heads * value_dim}")
        if key_dim > ops.MLSTM_MAX_KEY_SIZE:
            raise ValueError(f"key size {key_dim} is beyond the {ops.MLSTM_MAX_KEY_SIZE} the recurrence kernels take")
        if not gate_cap > 0:
            raise ValueError(f"the gate cap must be positive, found {gate_cap}")
        for name, t, n in (("input-gate bias", gate_bias_i, heads), ("forget-gate bias", gate_bias_f, heads),
                           ("head norm weight", head_norm_weight, heads * value_dim)):
            if t.numel() != n:
                raise ValueError(f"{name} has {t.numel()} entries, expected {n}")
        self.proj, self.out = proj, out
        self.bias_i, self.bias_f, self.head_norm_weight = gate_bias_i, gate_bias_f, head_norm_weight
        self.heads, self.key_dim, self.value_dim = heads, key_dim, value_dim
        self.gate_cap, self.eps, self.act_dtype = float(gate_cap), float(eps), act_dtype
        self.q_scale = float(key_dim) ** -0.5
        (self.col_q, self.col_k, self.col_v, self.col_g, self.col_i, self.col_f, _) = cols
        self.state_spec = StateSpec((ops.mlstm_state_floats(heads, key_dim, value_dim)[1],), torch.float32)

    def forward(self, ctx: StepContext, slot: LayerSlot, h: torch.Tensor) -> torch.Tensor:
        p = self.proj(h)                                                    # [T, fused] float32
        num, nq, coef = ops.mlstm_recurrence(
            p, col_q=self.col_q, col_k=self.col_k, col_v=self.col_v, col_i=self.col_i, col_f=self.col_f,
            bias_i=self.bias_i, bias_f=self.bias_f, row_offsets=ctx.row_offsets, state_slots=ctx.state_slots,
            state=slot.state, heads=self.heads, d=self.key_dim, dv=self.value_dim, cap=self.gate_cap,
            q_scale=self.q_scale)
        o = ops.mlstm_out(num, nq, coef, p, self.col_g, self.head_norm_weight, self.eps, self.heads, self.value_dim,
                          self.act_dtype)
        return self.out(o)
