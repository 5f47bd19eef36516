"""Gated linear attention: a recurrent mixer whose memory is one matrix per head.

  q = Wq h / sqrt(dim),  k = Wk h   [heads, dim];   v = Wv h   [heads, vdim]
  a = sigmoid(Wa2 (Wa1 h) + b)^(1/tau)  [heads, dim]      a decay per key channel, through a low rank
  S_t = diag(a_t) S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t   per head, S [dim, vdim] float32, zero at the start
  out = Wo ( rms(o_t) * g_n * silu(Wg h) )                 rms per head over vdim, g_n [vdim] shared by the heads

No cache of keys: the request's whole past is the state, kept in its state slot and carried from
step to step, so a prompt cut into portions, a decoded token and a whole prompt run the same
recurrence token by token.  The decay, its logarithm, the state and the head norm are float32; the
projections run in the compute dtype.  Sizes, tau, eps and tensor names are parameters; the rank of
the decay's two factors is taken from the checkpoint.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import ParamInfo, Part, StateNeed, register_part
from .linear import FUSE_PARTIALS, linear

_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm", "decay_in": "a1", "decay_out": "a2",
          "decay_bias": "a2.b"}


SEGMENT = 64       # tokens per segment of a prompt step (see csrc/recurrent.cu)


class GatedLinearAttention(Part):
    role = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, tau: float, eps: float,
                 decay_rank: int = 16, names=None, prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if min(hidden_size, num_heads, head_dim, value_dim, decay_rank) <= 0 or not tau > 0:
            raise ValueError("gated linear attention: sizes and tau must be positive")
        if head_dim > 256:
            raise ValueError(f"gated linear attention: key size {head_dim} exceeds 256, the most the recurrence kernel takes")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = hidden_size, num_heads, head_dim, value_dim
        self.tau, self.eps, self.decay_rank = float(tau), float(eps), int(decay_rank)
        self.names = dict(_NAMES, **(names or {}))
        self.qk_size, self.v_size = num_heads * head_dim, num_heads * value_dim
        self.w_in = None          # [q; k; v; gate; decay_in] stacked: one product per step
        self.w_decay = self.b_decay = self.w_o = self.gain = None

    def parameters(self):
        n = lambda k: self.name(self.names[k])
        W, R = self.hidden_size, self.decay_rank
        return {n("q"): ParamInfo((self.qk_size, W)), n("k"): ParamInfo((self.qk_size, W)),
                n("v"): ParamInfo((self.v_size, W)), n("gate"): ParamInfo((self.v_size, W)),
                n("out"): ParamInfo((W, self.v_size)),
                n("norm"): ParamInfo((self.value_dim,), kind="gain", init="ones_normal"),
                n("decay_in"): ParamInfo((R, W), free_dims=(0,)),
                n("decay_out"): ParamInfo((self.qk_size, R), free_dims=(1,)),
                n("decay_bias"): ParamInfo((self.qk_size,), kind="gain", init="normal")}

    def bind(self, tensors):
        n = lambda k: tensors[self.name(self.names[k])]
        a1, a2 = n("decay_in"), n("decay_out")
        if a1.shape[0] != a2.shape[1]:
            raise ValueError(f"{self.prefix}: the decay's factors disagree on their rank ({a1.shape[0]} and {a2.shape[1]})")
        self.decay_rank = int(a1.shape[0])
        self.w_in = torch.cat([n("q"), n("k"), n("v"), n("gate"), a1], dim=0).contiguous()
        self.w_decay = a2.contiguous()
        self.b_decay = n("decay_bias").contiguous()
        self.gain = n("norm").contiguous()
        self.w_o = n("out").contiguous()

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed((self.num_heads, self.head_dim, self.value_dim), torch.float32)

    def forward(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        T, ws = ctx.n_tokens, ctx.workspace
        QK, VS, R = self.qk_size, self.v_size, self.decay_rank
        proj = linear(x, self.w_in, ws.get("gla_in", T, self.w_in.shape[0], self.dtype), T)
        q, k, v = proj[:, :QK], proj[:, QK:2 * QK], proj[:, 2 * QK:2 * QK + VS]
        gate, low = proj[:, 2 * QK + VS:2 * QK + 2 * VS], proj[:, 2 * QK + 2 * VS:]
        # the decay's pre-activation in float32; bias, log-sigmoid and the power are the recurrence kernel's
        z = linear(low, self.w_decay, ws.get("gla_decay", T, QK, torch.float32), T)
        o = ws.get("gla_o", T, VS, torch.float32)
        # a step with prompt portions runs them as segments side by side (two passes); single tokens take one pass
        seg = 0 if (ctx.decode_only or T < 4 * SEGMENT) else SEGMENT
        seg_state = seg_decay = None
        if seg:
            cap = ws.max_rows // seg + ctx.cu_tokens.numel()
            seg_state = ws.flat("gla_seg_state", cap * self.num_heads * self.head_dim * self.value_dim, torch.float32)
            seg_decay = ws.flat("gla_seg_decay", cap * self.num_heads * self.head_dim, torch.float32)
        ops.gla_scan(o, q, k, v, z, self.b_decay, self.tau, self.head_dim ** -0.5, view.state, ctx.state_slots,
                     ctx.cu_tokens, ctx.n_entries, n_tokens=T, seg_len=seg, seg_state=seg_state, seg_decay=seg_decay)
        normed = ws.get("attn_out", T, VS, self.dtype)
        ops.head_rmsnorm_gate(normed, o, self.gain, gate, T, self.num_heads, self.eps)
        return linear(normed, self.w_o, ws.get("mixer_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS)


register_part("mixer", "gla", GatedLinearAttention)
