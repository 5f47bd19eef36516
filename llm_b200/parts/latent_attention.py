"""Latent attention: keys and values of every head are linear maps of one small vector per
token, and only that vector is cached.

  c_t   = rms(Wdkv h_t) * gain          [rank]      (kept in the layer's pages; a layer may
                                                      instead read the latents that another
                                                      layer stored, with maps of its own)
  k_t,h = Wuk_h c_t,  v_t,h = Wuv_h c_t
  o_i,h = sigmoid(Wg h_i)_h * sum_{j<=i} softmax_j(scale * q_i,h . k_j,h) v_j,h
  out_i = Wo concat_h(o_i,h)

No position enters: the mask alone orders the tokens.  Because k and v are linear in c, the
engine never forms them.  It carries the query through the key map, q'_i,h = Wuk_h^T q_i,h, so that
q . k = q' . c; runs a multi-query attention whose single key/value head of size `rank` is c
itself (the paged attention kernels the other mixers use, with the key pages given as value
pages too); and carries the result, a mix of latents, through the value map.  The cache holds
rank numbers per token and layer instead of heads x (dim + vdim), and prompts, portions and
decoded tokens all run the same arithmetic.  Sizes, the score scale, the norm's eps and the
tensor names are parameters.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import CacheNeed, ParamInfo, Part, register_part
from .linear import FUSE_PARTIALS, linear

_NAMES = {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "gate": "g", "out": "o"}


class LatentAttention(Part):
    role = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, rank: int, scale: float,
                 eps: float, gated: bool = True, shares_cache: bool = False, names=None, prefix: str = "", dtype=None,
                 device=None):
        super().__init__(prefix, dtype, device)
        if min(hidden_size, num_heads, head_dim, value_dim, rank) <= 0:
            raise ValueError("latent attention: sizes must be positive")
        if rank > 1024:
            raise ValueError(f"latent attention: rank {rank} exceeds 1024, the widest head the attention kernels take")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim, self.rank = hidden_size, num_heads, head_dim, value_dim, rank
        self.scale, self.eps = float(scale), float(eps)
        self.gated = bool(gated)
        self.shares_cache = bool(shares_cache)      # reads another layer's latents: no down-projection of its own
        self.names = dict(_NAMES, **(names or {}))
        self.q_size = num_heads * head_dim
        # The width of a cached row.  The tensor-core attention kernels (bfloat16) take heads of 64 or 128: a
        # smaller rank is padded up to the next of the two with zeros (in the cache rows and in the two per-head
        # maps), which changes no score and no output and costs cache, not correctness.  Other ranks, and
        # float32, keep their width and run on the general kernels.
        self.row_width = rank
        if dtype == torch.bfloat16 and rank < 128 and rank != 64:
            self.row_width = 64 if rank < 64 else 128
        self.w_in = None          # [q; down; gate] stacked: one product per step
        self.w_uk_t = None        # [heads, rank, dim]: the key map, transposed per head
        self.w_uv = None          # [heads, vdim, rank]
        self.w_o = None
        self.gain = None

    def parameters(self):
        n = lambda k: self.name(self.names[k])
        p = {n("q"): ParamInfo((self.q_size, self.hidden_size))}
        if not self.shares_cache:
            p[n("down")] = ParamInfo((self.rank, self.hidden_size))
            p[n("down_norm")] = ParamInfo((self.rank,), kind="gain", init="ones_normal")
        p[n("up_k")] = ParamInfo((self.q_size, self.rank))
        p[n("up_v")] = ParamInfo((self.num_heads * self.value_dim, self.rank))
        if self.gated:
            p[n("gate")] = ParamInfo((self.num_heads, self.hidden_size))
        p[n("out")] = ParamInfo((self.hidden_size, self.num_heads * self.value_dim))
        return p

    def bind(self, tensors):
        n = lambda k: tensors[self.name(self.names[k])]
        parts = [n("q")]
        if not self.shares_cache:
            parts.append(n("down"))
            self.gain = n("down_norm").contiguous()
        if self.gated:
            parts.append(n("gate"))
        self.w_in = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0].contiguous()
        H, D, V, R = self.num_heads, self.head_dim, self.value_dim, self.rank
        self.w_uk_t = n("up_k").view(H, D, R).transpose(1, 2).contiguous()
        self.w_uv = n("up_v").view(H, V, R).contiguous()
        if self.row_width != R:
            pad = self.row_width - R
            self.w_uk_t = torch.nn.functional.pad(self.w_uk_t, (0, 0, 0, pad)).contiguous()      # [H, width, D]: zero rows
            self.w_uv = torch.nn.functional.pad(self.w_uv, (0, pad)).contiguous()                # [H, V, width]: zero columns
        self.w_o = n("out").contiguous()

    def cache_need(self):
        if self.shares_cache:
            return None
        return CacheNeed("full", 1, self.row_width, None, values=False)

    def state_need(self):
        return None

    def forward(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        T, ws = ctx.n_tokens, ctx.workspace
        H, R, RW = self.num_heads, self.rank, self.row_width
        proj = linear(x, self.w_in, ws.get("latent_in", T, self.w_in.shape[0], self.dtype), T)
        col = self.q_size
        pages = view.k_pages                        # [pages, 1, page_size, rank]; also the value pages
        if not self.shares_cache:
            ops.latent_norm_store(proj[:, col:col + R], self.gain, self.eps, view.group.slot_map, pages, T)
            col += R
        gate = proj[:, col:col + H] if self.gated else None
        q_lat = ws.get("latent_q", T, H * RW, self.dtype)
        ops.gemm_heads(proj[:, :self.q_size], self.w_uk_t, q_lat, T, H)
        o_lat = ws.get("latent_o", T, H * RW, self.dtype)
        ops.paged_attention(o_lat, q_lat, pages, pages, view.group, ctx, H, 1, RW, 0, self.scale)
        attn = ws.get("attn_out", T, H * self.value_dim, self.dtype)
        ops.gemm_heads(o_lat, self.w_uv, attn, T, H, gate=gate)
        return linear(attn, self.w_o, ws.get("mixer_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS)


register_part("mixer", "latent_attention", LatentAttention)
