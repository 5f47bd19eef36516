"""Plain, slow implementation of the Tevudra decoder, for tests only.

Whole sequences, no cache, one function per mechanism, float64 on the CPU.  It shares
no code with the engine.  Notation: x is the residual stream [T, W]; h a normalised
input; every weight is [out, in] and applied as h @ W.T.

  layer:      x += mixer(dyt(x));  x += ff(dyt(x))          (ff may be absent)
  dyt:        tanh(alpha * x) * w + b                       (no mean, no variance)
  mixer:      q = h Wq^T; c = rms(h Wdkv^T) * g_c (or the latent of an earlier layer);
              k_h = c Wuk_h^T, v_h = c Wuv_h^T; p = softmax_{j<=i}(scale * q_h . k_h);
              o_h = sigmoid(h Wg^T)_h * sum_j p_j v_h,j; out = concat(o) Wo^T
  dense ff:   relu(h Wup^T)^2 Wdown^T
  routed ff:  z = h Wr^T + b_r; the `top` largest z; weights = softmax over those alone;
              sum_e w_e * gelu_erf(h Wup_e^T) Wdown_e^T  +  shared expert of the same form
  output:     dyt(x) Whead^T
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def dyt(x: torch.Tensor, alpha, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return torch.tanh(float(alpha) * x.to(F64)) * w.to(F64) + b.to(F64)


def rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.to(F64)


def latent(h: torch.Tensor, w_dkv: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """What a layer with a down-projection of its own caches per token: [T, rank]."""
    return rms(h.to(F64) @ w_dkv.to(F64).T, g, eps)


def latent_attention(h, c, w_q, w_uk, w_uv, w_g, w_o, heads: int, dim: int, vdim: int, scale: float):
    """h [T, W] the mixer's input, c [T, rank] the latents of the same tokens."""
    h, c = h.to(F64), c.to(F64)
    T = h.shape[0]
    q = (h @ w_q.to(F64).T).view(T, heads, dim)
    k = (c @ w_uk.to(F64).T).view(T, heads, dim)
    v = (c @ w_uv.to(F64).T).view(T, heads, vdim)
    gate = torch.sigmoid(h @ w_g.to(F64).T)                       # [T, heads]
    out = torch.zeros(T, heads, vdim, dtype=F64)
    for i in range(T):
        s = torch.einsum("hd,jhd->hj", q[i], k[: i + 1]) * scale  # [heads, i + 1]
        p = torch.softmax(s, dim=-1)
        out[i] = torch.einsum("hj,jhd->hd", p, v[: i + 1]) * gate[i][:, None]
    return out.reshape(T, heads * vdim) @ w_o.to(F64).T


def relu2_ff(h, w_up, w_down):
    a = torch.relu(h.to(F64) @ w_up.to(F64).T)
    return (a * a) @ w_down.to(F64).T


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def gelu_ff(h, w_up, w_down):
    return gelu_erf(h.to(F64) @ w_up.to(F64).T) @ w_down.to(F64).T


def route(h, w_r, b_r, top: int):
    """(ids [T, top], weights [T, top]): the largest logits and the softmax over them alone."""
    z = h.to(F64) @ w_r.to(F64).T + b_r.to(F64)
    vals, ids = torch.topk(z, top, dim=-1)
    return ids, torch.softmax(vals, dim=-1)


def routed_ff(h, w_r, b_r, top: int, experts: List[tuple], shared: Optional[tuple]):
    """experts: [(w_up, w_down)] by index; shared: (w_up, w_down) or None."""
    ids, wts = route(h, w_r, b_r, top)
    out = torch.zeros(h.shape[0], experts[0][1].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for j in range(top):
            up, down = experts[int(ids[t, j])]
            out[t] += wts[t, j] * gelu_ff(h[t: t + 1], up, down)[0]
    if shared is not None:
        out += gelu_ff(h, *shared)
    return out


def route_margin(h, w_r, b_r, top: int) -> torch.Tensor:
    """Per token, how far the last chosen logit lies above the first one left out (inf if all are chosen):
    where this is small, a rounding error elsewhere can change the choice."""
    z = h.to(F64) @ w_r.to(F64).T + b_r.to(F64)
    if top >= z.shape[1]:
        return torch.full((z.shape[0],), math.inf, dtype=F64)
    s = torch.sort(z, dim=-1, descending=True).values
    return s[:, top - 1] - s[:, top]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, keep_layers: bool = False, margins: Optional[list] = None):
    """Logits [T, vocab] in float64 of one whole sequence; with keep_layers also the residual
    stream after every layer [layers, T, W].  margins: a list that receives, per routed layer, the
    tokens' route_margin."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)]
    latents: Dict[int, torch.Tensor] = {}
    kept = []
    norm = lambda name, x: dyt(x, w[name + ".alpha"], w[name], w[name + ".b"])
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        h = norm(p + ".norm1", x)
        src = m.get("kv_from")
        if src is None:
            latents[i] = latent(h, w[p + ".mix.dkv"], w[p + ".mix.dkv.norm"], eps)
            c = latents[i]
        else:
            c = latents[int(src)]
        x = x + latent_attention(h, c, w[p + ".mix.q"], w[p + ".mix.uk"], w[p + ".mix.uv"], w[p + ".mix.g"],
                                 w[p + ".mix.o"], m["heads"], m["dim"], m["vdim"], float(m["scale"]))
        ff = layer.get("mlp")
        if ff is not None:
            h = norm(p + ".norm2", x)
            if ff["kind"] == "dense":
                x = x + relu2_ff(h, w[p + ".mlp.up"], w[p + ".mlp.down"])
            elif ff["kind"] == "moe":
                n, top = ff["router"]["experts"], ff["router"]["top"]
                experts = [(w[f"{p}.mlp.e{e}.up"], w[f"{p}.mlp.e{e}.down"]) for e in range(n)]
                shared = (w[p + ".mlp.shared.up"], w[p + ".mlp.shared.down"]) if ff.get("shared") else None
                if margins is not None:
                    margins.append(route_margin(h, w[p + ".mlp.router"], w[p + ".mlp.router.b"], top))
                x = x + routed_ff(h, w[p + ".mlp.router"], w[p + ".mlp.router.b"], top, experts, shared)
            else:
                raise ValueError(ff["kind"])
        if keep_layers:
            kept.append(x.clone())
    logits = norm("final.norm", x) @ w["head"].to(F64).T
    return (logits, torch.stack(kept)) if keep_layers else logits
