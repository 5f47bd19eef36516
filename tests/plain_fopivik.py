"""Plain, slow implementation of the Fopivik decoder, for tests only.

Whole sequences, no cache, one function per mechanism, float64 on the CPU.  It shares no
code with the engine.  Notation: x is the residual stream [T, W], e the embedding rows of the
same tokens, h a normalised input; every weight is [out, in] and applied as h @ W.T; m is the
residual multiplier.

  layer:      x += m * ln(mixer(ln(x)));  x += m * ln(ff(ln(x)))      (four norms a layer; ff may be absent)
  ln:         (x - mean) / sqrt(var + eps) * w                        (no bias)
  passes:     layers start..stop-1 run `times` times with the same weights; before the first layer of
              pass t:  x = [x, e] Win^T + step[t]
  attention:  GQA; q, k rotated pairwise (2i, 2i+1) on the first `dims` channels of a head with
              frequencies scaled by wavelength; s = cap * tanh(scale * q.k / cap); key j is seen by i
              when j <= i and (i - j < size or j < keep_first); p_j = exp(s_j) / (1 + sum_j exp(s_j))
  gla:        S_t = diag(a_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t / sqrt(dim), a = sigmoid(z)^(1/tau),
              z = (h Wa1^T) Wa2^T + b; out = (rms(o) * g_n * silu(h Wg^T)) Wo^T
  ff:         s = softmax(h Wr^T) over all experts; the `top` largest; sum_e s_e * down_e(silu(gate_e h) * up_e h)
  output:     cap * tanh(ln(x) Whead^T / cap)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.to(F64)
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w.to(F64)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scaled_frequencies(dims: int, base: float, scaling: Optional[dict]) -> torch.Tensor:
    """f_i for i < dims/2: base^(-2i/dims), divided by `factor` where the wavelength exceeds
    original/low, kept where it is under original/high, blended in between."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave > orig / lo:
                f = f / fac
            elif wave >= orig / hi:
                s = (orig / wave - lo) / (hi - lo)
                f = (1.0 - s) * f / fac + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x [T, heads, dim]; channels 2i and 2i+1 (i < len(freqs)) turn by positions * freqs[i]."""
    x = x.to(F64).clone()
    n = freqs.numel()
    ang = positions.to(F64)[:, None] * freqs[None, :]                  # [T, n]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0:2 * n:2].clone(), x[..., 1:2 * n:2].clone()
    x[..., 0:2 * n:2] = a * c - b * s
    x[..., 1:2 * n:2] = b * c + a * s
    return x


def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    return j <= i and (i - j < size or j < keep_first)


def sink_attention(q, k, v, scale: float, softcap: float, size: int, keep_first: int) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, V], already rotated -> [T, H, V]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, size, keep_first)]
        for h in range(H):
            g = h // (H // G)
            s = (k[js, g] @ q[i, h]) * scale
            s = softcap * torch.tanh(s / softcap)
            e = torch.exp(s)
            p = e / (1.0 + e.sum())
            out[i, h] = p @ v[js, g]
    return out


def attention_mixer(h, positions, w: Dict[str, torch.Tensor], m: dict) -> torch.Tensor:
    T = h.shape[0]
    h = h.to(F64)
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].to(F64).T).view(T, H, D)
    k = (h @ w["k"].to(F64).T).view(T, G, D)
    v = (h @ w["v"].to(F64).T).view(T, G, V)
    rot = m["rot"]
    f = scaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    q, k = rotate_pairs(q, positions, f), rotate_pairs(k, positions, f)
    o = sink_attention(q, k, v, m["scale"], m["softcap"], m["mask"]["size"], m["mask"]["keep_first"])
    return o.reshape(T, H * V) @ w["o"].to(F64).T


def decay(h, w_a1, w_a2, b_a2, tau: float) -> torch.Tensor:
    z = (h.to(F64) @ w_a1.to(F64).T) @ w_a2.to(F64).T + b_a2.to(F64)
    return torch.exp(torch.nn.functional.logsigmoid(z) / tau)


def gla_recurrence(q, k, v, a) -> torch.Tensor:
    """q, k, a [T, H, D], v [T, H, V] -> o [T, H, V]; the state starts at zero."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[2], dtype=F64)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def gla_mixer(h, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    h = h.to(F64)
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].to(F64).T).view(T, H, D) * D ** -0.5
    k = (h @ w["k"].to(F64).T).view(T, H, D)
    v = (h @ w["v"].to(F64).T).view(T, H, V)
    a = decay(h, w["a1"], w["a2"], w["a2.b"], m["tau"]).view(T, H, D)
    o = rms_unit(gla_recurrence(q, k, v, a), eps) * w["norm"].to(F64)
    gate = torch.nn.functional.silu(h @ w["g"].to(F64).T).view(T, H, V)
    return (o * gate).reshape(T, H * V) @ w["o"].to(F64).T


def route_all(h, w_r, top: int):
    """(ids [T, top], weights [T, top]): the largest of softmax(z) over all experts, as they are."""
    s = torch.softmax(h.to(F64) @ w_r.to(F64).T, dim=-1)
    vals, ids = torch.topk(s, top, dim=-1)
    return ids, vals


def route_margin(h, w_r, top: int) -> torch.Tensor:
    """Per token, how far the last chosen router logit lies above the first one left out (inf if none is left out)."""
    z = torch.sort(h.to(F64) @ w_r.to(F64).T, dim=-1, descending=True).values
    if top >= z.shape[-1]:
        return torch.full((z.shape[0],), math.inf, dtype=F64)
    return z[:, top - 1] - z[:, top]


def gated_expert(h, w_gate, w_up, w_down):
    h = h.to(F64)
    return (torch.nn.functional.silu(h @ w_gate.to(F64).T) * (h @ w_up.to(F64).T)) @ w_down.to(F64).T


def moe_ff(h, w_r, top: int, experts: List[tuple]) -> torch.Tensor:
    """experts: [(gate, up, down)] by index."""
    ids, wts = route_all(h, w_r, top)
    out = torch.zeros(h.shape[0], experts[0][2].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, s in zip(ids[t].tolist(), wts[t]):
            out[t] += s * gated_expert(h[t:t + 1], *experts[e])[0]
    return out


def loop_entry(x, e, w_in, step_row) -> torch.Tensor:
    return torch.cat([x.to(F64), e.to(F64)], dim=-1) @ w_in.to(F64).T + step_row.to(F64)


def layer_order(n_layers: int, loop: Optional[dict]):
    """[(layer, pass number or None when the layer opens no pass)] in execution order."""
    if not loop:
        return [(i, None) for i in range(n_layers)]
    a, b, n = loop["start"], loop["stop"], loop["times"]
    out = [(i, None) for i in range(a)]
    for t in range(n):
        out += [(i, t if i == a else None) for i in range(a, b)]
    return out + [(i, None) for i in range(b, n_layers)]


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, return_layers: bool = False, margins=None):
    """Logits [T, vocab] of one whole sequence (and, if asked, the stream after every layer run).  margins: a list
    that receives, per routed feed-forward that runs, every token's routing margin."""
    eps, m = config["norm"]["eps"], config["residual_mult"]
    tok = torch.as_tensor(tokens, dtype=torch.long)
    T = tok.numel()
    pos = torch.arange(T)
    e = weights["embed"].to(F64)[tok]
    x = e.clone()
    streams = []
    for i, opens in layer_order(len(config["layers"]), config.get("loop")):
        layer, p = config["layers"][i], f"l{i}"
        if opens is not None:
            x = loop_entry(x, e, weights["loop.in"], weights["loop.step"][opens])
        mix = {k[len(p) + 5:]: v for k, v in weights.items() if k.startswith(p + ".mix.")}
        hn = layer_norm(x, weights[p + ".norm1"], eps)
        if layer["type"] == "attention":
            y = attention_mixer(hn, pos, mix, layer["mixer"])
        elif layer["type"] == "gla":
            y = gla_mixer(hn, mix, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + m * layer_norm(y, weights[p + ".norm1b"], eps)
        ff = layer.get("mlp")
        if ff is not None:
            hn = layer_norm(x, weights[p + ".norm2"], eps)
            n_e = ff["router"]["experts"]
            experts = [tuple(weights[f"{p}.mlp.e{j}.{n}"] for n in ("gate", "up", "down")) for j in range(n_e)]
            y = moe_ff(hn, weights[p + ".mlp.router"], ff["router"]["top"], experts)
            if margins is not None:
                margins.append(route_margin(hn, weights[p + ".mlp.router"], ff["router"]["top"]))
            x = x + m * layer_norm(y, weights[p + ".norm2b"], eps)
        streams.append(x.clone())
    z = layer_norm(x, weights["final.norm"], eps) @ weights["head"].to(F64).T
    cap = config["logit_softcap"]
    logits = cap * torch.tanh(z / cap)
    return (logits, torch.stack(streams)) if return_layers else logits
