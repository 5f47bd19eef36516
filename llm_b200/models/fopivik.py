"""Fopivik laid out as a ModelSpec: a decoder whose config lists its layers one by one, a run of which
may be repeated with the same weights.

Every layer norms each sublayer on both sides (LayerNorm with a weight, no bias) and scales what joins
the residual: x += m ln(mixer(ln(x))); x += m ln(ff(ln(x))).  The mixer is a grouped-query attention
(pairs rotated on part of a head with wavelength-scaled frequencies, soft-capped scores, a window that
keeps the request's first tokens, a sink in the softmax) or a gated linear attention (a matrix state
per head); the feed-forward a mixture of gated experts weighted by their shares of the softmax over
all experts.  Layers start..stop-1 of `loop` run `times` times; each pass opens with the stream mixed
anew with the token embedding plus a vector per pass, and keeps a cache or state of its own.  The
logits pass a LayerNorm, the head and a soft cap.  Tensors: `embed`, `loop.in`, `loop.step`,
`l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.model_config import FopivikConfig, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec


def build_fopivik_spec(cfg: FopivikConfig) -> ModelSpec:
    norm = lambda prefix: PartSpec("layernorm", {"size": cfg.width, "eps": cfg.norm_eps}, prefix)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m, ff = f"l{i}", layer["mixer"], layer["mlp"]
        if layer["type"] == "attention":
            position = PartSpec("rope_pairs", {"dims": m["rot_dims"], "base": m["rot_base"], "scaling": m["rot_scaling"]})
            mixer = PartSpec("attention", {
                "hidden_size": cfg.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "value_dim": m["vdim"], "window": m["window"], "keep_first": m["keep_first"], "scale": m["scale"],
                "softcap": m["softcap"], "sink": True, "position": position,
                "names": {"q": "q", "k": "k", "v": "v", "o": "o"}}, p + ".mix")
        else:
            mixer = PartSpec("gla", {"hidden_size": cfg.width, "num_heads": m["heads"], "head_dim": m["dim"],
                                     "value_dim": m["vdim"], "tau": m["tau"], "eps": cfg.norm_eps}, p + ".mix")
        parts = {"norm1": norm(p + ".norm1"), "mixer": mixer, "post1": norm(p + ".norm1b"),
                 "norm2": None, "ffn": None, "post2": None}
        if ff is not None:
            parts.update({
                "norm2": norm(p + ".norm2"), "post2": norm(p + ".norm2b"),
                "ffn": PartSpec("routed", {"hidden_size": cfg.width, "experts": ff["experts"], "top": ff["top"],
                                           "expert_size": ff["ff"], "activation": "silu", "gated": True,
                                           "router": "softmax_all", "router_bias": False}, p + ".mlp")})
        layers.append(LayerSpec("sandwich", parts, params={"residual_mult": cfg.residual_mult}))
    n = len(layers)
    order = list(range(n))
    if cfg.loop is not None:
        start, stop, times = cfg.loop
        order = list(range(start))
        for t in range(times):
            # the opening of pass t is a place of its own in the order: it holds no layer, only the re-entry
            layers.append(LayerSpec("stream", {"stream": PartSpec("embedding_reinjection", {
                "hidden_size": cfg.width, "vocab_size": cfg.vocab, "passes": times, "pass_index": t,
                "table_name": "embed"}, "loop")}))
            order += [len(layers) - 1] + list(range(start, stop))
        order += list(range(stop, n))
    spec = ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=cfg.max_position,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight_name": ""}, "embed"),
        layers=tuple(layers), order=tuple(order),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"hidden_size": cfg.width, "vocab_size": cfg.vocab, "weight_name": "",
                                  "softcap": cfg.logit_softcap}, "head"),
        eos_token_id=cfg.eos_token_id,
    )
    spec.validate()
    return spec


register_architecture("Fopivik", FopivikConfig, build_fopivik_spec)
