"""Tevudra laid out as a ModelSpec: a decoder whose config lists its layers one by one.

Every layer is pre-norm with Dynamic Tanh norms: x += mixer(dyt(x)); x += ff(dyt(x)), the
second half absent where the layer has no feed-forward.  The mixer is a latent attention
without positions (a layer may read the latents an earlier layer cached); the feed-forward
is dense with a squared relu, or routed (erf gelu experts, softmax over the chosen logits,
an optional shared expert).  Tensors: `embed`, `l<i>.norm1|norm2` (+ `.b`, `.alpha`),
`l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.model_config import TevudraConfig, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec


def build_tevudra_spec(cfg: TevudraConfig) -> ModelSpec:
    norm = lambda prefix: PartSpec("dyt", {"size": cfg.width}, prefix)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m, ff = f"l{i}", layer["mixer"], layer["mlp"]
        parts = {
            "norm1": norm(p + ".norm1"),
            "mixer": PartSpec("latent_attention", {
                "hidden_size": cfg.width, "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                "rank": m["kv_rank"], "scale": m["scale"], "eps": cfg.norm_eps, "gated": True,
                "shares_cache": m["kv_from"] is not None}, p + ".mix"),
            "norm2": None, "ffn": None,
        }
        if ff is not None:
            parts["norm2"] = norm(p + ".norm2")
            if ff["kind"] == "dense":
                parts["ffn"] = PartSpec("mlp", {"hidden_size": cfg.width, "intermediate_size": ff["ff"],
                                                "activation": "relu2"}, p + ".mlp")
            else:
                parts["ffn"] = PartSpec("routed", {"hidden_size": cfg.width, "experts": ff["experts"], "top": ff["top"],
                                                   "expert_size": ff["ff"], "activation": "gelu", "router_bias": True,
                                                   "shared_size": ff["shared_ff"]}, p + ".mlp")
        layers.append(LayerSpec("prenorm", parts, cache_of=m["kv_from"]))
    spec = ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=cfg.max_position,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight_name": ""}, "embed"),
        layers=tuple(layers), order=tuple(range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"hidden_size": cfg.width, "vocab_size": cfg.vocab, "weight_name": ""}, "head"),
        eos_token_id=cfg.eos_token_id,
    )
    spec.validate()
    return spec


register_architecture("Tevudra", TevudraConfig, build_tevudra_spec)
