"""How a layer's parts are arranged on the residual stream.

"prenorm": x += mixer(norm1(x)); x += ffn(norm2(x)), the arrangement of the
reference's block (model/llm/tiny_llama.cpp:29-34).  Each sum is left pending on
the stream and folded in by the next norm.  A layer without a feed-forward leaves
out norm2 and ffn: it is x += mixer(norm1(x)) alone.
"""
from __future__ import annotations

from .base import ResidualStream, build_part, register_part


class PreNormBlock:
    role = "block"
    roles = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "ffn": "ffn"}

    def __init__(self, part_specs, dtype, device):
        optional = ("norm2", "ffn") if part_specs.get("ffn") is None else ()
        missing = [r for r in self.roles if part_specs.get(r) is None and r not in optional]
        if missing:
            raise ValueError(f"prenorm block lacks parts {missing}")
        self.parts = {r: build_part(self.roles[r], part_specs[r], dtype, device) if part_specs.get(r) is not None else None
                      for r in self.roles}
        self.norm1, self.mixer = self.parts["norm1"], self.parts["mixer"]
        self.norm2, self.ffn = self.parts["norm2"], self.parts["ffn"]

    def forward(self, stream: ResidualStream, ctx, view) -> None:
        stream.pending = self.mixer.forward(self.norm1.forward(stream, ctx), ctx, view)
        if self.ffn is not None:
            stream.pending = self.ffn.forward(self.norm2.forward(stream, ctx), ctx)


register_part("block", "prenorm", PreNormBlock)
