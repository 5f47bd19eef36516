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


class SandwichBlock:
    """x += m * post1(mixer(norm1(x))); x += m * post2(ffn(norm2(x))): every sublayer has a norm before it
    and a norm on its output, and the normed output joins the residual scaled by m.  The output is left
    pending on the stream with its norm still to do (norm.attach), so that the next norm adds and norms
    in one pass.  A layer without a feed-forward leaves out norm2, ffn and post2."""

    role = "block"
    roles = {"norm1": "norm", "mixer": "mixer", "post1": "norm", "norm2": "norm", "ffn": "ffn", "post2": "norm"}

    def __init__(self, part_specs, dtype, device, residual_mult: float = 1.0):
        self.mult = float(residual_mult)
        optional = ("norm2", "ffn", "post2") if part_specs.get("ffn") is None else ()
        missing = [r for r in self.roles if part_specs.get(r) is None and r not in optional]
        if missing:
            raise ValueError(f"sandwich block lacks parts {missing}")
        self.parts = {r: build_part(self.roles[r], part_specs[r], dtype, device) if part_specs.get(r) is not None else None
                      for r in self.roles}
        for r in ("post1", "post2"):
            if self.parts[r] is not None and not hasattr(self.parts[r], "attach"):
                raise ValueError(f"sandwich block: the norm '{part_specs[r].kind}' cannot stand behind a sublayer (no attach)")
        self.mixer, self.ffn = self.parts["mixer"], self.parts["ffn"]

    def forward(self, stream: ResidualStream, ctx, view) -> None:
        p = self.parts
        p["post1"].attach(stream, self.mixer.forward(p["norm1"].forward(stream, ctx), ctx, view), self.mult)
        if self.ffn is not None:
            p["post2"].attach(stream, self.ffn.forward(p["norm2"].forward(stream, ctx), ctx), self.mult)


register_part("block", "sandwich", SandwichBlock)


class StreamBlock:
    """A place in the layer order that holds no layer but one transform of the whole stream (role "stream")."""

    role = "block"

    def __init__(self, part_specs, dtype, device):
        self.parts = {"stream": build_part("stream", part_specs["stream"], dtype, device)}
        self.mixer = None

    def forward(self, stream: ResidualStream, ctx, view) -> None:
        self.parts["stream"].forward(stream, ctx)


register_part("block", "stream", StreamBlock)
