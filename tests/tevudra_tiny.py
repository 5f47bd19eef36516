"""Tiny Tevudra configurations and weights for the tests.

The configurations differ from each other in every size and constant, and include the corner
values: one head, one chosen expert, every expert chosen, no shared expert, a layer without a
feed-forward, key and value sizes that differ, ranks on and off the 16-grid, ranks the
tensor-core kernels take (64, 128) and a rank wider than 256, two layers that read the same
layer's latents.  The weights are drawn here (not by the package), with queries scaled so
that the attention is peaked: a wrong key, page or mask edge then moves the logits by far
more than rounding does.
"""
from __future__ import annotations

import math

import torch


def _mixer(heads, dim, vdim, rank, scale, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, shared=None):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


CONFIG_P = {"architecture": "Tevudra", "width": 64, "vocab": 200, "norm": {"eps": 1e-6}, "layers": [
    _layer(_mixer(4, 16, 8, 32, 0.3), _dense(96)),
    _layer(_mixer(2, 24, 16, 32, 0.21, kv_from=0), _moe(4, 2, 40, shared=48)),
    _layer(_mixer(3, 8, 8, 24, 0.4), None),
    _layer(_mixer(1, 32, 32, 24, 0.15, kv_from=2), _moe(3, 3, 16)),
]}
CONFIG_Q = {"architecture": "Tevudra", "width": 128, "vocab": 333, "norm": {"eps": 1e-5}, "layers": [
    _layer(_mixer(4, 32, 64, 64, 0.2), _moe(8, 1, 64, shared=32)),
    _layer(_mixer(8, 16, 16, 64, 0.25, kv_from=0), _dense(256)),
    _layer(_mixer(2, 64, 32, 128, 0.125), _dense(128)),
    _layer(_mixer(16, 8, 8, 128, 0.35, kv_from=2), _moe(5, 2, 24, shared=72)),
]}
CONFIG_R = {"architecture": "Tevudra", "width": 96, "vocab": 150, "norm": {"eps": 1e-4}, "layers": [
    _layer(_mixer(2, 16, 16, 320, 0.25), _dense(64)),
    _layer(_mixer(3, 16, 8, 320, 0.2, kv_from=0), _moe(6, 4, 32, shared=16)),
    _layer(_mixer(1, 48, 24, 320, 0.1, kv_from=0), _dense(40)),
]}
# one layer, nothing but the mixer: what the attention does shows in the logits undiluted
CONFIG_S = {"architecture": "Tevudra", "width": 64, "vocab": 120, "norm": {"eps": 1e-5}, "layers": [
    _layer(_mixer(2, 16, 16, 48, 0.25), None),
]}

# the same with a rank that the tensor-core attention kernels take, and more heads
CONFIG_T = {"architecture": "Tevudra", "width": 64, "vocab": 120, "norm": {"eps": 1e-5}, "layers": [
    _layer(_mixer(4, 16, 8, 64, 0.25), None),
]}

# U: nothing on a grid of 8 or 16 (width, vocabulary, head sizes, ranks, feed-forward sizes), so that bfloat16 too
# runs the any-size kernels; a rank above 128 that is not a multiple of 16
CONFIG_U = {"architecture": "Tevudra", "width": 100, "vocab": 97, "norm": {"eps": 3e-6}, "layers": [
    _layer(_mixer(3, 10, 6, 20, 0.3), _moe(5, 2, 14, shared=22)),
    _layer(_mixer(5, 6, 14, 20, 0.45, kv_from=0), _dense(30)),
    _layer(_mixer(2, 12, 10, 136, 0.28), _moe(7, 3, 10)),
]}

# V: ranks above 128 on the 16-grid, which in bfloat16 decode on the CUDA-core split-key kernel
CONFIG_V = {"architecture": "Tevudra", "width": 80, "vocab": 130, "norm": {"eps": 1e-5}, "layers": [
    _layer(_mixer(2, 24, 16, 160, 0.2), _dense(48)),
    _layer(_mixer(4, 16, 16, 256, 0.25), _moe(4, 2, 24, shared=16)),
    _layer(_mixer(3, 8, 24, 160, 0.3, kv_from=0), None),
]}

CONFIGS = {"V": (CONFIG_V, 16), "U": (CONFIG_U, 32), "P": (CONFIG_P, 16), "Q": (CONFIG_Q, 16), "R": (CONFIG_R, 8), "S": (CONFIG_S, 16), "T": (CONFIG_T, 16)}   # name -> (config, page size)


def make_weights(cfg: dict, seed: int, peak: float = 1.5) -> dict:
    """Seeded weights by tensor name, every value representable in bfloat16 (so that the 32-bit
    engine, the bfloat16 engine and the float64 plain implementation read the same numbers).
    peak: the standard deviation the attention scores are scaled to."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    rnd = lambda *shape, std=1.0: (torch.randn(*shape, generator=g) * std).to(torch.bfloat16).float()
    w = {"embed": rnd(cfg["vocab"], W), "head": rnd(cfg["vocab"], W, std=1.0 / math.sqrt(W))}

    def norm(name):
        w[name] = (1.0 + 0.1 * torch.randn(W, generator=g)).to(torch.bfloat16).float()
        w[name + ".b"] = rnd(W, std=0.1)
        w[name + ".alpha"] = torch.tensor(0.4 + 0.8 * float(torch.rand((), generator=g))).to(torch.bfloat16).float()

    norm("final.norm")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        H, D, V, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
        norm(p + ".norm1")
        q_std = peak / (math.sqrt(D) * 0.6 * m["scale"]) / math.sqrt(W)
        w[p + ".mix.q"] = rnd(H * D, W, std=q_std)
        if m.get("kv_from") is None:
            w[p + ".mix.dkv"] = rnd(R, W, std=1.0 / math.sqrt(W))
            w[p + ".mix.dkv.norm"] = (1.0 + 0.1 * torch.randn(R, generator=g)).to(torch.bfloat16).float()
        w[p + ".mix.uk"] = rnd(H * D, R, std=1.0 / math.sqrt(R))
        w[p + ".mix.uv"] = rnd(H * V, R, std=1.0 / math.sqrt(R))
        w[p + ".mix.g"] = rnd(H, W, std=2.0 / math.sqrt(W))
        w[p + ".mix.o"] = rnd(W, H * V, std=0.7 / math.sqrt(H * V))
        ff = layer["mlp"]
        if ff is None:
            continue
        norm(p + ".norm2")
        if ff["kind"] == "dense":
            w[p + ".mlp.up"] = rnd(ff["ff"], W, std=1.5 / math.sqrt(W))
            w[p + ".mlp.down"] = rnd(W, ff["ff"], std=0.7 / math.sqrt(ff["ff"]))
        else:
            E, F = ff["router"]["experts"], ff["expert"]["ff"]
            w[p + ".mlp.router"] = rnd(E, W, std=2.0 / math.sqrt(W))
            w[p + ".mlp.router.b"] = rnd(E, std=0.5)
            for e in range(E):
                w[f"{p}.mlp.e{e}.up"] = rnd(F, W, std=1.5 / math.sqrt(W))
                w[f"{p}.mlp.e{e}.down"] = rnd(W, F, std=1.0 / math.sqrt(F))
            if ff.get("shared"):
                S = ff["shared"]["ff"]
                w[p + ".mlp.shared.up"] = rnd(S, W, std=1.5 / math.sqrt(W))
                w[p + ".mlp.shared.down"] = rnd(W, S, std=0.7 / math.sqrt(S))
    return w


def make_engine(cfg, weights, dtype, page, num_blocks, max_tokens=512, max_seqs=4, poison=True, graphs=False):
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine
    opts = EngineOptions(dtype=dtype, kv_block_size=page, max_num_seqs=max_seqs, max_num_batched_tokens=max_tokens,
                         num_kv_blocks=num_blocks, use_cuda_graphs=graphs, poison_freed_pages=poison,
                         max_seq_len=min(num_blocks * page, 4096))
    return Engine(None, opts, random_config=cfg, tensors={k: v.clone() for k, v in weights.items()})
