"""Tiny Fopivik configurations and weights for the tests.

The configurations differ from each other in every size and constant and include the corner values:
one head, one kv head and as many as query heads, key and value sizes that differ, rotation of the
whole head, of part of it and of nothing, with and without frequency scaling, windows smaller and
larger than a page, no kept tokens and more kept tokens than a page holds, one chosen expert and
every expert chosen, a layer without a feed-forward, loops at the start, in the middle, over
everything and of a single pass, and no loop at all.  The weights are drawn here (not by the
package), with queries scaled so that attention is peaked and decays spread between fast and slow.
"""
from __future__ import annotations

import math

import torch


def attn(heads, kv_heads, dim, vdim, size, keep, rot_dims, scale, softcap=24.0, base=10000.0, scaling=None):
    rot = {"dims": rot_dims, "base": base}
    if scaling:
        rot["scaling"] = scaling
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                           "mask": {"size": size, "keep_first": keep}, "rot": rot,
                                           "scale": scale, "softcap": softcap}}


def gla(heads, dim, vdim, tau):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def config(width, vocab, layers, loop=None, eps=1e-5, mult=0.5, cap=25.0):
    cfg = {"architecture": "Fopivik", "width": width, "vocab": vocab, "norm": {"eps": eps}, "residual_mult": mult,
           "logit_softcap": cap, "layers": layers}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


SCALING = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}

# A: both mixers, a loop over the first two layers, window and kept tokens inside one page
CONFIG_A = config(64, 200, [
    layer(attn(4, 2, 16, 8, size=12, keep=3, rot_dims=8, scale=0.3, scaling=SCALING), moe(4, 2, 24)),
    layer(gla(2, 16, 24, tau=8.0), moe(3, 3, 16)),
    layer(attn(2, 1, 24, 24, size=40, keep=0, rot_dims=24, scale=0.25, softcap=12.0), None),
    layer(gla(1, 40, 8, tau=2.0), moe(5, 1, 32)),
], loop=(0, 2, 2), eps=1e-5, mult=0.4, cap=18.0)
# B: sizes the tensor-core kernels take; a loop in the middle that runs three times; kept tokens beyond a page
CONFIG_B = config(128, 333, [
    layer(gla(4, 32, 32, tau=16.0), moe(8, 2, 64)),
    layer(attn(8, 2, 64, 64, size=33, keep=20, rot_dims=32, scale=0.12, base=500000.0, scaling=SCALING), moe(6, 4, 40)),
    layer(attn(4, 4, 32, 64, size=100, keep=1, rot_dims=0, scale=0.2), moe(2, 1, 128)),
    layer(gla(2, 64, 128, tau=4.0), None),
], loop=(1, 3, 3), eps=1e-6, mult=0.35, cap=28.0)
# C: nothing on a grid of 8 (width, head sizes, feed-forward sizes); a loop over everything, once
CONFIG_C = config(100, 97, [
    layer(attn(3, 1, 10, 6, size=7, keep=2, rot_dims=6, scale=0.35), moe(5, 2, 14)),
    layer(gla(3, 10, 14, tau=3.0), moe(7, 3, 10)),
    layer(attn(5, 5, 6, 14, size=19, keep=9, rot_dims=2, scale=0.4, softcap=8.0), moe(1, 1, 22)),
], loop=(0, 3, 1), eps=3e-6, mult=1.0, cap=40.0)
# D: no loop; one attention layer, nothing else: what the attention does shows in the logits undiluted
CONFIG_D = config(64, 120, [layer(attn(2, 1, 32, 16, size=24, keep=4, rot_dims=8, scale=0.25, softcap=30.0), None)],
                  mult=1.0, cap=50.0)
# E: one gla layer alone, slow decays (a long memory), a loop of four passes over it
CONFIG_E = config(48, 150, [layer(gla(2, 24, 16, tau=32.0), None)], loop=(0, 1, 4), mult=0.7, cap=35.0)
# F: attention that decodes on the tensor-core kernels' sizes, window wider than any request here
CONFIG_F = config(128, 256, [
    layer(attn(6, 2, 64, 64, size=4096, keep=5, rot_dims=24, scale=0.11, base=5e5, scaling=SCALING), moe(4, 2, 64)),
    layer(attn(4, 2, 128, 128, size=50, keep=0, rot_dims=128, scale=0.08), moe(4, 2, 64)),
], loop=(1, 2, 2), mult=0.45)

CONFIGS = {"A": (CONFIG_A, 16), "B": (CONFIG_B, 16), "C": (CONFIG_C, 8), "D": (CONFIG_D, 16), "E": (CONFIG_E, 32),
           "F": (CONFIG_F, 16)}   # name -> (config, page size)


def make_weights(cfg: dict, seed: int, peak: float = 1.5, decay_rank: int = 6, slow: float = 0.0) -> dict:
    """Seeded weights by tensor name, every value representable in bfloat16 (so that the 32-bit engine, the
    bfloat16 engine and the float64 plain implementation read the same numbers).  peak: the standard
    deviation the attention scores are scaled to; slow: added to the decay's bias (larger: longer memory)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    rnd = lambda *shape, std=1.0: (torch.randn(*shape, generator=g) * std).to(torch.bfloat16).float()
    gain = lambda n: (1.0 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16).float()
    w = {"embed": rnd(cfg["vocab"], W), "head": rnd(cfg["vocab"], W, std=2.0 / math.sqrt(W)), "final.norm": gain(W)}
    loop = cfg.get("loop")
    if loop:
        eye = torch.cat([torch.eye(W), 0.5 * torch.eye(W)], dim=1)
        w["loop.in"] = (eye + torch.randn(W, 2 * W, generator=g) * 0.5 / math.sqrt(W)).to(torch.bfloat16).float()
        w["loop.step"] = rnd(loop["times"], W, std=0.3)
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}", lay["mixer"]
        for n in ("norm1", "norm1b"):
            w[f"{p}.{n}"] = gain(W)
        H, D, V = m["heads"], m["dim"], m["vdim"]
        if lay["type"] == "attention":
            G = m["kv_heads"]
            w[p + ".mix.q"] = rnd(H * D, W, std=peak / (math.sqrt(D) * m["scale"]) / math.sqrt(W))
            w[p + ".mix.k"] = rnd(G * D, W, std=1.0 / math.sqrt(W))
            w[p + ".mix.v"] = rnd(G * V, W, std=1.0 / math.sqrt(W))
        else:
            w[p + ".mix.q"] = rnd(H * D, W, std=1.0 / math.sqrt(W))
            w[p + ".mix.k"] = rnd(H * D, W, std=1.0 / math.sqrt(W))
            w[p + ".mix.v"] = rnd(H * V, W, std=1.0 / math.sqrt(W))
            w[p + ".mix.g"] = rnd(H * V, W, std=1.5 / math.sqrt(W))
            w[p + ".mix.norm"] = gain(V)
            w[p + ".mix.a1"] = rnd(decay_rank, W, std=1.0 / math.sqrt(W))
            w[p + ".mix.a2"] = rnd(H * D, decay_rank, std=2.0 / math.sqrt(decay_rank))
            w[p + ".mix.a2.b"] = rnd(H * D, std=1.5) + slow
        w[p + ".mix.o"] = rnd(W, H * V, std=1.0 / math.sqrt(H * V))
        ff = lay["mlp"]
        if ff is None:
            continue
        for n in ("norm2", "norm2b"):
            w[f"{p}.{n}"] = gain(W)
        E, F = ff["router"]["experts"], ff["expert"]["ff"]
        # router logits spread wide, so that few tokens sit on the edge between two experts (a loop sends a token
        # through the same router several times)
        w[p + ".mlp.router"] = rnd(E, W, std=4.0 / math.sqrt(W))
        for e in range(E):
            w[f"{p}.mlp.e{e}.gate"] = rnd(F, W, std=1.5 / math.sqrt(W))
            w[f"{p}.mlp.e{e}.up"] = rnd(F, W, std=1.5 / math.sqrt(W))
            w[f"{p}.mlp.e{e}.down"] = rnd(W, F, std=1.0 / math.sqrt(F))
    return w


def random_config(seed: int) -> dict:
    """Sizes, constants, layer order and loop drawn from a seed."""
    import random
    rng = random.Random(seed)
    width = rng.choice([40, 56, 72, 88, 100, 128, 136])
    layers = []
    for _ in range(rng.randint(2, 5)):
        if rng.random() < 0.5:
            kv = rng.choice([1, 2, 3])
            dim = rng.choice([4, 8, 10, 16, 24, 32, 64])
            rot = rng.choice([0, 2, dim // 2 // 2 * 2, dim // 2 * 2])
            mixer = attn(kv * rng.randint(1, 3), kv, dim, rng.choice([4, 8, 12, 16, 32, 64]), size=rng.choice([1, 5, 16, 17, 50, 300]),
                         keep=rng.choice([0, 0, 1, 5, 16, 40]), rot_dims=rot, scale=rng.uniform(0.1, 0.5),
                         softcap=rng.choice([5.0, 15.0, 50.0]), base=rng.choice([100.0, 10000.0, 1e6]),
                         scaling=rng.choice([None, SCALING, {"factor": 8.0, "low": 2.0, "high": 8.0, "original": 32}]))
        else:
            mixer = gla(rng.randint(1, 4), rng.choice([4, 10, 16, 24, 48, 80]), rng.choice([4, 8, 12, 16, 40, 64]),
                        tau=rng.choice([1.0, 4.0, 16.0, 64.0]))
        if rng.random() < 0.75:
            experts = rng.randint(1, 9)
            mlp = moe(experts, rng.randint(1, experts), rng.choice([8, 12, 24, 40]))
        else:
            mlp = None
        layers.append(layer(mixer, mlp))
    n = len(layers)
    loop = None
    if rng.random() < 0.8:
        start = rng.randint(0, n - 1)
        loop = (start, rng.randint(start + 1, n), rng.randint(1, 3))
    return config(width, rng.choice([61, 128, 200, 333]), layers, loop=loop, eps=rng.choice([1e-6, 1e-5, 1e-3]),
                  mult=rng.choice([0.2, 0.5, 1.0]), cap=rng.choice([10.0, 30.0, 100.0]))


def make_engine(cfg, weights, dtype, page, num_blocks, max_tokens=512, max_seqs=4, poison=True, graphs=False, max_seq_len=None):
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine
    opts = EngineOptions(dtype=dtype, kv_block_size=page, max_num_seqs=max_seqs, max_num_batched_tokens=max_tokens,
                         num_kv_blocks=num_blocks, use_cuda_graphs=graphs, poison_freed_pages=poison,
                         max_seq_len=max_seq_len or min(num_blocks * page, 4096))
    return Engine(None, opts, random_config=cfg, tensors={k: v.clone() for k, v in weights.items()})
