"""CPU tests of the Fopivik design: its config.json reader, the layout it builds (loops, caches, states), the
tensor names it expects, the pool's kept pages, and identities of the plain implementation."""
import copy
import json
import random

import pytest
import torch

import plain_fopivik as P
from fopivik_tiny import CONFIGS, make_weights, random_config
from llm_b200.cache.manager import CacheError, CacheManager, GroupSpec


def test_config_is_read_and_laid_out():
    from llm_b200.config.model_config import parse_config
    from llm_b200.engine.model import Model
    cfg, _ = CONFIGS["A"]
    arch, typed = parse_config(json.loads(json.dumps(cfg)))
    assert arch.name == "Fopivik" and typed.width == 64 and typed.vocab == 200 and typed.norm_eps == 1e-5
    assert typed.loop == (0, 2, 2) and typed.residual_mult == 0.4 and typed.logit_softcap == 18.0
    spec = arch.build_spec(typed)
    # four layers and one place per pass that holds the re-entry; layers 0 and 1 run twice
    kinds = [spec.layers[i].block for i in spec.order]
    assert kinds == ["stream", "sandwich", "sandwich", "stream", "sandwich", "sandwich", "sandwich", "sandwich"]
    assert [i for i in spec.order if spec.layers[i].block == "sandwich"] == [0, 1, 0, 1, 2, 3]
    assert spec.layers[2].parts["ffn"] is None and spec.layers[2].parts["post2"] is None
    model = Model(spec, torch.float32, torch.device("cpu"))
    # every run of an attention layer has pages of its own, every run of a gla layer a state of its own
    assert len(model.cache_instances) == 3 and len(model.state_needs) == 3
    assert [(c.num_kv_heads, c.head_dim, c.value_dim) for c in model.cache_instances] == [(2, 16, 8), (2, 16, 8), (1, 24, 24)]
    assert sorted(model.group_keys) == [("window", 12, 3), ("window", 40, 0)]
    assert [n.shape for n in model.state_needs] == [(2, 16, 24), (2, 16, 24), (1, 40, 8)]


@pytest.mark.parametrize("loop,order", [
    (None, [0, 1, 2, 3]), ((0, 4, 1), ["s", 0, 1, 2, 3]), ((1, 2, 3), [0, "s", 1, "s", 1, "s", 1, 2, 3]),
    ((2, 4, 2), [0, 1, "s", 2, 3, "s", 2, 3])])
def test_loops_anywhere(loop, order):
    from llm_b200.config.model_config import parse_config
    cfg = copy.deepcopy(CONFIGS["A"][0])
    cfg.pop("loop")
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    arch, typed = parse_config(cfg)
    spec = arch.build_spec(typed)
    assert ["s" if spec.layers[i].block == "stream" else i for i in spec.order] == order
    passes = [spec.layers[i].parts["stream"].params["pass_index"] for i in spec.order if spec.layers[i].block == "stream"]
    assert passes == list(range(loop[2] if loop else 0))
    # the plain side walks the same layers, and opens a pass where the engine has its re-entry
    plain = P.layer_order(4, cfg.get("loop"))
    assert [i for i, _ in plain] == [i for i in order if i != "s"]
    assert [t for _, t in plain if t is not None] == passes


def test_expected_tensors_match_the_weights_the_tests_draw(tmp_path):
    from llm_b200.weights.loader import expected_tensors, write_random_model
    from llm_b200.weights.safetensors_io import SafetensorsFile
    for name, (cfg, _) in CONFIGS.items():
        exp = expected_tensors(cfg)
        w = make_weights(cfg, 1)
        assert set(exp) == set(w), name
        assert all(exp[n].fits(w[n].shape) for n in exp), name
    exp = expected_tensors(CONFIGS["A"][0])
    assert exp["l1.mix.a1"].free_dims == (0,) and exp["l1.mix.a2"].free_dims == (1,) and not exp["l1.mix.q"].free_dims
    assert "l2.norm2" not in exp and "l2.norm1b" in exp and exp["loop.step"].shape == (2, 64) and "l0.mix.g" not in exp
    assert "loop.in" not in expected_tensors(CONFIGS["D"][0])
    d = write_random_model(str(tmp_path / "m"), CONFIGS["C"][0], seed=3)
    f = SafetensorsFile(str(tmp_path / "m" / "model.safetensors"))
    assert set(f.entries) == set(expected_tensors(CONFIGS["C"][0]))


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "positive"),
    (lambda c: c["layers"][1]["mixer"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=4), "top"),
    (lambda c: c["loop"].update(stop=5), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("low"), "low"),
])
def test_config_errors_name_the_key(change, message):
    from llm_b200.config.model_config import ConfigError, parse_config
    cfg = copy.deepcopy(CONFIGS["A"][0])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        parse_config(cfg)


def test_random_configurations_parse_and_name_their_tensors():
    from llm_b200.weights.loader import expected_tensors
    for seed in range(2000, 2030):
        cfg = random_config(seed)
        assert set(expected_tensors(cfg)) == set(make_weights(cfg, 1))


# ---- the pool: a window group that keeps a request's first tokens ----
@pytest.mark.parametrize("page,window,keep", [(8, 20, 3), (8, 20, 8), (8, 5, 9), (16, 24, 40), (4, 1, 1), (8, 16, 0)])
def test_window_group_keeps_the_first_pages(page, window, keep):
    c = CacheManager([GroupSpec("window", page, 64, window=window, keep_first=keep)], 2, 400)
    c.admit("a")
    pos = 0
    kept_pages = -(-keep // page)
    for n in (30, 1, 1, 7, 25, 2, 60, 1, 1, 90):
        need = c.pages_needed("a", n)[0]
        free = c.num_free_pages(0)
        assert c.extend("a", n) == pos
        assert c.num_free_pages(0) == free - need              # what was announced is what moved
        pos += n
        c.check()
        lowest_key = max(0, pos - n - window + 1)               # first key the first new token could see through the window
        for i, p in enumerate(c.table(0, "a")):
            if i < kept_pages or (i + 1) * page > lowest_key:
                assert p >= 0, (i, pos)
            else:
                assert p == -1, (i, pos)
        # every key that any new token may see is held
        for q in range(pos - n, pos):
            for j in range(q + 1):
                if P.visible(q, j, window, keep):
                    assert c.physical_slot(0, "a", j) >= 0
    c.release("a")
    assert c.num_free_pages(0) == 64
    c.check()


@pytest.mark.parametrize("seed", range(4))
def test_random_orders_with_kept_pages_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    c = CacheManager([GroupSpec("window", 8, 24, window=rng.choice([5, 16, 33]), keep_first=rng.choice([1, 8, 20])),
                      GroupSpec("full", 8, 30)], 5, 200)
    live, next_id = {}, 0
    for _ in range(500):
        op = rng.random()
        if op < 0.25 and c.num_free_slots():
            c.admit(next_id); live[next_id] = 0; next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 16, 40])
            if c.can_extend(rid, n):
                assert c.extend(rid, n) == live[rid]
                live[rid] += n
            else:
                with pytest.raises(CacheError):
                    c.extend(rid, n)
        elif live:
            rid = rng.choice(list(live))
            c.release(rid); del live[rid]
        c.check()
    for rid in list(live):
        c.release(rid)
    c.check()
    assert all(c.num_free_pages(g) == c.group_spec(g).num_pages for g in range(c.num_groups))


# ---- identities of the plain implementation ----
def test_plain_prefix_property_and_mechanisms():
    cfg, _ = CONFIGS["A"]
    w = make_weights(cfg, 2)
    toks = [5, 17, 3, 99, 140, 7, 7, 23, 51, 8, 160, 2, 44, 90, 31, 12, 77, 5, 6, 100]
    full = P.forward(cfg, w, toks)
    assert torch.allclose(P.forward(cfg, w, toks[:9]), full[:9], atol=1e-12)        # causal: a prefix stands alone
    assert float(full.abs().max()) < cfg["logit_softcap"]
    # the sink: weights of a row sum to less than one; with a huge score on one key nearly to one
    q, k, v = torch.zeros(1, 1, 4, dtype=torch.float64), torch.zeros(1, 1, 4, dtype=torch.float64), torch.ones(1, 1, 2, dtype=torch.float64)
    assert torch.allclose(P.sink_attention(q, k, v, 1.0, 10.0, 4, 0), torch.full((1, 1, 2), 0.5, dtype=torch.float64))
    # window and kept tokens
    assert [j for j in range(10) if P.visible(9, j, 3, 2)] == [0, 1, 7, 8, 9]
    # the decay: sigmoid(z)^(1/tau)
    z = torch.tensor([[-2.0, 0.0, 3.0]], dtype=torch.float64)
    a = P.decay(torch.eye(3, dtype=torch.float64)[:1], torch.eye(3), z.T.repeat(1, 3) * torch.eye(3), torch.zeros(3), 4.0)
    assert torch.allclose(a[0, 0], torch.sigmoid(z[0, 0]) ** 0.25)
    # the recurrence against its unrolled sum
    g = torch.Generator().manual_seed(0)
    qq, kk, aa = (torch.rand(5, 1, 3, generator=g, dtype=torch.float64) for _ in range(3))
    vv = torch.rand(5, 1, 2, generator=g, dtype=torch.float64)
    o = P.gla_recurrence(qq, kk, vv, aa)
    t = 4
    want = sum(((qq[t, 0] * kk[j, 0] * aa[j + 1:t + 1, 0].prod(0)).sum() * vv[j, 0]) for j in range(t + 1))
    assert torch.allclose(o[t, 0], want)
