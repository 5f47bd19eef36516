"""CPU tests of the Tevudra design: its config.json reader, the layout it builds, the tensor
names it expects, and identities of the plain implementation that the engine's arithmetic
rests on."""
import copy
import json

import pytest
import torch

import plain_tevudra as P
from tevudra_tiny import CONFIGS, make_weights


def test_config_is_read_and_laid_out():
    from llm_b200.config.model_config import parse_config
    from llm_b200.engine.model import Model
    cfg, _ = CONFIGS["P"]
    arch, typed = parse_config(json.loads(json.dumps(cfg)))
    assert arch.name == "Tevudra" and typed.width == 64 and typed.vocab == 200 and typed.norm_eps == 1e-6
    spec = arch.build_spec(typed)
    assert [l.cache_of for l in spec.layers] == [None, 0, None, 2]
    assert spec.layers[2].parts["ffn"] is None and spec.layers[2].parts["norm2"] is None
    model = Model(spec, torch.float32, torch.device("cpu"))
    assert len(model.cache_instances) == 2 and len(model.group_keys) == 1         # two layers keep latents, one group of pages
    assert all(not c.values and c.num_kv_heads == 1 for c in model.cache_instances)
    assert [c.head_dim for c in model.cache_instances] == [32, 24]
    assert [o.cache_instance for o in model.occurrences] == [0, 0, 1, 1]


def test_expected_tensors_match_the_weights_the_tests_draw():
    from llm_b200.weights.loader import expected_tensors
    for name, (cfg, _) in CONFIGS.items():
        exp = expected_tensors(cfg)
        w = make_weights(cfg, 1)
        assert set(exp) == set(w), name
        assert all(tuple(exp[n].shape) == tuple(w[n].shape) for n in exp), name
    exp = expected_tensors(CONFIGS["P"][0])
    assert "l1.mix.dkv" not in exp and "l0.mix.dkv.norm" in exp and "l2.norm2" not in exp
    assert exp["final.norm.alpha"].shape == () and "l3.mlp.shared.up" not in exp and "l1.mlp.shared.down" in exp


def test_random_model_folder_round_trip(tmp_path):
    from llm_b200.config.model_config import load_config
    from llm_b200.weights.loader import expected_tensors, write_random_model
    from llm_b200.weights.safetensors_io import SafetensorsFile
    cfg, _ = CONFIGS["R"]
    d = write_random_model(str(tmp_path / "m"), cfg, seed=3)
    arch, typed = load_config(d)
    assert arch.name == "Tevudra" and len(typed.layers) == 3
    f = SafetensorsFile(str(tmp_path / "m" / "model.safetensors"))
    assert set(f.entries) == set(expected_tensors(cfg))


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].update(kv_rank=40), "kv_rank"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_config_errors_are_named(change, message):
    from llm_b200.config.model_config import ConfigError, parse_config
    cfg = copy.deepcopy(CONFIGS["P"][0])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        parse_config(cfg)


def test_scores_and_values_through_the_latent_equal_the_expanded_form():
    """q . (Wuk c) = (Wuk^T q) . c and sum p (Wuv c) = Wuv (sum p c): the identity that lets the engine
    attend over the cached vectors themselves."""
    g = torch.Generator().manual_seed(0)
    T, W, H, D, V, R, scale = 9, 20, 3, 8, 6, 12, 0.3
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    h, c = r(T, W), r(T, R)
    w_q, w_uk, w_uv, w_g, w_o = r(H * D, W), r(H * D, R), r(H * V, R), r(H, W), r(W, H * V)
    want = P.latent_attention(h, c, w_q, w_uk, w_uv, w_g, w_o, H, D, V, scale)
    q = (h @ w_q.T).view(T, H, D)
    q_lat = torch.einsum("thd,hdr->thr", q, w_uk.view(H, D, R))
    out = torch.zeros(T, H, V, dtype=torch.float64)
    for i in range(T):
        p = torch.softmax(q_lat[i] @ c[: i + 1].T * scale, dim=-1)          # [H, i + 1]
        out[i] = torch.einsum("hr,hvr->hv", p @ c[: i + 1], w_uv.view(H, V, R))
    out = out * torch.sigmoid(h @ w_g.T)[:, :, None]
    assert torch.allclose(out.reshape(T, -1) @ w_o.T, want, atol=1e-10)


def test_plain_pieces():
    x = torch.tensor([[3.0, -4.0]])
    assert torch.allclose(P.rms(x, torch.ones(2), 0.0), x.double() / (12.5 ** 0.5))
    assert torch.allclose(P.dyt(x, 0.5, torch.tensor([2.0, 1.0]), torch.tensor([0.0, 1.0])),
                          torch.tanh(x.double() * 0.5) * torch.tensor([2.0, 1.0]).double() + torch.tensor([0.0, 1.0]).double())
    ids, wts = P.route(torch.eye(3), torch.tensor([[1.0, 0, 0], [0, 2.0, 0], [0, 0, 3.0], [0.5, 0.5, 0.5]]), torch.zeros(4), 2)
    assert ids.tolist() == [[0, 3], [1, 3], [2, 3]]
    assert torch.allclose(wts.sum(1), torch.ones(3, dtype=torch.float64))
    assert torch.allclose(wts[0], torch.softmax(torch.tensor([1.0, 0.5], dtype=torch.float64), 0))
    assert torch.allclose(P.relu2_ff(torch.tensor([[1.0, -1.0]]), torch.eye(2) * 2, torch.eye(2)), torch.tensor([[4.0, 0.0]], dtype=torch.float64))
