"""Movarax without a GPU: the configuration and the tensor names, and the plain implementation held to itself (the
recurrence against its closed form, attention over latents against attention over full-size keys, the weight on an
expert's input against its closed form)."""
import json

import numpy as np
import pytest

import movarax_models as mm
from plain import movarax_plain as plain


@pytest.mark.parametrize("name", sorted(mm.CONFIGS))
def test_a_configuration_is_read_written_and_named(tmp_path, name):
    from abacus_b200.config import ConfigError, MovaraxConfig, load_config
    from abacus_b200.weights.safetensors_io import folder_shapes
    folder, raw, tensors = mm.write_folder(tmp_path, name)
    arch, cfg = load_config(folder)
    assert arch.name == "Movarax" and isinstance(cfg, MovaraxConfig)
    assert MovaraxConfig.from_dict(cfg.to_dict()) == cfg
    spec = cfg.to_spec()
    expected, _ = arch.tensor_names(spec, None)
    assert {n: tuple(s) for n, s in expected.items()} == {n: tuple(s) for n, s in folder_shapes(folder).items()}
    # an entry that reads another layer's latents names it as its source, and has no cache of its own
    for i, (layer, entry) in enumerate(zip(raw["layers"], spec.schedule)):
        assert entry.layer == i and entry.source == layer["mixer"].get("kv_from")
    assert "movarax" in arch.info(spec)


def test_configurations_that_cannot_be_are_refused():
    from abacus_b200.config import ConfigError, MovaraxConfig
    raw = mm.config("U")
    for change in (lambda r: r["layers"][2]["mixer"].update(kv_from=0),            # layer 0 is no latent attention
                   lambda r: r["layers"][2]["mixer"].update(kv_from=2),            # not an earlier layer
                   lambda r: r["layers"][2]["mixer"].update(kv_rank=48),           # other latents than its source's
                   lambda r: r["layers"][1]["mixer"].update(kv_from=2),
                   lambda r: r["layers"][0]["mixer"].update(decay=[0.5]),          # a decay per head
                   lambda r: r["layers"][0]["mlp"]["router"].update(top=6),        # more than there are experts
                   lambda r: r["layers"][1]["mixer"]["rot"].update(dims=10),       # more than rot_dim
                   lambda r: r["layers"][3].update(type="lightning_3"),
                   lambda r: r["layers"][1]["mlp"].update(kind="sparse"),
                   lambda r: r.pop("norm")):
        bad = json.loads(json.dumps(raw))
        change(bad)
        with pytest.raises(ConfigError):
            MovaraxConfig.from_dict(bad)


def test_random_models_can_be_written_for_the_design(tmp_path):
    from abacus_b200.config import MovaraxConfig, load_config
    from abacus_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / "m"), MovaraxConfig.from_dict(mm.config("V")), seed=3)
    tensors = plain.read_safetensors(folder + "/model.safetensors")
    assert abs(tensors["l0.mix.dkv.norm"].mean() - 1.0) < 1e-6 and abs(tensors["l0.mix.sink"]).max() > 0.1
    assert load_config(folder)[1].to_dict() == MovaraxConfig.from_dict(mm.config("V")).to_dict()


def test_the_recurrence_is_the_decayed_sum_over_earlier_tokens():
    rng = np.random.default_rng(0)
    T, n, V, a = 23, 6, 4, 0.9
    q, k, v = rng.standard_normal((T, n)), rng.standard_normal((T, n)), rng.standard_normal((T, V))
    got = plain.decay_recurrence(q, k, v, a)
    want = np.stack([sum(a ** (t - j) * (q[t] @ k[j]) * v[j] for j in range(t + 1)) for t in range(T)])
    np.testing.assert_allclose(got, want, rtol=1e-10, atol=1e-10)


def test_attention_over_latents_equals_attention_over_full_size_keys():
    raw, tensors = mm.config("U"), mm.weights("U")
    tokens = [int(t) for t in np.random.default_rng(1).integers(0, raw["vocab"], 40)]
    full = plain.forward(raw, tensors, tokens, real=np.float64)
    over = plain.forward(raw, tensors, tokens, real=np.float64, latent_rows=np.ones(40, dtype=bool))
    np.testing.assert_allclose(over, full, rtol=1e-9, atol=1e-9)


def test_the_weight_on_an_experts_input_and_the_choice_of_experts():
    rng = np.random.default_rng(2)
    d, ff, E = 12, 7, 5
    h = rng.standard_normal((9, d))
    p = {"router": rng.standard_normal((E, d))}
    for e in range(E):
        p[f"e{e}.up"], p[f"e{e}.down"] = rng.standard_normal((ff, d)), rng.standard_normal((d, ff))
    mlp = {"router": {"experts": E, "top": 2}}
    got = plain.routed_feed_forward(h, p, mlp)
    s = plain.sigmoid(h @ p["router"].T)
    for t in range(9):
        first, second = np.argsort(-s[t])[:2]
        # the squared ReLU is of degree two: a weight on the input is its square on the output
        want = sum(s[t, e] ** 2 * plain.expert(h[t:t + 1], p[f"e{e}.up"], p[f"e{e}.down"])[0] for e in (first, second))
        np.testing.assert_allclose(got[t], want, rtol=1e-5, atol=1e-6)
    chosen, scores = plain.route(np.zeros((1, d)), p["router"], 3)   # all scores equal: the lowest indices
    assert chosen.tolist() == [[0, 1, 2]] and np.allclose(scores, 0.5)
