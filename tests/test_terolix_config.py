"""The Terolix configuration on the CPU: reading config.json, its faults, the model it describes and
the tensors that model reads."""
from __future__ import annotations

import json

import pytest

from terolix_helpers import CONFIGS, tensor_shapes


def _cfg(name):
    from kuiperllama_b200.config import config_from_dict
    return config_from_dict(json.loads(json.dumps(CONFIGS[name])))


@pytest.mark.parametrize("name", ["mixed", "odd", "wide", "only_ff"])
def test_manifest_names_and_shapes(name):
    from kuiperllama_b200.engine.model import model_manifest
    cfg = _cfg(name)
    assert type(cfg).__name__ == "TerolixConfig"
    got = {k: tuple(v.shape) for k, v in model_manifest(cfg.to_model_spec()).items()}
    assert got == tensor_shapes(CONFIGS[name])


def test_round_trip_and_spec():
    from kuiperllama_b200.config import config_from_dict
    cfg = _cfg("mixed")
    again = config_from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict() and again.to_dict()["layers"] == CONFIGS["mixed"]["layers"]
    spec = cfg.to_model_spec()
    assert spec.lm_head_name is None and spec.embedding_name == "embed" and spec.hidden_size == 64 and spec.vocab_size == 97
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds == ["mingru", "attention", "gated_delta", "attention", "gated_delta", "mingru"]
    assert all(l.arrangement == "sandwich" for l in spec.layers)
    att = spec.layers[1]
    assert att.feed_forward is None and att.feed_forward_norm is None and att.feed_forward_gate is None
    assert att.mixer["values"] == "keys" and att.mixer["scale"] == 0.2 and att.position["rotary_dim"] == 16
    assert att.position["scaling"]["original_max_position_embeddings"] == 64
    assert spec.layers[3].position["scaling"] is None and spec.layers[3].position["rotary_dim"] == 64
    d = spec.layers[2].mixer
    assert (d["heads"], d["kv_heads"], d["dim"], d["vdim"], d["conv"]) == (4, 2, 24, 40, 3) and d["q_scale"] == 24 ** -0.5
    assert "l1.norm2" in spec.ignorable_suffixes and "l0.norm2" not in spec.ignorable_suffixes


def test_rotary_frequencies_follow_the_scaling_rule():
    import plain_terolix as P
    from kuiperllama_b200.parts.position import rotary_inverse_frequencies
    spec = _cfg("wide").to_model_spec()
    pos = spec.layers[0].position
    got = rotary_inverse_frequencies(pos["rotary_dim"], pos["theta"], pos["scaling"])
    want = P.rotary_frequencies(CONFIGS["wide"]["layers"][0]["mixer"]["rot"]).tolist()
    assert got == pytest.approx(want, rel=1e-12)
    assert any(abs(g - float(pos["theta"]) ** (-2.0 * i / pos["rotary_dim"])) > 1e-9 for i, g in enumerate(got)), "the rule changed nothing"


@pytest.mark.parametrize("change, word", [
    (lambda c: c.pop("vocab"), '"vocab"'),
    (lambda c: c["layers"][0].update(type="lstm"), '"type"'),
    (lambda c: c["layers"][1]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=16), "vdim"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=34), "dims"),
    (lambda c: c["layers"][2]["mixer"].pop("conv"), '"conv"'),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), '"mlp"'),
    (lambda c: c["norm"].update(eps=0), "eps"),
])
def test_faults_are_named(change, word):
    from kuiperllama_b200.config import ConfigError, config_from_dict
    c = json.loads(json.dumps(CONFIGS["mixed"]))
    change(c)
    with pytest.raises(ConfigError) as e:
        config_from_dict(c)
    assert word in str(e.value)


def test_state_sizes_without_a_device():
    """What the mixers ask of the cache, from the specs alone."""
    spec = _cfg("mixed").to_model_spec()
    d = spec.layers[2].mixer
    channels = 2 * d["kv_heads"] * d["dim"] + d["heads"] * d["vdim"]
    assert channels == 256 and d["heads"] * d["vdim"] * d["dim"] + (d["conv"] - 1) * channels == 4352
