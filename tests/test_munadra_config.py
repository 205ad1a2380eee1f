"""The Munadra configuration on the CPU: reading config.json, its faults, the model it describes, the
tensors that model reads, the rotation's frequencies, and the plain implementation's own mechanisms
against values worked out by hand."""
from __future__ import annotations

import json
import math

import pytest
import torch

import plain_munadra as P
from munadra_helpers import CONFIGS, tensor_shapes


def _cfg(name):
    from kuiperllama_b200.config import config_from_dict
    return config_from_dict(json.loads(json.dumps(CONFIGS[name])))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_manifest_names_and_shapes(name):
    from kuiperllama_b200.engine.model import model_manifest
    cfg = _cfg(name)
    assert type(cfg).__name__ == "MunadraConfig"
    got = {k: tuple(v.shape) for k, v in model_manifest(cfg.to_model_spec()).items()}
    assert got == tensor_shapes(CONFIGS[name])


def test_round_trip_and_spec():
    from kuiperllama_b200.config import config_from_dict
    cfg = _cfg("mixed")
    again = config_from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict() and again.to_dict()["layers"] == CONFIGS["mixed"]["layers"]
    spec = cfg.to_model_spec()
    assert spec.lm_head_name is None and spec.embedding_name == "embed" and spec.hidden_size == 64 and spec.vocab_size == 97
    assert (spec.embedding_multiplier, spec.logit_scale, spec.logit_softcap) == (1.5, 0.2, 6.0)
    assert [l.mixer.kind for l in spec.layers] == ["rglru", "latent_attention", "latent_attention", "rglru", "latent_attention", "latent_attention"]
    assert [l.feed_forward.kind if l.feed_forward else None for l in spec.layers] == ["moe", "swiglu", None, "swiglu", "moe", "moe"]
    assert [e.cache_from for e in spec.schedule] == [None, None, 1, None, None, 1]
    assert all(l.arrangement == "sandwich" and l.mixer_norm.kind == "none" and l.mixer_post_norm["weight_offset"] == 1.0 for l in spec.layers)
    assert spec.final_norm["weight_offset"] == 1.0 and spec.final_norm.kind == "rmsnorm"
    att = spec.layers[2]
    assert att.mixer["own_latent"] is False and att.feed_forward_norm is None and att.feed_forward_post_norm is None
    assert att.position["pairing"] == "interleaved" and att.position["scaling"]["rope_type"] == "yarn"
    assert spec.layers[4].position["scaling"] is None and spec.layers[4].mixer["scale"] == 0.4
    moe = spec.layers[5].feed_forward
    assert (moe["experts"], moe["top"], moe["expert_size"], moe["limit"], moe["alpha"], moe["shift"], moe["renormalise"]) == (8, 3, 16, 0.75, 1.702, 1.0, False)
    assert spec.layers[0].mixer["decay_scale"] == 8.0 and "l2.norm2" in spec.ignorable_suffixes
    # plain scalars default to "absent"
    bare = config_from_dict({k: v for k, v in CONFIGS["only_rglru"].items() if k not in ("embedding", "logit_scale")}).to_model_spec()
    assert bare.embedding_multiplier is None and bare.logit_scale is None and bare.logit_softcap is None


def test_yarn_frequencies_against_worked_values():
    """dims 8, base 16, original 32, factor 4, fast 4, slow 1: index(t) = 8 ln(32 / (2 pi t)) / (2 ln 16), so
    index(4) = 0.349 -> lo 0 and index(1) = 2.349 -> hi 3; the ramp is i / 3; f_i = 16^(-i / 4) = 1, 1/2, 1/4, 1/8."""
    from kuiperllama_b200.parts.position import rotary_inverse_frequencies, rotary_magnitude
    sc = {"rope_type": "yarn", "factor": 4.0, "original": 32.0, "fast": 4.0, "slow": 1.0, "magnitude_slope": 0.1}
    got = rotary_inverse_frequencies(8, 16.0, sc)
    want = [1.0, 0.5 * (1 / 4 * 1 / 3 + 2 / 3), 0.25 * (1 / 4 * 2 / 3 + 1 / 3), 0.125 / 4]
    assert got == pytest.approx(want, rel=1e-12)
    assert rotary_magnitude(sc) == pytest.approx(0.1 * math.log(4.0) + 1.0) and rotary_magnitude(None) == 1.0
    plain, mag = P.yarn_frequencies(8, 16.0, {"factor": 4.0, "original": 32, "fast": 4.0, "slow": 1.0})
    assert plain == pytest.approx(want, rel=1e-12) and mag == pytest.approx(rotary_magnitude(sc))
    # ends that fall outside the pairs are kept inside; a ramp of no length does not divide by zero
    wide = {"rope_type": "yarn", "factor": 2.0, "original": 4096.0, "fast": 1e6, "slow": 1e-6}
    got = rotary_inverse_frequencies(4, 100.0, wide)
    assert got == pytest.approx([1.0, 0.1 / 2.0 * (1 / 3) + 0.1 * (2 / 3)], rel=1e-12)
    same = {"rope_type": "yarn", "factor": 2.0, "original": 64.0, "fast": 1.0, "slow": 1.0}
    assert len(rotary_inverse_frequencies(6, 10.0, same)) == 3
    for name in ("mixed", "odd", "wide"):
        pos = _cfg(name).to_model_spec().layers[[l["type"] for l in CONFIGS[name]["layers"]].index("latent_attention")].position
        rot = next(l["mixer"]["rot"] for l in CONFIGS[name]["layers"] if l["type"] == "latent_attention")
        want, _ = P.yarn_frequencies(rot["dims"], rot["base"], rot["scaling"])
        assert rotary_inverse_frequencies(pos["rotary_dim"], pos["theta"], pos["scaling"]) == pytest.approx(want, rel=1e-12)
        assert any(abs(w - rot["base"] ** (-2.0 * i / rot["dims"])) > 1e-9 for i, w in enumerate(want)), "the rule changed nothing"


def test_plain_mechanisms_against_hand_values():
    """The plain implementation itself, on numbers small enough to follow by hand."""
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert P.rms_norm(x, torch.tensor([0.0, 1.0]), 0.0, 1.0)[0].tolist() == pytest.approx([3 / math.sqrt(12.5), 8 / math.sqrt(12.5)])
    # a quarter turn of the pair (1, 0) at position 1 with frequency pi/2, times 2: (0, 2)
    r = P.rotate_interleaved(torch.tensor([[1.0, 0.0]], dtype=torch.float64), torch.tensor([1]), [math.pi / 2], 2.0)
    assert r[0].tolist() == pytest.approx([0.0, 2.0], abs=1e-12)
    # experts: g = min(2, 1) = 1, u = clamp(-3, -1, 1) = -1 -> y = sigmoid(1.702) * 0 = 0;   u = 0.5 -> sigmoid(1.702) * 1.5
    W = {"gate": torch.tensor([[2.0]]), "up": torch.tensor([[-3.0]]), "down": torch.tensor([[1.0]])}
    assert float(P.expert(torch.tensor([[1.0]], dtype=torch.float64), W, "", 1.0)) == pytest.approx(0.0)
    W["up"] = torch.tensor([[0.5]])
    assert float(P.expert(torch.tensor([[1.0]], dtype=torch.float64), W, "", 1.0)) == pytest.approx(1.5 / (1 + math.exp(-1.702)))
    # routing: scores over all three experts, the two largest, not renormalised
    idx, wgt = P.route(torch.tensor([[1.0]], dtype=torch.float64), {"router": torch.tensor([[0.0], [math.log(2.0)], [math.log(5.0)]])}, "", 2)
    assert idx.tolist() == [[2, 1]] and wgt[0].tolist() == pytest.approx([5 / 8, 2 / 8])
    # the recurrence from S = 0: one channel, one tap, gates at sigmoid(0) = 1/2
    m = {"width": 1, "blocks": 1, "conv": 1}
    z = lambda *s: torch.zeros(*s)
    W = {"y": torch.tensor([[1.0]]), "y.b": z(1), "x": torch.tensor([[1.0]]), "x.b": z(1), "conv": torch.tensor([[1.0]]), "conv.b": z(1),
         "ra": z(1, 1, 1), "ra.b": z(1, 1), "ri": z(1, 1, 1), "ri.b": z(1, 1), "lam": z(1), "o": torch.tensor([[1.0]])}
    a = math.exp(-8 * 0.5 * math.log(2.0))
    b = math.sqrt(1 - a * a) * 0.5
    h = torch.tensor([[1.0], [2.0]], dtype=torch.float64)
    got = P.rglru(h, W, "", m)
    g1, g2 = float(P.gelu_tanh(torch.tensor(1.0))), float(P.gelu_tanh(torch.tensor(2.0)))
    assert got.reshape(-1).tolist() == pytest.approx([b * 1.0 * g1, (a * b * 1.0 + b * 2.0) * g2])
    # a sink alone beside one key: weight 1 / (1 + exp(sink - score))
    m = {"heads": 1, "dim": 1, "rot_dim": 2, "vdim": 1, "kv_rank": 1, "scale": 1.0, "rot": {"base": 10.0, "dims": 2, "scaling": None}}
    W = {"q": torch.tensor([[1.0], [0.0], [0.0]]), "dkv": torch.tensor([[1.0], [0.0], [0.0]]), "dkv.norm": torch.ones(1), "uk": torch.tensor([[2.0]]),
         "uv": torch.tensor([[3.0]]), "sink": torch.tensor([0.5]), "g": torch.tensor([[0.0]]), "o": torch.tensor([[1.0]])}
    out, _ = P.latent_attention(torch.tensor([[1.0]], dtype=torch.float64), W, "", m, 0.0)
    assert float(out) == pytest.approx(3.0 / (1 + math.exp(0.5 - 2.0)) * 0.5)


@pytest.mark.parametrize("change, word", [
    (lambda c: c.pop("vocab"), '"vocab"'),
    (lambda c: c["layers"][0].update(type="lstm"), '"type"'),
    (lambda c: c["layers"][0]["mixer"].update(blocks=5), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), '"kv_rank"'),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][5]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=48), "must equal"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), '"top"'),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), '"mlp"'),
    (lambda c: c["norm"].update(eps=0), "eps"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
])
def test_faults_are_named(change, word):
    from kuiperllama_b200.config import ConfigError, config_from_dict
    c = json.loads(json.dumps(CONFIGS["mixed"]))
    change(c)
    with pytest.raises(ConfigError) as e:
        config_from_dict(c)
    assert word in str(e.value)


def test_cache_requests_without_a_device():
    """What the mixers ask of the cache, from the specs alone: one row of kv_rank + rot_dim per token and no second
    tensor, executions that share a latent in one group, and the recurrent state's size."""
    from kuiperllama_b200.cache import KVRequest, SequenceCache, StateRequest
    spec = _cfg("mixed").to_model_spec()
    kv, st = [], []
    for layer in spec.layers:
        m = layer.mixer
        kv.append(KVRequest(1, m["kv_rank"] + m["rot_dim"], kind="keys") if m.kind == "latent_attention" else None)
        st.append(StateRequest((m["width"] * m["conv"],)) if m.kind == "rglru" else None)
    cache = SequenceCache(kv, st, [e.cache_from for e in spec.schedule], max_tokens=256, max_seq_len=256, dtype=torch.float32, device="cpu")
    assert [g.request.head_dim for g in cache.groups] == [48, 40] and [len(g.entries) for g in cache.groups] == [1, 1]
    view, owner = cache.view(5), cache.view(1)
    assert view.k.data_ptr() == owner.k.data_ptr() == view.v.data_ptr() and not view.writable and owner.writable
    assert cache.view(0).state.shape == (4, 48 * 3) and cache.view(3).state.shape == (4, 96)
    assert cache.bytes() == 4 * (4 * 64 * (48 + 40) + 4 * (144 + 96))
