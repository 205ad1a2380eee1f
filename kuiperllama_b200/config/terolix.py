"""Typed configuration of the Terolix decoder, read from its config.json.

Terolix is a small decoder-only design whose layers each pick one of three mixers (a minGRU, a
gated delta rule, causal softmax attention whose values are its unrotated keys), all inside the
same block: a layer norm before and after every sublayer and a sigmoid gate on every sublayer's
result.  config.json lists the layers one by one::

    {"architecture": "Terolix", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "mingru",    "mixer": {"width": w},                                   "mlp": {...}},
                {"type": "delta",     "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"},   "mlp": {...}},
                {"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale",
                                                "rot": {"base", "dims", "scaling": {"factor", "low", "high", "original"}}},
                 "mlp": {"kind": "dense", "ff": F} or null}]}

Tensor names: ``embed``, ``final.norm`` (+ ``.b``), and under ``l<i>.``: ``norm1``, ``norm1b``,
``norm2``, ``norm2b`` (+ ``.b`` each), ``rg1``, ``rg2`` (+ ``.b``), ``mix.*`` and ``mlp.*``.  The
classifier is the embedding table.  ExiledOfCode/KuiperLLama has no such model; its model classes
are picked in ``main`` (demo/main.cpp:58).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .registry import ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, default_schedule

MIXER_TYPES = ("mingru", "attention", "delta")
# Constants the design fixes (they are parameters of the parts, so another design may choose others).
DELTA_UNIT_EPS = 1e-6            # inside the root when q and k are made unit vectors
DEFAULT_MAX_POSITIONS = 1 << 17  # the design names no longest sequence; "max_positions" may raise it


def _is_int(v: Any) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@register_architecture("Terolix")
@dataclass(frozen=True)
class TerolixConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[dict, ...]              # as in config.json, checked
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Terolix"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TerolixConfig":
        problems: List[str] = []

        def positive_int(where: str, obj: Any, key: str) -> int:
            v = obj.get(key) if isinstance(obj, dict) else None
            if not _is_int(v) or v <= 0:
                problems.append(f'{where}"{key}" must be a positive integer, got {v!r}')
                return 1
            return v

        vocab = positive_int("", d, "vocab")
        width = positive_int("", d, "width")
        norm = d.get("norm")
        eps = norm.get("eps") if isinstance(norm, dict) else None
        if not _is_num(eps) or eps <= 0:
            problems.append(f'"norm": {{"eps"}} must be a positive number, got {eps!r}')
            eps = 1e-5
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            problems.append('"layers" must be a list with at least one layer')
            layers = []
        for i, layer in enumerate(layers):
            at = f"layers[{i}]: "
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
                problems.append(f'{at}"type" must be one of {list(MIXER_TYPES)}, got {layer.get("type") if isinstance(layer, dict) else layer!r}')
                continue
            m = layer.get("mixer")
            if not isinstance(m, dict):
                problems.append(f'{at}"mixer" must be an object')
                continue
            kind = layer["type"]
            if kind == "mingru":
                positive_int(at, m, "width")
            else:
                H, G = positive_int(at, m, "heads"), positive_int(at, m, "kv_heads")
                dim, vdim = positive_int(at, m, "dim"), positive_int(at, m, "vdim")
                if H % G:
                    problems.append(f'{at}"heads" {H} is not a multiple of "kv_heads" {G}')
                if kind == "delta":
                    positive_int(at, m, "conv")
                else:
                    if vdim != dim:
                        problems.append(f'{at}the values are the keys, so "vdim" {vdim} must equal "dim" {dim}')
                    if not _is_num(m.get("scale")):
                        problems.append(f'{at}"scale" must be a number, got {m.get("scale")!r}')
                    rot = m.get("rot")
                    if rot is not None:
                        if not isinstance(rot, dict) or not _is_num(rot.get("base")) or rot.get("base", 0) <= 0:
                            problems.append(f'{at}"rot" needs a positive "base"')
                        else:
                            dims = positive_int(at + '"rot": ', rot, "dims")
                            if dims % 2 or dims > dim:
                                problems.append(f'{at}"rot": "dims" {dims} must be even and at most "dim" {dim}')
                            sc = rot.get("scaling")
                            if sc is not None:
                                missing = [k for k in ("factor", "low", "high", "original") if not (isinstance(sc, dict) and _is_num(sc.get(k)))]
                                if missing:
                                    problems.append(f'{at}"rot": "scaling" lacks numbers for {missing}')
                                elif sc["high"] <= sc["low"] or sc["factor"] <= 0:
                                    problems.append(f'{at}"rot": "scaling" needs high > low and factor > 0')
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    problems.append(f'{at}"mlp" must be null or have "kind": "dense", got {mlp!r}')
                else:
                    positive_int(at + '"mlp": ', mlp, "ff")
        max_positions = d.get("max_positions", DEFAULT_MAX_POSITIONS)
        if not _is_int(max_positions) or max_positions <= 0:
            problems.append(f'"max_positions" must be a positive integer, got {max_positions!r}')
        if problems:
            raise ConfigError("config.json (Terolix): " + "; ".join(problems))
        return cls(vocab=vocab, width=width, norm_eps=float(eps), layers=tuple(json.loads(json.dumps(l)) for l in layers),
                   max_positions=max_positions)

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "layers": json.loads(json.dumps(list(self.layers))),
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d

    # ------------------------------------------------------------------ the model it describes
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("layernorm", {"size": self.width, "eps": self.norm_eps, "name": name, "bias": name + ".b"})

    def _mixer(self, kind: str, m: dict) -> Tuple[PartSpec, Optional[PartSpec]]:
        """The mixer's part and, for attention, its position encoding."""
        if kind == "mingru":
            return PartSpec("mingru", {"hidden_size": self.width, "width": m["width"],
                                       "names": {"z": "mix.z", "x": "mix.x", "g": "mix.g", "o": "mix.o",
                                                 "z_bias": "mix.z.b", "x_bias": "mix.x.b"}}), None
        if kind == "delta":
            return PartSpec("gated_delta", {
                "hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                "conv": m["conv"], "norm_eps": self.norm_eps, "unit_eps": DELTA_UNIT_EPS, "q_scale": float(m["dim"]) ** -0.5,
                "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "g": "mix.g", "o": "mix.o", "beta": "mix.b", "a": "mix.a",
                          "q_conv": "mix.q.conv", "k_conv": "mix.k.conv", "v_conv": "mix.v.conv", "A_log": "mix.A_log",
                          "dt_bias": "mix.dt_bias", "norm": "mix.norm"}}), None
        rot, position = m.get("rot"), None
        if rot is not None:
            sc = rot.get("scaling")
            position = PartSpec("rope", {
                "head_dim": m["dim"], "rotary_dim": rot["dims"], "theta": float(rot["base"]),
                "scaling": None if sc is None else {"rope_type": "llama3", "factor": float(sc["factor"]),
                                                    "low_freq_factor": float(sc["low"]), "high_freq_factor": float(sc["high"]),
                                                    "original_max_position_embeddings": float(sc["original"])}})
        return PartSpec("attention", {
            "hidden_size": self.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "window": None, "scale": float(m["scale"]), "values": "keys",
            "names": {"q": "mix.q", "k": "mix.k", "g": "mix.g", "o": "mix.o"}}), position

    def to_model_spec(self) -> ModelSpec:
        layers = []
        for i, layer in enumerate(self.layers):
            mixer, position = self._mixer(layer["type"], layer["mixer"])
            gate = lambda name: PartSpec("sigmoid_linear", {"hidden_size": self.width, "name": name, "bias": name + ".b"})
            mlp = layer.get("mlp")
            ff = None
            if mlp is not None:
                ff = PartSpec("dense", {"hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "xielu",
                                        "names": {"up": "mlp.up", "down": "mlp.down", "act": "mlp.act"}})
            layers.append(LayerSpec(
                prefix=f"l{i}.", arrangement="sandwich", mixer=mixer, feed_forward=ff, position=position,
                mixer_norm=self._norm("norm1"), mixer_post_norm=self._norm("norm1b"), mixer_gate=gate("rg1"),
                feed_forward_norm=self._norm("norm2") if ff else None,
                feed_forward_post_norm=self._norm("norm2b") if ff else None,
                feed_forward_gate=gate("rg2") if ff else None))
        # a layer without a feed-forward reads none of the second sublayer's tensors, should a checkpoint hold them
        unread = tuple(f"l{i}.{name}{b}" for i, layer in enumerate(self.layers) if layer.get("mlp") is None
                       for name in ("norm2", "norm2b", "rg2") for b in ("", ".b"))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
            layers=tuple(layers), schedule=default_schedule(len(layers)), embedding_name="embed",
            final_norm=self._norm("norm"), final_norm_prefix="final.", lm_head_name=None, ignorable_suffixes=unread)
        spec.validate()
        return spec
