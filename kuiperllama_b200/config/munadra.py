"""Typed configuration of the Munadra decoder, read from its config.json.

Munadra is a small decoder-only design.  Every layer adds its sublayers' results after a norm,
x += norm1(mixer(x)); x += norm2(ff(x)), the sublayers reading the stream itself; the norms are RMS norms
whose stored weight lies around zero (the factor is 1 + w).  The mixer is attention over a latent that
all heads share (one short row per token in the cache; a layer may read an earlier layer's rows instead
of making its own) or a recurrent block with a real-gated linear recurrent unit; the feed-forward is
a dense SiLU-gated one or a mixture of experts.  config.json lists the layers one by one::

    {"architecture": "Munadra", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "logit_scale": a, "logit_softcap": c,
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "kv_from": j (optional),
                           "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "rglru", "mixer": {"width", "blocks", "conv"},
                 "mlp": {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff", "limit"}} or null}]}

Tensor names: ``embed`` (also the classifier), ``final.norm``, and under ``l<i>.``: ``norm1``, ``norm2``,
``mix.*`` and ``mlp.*`` (experts: ``mlp.e<k>.gate|up|down``, ``mlp.router``).  ExiledOfCode/KuiperLLama has no
such model; its model classes are picked in ``main`` (demo/main.cpp:58).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .registry import ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXER_TYPES = ("latent_attention", "rglru")
# Constants the design fixes (parameters of the parts, so another design may choose others).
NORM_WEIGHT_OFFSET = 1.0         # every block norm and the final norm multiply by 1 + w
RGLRU_DECAY_SCALE = 8.0          # log a = -8 r softplus(lambda)
EXPERT_ALPHA = 1.702             # y = g sigmoid(1.702 g) (u + 1)
EXPERT_SHIFT = 1.0
YARN_MAGNITUDE_SLOPE = 0.1       # cos and sin times 0.1 ln(factor) + 1
DEFAULT_MAX_POSITIONS = 1 << 17  # the design names no longest sequence; "max_positions" may raise it


def _is_int(v: Any) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@register_architecture("Munadra")
@dataclass(frozen=True)
class MunadraConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[dict, ...]              # as in config.json, checked
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: Optional[float] = None
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Munadra"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MunadraConfig":
        problems: List[str] = []

        def positive_int(where: str, obj: Any, key: str) -> int:
            v = obj.get(key) if isinstance(obj, dict) else None
            if not _is_int(v) or v <= 0:
                problems.append(f'{where}"{key}" must be a positive integer, got {v!r}')
                return 1
            return v

        def number(where: str, obj: Any, key: str, default=None, positive: bool = False) -> float:
            v = obj.get(key, default) if isinstance(obj, dict) else default
            if not _is_num(v) or (positive and v <= 0):
                problems.append(f'{where}"{key}" must be a {"positive " if positive else ""}number, got {v!r}')
                return 1.0
            return float(v)

        vocab = positive_int("", d, "vocab")
        width = positive_int("", d, "width")
        eps = number('"norm": ', d.get("norm"), "eps", positive=True)
        emb = d.get("embedding")
        emb_scale = number('"embedding": ', emb, "scale", 1.0) if emb is not None else 1.0
        logit_scale = number("", d, "logit_scale", 1.0)
        cap = d.get("logit_softcap")
        if cap is not None and (not _is_num(cap) or cap <= 0):
            problems.append(f'"logit_softcap" must be a positive number or absent, got {cap!r}')
            cap = None
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
            if layer["type"] == "rglru":
                w, B = positive_int(at, m, "width"), positive_int(at, m, "blocks")
                positive_int(at, m, "conv")
                if w % B:
                    problems.append(f'{at}"width" {w} is not a multiple of "blocks" {B}')
            else:
                for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
                    positive_int(at, m, k)
                number(at, m, "scale")
                rot = m.get("rot")
                if not isinstance(rot, dict) or not _is_num(rot.get("base")) or rot.get("base", 0) <= 1:
                    problems.append(f'{at}"rot" needs a "base" above 1')
                else:
                    dims = positive_int(at + '"rot": ', rot, "dims")
                    if dims % 2 or (_is_int(m.get("rot_dim")) and dims > m["rot_dim"]):
                        problems.append(f'{at}"rot": "dims" {dims} must be even and at most "rot_dim" {m.get("rot_dim")!r}')
                    sc = rot.get("scaling")
                    if sc is not None:
                        missing = [k for k in ("factor", "original", "fast", "slow") if not (isinstance(sc, dict) and _is_num(sc.get(k)) and sc[k] > 0)]
                        if missing:
                            problems.append(f'{at}"rot": "scaling" lacks positive numbers for {missing}')
                src = m.get("kv_from")
                if src is not None:
                    ok = _is_int(src) and 0 <= src < i and isinstance(layers[src], dict) and layers[src].get("type") == "latent_attention" \
                        and isinstance(layers[src].get("mixer"), dict) and layers[src]["mixer"].get("kv_from") is None
                    if not ok:
                        problems.append(f'{at}"kv_from" {src!r} must name an earlier latent_attention layer that makes its own latent')
                    elif any(layers[src]["mixer"].get(k) != m.get(k) for k in ("kv_rank", "rot_dim", "rot")):
                        problems.append(f'{at}"kv_from" {src}: "kv_rank", "rot_dim" and "rot" must equal that layer\'s')
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                problems.append(f'{at}"mlp" must be null or have "kind": "dense" or "moe", got {mlp!r}')
            elif mlp["kind"] == "dense":
                positive_int(at + '"mlp": ', mlp, "ff")
            else:
                E = positive_int(at + '"mlp": "router": ', mlp.get("router"), "experts")
                top = positive_int(at + '"mlp": "router": ', mlp.get("router"), "top")
                if top > E:
                    problems.append(f'{at}"mlp": "top" {top} exceeds "experts" {E}')
                positive_int(at + '"mlp": "expert": ', mlp.get("expert"), "ff")
                number(at + '"mlp": "expert": ', mlp.get("expert"), "limit", positive=True)
        max_positions = d.get("max_positions", DEFAULT_MAX_POSITIONS)
        if not _is_int(max_positions) or max_positions <= 0:
            problems.append(f'"max_positions" must be a positive integer, got {max_positions!r}')
        if problems:
            raise ConfigError("config.json (Munadra): " + "; ".join(problems))
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(json.loads(json.dumps(l)) for l in layers),
                   embedding_scale=emb_scale, logit_scale=logit_scale, logit_softcap=None if cap is None else float(cap),
                   max_positions=max_positions)

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
             "layers": json.loads(json.dumps(list(self.layers))), "logit_scale": self.logit_scale,
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d

    # ------------------------------------------------------------------ the model it describes
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "name": name, "weight_offset": NORM_WEIGHT_OFFSET})

    def _mixer(self, kind: str, m: dict) -> Tuple[PartSpec, Optional[PartSpec]]:
        if kind == "rglru":
            return PartSpec("rglru", {
                "hidden_size": self.width, "width": m["width"], "blocks": m["blocks"], "conv": m["conv"], "decay_scale": RGLRU_DECAY_SCALE,
                "names": {"y": "mix.y", "x": "mix.x", "y_bias": "mix.y.b", "x_bias": "mix.x.b", "conv": "mix.conv",
                          "conv_bias": "mix.conv.b", "ra": "mix.ra", "ra_bias": "mix.ra.b", "ri": "mix.ri", "ri_bias": "mix.ri.b",
                          "lam": "mix.lam", "o": "mix.o"}}), None
        rot = m["rot"]
        sc = rot.get("scaling")
        position = PartSpec("rope", {
            "head_dim": m["rot_dim"], "rotary_dim": rot["dims"], "theta": float(rot["base"]), "pairing": "interleaved",
            "scaling": None if sc is None else {"rope_type": "yarn", "factor": float(sc["factor"]), "original": float(sc["original"]),
                                                "fast": float(sc["fast"]), "slow": float(sc["slow"]),
                                                "magnitude_slope": YARN_MAGNITUDE_SLOPE}})
        return PartSpec("latent_attention", {
            "hidden_size": self.width, "num_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
            "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "norm_eps": self.norm_eps, "own_latent": m.get("kv_from") is None,
            "names": {"q": "mix.q", "dkv": "mix.dkv", "dkv_norm": "mix.dkv.norm", "uk": "mix.uk", "uv": "mix.uv", "sink": "mix.sink",
                      "g": "mix.g", "o": "mix.o"}}), position

    def _feed_forward(self, mlp: Optional[dict]) -> Optional[PartSpec]:
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": mlp["ff"],
                                       "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
        return PartSpec("moe", {
            "hidden_size": self.width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
            "expert_size": mlp["expert"]["ff"], "limit": float(mlp["expert"]["limit"]), "alpha": EXPERT_ALPHA, "shift": EXPERT_SHIFT,
            "renormalise": False,
            "names": {"router": "mlp.router", "gate": "mlp.e{e}.gate", "up": "mlp.e{e}.up", "down": "mlp.e{e}.down"}})

    def to_model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        none = PartSpec("none", {"size": self.width})
        for i, layer in enumerate(self.layers):
            mixer, position = self._mixer(layer["type"], layer["mixer"])
            ff = self._feed_forward(layer.get("mlp"))
            layers.append(LayerSpec(
                prefix=f"l{i}.", arrangement="sandwich", mixer=mixer, feed_forward=ff, position=position,
                mixer_norm=none, mixer_post_norm=self._norm("norm1"),
                feed_forward_norm=none if ff else None, feed_forward_post_norm=self._norm("norm2") if ff else None))
            schedule.append(ScheduleEntry(layer=i, cache_from=layer["mixer"].get("kv_from")))
        unread = tuple(f"l{i}.norm2" for i, layer in enumerate(self.layers) if layer.get("mlp") is None)
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
            layers=tuple(layers), schedule=tuple(schedule), embedding_name="embed", final_norm=self._norm("norm"),
            final_norm_prefix="final.", lm_head_name=None, ignorable_suffixes=unread,
            embedding_multiplier=None if self.embedding_scale == 1.0 else self.embedding_scale,
            logit_scale=None if self.logit_scale == 1.0 else self.logit_scale, logit_softcap=self.logit_softcap)
        spec.validate()
        return spec
