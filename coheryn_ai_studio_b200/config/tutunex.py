"""Typed configuration of the Tutunex decoder and its layout as parts.

The design: an embedding multiplied by a constant; layers with a norm before and after each sub-layer,
x <- x + norm_b(mixer(norm(x))), then x <- x + norm_b(ff(norm(x))) (arrangement ``sandwich_residual``); two kinds of
mixer, chosen per layer by ``type``:

* ``attention``  differential attention (``parts/attention.py``: ``MapsAttention`` with two score maps per head): grouped
                 queries, keys of ``dim`` and values of ``vdim`` channels, a rotation of the first ``rot.dims`` channels
                 of every map with optional YaRN scaling (``parts/position.py``: ``ComputedRope``), a mask by chunks of
                 ``mask.size`` positions (absent: every earlier position), the heads' outputs normalised; a layer with
                 ``kv_from: j`` has no key and value projections and reads the cache of layer j;
* ``parallel``   two mixers side by side on the same input (``SideBySide`` with ``normed_mean``): softmax attention with a
                 sink in its denominator, queries and keys normalised per head, no rotation (``MapsAttention`` with one
                 map), and a gated delta rule with one decay per head behind short convolutions (``GatedDeltaRule``);
                 each side's output is normalised over the model width with a weight, the result is their mean;

a feed-forward per layer (gated, g <- min(g, limit), u <- clamp(u, -limit, limit), g sigmoid(1.702 g) (u + 1)) or none;
a final norm and a head.

``config.json`` (key ``architecture``) gives every size and every constant that differs between models of the design.
Tensor names follow the checkpoint: ``embed``, ``head``, ``final.norm`` and ``l<i>.norm1``, ``l<i>.norm1b``,
``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .kapudra import DEFAULT_MAX_POSITIONS, _int, _num, _obj
from .qwen2 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


@dataclass(frozen=True)
class TutunexConfig:
    """The parsed ``config.json``; ``layers`` keeps each layer's object as read (validated)."""

    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()

    architecture = "Tutunex"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TutunexConfig":
        if d.get("architecture", d.get("architectures", ["Tutunex"])) not in ("Tutunex", ["Tutunex"]):
            raise ConfigError("not a Tutunex configuration")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("layers must be a non-empty list")
        for i, L in enumerate(layers):
            _check_layer(_obj(L, f"layers[{i}]"), f"layers[{i}]", i, layers)
        return cls(
            vocab=_int(d, "vocab", "config"), width=_int(d, "width", "config"),
            embedding_scale=_num(_obj(d.get("embedding"), "embedding"), "scale", "embedding"),
            norm_eps=_num(_obj(d.get("norm"), "norm"), "eps", "norm"), layers=tuple(layers),
            max_positions=_int(d, "max_positions", "config") if "max_positions" in d else DEFAULT_MAX_POSITIONS)

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "layers": list(self.layers)}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out


def _check_heads(o: Dict[str, Any], what: str) -> None:
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _int(o, key, what)
    if o["heads"] % o["kv_heads"]:
        raise ConfigError(f"{what}: {o['heads']} heads do not divide into {o['kv_heads']} kv_heads")


def _check_rot(rot: Dict[str, Any], dim: int, what: str) -> None:
    dims = _int(rot, "dims", what, 2)
    if dims % 2 or dims > dim:
        raise ConfigError(f"{what}.dims {dims} must be even and at most the map's {dim} channels")
    if not _num(rot, "base", what) > 1:
        raise ConfigError(f"{what}.base must exceed 1")
    if rot.get("scaling") is not None:
        sc = _obj(rot["scaling"], what + ".scaling")
        for key in ("factor", "original", "fast", "slow"):
            _num(sc, key, what + ".scaling")


def _check_layer(L: Dict[str, Any], what: str, index: int, layers: List[Any]) -> None:
    kind = L.get("type")
    m = _obj(L.get("mixer"), what + ".mixer")
    if kind == "attention":
        _check_heads(m, what + ".mixer")
        _num(m, "scale", what + ".mixer")
        _num(m, "diff", what + ".mixer", positive=False)
        if m.get("rot") is not None:
            _check_rot(_obj(m["rot"], what + ".mixer.rot"), m["dim"], what + ".mixer.rot")
        if m.get("mask") is not None:
            _int(_obj(m["mask"], what + ".mixer.mask"), "size", what + ".mixer.mask")
        src = m.get("kv_from")
        if src is not None:
            if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < index:
                raise ConfigError(f"{what}.mixer.kv_from {src!r} must name an earlier layer")
            other = layers[src] if isinstance(layers[src], dict) else {}
            om = other.get("mixer") if isinstance(other.get("mixer"), dict) else {}
            if other.get("type") != "attention" or om.get("kv_from") is not None:
                raise ConfigError(f"{what}.mixer.kv_from: layer {src} has no keys and values of its own to share")
            if any(om.get(key) != m.get(key) for key in ("kv_heads", "dim", "vdim", "rot")):
                raise ConfigError(f"{what}.mixer.kv_from: layer {src}'s keys and values have other sizes or another rotation")
    elif kind == "parallel":
        left, right = _obj(m.get("left"), what + ".mixer.left"), _obj(m.get("right"), what + ".mixer.right")
        _check_heads(left, what + ".mixer.left")
        _check_heads(right, what + ".mixer.right")
        _num(left, "scale", what + ".mixer.left")
        _int(right, "conv", what + ".mixer.right", 1, 16)
    else:
        raise ConfigError(f"{what}.type {kind!r} is not a mixer of this design (attention, parallel)")
    mlp = L.get("mlp")
    if mlp is not None:
        if _obj(mlp, what + ".mlp").get("kind") != "dense":
            raise ConfigError(f"{what}.mlp.kind {mlp.get('kind')!r} is not implemented (dense, or null for none)")
        _int(mlp, "ff", what + ".mlp")
        _num(mlp, "limit", what + ".mlp")


def _mixer_spec(L: Dict[str, Any], width: int, eps: float) -> Tuple[PartSpec, Optional[PartSpec]]:
    """(mixer, position encoding of the layer)."""
    m = L["mixer"]
    if L["type"] == "attention":
        rot = m.get("rot")
        position = None
        if rot is not None:
            position = PartSpec("rope_computed", dict(rotary_dim=rot["dims"], theta=float(rot["base"]),
                                                      scaling=dict(rot["scaling"]) if rot.get("scaling") is not None else None))
        mask = m.get("mask")
        return PartSpec("attention_maps", dict(
            hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
            scale=float(m["scale"]), maps=2, lambda_init=float(m["diff"]), chunk=mask["size"] if mask is not None else None,
            eps=eps, own_kv=m.get("kv_from") is None, float32_output=True)), position
    left, right = m["left"], m["right"]
    attention = PartSpec("attention_maps", dict(
        hidden_size=width, num_heads=left["heads"], num_kv_heads=left["kv_heads"], head_dim=left["dim"],
        v_head_dim=left["vdim"], scale=float(left["scale"]), maps=1, sink=True, qk_norm="head", eps=eps))
    delta = PartSpec("gated_delta_rule", dict(
        hidden_size=width, num_heads=right["heads"], num_kv_heads=right["kv_heads"], head_dim=right["dim"],
        v_head_dim=right["vdim"], conv_taps=right["conv"], eps=eps, decay="head", low_rank=False, gate_activation="silu"))
    return PartSpec("side_by_side", dict(hidden_size=width, mixers=(("left", attention, 1.0), ("right", delta, 1.0)),
                                         combine="normed_mean", eps=eps)), None


def tutunex_schedule(layers) -> List[ScheduleEntry]:
    """Every layer once, in order; a layer with ``kv_from: j`` reads the cache that layer j's entry wrote."""
    return [ScheduleEntry(i, cache_from=L["mixer"].get("kv_from") if L["type"] == "attention" else None)
            for i, L in enumerate(layers)]


def tutunex_model_spec(c: TutunexConfig) -> ModelSpec:
    norm = lambda: PartSpec("rmsnorm", dict(size=c.width, eps=c.norm_eps, tensor=""))
    layers = []
    for i, L in enumerate(c.layers):
        mixer, position = _mixer_spec(L, c.width, c.norm_eps)
        parts = {"mixer_norm": norm(), "mixer": mixer, "mixer_post_norm": norm()}
        if L.get("mlp") is not None:
            parts.update({"feed_forward_norm": norm(), "feed_forward_post_norm": norm(),
                          "feed_forward": PartSpec("gated_mlp", dict(
                              hidden_size=c.width, intermediate_size=L["mlp"]["ff"], activation="swish_clamped",
                              activation_constant=float(L["mlp"]["limit"]), tensors=("gate", "up", "down"),
                              float32_output=True))})
        layers.append(LayerSpec(f"l{i}", "sandwich_residual", parts, position,
                                names={"mixer_norm": "norm1", "mixer": "mix", "mixer_post_norm": "norm1b",
                                       "feed_forward_norm": "norm2", "feed_forward": "mlp",
                                       "feed_forward_post_norm": "norm2b"}))
    return ModelSpec(
        architecture=c.architecture, hidden_size=c.width, vocab_size=c.vocab, max_positions=c.max_positions,
        embedding_name="embed", layers=layers, schedule=tutunex_schedule(c.layers), final_norm=norm(),
        final_norm_name="final.norm", head_name="head", embedding_scale=c.embedding_scale, bare_tensor_names=True)
