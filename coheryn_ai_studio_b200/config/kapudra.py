"""Typed configuration of the Kapudra decoder and its layout as parts.

The design: an embedding multiplied by a constant; layers of the form x <- x + mixer(h) + ff(h) with ONE
norm h = rmsnorm(x) read by both; two kinds of mixer, chosen per layer by ``type``:

* ``mlstm``     a stabilised matrix memory per head (``parts/recurrent.py``: ``MatrixMemory``);
* ``parallel``  two mixers side by side on the same input, their outputs added with a weight each:
                windowed softmax attention whose scores lose a slope times the distance, with queries and
                keys normalised over the whole projection and no rotation (``DistanceBiasAttention``), and a
                gated delta rule behind short convolutions (``GatedDeltaRule``);

a feed-forward per layer (gated, tanh-form GELU) or none; a span of layers that runs several times in a row
with the same weights and a cache or state per run, each pass opened by adding a vector of the pass (and, from
the second pass on, the embedding output once more); a final norm, a head, scaled and softly capped logits.

``config.json`` gives every size and every constant; nothing of them stands in code.  Tensor names follow the
checkpoint: ``embed``, ``head``, ``final.norm``, ``loop.step`` and ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .qwen2 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, StreamInject

# No table depends on the position (the attention's bias is a function of the distance and the other mixers
# are recurrences), so the bound on positions is only what the engine's index arithmetic is sized for.
DEFAULT_MAX_POSITIONS = 1 << 20


def _obj(d: Any, what: str) -> Dict[str, Any]:
    if not isinstance(d, dict):
        raise ConfigError(f"{what} must be an object")
    return d


def _int(d: Dict[str, Any], key: str, what: str, minimum: int = 1, maximum: int = 1 << 24) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or not minimum <= v <= maximum:
        raise ConfigError(f"{what}.{key} must be an integer in {minimum}..={maximum}, got {v!r}")
    return v


def _num(d: Dict[str, Any], key: str, what: str, positive: bool = True) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or (positive and v <= 0):
        raise ConfigError(f"{what}.{key} must be a finite{' positive' if positive else ''} number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class KapudraConfig:
    """The parsed ``config.json``; ``layers`` keeps each layer's object as read (validated)."""

    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    logit_scale: float
    logit_softcap: float
    layers: Tuple[Dict[str, Any], ...]
    loop: Optional[Tuple[int, int, int]]          # (start, stop, times)
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()

    architecture = "Kapudra"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "KapudraConfig":
        if d.get("architecture", d.get("architectures", ["Kapudra"])) not in ("Kapudra", ["Kapudra"]):
            raise ConfigError("not a Kapudra configuration")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("layers must be a non-empty list")
        for i, L in enumerate(layers):
            _check_layer(_obj(L, f"layers[{i}]"), f"layers[{i}]")
        loop = None
        if d.get("loop") is not None:
            lo = _obj(d["loop"], "loop")
            start = _int(lo, "start", "loop", 0, len(layers))
            stop = _int(lo, "stop", "loop", 0, len(layers))
            times = _int(lo, "times", "loop", 1, 1 << 10)
            if stop <= start:
                raise ConfigError(f"loop.stop {stop} must lie beyond loop.start {start}")
            loop = (start, stop, times)
        return cls(
            vocab=_int(d, "vocab", "config"), width=_int(d, "width", "config"),
            embedding_scale=_num(_obj(d.get("embedding"), "embedding"), "scale", "embedding"),
            norm_eps=_num(_obj(d.get("norm"), "norm"), "eps", "norm"),
            logit_scale=_num(d, "logit_scale", "config"), logit_softcap=_num(d, "logit_softcap", "config"),
            layers=tuple(layers), loop=loop,
            max_positions=_int(d, "max_positions", "config") if "max_positions" in d else DEFAULT_MAX_POSITIONS)

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "logit_scale": self.logit_scale, "logit_softcap": self.logit_softcap, "layers": list(self.layers)}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out


def _check_layer(L: Dict[str, Any], what: str) -> None:
    kind = L.get("type")
    m = _obj(L.get("mixer"), what + ".mixer")
    if kind == "mlstm":
        for key in ("heads", "dim", "vdim"):
            _int(m, key, what + ".mixer")
        _num(m, "gate_cap", what + ".mixer")
    elif kind == "parallel":
        left, right = _obj(m.get("left"), what + ".mixer.left"), _obj(m.get("right"), what + ".mixer.right")
        for side, o in (("left", left), ("right", right)):
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _int(o, key, f"{what}.mixer.{side}")
            if o["heads"] % o["kv_heads"]:
                raise ConfigError(f"{what}.mixer.{side}: {o['heads']} heads do not divide into {o['kv_heads']} kv_heads")
        _num(left, "scale", what + ".mixer.left")
        _int(_obj(left.get("mask"), what + ".mixer.left.mask"), "size", what + ".mixer.left.mask")
        _int(right, "conv", what + ".mixer.right", 1, 16)
        for key in ("a_rank", "g_rank"):      # the inner sizes of the two-step projections: a checkpoint's tensors give
            if key in right:                  # them; a configuration names them only so that random weights can be made
                _int(right, key, what + ".mixer.right")
        _num(m, "left_scale", what + ".mixer", positive=False)
        _num(m, "right_scale", what + ".mixer", positive=False)
    else:
        raise ConfigError(f"{what}.type {kind!r} is not a mixer of this design (mlstm, parallel)")
    mlp = L.get("mlp")
    if mlp is not None:
        if _obj(mlp, what + ".mlp").get("kind") != "dense":
            raise ConfigError(f"{what}.mlp.kind {mlp.get('kind')!r} is not implemented (dense, or null for none)")
        _int(mlp, "ff", what + ".mlp")


def _mixer_spec(L: Dict[str, Any], width: int, eps: float) -> PartSpec:
    m = L["mixer"]
    if L["type"] == "mlstm":
        return PartSpec("matrix_memory", dict(hidden_size=width, num_heads=m["heads"], head_dim=m["dim"],
                                              v_head_dim=m["vdim"], gate_cap=float(m["gate_cap"]), eps=eps))
    left, right = m["left"], m["right"]
    attention = PartSpec("attention_distance_bias", dict(
        hidden_size=width, num_heads=left["heads"], num_kv_heads=left["kv_heads"], head_dim=left["dim"],
        v_head_dim=left["vdim"], window=left["mask"]["size"], scale=float(left["scale"]), slope_exponent=8.0,
        qk_norm="projection", eps=eps))
    delta = PartSpec("gated_delta_rule", dict(
        hidden_size=width, num_heads=right["heads"], num_kv_heads=right["kv_heads"], head_dim=right["dim"],
        v_head_dim=right["vdim"], conv_taps=right["conv"], eps=eps,
        decay_rank=right.get("a_rank"), gate_rank=right.get("g_rank")))
    return PartSpec("side_by_side", dict(hidden_size=width, mixers=(("left", attention, float(m["left_scale"])),
                                                                    ("right", delta, float(m["right_scale"])))))


def kapudra_schedule(n_layers: int, loop: Optional[Tuple[int, int, int]]) -> List[ScheduleEntry]:
    """Layers before the span once, the span ``times`` times (each run an entry of its own, hence a cache or
    state of its own), the rest once.  The first entry of pass t adds row t of ``loop.step``, and from the
    second pass on the embedding output before it."""
    if loop is None:
        return [ScheduleEntry(i) for i in range(n_layers)]
    start, stop, times = loop
    entries = [ScheduleEntry(i) for i in range(start)]
    for t in range(times):
        for i in range(start, stop):
            inject = StreamInject(embedding=t > 0, vector=("loop.step", t)) if i == start else None
            entries.append(ScheduleEntry(i, inject=inject))
    return entries + [ScheduleEntry(i) for i in range(stop, n_layers)]


def kapudra_model_spec(c: KapudraConfig) -> ModelSpec:
    norm = lambda: PartSpec("rmsnorm", dict(size=c.width, eps=c.norm_eps, tensor=""))
    layers = []
    for i, L in enumerate(c.layers):
        parts = {"norm": norm(), "mixer": _mixer_spec(L, c.width, c.norm_eps)}
        if L.get("mlp") is not None:
            parts["feed_forward"] = PartSpec("gated_mlp", dict(
                hidden_size=c.width, intermediate_size=L["mlp"]["ff"], activation="gelu_tanh",
                tensors=("gate", "up", "down")))
        layers.append(LayerSpec(f"l{i}", "parallel_residual", parts,
                                names={"norm": "norm1", "mixer": "mix", "feed_forward": "mlp"}))
    extra = {}
    if c.loop is not None:
        extra["loop.step"] = ((c.loop[2], c.width), "vector", "bias")
    return ModelSpec(
        architecture=c.architecture, hidden_size=c.width, vocab_size=c.vocab, max_positions=c.max_positions,
        embedding_name="embed", layers=layers, schedule=kapudra_schedule(len(c.layers), c.loop),
        final_norm=norm(), final_norm_name="final.norm", head_name="head", embedding_scale=c.embedding_scale,
        logit_scale=c.logit_scale, logit_softcap=c.logit_softcap, bare_tensor_names=True, extra_tensors=extra)
