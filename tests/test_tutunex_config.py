"""The Tutunex configuration without a GPU: what config.json must hold, what is refused, how the layers are laid out
as parts, which tensors a checkpoint must have, and the host-side numbers the kernels get."""
import copy
import math
import struct

import numpy as np
import pytest
import torch

import plain_tutunex as plain
import tutunex_cases as tc
from coheryn_ai_studio_b200.config.qwen2 import ConfigError
from coheryn_ai_studio_b200.config.registry import architecture_for, registered_architectures
from coheryn_ai_studio_b200.config.tutunex import TutunexConfig, tutunex_model_spec
from coheryn_ai_studio_b200.parts.base import FixedState, PagedKV, Runtime
from coheryn_ai_studio_b200.parts.model import DecoderModel


def model_of(cfg):
    return DecoderModel(tutunex_model_spec(TutunexConfig.from_dict(cfg)), Runtime(torch.bfloat16, torch.device("cpu")))


def test_registered_by_name():
    assert "Tutunex" in registered_architectures()
    assert architecture_for({"architecture": "Tutunex"}).name == "Tutunex"


@pytest.mark.parametrize("name", sorted(tc.CASES))
def test_round_trip_and_layout(name):
    cfg = tc.CASES[name][0]
    c = TutunexConfig.from_dict(cfg)
    assert TutunexConfig.from_dict(c.to_dict()) == c
    spec = tutunex_model_spec(c)
    spec.validate()
    assert [e.layer for e in spec.schedule] == list(range(len(cfg["layers"])))
    for e, L in zip(spec.schedule, cfg["layers"]):
        assert e.cache_from == (L["mixer"].get("kv_from") if L["type"] == "attention" else None)
        assert spec.layers[e.layer].arrangement == "sandwich_residual"
    m = model_of(cfg)
    needs = m.cache_requirements()
    for need, L in zip(needs, cfg["layers"]):
        mx = L["mixer"]
        if L["type"] == "attention":
            want = None if mx.get("kv_from") is not None else PagedKV(mx["kv_heads"], 2 * mx["dim"], None, mx["vdim"])
            assert need == want
        else:
            left, right = mx["left"], mx["right"]
            assert need[0] == PagedKV(left["kv_heads"], left["dim"], None, left["vdim"])
            channels = 2 * right["kv_heads"] * right["dim"] + right["heads"] * right["vdim"]
            assert need[1] == FixedState((right["heads"] * right["dim"] * right["vdim"] + (right["conv"] - 1) * channels,), torch.float32)


def test_tensor_names_and_shapes():
    cfg = tc.T1
    specs = model_of(cfg).tensor_specs()
    W = cfg["width"]
    want = {"embed": (300, W), "head": (300, W), "final.norm": (W,)}
    for i, L in enumerate(cfg["layers"]):
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if L["mlp"] else ()):
            want[f"l{i}.{n}"] = (W,)
        if L["mlp"]:
            want.update({f"l{i}.mlp.gate": (L["mlp"]["ff"], W), f"l{i}.mlp.up": (L["mlp"]["ff"], W), f"l{i}.mlp.down": (W, L["mlp"]["ff"])})
        m = L["mixer"]
        if L["type"] == "attention":
            want.update({f"l{i}.mix.q": (m["heads"] * 2 * m["dim"], W), f"l{i}.mix.o": (W, m["heads"] * m["vdim"])})
            want.update({f"l{i}.mix.{n}": (m["dim"],) for n in ("lq1", "lk1", "lq2", "lk2")})
            if m.get("kv_from") is None:
                want.update({f"l{i}.mix.k": (m["kv_heads"] * 2 * m["dim"], W), f"l{i}.mix.v": (m["kv_heads"] * m["vdim"], W)})
        else:
            a, b = m["left"], m["right"]
            p = f"l{i}.mix.left"
            want.update({p + ".q": (a["heads"] * a["dim"], W), p + ".k": (a["kv_heads"] * a["dim"], W), p + ".v": (a["kv_heads"] * a["vdim"], W),
                         p + ".q.norm": (a["dim"],), p + ".k.norm": (a["dim"],), p + ".o": (W, a["heads"] * a["vdim"]), p + ".out": (W,)})
            p = f"l{i}.mix.right"
            want.update({p + ".q": (b["kv_heads"] * b["dim"], W), p + ".q.conv": (b["kv_heads"] * b["dim"], b["conv"]),
                         p + ".k": (b["kv_heads"] * b["dim"], W), p + ".k.conv": (b["kv_heads"] * b["dim"], b["conv"]),
                         p + ".v": (b["heads"] * b["vdim"], W), p + ".v.conv": (b["heads"] * b["vdim"], b["conv"]),
                         p + ".b": (b["heads"], W), p + ".a": (b["heads"], W), p + ".A_log": (b["heads"],), p + ".dt_bias": (b["heads"],),
                         p + ".g": (b["heads"] * b["vdim"], W), p + ".norm": (b["vdim"],), p + ".o": (W, b["heads"] * b["vdim"]),
                         p + ".out": (W,)})
    assert {n: tuple(s.shape) for n, s in specs.items()} == want


def _changed(path, value, base=tc.T1):
    cfg = copy.deepcopy(base)
    node = cfg
    for key in path[:-1]:
        node = node[key]
    if value is KeyError:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value", [
    (("layers", 0, "type"), "mlstm"), (("layers", 0, "mixer", "heads"), 3), (("layers", 0, "mixer", "scale"), KeyError),
    (("layers", 0, "mixer", "diff"), "x"), (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "rot", "dims"), 34),
    (("layers", 0, "mixer", "rot", "scaling", "factor"), 0), (("layers", 0, "mixer", "mask", "size"), 0),
    (("layers", 2, "mixer", "kv_from"), 2), (("layers", 2, "mixer", "kv_from"), 1), (("layers", 2, "mixer", "dim"), 16),
    (("layers", 1, "mixer", "right", "conv"), 0), (("layers", 1, "mixer", "left", "scale"), -1.0),
    (("layers", 0, "mlp", "kind"), "moe"), (("layers", 0, "mlp", "limit"), 0), (("norm", "eps"), KeyError), (("vocab",), 0)])
def test_refused(path, value):
    with pytest.raises(ConfigError):
        TutunexConfig.from_dict(_changed(path, value))


def test_options_that_may_be_absent():
    """No rotation, no scaling, no chunks, no feed-forward: each is a model of the design."""
    for path in (("layers", 0, "mixer", "rot", "scaling"), ("layers", 0, "mixer", "mask")):
        cfg = _changed(path, KeyError)
        cfg = _changed(("layers", 2, "mixer") + path[3:], KeyError, cfg)
        model_of(cfg)
    cfg = _changed(("layers", 0, "mixer", "rot"), KeyError)
    cfg = _changed(("layers", 2, "mixer", "rot"), KeyError, cfg)
    m = model_of(cfg)
    assert m.layers[0].mixer.position is None
    assert model_of(_changed(("layers", 0, "mlp"), None)).layers[0].feed_forward is None


@pytest.mark.parametrize("rot", [{"dims": 16, "base": 1000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}},
                                 {"dims": 64, "base": 500000.0, "scaling": {"factor": 32.0, "original": 8192, "fast": 32.0, "slow": 1.0}},
                                 {"dims": 6, "base": 77.0}])
def test_frequencies_as_pairs_of_floats(rot):
    from coheryn_ai_studio_b200.parts.position import ComputedRope
    part = ComputedRope(Runtime(torch.float32, torch.device("cpu")), rot["dims"], rot["base"], rot.get("scaling"))
    f, amp = plain.rotary_frequencies(rot)
    assert np.allclose(part.frequencies(), f, rtol=1e-14, atol=0) and math.isclose(part.amplitude, amp, rel_tol=1e-14)
    pairs = part.frequency_pairs().numpy().astype(np.float64)
    assert np.abs(pairs.sum(-1) - f).max() <= 1e-14 * f.max() + 1e-15          # the pair carries what one float loses
    if "scaling" in rot:
        assert f[0] == rot["base"] ** 0.0 and f[-1] < rot["base"] ** (-2.0 * (len(f) - 1) / rot["dims"])   # fast pairs kept, slow ones stretched


@pytest.mark.parametrize("limit", [0.25, 1.5, 7.0, 1.3, 1e-3, 3e4])
def test_the_epilogue_word_carries_the_constant(limit):
    from coheryn_ai_studio_b200 import ops
    word = ops.gated_epilogue_word("swish_clamped", limit)
    assert word & 0xff == 3 and word > 0
    back = struct.unpack("<f", struct.pack("<I", word & 0xffffff00))[0]
    assert abs(back - limit) <= limit * 2.0 ** -16
    assert ops.gated_epilogue_word("silu") == 1 and ops.gated_epilogue_word("gelu_tanh") == 2
    with pytest.raises(ops.KernelError):
        ops.gated_epilogue_word("swish_clamped", None)


def test_the_plain_mask_and_sink():
    m = plain.visible(7, 3)
    assert m.sum() == 1 + 2 + 3 + 1 + 2 + 3 + 1 and m[3, 2] == 0 and m[5, 3] == 1
    s = np.zeros((1, 4))
    assert np.allclose(plain.softmax_rows(s, np.ones((1, 4), bool), sink=True), 0.2)
    assert np.allclose(plain.softmax_rows(s, np.ones((1, 4), bool)), 0.25)
