"""Small Kapudra configurations of the tests (they differ from each other in every size and option), folders of
seeded random weights for them, and the comparison of engine rows with the plain implementation."""
from __future__ import annotations

import json
from typing import Dict, List

import numpy as np
import torch

import plain_kapudra as plain
from plain_qwen2 import read_safetensors

LOUD = dict(matrix_std=0.12, bias_std=0.4, norm_jitter=0.1, conv_std=0.5)


def _parallel(left, right, ls, rs, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _mlstm(heads, dim, vdim, cap, ff):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


# K1: values wider than keys in the attention, grouped query/key heads in the delta rule, four taps, a span that
# starts at layer 0 and runs three times, a layer without feed-forward.
K1 = {
    "architecture": "Kapudra", "vocab": 300, "width": 80, "embedding": {"scale": 3.5}, "norm": {"eps": 1e-5},
    "logit_scale": 0.5, "logit_softcap": 12.0, "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [
        _parallel({"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.2, "mask": {"size": 24}},
                  {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 4, "a_rank": 8, "g_rank": 16}, 0.7, 1.3, 96),
        _mlstm(2, 24, 40, 8.0, None),
        _parallel({"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.3, "mask": {"size": 9}},
                  {"heads": 2, "kv_heads": 1, "dim": 40, "vdim": 32, "conv": 2, "a_rank": 4, "g_rank": 4}, 1.0, 0.5, 64),
    ]}

# K2: three heads over one kv head, a window of five, one head of matrix memory, a width that is no multiple
# of sixteen, no repeated span, the span's vector absent.
K2 = {
    "architecture": "Kapudra", "vocab": 515, "width": 72, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "logit_scale": 1.5, "logit_softcap": 50.0,
    "layers": [
        _mlstm(1, 64, 16, 15.0, 104),
        _parallel({"heads": 3, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.18, "mask": {"size": 5}},
                  {"heads": 3, "kv_heads": 3, "dim": 8, "vdim": 64, "conv": 3, "a_rank": 12, "g_rank": 8}, 1.2, 0.9, 48),
        _mlstm(3, 16, 16, 6.0, 40),
    ]}

# K3: a span in the middle that runs once (its vector is still added), one tap (no convolution state).
K3 = {
    "architecture": "Kapudra", "vocab": 128, "width": 64, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6},
    "logit_scale": 0.25, "logit_softcap": 30.0, "loop": {"start": 1, "stop": 2, "times": 1},
    "layers": [
        _mlstm(2, 32, 32, 10.0, 128),
        _parallel({"heads": 2, "kv_heads": 1, "dim": 48, "vdim": 80, "scale": 0.15, "mask": {"size": 40}},
                  {"heads": 1, "kv_heads": 1, "dim": 64, "vdim": 128, "conv": 1, "a_rank": 16, "g_rank": 16}, 0.9, 1.1, 128),
    ]}

# K4: sizes that no vector width divides (a width of 100, head sizes of 12, 20, 24 and 30, 50 feed-forward channels, five
# taps, 101 ids): every kernel's scalar path and the products' fallback.
K4 = {
    "architecture": "Kapudra", "vocab": 101, "width": 100, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
    "logit_scale": 0.7, "logit_softcap": 20.0, "loop": {"start": 0, "stop": 3, "times": 2},
    "layers": [
        _parallel({"heads": 6, "kv_heads": 3, "dim": 24, "vdim": 24, "scale": 0.2, "mask": {"size": 17}},
                  {"heads": 3, "kv_heads": 1, "dim": 20, "vdim": 30, "conv": 5, "a_rank": 6, "g_rank": 10}, 0.6, 1.4, 50),
        _mlstm(5, 12, 20, 9.0, None),
        _mlstm(1, 20, 30, 11.0, 50),
    ]}

CASES = {"K1": (K1, 11), "K2": (K2, 12), "K3": (K3, 13), "K4": (K4, 14)}


def make_folder(tmp_path, name: str) -> str:
    from coheryn_ai_studio_b200.config.kapudra import KapudraConfig
    from coheryn_ai_studio_b200.engine import write_random_model
    from coheryn_ai_studio_b200.weights import InitPolicy
    cfg, seed = CASES[name]
    d = str(tmp_path / f"kapudra_{name}")
    write_random_model(d, KapudraConfig.from_dict(cfg), seed, InitPolicy(**LOUD))
    return d


def read_model(folder: str):
    with open(f"{folder}/config.json") as f:
        config = json.load(f)
    return config, read_safetensors(f"{folder}/model.safetensors")


_rows: Dict[tuple, np.ndarray] = {}


def plain_rows(folder: str, tokens: List[int], rounded: bool = False) -> np.ndarray:
    key = (folder, tuple(tokens), rounded)
    if key not in _rows:
        config, w = read_model(folder)
        _rows[key] = plain.forward(config, w, tokens, rounded=rounded)
    return _rows[key]


# float32: only the order of sums differs.  bfloat16: weights are the same bits, activations are rounded to eight bits of
# mantissa between the kernels.  What that costs a row by itself is measured on the plain model's rounded twin
# (``plain.forward(rounded=True)``); the engine's rounding errors are other draws of the same noise, so a bfloat16 engine row
# may be a small factor further from the unrounded row than the twin is (``replay.bf16_excess``: twice in root mean square,
# three times in its largest element, in units of which 1.0 is the bound).  Over the rows of a test: none beyond one and a
# half bounds, at most one in twenty (or one) beyond one.  The tests with a key or a state made to stand out show that a lost
# key, state or window edge moves a row by far more than this.  K4 (heads of 12 to 30 channels) is the exception: where a
# head's output nearly cancels before its norm, rounding noise is amplified at single rows, in the twin and in the engine
# at different ones; its bfloat16 rows are held to the bound in the median and to eight bounds at most, and its float32
# rows, which run the same kernels' scalar paths, to 2e-4 like all others.
TOL_F32 = 2e-4
WORST = {"float32": 0.0, "bfloat16": 0.0}


def check_rows(rows: Dict[tuple, np.ndarray], folder: str, sequences: Dict[str, List[int]], dtype: str, label: str = ""):
    from replay import bf16_excess
    assert rows, "nothing was compared"
    excesses = []
    for (rid, pos), row in sorted(rows.items()):
        ref = plain_rows(folder, sequences[rid])[pos]
        if dtype == "float32":
            d = np.abs(row.astype(np.float64) - ref).max()
            WORST[dtype] = max(WORST[dtype], float(d))
            assert d <= TOL_F32 * max(1.0, float(np.std(ref))), f"{label} {rid}@{pos}: |d| = {d:.3e}"
        else:
            twin = plain_rows(folder, sequences[rid], rounded=True)[pos]
            excesses.append((bf16_excess(row, ref.astype(np.float32), twin.astype(np.float32)), rid, pos))
    if excesses:
        values = np.array([e[0] for e in excesses])
        worst = max(excesses)
        if folder.endswith("K4"):
            assert np.median(values) <= 1.0 and worst[0] <= 8.0, f"{label}: median {np.median(values):.2f}, worst {worst}"
            return
        WORST[dtype] = max(WORST[dtype], worst[0])
        over = int((values > 1.0).sum())
        assert worst[0] <= 1.5, f"{label} {worst[1]}@{worst[2]}: {worst[0]:.2f} of the bfloat16 bound"
        assert over <= max(1, len(values) // 20), f"{label}: {over} of {len(values)} rows beyond the bfloat16 bound"


def noisy_replay(folder: str, dtype: str, max_tokens: int, model, max_requests: int = 4, page_size: int = 16, **kw):
    """The replay harness with the state slots full of noise as well as the pages: a request then has to start from
    a slot that its admission zeroed, and a slot that is used again shows what its last owner left."""
    from replay import Replay
    r = Replay(folder, dtype, max_tokens=max_tokens, model=model, max_requests=max_requests, page_size=page_size, **kw)
    for t in r.cache.state_tensors():
        t.normal_(0.0, 4.0)
    return r


def prompt(seed: int, n: int, vocab: int) -> List[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
