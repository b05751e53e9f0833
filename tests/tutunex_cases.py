"""Small Tutunex configurations of the tests (they differ from each other in every size and option), folders of
seeded random weights for them, and the comparison of engine rows with the plain implementation."""
from __future__ import annotations

import json
from typing import Dict, List

import numpy as np

import plain_tutunex as plain
from plain_qwen2 import read_safetensors

LOUD = dict(matrix_std=0.12, bias_std=0.4, norm_jitter=0.1, conv_std=0.5)


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _attention(heads, kv_heads, dim, vdim, scale, diff, rot=None, chunk=None, kv_from=None, ff=None, limit=2.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if rot is not None:
        m["rot"] = rot
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def _parallel(left, right, ff=None, limit=2.0):
    return {"type": "parallel", "mixer": {"left": left, "right": right},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def _side(heads, kv_heads, dim, vdim, **more):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, **more)


# T1: sizes the tensor-core kernels take.  Half of every map rotated with YaRN scaling, chunks of 24 positions (a page
# and a half), a layer that reads the first one's keys and values, a side-by-side layer, a layer without feed-forward.
T1 = {
    "architecture": "Tutunex", "vocab": 300, "width": 64, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "layers": [
        _attention(4, 2, 32, 16, 0.25, 0.35, _rot(16, 1000.0, (4.0, 64, 8.0, 1.0)), chunk=24, ff=96, limit=0.75),
        _parallel(_side(4, 2, 16, 32, scale=0.3), _side(4, 2, 16, 24, conv=4), ff=None),
        _attention(4, 2, 32, 16, 0.2, 0.5, _rot(16, 1000.0, (4.0, 64, 8.0, 1.0)), chunk=24, kv_from=0, ff=64, limit=1.25),
    ]}

# T2: the side-by-side layer first; one kv head under three heads; a whole map rotated without scaling; no chunks
# (every earlier position is seen); three taps; widths and head sizes that are multiples of 16 but differ everywhere.
T2 = {
    "architecture": "Tutunex", "vocab": 515, "width": 80, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "layers": [
        _parallel(_side(3, 1, 32, 16, scale=0.18), _side(2, 1, 32, 16, conv=3), ff=48, limit=0.5),
        _attention(3, 1, 16, 48, 0.3, 0.8, _rot(16, 50.0), chunk=None, ff=None),
        _attention(2, 2, 48, 32, 0.15, 0.2, None, chunk=7, ff=112, limit=3.0),
    ]}

# T3: sizes that no vector width and no tensor-core tile divides (a width of 100, maps of 12 and 20 channels, values of 10,
# 30 and 36, 50 feed-forward channels, five taps, one tap, 101 ids): the float32-arithmetic kernels in both precisions and
# the products' fallback.  One head everywhere in the last layer; chunks of one position (a row sees itself only).
T3 = {
    "architecture": "Tutunex", "vocab": 101, "width": 100, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
    "layers": [
        _attention(6, 3, 12, 10, 0.3, 0.6, _rot(6, 77.0, (2.0, 16, 4.0, 0.5)), chunk=17, ff=50, limit=1.0),
        _parallel(_side(2, 1, 20, 30, scale=0.25), _side(3, 1, 20, 36, conv=5), ff=50, limit=1.5),
        _attention(6, 3, 12, 10, 0.3, 0.1, _rot(6, 77.0, (2.0, 16, 4.0, 0.5)), chunk=5, kv_from=0),
        _parallel(_side(1, 1, 12, 12, scale=0.4), _side(1, 1, 12, 20, conv=1), ff=None),
        _attention(1, 1, 20, 30, 0.2, 0.45, _rot(20, 9.0), chunk=1, ff=50, limit=0.25),
    ]}

CASES = {"T1": (T1, 21), "T2": (T2, 22), "T3": (T3, 23)}


def make_folder(tmp_path, name: str) -> str:
    from coheryn_ai_studio_b200.config.tutunex import TutunexConfig
    from coheryn_ai_studio_b200.engine import write_random_model
    from coheryn_ai_studio_b200.weights import InitPolicy
    cfg, seed = CASES[name]
    d = str(tmp_path / f"tutunex_{name}")
    write_random_model(d, TutunexConfig.from_dict(cfg), seed, InitPolicy(**LOUD))
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


# float32: only the order of sums differs.  bfloat16: the weights are the same bits, activations are rounded to eight bits
# of mantissa between the kernels; what that costs a row by itself is measured on the plain model's rounded twin, and an
# engine row may be a small factor further from the unrounded row than the twin is (``replay.bf16_excess``).  Over the rows
# of a test: none beyond one and a half bounds, at most one in twenty (or one) beyond one.  T3 (maps of 12 channels, values
# of 10) is held to the bound in the median and to eight bounds at most: with so few channels a head's output can nearly
# cancel before its norm at single rows, which amplifies rounding noise there, in the twin and in the engine at different rows.
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
        if folder.endswith("T3"):
            assert np.median(values) <= 1.0 and worst[0] <= 8.0, f"{label}: median {np.median(values):.2f}, worst {worst}"
            return
        WORST[dtype] = max(WORST[dtype], worst[0])
        over = int((values > 1.0).sum())
        assert worst[0] <= 1.5, f"{label} {worst[1]}@{worst[2]}: {worst[0]:.2f} of the bfloat16 bound"
        assert over <= max(1, len(values) // 20), f"{label}: {over} of {len(values)} rows beyond the bfloat16 bound"


def noisy_replay(folder: str, dtype: str, max_tokens: int, model, max_requests: int = 4, page_size: int = 16, **kw):
    """The replay harness with the state slots full of noise as well as the pages."""
    from replay import Replay
    r = Replay(folder, dtype, max_tokens=max_tokens, model=model, max_requests=max_requests, page_size=page_size, **kw)
    for t in r.cache.state_tensors():
        t.normal_(0.0, 4.0)
    return r


def prompt(seed: int, n: int, vocab: int) -> List[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
