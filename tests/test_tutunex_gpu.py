"""The Tutunex decoder on the GPU against the plain implementation (``plain_tutunex.py``): each mechanism's kernel
alone, then whole models through the step function, the cache and the scheduler, in float32 and in bfloat16."""
import math
import types

import numpy as np
import pytest
import torch

import plain_tutunex as plain
import tutunex_cases as tc

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = ["T1", "T2", "T3"]
DEV = "cuda:0"


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("tutunex")
    return {n: tc.make_folder(base, n) for n in NAMES}


@pytest.fixture(scope="module")
def models(folders):
    from coheryn_ai_studio_b200.engine import load_model
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = load_model(folders[name], dtype)[1]
        return cache[(name, dtype)]
    return get


def vocab(name):
    return tc.CASES[name][0]["vocab"]


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=dtype).to(DEV)


def bf(a):
    """A float64 array rounded to bfloat16 values."""
    return torch.as_tensor(np.asarray(a), dtype=torch.float32).bfloat16().float().numpy().astype(np.float64)


class Paged:
    """A hand-made paged cache for one attention: requests of given lengths whose pages are handed out in a scrambled
    order, filled by the engine's own kernel, and steps over any runs of their positions."""

    def __init__(self, lengths, G, key_channels, dv, page, dtype, seed=0):
        self.page, self.G, self.kc, self.dv, self.dtype = page, G, key_channels, dv, dtype
        pages = [-(-n // page) for n in lengths]
        order = np.random.default_rng(seed).permutation(sum(pages) + 3)
        self.tables = np.full((len(lengths), max(pages) + 1), -1, dtype=np.int32)
        at = 0
        for r, n in enumerate(pages):
            self.tables[r, :n] = order[at:at + n]
            at += n
        self.k = torch.full((len(order), G, page, key_channels), 7.0, dtype=dtype, device=DEV)     # noise where nothing is written
        self.v = torch.full((len(order), G, page, dv), -5.0, dtype=dtype, device=DEV)

    def step(self, runs):
        """``runs``: (request, first position, tokens) in batch order; the requests' lengths are first + tokens."""
        req = np.concatenate([np.full(n, i) for i, (_, _, n) in enumerate(runs)]).astype(np.int32)
        pos = np.concatenate([np.arange(s, s + n) for _, s, n in runs]).astype(np.int32)
        cu = np.concatenate([[0], np.cumsum([n for _, _, n in runs])]).astype(np.int32)
        tables = np.stack([self.tables[r] for r, _, _ in runs])
        slots = np.concatenate([self.tables[r][np.arange(s, s + n) // self.page] * self.page + np.arange(s, s + n) % self.page
                                for r, s, n in runs]).astype(np.int32)
        kv = [s + n for _, s, n in runs]
        return types.SimpleNamespace(
            num_requests=len(runs), num_tokens=int(cu[-1]), token_req=dev(req, torch.int32), positions=dev(pos, torch.int32),
            cu_q=dev(cu, torch.int32), kv_lens=dev(kv, torch.int32), block_tables=[dev(tables, torch.int32)],
            slots=[dev(slots, torch.int32)], q_lens=[n for _, _, n in runs], max_q_len=max(n for _, _, n in runs),
            max_kv_len=max(kv), prior_positions_settled=True)


def write_and_attend(cache, step, q, k, v, heads, dk, maps, ops, simple=False, rot=None, norm=None, eps=1e-5, **opts):
    """q [T, heads*maps*dk], k [T, G*maps*dk], v [T, G*dv] (float64) through the engine's two kernels."""
    G, dv = cache.G, cache.dv
    wide = torch.zeros((q.shape[0], q.shape[1] + k.shape[1] + v.shape[1] + 3), device=DEV)     # slices of one wider buffer
    nq, nk = q.shape[1], k.shape[1]
    wide[:, :nq], wide[:, nq:nq + nk], wide[:, nq + nk:nq + nk + v.shape[1]] = dev(q), dev(k), dev(v)
    freq, rdims, amp = (None, 0, 1.0) if rot is None else rot
    qn, kn = (None, None) if norm is None else norm
    qd = ops.unit_norm_rope_kv_write(wide[:, :nq], wide[:, nq:nq + nk], wide[:, nq + nk:nq + nk + v.shape[1]], qn, kn, eps,
                                     step.positions, freq, rdims, amp, step.slots[0], cache.k, cache.v, heads * maps, G * maps, G,
                                     dk, dv, cache.page, cache.dtype)
    out = torch.empty((q.shape[0], heads * dv), dtype=cache.dtype, device=DEV)
    ops.attention_maps(qd, out, cache.k, cache.v, step, 0, heads, G, dk, dv, maps, cache.page, opts.get("window"),
                       opts.get("chunk"), opts.get("sink", False), opts.get("scale", 1.0), opts.get("lam", 0.0),
                       opts.get("head_norm", False), eps, opts.get("out_scale", 1.0), force_simple=simple)
    return out.float().cpu().numpy().astype(np.float64)


def plain_maps(q, k, v, heads, G, dk, dv, maps, scale, lam, chunk, sink, head_norm, eps, out_scale):
    """The plain attention of one whole sequence with the given options."""
    T = q.shape[0]
    q, k, v = q.reshape(T, heads * maps, dk), k.reshape(T, G * maps, dk), v.reshape(T, G, dv)
    mask = plain.visible(T, chunk)
    out = np.zeros((T, heads, dv))
    for h in range(heads):
        g = h // (heads // G)
        a = [plain.softmax_rows((q[:, maps * h + i] @ k[:, maps * g + i].T) * scale, mask, sink=sink) @ v[:, g] for i in range(maps)]
        o = a[0] - lam * a[1] if maps == 2 else a[0]
        out[:, h] = (plain.rms(o, eps) if head_norm else o) * out_scale
    return out.reshape(T, heads * dv)


# ------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dims,channels,scaling", [(16, 32, (4.0, 64, 8.0, 1.0)), (20, 20, None), (6, 12, (2.0, 16, 4.0, 0.5)),
                                                    (64, 64, (8.0, 4096, 32.0, 1.0))])
def test_norm_rotation_and_cache_write(dims, channels, scaling):
    """Units normalised with a shared weight, their first channels turned by computed angles (positions up to a million),
    keys laid into pages with the maps of a head side by side, values beside them."""
    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.parts.base import Runtime
    from coheryn_ai_studio_b200.parts.position import ComputedRope
    rng = np.random.default_rng(dims)
    rot = {"dims": dims, "base": 5000.0}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    part = ComputedRope(Runtime(torch.float32, torch.device(DEV)), dims, 5000.0, rot.get("scaling"))
    assert np.allclose(part.frequencies(), plain.rotary_frequencies(rot)[0], rtol=1e-14) and \
        math.isclose(part.amplitude, plain.rotary_frequencies(rot)[1], rel_tol=1e-14)
    H, G, maps, dv, page, n = 3, 1, 2, 10, 4, 9
    for first in (0, 5, 1_000_003):
        cache = Paged([first + n], G, maps * channels, dv, page, torch.float32)
        step = cache.step([(0, first, n)])
        q, k, v = rng.normal(size=(n, H * maps * channels)), rng.normal(size=(n, G * maps * channels)), rng.normal(size=(n, G * dv))
        wq, wk = rng.normal(size=channels) + 1, rng.normal(size=channels) + 1
        wide = torch.zeros((n, q.shape[1] + k.shape[1] + v.shape[1]), device=DEV)
        wide[:, :q.shape[1]], wide[:, q.shape[1]:q.shape[1] + k.shape[1]], wide[:, q.shape[1] + k.shape[1]:] = dev(q), dev(k), dev(v)
        got = ops.unit_norm_rope_kv_write(wide[:, :q.shape[1]], wide[:, q.shape[1]:q.shape[1] + k.shape[1]], wide[:, q.shape[1] + k.shape[1]:],
                                          dev(wq), dev(wk), 1e-5, step.positions, part.frequency_pairs(), dims, part.amplitude,
                                          step.slots[0], cache.k, cache.v, H * maps, G * maps, G, channels, dv, page, torch.float32)
        pos = np.arange(first, first + n)
        want_q = plain.rotate(plain.rms(q.reshape(n, -1, channels), 1e-5) * wq, pos, rot).reshape(n, -1)
        want_k = plain.rotate(plain.rms(k.reshape(n, -1, channels), 1e-5) * wk, pos, rot).reshape(n, -1)
        assert np.abs(got.cpu().numpy() - want_q).max() < 2e-5, first
        slots = step.slots[0].cpu().numpy()
        kc = cache.k.cpu().numpy().reshape(-1, G, page, maps * channels)
        vc = cache.v.cpu().numpy()
        for t in range(n):
            assert np.abs(kc[slots[t] // page, 0, slots[t] % page] - want_k[t]).max() < 2e-5, (first, t)
            assert np.abs(vc[slots[t] // page, 0, slots[t] % page] - v[t]).max() < 1e-6


SHAPES = [  # heads, kv heads, channels per map, value channels, maps, chunk, sink, page
    (4, 2, 32, 16, 2, 24, False, 16), (3, 1, 16, 48, 2, None, False, 8), (4, 2, 16, 32, 1, None, True, 16),
    (2, 2, 48, 80, 2, 40, False, 16), (6, 3, 12, 10, 2, 17, False, 4), (1, 1, 20, 30, 1, 5, True, 3),
    (8, 2, 64, 128, 2, 100, False, 16), (2, 1, 128, 256, 2, 64, False, 16), (2, 1, 128, 128, 1, None, True, 32)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,G,dk,dv,maps,chunk,sink,page", SHAPES)
def test_attention_with_maps_in_portions_and_decoded(dtype, heads, G, dk, dv, maps, chunk, sink, page):
    """Two sequences at once, cut into portions (down to one token, which takes the decoding kernels in bfloat16) across
    pages, tiles and chunks: equal to the plain attention of the whole sequences.  bfloat16 runs the tensor-core kernels
    where the sizes allow and is compared with the plain attention of the rounded inputs."""
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(heads * 1000 + dk)
    lengths = [150, 83]
    lam, scale, eps = 0.55, 1.0 / math.sqrt(dk), 1e-5
    seqs = []
    for n in lengths:
        q, k, v = rng.normal(size=(n, heads * maps * dk)) * 1.5, rng.normal(size=(n, G * maps * dk)) * 1.5, rng.normal(size=(n, G * dv))
        if dtype == torch.bfloat16:
            q, k, v = bf(q), bf(k), bf(v)
        seqs.append((q, k, v, plain_maps(q, k, v, heads, G, dk, dv, maps, scale, lam, chunk, sink, maps == 2, eps, 0.7)))
    cache = Paged(lengths, G, maps * dk, dv, page, dtype, seed=dk)
    cuts = [[70, 1, 1, 2, 39, 1, 36], [1, 1, 30, 17, 2, 1, 31]]
    at = [0, 0]
    tol = 2e-5 if dtype == torch.float32 else 0.02
    for a, b in zip(*cuts):
        step = cache.step([(0, at[0], a), (1, at[1], b)])
        q = np.concatenate([seqs[0][0][at[0]:at[0] + a], seqs[1][0][at[1]:at[1] + b]])
        k = np.concatenate([seqs[0][1][at[0]:at[0] + a], seqs[1][1][at[1]:at[1] + b]])
        v = np.concatenate([seqs[0][2][at[0]:at[0] + a], seqs[1][2][at[1]:at[1] + b]])
        got = write_and_attend(cache, step, q, k, v, heads, dk, maps, ops, chunk=chunk, sink=sink, scale=scale, lam=lam,
                               head_norm=maps == 2, out_scale=0.7, eps=eps)
        want = np.concatenate([seqs[0][3][at[0]:at[0] + a], seqs[1][3][at[1]:at[1] + b]])
        assert np.abs(got - want).max() < tol * max(1.0, np.abs(want).max()), (at, a, b, np.abs(got - want).max())
        at = [at[0] + a, at[1] + b]
    assert at == lengths


@pytest.mark.parametrize("simple", [False, True])
@pytest.mark.parametrize("dk,dv,maps,chunk,page", [(32, 16, 2, 24, 16), (16, 32, 1, 40, 8), (64, 64, 2, 128, 16), (48, 80, 2, 100, 16)])
def test_a_key_that_stands_out_at_every_edge(simple, dk, dv, maps, chunk, page):
    """One key of the sequence carries a large component that every query shares, so a row that may see it puts all its
    weight there and returns its value.  The key sits at position 0, at the first and the last position of a chunk, on both
    sides of page and tile borders, and far back; rows just inside and just outside its chunk are read in a prompt's
    portion and decoded alone.  A row of a later chunk must not see it at all."""
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(dk + chunk)
    heads, G, n = 2, 1, 3 * chunk + 9
    dtype = torch.bfloat16
    places = (0, chunk - 1, chunk, chunk + page - 1, chunk + page, chunk + 63, chunk + 64, 2 * chunk - 1, 2 * chunk + 3)
    for marked in sorted({m for m in places if m < n - 4}):
        q = rng.normal(size=(n, heads * maps * dk)) * 0.1
        k = rng.normal(size=(n, G * maps * dk)) * 0.1
        v = rng.normal(size=(n, G * dv))
        q = q.reshape(n, heads * maps, dk); k = k.reshape(n, G * maps, dk)
        q[:, 0::maps, 0] = 8.0                       # the first map of every head asks for the marked key
        k[marked, 0, 0] = 8.0
        q, k = bf(q.reshape(n, -1)), bf(k.reshape(n, -1))
        v = bf(v)
        want = plain_maps(q, k, v, heads, G, dk, dv, maps, 1.0, 0.0, chunk, False, False, 1e-5, 1.0)
        end = (marked // chunk + 1) * chunk             # the first position that no longer sees the key
        for first_decoded in (end - 2, end + 1):
            cache = Paged([n], G, maps * dk, dv, page, dtype, seed=marked)
            got = [write_and_attend(cache, cache.step([(0, 0, first_decoded)]), q[:first_decoded], k[:first_decoded],
                                    v[:first_decoded], heads, dk, maps, ops, simple=simple, chunk=chunk)]
            for t in range(first_decoded, min(n, end + 3)):
                got.append(write_and_attend(cache, cache.step([(0, t, 1)]), q[t:t + 1], k[t:t + 1], v[t:t + 1], heads, dk, maps,
                                            ops, simple=simple, chunk=chunk))
            got = np.concatenate(got)
            assert np.abs(got - want[:len(got)]).max() < 0.03, (marked, first_decoded)
            inside, outside = got[end - 1].reshape(heads, dv), got[end].reshape(heads, dv)
            assert np.abs(inside - v[marked].reshape(G, dv)[0]).max() < 0.03, (marked, "the last row of the chunk lost the key")
            if end < n:
                assert np.abs(outside - v[marked].reshape(G, dv)[0]).max() > 0.3, (marked, "a row of the next chunk saw the key")


@pytest.mark.parametrize("simple", [False, True])
@pytest.mark.parametrize("dk,dv,sink,page", [(32, 32, True, 16), (64, 16, False, 8)])
def test_a_far_key_among_hundreds_without_chunks(simple, dk, dv, sink, page):
    """No chunks: every earlier position is seen.  One of the first keys of 420 stands out; rows hundreds of positions later
    return its value, in a prompt's portion (several row tiles and key tiles away), in a second portion, and decoded alone
    (several splits away)."""
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(dk)
    heads, G, n = 4, 2, 420
    for marked in (0, 5, 17):
        q, k = rng.normal(size=(n, heads, dk)) * 0.1, rng.normal(size=(n, G, dk)) * 0.1
        v = bf(rng.normal(size=(n, G * dv)))
        q[:, :, 1] = 8.0
        k[marked, :, 1] = 8.0
        q, k = bf(q.reshape(n, -1)), bf(k.reshape(n, -1))
        want = plain_maps(q, k, v, heads, G, dk, dv, 1, 1.0, 0.0, None, sink, False, 1e-5, 1.0)
        cache = Paged([n], G, dk, dv, page, torch.bfloat16, seed=marked)
        got, at = [], 0
        for portion in (300, 110, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1):
            got.append(write_and_attend(cache, cache.step([(0, at, portion)]), q[at:at + portion], k[at:at + portion], v[at:at + portion],
                                        heads, dk, 1, ops, simple=simple, sink=sink))
            at += portion
        got = np.concatenate(got)
        assert at == n and np.abs(got - want).max() < 0.03, marked
        value = v[marked].reshape(G, dv)
        for row in (marked, 299, 300, 409, 410, 419):
            assert np.abs(got[row].reshape(heads, dv) - np.repeat(value, heads // G, axis=0)).max() < 0.03, (marked, row)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_sink_takes_weight_and_carries_no_value(dtype):
    """Scores far below zero: with the sink nearly all weight goes to it and the output nearly vanishes; without it the
    output is the mean of the values.  Scores far above zero: the sink changes nothing."""
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(5)
    heads, G, dk, dv, n, page = 2, 1, 32, 32, 40, 16
    v = bf(rng.normal(size=(n, G * dv)) + 2.0)
    for sign in (-1.0, 1.0):
        q = bf(np.full((n, heads * dk), 1.0))
        k = bf(np.full((n, G * dk), sign * 0.5))
        for portion in (n, 1):
            outs = {}
            for sink in (True, False):
                cache = Paged([n], G, dk, dv, page, dtype)
                if portion == 1:
                    write_and_attend(cache, cache.step([(0, 0, n - 1)]), q[:n - 1], k[:n - 1], v[:n - 1], heads, dk, 1, ops, sink=sink)
                    outs[sink] = write_and_attend(cache, cache.step([(0, n - 1, 1)]), q[n - 1:], k[n - 1:], v[n - 1:], heads, dk, 1, ops, sink=sink)[-1]
                else:
                    outs[sink] = write_and_attend(cache, cache.step([(0, 0, n)]), q, k, v, heads, dk, 1, ops, sink=sink)[-1]
            mean = np.tile(v.mean(0), heads)
            assert np.abs(outs[False] - mean).max() < 0.02
            if sign < 0:
                assert np.abs(outs[True]).max() < 1e-4          # 40 e^-16 against the sink's 1
            else:
                assert np.abs(outs[True] - mean).max() < 0.02    # the sink's 1 against 40 e^16


@pytest.mark.parametrize("rows,width,parts,inner", [(5, 64, 1, False), (70, 100, 3, False), (9, 256, 2, True), (300, 80, 2, True), (3, 8192, 2, True)])
def test_normalised_summand_and_the_next_norm_in_one_kernel(rows, width, parts, inner):
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(rows)
    eps = 1e-5
    x = rng.normal(size=(rows, width)) * 3
    p = rng.normal(size=(parts, rows, width)) * np.array([1.0, 30.0, 0.01])[:parts, None, None]
    wi, wb, w = rng.normal(size=(parts, width)), rng.normal(size=width), rng.normal(size=width)
    y = 0.5 * sum(plain.rms(p[i], eps) * wi[i] for i in range(parts)) if inner else p.sum(0)
    want_x = x + plain.rms(y, eps) * wb
    want_h = plain.rms(want_x, eps) * w
    resid = dev(x)
    out = torch.empty((rows, width), device=DEV)
    ops.add_normed_rmsnorm(resid, dev(p), dev(wi) if inner else None, 0.5, dev(wb), dev(w), eps, out)
    assert np.abs(resid.cpu().numpy() - want_x).max() < 1e-4 and np.abs(out.cpu().numpy() - want_h).max() < 1e-4
    pick = np.array([rows - 1, 0, rows // 2], dtype=np.int32)               # a gather leaves the stream as it is
    resid = dev(x)
    out = torch.empty((3, width), device=DEV)
    ops.add_normed_rmsnorm(resid, dev(p), dev(wi) if inner else None, 0.5, dev(wb), dev(w), eps, out, rows=dev(pick, torch.int32))
    assert np.abs(out.cpu().numpy() - want_h[pick]).max() < 1e-4 and np.array_equal(resid.cpu().numpy(), x.astype(np.float32))
    resid = dev(x)                                                           # no reader: the stream is only updated
    ops.add_normed_rmsnorm(resid, dev(p), dev(wi) if inner else None, 0.5, dev(wb), None, eps, None)
    assert np.abs(resid.cpu().numpy() - want_x).max() < 1e-4


@pytest.mark.parametrize("rows", [3, 40, 300])
@pytest.mark.parametrize("limit", [0.25, 1.5, 7.0, 1.3])
def test_clamped_gate(rows, limit):
    """The gate capped from above, the other factor from both sides, g sigmoid(1.702 g) (u + 1): in the products' epilogues
    (every kernel family by its row count) and in the unfused kernel."""
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(rows)
    K, I = 64, 48
    x, wg, wu = bf(rng.normal(size=(rows, K))), bf(rng.normal(size=(I, K)) * 0.4), bf(rng.normal(size=(I, K)) * 0.4)
    g, u = np.minimum(x @ wg.T, limit), np.clip(x @ wu.T, -limit, limit)
    want = g * plain.sigmoid(1.702 * g) * (u + 1.0)
    assert (x @ wg.T > limit).any() and (np.abs(x @ wu.T) > limit).any()
    w = np.stack([wg, wu], axis=1).reshape(2 * I, K)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 0.02)):
        got = ops.gated_linear(dev(x, dtype), dev(w, dtype), "swish_clamped", param=limit).float().cpu().numpy()
        assert np.abs(got - want).max() < tol * max(1.0, np.abs(want).max()), (dtype, np.abs(got - want).max())


@pytest.mark.parametrize("heads,groups,dk,dv", [(4, 2, 16, 24), (1, 1, 40, 64), (3, 1, 20, 36), (2, 1, 128, 128), (2, 2, 64, 200)])
def test_delta_rule_with_one_decay_per_head_and_a_silu_gate(heads, groups, dk, dv):
    """Two sequences in portions down to one token, in slots 2 and 0 of a pool full of noise: the recurrence, the norm
    per head, its weight and the gate equal the plain recurrence of the whole sequences."""
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(dk)
    lengths, eps = [37, 20], 1e-5
    rate_log, bias, weight = rng.normal(size=heads) * 0.5, rng.normal(size=heads), rng.normal(size=dv) + 1
    seqs = []
    for n in lengths:
        q, k, v = rng.normal(size=(n, groups, dk)), rng.normal(size=(n, groups, dk)), rng.normal(size=(n, heads, dv))
        b, a, g = rng.normal(size=(n, heads)), rng.normal(size=(n, heads)), rng.normal(size=(n, heads, dv))
        unit = lambda x: x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + 1e-6)
        decay = np.exp(-np.exp(rate_log) * plain.softplus(a + bias))
        rep = heads // groups
        o = plain.gated_delta_rule(np.repeat(unit(q) * dk ** -0.5, rep, 1), np.repeat(unit(k), rep, 1), v, plain.sigmoid(b), decay)
        seqs.append((q, k, v, b, a, g, (plain.rms(o, eps) * weight * plain.silu(g)).reshape(n, heads * dv)))
    state = torch.randn((4, heads * dk * dv + 5), device=DEV)
    view = state[:, 5:]
    view[2].zero_(); view[0].zero_()
    cuts = [[1, 9, 1, 2, 24], [5, 1, 1, 12, 1]]
    at = [0, 0]
    for a_n, b_n in zip(*cuts):
        cu = np.array([0, a_n, a_n + b_n], dtype=np.int32)
        step = types.SimpleNamespace(num_requests=2, cu_q=dev(cu, torch.int32), state_slots=dev([2, 0], torch.int32))
        cat = lambda i: np.concatenate([seqs[0][i][at[0]:at[0] + a_n].reshape(a_n, -1), seqs[1][i][at[1]:at[1] + b_n].reshape(b_n, -1)])
        qkv = dev(np.concatenate([cat(0), cat(1), cat(2)], axis=1))
        nq = groups * dk
        out = torch.empty((a_n + b_n, heads * dv), device=DEV)
        ops.gated_delta_scan(qkv[:, :nq], qkv[:, nq:2 * nq], qkv[:, 2 * nq:], dev(cat(3)), dev(cat(4)), dev(bias), dev(rate_log), view,
                             step, heads, groups, dk, dv, out, dev(weight), dev(cat(5)), eps, decay_per_channel=False,
                             gate_activation="silu")
        want = np.concatenate([seqs[0][6][at[0]:at[0] + a_n], seqs[1][6][at[1]:at[1] + b_n]])
        assert np.abs(out.cpu().numpy() - want).max() < 2e-4 * max(1.0, np.abs(want).max()), (at, np.abs(out.cpu().numpy() - want).max())
        at = [at[0] + a_n, at[1] + b_n]


# ------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(name, dtype, folders, models):
    for i, n in enumerate([1, 2, 23, 97]):
        seq = tc.prompt(30 + i, n, vocab(name))
        r = tc.noisy_replay(folders[name], dtype, 128, models(name, dtype))
        r.step([("r", seq, list(range(n)))], end=["r"])
        tc.check_rows(r.rows, folders[name], {"r": seq}, dtype, f"whole {n}")


def test_layer_outputs_equal_the_plain_layers(folders, models):
    for name in NAMES:
        seq = tc.prompt(3, 29, vocab(name))
        config, w = tc.read_model(folders[name])
        want = []
        plain.forward(config, w, seq, want)
        r = tc.noisy_replay(folders[name], "float32", 64, models(name, "float32"), layer_outputs=True)
        r.step([("r", seq, [28])])
        assert len(want) == len(models(name, "float32").spec.schedule)
        for t in range(29):
            got = r.layers[("r", t)]
            for i in range(len(want)):
                assert np.abs(got[i] - want[i][t]).max() <= 2e-4 * max(1.0, np.abs(want[i][t]).max()), (name, i, t)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_token_by_token(name, dtype, folders, models):
    """The last 50 tokens one by one: several chunks of the tiny models begin and end among decoded tokens."""
    n = 120
    seq = tc.prompt(41, n, vocab(name))
    r = tc.noisy_replay(folders[name], dtype, 128, models(name, dtype))
    r.step([("r", seq[:n - 50], list(range(0, n - 50, 3)))])
    for t in range(n - 50, n):
        r.step([("r", [seq[t]], [0])])
    tc.check_rows(r.rows, folders[name], {"r": seq}, dtype, "tail")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_every_token_decoded(name, dtype, folders, models):
    n = 70 if dtype == "bfloat16" else 260
    seq = tc.prompt(42, n, vocab(name))
    r = tc.noisy_replay(folders[name], dtype, 272, models(name, dtype))
    for t in range(n):
        r.step([("r", [seq[t]], [0] if t % 4 == 0 or t > n - 5 else [])])
    tc.check_rows(r.rows, folders[name], {"r": seq}, dtype, "decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_down_to_two_tokens(name, dtype, folders, models):
    portions = [7, 2, 16, 3, 2, 33, 1, 15, 2, 17, 2, 5, 1, 1, 2, 40]
    n = sum(portions)
    seq = tc.prompt(43, n, vocab(name))
    r = tc.noisy_replay(folders[name], dtype, 160, models(name, dtype), page_size=8)
    o = 0
    for p in portions:
        r.step([("r", seq[o:o + p], list(range(p)))])
        o += p
    tc.check_rows(r.rows, folders[name], {"r": seq}, dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(name, dtype, folders, models):
    """Five requests over three state slots and a pool of 14 pages of 16: portions of some beside single tokens of others;
    a request that ends gives its pages and its slot to the next, which must not see what they held."""
    V = vocab(name)
    seqs = {f"s{i}": tc.prompt(50 + i, n, V) for i, n in enumerate([61, 9, 130, 33, 47])}
    r = tc.noisy_replay(folders[name], dtype, 14 * 16, models(name, dtype), max_requests=3)
    at = {k: 0 for k in seqs}

    def take(rid, n):
        toks = seqs[rid][at[rid]:at[rid] + n]
        want = [i for i in range(len(toks)) if (at[rid] + i) % 3 == 0 or at[rid] + i == len(seqs[rid]) - 1]
        at[rid] += len(toks)
        return (rid, toks, want)

    def done(*rids):
        return [x for x in rids if at[x] == len(seqs[x])]

    r.step([take("s0", 20), take("s1", 2)])
    r.step([take("s0", 1), take("s1", 1), take("s2", 50)])
    r.step([take("s0", 40), take("s1", 6), take("s2", 1)], end=["s0", "s1"])           # s0 and s1 end: slots and pages go back
    r.step([take("s2", 1), take("s3", 33)], end=["s3"])                                   # s3 takes a used slot and used pages
    r.step([take("s4", 2), take("s2", 30)])
    while at["s2"] < 130 or at["s4"] < 47:
        batch = [take(x, 1 if x == "s2" else 5) for x in ("s2", "s4") if at[x] < len(seqs[x])]
        r.step(batch, end=done(*[b[0] for b in batch]))
    assert all(at[k] == len(seqs[k]) for k in seqs)
    tc.check_rows(r.rows, folders[name], seqs, dtype, "mixed")
    assert len(r.cache.requests) == 0 and r.cache.available_pages() == [14] * len(r.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
def test_batched_rows_equal_the_rows_of_each_request_alone(dtype, folders, models):
    """What a request's rows are does not depend on what else is in the batch, nor on pages and slots (float32: to the bit)."""
    name = "T1"
    a, b = tc.prompt(60, 45, vocab(name)), tc.prompt(61, 18, vocab(name))
    alone = tc.noisy_replay(folders[name], dtype, 128, models(name, dtype))
    alone.step([("a", a[:30], list(range(30)))]); alone.step([("a", a[30:], list(range(15)))])
    both = tc.noisy_replay(folders[name], dtype, 128, models(name, dtype))
    both.step([("b", b[:10], [9]), ("a", a[:30], list(range(30)))])
    both.step([("a", a[30:], list(range(15))), ("b", b[10:], [7])])
    for p in range(45):
        assert np.array_equal(alone.rows[("a", p)], both.rows[("a", p)]) or dtype == "bfloat16", p
        assert np.abs(alone.rows[("a", p)] - both.rows[("a", p)]).max() <= (0 if dtype == "float32" else 0.05 * np.std(alone.rows[("a", p)]))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_few_wanted_rows_take_the_last_layers_shortcut(name, dtype, folders, models):
    """Steps that want few rows (or none) run the last layer's attention, feed-forward and norms for those rows only (T1:
    a last layer that reads another layer's keys and values; T2, T3: one that writes its own): the logits equal the plain
    implementation's, the cache that later steps read is complete, and switching the shortcut off changes nothing beyond
    rounding."""
    n = 131
    seq, other = tc.prompt(33, n, vocab(name)), tc.prompt(34, 40, vocab(name))
    runs = {}
    for shortcut in (True, False):
        r = tc.noisy_replay(folders[name], dtype, 256, models(name, dtype))
        r.runner.tail_shortcut = shortcut
        r.step([("r", seq[:30], [])])                                   # nothing wanted
        r.step([("r", seq[30:60], [29, 3]), ("o", other[:20], [19])])    # few rows, out of order, two requests
        r.step([("r", seq[60:n - 5], [0]), ("o", other[20:], [])])
        r.step([("r", seq[n - 5:], list(range(5)))])                     # everything wanted: no shortcut
        assert set(k for k in r.rows if k[0] == "r") == {("r", p) for p in [59, 33, 60] + list(range(n - 5, n))}
        tc.check_rows(r.rows, folders[name], {"r": seq, "o": other}, dtype, f"shortcut {shortcut}")
        runs[shortcut] = r.rows
    assert models(name, dtype).layers[-1].supports_tail
    for key, row in runs[True].items():
        d = np.abs(row - runs[False][key]).max()
        assert d <= (1e-4 if dtype == "float32" else 0.08 * np.std(row)), (key, d)


@pytest.mark.parametrize("dtype", DTYPES)
def test_tensor_core_attention_equals_the_float32_arithmetic_one_in_a_model(dtype, folders, models):
    """The same steps with the tensor-core kernels switched off: rows agree within rounding (bfloat16), and float32
    never takes them."""
    from coheryn_ai_studio_b200 import ops
    name = "T1"
    seq = tc.prompt(62, 90, vocab(name))
    rows = {}
    for on in (True, False):
        ops.set_maps_tc(on)
        try:
            r = tc.noisy_replay(folders[name], dtype, 128, models(name, dtype))
            r.step([("r", seq[:61], list(range(0, 61, 2)))])
            for t in range(61, 90):
                r.step([("r", [seq[t]], [0])])
            rows[on] = r.rows
        finally:
            ops.set_maps_tc(True)
    for key in rows[True]:
        d = np.abs(rows[True][key] - rows[False][key]).max()
        assert d <= (0 if dtype == "float32" else 0.05 * np.std(rows[False][key])), (key, d)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["T1", "T2"])
def test_greedy_generation_through_the_engine(name, dtype, folders):
    """The Python entry point with its scheduler, continuous batching, portions of 16 tokens and decode steps replayed
    from CUDA graphs: every generated token is the plain implementation's first maximum given the tokens before it (in
    bfloat16: or a near tie)."""
    from coheryn_ai_studio_b200.engine import Engine
    eng = Engine.from_folder(folders[name], dtype, context=128, max_num_seqs=3, max_num_batched_tokens=16, page_size=8)
    prompts = [tc.prompt(70 + i, n, vocab(name)) for i, n in enumerate((3, 29, 50, 1))]
    res = eng.generate(prompts, max_tokens=12)
    for p, out in zip(prompts, res):
        ids = list(p)
        assert out.completion_tokens == 12 and out.finish_reason == "length"
        for tok in out.token_ids:
            ref = tc.plain_rows(folders[name], ids)[-1]
            best = int(np.argmax(ref))
            if tok != best:
                gap = float(ref[best] - ref[tok]) / float(np.std(ref))
                assert gap <= (1e-3 if dtype == "float32" else 0.4), (name, len(ids), tok, best, gap)
            ids.append(tok)
    eng.cache.check()
    assert len(eng.cache.requests) == 0


def test_trace_program_replays_a_schedule(folders, tmp_path):
    """bin/trace_run on a folder of this design: portions, a second request, an ended request, a step that wants nothing."""
    import json, os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "T2"
    a, b = tc.prompt(80, 40, vocab(name)), tc.prompt(81, 12, vocab(name))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:25], "want": [0, 24]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[25:27], "want": []}, {"id": "b", "tokens": b, "want": [11]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[27:], "want": [12]}], "end": ["a"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders[name], "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    V = vocab(name)
    got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, V)
    got1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, V)
    got2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(1, V)
    rows = {("a", 0): got0[0], ("a", 24): got0[1], ("b", 11): got1[0], ("a", 39): got2[0]}
    tc.check_rows(rows, folders[name], {"a": a, "b": b}, "float32", "trace")


def test_command_line_runs_and_traces_the_design(folders):
    """`coheryn run` (greedy tokens) and `coheryn trace` (every layer's output and the logits per position) on a folder of
    this design, and the Python entry point, against the plain implementation."""
    import json, os, subprocess, sys
    from coheryn_ai_studio_b200 import api
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "T1"
    p = tc.prompt(85, 27, vocab(name))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "coheryn"), "run", folders[name], "--tokens", ",".join(map(str, p)),
                        "--max-tokens", "5", "--context", "64", "--dtype", "float32", "--stream"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [int(t) for t in r.stdout.split()]
    ids = list(p)
    for tok in got:
        assert tok == int(np.argmax(tc.plain_rows(folders[name], ids)[-1]))
        ids.append(tok)
    assert api.generate(folders[name], [p], max_tokens=5, context=64, dtype="float32")[0]["token_ids"] == got
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "coheryn"), "trace", folders[name], "--tokens", ",".join(map(str, p)),
                        "--context", "64", "--dtype", "float32"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    config, w = tc.read_model(folders[name])
    layers = []
    ref = plain.forward(config, w, p, layers)
    assert len(lines) == len(p) * (len(layers) + 1)
    for l in lines:
        want = ref[l["position"]] if l["name"] == "logits" else layers[int(l["name"].split(".")[1])][l["position"]]
        assert np.abs(np.asarray(l["values"], np.float64) - want).max() <= 2e-4 * max(1.0, float(np.abs(want).max())), l["name"]
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "coheryn"), "models", "inspect", folders[name]], capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0 and "Tutunex" in r.stdout, r.stderr[-2000:]


def test_zz_report():
    print(f"\nTutunex rows against the plain implementation: float32 largest |d| = {tc.WORST['float32']:.2e}; "
          f"bfloat16 largest distance = {tc.WORST['bfloat16']:.2f} of the bound")
