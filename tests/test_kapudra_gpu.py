"""The Kapudra decoder on the GPU against the plain implementation (``plain_kapudra.py``): each mechanism's kernel
alone, then whole models through the step function, the cache and the scheduler, in float32 and in bfloat16."""
import types

import numpy as np
import pytest
import torch

import kapudra_cases as kc
import plain_kapudra as plain

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = ["K1", "K2", "K3", "K4"]
DEV = "cuda:0"


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("kapudra")
    return {n: kc.make_folder(base, n) for n in NAMES}


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
    return kc.CASES[name][0]["vocab"]


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=dtype).to(DEV)


def step_of(lengths, slots=None, starts=None):
    """What the kernels read of a step: runs of ``lengths`` tokens, one per request."""
    cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    req = np.repeat(np.arange(len(lengths)), lengths).astype(np.int32)
    starts = starts or [0] * len(lengths)
    pos = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lengths)]).astype(np.int32)
    slots = list(range(len(lengths))) if slots is None else slots
    return types.SimpleNamespace(num_requests=len(lengths), num_tokens=int(cu[-1]), cu_q=dev(cu, torch.int32),
                                 token_req=dev(req, torch.int32), positions=dev(pos, torch.int32),
                                 state_slots=dev(slots, torch.int32))


# ------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_convolution_in_portions(taps):
    """Two sequences cut into portions of 1 to 9 tokens (shorter than the taps reach back, too), in slots 3 and 1 of a
    pool full of noise that is zeroed for them: equal to the convolution of the whole sequences."""
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(taps)
    C, n = 37, 31
    w = rng.normal(size=(C, taps))
    xs = [rng.normal(size=(n, C)), rng.normal(size=(n - 6, C))]
    want = [plain.silu(plain.causal_short_conv(x, w)) for x in xs]
    state = torch.randn((5, 11 + (taps - 1) * C), device=DEV)
    view = state[:, 11:]
    view[3].zero_(); view[1].zero_()
    cuts = [[1, 1, 2, 9, 1, 3, 5, 2, 7], [2, 1, 1, 1, 8, 3, 4, 4, 1]]
    at = [0, 0]
    for a, b in zip(*cuts):
        step = step_of([a, b], slots=[3, 1])
        x = np.concatenate([xs[0][at[0]:at[0] + a], xs[1][at[1]:at[1] + b]])
        wide = torch.zeros((a + b, C + 5), device=DEV)          # the input is a column slice of a wider buffer
        wide[:, 2:2 + C] = dev(x)
        y = ops.short_conv_silu(wide[:, 2:2 + C], dev(w), view, step).cpu().numpy()
        assert np.abs(y[:a] - want[0][at[0]:at[0] + a]).max() < 1e-5
        assert np.abs(y[a:] - want[1][at[1]:at[1] + b]).max() < 1e-5
        at = [at[0] + a, at[1] + b]
    assert at == [n, n - 6]


def _norm_gate(o, weight, gate, eps):
    return plain.rms(o, eps) * weight * plain.sigmoid(gate)


@pytest.mark.parametrize("heads,groups,dk,dv", [(4, 2, 16, 24), (1, 1, 40, 64), (3, 3, 8, 130), (2, 1, 128, 32), (2, 2, 20, 30), (1, 1, 200, 256)])
def test_gated_delta_rule_kernel(heads, groups, dk, dv):
    """Three requests in one batch, cut into portions, against the recurrence written token by token."""
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(dk + dv)
    lens, eps = [37, 5, 18], 1e-5
    data = []
    for n in lens:
        d = dict(q=rng.normal(size=(n, groups * dk)), k=rng.normal(size=(n, groups * dk)), v=rng.normal(size=(n, heads * dv)),
                 beta=rng.normal(size=(n, heads)), step=rng.normal(size=(n, heads * dk)), gate=rng.normal(size=(n, heads * dv)))
        data.append(d)
    bias, rate_log, weight = rng.normal(size=heads * dk), rng.normal(size=heads) * 0.5, rng.normal(size=dv)
    want = []
    for d, n in zip(data, lens):
        q = d["q"].reshape(n, groups, dk); k = d["k"].reshape(n, groups, dk)
        q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dk ** -0.5
        k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
        decay = np.exp(-np.exp(rate_log)[None, :, None] * plain.softplus(d["step"] + bias).reshape(n, heads, dk))
        per = heads // groups
        o = np.stack([plain.gated_delta_rule(q[:, h // per], k[:, h // per], d["v"].reshape(n, heads, dv)[:, h],
                                             plain.sigmoid(d["beta"][:, h]), decay[:, h]) for h in range(heads)], axis=1)
        want.append((_norm_gate(o, weight, d["gate"].reshape(n, heads, dv), eps) * 1.7).reshape(n, heads * dv))
    state = torch.randn((4, heads * dk * dv + 3), device=DEV)
    view = state[:, :heads * dk * dv]
    view.zero_()
    cuts = [[17, 1, 2, 17], [1, 1, 2, 1], [2, 16, 0, 0]]
    at = [0, 0, 0]
    for s in range(4):
        parts = [(r, cuts[r][s]) for r in range(3) if cuts[r][s]]
        step = step_of([n for _, n in parts], slots=[[2, 0, 3][r] for r, _ in parts])
        cat = lambda key: dev(np.concatenate([data[r][key][at[r]:at[r] + n] for r, n in parts]))
        qkv = torch.cat([cat("q"), cat("k"), cat("v")], dim=1)
        G = groups * dk
        out = torch.empty((step.num_tokens, heads * dv), device=DEV)
        ops.gated_delta_scan(qkv[:, :G], qkv[:, G:2 * G], qkv[:, 2 * G:], cat("beta"), cat("step"), dev(bias), dev(rate_log), view, step,
                             heads, groups, dk, dv, out, dev(weight), cat("gate"), eps, out_scale=1.7)
        got, o = out.cpu().numpy(), 0
        for r, n in parts:
            ref = want[r][at[r]:at[r] + n]
            assert np.abs(got[o:o + n] - ref).max() <= 2e-4 * max(1.0, np.abs(ref).max()), (s, r)
            o += n; at[r] += n
    assert at == lens


@pytest.mark.parametrize("heads,dk,dv,cap", [(2, 24, 40, 8.0), (1, 64, 16, 15.0), (3, 16, 200, 4.0), (2, 192, 32, 10.0), (2, 20, 30, 9.0), (1, 128, 256, 12.0)])
def test_matrix_memory_kernel(heads, dk, dv, cap):
    """Two requests in portions against the token-by-token recurrence; the second request's forget gate is held open and
    one early token's input gate stands out, so that what the rows 300 tokens later read is that token's value: a state
    lost at a portion's edge would change them altogether."""
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(dk)
    lens, eps = [29, 330], 1e-6
    data = []
    for r, n in enumerate(lens):
        d = dict(q=rng.normal(size=(n, heads * dk)), k=rng.normal(size=(n, heads * dk)), v=rng.normal(size=(n, heads * dv)),
                 gi=rng.normal(size=(n, heads)) * 2, gf=rng.normal(size=(n, heads)) * 2, gate=rng.normal(size=(n, heads * dv)))
        if r == 1:
            d["gf"] += 30.0; d["gi"] -= 6.0; d["gi"][7] += 14.0
        data.append(d)
    bi, bf, weight = rng.normal(size=heads), rng.normal(size=heads), rng.normal(size=heads * dv)
    want = []
    for d, n in zip(data, lens):
        li = cap * np.tanh((d["gi"] + bi) / cap)
        lf = plain.log_sigmoid(cap * np.tanh((d["gf"] + bf) / cap))
        o = np.stack([plain.matrix_memory(d["q"].reshape(n, heads, dk)[:, h] * dk ** -0.5, d["k"].reshape(n, heads, dk)[:, h],
                                          d["v"].reshape(n, heads, dv)[:, h], li[:, h], lf[:, h]) for h in range(heads)], axis=1)
        want.append(plain.rms(o, eps).reshape(n, heads * dv) * weight * plain.sigmoid(d["gate"]))
    size = heads * (dk * dv + dk + 1)
    state = torch.randn((3, size), device=DEV)
    state[0].zero_(); state[2].zero_()
    cuts = [[9, 1, 2, 17, 0], [100, 1, 2, 129, 98]]
    at = [0, 0]
    for s in range(5):
        parts = [(r, cuts[r][s]) for r in range(2) if cuts[r][s]]
        step = step_of([n for _, n in parts], slots=[[2, 0][r] for r, _ in parts])
        cat = lambda key: dev(np.concatenate([data[r][key][at[r]:at[r] + n] for r, n in parts]))
        qkv = torch.cat([cat("q"), cat("k"), cat("v")], dim=1)
        gates = torch.cat([cat("gi"), cat("gf")], dim=1)
        out = torch.empty((step.num_tokens, heads * dv), device=DEV)
        ops.matrix_memory_scan(qkv[:, :heads * dk], qkv[:, heads * dk:2 * heads * dk], qkv[:, 2 * heads * dk:], gates[:, :heads],
                               gates[:, heads:], dev(bi), dev(bf), cap, state, step, heads, dk, dv, out, dev(weight), cat("gate"), eps)
        got, o = out.cpu().numpy(), 0
        for r, n in parts:
            ref = want[r][at[r]:at[r] + n]
            # (a float32 recurrence is itself up to 5e-4 from float64 here, where a row's output nearly cancels before its norm)
            assert np.abs(got[o:o + n] - ref).max() <= 1e-3 * max(1.0, np.abs(ref).max()), (s, r)
            o += n; at[r] += n
    assert at == lens
    # the far token is what the late rows of the second request hold: without it they are something else
    d = {k: v.copy() for k, v in data[1].items()}
    d["v"][7] = 0.0
    n = lens[1]
    li = cap * np.tanh((d["gi"] + bi) / cap); lf = plain.log_sigmoid(cap * np.tanh((d["gf"] + bf) / cap))
    o = plain.matrix_memory(d["q"].reshape(n, heads, dk)[:, 0] * dk ** -0.5, d["k"].reshape(n, heads, dk)[:, 0],
                            d["v"].reshape(n, heads, dv)[:, 0], li[:, 0], lf[:, 0])
    other = plain.rms(o, eps) * weight[:dv] * plain.sigmoid(d["gate"][:, :dv])
    assert np.abs(other[-1] - want[1][-1, :dv]).max() > 0.05


@pytest.mark.parametrize("heads,dk,dv", [(2, 24, 200), (1, 128, 256), (3, 64, 72)])
def test_scans_of_long_portions_split_a_heads_columns_over_ctas(heads, dk, dv):
    """One request whose long portions (64 tokens and more) run as several CTAs per head, with norm and gate in a kernel of
    their own (the delta rule from prepared inputs, staged asynchronously), and whose short portions run the one-CTA kernels:
    both against the token-by-token recurrences, continuing each other's state."""
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(dv)
    cuts, eps, cap, groups = [130, 1, 70, 2, 64, 33], 1e-6, 9.0, 1
    n = sum(cuts)
    f = lambda *shape: rng.normal(size=shape)
    # the delta rule
    d = dict(q=f(n, groups * dk), k=f(n, groups * dk), v=f(n, heads * dv), beta=f(n, heads), step=f(n, heads * dk), gate=f(n, heads * dv))
    bias, rate_log, weight = f(heads * dk), f(heads) * 0.5, f(dv)
    q = d["q"].reshape(n, groups, dk); k = d["k"].reshape(n, groups, dk)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    decay = np.exp(-np.exp(rate_log)[None, :, None] * plain.softplus(d["step"] + bias).reshape(n, heads, dk))
    o = np.stack([plain.gated_delta_rule(q[:, 0], k[:, 0], d["v"].reshape(n, heads, dv)[:, h], plain.sigmoid(d["beta"][:, h]), decay[:, h])
                  for h in range(heads)], axis=1)
    want = _norm_gate(o, weight, d["gate"].reshape(n, heads, dv), eps).reshape(n, heads * dv)
    state = torch.zeros((2, heads * dk * dv), device=DEV)
    at = 0
    for m in cuts:
        step = step_of([m], slots=[1])
        cat = lambda key: dev(d[key][at:at + m])
        qkv = torch.cat([cat("q"), cat("k"), cat("v")], dim=1)
        out = torch.empty((m, heads * dv), device=DEV)
        ops.gated_delta_scan(qkv[:, :groups * dk], qkv[:, groups * dk:2 * groups * dk], qkv[:, 2 * groups * dk:], cat("beta"), cat("step"),
                             dev(bias), dev(rate_log), state, step, heads, groups, dk, dv, out, dev(weight), cat("gate"), eps)
        ref = want[at:at + m]
        assert np.abs(out.cpu().numpy() - ref).max() <= 3e-4 * max(1.0, np.abs(ref).max()), ("delta", at, m)
        at += m
    # the matrix memory
    d = dict(q=f(n, heads * dk), k=f(n, heads * dk), v=f(n, heads * dv), gi=f(n, heads) * 2, gf=f(n, heads) * 2 + 3.0, gate=f(n, heads * dv))
    bi, bf, weight = f(heads), f(heads), f(heads * dv)
    li = cap * np.tanh((d["gi"] + bi) / cap); lf = plain.log_sigmoid(cap * np.tanh((d["gf"] + bf) / cap))
    o = np.stack([plain.matrix_memory(d["q"].reshape(n, heads, dk)[:, h] * dk ** -0.5, d["k"].reshape(n, heads, dk)[:, h],
                                      d["v"].reshape(n, heads, dv)[:, h], li[:, h], lf[:, h]) for h in range(heads)], axis=1)
    want = plain.rms(o, eps).reshape(n, heads * dv) * weight * plain.sigmoid(d["gate"])
    state = torch.zeros((2, heads * (dk * dv + dk + 1)), device=DEV)
    at = 0
    for m in cuts:
        step = step_of([m], slots=[1])
        cat = lambda key: dev(d[key][at:at + m])
        qkv = torch.cat([cat("q"), cat("k"), cat("v")], dim=1)
        gates = torch.cat([cat("gi"), cat("gf")], dim=1)
        out = torch.empty((m, heads * dv), device=DEV)
        ops.matrix_memory_scan(qkv[:, :heads * dk], qkv[:, heads * dk:2 * heads * dk], qkv[:, 2 * heads * dk:], gates[:, :heads], gates[:, heads:],
                               dev(bi), dev(bf), cap, state, step, heads, dk, dv, out, dev(weight), cat("gate"), eps)
        ref = want[at:at + m]
        assert np.abs(out.cpu().numpy() - ref).max() <= 1e-3 * max(1.0, np.abs(ref).max()), ("memory", at, m)
        at += m


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dk,dv,window,page", [(16, 32, 24, 16), (32, 32, 5, 4), (64, 64, 72, 16), (48, 80, 40, 8), (128, 64, 130, 16)])
def test_distance_bias_attention_window_edges(dtype, dk, dv, window, page):
    """One key is made to stand out (its key and every query are aligned and long), so a row's output is that key's value
    as long as the key lies inside the window and something else from the next row on.  The key sits at position 0, at
    a page's last and first slot, and in the middle; the rows come as one prompt, and again one by one (decoding)."""
    from coheryn_ai_studio_b200 import ops
    H, G, n = 4, 2, window + 40
    rng = np.random.default_rng(dk + window)
    tol = 2e-4 if dtype == torch.float32 else 3e-2
    slopes = np.array([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)])
    for marked in (0, page - 1, page, 2 * page + 1):
        q = rng.normal(size=(n, H, dk)) * 0.3
        k = rng.normal(size=(n, G, dk)) * 0.3
        v = rng.normal(size=(n, G, dv))
        axis = rng.normal(size=dk); axis /= np.linalg.norm(axis)
        k[marked] += 6.0 * axis
        q += 6.0 * axis
        qd, kd, vd = (torch.as_tensor(a).to(dtype).to(DEV) for a in (q, k, v * 0.6))    # the output's constant rides on the values
        q64, k64, v64 = (t.double().cpu().numpy() for t in (qd, kd, vd))
        want = plain.biased_window_attention(q64, k64, v64, H, G, 0.9, window)
        # the marked key holds nearly all the weight while it is seen, and none afterwards
        inside, outside = marked + window - 1, marked + window
        last = H - 1                                 # the head with the smallest slope: distance costs it least
        assert np.abs(want[inside, last] - v64[marked, G - 1]).max() < 0.2
        assert np.abs(want[outside, last] - v64[marked, G - 1]).max() > 0.3
        pages = -(-n // page)
        table = rng.permutation(pages + 3)[:pages].astype(np.int32)          # pages in no order
        kc_, vc_ = (torch.randn((pages + 3, G, page, d), device=DEV).to(dtype) * 5 for d in (dk, dv))
        for t in range(n):
            kc_[table[t // page], :, t % page] = kd[t]
            vc_[table[t // page], :, t % page] = vd[t]
        tables = dev(table[None, :], torch.int32)
        for simple in (False, True):          # the tensor-core kernels where they take the shape, and the plain kernel
            for cut in ([n], [n - 35] + [1] * 35, [3, 2, n - 5]):
                got, at = [], 0
                for m in cut:
                    step = step_of([m], starts=[at])
                    step.block_tables, step.q_lens, step.kv_lens_host = [tables], [m], [at + m]
                    step.kv_lens, step.max_q_len, step.max_kv_len = dev([at + m], torch.int32), m, at + m
                    step.prior_positions_settled = True
                    out = torch.empty((m, H * dv), dtype=dtype, device=DEV)
                    ops.attention_biased(qd[at:at + m].reshape(m, H * dk).contiguous(), out, kc_, vc_, step, 0, H, G, dk, dv, page,
                                         window, 0.9, dev(slopes), force_simple=simple)
                    got.append(out.float().cpu().numpy()); at += m
                got = np.concatenate(got).reshape(n, H, dv)
                assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max()), (marked, cut[:2], simple)


def test_whole_projection_norm_and_cache_write():
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(5)
    H, G, dk, dv, page, T = 3, 1, 24, 40, 8, 11
    q, k, v = rng.normal(size=(T, H * dk)), rng.normal(size=(T, G * dk)), rng.normal(size=(T, G * dv))
    wq, wk = rng.normal(size=H * dk), rng.normal(size=G * dk)
    buf = dev(np.concatenate([q, k, v], axis=1))
    slots = rng.permutation(5 * page)[:T].astype(np.int32)
    kc_, vc_ = torch.zeros((5, G, page, dk), device=DEV), torch.zeros((5, G, page, dv), device=DEV)
    got = ops.qk_norm_kv_write(buf[:, :H * dk], buf[:, H * dk:H * dk + G * dk], buf[:, H * dk + G * dk:], dev(wq), dev(wk), 1e-5,
                               dev(slots, torch.int32), kc_, vc_, H, G, dk, dv, page, torch.float32)
    assert np.abs(got.cpu().numpy() - plain.rms(q, 1e-5) * wq).max() < 1e-5
    kn = plain.rms(k, 1e-5) * wk
    for t, s in enumerate(slots):
        assert np.abs(kc_[s // page, :, s % page].cpu().numpy().reshape(-1) - kn[t]).max() < 1e-5
        assert np.abs(vc_[s // page, :, s % page].cpu().numpy().reshape(-1) - v[t]).max() < 1e-6


@pytest.mark.parametrize("rows", [3, 40, 300])
def test_tanh_gelu_gate_and_logit_cap(rows):
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(rows)
    K, I = 64, 88
    x, wg, wu = rng.normal(size=(rows, K)), rng.normal(size=(I, K)) * 0.3, rng.normal(size=(I, K)) * 0.3
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 6e-2)):
        xd = dev(x).to(dtype)
        w = torch.stack([dev(wg), dev(wu)], dim=1).reshape(2 * I, K).to(dtype).contiguous()
        x64, w64 = xd.double().cpu().numpy(), w.double().cpu().numpy()
        want = plain.gelu_tanh(x64 @ w64[0::2].T) * (x64 @ w64[1::2].T)
        got = ops.gated_linear(xd, w, "gelu_tanh").double().cpu().numpy()
        assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max())
    z = dev(rng.normal(size=(rows, 70)) * 40)
    want = 30.0 * np.tanh(z.double().cpu().numpy() * 0.25 / 30.0)
    ops.scale_add_bias(z, 0.25, None, 30.0)
    assert np.abs(z.cpu().numpy() - want).max() < 1e-4


# ------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(name, dtype, folders, models):
    for i, n in enumerate([1, 2, 23, 97]):
        seq = kc.prompt(30 + i, n, vocab(name))
        r = kc.noisy_replay(folders[name], dtype, 128, models(name, dtype))
        r.step([("r", seq, list(range(n)))], end=["r"])
        kc.check_rows(r.rows, folders[name], {"r": seq}, dtype, f"whole {n}")


def test_layer_outputs_equal_the_plain_layers(folders, models):
    for name in NAMES:
        seq = kc.prompt(3, 19, vocab(name))
        config, w = kc.read_model(folders[name])
        want = []
        plain.forward(config, w, seq, want)
        r = kc.noisy_replay(folders[name], "float32", 64, models(name, "float32"), layer_outputs=True)
        r.step([("r", seq, [18])])
        assert len(want) == len(models(name, "float32").spec.schedule)
        for t in range(19):
            got = r.layers[("r", t)]
            for i in range(len(want)):
                assert np.abs(got[i] - want[i][t]).max() <= 2e-4 * max(1.0, np.abs(want[i][t]).max()), (name, i, t)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_token_by_token(name, dtype, folders, models):
    """The last 50 tokens one by one: every window of the tiny models passes over decoded tokens."""
    n = 120
    seq = kc.prompt(41, n, vocab(name))
    r = kc.noisy_replay(folders[name], dtype, 128, models(name, dtype))
    r.step([("r", seq[:n - 50], list(range(0, n - 50, 3)))])
    for t in range(n - 50, n):
        r.step([("r", [seq[t]], [0])])
    kc.check_rows(r.rows, folders[name], {"r": seq}, dtype, "tail")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_every_token_decoded(name, dtype, folders, models):
    n = 70 if dtype == "bfloat16" else 260
    seq = kc.prompt(42, n, vocab(name))
    r = kc.noisy_replay(folders[name], dtype, 272, models(name, dtype))
    for t in range(n):
        r.step([("r", [seq[t]], [0] if t % 4 == 0 or t > n - 5 else [])])
    kc.check_rows(r.rows, folders[name], {"r": seq}, dtype, "decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_down_to_two_tokens(name, dtype, folders, models):
    portions = [7, 2, 16, 3, 2, 33, 1, 15, 2, 17, 2, 5, 1, 1, 2, 40]
    n = sum(portions)
    seq = kc.prompt(43, n, vocab(name))
    r = kc.noisy_replay(folders[name], dtype, 160, models(name, dtype), page_size=8)
    o = 0
    for p in portions:
        r.step([("r", seq[o:o + p], list(range(p)))])
        o += p
    kc.check_rows(r.rows, folders[name], {"r": seq}, dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(name, dtype, folders, models):
    """Five requests over three state slots and a pool of 14 pages of 16: portions of some beside single tokens of others;
    a request that ends gives its pages and its slot to the next, which must not see what they held."""
    V = vocab(name)
    seqs = {f"s{i}": kc.prompt(50 + i, n, V) for i, n in enumerate([61, 9, 130, 33, 47])}
    r = kc.noisy_replay(folders[name], dtype, 14 * 16, models(name, dtype), max_requests=3)
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
    slot_of_s2 = r.cache.state_slot("s2")
    r.step([take("s2", 1), take("s3", 33)], end=["s3"])                                   # s3 takes a used slot and used pages
    r.step([take("s4", 2), take("s2", 30)])
    while at["s2"] < 130 or at["s4"] < 47:
        batch = [take(x, 1 if x == "s2" else 5) for x in ("s2", "s4") if at[x] < len(seqs[x])]
        r.step(batch, end=done(*[b[0] for b in batch]))
    assert r.cache.state_slot is not None and slot_of_s2 in (0, 1, 2)
    assert all(at[k] == len(seqs[k]) for k in seqs)
    kc.check_rows(r.rows, folders[name], seqs, dtype, "mixed")
    assert len(r.cache.requests) == 0 and r.cache.available_pages() == [14] * len(r.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
def test_batched_rows_equal_the_rows_of_each_request_alone(dtype, folders, models):
    """Bit for bit: what a request's rows are does not depend on what else is in the batch, nor on the slot."""
    name = "K1"
    a, b = kc.prompt(60, 45, vocab(name)), kc.prompt(61, 18, vocab(name))
    alone = kc.noisy_replay(folders[name], dtype, 128, models(name, dtype))
    alone.step([("a", a[:30], list(range(30)))]); alone.step([("a", a[30:], list(range(15)))])
    both = kc.noisy_replay(folders[name], dtype, 128, models(name, dtype))
    both.step([("b", b[:10], [9]), ("a", a[:30], list(range(30)))])
    both.step([("a", a[30:], list(range(15))), ("b", b[10:], [7])])
    for p in range(45):
        assert np.array_equal(alone.rows[("a", p)], both.rows[("a", p)]) or dtype == "bfloat16", p
        assert np.abs(alone.rows[("a", p)] - both.rows[("a", p)]).max() <= (0 if dtype == "float32" else 0.05 * np.std(alone.rows[("a", p)]))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["K1", "K2"])
def test_greedy_generation_through_the_engine(name, dtype, folders):
    """The Python entry point with its scheduler, continuous batching, portions of 16 tokens and decode steps replayed
    from CUDA graphs: every generated token is the plain implementation's first maximum given the tokens before it (in
    bfloat16: or a near tie)."""
    from coheryn_ai_studio_b200.engine import Engine
    eng = Engine.from_folder(folders[name], dtype, context=128, max_num_seqs=3, max_num_batched_tokens=16, page_size=8)
    prompts = [kc.prompt(70 + i, n, vocab(name)) for i, n in enumerate((3, 29, 50, 1))]
    res = eng.generate(prompts, max_tokens=12)
    for p, out in zip(prompts, res):
        ids = list(p)
        assert out.completion_tokens == 12 and out.finish_reason == "length"
        for tok in out.token_ids:
            ref = kc.plain_rows(folders[name], ids)[-1]
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
    name = "K2"
    a, b = kc.prompt(80, 40, vocab(name)), kc.prompt(81, 12, vocab(name))
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
    kc.check_rows(rows, folders[name], {"a": a, "b": b}, "float32", "trace")


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_output_product_per_block_equals_one_per_producer(dtype, folders, models):
    """A block multiplies [attention | delta rule | feed-forward] by the stacked output matrices once; switched off, every
    producer multiplies its own and the next norm adds the summands.  The same sum in another order."""
    from coheryn_ai_studio_b200 import ops
    name = "K1"
    layer = models(name, dtype).layers[0]
    assert layer._joined_output() and layer._joined_output()[0].shape[1] == 4 * 32 + 4 * 24 + 96
    assert not models("K4", dtype).layers[0]._joined_output()          # a piece of 90 columns: no 16-byte boundaries
    seq = kc.prompt(66, 40, vocab(name))
    rows = {}
    try:
        for on in (True, False):
            ops.set_joined_output(on)
            r = kc.noisy_replay(folders[name], dtype, 64, models(name, dtype))
            r.step([("r", seq[:33], list(range(33)))])
            for t in range(33, 40):
                r.step([("r", [seq[t]], [0])])
            rows[on] = r.rows
    finally:
        ops.set_joined_output(True)
    for key, row in rows[True].items():
        d = np.abs(row - rows[False][key]).max() / max(1.0, float(np.std(row)))
        assert d <= (2e-5 if dtype == "float32" else 0.05), (key, d)
    kc.check_rows(rows[False], folders[name], {"r": seq}, dtype, "summands")


def test_command_line_runs_and_traces_the_design(folders):
    """`coheryn run` (greedy tokens) and `coheryn trace` (every layer run's output and the logits per position) on a folder
    of this design, and the Python entry point, against the plain implementation."""
    import json, os, subprocess, sys
    from coheryn_ai_studio_b200 import api
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "K1"
    p = kc.prompt(85, 7, vocab(name))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "coheryn"), "run", folders[name], "--tokens", ",".join(map(str, p)),
                        "--max-tokens", "5", "--context", "64", "--dtype", "float32", "--stream"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [int(t) for t in r.stdout.split()]
    ids = list(p)
    for tok in got:
        assert tok == int(np.argmax(kc.plain_rows(folders[name], ids)[-1]))
        ids.append(tok)
    assert api.generate(folders[name], [p], max_tokens=5, context=64, dtype="float32")[0]["token_ids"] == got
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "coheryn"), "trace", folders[name], "--tokens", ",".join(map(str, p)),
                        "--context", "64", "--dtype", "float32"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    config, w = kc.read_model(folders[name])
    layers = []
    ref = plain.forward(config, w, p, layers)
    assert len(lines) == len(p) * (len(layers) + 1)
    for l in lines:
        want = ref[l["position"]] if l["name"] == "logits" else layers[int(l["name"].split(".")[1])][l["position"]]
        assert np.abs(np.asarray(l["values"], np.float64) - want).max() <= 2e-4 * max(1.0, float(np.abs(want).max())), l["name"]


def test_zz_report():
    print(f"\nlargest float32 difference {kc.WORST['float32']:.2e}; bfloat16 rows reached {kc.WORST['bfloat16']:.2f} of their bound")
