"""The Nuzinex decoder through the engine, against the plain implementation (`plain_nuzinex.py`).

Every test makes its own small configuration and random weights.  The configurations differ from each other in every
size and constant and exercise the values that are easily 1 or equal: one head and many, as many key/value heads as
query heads and one for all, keys and values of different widths, all of a head rotated, a part of it and none, windows
of one position, of a page and of a page and one, a borrower that looks further back than the layer it borrows from and
one that looks less far, convolutions of one tap and of several, decays of exactly one, layers without feed-forward,
sizes that are multiples of 8 (the tensor-core kernels) and sizes that are not (the plain ones).  Where random weights
would hide a fault the weights are made: a query that finds one key among hundreds, or one key at a window's edge.
"""
import json
import os

import numpy as np
import pytest
import torch

import ghost_infer_b200 as gi
import plain_nuzinex as pz

pytestmark = pytest.mark.gpu


def att(heads, kv, dim, vdim, scale, window, rot_dims, base=10000.0, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": rot_dims}}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def delta(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def layer(kind, m, ff=None):
    return {"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def par(left, right, ls=1.0, rs=1.0, ff=None):
    return layer("parallel", {"left": left, "right": right, "left_scale": ls, "right_scale": rs}, ff)


def light(heads, dim, vdim, decay, ff=None):
    return layer("lightning", {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, ff)


def model_cfg(width, vocab, side, layers, eps=1e-5):
    return {"architecture": "Nuzinex", "width": width, "vocab": vocab, "norm": {"eps": eps}, "token_side": {"dim": side}, "layers": layers}


# multiples of 8 everywhere: the tensor-core kernels in 16 bits.  The second borrower looks further back than the lender
# (which then keeps 70 positions, across a page border), the first one less far.
A_ATT = att(4, 2, 16, 24, 0.4, 20, 8, base=500.0)
CFG_A = model_cfg(96, 200, 8, [
    layer("attention", A_ATT, 136),
    par(att(4, 1, 16, 16, 0.35, None, 16, base=40000.0), delta(4, 2, 16, 24, 4), 1.3, 0.8, 72),
    light(2, 16, 8, (0.8, 1.0)),
    layer("attention", att(4, 2, 16, 24, 0.5, 12, 8, base=500.0, kv_from=0), 64),
    par(att(2, 2, 24, 8, 0.3, None, 8), delta(2, 2, 24, 16, 2), 0.6, 1.5),
    layer("attention", att(8, 2, 16, 24, 0.3, 70, 8, base=500.0, kv_from=0), 40),
])
# nothing a multiple of 8: the plain kernels.  A window of one position, a convolution of one tap, one head.
CFG_B = model_cfg(52, 301, 3, [
    par(att(3, 3, 10, 6, 0.45, None, 6, base=77.0), delta(5, 1, 6, 10, 1), 1.0, 1.0),
    layer("attention", att(5, 5, 6, 10, 0.5, 1, 2, base=9.0), 36),
    layer("attention", att(1, 1, 14, 5, 0.3, 65, 14, base=1e6), None),
    light(1, 5, 7, (0.93,), 20),
    layer("attention", att(2, 1, 14, 5, 0.6, 64, 14, base=1e6, kv_from=2), 28),
    par(att(6, 2, 4, 4, 0.7, None, 2), delta(3, 3, 10, 3, 3), 2.0, 0.25, 44),
], eps=3e-6)
# heads as wide as a served model's: keys of 64 and 128 numbers in the recurrences, heads of 64 in the attention
CFG_C = model_cfg(128, 150, 16, [
    layer("attention", att(8, 2, 64, 64, 0.125, 100, 64, base=30000.0), 256),
    par(att(4, 4, 32, 32, 0.18, None, 32), delta(2, 1, 128, 40, 4), 1.0, 1.0, 128),
    light(4, 32, 64, (0.5, 0.97, 0.999, 1.0)),
    layer("attention", att(8, 2, 64, 64, 0.125, 100, 64, base=30000.0, kv_from=0), None),
    light(2, 64, 16, (0.9, 0.99), 96),
])
CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C}
_made = {}


def tensors_of(w, bf16=True):
    out = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)) for k, v in w.items()}
    return {k: v.to(torch.bfloat16) for k, v in out.items()} if bf16 else out


def made(name):
    if name not in _made:
        cfg = CONFIGS[name]
        w = pz.random_weights(cfg, seed=len(name) + ord(name[0]))
        _made[name] = (cfg, w, tensors_of(w))
    return _made[name]


def engine_of(cfg, tensors, dtype, max_tokens=64 * 40, max_slots=None, max_seq_len=4096):
    model = gi.Model.from_config_dict(cfg).bind(tensors, dtype, "cuda:0")
    cache = model.new_cache(max_tokens=max_tokens, max_seq_len=max_seq_len, max_slots=max_slots, beyond_trained_positions=True)
    return gi.Engine(model, cache)


def engine_for(name, dtype, **kw):
    cfg, _, tensors = made(name)
    return engine_of(cfg, tensors, dtype, **kw)


_plain = {}


def plain(name, tokens):
    key = (name, tuple(tokens))
    if key not in _plain:
        cfg, w, _ = made(name)
        _plain[key] = pz.forward(cfg, w, list(tokens))
    return _plain[key]


def toks(name, n, seed):
    return np.random.default_rng(seed).integers(0, CONFIGS[name]["vocab"], size=n).tolist()


def check(got, ref, dtype, what="", keep=None):
    """`keep`: the positions that count (all, if None).  32-bit: sums of a few hundred terms over a dozen dependent stages, relative to the largest logit.  bfloat16:
    activations rounded to 8 bits between kernels; every sublayer's output is normed, so errors do not grow with depth.
    A key one position off, a lost state or a wrong angle moves logits by tens of percent."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    scale = max(1.0, float(np.abs(ref).max()))
    err = np.abs(got - ref)
    if keep is not None:
        err = err[np.asarray(keep, dtype=bool)]
    if dtype == "float32":
        assert err.max() <= 5e-5 * scale, f"{what}: max error {err.max():.3e} (scale {scale:.2f}) at {np.unravel_index(err.argmax(), err.shape)}"
    else:
        rms = float(np.sqrt((err ** 2).mean()))
        assert err.max() <= 0.08 * scale and rms <= 0.012 * scale, f"{what}: max {err.max():.3e} rms {rms:.3e} (scale {scale:.2f})"


def run_whole(eng, tokens):
    s = eng.cache.open_slot()
    out = eng.step([gi.StepEntry(s, tokens, list(range(len(tokens))))]).cpu().numpy()
    eng.cache.close_slot(s)
    return out


def prompt_then_tokens(eng, t, cut, graph=None):
    """The first `cut` tokens in one step, the rest one by one through the decode runner."""
    s = eng.cache.open_slot()
    rows = [eng.step([gi.StepEntry(s, t[:cut], list(range(cut)))]).cpu().numpy()]
    run = eng.decoder([s]) if graph is None else eng.decoder([s], use_graph=graph)
    rows += [run.forward(tokens=[x]).cpu().numpy().copy() for x in t[cut:]]
    eng.cache.close_slot(s)
    return np.concatenate(rows, 0)


PATHS = [("A", "float32"), ("B", "float32"), ("C", "float32"), ("A", "bfloat16"), ("C", "bfloat16")]

# ---- the row kernels of a layer that norms what it adds, against 64-bit torch ---------------------------------------------
@pytest.mark.parametrize("rows,width", [(5, 52), (3, 96), (70, 1028), (2, 7)])
def test_norm_on_a_sublayers_output_with_the_next_input_and_a_zeroed_sum(rows, width):
    from ghost_infer_b200.kernels import ops
    g = torch.Generator(device="cuda:0").manual_seed(rows * 1000 + width)
    x = torch.randn((rows, width), device="cuda:0", generator=g)
    y = torch.randn((rows, width), device="cuda:0", generator=g) * 3.0
    w = torch.rand((width,), device="cuda:0", generator=g) + 0.5
    sc = torch.rand((width,), device="cuda:0", generator=g) * 2.0
    eps = 1e-5
    ref = x.double() + y.double() / torch.sqrt((y.double() ** 2).mean(-1, keepdim=True) + eps) * w.double() * sc.double()
    for low in (True, False):
        xs, ys = x.clone(), y.clone()
        h = torch.full((rows, width), 7.0, device="cuda:0", dtype=torch.bfloat16 if low else torch.float32)
        ops.postnorm_add(xs, ys, w, eps, sc, cast_out=h, zero_y=True)
        torch.testing.assert_close(xs.double(), ref, rtol=1e-5, atol=1e-5)
        assert float(ys.abs().max()) == 0.0
        assert torch.equal(h, xs.to(h.dtype))                    # the next reader gets the new stream, rounded once
    xs, ys = x.clone(), y.clone()
    ops.postnorm_add(xs, ys, w, eps)                             # no scale, nothing else written
    ref1 = x.double() + y.double() / torch.sqrt((y.double() ** 2).mean(-1, keepdim=True) + eps) * w.double()
    torch.testing.assert_close(xs.double(), ref1, rtol=1e-5, atol=1e-5)
    assert torch.equal(ys, y)
    z = torch.full((rows, width), 3.0, device="cuda:0")
    hb = ops.cast_rows(x, torch.bfloat16, zero=z)
    assert torch.equal(hb, x.to(torch.bfloat16)) and float(z.abs().max()) == 0.0
    assert torch.equal(ops.cast_rows(x, torch.bfloat16), x.to(torch.bfloat16))
    a = torch.randn((rows, width), device="cuda:0", generator=g)
    out = x.clone()
    ops.axpy(out, a, 1.3)
    torch.testing.assert_close(out.double(), x.double() + 1.3 * a.double(), rtol=1e-6, atol=1e-6)


# ---- each mechanism alone: one- and two-layer models ------------------------------------------------------------------
ALONE = {
    "window": [layer("attention", att(3, 1, 8, 12, 0.4, 7, 8))],
    "window_partly_rotated": [layer("attention", att(2, 2, 12, 4, 0.5, 33, 4, base=50.0))],
    "window_not_rotated": [layer("attention", att(2, 1, 6, 6, 0.5, 5, 0))],
    "window_longer_than_the_prompt": [layer("attention", att(2, 1, 8, 8, 0.5, 500, 8))],
    "borrowed_keys": [layer("attention", att(2, 2, 8, 4, 0.5, 9, 4)), layer("attention", att(4, 2, 8, 4, 0.9, 21, 4, kv_from=0))],
    "side_by_side": [par(att(3, 1, 8, 6, 0.4, None, 8), delta(4, 2, 6, 5, 3), 0.9, 1.2)],
    "linear": [light(3, 6, 9, (0.7, 0.95, 1.0))],
    "dense": [layer("attention", att(1, 1, 4, 4, 0.5, 3, 4), 52)],
}


def one(which, seed=11, width=48, vocab=90, side=5):
    cfg = model_cfg(width, vocab, side, ALONE[which])
    return cfg, pz.random_weights(cfg, seed=seed)


@pytest.mark.parametrize("which", sorted(ALONE))
def test_each_mechanism_alone(which):
    cfg, w = one(which)
    eng = engine_of(cfg, tensors_of(w, False), "float32", max_tokens=256, max_seq_len=256)
    t = np.random.default_rng(5).integers(0, 90, size=70).tolist()
    check(run_whole(eng, t), pz.forward(cfg, w, t), "float32", which)


@pytest.mark.parametrize("side", ["left", "right"])
def test_each_of_the_two_mixers_side_by_side_alone(side):
    """With the other one's output projection zero, what the layer adds is one mixer's: gated attention, or the delta rule."""
    cfg, w = one("side_by_side")
    other = "right" if side == "left" else "left"
    w[f"l0.mix.{other}.o"] = w[f"l0.mix.{other}.o"] * 0
    eng = engine_of(cfg, tensors_of(w, False), "float32", max_tokens=256, max_seq_len=256)
    t = np.random.default_rng(6).integers(0, 90, size=80).tolist()
    ref = pz.forward(cfg, w, t)
    check(run_whole(eng, t), ref, "float32", side)
    check(prompt_then_tokens(eng, t, 30), ref, "float32", side + ", decoded")


def test_token_side_input_and_head_alone():
    """A layer whose mixer gives nothing (its output projection is zero, and the norm of zeros is zero): what reaches the
    head is the embedding plus the per-token input of each layer's own slice of the table."""
    cfg = model_cfg(40, 60, 7, [light(1, 4, 4, (0.5,)), light(1, 4, 4, (0.5,))])
    w = pz.random_weights(cfg, seed=2)
    for i in range(2):
        w[f"l{i}.mix.o"] = w[f"l{i}.mix.o"] * 0
    eng = engine_of(cfg, tensors_of(w, False), "float32", max_tokens=128, max_seq_len=128)
    t = list(range(0, 60, 7))
    x = w["embed"][t]
    for i in range(2):
        x = x + pz.token_side(x, t, w["side.embed"], pz.under(w, f"l{i}.side."), i, 7, 1e-5)
    check(run_whole(eng, t), pz.rms_norm(x, w["final.norm"], 1e-5) @ w["head"].T, "float32")


# ---- whole prompts, decoding, portions, batches -----------------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", PATHS)
def test_whole_prompt(name, dtype):
    eng = engine_for(name, dtype)
    for n, seed in ((1, 1), (2, 2), (64, 3), (65, 4), (200, 5)):
        t = toks(name, n, seed)
        check(run_whole(eng, t), plain(name, t), dtype, f"{name} {n} tokens")


@pytest.mark.parametrize("name,dtype", PATHS)
@pytest.mark.parametrize("graph", [False, True])
def test_prompt_then_token_by_token(name, dtype, graph):
    eng = engine_for(name, dtype)
    t = toks(name, 150, 21)          # decoded across the page borders at 64 and 128 and out of every window
    check(prompt_then_tokens(eng, t, 60, graph), plain(name, t), dtype)


@pytest.mark.parametrize("name", ["A", "B"])
def test_decoding_from_the_first_token(name):
    eng = engine_for(name, "float32")
    t = toks(name, 80, 8)
    s = eng.cache.open_slot()
    rows = [eng.step([gi.StepEntry(s, [x], [0])]).cpu().numpy() for x in t]
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), plain(name, t), "float32")


@pytest.mark.parametrize("name,dtype", PATHS)
def test_portions_of_several_sizes(name, dtype):
    eng = engine_for(name, dtype)
    t = toks(name, 140, 31)
    ref = plain(name, t)
    for cuts in ((2, 4, 66, 130, 140), (63, 64, 65, 128, 140), (1, 3, 5, 7, 140), (20, 40, 41, 43, 110, 140)):
        s = eng.cache.open_slot()
        rows, a = [], 0
        for b in cuts:
            rows.append(eng.step([gi.StepEntry(s, t[a:b], list(range(b - a)))]).cpu().numpy())
            a = b
        eng.cache.close_slot(s)
        check(np.concatenate(rows, 0), ref, dtype, f"{name} cut at {cuts}")


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_does_not_depend_on_the_cut_or_the_batch(name):
    eng = engine_for(name, "float32")
    t, other = toks(name, 100, 41), toks(name, 37, 42)
    whole = run_whole(eng, t)
    s = eng.cache.open_slot()
    cut = np.concatenate([eng.step([gi.StepEntry(s, t[a:b], list(range(b - a)))]).cpu().numpy() for a, b in ((0, 7), (7, 71), (71, 100))], 0)
    eng.cache.close_slot(s)
    assert np.array_equal(whole, cut)
    s1, s2 = eng.cache.open_slot(), eng.cache.open_slot()
    both = eng.step([gi.StepEntry(s2, other, [0]), gi.StepEntry(s1, t, list(range(100)))]).cpu().numpy()
    eng.cache.close_slot(s1); eng.cache.close_slot(s2)
    assert np.array_equal(whole, both[1:])


@pytest.mark.parametrize("name,dtype", PATHS)
def test_unequal_batch_against_each_alone(name, dtype):
    eng = engine_for(name, dtype)
    prompts = [toks(name, n, 50 + n) for n in (90, 3, 66, 1, 130)]
    tails = 6
    slots = [eng.cache.open_slot() for _ in prompts]
    cut = [max(1, len(p) - tails) for p in prompts]
    out = eng.step([gi.StepEntry(s, p[:c], list(range(c))) for s, p, c in zip(slots, prompts, cut)]).cpu().numpy()
    got = [[out[sum(cut[:i]):sum(cut[:i + 1])]] for i in range(len(prompts))]
    live = list(range(len(prompts)))
    fed = list(cut)
    while live:
        live = [i for i in live if fed[i] < len(prompts[i])]
        if not live:
            break
        run = eng.decoder([slots[i] for i in live])          # the shorter requests end earlier
        rows = run.forward(tokens=[prompts[i][fed[i]] for i in live]).cpu().numpy()
        for k, i in enumerate(live):
            got[i].append(rows[k:k + 1].copy())
            fed[i] += 1
    for s in slots:
        eng.cache.close_slot(s)
    for i, p in enumerate(prompts):
        check(np.concatenate(got[i], 0), plain(name, p), dtype, f"{name}: request {i} of the batch")


def test_mixed_step_of_fresh_prompts_and_sequences_under_way():
    """One step holds the second portion of one request and the whole of another: positions count from 0 in each."""
    eng = engine_for("A", "float32")
    a, b = toks("A", 120, 61), toks("A", 40, 62)
    s1, s2 = eng.cache.open_slot(), eng.cache.open_slot()
    r0 = eng.step([gi.StepEntry(s1, a[:50], list(range(50)))]).cpu().numpy()
    r1 = eng.step([gi.StepEntry(s2, b, list(range(40))), gi.StepEntry(s1, a[50:110], list(range(60)))]).cpu().numpy()
    r2 = eng.step([gi.StepEntry(s1, a[110:], list(range(10)))]).cpu().numpy()
    eng.cache.close_slot(s1); eng.cache.close_slot(s2)
    check(np.concatenate([r0, r1[40:], r2], 0), plain("A", a), "float32", "under way")
    check(r1[:40], plain("A", b), "float32", "fresh")


# ---- pages and slots given back and used again ---------------------------------------------------------------------
def test_slots_and_pages_used_again():
    """A pool of five pages and two slots: sequences come and go; whoever gets a used slot must find the recurrent state
    and the convolution's inputs zero and must not see the keys the pages held before."""
    eng = engine_for("A", "float32", max_tokens=64 * 5, max_slots=2)
    for round_ in range(3):
        p, q = toks("A", 100 + round_, 40 + round_), toks("A", 70, 50 + round_)
        s1, s2 = eng.cache.open_slot(), eng.cache.open_slot()
        out = eng.step([gi.StepEntry(s1, p, [len(p) - 1]), gi.StepEntry(s2, q, list(range(70)))]).cpu().numpy()
        check(out[0], plain("A", p)[-1], "float32", f"round {round_}")
        check(out[1:], plain("A", q), "float32", f"round {round_}")
        run = eng.decoder([s2])
        extra = toks("A", 3, 90 + round_)
        rows = [run.forward(tokens=[x]).cpu().numpy().copy() for x in extra]
        check(np.concatenate(rows, 0), plain("A", q + extra)[70:], "float32", f"round {round_}, decoded")
        eng.cache.close_slot(s1)
        eng.cache.close_slot(s2)
    assert eng.cache.free_pages == eng.cache.n_pages


def test_a_windowed_cache_gives_pages_back_as_it_goes():
    """Windows of at most 70 positions and recurrences: a sequence of 700 tokens lives in a pool of four pages, because
    pages wholly before every reader's window are given back; a lender keeps what its furthest-looking borrower reads."""
    cfg = model_cfg(64, 120, 4, [
        layer("attention", att(2, 1, 16, 8, 0.4, 9, 8), 40),
        light(2, 8, 8, (0.9, 1.0)),
        layer("attention", att(4, 1, 16, 8, 0.3, 70, 8, kv_from=0), None),
        layer("attention", att(2, 2, 8, 8, 0.5, 33, 4), 24),
    ])
    w = pz.random_weights(cfg, seed=17)
    eng = engine_of(cfg, tensors_of(w, False), "float32", max_tokens=64 * 4, max_slots=1)
    t = np.random.default_rng(61).integers(0, 120, size=700).tolist()
    s = eng.cache.open_slot()
    rows, at = [], 0
    while at < 600:
        rows.append(eng.step([gi.StepEntry(s, t[at:at + 50], list(range(50)))]).cpu().numpy())
        at += 50
    run = eng.decoder([s])
    rows += [run.forward(tokens=[x]).cpu().numpy().copy() for x in t[600:]]
    eng.cache.close_slot(s)
    assert eng.cache.free_pages == eng.cache.n_pages
    check(np.concatenate(rows, 0), pz.forward(cfg, w, t), "float32")


# ---- edges made to show ------------------------------------------------------------------------------------------------
LOVED = 5          # the token whose key every query finds


def loved_key_model(layers, q_prefixes, k_prefix, seed):
    """A model of width 32 over 16 tokens in which one token (`LOVED`) has a key that every query scores far above all
    others (16 against 0 before the scale) and a value unlike the rest: the embedding gives every token a shared
    direction (9) that the queries are made of, and only the loved token the direction (8) that keys are made of.  The
    signal sits in number 8 of a head of 16, beyond the 8 rotated numbers, so the score does not turn with distance."""
    cfg = model_cfg(32, 16, 3, layers)
    w = pz.random_weights(cfg, seed=seed)
    e = np.zeros((16, 32))
    e[:, :8] = np.random.default_rng(0).standard_normal((16, 8)).round(1) * 0.25
    e[LOVED] = 0.0
    e[LOVED, 8] = 4.0
    e[:, 9] = 1.0
    w["embed"] = e
    for p in q_prefixes:
        w[p + "q"] = np.zeros_like(w[p + "q"])
        w[p + "q"][8::16, 9] = 1.0                         # number 8 of every query head: the shared direction
        w[p + "q.norm"] = np.ones_like(w[p + "q.norm"])
        if p + "q.b" in w:
            w[p + "q.b"] = np.zeros_like(w[p + "q.b"])
    w[k_prefix + "k"] = np.zeros_like(w[k_prefix + "k"])
    w[k_prefix + "k"][8::16, 8] = 8.0                      # number 8 of every key head: only the loved token has any
    w[k_prefix + "k.norm"] = np.ones_like(w[k_prefix + "k.norm"])
    if k_prefix + "k.b" in w:
        w[k_prefix + "k.b"] = np.zeros_like(w[k_prefix + "k.b"])
    return cfg, w


def with_window(cfg, i, size):
    out = json.loads(json.dumps(cfg))
    out["layers"][i]["mixer"]["mask"]["size"] = size
    return out


def tokens_with_loved_at(n, places, seed=6):
    t = [int(x) for x in np.random.default_rng(seed).integers(6, 16, size=n)]
    for p in places:
        t[p] = LOVED
    return t


def edge_case(which):
    """(cfg, weights, tokens, reference logits, first decoded position): the oracle itself is checked to show the edge, by
    running it with the window one position shorter and one longer."""
    if which == "own_keys":
        W, i = 12, 0
        cfg, w = loved_key_model([layer("attention", att(2, 1, 16, 16, 1.0, W, 8))], ["l0.mix."], "l0.mix.", 8)
    else:                          # a borrower that looks further back than the lender, whose window is 6
        W, i = 20, 1
        cfg, w = loved_key_model([layer("attention", att(2, 1, 16, 16, 1.0, 6, 8)),
                                  layer("attention", att(2, 1, 16, 16, 1.0, W, 8, kv_from=0))], ["l0.mix.", "l1.mix."], "l0.mix.", 9)
    p1, p2 = 10, 10 + 2 * W + 3
    t = tokens_with_loved_at(p2 + W + 8, [p1, p2])
    ref = pz.forward(cfg, w, t)
    shorter, longer = pz.forward(with_window(cfg, i, W - 1), w, t), pz.forward(with_window(cfg, i, W + 1), w, t)
    for p in (p1, p2):
        last_in, first_out = p + W - 1, p + W
        assert np.abs(shorter[last_in] - ref[last_in]).max() > 0.1      # the last query that sees the key would lose it
        assert np.abs(longer[first_out] - ref[first_out]).max() > 0.1   # the first one that does not would gain it
    return cfg, w, t, ref, p1 + W - 3


@pytest.mark.parametrize("which", ["own_keys", "borrowed_keys"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_key_at_the_windows_edge_is_seen_and_the_next_one_is_not(which, dtype):
    """In a prompt, in portions that end on the edge, and token by token (the second loved key is decoded itself)."""
    cfg, w, t, ref, cut = edge_case(which)
    eng = engine_of(cfg, tensors_of(w, dtype == "bfloat16"), dtype, max_tokens=512, max_seq_len=256)
    check(run_whole(eng, t), ref, dtype, "whole")
    check(prompt_then_tokens(eng, t, cut), ref, dtype, "decoded")
    s = eng.cache.open_slot()
    rows, a = [], 0
    for b in (cut + 2, cut + 3, cut + 5, len(t)):          # portions that end just inside and just outside the window
        rows.append(eng.step([gi.StepEntry(s, t[a:b], list(range(b - a)))]).cpu().numpy())
        a = b
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), ref, dtype, "portions")


def far_key_case(n=700):
    cfg, w = loved_key_model([par(att(2, 1, 16, 16, 1.0, None, 8), delta(2, 1, 8, 8, 2), 1.0, 0.5)], ["l0.mix.left."], "l0.mix.left.", 10)
    t = tokens_with_loved_at(n, [3], seed=7)
    ref = pz.forward(cfg, w, t)
    other = list(t)
    other[3] = 7
    assert np.abs(pz.forward(cfg, w, other)[-1] - ref[-1]).max() > 0.1    # the last token still listens to the fourth
    return cfg, w, t, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds(dtype):
    """Causal attention: the fourth token's key, eleven pages back, is the one every query wants; whole and decoded."""
    cfg, w, t, ref = far_key_case()
    eng = engine_of(cfg, tensors_of(w, dtype == "bfloat16"), dtype, max_tokens=64 * 30, max_seq_len=1024)
    check(run_whole(eng, t), ref, dtype, "whole")
    check(prompt_then_tokens(eng, t, 640), ref, dtype, "decoded")      # decoded across the page border at 640..704
    s = eng.cache.open_slot()
    rows = [eng.step([gi.StepEntry(s, t[a:b], list(range(b - a)))]).cpu().numpy() for a, b in ((0, 2), (2, 64), (64, 449), (449, 700))]
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), ref, dtype, "portions")


def test_a_decay_of_one_keeps_the_first_token():
    """Linear attention with decay exactly 1 forgets nothing: the first token moves the last logits of a long prompt; with
    a decay of 0.5 it is gone.  Both through the engine, whole and decoded."""
    for decay, stays in ((1.0, True), (0.5, False)):
        cfg = model_cfg(40, 30, 4, [light(2, 8, 8, (decay, decay))])
        w = pz.random_weights(cfg, seed=3)
        t = np.random.default_rng(4).integers(0, 30, size=300).tolist()
        ref = pz.forward(cfg, w, t)
        other = [(t[0] + 1) % 30] + t[1:]
        assert (np.abs(pz.forward(cfg, w, other)[-1] - ref[-1]).max() > 1e-3) == stays
        eng = engine_of(cfg, tensors_of(w, False), "float32", max_tokens=512, max_seq_len=512)
        check(run_whole(eng, t), ref, "float32", f"decay {decay}")
        check(prompt_then_tokens(eng, t, 250), ref, "float32", f"decay {decay}, decoded")


# ---- long decoding -------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_through_the_graph_runner(name):
    """320 decoded tokens after a prompt of 10: the 256-position length bucket, five page borders, every window passed
    several times, the recurrent state written 320 times."""
    eng = engine_for(name, "bfloat16")
    t = toks(name, 330, 71)
    check(prompt_then_tokens(eng, t, 10, True), plain(name, t), "bfloat16")


# ---- generation through the entry point ----------------------------------------------------------------------------------
def write_model(folder, cfg, w):
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    pz.write_safetensors_bf16(str(folder / "model.safetensors"), w)
    return str(folder)


def test_greedy_generation_through_the_entry_point(tmp_path):
    """`LLM.generate` on a model folder: the scheduler cuts prompts into portions of 16 tokens and decodes two requests at
    a time; every greedy token is the plain implementation's, as long as that one's choice is clear."""
    cfg, w, _ = made("A")
    llm = gi.LLM(write_model(tmp_path / "model", cfg, w), dtype="float32", max_tokens=64 * 16, max_seq_len=512)
    prompts = [toks("A", n, 80 + i) for i, n in enumerate([3, 30, 11, 75])]
    res = llm.generate(prompts, max_new=6, temperature=0.0, stop_token_ids=(), batch_size=2, max_step_tokens=16)
    for p, r in zip(prompts, res):
        seq = list(p)
        for _ in range(6):
            logits = pz.forward(cfg, w, seq)[-1]
            order = np.argsort(-logits, kind="stable")
            if logits[order[0]] - logits[order[1]] < 1e-3:
                break
            seq.append(int(order[0]))
        want = seq[len(p):]
        assert r.tokens[:len(want)] == want, f"prompt of {len(p)}: {r.tokens} vs {want}"
    assert llm.cache.free_pages == llm.cache.n_pages


# ---- configurations drawn at random ------------------------------------------------------------------------------------
def random_config(seed, sixteen_bit):
    """Sizes drawn from lists that mix multiples of 8 with numbers that are not (which take the kernels' plain paths; the
    16-bit path is drawn from multiples of 8 only), layers in any order, borrowers after any lender."""
    r = np.random.default_rng(seed)
    pick = lambda xs: int(xs[r.integers(len(xs))])
    even = lambda top: 2 * int(r.integers(0, top // 2 + 1))
    dims = [8, 16, 24, 64] if sixteen_bit else [4, 6, 10, 16, 36]
    vdims = [8, 16, 40] if sixteen_bit else [3, 8, 12, 20]
    width = pick([64, 96, 128] if sixteen_bit else [40, 52, 72, 100])
    layers, lenders = [], []
    for i in range(pick([2, 3, 4, 5])):
        kind = pick([0, 1, 2, 3]) if lenders else pick([0, 1, 2])
        ff = pick([0, 24, 40, 64]) or None
        if kind == 0:
            kv, dim = pick([1, 2, 3]), pick(dims)
            m = att(kv * pick([1, 2, 4]), kv, dim, pick(vdims), float(r.uniform(0.1, 0.6)), pick([1, 2, 7, 33, 64, 65, 90, 300]),
                    (8 * int(r.integers(0, dim // 8 + 1))) if sixteen_bit else even(dim), base=float(10 ** r.uniform(1, 6)))
            lenders.append((i, m))
            layers.append(layer("attention", m, ff))
        elif kind == 3:
            j, src = lenders[int(r.integers(len(lenders)))]
            m = dict(src, heads=src["kv_heads"] * pick([1, 2, 3]), scale=float(r.uniform(0.1, 0.6)), mask={"size": pick([1, 5, 64, 70, 200])},
                     kv_from=j)
            layers.append(layer("attention", m, ff))
        elif kind == 1:
            kv, dim = pick([1, 2]), pick(dims)
            left = att(kv * pick([1, 3]), kv, dim, pick(vdims), float(r.uniform(0.1, 0.6)), None,
                       (8 * int(r.integers(0, dim // 8 + 1))) if sixteen_bit else even(dim), base=float(10 ** r.uniform(1, 6)))
            qk = pick([1, 2, 3])
            right = delta(qk * pick([1, 2]), qk, pick(dims + [128]), pick(vdims), pick([1, 2, 3, 4, 5]))
            layers.append(par(left, right, float(r.uniform(0.3, 2.0)), float(r.uniform(0.3, 2.0)), ff))
        else:
            heads = pick([1, 2, 5])
            layers.append(light(heads, pick(dims), pick(vdims), [float(x) for x in r.choice([0.3, 0.9, 0.99, 1.0], size=heads)], ff))
    side = pick([8, 16] if sixteen_bit else [1, 3, 7, 12])
    return model_cfg(width, pick([64, 200] if sixteen_bit else [50, 97, 260]), side, layers, eps=float(10 ** r.uniform(-6, -4)))


def well_conditioned(cfg, w, tokens, ref):
    """The positions whose logits the plain implementation itself keeps when its weights and the sums that take their type
    are 32-bit.  Where a drawn model norms a vector that nearly cancelled (a read-out of a few terms in a sequence's first
    tokens), rounding alone moves the logits by more than a fault would elsewhere; such a position says nothing about the
    kernels.  They are few: more than one in twenty-five fails the test."""
    w32 = {k: (v.astype(np.float32) if v.dtype.kind == "f" else v) for k, v in w.items()}
    low = np.asarray(pz.forward(cfg, w32, tokens), dtype=np.float64)
    keep = np.abs(low - ref).max(axis=1) <= 1e-5 * max(1.0, float(np.abs(ref).max()))
    assert keep.mean() >= 0.96, f"{cfg}: {int((~keep).sum())} of {len(keep)} positions are ill-conditioned"
    return keep


@pytest.mark.parametrize("seed,dtype", [(s, "float32") for s in range(8)] + [(s, "bfloat16") for s in range(100, 105)])
def test_configurations_drawn_at_random(seed, dtype):
    """Whole prompt, prompt cut in three, the tail token by token, and a batch of three, on a model nobody chose."""
    cfg = random_config(seed, dtype == "bfloat16")
    w = pz.random_weights(cfg, seed=seed)
    eng = engine_of(cfg, tensors_of(w), dtype, max_tokens=64 * 24, max_seq_len=1024)
    r = np.random.default_rng(seed + 1)
    prompts = [r.integers(0, cfg["vocab"], size=n).tolist() for n in (150, 70, 9)]
    refs = [pz.forward(cfg, w, p) for p in prompts]
    keeps = [well_conditioned(cfg, w, p, ref) for p, ref in zip(prompts, refs)]
    check(run_whole(eng, prompts[0]), refs[0], dtype, f"{cfg}: whole", keeps[0])
    s = eng.cache.open_slot()
    rows = [eng.step([gi.StepEntry(s, prompts[0][a:b], list(range(b - a)))]).cpu().numpy() for a, b in ((0, 2), (2, 67), (67, 130))]
    run = eng.decoder([s])
    rows += [run.forward(tokens=[t]).cpu().numpy().copy() for t in prompts[0][130:]]
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), refs[0], dtype, f"{cfg}: cut and decoded", keeps[0])
    slots = [eng.cache.open_slot() for _ in prompts]
    cut = [len(p) - 5 for p in prompts]
    out = eng.step([gi.StepEntry(sl, p[:c], list(range(c))) for sl, p, c in zip(slots, prompts, cut)]).cpu().numpy()
    got = [[out[sum(cut[:i]):sum(cut[:i + 1])]] for i in range(3)]
    run = eng.decoder(slots)
    for k in range(5):
        step_rows = run.forward(tokens=[p[c + k] for p, c in zip(prompts, cut)]).cpu().numpy()
        for i in range(3):
            got[i].append(step_rows[i:i + 1].copy())
    for sl in slots:
        eng.cache.close_slot(sl)
    for i in range(3):
        check(np.concatenate(got[i], 0), refs[i], dtype, f"{cfg}: request {i} of a batch", keeps[i])


# ---- the replay program as a user runs it ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(tmp_path, dtype):
    """`bin/trace_run` on a model folder: requests whole, tails token by token, and unequal batches decoded together."""
    import subprocess
    import sys
    from test_gpu_trace_run import build_trace
    cfg, w, _ = made("A" if dtype == "bfloat16" else "B")
    d = write_model(tmp_path / "model", cfg, w)
    reqs, steps = build_trace({"vocab_size": cfg["vocab"]})
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(64 * 8)], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                       text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    assert p.stdout.split("\n")[:len(steps)] == [f"done {i}" for i in range(len(steps))]
    refs = {rid: pz.forward(cfg, w, ts) for rid, ts in reqs.items()}
    place = {}
    for s in steps:
        want_rows = []
        for e in s["entries"]:
            base = place.get(e["id"], 0)
            want_rows += [refs[e["id"][:2]][base + k] for k in e["want"]]
            place[e["id"]] = base + len(e["tokens"])
        f = out / f"{s['step']}.f32"
        if want_rows:
            check(np.fromfile(f, dtype="<f4").reshape(-1, cfg["vocab"]), np.stack(want_rows), dtype, f"step {s['step']}")
        else:
            assert not f.exists()
