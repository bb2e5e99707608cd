"""The Torutar decoder through the engine, against the plain implementation (`plain_torutar.py`).

Every test makes its own small configuration and random weights.  The configurations differ from each other in every size
and constant and exercise the values that are easily 1 or equal: one copy of the stream and several, a convolution of one
tap and of several, one head and many, as many key/value heads as query heads and one for all, keys and values of different
widths, all of a head rotated, a part and none, windows of one position, of a page and of a page and one, no kept first
positions, a few and more than a page, a borrower that looks further back than the layer it borrows from and one that looks
less far, every expert chosen and one of many, layers without feed-forward, sizes that are multiples of 8 (the tensor-core
kernels) and sizes that are not (the plain ones).  Where random weights would hide a fault the inputs are made: one key
whose score stands out, placed just inside and just outside a window's edge and the kept first positions.
"""
import numpy as np
import pytest
import torch

import ghost_infer_b200 as gi
import plain_torutar as pt

pytestmark = pytest.mark.gpu


def att(heads, kv, dim, vdim, scale, window, keep, rot_dims, base=10000.0, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": rot_dims},
         "mask": {"size": window, "keep_first": keep}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def lat(heads, dim, rot_dim, vdim, rank, q_rank, scale, base=10000.0):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank, "scale": scale,
            "rot": {"base": base, "dims": rot_dim}}


def mem(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def moe(experts, top, ff, limit, shared_ff, shared_limit, scale):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff, "limit": limit},
            "shared": {"ff": shared_ff, "limit": shared_limit}}


def layer(kind, m, mlp=None):
    return {"type": kind, "mixer": m, "mlp": mlp}


def model_cfg(width, vocab, streams, taps, layers, eps=1e-5, logit_scale=1.0):
    return {"architecture": "Torutar", "width": width, "vocab": vocab, "streams": streams, "canon": {"taps": taps},
            "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}


# multiples of 8 everywhere.  The second borrower looks further back than the lender and keeps more first positions.
CFG_A = model_cfg(96, 200, 3, 3, [
    layer("latent_attention", lat(4, 16, 8, 16, 32, 24, 0.25, base=500.0), moe(4, 2, 24, 1.0, 40, 2.0, 2.0)),
    layer("mlstm", mem(2, 16, 24, 12.0), moe(8, 3, 16, 0.7, 24, 1.5, 1.0)),
    layer("attention", att(4, 2, 16, 24, 0.4, 20, 4, 8, base=500.0), moe(4, 4, 16, 1.0, 16, 1.0, 0.5)),
    layer("attention", att(4, 2, 16, 24, 0.5, 12, 2, 8, base=500.0, kv_from=2)),
    layer("mlstm", mem(4, 8, 8, 3.0)),
    layer("attention", att(8, 2, 16, 24, 0.3, 70, 9, 8, base=500.0, kv_from=2), moe(5, 1, 24, 2.0, 8, 0.5, 1.3)),
], logit_scale=0.5)
# nothing a multiple of 8; one copy of the stream, one tap, one head, a window of one position, nothing kept, nothing rotated
CFG_B = model_cfg(52, 301, 1, 1, [
    layer("attention", att(3, 3, 10, 6, 0.45, 1, 0, 0), moe(3, 1, 9, 1.0, 7, 2.0, 1.0)),
    layer("mlstm", mem(1, 5, 7, 8.0)),
    layer("latent_attention", lat(3, 6, 4, 5, 11, 13, 0.4, base=77.0), moe(2, 2, 5, 0.5, 3, 0.5, 3.0)),
    layer("attention", att(1, 1, 14, 5, 0.3, 65, 1, 14, base=1e6)),
    layer("attention", att(2, 1, 14, 5, 0.6, 64, 3, 14, base=1e6, kv_from=3), moe(6, 2, 4, 1.0, 6, 1.0, 1.0)),
    layer("mlstm", mem(3, 9, 4, 15.0), moe(4, 3, 6, 1.5, 5, 1.0, 0.8)),
], eps=3e-6, logit_scale=1.7)
# heads as wide as a served model's; kept first positions across a page border; four taps, four copies
CFG_C = model_cfg(128, 150, 4, 4, [
    layer("attention", att(8, 2, 64, 64, 0.125, 100, 70, 32, base=30000.0), moe(8, 2, 32, 1.0, 64, 2.0, 2.0)),
    layer("mlstm", mem(2, 64, 64, 12.0)),
    layer("latent_attention", lat(4, 32, 32, 32, 64, 48, 0.125, base=500000.0), moe(4, 2, 64, 1.0, 32, 2.0, 1.0)),
    layer("attention", att(8, 2, 64, 64, 0.125, 40, 70, 32, base=30000.0, kv_from=0)),
    layer("mlstm", mem(1, 128, 40, 6.0), moe(4, 1, 48, 0.8, 24, 1.2, 1.0)),
])
CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C}
_made = {}


def tensors_of(w, bf16=True):
    out = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)) for k, v in w.items()}
    return {k: v.to(torch.bfloat16) for k, v in out.items()} if bf16 else out


def made(name):
    if name not in _made:
        cfg = CONFIGS[name]
        w = pt.random_weights(cfg, seed=len(name) + ord(name[0]))
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
    """(logits, positions that count in 16 bits): a position does not count where a router's choice rests on a gap that a
    bfloat16 rounding could close (and the choice matters)."""
    key = (name, tuple(tokens))
    if key not in _plain:
        cfg, w, _ = made(name)
        gaps = []
        ref = pt.forward(cfg, w, list(tokens), gaps=gaps)
        close = np.min(np.stack(gaps), axis=0) < 0.01 if gaps else np.zeros(len(tokens), dtype=bool)
        _plain[key] = (ref, ~close)
    return _plain[key]


def toks(name, n, seed):
    return np.random.default_rng(seed).integers(0, CONFIGS[name]["vocab"], size=n).tolist()


def check(got, ref, dtype, what="", keep=None):
    """32-bit: sums of a few hundred terms over a dozen dependent stages, relative to the largest logit.  bfloat16: activations
    rounded to 8 bits between kernels; `keep` leaves out what follows a router's close call.  A key one position off, a lost
    state or a wrong angle moves logits by tens of percent."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    scale = max(1.0, float(np.abs(ref).max()))
    err = np.abs(got - ref)
    if dtype == "float32":
        assert err.max() <= 5e-5 * scale, f"{what}: max error {err.max():.3e} (scale {scale:.2f}) at {np.unravel_index(err.argmax(), err.shape)}"
        return
    if keep is not None and err.ndim == 2:
        keep = np.asarray(keep, dtype=bool)
        assert len(keep) < 20 or keep.sum() * 4 >= 3 * len(keep), f"{what}: too few positions count ({keep.sum()} of {len(keep)})"
        err = err[keep]
        if err.size == 0:
            return
        # Roundings move a router's shares by a percent or so, and where two experts' choice scores lie closer than that the
        # 16-bit run may choose the other one: that position's logits then differ by an expert's whole contribution, and later
        # positions feel it through the caches and states (a layer that gives a token one expert of three changes most of all).
        # So one position in five may be off; a window one position off,
        # a lost state or a wrong angle puts nearly all of them off (and the 32-bit runs of the same tests allow none).
        worst = err.max(axis=1)
        off = worst > 0.08 * scale
        assert off.sum() <= max(1, len(worst) // 5), f"{what}: {off.sum()} of {len(worst)} positions are off (worst {worst.max():.3e}, scale {scale:.2f})"
        err = err[~off]
        if err.size == 0:
            return
    rms = float(np.sqrt((err ** 2).mean()))
    assert err.max() <= 0.08 * scale and rms <= 0.012 * scale, f"{what}: max {err.max():.3e} rms {rms:.3e} (scale {scale:.2f})"


def check_plain(got, name, tokens, dtype, what="", rows=None):
    ref, keep = plain(name, tokens)
    if rows is not None:
        ref, keep = ref[rows], keep[rows]
    check(got, ref, dtype, what, keep)


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


PATHS = [("A", "float32"), ("B", "float32"), ("C", "float32"), ("A", "bfloat16"), ("B", "bfloat16"), ("C", "bfloat16")]


# ---- the row kernels of a layer over several copies of the stream, against 64-bit torch ------------------------------------
@pytest.mark.parametrize("rows,width,streams", [(5, 52, 1), (3, 96, 3), (70, 1028, 4), (2, 7, 16)])
def test_copies_of_the_stream_are_read_and_written(rows, width, streams):
    from ghost_infer_b200.kernels import ops
    g = torch.Generator(device="cuda:0").manual_seed(rows * 1000 + width)
    rnd = lambda *shape: torch.randn(shape, device="cuda:0", generator=g)
    e = rnd(rows, width)
    x = ops.stream_expand(e, streams)
    assert torch.equal(x.view(rows, streams, width), e[:, None, :].expand(rows, streams, width))
    x = rnd(rows, streams * width)
    pick = torch.tensor([rows - 1, 0], dtype=torch.int32, device="cuda:0")
    torch.testing.assert_close(ops.stream_sum(x, streams).double(), x.view(rows, streams, width).double().sum(1), rtol=1e-6, atol=1e-5)
    torch.testing.assert_close(ops.stream_sum(x, streams, pick), ops.stream_sum(x, streams)[pick.long()])
    blend, w, eps = rnd(streams), torch.rand((width,), device="cuda:0", generator=g) + 0.5, 1e-5
    u = (x.view(rows, streams, width).double() * blend.double()[None, :, None]).sum(1)
    ref = u / torch.sqrt((u ** 2).mean(-1, keepdim=True) + eps) * w.double()
    z = torch.full((rows, width), 3.0, device="cuda:0")
    h = ops.hyper_read(x, blend, w, eps, torch.float32, zero=z)
    torch.testing.assert_close(h.double(), ref, rtol=1e-5, atol=1e-5)
    assert float(z.abs().max()) == 0.0
    assert torch.equal(ops.hyper_read(x, blend, w.bfloat16(), eps, torch.bfloat16),
                       ops.hyper_read(x, blend, w.bfloat16().float(), eps, torch.float32).bfloat16())
    y, gate, bias = rnd(rows, width), rnd(rows, width), rnd(width)
    mix, share = rnd(streams, streams), rnd(streams)
    step = type("S", (), {"token_slots": torch.zeros(rows, dtype=torch.int32, device="cuda:0")})()
    v = y.double() * torch.sigmoid(gate.double() + bias.double())
    want = torch.einsum("st,nsd->ntd", mix.double(), x.view(rows, streams, width).double()) + share.double()[None, :, None] * v[:, None, :]
    xs = x.clone()
    ops.hyper_write(xs, y, mix, share, gate, bias, step=step)
    torch.testing.assert_close(xs.view(rows, streams, width).double(), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("taps", [1, 2, 4, 8])
def test_input_convolution_across_portions_and_in_a_batch(taps):
    """Two sequences side by side, fed in portions of unequal sizes down to one token: every portion reads the inputs before it
    from the state the portion before left."""
    from ghost_infer_b200.kernels import ops
    g = torch.Generator(device="cuda:0").manual_seed(taps)
    d, lens = 20, (23, 9)
    hs = [torch.randn((n, d), device="cuda:0", generator=g) for n in lens]
    w = torch.randn((d, taps), device="cuda:0", generator=g)
    want = [torch.from_numpy(pt.causal_conv_added(h.double().cpu().numpy(), w.double().cpu().numpy())) for h in hs]
    state = torch.zeros((3, (taps - 1) * d + 5), device="cuda:0")[:, :max(1, (taps - 1) * d)]      # rows further apart than they are long
    x = torch.zeros((1, d), device="cuda:0")
    one = torch.ones((1,), device="cuda:0")
    got = [[], []]
    at = [0, 0]
    for portion in ((1, 1), (2, 3), (1, 0), (7, 1), (3, 4), (9, 0)):
        rows, slots, who = [], [], []
        for b, n in enumerate(portion):
            if n:
                rows.append(hs[b][at[b]:at[b] + n]); slots += [b] * n; who.append((b, n)); at[b] += n
        h = torch.cat(rows).contiguous()
        step = type("S", (), {"token_slots": torch.tensor(slots, dtype=torch.int32, device="cuda:0")})()
        out = ops.input_conv(h, w, state if taps > 1 else None, step)
        ops.hyper_write(torch.zeros((h.shape[0], d), device="cuda:0"), torch.zeros((h.shape[0], d), device="cuda:0"), one.view(1, 1), one,
                        h=h if taps > 1 else None, state=state if taps > 1 else None, taps=taps, step=step)
        o = 0
        for b, n in who:
            got[b].append(out[o:o + n]); o += n
    for b in range(2):
        torch.testing.assert_close(torch.cat(got[b]).double().cpu(), want[b], rtol=1e-5, atol=1e-5)


# ---- edges made to show: one key whose score stands out, just inside and just outside what a query sees ------------------
def _standout_case(n, window, keep, loved, heads=4, kv=2, dim=16, vdim=24, seed=3):
    """Queries all alike, keys small but for the loved positions, whose score is far above the rest; values unlike each other."""
    rng = np.random.default_rng(seed)
    q = np.tile(rng.standard_normal((1, heads, dim)), (n, 1, 1)) * 4.0 / np.sqrt(dim)
    k = rng.standard_normal((n, kv, dim)) * 0.05
    for p in loved:
        k[p] = q[0, ::heads // kv] * 1.5
    v = rng.standard_normal((n, kv, vdim))
    sink = rng.standard_normal(heads)
    ref = pt.softmax_attention(q, k, v, 0.5, pt.visible(n, window, keep), sink)
    return q, k, v, sink, ref


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim,vdim", [(16, 24), (64, 64), (128, 128)])      # the plain kernels; in 16 bits mma.sync, tcgen05 at 64 and 128
@pytest.mark.parametrize("window,keep", [(33, 0), (33, 5), (64, 64), (65, 65), (20, 70), (1, 1), (100, 3), (90, 17)])
def test_a_key_at_the_windows_edge_and_among_the_kept_first(dtype, dim, vdim, window, keep):
    """Loved keys sit at the last kept position, the first one not kept, and far back; the queries just inside and just outside
    their reach show them or not, in a prompt, in portions that end on the edges, and token by token."""
    from ghost_infer_b200.kernels import ops
    from ghost_infer_b200.cache.sequence_cache import CacheRequest, SequenceCache
    n, H, G = 300, 4, 2
    loved = sorted({max(keep - 1, 0), keep, 130})
    q, k, v, sink, ref = _standout_case(n, window, keep, loved, dim=dim, vdim=vdim)
    for p in loved:            # the oracle itself shows the edge
        if p >= keep and p + window < n:
            assert np.abs(ref[p + window - 1] - ref[p + window]).max() > 0.05
    cache = SequenceCache([(0, CacheRequest("window", G, dim, window, vdim, keep_first=keep), None, None)], max_tokens=64 * 8, max_slots=2,
                          max_seq_len=1024, dtype=dtype, device="cuda:0")
    dev = lambda a: torch.from_numpy(a.reshape(a.shape[0], -1)).to(device="cuda:0", dtype=dtype).contiguous()
    qd, kd, vd, sk = dev(q), dev(k), dev(v), torch.from_numpy(sink).to(device="cuda:0", dtype=torch.float32)
    for cuts in ([n], [keep + 1, 130 + window - 1, 130 + window, 131 + window, n] if 131 + window < n else [2, n], "tokens"):
        slot = cache.open_slot()
        bounds = list(range(1, n + 1)) if cuts == "tokens" else cuts
        out, a = [], 0
        for b in bounds:
            if b <= a:
                continue
            cache.reserve([(slot, b)]); cache.sync_tables()
            mem_ = cache.memory(0)
            pos = torch.arange(a, b, dtype=torch.int32, device="cuda:0")
            pages = mem_.block_table[slot, (pos // 64).long()].long()
            mem_.k[pages, :, (pos % 64).long()] = kd[a:b].view(b - a, G, dim)
            mem_.v[pages, :, (pos % 64).long()] = vd[a:b].view(b - a, G, vdim)
            step = type("S", (), {})()
            step.is_decode, step.n_seqs, step.max_q_len, step.max_kv_len, step.sm_count = (b - a == 1 and a > 0), 1, b - a, b, 148
            i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda:0")
            step.cu_seqlens, step.seq_slots, step.seq_pos0, step.seq_lens = i32([0, b - a]), i32([slot]), i32([a]), i32([b])
            o = torch.empty((b - a, H * vdim), dtype=dtype, device="cuda:0")
            ops.attention_general(qd[a:b].contiguous(), mem_, step, H, G, dim, vdim, 0.5, o, window=window, sinks=sk, keep_first=keep)
            out.append(o.float().cpu().numpy())
            cache.commit(slot, b)
            a = b
        cache.close_slot(slot)
        got = np.concatenate(out, 0).reshape(n, H, vdim)
        tol = 2e-5 if dtype == torch.float32 else 0.03
        assert np.abs(got - ref).max() <= tol, f"window {window}, kept {keep}, {cuts if cuts == 'tokens' else 'portions'}: {np.abs(got - ref).max():.3e}"
    assert cache.free_pages == cache.n_pages


# ---- each mechanism alone: one- and two-layer models ------------------------------------------------------------------
ALONE = {
    "window": [layer("attention", att(3, 1, 8, 12, 0.4, 7, 2, 8))],
    "window_partly_rotated": [layer("attention", att(2, 2, 12, 4, 0.5, 33, 0, 4, base=50.0))],
    "window_longer_than_the_prompt": [layer("attention", att(2, 1, 8, 8, 0.5, 500, 3, 8))],
    "kept_more_than_the_window": [layer("attention", att(2, 1, 8, 8, 0.5, 3, 30, 0))],
    "borrowed_keys": [layer("attention", att(2, 2, 8, 4, 0.5, 9, 1, 4)), layer("attention", att(4, 2, 8, 4, 0.9, 21, 6, 4, kv_from=0))],
    "latent": [layer("latent_attention", lat(3, 6, 4, 5, 12, 10, 0.4))],
    "latent_all_rotated_queries_wide": [layer("latent_attention", lat(2, 8, 8, 8, 16, 40, 0.3, base=50.0))],
    "matrix_memory": [layer("mlstm", mem(3, 6, 9, 12.0))],
    "matrix_memory_tight_cap": [layer("mlstm", mem(2, 4, 4, 0.5))],
    "matrix_memory_wide_keys": [layer("mlstm", mem(1, 200, 8, 10.0))],
    "matrix_memory_widest_keys": [layer("mlstm", mem(1, 256, 4, 10.0))],
    "experts": [layer("mlstm", mem(1, 4, 4, 5.0), moe(6, 2, 10, 1.0, 12, 2.0, 2.0))],
    "experts_all_chosen_no_clamp_reached": [layer("mlstm", mem(1, 4, 4, 5.0), moe(3, 3, 8, 50.0, 4, 50.0, 1.0))],
}


@pytest.mark.parametrize("which", sorted(ALONE))
@pytest.mark.parametrize("streams,taps", [(1, 1), (3, 3)])
def test_each_mechanism_alone(which, streams, taps):
    cfg = model_cfg(48, 90, streams, taps, ALONE[which], logit_scale=0.75)
    w = pt.random_weights(cfg, seed=11)
    eng = engine_of(cfg, tensors_of(w, False), "float32", max_tokens=256, max_seq_len=256)
    t = np.random.default_rng(5).integers(0, 90, size=70).tolist()
    ref = pt.forward(cfg, w, t)
    check(run_whole(eng, t), ref, "float32", which)
    check(prompt_then_tokens(eng, t, 30), ref, "float32", which + ", decoded")


def test_the_matrix_memory_and_the_routers_choice_by_themselves():
    """The recurrence's kernels against the plain walk, state carried over a cut; the router's ids and weights."""
    from ghost_infer_b200.kernels import ops
    cfg = model_cfg(40, 60, 1, 1, [layer("mlstm", mem(3, 10, 6, 4.0), moe(7, 3, 8, 1.0, 8, 1.0, 1.7))])
    w = pt.random_weights(cfg, seed=4)
    h = np.random.default_rng(1).standard_normal((50, 40))
    ref, _ = pt.mlstm(h, w, "l0.mix.", cfg["layers"][0]["mixer"], 1e-5)
    model = gi.Model.from_config_dict(cfg).bind(tensors_of(w, False), "float32", "cuda:0")
    cache = model.new_cache(max_tokens=128, max_seq_len=128)
    eng = gi.Engine(model, cache)
    mixer, ffn = model.layers[0].block.mixer, model.layers[0].block.ffn
    hd = torch.from_numpy(h).to("cuda:0", torch.float32)
    s = cache.open_slot()
    got = []
    for a, b in ((0, 17), (17, 18), (18, 50)):
        cache.reserve([(s, b)]); cache.sync_tables()
        ctx = eng.build_context([gi.StepEntry(s, [0] * (b - a), [])])
        y = torch.zeros((b - a, 40), device="cuda:0")
        mixer.forward(hd[a:b].contiguous(), y, ctx, cache.memory(0))
        got.append(y.cpu().numpy())
        cache.commit(s, b)
    assert np.abs(np.concatenate(got) - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max())
    ids, wts = ops.moe_route_shares(hd, ffn.w_router, 3, ffn.correction, 1.7)
    rid, rw = pt.route(h, w, "l0.mlp.", cfg["layers"][0]["mlp"]["router"])
    assert np.array_equal(ids.cpu().numpy(), rid)
    assert np.abs(wts.cpu().numpy() - rw).max() <= 1e-5


@pytest.mark.parametrize("rows", [5, 64, 65, 300])
@pytest.mark.parametrize("limit", [0.6, 7.0])
def test_clamped_gated_value_in_the_products(rows, limit):
    """min(g, limit) * sigmoid(alpha g') * (clamp(u) + 1) in the epilogue of the streamed product (up to 64 rows) and of the
    tcgen05 product (more), and as a step of its own over either layout of the rows, against 64-bit torch."""
    from ghost_infer_b200.kernels import ops
    g = torch.Generator(device="cuda:0").manual_seed(rows)
    k, f, alpha = 128, 72, 1.702
    h = torch.randn((rows, k), device="cuda:0", generator=g).bfloat16()
    wg, wu = (torch.randn((f, k), device="cuda:0", generator=g) * 0.15).bfloat16(), (torch.randn((f, k), device="cuda:0", generator=g) * 0.15).bfloat16()
    gate, up = h.double() @ wg.double().T, h.double() @ wu.double().T
    gc, uc = gate.clamp(max=limit), up.clamp(-limit, limit)
    ref = gc * torch.sigmoid(alpha * gc) * (uc + 1.0)
    inter = torch.stack([wg.view(f // 8, 8, k), wu.view(f // 8, 8, k)], dim=1).reshape(2 * f, k).contiguous()
    got = ops.clamped_glu_interleaved(h, inter, limit, alpha)
    assert got.dtype == torch.bfloat16 and tuple(got.shape) == (rows, f)
    torch.testing.assert_close(got.double(), ref, rtol=2e-2, atol=2e-2)
    rows32 = torch.cat([gate, up], dim=1).float().contiguous()
    torch.testing.assert_close(ops.clamped_glu(rows32, limit, alpha).double(), ref, rtol=1e-5, atol=1e-5)
    inter32 = torch.stack([gate.view(rows, f // 8, 8), up.view(rows, f // 8, 8)], dim=2).reshape(rows, 2 * f).float().contiguous()
    torch.testing.assert_close(ops.clamped_glu(inter32, limit, alpha, interleaved=True).double(), ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_experts_of_a_long_prompt(dtype):
    """Enough rows per expert for the products expert by expert on the tensor cores (16 bits), and more (token, expert) pairs
    than the few-row kernels take (both precisions)."""
    cfg = model_cfg(64, 80, 2, 2, [layer("mlstm", mem(2, 8, 8, 6.0), moe(4, 2, 64, 1.0, 64, 2.0, 1.5))])
    w = pt.random_weights(cfg, seed=23)
    eng = engine_of(cfg, tensors_of(w, dtype == "bfloat16"), dtype, max_tokens=1024, max_seq_len=1024)
    t = np.random.default_rng(3).integers(0, 80, size=400).tolist()
    gaps = []
    ref = pt.forward(cfg, w, t, gaps=gaps)
    check(run_whole(eng, t), ref, dtype, "long prompt", np.min(np.stack(gaps), axis=0) >= 0.01)


# ---- whole prompts, decoding, portions, batches -----------------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", PATHS)
def test_whole_prompt(name, dtype):
    eng = engine_for(name, dtype)
    for n, seed in ((1, 1), (2, 2), (64, 3), (65, 4), (200, 5)):
        t = toks(name, n, seed)
        check_plain(run_whole(eng, t), name, t, dtype, f"{name} {n} tokens")


@pytest.mark.parametrize("name,dtype", PATHS)
@pytest.mark.parametrize("graph", [False, True])
def test_prompt_then_token_by_token(name, dtype, graph):
    eng = engine_for(name, dtype)
    t = toks(name, 150, 21)          # decoded across the page borders at 64 and 128, out of every window and past the kept positions
    check_plain(prompt_then_tokens(eng, t, 60, graph), name, t, dtype)


@pytest.mark.parametrize("name", ["A", "B"])
def test_decoding_from_the_first_token(name):
    eng = engine_for(name, "float32")
    t = toks(name, 80, 8)
    s = eng.cache.open_slot()
    rows = [eng.step([gi.StepEntry(s, [x], [0])]).cpu().numpy() for x in t]
    eng.cache.close_slot(s)
    check_plain(np.concatenate(rows, 0), name, t, "float32")


@pytest.mark.parametrize("name,dtype", PATHS)
def test_portions_of_several_sizes(name, dtype):
    eng = engine_for(name, dtype)
    t = toks(name, 140, 31)
    for cuts in ((2, 4, 66, 130, 140), (63, 64, 65, 128, 140), (1, 3, 5, 7, 140), (20, 40, 41, 43, 110, 140)):
        s = eng.cache.open_slot()
        rows, a = [], 0
        for b in cuts:
            rows.append(eng.step([gi.StepEntry(s, t[a:b], list(range(b - a)))]).cpu().numpy())
            a = b
        eng.cache.close_slot(s)
        check_plain(np.concatenate(rows, 0), name, t, dtype, f"{name} cut at {cuts}")


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_does_not_depend_on_the_cut_or_the_batch(name):
    eng = engine_for(name, "float32")
    t, other = toks(name, 100, 41), toks(name, 20, 42)       # few enough (token, expert) pairs for one kind of expert product
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
        check_plain(np.concatenate(got[i], 0), name, p, dtype, f"{name}: request {i} of the batch")


def test_mixed_step_of_fresh_prompts_and_sequences_under_way():
    """One step holds the second portion of one request and the whole of another: positions count from 0 in each."""
    eng = engine_for("A", "float32")
    a, b = toks("A", 120, 61), toks("A", 40, 62)
    s1, s2 = eng.cache.open_slot(), eng.cache.open_slot()
    r0 = eng.step([gi.StepEntry(s1, a[:50], list(range(50)))]).cpu().numpy()
    r1 = eng.step([gi.StepEntry(s2, b, list(range(40))), gi.StepEntry(s1, a[50:110], list(range(60)))]).cpu().numpy()
    r2 = eng.step([gi.StepEntry(s1, a[110:], list(range(10)))]).cpu().numpy()
    eng.cache.close_slot(s1); eng.cache.close_slot(s2)
    check_plain(np.concatenate([r0, r1[40:], r2], 0), "A", a, "float32", "under way")
    check_plain(r1[:40], "A", b, "float32", "fresh")


# ---- pages and slots given back and used again ---------------------------------------------------------------------
def test_slots_and_pages_used_again():
    """A pool of six pages and two slots: sequences come and go; whoever gets a used slot must find the matrix memory, its
    normalizer and maximum and the convolutions' inputs zero, and must not see the keys the pages held before."""
    eng = engine_for("A", "float32", max_tokens=64 * 6, max_slots=2)
    for round_ in range(3):
        p, q = toks("A", 100 + round_, 40 + round_), toks("A", 70, 50 + round_)
        s1, s2 = eng.cache.open_slot(), eng.cache.open_slot()
        out = eng.step([gi.StepEntry(s1, p, [len(p) - 1]), gi.StepEntry(s2, q, list(range(70)))]).cpu().numpy()
        check(out[0], plain("A", p)[0][-1], "float32", f"round {round_}")
        check(out[1:], plain("A", q)[0], "float32", f"round {round_}")
        run = eng.decoder([s2])
        extra = toks("A", 3, 90 + round_)
        rows = [run.forward(tokens=[x]).cpu().numpy().copy() for x in extra]
        check(np.concatenate(rows, 0), plain("A", q + extra)[0][70:], "float32", f"round {round_}, decoded")
        eng.cache.close_slot(s1)
        eng.cache.close_slot(s2)
    assert eng.cache.free_pages == eng.cache.n_pages


def test_a_windowed_cache_keeps_its_first_pages_and_gives_the_others_back():
    """Windows of at most 70 positions that keep up to 66 first positions, and a recurrence: a sequence of 700 tokens lives in a
    pool of five pages, because pages wholly before every reader's window and after the kept positions are given back; a
    lender keeps what its furthest-looking borrower reads."""
    cfg = model_cfg(64, 120, 2, 2, [
        layer("attention", att(2, 1, 16, 8, 0.4, 9, 66, 8), moe(4, 2, 8, 1.0, 8, 1.0, 1.0)),
        layer("mlstm", mem(2, 8, 8, 6.0)),
        layer("attention", att(4, 1, 16, 8, 0.3, 70, 3, 8, kv_from=0)),
        layer("attention", att(2, 2, 8, 8, 0.5, 33, 0, 4), moe(2, 1, 8, 1.0, 8, 1.0, 1.0)),
    ])
    w = pt.random_weights(cfg, seed=17)
    eng = engine_of(cfg, tensors_of(w, False), "float32", max_tokens=64 * 5, max_slots=1)
    t = np.random.default_rng(61).integers(0, 120, size=700).tolist()
    s = eng.cache.open_slot()
    rows, at = [], 0
    while at < 600:
        rows.append(eng.step([gi.StepEntry(s, t[at:at + 50], list(range(50)))]).cpu().numpy())
        at += 50
    run = eng.decoder([s])
    rows += [run.forward(tokens=[x]).cpu().numpy().copy() for x in t[600:]]          # a long run of one-token steps
    eng.cache.close_slot(s)
    assert eng.cache.free_pages == eng.cache.n_pages
    check(np.concatenate(rows, 0), pt.forward(cfg, w, t), "float32")


# ---- greedy generation through the library's own entry point ---------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype):
    """`LLM.generate` on a model folder: the scheduler cuts prompts into portions of 16 tokens and decodes two requests at a
    time; every greedy token is the plain implementation's, as long as that one's choice is clear."""
    import json
    from ghost_infer_b200.weights.safetensors_io import save_safetensors
    cfg, w, tensors = made("A")
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    save_safetensors(str(folder / "model.safetensors"), tensors)
    llm = gi.LLM(str(folder), dtype=dtype, max_tokens=64 * 16, max_seq_len=512)
    prompts = [toks("A", n, 80 + i) for i, n in enumerate([3, 30, 11, 75])]
    res = llm.generate(prompts, max_new=6, temperature=0.0, stop_token_ids=(), batch_size=2, max_step_tokens=16)
    clear = 1e-3 if dtype == "float32" else 0.2
    for p, r in zip(prompts, res):
        seq = list(p)
        for _ in range(6):
            gaps = []
            logits = pt.forward(cfg, w, seq, gaps=gaps)[-1]
            order = np.argsort(-logits, kind="stable")
            if logits[order[0]] - logits[order[1]] < clear or (dtype != "float32" and np.min(np.stack(gaps)) < 0.01):
                break
            seq.append(int(order[0]))
        want = seq[len(p):]
        assert r.tokens[:len(want)] == want, f"prompt of {len(p)}: {r.tokens} vs {want}"
    assert llm.cache.free_pages == llm.cache.n_pages


# ---- the replay program as a user runs it ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(tmp_path, dtype):
    """`bin/trace_run` on a model folder: requests whole, tails token by token, and unequal batches decoded together."""
    import json
    import os
    import subprocess
    import sys
    from ghost_infer_b200.weights.safetensors_io import save_safetensors
    from test_gpu_trace_run import build_trace
    name = "A" if dtype == "bfloat16" else "B"
    cfg, w, tensors = made(name)
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    save_safetensors(str(folder / "model.safetensors"), tensors)
    reqs, steps = build_trace({"vocab_size": cfg["vocab"]})
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(64 * 8)], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                       text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    assert p.stdout.split("\n")[:len(steps)] == [f"done {i}" for i in range(len(steps))]
    refs = {rid: plain(name, ts) for rid, ts in reqs.items()}
    place, got, want, keep = {}, [], [], []
    for s in steps:
        rows = []
        for e in s["entries"]:
            base = place.get(e["id"], 0)
            rows += [(refs[e["id"][:2]][0][base + k], refs[e["id"][:2]][1][base + k]) for k in e["want"]]
            place[e["id"]] = base + len(e["tokens"])
        f = out / f"{s['step']}.f32"
        if rows:
            got.append(np.fromfile(f, dtype="<f4").reshape(-1, cfg["vocab"]))
            want += [r for r, _ in rows]
            keep += [k for _, k in rows]
        else:
            assert not f.exists()
    check(np.concatenate(got, 0), np.stack(want), dtype, "all steps", np.array(keep))


# ---- schedules drawn at random ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_drawn_schedules(name):
    """One to four requests of 1 to 200 tokens; every step takes some of the live requests and gives each a portion of 1 to 130
    of its next tokens, so a step holds fresh prompts, portions in mid-sequence and single tokens side by side and some
    requests sit a step out; the places whose logits are wanted are drawn too.  32-bit, so that every row must agree."""
    eng = engine_for(name, "float32", max_tokens=64 * 32, max_seq_len=1024)
    rng = np.random.default_rng(sum(map(ord, name)) + 5)
    rows = 0
    for draw in range(5):
        n_req = int(rng.integers(1, 5))
        lens = [int(rng.integers(1, 200)) for _ in range(n_req)]
        seqs = [toks(name, n, int(rng.integers(1 << 30))) for n in lens]
        refs = [plain(name, t)[0] for t in seqs]
        slots = [eng.cache.open_slot() for _ in seqs]
        done = [0] * n_req
        while any(done[i] < lens[i] for i in range(n_req)):
            live = [i for i in range(n_req) if done[i] < lens[i]]
            pick = [i for i in live if rng.random() < 0.7] or [live[0]]
            entries, wants = [], []
            for i in pick:
                n = int(min(lens[i] - done[i], rng.choice([1, 1, 2, 3, 7, 33, 64, 65, 130])))
                w = sorted(set(int(x) for x in rng.integers(0, n, size=int(rng.integers(0, 3))))) or [n - 1]
                entries.append(gi.StepEntry(slots[i], seqs[i][done[i]:done[i] + n], w))
                wants.append((i, done[i], w))
                done[i] += n
            lg = eng.step(entries).cpu().numpy()
            r = 0
            for i, base, w in wants:
                for x in w:
                    check(lg[r:r + 1], refs[i][base + x:base + x + 1], "float32", f"{name} draw {draw}, request {i} of lengths {lens}, place {base + x}")
                    r += 1
            rows += r
        for s in slots:
            eng.cache.close_slot(s)
    assert rows > 50 and eng.cache.free_pages == eng.cache.n_pages
