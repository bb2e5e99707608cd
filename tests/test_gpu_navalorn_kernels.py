"""Each kernel behind the Navalorn decoder's parts alone, against the same operation written out in 64-bit torch, at
sizes that are not an engine's: the layer norm; bias and squared relu; the latent's row (two RMS norms, the turn of the
shared key part in neighbouring pairs with stretched frequencies, the write into shuffled pages); one small product per
head; attention over one shared row per position (the plain kernels in both precisions and the tensor-core kernel: prompt
rows after a cached prefix in a ragged batch, one-token rows cut into slices, few heads and many, values wider than one
warp holds, a far key made to stand out, pages shuffled and unused rows poisoned); the router with sigmoid weights,
rows gathered with their weights on, the ungated experts' products and the unweighted sum."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from ghost_infer_b200.cache.sequence_cache import LayerMemory
from ghost_infer_b200.kernels import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)


def step_of(q_lens, pos0, slots):
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    positions = np.concatenate([np.arange(p, p + n) for p, n in zip(pos0, q_lens)]).astype(np.int32)
    token_slots = np.concatenate([np.full(n, s) for s, n in zip(slots, q_lens)]).astype(np.int32)
    t = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
    return SimpleNamespace(n_seqs=len(q_lens), n_tokens=int(sum(q_lens)), max_q_len=int(max(q_lens)),
                           max_kv_len=int(max(p + n for p, n in zip(pos0, q_lens))), is_decode=max(q_lens) == 1,
                           cu_seqlens=t(cu), positions=t(positions), token_slots=t(token_slots), seq_slots=t(slots),
                           seq_pos0=t(pos0), seq_lens=t([p + n for p, n in zip(pos0, q_lens)]), sm_count=148)


def paged_rows(dense, lens, seed=0):
    """Dense [B, S, d] rows into shuffled pages [pages, 1, 64, d]; unused rows and pages hold NaN."""
    B, S, d = dense.shape
    per = (S + 63) // 64
    total = B * per + 4
    order = (torch.randperm(total - 1, generator=torch.Generator().manual_seed(seed)) + 1).tolist()
    kc = torch.full((total, 1, 64, d), float("nan"), dtype=dense.dtype, device=DEV)
    kc[0] = 0
    bt = torch.zeros((B, per), dtype=torch.int32)
    it = iter(order)
    for b in range(B):
        for p in range((lens[b] + 63) // 64):
            page = next(it)
            bt[b, p] = page
            n = min(64, lens[b] - p * 64)
            kc[page, 0, :n] = dense[b, p * 64:p * 64 + n]
    return kc, bt.to(DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,width", [(5, 48), (3, 2050), (2, 4100)])
def test_layernorm(dtype, rows, width):
    g = torch.Generator(device=DEV).manual_seed(rows * width)
    x = torch.randn((rows, width), device=DEV, generator=g) * 3 + 1.5
    w = (torch.randn((width,), device=DEV, generator=g) * 0.3 + 1).to(DT[dtype])
    got = ops.layernorm(x, w, 1e-3, DT[dtype])
    xd, wd = x.double(), w.double()
    mu = xd.mean(-1, keepdim=True)
    ref = (xd - mu) / torch.sqrt(((xd - mu) ** 2).mean(-1, keepdim=True) + 1e-3) * wd
    torch.testing.assert_close(got.double(), ref, **tol(dtype))
    pick = torch.tensor([rows - 1, 0, rows - 1], dtype=torch.int32, device=DEV)
    torch.testing.assert_close(ops.layernorm(x, w, 1e-3, torch.float32, rows=pick).double(), ref[pick.long()], rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_bias_and_squared_relu(dtype):
    g = torch.Generator(device=DEV).manual_seed(3)
    a = torch.randn((7, 44), device=DEV, generator=g).to(DT[dtype])
    b = torch.randn((44,), device=DEV, generator=g).to(DT[dtype])
    rb = torch.randn((20,), device=DEV, generator=g).to(DT[dtype])
    res = torch.randn((7, 20), device=DEV, generator=g)
    before = res.clone()
    got = ops.bias_act(a, b, "relu2", res, rb)
    torch.testing.assert_close(got.double(), torch.relu(a.double() + b.double()) ** 2, **tol(dtype))
    torch.testing.assert_close(res.double(), before.double() + rb.double(), rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(ops.bias_act(a[:, :12], None, None).double(), a[:, :12].double(), rtol=0, atol=0)


def frequencies(dims, base, factor, original, fast, slow):
    idx = lambda turns: dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))
    lo, hi = max(math.floor(idx(fast)), 0), min(math.ceil(idx(slow)), dims - 1)
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def test_yarn_frequencies_against_hand_values():
    """Eight numbers turn, base 100, 64 original positions stretched 4 times, ramp between 4 turns and 1 turn: the pair
    index that makes t turns is 8 ln(64 / (2 pi t)) / (2 ln 100) = 0.812 (t = 4) and 2.016 (t = 1), so lo = 0, hi = 3, and
    the ramp over pairs 0..3 is 0, 1/3, 2/3, 1."""
    from ghost_infer_b200.parts.rope import Rotary, rotary_inv_freq
    sc = {"rope_type": "yarn", "factor": 4.0, "original": 64, "fast": 4.0, "slow": 1.0}
    got = rotary_inv_freq(8, 100.0, sc).double().tolist()
    plain = [100.0 ** (-2 * i / 8) for i in range(4)]
    want = [plain[0], plain[1] * (1 / 4 * 1 / 3 + 2 / 3), plain[2] * (1 / 4 * 2 / 3 + 1 / 3), plain[3] / 4]
    assert np.allclose(got, want, rtol=1e-6)
    assert abs(Rotary({"head_dim": 8, "theta": 100.0, "pairing": "adjacent", "scaling": sc}).magnitude - (0.1 * math.log(4) + 1)) < 1e-12


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rq,r,dr,rot", [(24, 40, 8, 8), (56, 72, 24, 16), (8, 16, 6, 4)])
def test_latent_rows(dtype, rq, r, dr, rot):
    dt = DT[dtype]
    g = torch.Generator(device=DEV).manual_seed(rq + r)
    q_lens, pos0, slots = [70, 3, 1], [0, 130, 63], [2, 0, 1]
    st = step_of(q_lens, pos0, slots)
    T = st.n_tokens
    rows = torch.randn((T, rq + r + dr), device=DEV, generator=g).to(dt)
    wq = (torch.randn((rq,), device=DEV, generator=g) * 0.2 + 1).to(dt)
    wc = (torch.randn((r,), device=DEV, generator=g) * 0.2 + 1).to(dt)
    freqs, mag = frequencies(rot, 1000.0, 8.0, 32, 8.0, 1.0)
    inv = torch.tensor(freqs, dtype=torch.float64).float().to(DEV)
    table = ops.rope_table(st.positions, inv, mag)
    kc = torch.full((8, 1, 64, r + dr), float("nan"), dtype=dt, device=DEV)
    bt = torch.tensor([[5, 2, 7], [1, 0, 0], [3, 6, 0]], dtype=torch.int32, device=DEV)     # slot -> pages
    mem = LayerMemory(kc, None, bt, None, True, None)
    cq = ops.latent_prepare(rows, wq, wc, 1e-4, table, rot, st.positions, st.token_slots, mem, rq, r, dr)
    x = rows.double()
    rms = lambda v, w: v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-4) * w.double()
    torch.testing.assert_close(cq.double(), rms(x[:, :rq], wq), **tol(dtype))
    c = rms(x[:, rq:rq + r], wc)
    kr = x[:, rq + r:].clone()
    ang = st.positions.double()[:, None] * torch.tensor(freqs, dtype=torch.float64, device=DEV)[None, :]
    co, si = torch.cos(ang) * mag, torch.sin(ang) * mag
    u, v = kr[:, 0:rot:2].clone(), kr[:, 1:rot:2].clone()
    kr[:, 0:rot:2], kr[:, 1:rot:2] = u * co - v * si, v * co + u * si
    want = torch.cat([c, kr], dim=1)
    pos, sl = st.positions.tolist(), st.token_slots.tolist()
    got = torch.stack([kc[bt[sl[t], pos[t] // 64], 0, pos[t] % 64] for t in range(T)])
    torch.testing.assert_close(got.double(), want, **tol(dtype))
    # nothing else was written
    written = {(int(bt[sl[t], pos[t] // 64]), pos[t] % 64) for t in range(T)}
    assert int((~torch.isnan(kc[:, 0, :, 0])).sum()) == len(written)
    # the queries' rotated parts, into rows of another layout
    H, dn = 3, 10
    q = torch.randn((T, H * (dn + dr)), device=DEV, generator=g).to(dt)
    qa = torch.zeros((T, H * (r + dr)), dtype=dt, device=DEV)
    ops.latent_query_rot(qa, q, table, rot, H, dn, dr, r)
    qr = q.double().view(T, H, dn + dr)[:, :, dn:].clone()
    u, v = qr[:, :, 0:rot:2].clone(), qr[:, :, 1:rot:2].clone()
    qr[:, :, 0:rot:2], qr[:, :, 1:rot:2] = u * co[:, None] - v * si[:, None], v * co[:, None] + u * si[:, None]
    torch.testing.assert_close(qa.double().view(T, H, r + dr)[:, :, r:], qr, **tol(dtype))
    assert float(qa.view(T, H, r + dr)[:, :, :r].abs().max()) == 0.0


@pytest.mark.parametrize("dtype,tc", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("M,H,N,K,pad", [(5, 3, 40, 24, 6), (130, 2, 72, 100, 6), (64, 5, 8, 16, 6), (1, 16, 128, 64, 6),
                                         (5, 3, 40, 24, 8), (1, 16, 128, 64, 8), (19, 2, 33, 512, 0),       # few rows, 16-byte rows
                                         (130, 2, 72, 104, 8), (40, 3, 100, 256, 8), (300, 2, 512, 128, 64)])  # many rows, 16-byte rows
def test_one_product_per_head(dtype, tc, M, H, N, K, pad):
    dt = DT[dtype]
    g = torch.Generator(device=DEV).manual_seed(M + N)
    a = torch.randn((M, H * (K + pad)), device=DEV, generator=g).to(dt)      # a head's numbers start every K + pad
    w = (torch.randn((H, N, K), device=DEV, generator=g) * 0.2).to(dt)
    out = torch.full((M, H * (N + 2)), 7.0, dtype=dt, device=DEV)
    old = ops.TUNE["bmm_heads_tc"]
    ops.TUNE["bmm_heads_tc"] = tc
    try:
        ops.bmm_heads(out, N + 2, a, K + pad, w, N, K)
    finally:
        ops.TUNE["bmm_heads_tc"] = old
    ref = torch.einsum("mhk,hnk->mhn", a.double().view(M, H, K + pad)[:, :, :K], w.double())
    got = out.double().view(M, H, N + 2)
    torch.testing.assert_close(got[:, :, :N], ref, **tol(dtype))
    assert float((got[:, :, N:] - 7.0).abs().max()) == 0.0          # nothing past a head's columns is touched


def latent_attention_reference(qa, rows, pos0, q_lens, H, r, scale):
    """qa [T, H, dk], rows [B, S, dk] in 64-bit; returns [T, H * r]."""
    out, at = [], 0
    for b, (p0, n) in enumerate(zip(pos0, q_lens)):
        for i in range(n):
            k = rows[b, :p0 + i + 1]
            s = (qa[at + i] @ k.T) * scale                         # [H, keys]
            p = torch.softmax(s, dim=-1)
            out.append((p @ k[:, :r]).reshape(-1))
        at += n
    return torch.stack(out)


CASES = [  # heads, latent, rotary part
    (3, 40, 8), (5, 64, 16), (20, 128, 32), (16, 512, 64), (70, 24, 8), (2, 36, 4)]


@pytest.mark.parametrize("dtype,tc", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("H,r,dr", CASES)
def test_latent_attention_prompt_rows(dtype, tc, H, r, dr):
    if tc and not ops.attn_latent_tc_ok(torch.bfloat16, r, dr):
        pytest.skip("sizes the tensor-core kernel leaves to the plain one")
    dt = DT[dtype]
    dk = r + dr
    g = torch.Generator(device=DEV).manual_seed(H * r)
    q_lens, pos0, slots = [67, 1, 130, 5], [0, 64, 190, 63], [1, 3, 0, 2]
    lens = [p + n for p, n in zip(pos0, q_lens)]
    S = max(lens)
    dense = (torch.randn((4, S, dk), device=DEV, generator=g) * 0.5).to(dt)
    st = step_of(q_lens, pos0, list(range(4)))
    qa = (torch.randn((st.n_tokens, H * dk), device=DEV, generator=g) * 0.5).to(dt)
    # one far key made to stand out for one row: the last token of the third sequence looks at position 2
    dense[2, 2] = dense[2, 2] * 0 + 1.0
    far_row = sum(q_lens[:3]) - 1
    qa.view(-1, H, dk)[far_row, 0] = 2.0
    kc, bt = paged_rows(dense, lens, seed=H)
    order = torch.tensor(slots, device=DEV)
    bt_by_slot = torch.zeros_like(bt)
    bt_by_slot[order] = bt
    st = step_of(q_lens, pos0, slots)
    mem = LayerMemory(kc, None, bt_by_slot, None, True, None)
    out = torch.full((st.n_tokens, H * r), float("nan"), dtype=dt, device=DEV)
    old = ops.TUNE["attn_latent_tc"]
    ops.TUNE["attn_latent_tc"] = tc
    try:
        ops.attention_latent(qa, mem, st, H, r, dr, 0.3, out)
    finally:
        ops.TUNE["attn_latent_tc"] = old
    ref = latent_attention_reference(qa.double().view(-1, H, dk), dense.double(), pos0, q_lens, H, r, 0.3)
    torch.testing.assert_close(out.double(), ref, **tol(dtype))
    # the row that looks far back is mostly that key's latent
    assert float((out.double().view(-1, H, r)[far_row, 0] - 1.0).abs().max()) < 0.2


@pytest.mark.parametrize("dtype,tc", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("H,r,dr", CASES)
@pytest.mark.parametrize("splits", [1, 3])
def test_latent_attention_one_token_rows(dtype, tc, H, r, dr, splits):
    if tc and not ops.attn_latent_tc_ok(torch.bfloat16, r, dr):
        pytest.skip("sizes the tensor-core kernel leaves to the plain one")
    dt = DT[dtype]
    dk = r + dr
    g = torch.Generator(device=DEV).manual_seed(H + r)
    lens = [1, 64, 65, 300, 129]
    slots = [4, 0, 3, 1, 2]
    dense = (torch.randn((5, max(lens), dk), device=DEV, generator=g) * 0.5).to(dt)
    dense[3, 1] = dense[3, 1] * 0 + 1.0               # a key 298 positions back that one head looks for
    qa = (torch.randn((5, H * dk), device=DEV, generator=g) * 0.5).to(dt)
    qa.view(5, H, dk)[3, H - 1] = 2.0
    kc, bt = paged_rows(dense, lens, seed=r)
    bt_by_slot = torch.zeros_like(bt)
    bt_by_slot[torch.tensor(slots, device=DEV)] = bt
    st = step_of([1] * 5, [n - 1 for n in lens], slots)
    mem = LayerMemory(kc, None, bt_by_slot, None, True, None)
    out = torch.full((5, H * r), float("nan"), dtype=dt, device=DEV)
    old = ops.TUNE["attn_latent_tc"]
    ops.TUNE["attn_latent_tc"] = tc
    try:
        if tc:
            plan = ("tensor cores", splits, 0)
        else:
            plan = ("plain", splits, 0) if splits > 1 else ops.attn_latent_decode_plan(5, max(lens), 148, H, r, dr, dt)
        ops.attention_latent(qa, mem, st, H, r, dr, 0.25, out, plan=plan)
    finally:
        ops.TUNE["attn_latent_tc"] = old
    ref = latent_attention_reference(qa.double().view(-1, H, dk), dense.double(), [n - 1 for n in lens], [1] * 5, H, r, 0.25)
    torch.testing.assert_close(out.double(), ref, **tol(dtype))
    assert float((out.double().view(5, H, r)[3, H - 1] - 1.0).abs().max()) < 0.2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tokens,experts,top", [(6, 5, 1), (9, 12, 3), (700, 4, 2)])
def test_scored_experts_pieces(dtype, tokens, experts, top):
    dt = DT[dtype]
    width, ff = 48, 24
    g = torch.Generator(device=DEV).manual_seed(tokens)
    h = torch.randn((tokens, width), device=DEV, generator=g).to(dt)
    wr = (torch.randn((experts, width), device=DEV, generator=g) * 0.3).to(dt)
    ids, wts, _ = ops.moe_route(h, wr, top, None, scores="sigmoid")
    z = h.double() @ wr.double().T
    want_ids = torch.argsort(-z, dim=-1, stable=True)[:, :top]
    assert torch.equal(ids.long(), want_ids)
    torch.testing.assert_close(wts.double(), torch.sigmoid(torch.gather(z, 1, want_ids)), rtol=1e-5, atol=1e-6)
    offsets, perm, inv = ops.moe_plan(ids, experts)
    rows = ops.moe_gather_rows(h, perm, top, wts.view(-1))
    src = (perm // top).long()
    scaled = (h.double()[src] * wts.view(-1).double()[perm.long()][:, None])
    torch.testing.assert_close(rows.double(), scaled, **tol(dtype))
    w_up = (torch.randn((experts, ff, width), device=DEV, generator=g) * 0.2).to(dt)
    w_down = (torch.randn((experts, width, ff), device=DEV, generator=g) * 0.2).to(dt)
    hidden = ops.moe_rows_product(rows, w_up, offsets, act="relu2")
    which = ids.view(-1).long()[perm.long()]                            # the expert of every sorted row
    ref_hidden = torch.relu(torch.einsum("rk,rnk->rn", rows.double(), w_up.double()[which])) ** 2
    torch.testing.assert_close(hidden.double(), ref_hidden, **tol(dtype))
    down = ops.moe_rows_product(hidden, w_down, offsets)
    ref_down = torch.einsum("rk,rnk->rn", hidden.double(), w_down.double()[which])
    torch.testing.assert_close(down.double(), ref_down, rtol=2e-4, atol=2e-4)
    res = torch.randn((tokens, width), device=DEV, generator=g)
    before = res.double().clone()
    ops.moe_combine(res, down, inv, None)
    want = before + down.double()[inv.long()].view(tokens, top, width).sum(1)
    torch.testing.assert_close(res.double(), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("rows,n,k,with_bias", [(70, 136, 96, True), (300, 264, 128, False), (65, 8, 8, True)])
def test_squared_relu_in_the_product_epilogue(rows, n, k, with_bias):
    g = torch.Generator(device=DEV).manual_seed(rows)
    h = torch.randn((rows, k), device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn((n, k), device=DEV, generator=g) * 0.2).to(torch.bfloat16)
    b = torch.randn((n,), device=DEV, generator=g).to(torch.bfloat16) if with_bias else None
    got = ops.linear_act(h, w, b, "relu2")
    ref = torch.relu(h.double() @ w.double().T + (b.double() if with_bias else 0.0)) ** 2
    torch.testing.assert_close(got.double(), ref, rtol=2e-2, atol=2e-2)
    few = ops.linear_act(h[:9], w, b, "relu2")                     # few rows: product, then bias and activation
    torch.testing.assert_close(few.double(), ref[:9], rtol=2e-2, atol=2e-2)
    res = torch.randn((rows, 12), device=DEV, generator=g)
    before = res.clone()
    rb = torch.randn((12,), device=DEV, generator=g).to(torch.bfloat16)
    ops.add_row_bias(res, rb)
    torch.testing.assert_close(res.double(), before.double() + rb.double(), rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("rows,n,k", [(70, 136, 96), (300, 264, 128), (65, 8, 8), (129, 520, 72)])
def test_exact_gelu_in_the_product_epilogue(rows, n, k):
    g = torch.Generator(device=DEV).manual_seed(rows + 1)
    h = torch.randn((rows, k), device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn((n, k), device=DEV, generator=g) * 0.3).to(torch.bfloat16)
    z = h.double() @ w.double().T
    ref = 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))
    got = ops.linear_act(h, w, None, "gelu")                       # many rows: the activation on the product's 32-bit sums
    assert got.dtype == torch.bfloat16 and tuple(got.shape) == (rows, n)
    torch.testing.assert_close(got.double(), ref, rtol=1e-2, atol=1e-2)
    few = ops.linear_act(h[:9], w, None, "gelu")                   # few rows: product, then the activation
    torch.testing.assert_close(few.double(), ref[:9], rtol=2e-2, atol=2e-2)
    with pytest.raises(ops.KernelError):
        ops.linear_act(h, w, torch.zeros((n,), device=DEV, dtype=torch.bfloat16), "gelu")


def test_ungated_experts_stretch_by_stretch():
    experts, width, ff = 5, 64, 40
    g = torch.Generator(device=DEV).manual_seed(1)
    counts = [130, 0, 7, 64, 200]
    offs = [0] + np.cumsum(counts).tolist()
    rows = torch.randn((offs[-1], width), device=DEV, generator=g).to(torch.bfloat16)
    w_up = (torch.randn((experts, ff, width), device=DEV, generator=g) * 0.2).to(torch.bfloat16)
    w_down = (torch.randn((experts, width, ff), device=DEV, generator=g) * 0.2).to(torch.bfloat16)
    got = ops.moe_experts_by_expert_ungated(rows, w_up, w_down, offs)
    for e in range(experts):
        lo, hi = offs[e], offs[e + 1]
        hid = (torch.relu(rows[lo:hi].double() @ w_up[e].double().T) ** 2).to(torch.bfloat16).double()
        torch.testing.assert_close(got[lo:hi].double(), hid @ w_down[e].double().T, rtol=2e-2, atol=2e-2)
