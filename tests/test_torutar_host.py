"""What the Torutar decoder decides on the host: its configuration, the layers it is built from, the cache and state it asks
for (kept first pages, state of the layer's arrangement beside the mixer's); and the plain implementation's own properties (the
oracle is checked apart from the code it judges)."""
import numpy as np
import pytest
import torch

import plain_torutar as pt
from ghost_infer_b200.cache.sequence_cache import CacheRequest, SequenceCache, StateRequest
from ghost_infer_b200.config import ConfigError, architecture_of, parse_config
from ghost_infer_b200.engine.model import Model

ATT = {"heads": 6, "kv_heads": 3, "dim": 12, "vdim": 20, "scale": 0.3, "mask": {"size": 9, "keep_first": 4}, "rot": {"base": 700.0, "dims": 8}}
LAT = {"heads": 4, "dim": 10, "rot_dim": 6, "vdim": 8, "kv_rank": 14, "q_rank": 18, "scale": 0.2, "rot": {"base": 3000.0, "dims": 6}}
MEM = {"heads": 3, "dim": 8, "vdim": 12, "gate_cap": 9.0}
MOE = {"kind": "moe", "router": {"experts": 5, "top": 2, "scale": 1.5}, "expert": {"ff": 12, "limit": 1.0}, "shared": {"ff": 10, "limit": 2.0}}
CFG = {"architecture": "Torutar", "width": 40, "vocab": 70, "streams": 3, "canon": {"taps": 4}, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
       "layers": [
           {"type": "attention", "mixer": ATT, "mlp": MOE},
           {"type": "mlstm", "mixer": MEM, "mlp": None},
           {"type": "latent_attention", "mixer": LAT, "mlp": MOE},
           {"type": "attention", "mixer": dict(ATT, kv_from=0, mask={"size": 30, "keep_first": 70}, heads=3), "mlp": None},
       ]}


def test_configuration_is_typed_and_checked():
    assert architecture_of(CFG) == "Torutar"
    cfg = parse_config(CFG)
    assert (cfg.width, cfg.vocab_size, cfg.num_hidden_layers, cfg.norm_eps, cfg.streams, cfg.taps, cfg.logit_scale) == (40, 70, 4, 1e-5, 3, 4, 0.5)
    assert cfg.layers[1].mlp is None and cfg.layers[3].mixer.kv_from == 0 and cfg.layers[0].mixer.window == 9 and cfg.layers[0].mixer.keep_first == 4
    assert cfg.layers[2].mixer.kv_rank == 14 and cfg.layers[1].mixer.gate_cap == 9.0 and cfg.layers[0].mlp.route_scale == 1.5
    first = lambda **kw: dict(CFG["layers"][0], **kw)
    for bad in (dict(CFG, layers=[]), dict(CFG, layers=[first(type="lightning")]),
                dict(CFG, layers=[first(mixer=dict(ATT, kv_heads=4))]),                               # 6 heads over 4
                dict(CFG, layers=[first(mixer=dict(ATT, rot={"base": 10.0, "dims": 14}))]),           # more numbers turn than a head has
                dict(CFG, layers=[first(mixer=dict(ATT, rot={"base": 10.0, "dims": 5}))]),
                dict(CFG, layers=[first(mixer={k: v for k, v in ATT.items() if k != "scale"})]),
                dict(CFG, layers=[first(mlp={"kind": "dense", "ff": 8})]),
                dict(CFG, layers=[first(mlp=dict(MOE, router={"experts": 2, "top": 3, "scale": 1.0}))]),
                dict(CFG, layers=[first(), first(mixer=dict(ATT, kv_from=1))]),                       # itself
                dict(CFG, layers=[first(), first(mixer=dict(ATT, kv_from=0, vdim=8))]),               # other sizes than the lender's
                dict(CFG, layers=[first(), first(mixer=dict(ATT, kv_from=0)), first(mixer=dict(ATT, kv_from=1))]),   # a borrower lends nothing
                dict(CFG, layers=[CFG["layers"][1], first(mixer=dict(ATT, kv_from=0))]),
                dict(CFG, layers=[{"type": "mlstm", "mixer": dict(MEM, gate_cap=0.0), "mlp": None}]),
                dict(CFG, layers=[{"type": "latent_attention", "mixer": dict(LAT, rot={"base": 5.0, "dims": 8}), "mlp": None}]),
                {k: v for k, v in CFG.items() if k != "streams"}, {k: v for k, v in CFG.items() if k != "norm"}):
        with pytest.raises(ConfigError):
            parse_config(bad)


def test_layers_are_put_together_from_the_configuration():
    model = Model.from_config_dict(CFG)
    assert model.spec.streams == 3 and model.spec.embedding_norm is not None and model.head.scale == 0.5
    assert [(e.layer, e.memory_of) for e in model.spec.schedule] == [(0, None), (1, None), (2, None), (3, 0)]
    assert [type(l.block).__name__ for l in model.layers] == ["HyperConnections"] * 4
    assert [type(l.block.mixer).__name__ for l in model.layers] == ["HeadNormedAttention", "MLstm", "LatentAttention", "HeadNormedAttention"]
    assert [type(l.block.ffn).__name__ for l in model.layers] == ["ShareRoutedExperts", "NoneType", "ShareRoutedExperts", "NoneType"]
    assert list(model.layers[0].block.extra) == ["connect1", "connect2"] and list(model.layers[1].block.extra) == ["connect1"]
    names = {w.name: tuple(w.shape) for w in model.weight_manifest()}
    for name, shape in {"embed": (70, 40), "embed.norm": (40,), "final.norm": (40,), "head": (70, 40), "l0.norm2": (40,),
                        "l0.hc1.in": (3,), "l0.hc2.mix": (3, 3), "l1.hc1.out": (3,), "l0.canon1": (40, 4), "l2.rg2": (40, 40),
                        "l2.rg2.b": (40,), "l0.mix.q": (72, 40), "l0.mix.q.b": (72,), "l0.mix.q.norm": (12,), "l0.mix.k.norm": (12,),
                        "l0.mix.v": (60, 40), "l0.mix.sink": (6,), "l0.mix.g": (6, 40), "l0.mix.o": (40, 120), "l0.mix.o.b": (40,),
                        "l3.mix.q": (36, 40), "l3.mix.g": (3, 40), "l1.mix.i": (3, 40), "l1.mix.f.b": (3,), "l1.mix.norm": (36,),
                        "l1.mix.g": (36, 40), "l2.mix.dkv": (20, 40), "l2.mix.uq": (64, 18), "l2.mix.g": (32, 40),
                        "l0.mlp.router": (5, 40), "l0.mlp.correction": (5,), "l0.mlp.e4.down": (40, 12), "l0.mlp.shared.up": (10, 40)}.items():
        assert names[name] == shape, name
    for absent in ("l3.mix.k", "l3.mix.v", "l3.mix.k.norm", "l1.norm2", "l1.hc2.in", "l1.canon2", "l3.rg2"):
        assert absent not in names
    assert set(names) == set(pt.random_weights(CFG, 0))


def test_memory_asked_for():
    """A lender's cache keeps what the borrower that looks furthest back reads and the most first positions anyone keeps; every
    layer's arrangement keeps the last taps - 1 inputs of both sublayers, a borrower too; the matrix memory keeps S, n and m."""
    model = Model.from_config_dict(CFG)
    reqs = model.memory_requests()
    conv = StateRequest((2, 3 * 40), torch.float32)
    assert reqs[0] == (0, CacheRequest("window", 3, 12, 30, 20, keep_first=70), None, None, conv)
    assert reqs[1] == (1, None, StateRequest((3 * 8 * 12 + 3 * 9,), torch.float32), None, conv)
    assert reqs[2] == (2, CacheRequest("full", 1, 20, None, 14, values_in_keys=True), None, None, conv)
    assert reqs[3] == (3, None, None, 0, conv)
    one_tap = Model.from_config_dict(dict(CFG, canon={"taps": 1}))
    assert all(r[4] is None for r in one_tap.memory_requests())
    with pytest.raises(ValueError):
        CacheRequest("full", 1, 8, None, keep_first=3)


def test_a_window_cache_keeps_the_pages_of_its_first_positions():
    reqs = [(0, CacheRequest("window", 1, 8, 70, keep_first=65), None, None, StateRequest((2, 6), torch.float32)),
            (1, None, None, 0, StateRequest((2, 6), torch.float32))]
    cache = SequenceCache(reqs, max_tokens=64 * 6, max_slots=2, max_seq_len=4096, dtype=torch.float32)
    s = cache.open_slot()
    for n in list(range(50, 1500, 50)) + [1501, 1502]:       # portions of 50 tokens, then single ones
        cache.reserve([(s, n)])
        cache.commit(s, n)
        pages = cache.groups[0].pages[s]
        live = [i for i, p in enumerate(pages) if p != 0]
        first_needed = (n - 70 + 1) // 64
        assert live[:2] == [0, 1][:len(pages)] and all(i >= first_needed for i in live[2:]) and pages[n // 64 if n % 64 else n // 64 - 1] != 0, (n, live)
    assert cache.free_pages >= cache.n_pages - 5
    own, borrowed = cache.memory(0), cache.memory(1)
    assert own.block_state is not None and borrowed.block_state is not None and own.block_state.data_ptr() != borrowed.block_state.data_ptr()
    assert borrowed.k is own.k or borrowed.k.data_ptr() == own.k.data_ptr()
    assert not borrowed.writes and own.writes
    own.block_state[s] = 3.0
    cache.close_slot(s)
    assert cache.free_pages == cache.n_pages
    s2 = cache.open_slot()
    assert s2 == s and float(cache.memory(0).block_state[s2].abs().max()) == 0.0      # a used slot starts from zero


# ---- the plain implementation by itself --------------------------------------------------------------------------------
def test_plain_matrix_memory_carries_its_state_over_a_cut():
    w = pt.random_weights(CFG, seed=3)
    h = np.random.default_rng(0).standard_normal((30, 40))
    whole, _ = pt.mlstm(h, w, "l1.mix.", MEM, 1e-5)
    a, st = pt.mlstm(h[:11], w, "l1.mix.", MEM, 1e-5)
    b, _ = pt.mlstm(h[11:], w, "l1.mix.", MEM, 1e-5, st)
    assert np.allclose(np.concatenate([a, b]), whole, rtol=1e-12, atol=1e-12)


def test_plain_window_and_kept_positions():
    ok = pt.visible(12, 3, 2)
    assert ok[11].tolist() == [True, True] + [False] * 7 + [True] * 3
    assert ok[2].tolist() == [True, True, True] + [False] * 9
    assert pt.visible(5).tolist() == np.tril(np.ones((5, 5), dtype=bool)).tolist()


def test_plain_router_weights_and_choice():
    w = {"p.router": np.array([[1.0, 0.0], [0.0, 1.0], [0.0, 0.0]]), "p.correction": np.array([0.0, 0.0, 10.0])}
    ids, wt = pt.route(np.array([[2.0, 1.0]]), w, "p.", {"top": 2, "scale": 3.0})
    s = np.exp([2.0, 1.0, 0.0]) / np.exp([2.0, 1.0, 0.0]).sum()
    assert ids.tolist() == [[2, 0]]                                  # the correction decides the choice ...
    assert np.allclose(wt[0], np.array([s[2], s[0]]) / (s[2] + s[0]) * 3.0)      # ... and does not enter the weights


def test_plain_input_convolution_and_rotation():
    h = np.arange(12.0).reshape(6, 2)
    k = np.array([[0.5, 0.25, 2.0], [0.0, 0.0, 0.0]])
    out = pt.causal_conv_added(h, k)
    assert np.allclose(out[:, 1], h[:, 1])
    assert np.allclose(out[3, 0], h[3, 0] + 0.5 * h[1, 0] + 0.25 * h[2, 0] + 2.0 * h[3, 0]) and np.allclose(out[0, 0], 3.0 * h[0, 0])
    x = np.random.default_rng(1).standard_normal((4, 2, 8))
    for layout in ("half", "adjacent"):
        r = pt.rotate(x, [0, 1, 5, 9], 4, 100.0, layout)
        assert np.allclose(r[0], x[0]) and np.allclose(r[..., 4:], x[..., 4:]) and np.allclose((r ** 2).sum(-1), (x ** 2).sum(-1))
    a = pt.rotate(x, [3] * 4, 4, 100.0, "half")
    assert np.allclose(a[..., 0], x[..., 0] * np.cos(3.0) - x[..., 2] * np.sin(3.0))
    b = pt.rotate(x, [3] * 4, 4, 100.0, "adjacent")
    assert np.allclose(b[..., 1], x[..., 1] * np.cos(3.0) + x[..., 0] * np.sin(3.0))
