"""What the Nuzinex decoder decides on the host: its configuration, the layers it is built from, the cache and state it
asks for; and the plain implementation's own properties (the oracle is checked apart from the code it judges)."""
import json
import math

import numpy as np
import pytest
import torch

import plain_nuzinex as pz
from ghost_infer_b200.cache.sequence_cache import CacheRequest, StateRequest
from ghost_infer_b200.config import ConfigError, architecture_of, parse_config
from ghost_infer_b200.engine.model import Model

ATT = {"heads": 6, "kv_heads": 3, "dim": 12, "vdim": 20, "scale": 0.3, "mask": {"size": 9}, "rot": {"base": 700.0, "dims": 8}}
LEFT = {"heads": 4, "kv_heads": 1, "dim": 16, "vdim": 8, "scale": 0.2, "rot": {"base": 3000.0, "dims": 16}}
RIGHT = {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 10, "conv": 4}
LIGHT = {"heads": 3, "dim": 8, "vdim": 12, "decay": [0.5, 0.9, 1.0]}
CFG = {"architecture": "Nuzinex", "width": 40, "vocab": 70, "norm": {"eps": 1e-5}, "token_side": {"dim": 6}, "layers": [
    {"type": "attention", "mixer": ATT, "mlp": {"kind": "dense", "ff": 56}},
    {"type": "lightning", "mixer": LIGHT, "mlp": None},
    {"type": "parallel", "mixer": {"left": LEFT, "right": RIGHT, "left_scale": 0.7, "right_scale": 1.4}, "mlp": {"kind": "dense", "ff": 24}},
    {"type": "attention", "mixer": dict(ATT, kv_from=0, mask={"size": 30}, heads=3), "mlp": None},
]}


def test_configuration_is_typed_and_checked():
    assert architecture_of(CFG) == "Nuzinex"
    cfg = parse_config(CFG)
    assert cfg.width == 40 and cfg.vocab_size == 70 and cfg.num_hidden_layers == 4 and cfg.norm_eps == 1e-5 and cfg.side_dim == 6
    assert cfg.layers[1].mlp is None and cfg.layers[3].mixer.kv_from == 0 and cfg.layers[0].mixer.window == 9
    assert cfg.layers[2].mixer.right.conv == 4 and cfg.layers[2].mixer.left.window is None and cfg.layers[1].mixer.decay == (0.5, 0.9, 1.0)
    first = lambda **kw: dict(CFG["layers"][0], **kw)
    par = lambda **kw: {"type": "parallel", "mixer": dict(CFG["layers"][2]["mixer"], **kw), "mlp": None}
    for bad in (dict(CFG, layers=[]), dict(CFG, layers=[first(type="latent_attention")]),
                dict(CFG, layers=[first(mixer=dict(ATT, kv_heads=4))]),                               # 6 heads over 4
                dict(CFG, layers=[first(mixer=dict(ATT, rot={"base": 10.0, "dims": 14}))]),           # more numbers turn than a head has
                dict(CFG, layers=[first(mixer=dict(ATT, rot={"base": 10.0, "dims": 5}))]),
                dict(CFG, layers=[first(mixer={k: v for k, v in ATT.items() if k != "scale"})]),
                dict(CFG, layers=[first(mlp={"kind": "gated", "ff": 8})]),
                dict(CFG, layers=[first(), first(mixer=dict(ATT, kv_from=1))]),                       # itself
                dict(CFG, layers=[first(), first(mixer=dict(ATT, kv_from=0, vdim=8))]),               # other sizes than the lender's
                dict(CFG, layers=[first(), first(mixer=dict(ATT, kv_from=0)), first(mixer=dict(ATT, kv_from=1))]),   # a borrower lends nothing
                dict(CFG, layers=[CFG["layers"][1], first(mixer=dict(ATT, kv_from=0))]),
                dict(CFG, layers=[{"type": "lightning", "mixer": dict(LIGHT, decay=[0.5]), "mlp": None}]),
                dict(CFG, layers=[par(right=dict(RIGHT, kv_heads=3))]),
                dict(CFG, layers=[par(right={k: v for k, v in RIGHT.items() if k != "conv"})]),
                {k: v for k, v in CFG.items() if k != "token_side"}, {k: v for k, v in CFG.items() if k != "norm"}):
        with pytest.raises(ConfigError):
            parse_config(bad)


def test_layers_are_put_together_from_the_configuration():
    model = Model.from_config_dict(CFG)
    assert [(e.layer, e.memory_of) for e in model.spec.schedule] == [(0, None), (1, None), (2, None), (3, 0)]
    assert [type(l.block).__name__ for l in model.layers] == ["ResidualPostNorm"] * 4
    assert [type(l.block.mixer).__name__ for l in model.layers] == ["NormedAttention", "DecayedLinearAttention", "ParallelMixers", "NormedAttention"]
    assert [type(l.block.ffn).__name__ for l in model.layers] == ["Mlp", "NoneType", "Mlp", "NoneType"]
    assert list(model.layers[0].block.extra) == ["mixer_scale", "ffn_scale", "after_token_side"]
    assert list(model.layers[1].block.extra) == ["mixer_scale", "after_token_side"]
    names = {w.name: tuple(w.shape) for w in model.weight_manifest()}
    assert set(names) == set(pz.random_weights(CFG))
    assert names["l0.mix.q"] == (72, 40) and names["l0.mix.k"] == (36, 40) and names["l0.mix.v"] == (60, 40) and names["l0.mix.o"] == (40, 120)
    assert names["l0.mix.q.norm"] == (72,) and names["l0.mix.k.norm"] == (36,) and names["l0.mix.v.b"] == (60,)
    assert names["l3.mix.q"] == (36, 40) and "l3.mix.k" not in names and "l3.mix.k.norm" not in names and "l3.mix.v.b" not in names
    assert names["l2.mix.left.g"] == (32, 40) and "l2.mix.left.q.b" not in names and names["l2.mix.left.q.norm"] == (64,)
    assert names["l2.mix.right.q.conv"] == (24, 4) and names["l2.mix.right.v.conv"] == (40, 4) and names["l2.mix.right.norm"] == (10,)
    assert names["l2.mix.right.A_log"] == (4,) and names["l2.mix.right.a"] == (4, 40) and names["l2.mix.right.b"] == (4, 40)
    assert names["l1.mix.norm"] == (36,) and names["l1.mix.g"] == (36, 40) and "l1.norm2" not in names and "l1.ls2" not in names
    assert names["side.embed"] == (70, 24) and names["l3.side.gate"] == (6, 40) and names["l3.side.proj"] == (40, 6) and names["head"] == (70, 40)
    side = [l.block.extra["after_token_side"] for l in model.layers]
    assert [s.col0 for s in side] == [0, 6, 12, 18]
    # the lender keeps what the borrower that looks furthest back needs; the borrower asks for nothing
    reqs = model.memory_requests()
    assert reqs[0][1] == CacheRequest("window", 3, 12, 30, 20) and reqs[0][2] is None
    assert reqs[1][1] is None and reqs[1][2] == StateRequest((3 * 8 * 12,), torch.float32)
    assert reqs[2][1] == CacheRequest("full", 1, 16, None, 8) and reqs[2][2] == StateRequest((4 * 12 * 10 + 3 * (2 * 24 + 40),), torch.float32)
    assert reqs[3][1] is None and reqs[3][2] is None and reqs[3][3] == 0
    a0, a3 = model.layers[0].block.mixer, model.layers[3].block.mixer
    assert a0.window == 9 and a0.cache_window == 30 and a3.window == 30 and a3.borrows_kv and a0.adjacent and a0.rot_dims == 8
    left = model.layers[2].block.mixer.subs[0][0]
    assert left.rotary.pairing == "half" and left.window is None and left.out_gate == "sigmoid" and not left.bias
    assert [s for _, s in model.layers[2].block.mixer.subs] == [0.7, 1.4]


def test_a_lender_without_a_window_of_its_own_keeps_everything_a_borrower_wants():
    both = dict(CFG, layers=[dict(CFG["layers"][0]), {"type": "attention", "mixer": {k: v for k, v in dict(ATT, kv_from=0).items() if k != "mask"}, "mlp": None}])
    reqs = Model.from_config_dict(both).memory_requests()
    assert reqs[0][1] == CacheRequest("full", 3, 12, None, 20)


# ---- the plain implementation's own properties ---------------------------------------------------------------------
def test_plain_model_is_causal_and_carries_what_lies_outside_a_window():
    w = pz.random_weights(CFG, seed=1)
    t = np.random.default_rng(0).integers(0, 70, size=60).tolist()
    layers = []
    full = pz.forward(CFG, w, t, layers_out=layers)
    assert len(layers) == 4 and layers[0].shape == (60, 40)
    assert np.allclose(pz.forward(CFG, w, t[:33]), full[:33], rtol=0, atol=1e-11)
    t2 = list(t)
    t2[40] = (t2[40] + 1) % 70
    b = pz.forward(CFG, w, t2)
    assert np.allclose(b[:40], full[:40], rtol=0, atol=1e-11) and np.abs(b[40:] - full[40:]).max() > 1e-6
    # the recurrent layers carry token 0 to the end, far outside both windows
    t3 = list(t)
    t3[0] = (t3[0] + 1) % 70
    assert np.abs(pz.forward(CFG, w, t3)[-1] - full[-1]).max() > 1e-9
    # with the attention layers alone, nothing older than the windows reaches the last token
    only = dict(CFG, layers=[CFG["layers"][0], dict(CFG["layers"][3], mixer=dict(CFG["layers"][3]["mixer"], kv_from=0))])
    only["layers"][1]["mixer"]["kv_from"] = 0
    w2 = pz.random_weights(only, seed=2)
    a, c = pz.forward(only, w2, t), pz.forward(only, w2, t3)
    assert np.abs(a[1] - c[1]).max() > 1e-9 and np.allclose(a[-1], c[-1], rtol=0, atol=1e-12)


def test_plain_mechanisms_on_small_cases_worked_by_hand():
    assert np.allclose(pz.rms_norm(np.array([[3.0, 4.0]]), np.array([1.0, 2.0]), 0.0), [[3.0 / math.sqrt(12.5), 8.0 / math.sqrt(12.5)]])
    # a quarter turn: base 1 makes every frequency 1, position pi / 2
    x = np.array([[[1.0, 0.0, 0.0, 2.0, 7.0]]])
    near = pz.rotate(x, [math.pi / 2], {"dims": 4, "base": 1.0}, "neighbours")       # pairs (0, 1), (2, 3)
    assert np.allclose(near, [[[0.0, 1.0, -2.0, 0.0, 7.0]]], atol=1e-12)
    half = pz.rotate(x, [math.pi / 2], {"dims": 4, "base": 1.0}, "halves")           # pairs (0, 2), (1, 3)
    assert np.allclose(half, [[[0.0, -2.0, 1.0, 0.0, 7.0]]], atol=1e-12)
    assert np.allclose(pz.rotate(x, [3], {"dims": 4, "base": 100.0}, "halves")[0, 0, :1], [math.cos(3.0)])     # pair 0 turns by p
    assert np.allclose(pz.rotate(x, [3], {"dims": 4, "base": 100.0}, "halves")[0, 0, 1], -2.0 * math.sin(0.3))  # pair 1 by p / 10
    # convolution: the last column is the current token's
    u = np.array([[1.0], [10.0], [100.0]])
    assert np.allclose(pz.short_conv(u, np.array([[3.0, 2.0, 1.0]])), [[1.0], [12.0], [123.0]])
    # a window of 2: the last of three sees the last two
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": 1.0, "mask": {"size": 2}, "rot": {"dims": 0, "base": 10.0}}
    eye = np.eye(2)
    wts = {"q": eye, "k": eye, "v": np.array([[1.0, 0.0]]), "q.b": np.zeros(2), "k.b": np.zeros(2), "v.b": np.zeros(1),
           "q.norm": np.ones(2), "k.norm": np.ones(2)}
    h = np.array([[5.0, 0.0], [1.0, 0.0], [0.0, 0.0]])                               # the last query is zero: equal weights
    out = pz.softmax_heads(h, wts, m, 1e-9, "neighbours", True)
    assert np.allclose(out[2], [0.5]) and np.allclose(out[0], [5.0])
    # gelu both ways
    assert abs(pz.gelu_erf(np.array([1.0]))[0] - 0.8413447460685429) < 1e-12 and abs(pz.gelu_tanh(np.array([1.0]))[0] - 0.8411919906082768) < 1e-12
    # decayed linear attention, one head of one number: S = 0.5 S + k v, o = S q, all silu(1) = s: o_1 = s^3, o_2 = 1.5 s^3;
    # the norm over the one number gives its sign
    s = 1.0 / (1.0 + math.exp(-1.0))
    one = np.array([[1.0]])
    lw = {"q": one, "k": one, "v": one, "g": one * 0, "o": one, "norm": one[0] * 4}
    assert np.allclose(pz.lightning(np.array([[1.0], [1.0]]), lw, {"heads": 1, "dim": 1, "vdim": 1, "decay": [0.5]}, 0.0), [[2.0], [2.0]])
    lw["norm"] = one[0]
    big = pz.lightning(np.array([[1.0], [1.0]]), lw, {"heads": 1, "dim": 1, "vdim": 1, "decay": [0.5]}, 1.0)     # eps 1: o / sqrt(o^2 + 1) / 2
    assert np.allclose(big[:, 0], [s ** 3 / math.sqrt(s ** 6 + 1) / 2, 1.5 * s ** 3 / math.sqrt(2.25 * s ** 6 + 1) / 2])


def test_plain_delta_rule_overwrites_what_a_key_holds():
    """With beta = 1, no decay and unit keys the rule stores v under k: writing twice under the same key keeps the second
    value, and a read with that key returns it."""
    dim = 4
    m = {"heads": 1, "kv_heads": 1, "dim": dim, "vdim": 2, "conv": 1}
    big = 40.0
    w = {"q": np.eye(dim) * big, "k": np.eye(dim) * big, "v": np.zeros((2, dim)), "q.conv": np.ones((dim, 1)), "k.conv": np.ones((dim, 1)),
         "v.conv": np.ones((2, 1)), "b": np.full((1, dim), big), "a": np.full((1, dim), -big), "A_log": np.zeros(1), "dt_bias": np.zeros(1),
         "norm": np.ones(2), "g": np.zeros((2, dim)), "o": np.eye(2)}
    w["v"][0, 0], w["v"][1, 1] = 3.0, 5.0
    # silu(big x) of a one-hot input is a one-hot key; beta = sigmoid(40) = 1; decay = exp(-softplus(-40)) = 1
    h = np.array([[1.0, 0, 0, 0], [0, 1.0, 0, 0], [1.0, 0, 0, 0]])
    T = 3
    q = pz.silu(h @ w["q"].T)
    k = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6)
    v = pz.silu(h @ w["v"].T)
    S = np.zeros((dim, 2))
    outs = []
    for t in range(T):
        S = S + np.outer(k[t], v[t] - S.T @ k[t])
        outs.append(S.T @ k[t] * dim ** -0.5)
    assert np.allclose(outs[2], v[2] * dim ** -0.5, atol=1e-4)
    got = pz.delta_rule(h, w, m, 0.0)          # gate silu(0) = 0 would hide everything: give the gate a value
    assert np.allclose(got, 0.0)
    w["g"] = np.full((2, dim), 2.0)
    got = pz.delta_rule(h, w, m, 0.0)
    o = np.stack(outs)
    want = o / np.sqrt((o * o).mean(-1, keepdims=True)) * pz.silu(h @ w["g"].T)
    assert np.allclose(got, want, atol=1e-6)


def test_token_side_input_reads_its_own_slice_of_the_table():
    table = np.arange(24, dtype=np.float64).reshape(2, 12)
    w = {"gate": np.ones((3, 2)), "proj": np.eye(3)[:2].T.copy().T, "norm": np.ones(2)}
    w["proj"] = np.array([[1.0, 0.0, 0.0], [0.0, 1.0, 0.0]])
    x = np.array([[0.5, 0.5]])
    g = pz.gelu_tanh(np.array([1.0]))[0]
    y = pz.token_side(x, [1], table, w, 2, 3, 0.0)              # layer 2 of slices 3 wide: columns 6..8 of row 1: 18, 19, 20
    raw = np.array([18.0 * g, 19.0 * g])
    assert np.allclose(y, [raw / math.sqrt((raw ** 2).mean())])


def test_command_line_makes_and_lists_a_model_folder(tmp_path, capsys):
    from ghost_infer_b200 import cli
    from ghost_infer_b200.weights.loader import load_model_tensors
    from ghost_infer_b200.weights.safetensors_io import SafetensorsFile
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(CFG))
    out = tmp_path / "model"
    assert cli.main(["random", str(cfg_file), str(out), "--seed", "3"]) == 0
    names = set(SafetensorsFile(str(out / "model.safetensors")).names())
    assert names == {w.name for w in Model.from_config_dict(CFG).weight_manifest()}
    assert cli.main(["inspect", str(out)]) == 0
    text = capsys.readouterr().out
    assert "l0.mix.q.norm" in text and "token_side" in text and f"{len(names)} tensors" in text
    w = pz.random_weights(CFG, seed=4)
    other = tmp_path / "other"
    other.mkdir()
    (other / "config.json").write_text(json.dumps(CFG))
    pz.write_safetensors_bf16(str(other / "model.safetensors"), w)
    model = Model.from_config_dict(CFG)
    got = load_model_tensors(str(other), model.weight_manifest(), model.ignorable_tensors())
    assert torch.equal(got["l2.mix.right.q.conv"].float(), torch.from_numpy(w["l2.mix.right.q.conv"]).float())
    assert torch.equal(got["side.embed"].float(), torch.from_numpy(w["side.embed"]).float())
