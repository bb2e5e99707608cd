"""Typed configuration of the Nuzinex decoder, read from config.json, and the layers it is made of.

A Nuzinex model is a list of layers, each with its own sizes.  A layer reads the residual stream itself and norms what
its sublayers give back: x += ls1 * rms(mixer(x)), then, unless `mlp` is null, x += ls2 * rms(ff(x)), then a per-token
input from a second embedding table (`token_side.dim` columns per layer).  `layers[i].type` names the mixer:

* "attention": grouped-query attention inside a sliding window (`mask.size`), with biases, an RMS norm over the whole
  query and key projections, rotation of neighbouring pairs on the first `rot.dims` numbers of a head (`rot.base`), and
  `scale`; with `kv_from`: j it has no keys and values of its own and reads layer j's cache.
* "parallel": `left` (causal attention without biases, the same whole-projection norm, rotation of pairs half the
  rotated width apart, a sigmoid gate on the heads' outputs) and `right` (a gated delta rule with short convolutions)
  side by side, added with `left_scale` and `right_scale`.
* "lightning": linear attention with a constant `decay` per head.

The feed-forward (`mlp.kind` "dense") is W_down gelu(W_up h) with the exact gelu.  Every norm is an RMS norm with
`norm.eps`; the head is a matrix of its own.  Nothing about a model lives in code: sizes, counts, constants and the order
of layers come from config.json.

Tensors: "embed", "side.embed", "l<i>.norm1", "l<i>.norm2", "l<i>.ls1", "l<i>.ls2", "l<i>.mix.*", "l<i>.mlp.{up,down}",
"l<i>.side.{gate,proj,norm}", "final.norm", "head".
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..parts.spec import ExtraPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .errors import ConfigError

ARCHITECTURE = "Nuzinex"
# rotary angles are formed from the position itself: no length the design was trained for is written anywhere
NO_POSITION_LIMIT = 1 << 20
# fixed by the design: the floor under the sum of squares when the delta rule's queries and keys are made unit vectors
UNIT_NORM_EPS = 1e-6


def _need(d: Any, key: str, where: str):
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json of {ARCHITECTURE}: missing key \"{key}\" in {where}")
    return d[key]


def _int(d: Any, key: str, where: str, least: int = 1) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or int(v) < least:
        raise ConfigError(f"config.json of {ARCHITECTURE}: \"{key}\" in {where} must be an integer >= {least}, got {v!r}")
    return int(v)


def _num(d: Any, key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json of {ARCHITECTURE}: \"{key}\" in {where} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float


@dataclass(frozen=True)
class SoftmaxMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[Rotation]
    window: Optional[int]
    kv_from: Optional[int]


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class ParallelMixer:
    left: SoftmaxMixer
    right: DeltaMixer
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class LightningMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class NuzinexLayer:
    type: str
    mixer: Any
    mlp: Optional[DenseMlp]


def _softmax_mixer(m: Any, where: str, n_layers: int, index: int, windowed: bool) -> SoftmaxMixer:
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: {heads} heads do not divide into {kv} kv heads")
    dim = _int(m, "dim", where)
    rot = None
    if isinstance(m, Mapping) and m.get("rot") is not None:
        r = m["rot"]
        dims = _int(r, "dims", where + ".rot", least=0)
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json of {ARCHITECTURE}: {where}.rot: {dims} rotated numbers must be even and at most {dim}")
        rot = Rotation(dims, _num(r, "base", where + ".rot")) if dims else None
    window = None
    if windowed and m.get("mask") is not None:
        window = _int(m["mask"], "size", where + ".mask")
    kv_from = None
    if windowed and m.get("kv_from") is not None:
        kv_from = _int(m, "kv_from", where, least=0)
        if kv_from >= index:
            raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: kv_from {kv_from} must name an earlier layer")
    return SoftmaxMixer(heads, kv, dim, _int(m, "vdim", where), _num(m, "scale", where), rot, window, kv_from)


@dataclass(frozen=True)
class NuzinexConfig:
    architecture: str
    width: int
    vocab: int
    norm_eps: float
    side_dim: int
    layers: Tuple[NuzinexLayer, ...]
    stop_token_ids: Tuple[int, ...] = ()

    # what the rest of the library asks of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return NO_POSITION_LIMIT

    @property
    def eos_token_ids(self) -> Tuple[int, ...]:
        return self.stop_token_ids

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "NuzinexConfig":
        width = _int(raw, "width", "the top level")
        vocab = _int(raw, "vocab", "the top level")
        layers_raw = _need(raw, "layers", "the top level")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError(f"config.json of {ARCHITECTURE}: \"layers\" must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            kind = _need(lr, "type", where)
            m = _need(lr, "mixer", where)
            if kind == "attention":
                mixer = _softmax_mixer(m, where, len(layers_raw), i, True)
                if mixer.kv_from is not None:
                    src = layers[mixer.kv_from]
                    if src.type != "attention" or src.mixer.kv_from is not None:
                        raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: layer {mixer.kv_from} has no keys and values of its own to lend")
                    s = src.mixer
                    if (s.kv_heads, s.dim, s.vdim) != (mixer.kv_heads, mixer.dim, mixer.vdim):
                        raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: layer {mixer.kv_from}'s keys and values have other sizes")
            elif kind == "parallel":
                left = _softmax_mixer(_need(m, "left", where), where + ".left", len(layers_raw), i, False)
                r = _need(m, "right", where)
                rw = where + ".right"
                right = DeltaMixer(_int(r, "heads", rw), _int(r, "kv_heads", rw), _int(r, "dim", rw), _int(r, "vdim", rw), _int(r, "conv", rw))
                if right.heads % right.kv_heads:
                    raise ConfigError(f"config.json of {ARCHITECTURE}: {rw}: {right.heads} heads do not divide into {right.kv_heads} query/key heads")
                mixer = ParallelMixer(left, right, _num(m, "left_scale", where), _num(m, "right_scale", where))
            elif kind == "lightning":
                heads = _int(m, "heads", where)
                decay = _need(m, "decay", where)
                if not isinstance(decay, (list, tuple)) or len(decay) != heads or any(isinstance(g, bool) or not isinstance(g, (int, float)) for g in decay):
                    raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: \"decay\" must list one number per head ({heads})")
                mixer = LightningMixer(heads, _int(m, "dim", where), _int(m, "vdim", where), tuple(float(g) for g in decay))
            else:
                raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: unknown layer type {kind!r} (attention, parallel, lightning)")
            mr = lr.get("mlp") if isinstance(lr, Mapping) else None
            if mr is None:
                mlp = None
            elif _need(mr, "kind", where + ".mlp") == "dense":
                mlp = DenseMlp(_int(mr, "ff", where + ".mlp"))
            else:
                raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: unknown feed-forward kind {mr['kind']!r} (dense)")
            layers.append(NuzinexLayer(kind, mixer, mlp))
        stops = raw.get("eos_token_id")
        stops = () if stops is None else tuple(int(t) for t in (stops if isinstance(stops, (list, tuple)) else [stops]))
        return cls(ARCHITECTURE, width, vocab, _num(_need(raw, "norm", "the top level"), "eps", "norm"),
                   _int(_need(raw, "token_side", "the top level"), "dim", "token_side"), tuple(layers), stops)


def _attention_params(cfg: NuzinexConfig, m: SoftmaxMixer, *, base: str, pairing: str, bias: bool, gate: Optional[str],
                      cache_window: Optional[int]) -> dict:
    rot = {"dims": m.rot.dims, "base": m.rot.base, "pairing": pairing} if m.rot is not None else None
    return {"hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
            "scale": m.scale, "window": m.window, "cache_window": cache_window, "bias": bias, "qk_norm": True, "eps": cfg.norm_eps,
            "rotary": rot, "out_gate": gate, "borrows_kv": m.kv_from is not None, "base": base}


def build_nuzinex_spec(cfg: NuzinexConfig) -> ModelSpec:
    bare = {"tensor_names": {"weight": ""}}      # "l0.norm1", "embed", "head": the tensor is the prefix itself
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, **bare})
    scale = PartSpec("channel_scale", {"size": cfg.width, **bare})
    table_width = cfg.side_dim * len(cfg.layers)
    # a layer that lends its keys and values keeps them as long as the borrower that looks furthest back needs them
    keep = {}
    for i, layer in enumerate(cfg.layers):
        if layer.type == "attention":
            src = i if layer.mixer.kv_from is None else layer.mixer.kv_from
            w = layer.mixer.window
            keep[src] = w if src not in keep else (None if (w is None or keep[src] is None) else max(w, keep[src]))
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "attention":
            mixer = PartSpec("normed_attention", _attention_params(cfg, m, base="mix.", pairing="adjacent", bias=True, gate=None,
                                                                   cache_window=keep.get(i) if m.kv_from is None else None))
        elif layer.type == "parallel":
            left = PartSpec("normed_attention", _attention_params(cfg, m.left, base="mix.left.", pairing="half", bias=False,
                                                                  gate="sigmoid", cache_window=None))
            r = m.right
            right = PartSpec("gated_delta_rule", {"hidden_size": cfg.width, "heads": r.heads, "qk_heads": r.kv_heads, "key_dim": r.dim,
                                                  "v_dim": r.vdim, "conv": r.conv, "eps": cfg.norm_eps, "unit_eps": UNIT_NORM_EPS,
                                                  "base": "mix.right."})
            mixer = PartSpec("parallel_mixers", {"mixers": ({"spec": left, "scale": m.left_scale}, {"spec": right, "scale": m.right_scale})})
        else:
            mixer = PartSpec("decayed_linear_attention", {"hidden_size": cfg.width, "heads": m.heads, "key_dim": m.dim, "v_dim": m.vdim,
                                                          "decay": m.decay, "eps": cfg.norm_eps, "base": "mix."})
        ffn = None
        if layer.mlp is not None:
            ffn = PartSpec("mlp", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "activation": "gelu", "bias": False})
        extra = [ExtraPart("mixer_scale", "norm", scale, "ls1")]
        if ffn is not None:
            extra.append(ExtraPart("ffn_scale", "norm", scale, "ls2"))
        extra.append(ExtraPart("after_token_side", "feed_forward",
                               PartSpec("token_side", {"hidden_size": cfg.width, "dim": cfg.side_dim, "col0": i * cfg.side_dim,
                                                       "table_width": table_width, "vocab_size": cfg.vocab, "eps": cfg.norm_eps,
                                                       "table": "side.embed"})))
        layers.append(LayerSpec(prefix=f"l{i}.", block="residual_postnorm", mixer_norm=norm, mixer=mixer,
                                ffn_norm=norm if ffn is not None else None, ffn=ffn, mixer_norm_prefix="norm1",
                                ffn_norm_prefix="norm2", extra=tuple(extra)))
        schedule.append(ScheduleEntry(i, memory_of=m.kv_from if layer.type == "attention" else None))
    spec = ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=NO_POSITION_LIMIT,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, **bare}),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm,
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": False, **bare}),
        stop_token_ids=cfg.stop_token_ids, embedding_prefix="embed", final_norm_prefix="final.norm", head_prefix="head")
    spec.validate()
    return spec
