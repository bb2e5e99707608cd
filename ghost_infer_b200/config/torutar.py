"""Typed configuration of the Torutar decoder, read from config.json, and the layers it is made of.

A Torutar model keeps `streams` copies of the residual stream.  Every layer has a mixer and, unless `mlp` is null, a routed
feed-forward; each sublayer reads a learned blend of the copies through an RMS norm, adds a short causal convolution of its
input (`canon.taps`), is gated by a sigmoid of a projection of its input, and is written back into every copy with learned
weights.  `layers[i].type` names the mixer, `layers[i].mixer` gives its sizes:

* "attention": grouped-query attention with biases, per-head RMS norms of queries and keys (one weight shared by the heads),
  rotation of pairs half the rotated width apart on the first `rot.dims` numbers of a head, values divided by their root mean
  square, a window of `mask.size` positions that keeps the first `mask.keep_first` visible, a learned sink per head, one
  sigmoid gate per head, `scale`; with `kv_from`: j the layer has no keys and values and reads layer j's cache;
* "latent_attention": causal attention whose keys and values come out of one cached latent per token (`kv_rank`), queries
  through a latent of their own (`q_rank`), `dim` unrotated and `rot_dim` rotated numbers per head (neighbouring pairs
  turn), a sigmoid gate on the heads' outputs;
* "mlstm": a matrix memory with exponential gates capped at `gate_cap` and a running maximum.

The feed-forward (`mlp.kind` "moe"): `router.experts` clamped gated experts of width `expert.ff` (`expert.limit`), of which a
token uses `router.top`, chosen by softmax share plus a stored correction and weighted by their shares times `router.scale`;
beside them a shared expert (`shared.ff`, `shared.limit`).  The embedded tokens pass an RMS norm; the logits are multiplied by
`logit_scale`.  Nothing about a model lives in code: sizes, counts, constants and the order of layers come from config.json.

Tensors: "embed", "embed.norm", "l<i>.norm1", "l<i>.norm2", "l<i>.hc{1,2}.{in,mix,out}", "l<i>.canon{1,2}", "l<i>.rg{1,2}",
"l<i>.rg{1,2}.b", "l<i>.mix.*", "l<i>.mlp.*", "final.norm", "head".
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..parts.spec import ExtraPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .errors import ConfigError

ARCHITECTURE = "Torutar"
# rotary angles are formed from the position itself: no length the design was trained for is written anywhere
NO_POSITION_LIMIT = 1 << 20
# fixed by the design: the slope inside the sigmoid of an expert's gate half
EXPERT_SIGMOID_SLOPE = 1.702


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
class WindowMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[Rotation]
    window: Optional[int]
    keep_first: int
    kv_from: Optional[int]


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: Optional[Rotation]


@dataclass(frozen=True)
class MatrixMemoryMixer:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ExpertsMlp:
    experts: int
    top: int
    route_scale: float
    ff: int
    limit: float
    shared_ff: Optional[int]
    shared_limit: float


@dataclass(frozen=True)
class TorutarLayer:
    type: str
    mixer: Any
    mlp: Optional[ExpertsMlp]


def _rotation(m: Any, where: str, most: int) -> Optional[Rotation]:
    if not isinstance(m, Mapping) or m.get("rot") is None:
        return None
    r = m["rot"]
    dims = _int(r, "dims", where + ".rot", least=0)
    if dims % 2 or dims > most:
        raise ConfigError(f"config.json of {ARCHITECTURE}: {where}.rot: {dims} rotated numbers must be even and at most {most}")
    return Rotation(dims, _num(r, "base", where + ".rot")) if dims else None


def _window_mixer(m: Any, where: str, index: int) -> WindowMixer:
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: {heads} heads do not divide into {kv} kv heads")
    dim = _int(m, "dim", where)
    window, keep_first = None, 0
    if m.get("mask") is not None:
        window = _int(m["mask"], "size", where + ".mask")
        if m["mask"].get("keep_first") is not None:
            keep_first = _int(m["mask"], "keep_first", where + ".mask", least=0)
    kv_from = None
    if m.get("kv_from") is not None:
        kv_from = _int(m, "kv_from", where, least=0)
        if kv_from >= index:
            raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: kv_from {kv_from} must name an earlier layer")
    return WindowMixer(heads, kv, dim, _int(m, "vdim", where), _num(m, "scale", where), _rotation(m, where, dim), window, keep_first, kv_from)


def _mlp(mr: Any, where: str) -> Optional[ExpertsMlp]:
    if mr is None:
        return None
    if _need(mr, "kind", where) != "moe":
        raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: unknown feed-forward kind {mr['kind']!r} (moe)")
    r, e = _need(mr, "router", where), _need(mr, "expert", where)
    experts, top = _int(r, "experts", where + ".router"), _int(r, "top", where + ".router")
    if top > experts:
        raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: a token cannot use {top} of {experts} experts")
    sh = mr.get("shared")
    return ExpertsMlp(experts, top, _num(r, "scale", where + ".router"), _int(e, "ff", where + ".expert"), _num(e, "limit", where + ".expert"),
                      _int(sh, "ff", where + ".shared") if sh is not None else None,
                      _num(sh, "limit", where + ".shared") if sh is not None else 0.0)


@dataclass(frozen=True)
class TorutarConfig:
    architecture: str
    width: int
    vocab: int
    norm_eps: float
    streams: int
    taps: int
    logit_scale: float
    layers: Tuple[TorutarLayer, ...]
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
    def from_dict(cls, raw: Mapping[str, Any]) -> "TorutarConfig":
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
                mixer = _window_mixer(m, where, i)
                if mixer.kv_from is not None:
                    src = layers[mixer.kv_from]
                    if src.type != "attention" or src.mixer.kv_from is not None:
                        raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: layer {mixer.kv_from} has no keys and values of its own to lend")
                    s = src.mixer
                    if (s.kv_heads, s.dim, s.vdim) != (mixer.kv_heads, mixer.dim, mixer.vdim):
                        raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: layer {mixer.kv_from}'s keys and values have other sizes")
            elif kind == "latent_attention":
                rot_dim = _int(m, "rot_dim", where, least=0)
                mixer = LatentMixer(_int(m, "heads", where), _int(m, "dim", where), rot_dim, _int(m, "vdim", where), _int(m, "kv_rank", where),
                                    _int(m, "q_rank", where), _num(m, "scale", where), _rotation(m, where, rot_dim))
            elif kind == "mlstm":
                mixer = MatrixMemoryMixer(_int(m, "heads", where), _int(m, "dim", where), _int(m, "vdim", where), _num(m, "gate_cap", where))
                if not mixer.gate_cap > 0:
                    raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: gate_cap must be positive")
            else:
                raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: unknown layer type {kind!r} (attention, latent_attention, mlstm)")
            layers.append(TorutarLayer(kind, mixer, _mlp(lr.get("mlp") if isinstance(lr, Mapping) else None, where + ".mlp")))
        stops = raw.get("eos_token_id")
        stops = () if stops is None else tuple(int(t) for t in (stops if isinstance(stops, (list, tuple)) else [stops]))
        canon = raw.get("canon")
        return cls(ARCHITECTURE, width, vocab, _num(_need(raw, "norm", "the top level"), "eps", "norm"),
                   _int(raw, "streams", "the top level"), _int(canon, "taps", "canon") if canon is not None else 0,
                   float(raw["logit_scale"]) if raw.get("logit_scale") is not None else 1.0, tuple(layers), stops)


def build_torutar_spec(cfg: TorutarConfig) -> ModelSpec:
    bare = {"tensor_names": {"weight": ""}}      # "l0.norm1", "embed", "head": the tensor is the prefix itself
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, **bare})
    # a layer that lends its keys and values keeps them as long as the borrower that looks furthest back needs them
    keep_window, keep_first = {}, {}
    for i, layer in enumerate(cfg.layers):
        if layer.type == "attention":
            src = i if layer.mixer.kv_from is None else layer.mixer.kv_from
            w = layer.mixer.window
            keep_window[src] = w if src not in keep_window else (None if (w is None or keep_window[src] is None) else max(w, keep_window[src]))
            keep_first[src] = max(keep_first.get(src, 0), layer.mixer.keep_first)
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "attention":
            own = m.kv_from is None
            mixer = PartSpec("head_normed_attention", {
                "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "scale": m.scale, "window": m.window, "keep_first": m.keep_first,
                "cache_window": keep_window.get(i) if own else m.window, "cache_keep_first": keep_first.get(i, 0) if own else m.keep_first,
                "bias": True, "qk_norm": True, "v_norm": True, "sink": True, "head_gate": True, "eps": cfg.norm_eps,
                "rotary": {"dims": m.rot.dims, "base": m.rot.base, "pairing": "half"} if m.rot is not None else None,
                "borrows_kv": not own, "base": "mix."})
        elif layer.type == "latent_attention":
            position = None
            if m.rot is not None:
                position = PartSpec("rotary", {"head_dim": m.rot_dim, "rotary_dim": m.rot.dims, "theta": m.rot.base, "pairing": "adjacent"})
            mixer = PartSpec("latent_attention", {"hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim,
                                                  "v_head_dim": m.vdim, "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale,
                                                  "eps": cfg.norm_eps, "position": position, "out_gate": "sigmoid"})
        else:
            mixer = PartSpec("mlstm", {"hidden_size": cfg.width, "heads": m.heads, "key_dim": m.dim, "v_dim": m.vdim,
                                       "gate_cap": m.gate_cap, "eps": cfg.norm_eps, "base": "mix."})
        ffn = None
        if layer.mlp is not None:
            f = layer.mlp
            ffn = PartSpec("share_routed_experts", {"hidden_size": cfg.width, "experts": f.experts, "top": f.top, "expert_ff": f.ff,
                                                    "limit": f.limit, "alpha": EXPERT_SIGMOID_SLOPE, "route_scale": f.route_scale,
                                                    "correction": True, "shared_ff": f.shared_ff, "shared_limit": f.shared_limit})
        connect = lambda q: PartSpec("hyper_connection", {"hidden_size": cfg.width, "streams": cfg.streams, "conv_taps": cfg.taps,
                                                          "gate": True, "index": q})
        extra = [ExtraPart("connect1", "feed_forward", connect(1))]
        if ffn is not None:
            extra.append(ExtraPart("connect2", "feed_forward", connect(2)))
        layers.append(LayerSpec(prefix=f"l{i}.", block="hyper_connections", mixer_norm=norm, mixer=mixer,
                                ffn_norm=norm if ffn is not None else None, ffn=ffn, mixer_norm_prefix="norm1",
                                ffn_norm_prefix="norm2", extra=tuple(extra)))
        schedule.append(ScheduleEntry(i, memory_of=m.kv_from if layer.type == "attention" else None))
    spec = ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=NO_POSITION_LIMIT,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, **bare}),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm,
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": False, "scale": cfg.logit_scale, **bare}),
        stop_token_ids=cfg.stop_token_ids, embedding_prefix="embed", final_norm_prefix="final.norm", head_prefix="head",
        embedding_norm=norm, embedding_norm_prefix="embed.norm", streams=cfg.streams)
    spec.validate()
    return spec
