"""Kevatar: config.json -> typed configuration -> :class:`ModelSpec`.

A decoder-only model whose config.json lists its layers one by one (``layers``: ``type``, the mixer's sizes under
``mixer``, the feed-forward under ``mlp`` or null).  The norm of a layer sits on each branch's *output*, and the branches
read the residual stream itself: ``x += N1(mixer(x)); x += N2(ff(x))``; with ``token_side`` every layer then adds a third
branch, a gate on the token's own entry in a table that all layers divide among themselves: ``x += Ns(P (gelu_tanh(G x) *
T[token, l d : (l + 1) d]))``.  The embedding is multiplied by ``embedding.scale``; the head is the embedding table itself.
Three kinds of mixer:

* ``attention``: grouped-query attention with value heads of their own size, the first ``rot.dims`` entries of every query
  and key head turned in interleaved pairs (frequencies stretched by ``rot.scaling``), every turned head divided by its root
  mean square, ``scale`` from the config, scores through ``softcap * tanh(s / softcap)``, a window of ``mask.size`` keys; a
  layer with ``kv_from: j`` has no key and value projections and reads the cache of layer j;
* ``channel_delta``: a gated delta rule with a decay per head and key entry, short causal convolutions on q, k and v;
* ``lightning``: a matrix state per head with a constant decay.

The feed-forward is a dense gated one (SiLU).  Tensor names: ``embed``, ``side.embed``, ``final.norm``, and per layer i
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

MIXER_TYPES = ("attention", "channel_delta", "lightning")
# the framework's context limit when config.json names none: the design has no learned positions
DEFAULT_MAX_POSITIONS = 1 << 15
SIDE_TABLE = "side"              # the key under which the embedding leaves the per-token table for the layers


@dataclass(frozen=True)
class KevatarRotation:
    base: float
    dims: int
    scaling: Optional[Mapping[str, float]]         # factor, original, fast, slow


@dataclass(frozen=True)
class KevatarLayer:
    type: str
    mixer: Mapping[str, Any]              # the mixer's sizes and constants, checked
    rot: Optional[KevatarRotation]
    kv_from: Optional[int]
    ff: int = 0                           # 0: no feed-forward


@dataclass(frozen=True)
class KevatarConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    side_dim: int                         # 0: no per-token table
    layers: Tuple[KevatarLayer, ...]
    max_positions: int
    raw: Mapping[str, Any]

    def to_json_dict(self) -> dict:
        return dict(self.raw)


def _int(obj: Mapping[str, Any], key: str, where: str) -> int:
    v = obj.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}'{key}' must be a positive integer, got {v!r}")
    return v


def _num(obj: Mapping[str, Any], key: str, where: str) -> float:
    v = obj.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {v!r}")
    return float(v)


def _rotation(m: Mapping[str, Any], where: str, limit: int) -> Optional[KevatarRotation]:
    rot = m.get("rot")
    if rot is None:
        return None
    if not isinstance(rot, Mapping):
        raise ConfigError(f"config.json: {where}rot must be an object with 'base' and 'dims'")
    base, dims = _num(rot, "base", where + "rot."), _int(rot, "dims", where + "rot.")
    if not base > 0.0 or dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}rot: base={base} must be positive and dims={dims} even and at most {limit}")
    scaling = rot.get("scaling")
    if scaling is not None:
        if not isinstance(scaling, Mapping):
            raise ConfigError(f"config.json: {where}rot.scaling must be an object or null")
        scaling = {k: _num(scaling, k, where + "rot.scaling.") for k in ("factor", "original", "fast", "slow")}
        if min(scaling.values()) <= 0.0 or base == 1.0:
            raise ConfigError(f"config.json: {where}rot.scaling: every entry must be positive (and rot.base differ from 1)")
    return KevatarRotation(base, dims, scaling)


def parse_kevatar_config(raw: Mapping[str, Any]) -> KevatarConfig:
    missing = [k for k in ("vocab", "width", "layers", "norm") if k not in raw]
    if missing:
        raise ConfigError("config.json: missing required key(s): " + ", ".join(missing))
    if not isinstance(raw["layers"], list) or not raw["layers"]:
        raise ConfigError("config.json: 'layers' must be a list with at least one layer")
    if not isinstance(raw["norm"], Mapping):
        raise ConfigError("config.json: 'norm' must be an object with 'eps'")
    eps = _num(raw["norm"], "eps", "norm.")
    if not eps > 0.0:
        raise ConfigError(f"config.json: norm.eps={eps} must be positive")
    emb = raw.get("embedding")
    if emb is not None and not isinstance(emb, Mapping):
        raise ConfigError("config.json: 'embedding' must be an object with 'scale'")
    emb_scale = _num(emb, "scale", "embedding.") if emb and "scale" in emb else 1.0
    side = raw.get("token_side")
    if side is not None and not isinstance(side, Mapping):
        raise ConfigError("config.json: 'token_side' must be an object with 'dim', or null")
    side_dim = _int(side, "dim", "token_side.") if side is not None else 0
    layers = []
    for i, entry in enumerate(raw["layers"]):
        where = f"layers[{i}]."
        if not isinstance(entry, Mapping) or not isinstance(entry.get("mixer"), Mapping):
            raise ConfigError(f"config.json: {where}mixer must be an object")
        kind, m, mw = entry.get("type"), entry["mixer"], where + "mixer."
        rot, kv_from = None, None
        sizes: Dict[str, Any]
        if kind == "attention":
            sizes = {k: _int(m, k, mw) for k in ("heads", "kv_heads", "dim")}
            sizes["vdim"] = _int(m, "vdim", mw) if "vdim" in m else sizes["dim"]
            if sizes["heads"] % sizes["kv_heads"]:
                raise ConfigError(f"config.json: {mw}heads={sizes['heads']} is no multiple of kv_heads={sizes['kv_heads']}")
            sizes["scale"] = _num(m, "scale", mw)
            sizes["softcap"] = _num(m, "softcap", mw) if m.get("softcap") is not None else None
            if sizes["softcap"] is not None and not sizes["softcap"] > 0.0:
                raise ConfigError(f"config.json: {mw}softcap={sizes['softcap']} must be positive")
            mask = m.get("mask")
            if mask is not None and not isinstance(mask, Mapping):
                raise ConfigError(f"config.json: {mw}mask must be an object with 'size', or null")
            sizes["window"] = _int(mask, "size", mw + "mask.") if mask is not None else None
            rot = _rotation(m, mw, sizes["dim"])
            if m.get("kv_from") is not None:
                kv_from = m["kv_from"]
                if isinstance(kv_from, bool) or not isinstance(kv_from, int) or not 0 <= kv_from < i:
                    raise ConfigError(f"config.json: {mw}kv_from={kv_from!r} must name an earlier layer")
                src = layers[kv_from]
                if src.type != "attention" or src.kv_from is not None:
                    raise ConfigError(f"config.json: {mw}kv_from={kv_from} must name an attention layer with projections of its own")
                same = all(src.mixer[k] == sizes[k] for k in ("heads", "kv_heads", "dim", "vdim")) and src.rot == rot
                if not same:
                    raise ConfigError(f"config.json: {mw}kv_from={kv_from}: head counts, head sizes and rotation must equal that layer's")
        elif kind == "channel_delta":
            sizes = {k: _int(m, k, mw) for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
            if sizes["heads"] % sizes["kv_heads"]:
                raise ConfigError(f"config.json: {mw}heads={sizes['heads']} is no multiple of kv_heads={sizes['kv_heads']}")
            # the two low ranks are sizes that only the tensors' shapes give; config.json may name them
            for k in ("decay_rank", "gate_rank"):
                sizes[k] = _int(m, k, mw) if k in m else None
        elif kind == "lightning":
            sizes = {k: _int(m, k, mw) for k in ("heads", "dim", "vdim")}
            decay = m.get("decay")
            if not isinstance(decay, list) or len(decay) != sizes["heads"] or any(
                    isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
                raise ConfigError(f"config.json: {mw}decay must list one number per head ({sizes['heads']})")
            sizes["decay"] = tuple(float(d) for d in decay)
        else:
            raise ConfigError(f"config.json: {where}type={kind!r} is not a mixer of this design ({', '.join(MIXER_TYPES)})")
        f = entry.get("mlp")
        ff = 0
        if f is not None:
            if not isinstance(f, Mapping):
                raise ConfigError(f"config.json: {where}mlp must be an object or null")
            if f.get("kind", "dense") != "dense":
                raise ConfigError(f"config.json: {where}mlp.kind={f.get('kind')!r} is not 'dense'")
            ff = _int(f, "ff", where + "mlp.")
        layers.append(KevatarLayer(kind, sizes, rot, kv_from, ff))
    max_positions = _int(raw, "max_positions", "") if "max_positions" in raw else DEFAULT_MAX_POSITIONS
    return KevatarConfig(vocab=_int(raw, "vocab", ""), width=_int(raw, "width", ""), eps=eps, embedding_scale=emb_scale,
                         side_dim=side_dim, layers=tuple(layers), max_positions=max_positions, raw=dict(raw))


def low_ranks_from_shapes(raw: Dict[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Dict[str, Any]:
    """config.json with the low ranks of every ``channel_delta`` layer filled in from the tensors' shapes (``l<i>.mix.a1`` is
    ``[decay_rank, width]``, ``l<i>.mix.g1`` ``[gate_rank, width]``) where it does not name them."""
    out = dict(raw)
    layers = []
    for i, entry in enumerate(raw.get("layers", [])):
        if isinstance(entry, Mapping) and entry.get("type") == "channel_delta" and isinstance(entry.get("mixer"), Mapping):
            m = dict(entry["mixer"])
            for key, tensor in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                if key not in m and tensor in shapes:
                    m[key] = int(shapes[tensor][0])
            entry = dict(entry)
            entry["mixer"] = m
        layers.append(entry)
    out["layers"] = layers
    return out


def build_kevatar_spec(cfg: KevatarConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.eps, "name": name})

    # what a layer's cache must keep: its own window, or more where a layer that reads it looks further back
    keep: Dict[int, Optional[int]] = {}
    for i, layer in enumerate(cfg.layers):
        if layer.type == "attention":
            owner = i if layer.kv_from is None else layer.kv_from
            w = layer.mixer["window"]
            if owner not in keep:
                keep[owner] = w
            elif keep[owner] is not None:
                keep[owner] = None if w is None else max(keep[owner], w)
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "attention":
            rot = layer.rot
            position = PartSpec("rope_span", {
                "head_dim": m["dim"], "dims": rot.dims if rot else 0, "theta": rot.base if rot else 10000.0, "interleaved": True,
                "scaling": dict(rot.scaling) if rot and rot.scaling else None, "unit_rms_eps": cfg.eps})
            names = {"q": "q", "o": "o"} if layer.kv_from is not None else {"q": "q", "k": "k", "v": "v", "o": "o"}
            own = layer.kv_from is None
            mixer = PartSpec("attention", {
                "hidden_size": cfg.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "v_head_dim": m["vdim"], "position": position, "qkv_bias": False, "scale": m["scale"], "softcap": m["softcap"],
                "window": m["window"], "shared_kv": not own, "names": names,
                "cache_window": keep[i] if own else "own"})
        elif layer.type == "channel_delta":
            if m["decay_rank"] is None or m["gate_rank"] is None:
                raise ConfigError(f"config.json: layers[{i}].mixer: 'decay_rank' and 'gate_rank' are neither named nor known "
                                  "from the tensors' shapes")
            mixer = PartSpec("channel_delta", {
                "hidden_size": cfg.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                "conv": m["conv"], "decay_rank": m["decay_rank"], "gate_rank": m["gate_rank"], "eps": cfg.eps})
        else:
            mixer = PartSpec("lightning", {"hidden_size": cfg.width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                           "decay": m["decay"], "eps": cfg.eps})
        ffn, norms = None, {"norm1": norm("norm1")}
        prefixes = {"mixer": "mix.", "ffn": "mlp.", "norm1": "", "norm2": "", "side": "side.", "norm_side": "side."}
        extra = {}
        if layer.ff:
            norms["norm2"] = norm("norm2")
            ffn = PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.ff,
                                         "names": {"gate": "gate", "up": "up", "down": "down"}})
        if cfg.side_dim:
            norms["norm_side"] = norm("norm")
            extra["side"] = ("ffn", PartSpec("token_gated_table", {"hidden_size": cfg.width, "dim": cfg.side_dim, "table": SIDE_TABLE,
                                                                     "col0": i * cfg.side_dim}))
        layers.append(LayerSpec(block="branch_norm", mixer=mixer, ffn=ffn, norms=norms, prefixes=prefixes, extra=extra))
    schedule = []
    for i, layer in enumerate(cfg.layers):
        schedule.append(LayerCall(i, cache_of=layer.kv_from))          # no loops: call i is layer i
    tables = {SIDE_TABLE: ("side.embed", len(cfg.layers) * cfg.side_dim)} if cfg.side_dim else {}
    return ModelSpec(
        architecture="Kevatar", vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers), schedule=tuple(schedule),
        final_norm=norm("norm"), tie_word_embeddings=True, max_position_embeddings=cfg.max_positions,
        layer_prefix="l{i}.", embed_name="embed", final_norm_prefix="final.", head_name="head",
        embedding=PartSpec("scaled_token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": cfg.embedding_scale,
                                                      "name": "embed", "token_tables": tables}),
        head=PartSpec("output_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": True, "name": "head"}))


KEVATAR = register_architecture("Kevatar", model_types=("kevatar",), parse=parse_kevatar_config, build_spec=build_kevatar_spec,
                                kernel_libraries=("rowwise", "ssm", "linrec"), sizes_from_shapes=low_ranks_from_shapes)
