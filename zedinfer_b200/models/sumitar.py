"""Sumitar: config.json -> typed configuration -> :class:`ModelSpec`.

A decoder-only model whose config.json lists its layers one by one (``layers``: ``type``, the mixer's sizes under ``mixer``,
the feed-forward under ``mlp`` or null).  Every sublayer has a norm before and a norm after it, ``x += N1b(mixer(N1(x)));
x += N2b(ff(N2(x)))``, and every norm of the layers and the model's last one is the tanh norm ``tanh(alpha v) * w + b``
(``norm.eps`` belongs to the root-mean-square norms inside the sublayers).  The head is the embedding table.  Two kinds of
layer:

* ``parallel``: two mixers read the same input and are joined as ``(U(left) * w_l + U(right) * w_r) / 2``.  ``left`` is
  grouped-query attention with biases on q, k and v, value heads of their own size, the first ``rot.dims`` entries of every
  query and key head turned in the rotate-half pairing, ``scale`` from the config times one learned number per head
  (``temp``), and a window of ``mask.size`` keys.  ``right`` is a matrix-state recurrence with one gate per key entry, bounded below,
  that fades the state and whose complement stands where a key would (``forget_gate``).
* ``delta``: a gated delta rule with one decay per head, short causal convolutions on q, k and v, and a SiLU gate on the
  normed read-out (``gated_delta``).

The feed-forward is dense, ``down(P(up h))`` with ``P`` a sum of normed powers (``poly_norm_mlp``), or routed: scores are the
softmax over all experts, the choice goes by score + ``correction``, weights are the scores unrenormalised, the last
``router.identity`` router outputs are experts that return their input, and a shared expert, gated by one sigmoid per token,
runs for every token.  Tensor names: ``embed``, ``final.norm`` (+ ``.alpha``, ``.b``), and per layer i ``l<i>.norm1``,
``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.*`` (``left.*`` and ``right.*`` in a parallel layer), ``l<i>.mlp.*``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

LAYER_TYPES = ("parallel", "delta")
# the framework's context limit when config.json names none: the design has no learned positions
DEFAULT_MAX_POSITIONS = 1 << 15


@dataclass(frozen=True)
class SumitarLayer:
    type: str
    mixer: Mapping[str, Any]              # the mixer's sizes and constants, checked (a parallel layer: {"left": ..., "right": ...})
    mlp: Optional[Mapping[str, Any]]      # None: no feed-forward


@dataclass(frozen=True)
class SumitarConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[SumitarLayer, ...]
    max_positions: int
    raw: Mapping[str, Any]

    def to_json_dict(self) -> dict:
        return dict(self.raw)


def _int(obj: Mapping[str, Any], key: str, where: str, least: int = 1) -> int:
    v = obj.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < least:
        raise ConfigError(f"config.json: {where}'{key}' must be an integer of at least {least}, got {v!r}")
    return v


def _num(obj: Mapping[str, Any], key: str, where: str) -> float:
    v = obj.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {v!r}")
    return float(v)


def _obj(obj: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = obj.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


def _left(m: Mapping[str, Any], where: str) -> Dict[str, Any]:
    sizes: Dict[str, Any] = {k: _int(m, k, where) for k in ("heads", "kv_heads", "dim", "vdim")}
    if sizes["heads"] % sizes["kv_heads"]:
        raise ConfigError(f"config.json: {where}heads={sizes['heads']} is no multiple of kv_heads={sizes['kv_heads']}")
    sizes["scale"] = _num(m, "scale", where)
    # a layer without a mask (null, or no key at all) sees every key
    sizes["window"] = _int(_obj(m, "mask", where), "size", where + "mask.") if m.get("mask") is not None else None
    rot = _obj(m, "rot", where)
    sizes["rot_base"], sizes["rot_dims"] = _num(rot, "base", where + "rot."), _int(rot, "dims", where + "rot.")
    if not sizes["rot_base"] > 0.0 or sizes["rot_dims"] % 2 or sizes["rot_dims"] > sizes["dim"]:
        raise ConfigError(f"config.json: {where}rot: base={sizes['rot_base']} must be positive and dims={sizes['rot_dims']} even "
                          f"and at most {sizes['dim']}")
    return sizes


def _mlp(f: Any, where: str) -> Optional[Dict[str, Any]]:
    if f is None:
        return None
    if not isinstance(f, Mapping):
        raise ConfigError(f"config.json: {where}mlp must be an object or null")
    kind = f.get("kind")
    if kind == "dense":
        return {"kind": "dense", "ff": _int(f, "ff", where + "mlp.")}
    if kind == "moe":
        r = _obj(f, "router", where + "mlp.")
        out: Dict[str, Any] = {"kind": "moe", "ff": _int(_obj(f, "expert", where + "mlp."), "ff", where + "mlp.expert."),
                               "experts": _int(r, "experts", where + "mlp.router."), "top": _int(r, "top", where + "mlp.router."),
                               "identity": _int(r, "identity", where + "mlp.router.", least=0) if "identity" in r else 0}
        if out["top"] > out["experts"] + out["identity"]:
            raise ConfigError(f"config.json: {where}mlp.router: top={out['top']} of {out['experts']} + {out['identity']} experts")
        shared = f.get("shared")
        if shared is not None and not isinstance(shared, Mapping):
            raise ConfigError(f"config.json: {where}mlp.shared must be an object or null")
        out["shared_ff"] = _int(shared, "ff", where + "mlp.shared.") if shared is not None else 0
        return out
    raise ConfigError(f"config.json: {where}mlp.kind={kind!r} is neither 'dense' nor 'moe'")


def parse_sumitar_config(raw: Mapping[str, Any]) -> SumitarConfig:
    missing = [k for k in ("vocab", "width", "layers", "norm") if k not in raw]
    if missing:
        raise ConfigError("config.json: missing required key(s): " + ", ".join(missing))
    if not isinstance(raw["layers"], list) or not raw["layers"]:
        raise ConfigError("config.json: 'layers' must be a list with at least one layer")
    eps = _num(_obj(raw, "norm", ""), "eps", "norm.")
    if not eps > 0.0:
        raise ConfigError(f"config.json: norm.eps={eps} must be positive")
    layers = []
    for i, entry in enumerate(raw["layers"]):
        where = f"layers[{i}]."
        if not isinstance(entry, Mapping):
            raise ConfigError(f"config.json: layers[{i}] must be an object")
        kind, m, mw = entry.get("type"), _obj(entry, "mixer", where), where + "mixer."
        if kind == "parallel":
            right = _obj(m, "right", mw)
            sizes: Dict[str, Any] = {"left": _left(_obj(m, "left", mw), mw + "left."),
                                     "right": {k: _int(right, k, mw + "right.") for k in ("heads", "dim", "vdim")}}
        elif kind == "delta":
            sizes = {k: _int(m, k, mw) for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
            if sizes["heads"] % sizes["kv_heads"]:
                raise ConfigError(f"config.json: {mw}heads={sizes['heads']} is no multiple of kv_heads={sizes['kv_heads']}")
        else:
            raise ConfigError(f"config.json: {where}type={kind!r} is not a layer of this design ({', '.join(LAYER_TYPES)})")
        layers.append(SumitarLayer(kind, sizes, _mlp(entry.get("mlp"), where)))
    max_positions = _int(raw, "max_positions", "") if "max_positions" in raw else DEFAULT_MAX_POSITIONS
    return SumitarConfig(vocab=_int(raw, "vocab", ""), width=_int(raw, "width", ""), eps=eps, layers=tuple(layers),
                         max_positions=max_positions, raw=dict(raw))


def build_sumitar_spec(cfg: SumitarConfig) -> ModelSpec:
    def tanh_norm(name: str) -> PartSpec:
        return PartSpec("tanh_norm", {"size": cfg.width, "name": name})

    def gated(ff: int) -> PartSpec:                       # silu(gate) * up, then down: the clamped form without a limit
        return PartSpec("clamped_gated_mlp", {"hidden_size": cfg.width, "intermediate_size": ff, "limit": None})

    layers = []
    for layer in cfg.layers:
        m = layer.mixer
        norms = {"norm1": tanh_norm("norm1"), "norm1b": tanh_norm("norm1b")}
        prefixes = {"mixer": "mix.", "ffn": "mlp.", "norm1": "", "norm1b": "", "norm2": "", "norm2b": ""}
        extra = {}
        if layer.type == "parallel":
            lf, rt = m["left"], m["right"]
            position = PartSpec("rope_span", {"head_dim": lf["dim"], "dims": lf["rot_dims"], "theta": lf["rot_base"], "interleaved": False})
            mixer = PartSpec("attention", {
                "hidden_size": cfg.width, "num_heads": lf["heads"], "num_kv_heads": lf["kv_heads"], "head_dim": lf["dim"],
                "v_head_dim": lf["vdim"], "position": position, "qkv_bias": True, "scale": lf["scale"], "window": lf["window"],
                "head_scale": "temp",
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b"}})
            extra["mixer2"] = ("mixer", PartSpec("forget_gate", {"hidden_size": cfg.width, "heads": rt["heads"], "dim": rt["dim"],
                                                                  "vdim": rt["vdim"], "eps": cfg.eps}))
            for role, prefix in (("mix_out", "mix.left."), ("mix2_out", "mix.right.")):
                norms[role] = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.eps, "name": "out", "float32_weight": True})
                prefixes[role] = prefix
            prefixes.update({"mixer": "mix.left.", "mixer2": "mix.right."})
        else:
            mixer = PartSpec("gated_delta", {"hidden_size": cfg.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
                                             "vdim": m["vdim"], "conv": m["conv"], "eps": cfg.eps})
        ffn = None
        f = layer.mlp
        if f is not None:
            norms.update({"norm2": tanh_norm("norm2"), "norm2b": tanh_norm("norm2b")})
            if f["kind"] == "dense":
                ffn = PartSpec("poly_norm_mlp", {"hidden_size": cfg.width, "intermediate_size": f["ff"], "eps": cfg.eps})
            else:
                ffn = PartSpec("routed_experts", {
                    "hidden_size": cfg.width, "intermediate_size": f["ff"], "experts": f["experts"], "top": f["top"],
                    "identity": f["identity"], "router_bias": False, "score": "softmax_all", "choice_bias_name": "correction",
                    "shared": gated(f["shared_ff"]) if f["shared_ff"] else None,
                    "shared_gate_name": "sg" if f["shared_ff"] else None})
        layers.append(LayerSpec(block="sandwich_norm", mixer=mixer, ffn=ffn, norms=norms, prefixes=prefixes, extra=extra))
    schedule = tuple(LayerCall(i) for i in range(len(layers)))          # no loops: call i is layer i
    return ModelSpec(
        architecture="Sumitar", vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers), schedule=schedule,
        final_norm=tanh_norm("norm"), tie_word_embeddings=True, max_position_embeddings=cfg.max_positions,
        layer_prefix="l{i}.", embed_name="embed", final_norm_prefix="final.", head_name="head")


SUMITAR = register_architecture("Sumitar", model_types=("sumitar",), parse=parse_sumitar_config, build_spec=build_sumitar_spec,
                                kernel_libraries=("rowwise", "moe", "ssm", "linrec"))
