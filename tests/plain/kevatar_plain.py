"""A plain, slow implementation of the Kevatar forward pass: whole sequences, no cache, one function per mechanism,
on the CPU in float64 (or float32).  It shares no code with ``zedinfer_b200``: it reads ``config.json`` with ``json``
and ``model.safetensors`` with its own few lines.

The design in this file's notation (``x`` the residual stream, ``U(v) = v / sqrt(mean(v^2) + eps)``, ``t`` a token's
index in its sequence, ``sg`` the logistic function):

    x_t = c_e * E[token_t]
    per layer l:   x += U(mixer(x)) * w1;   x += U(ff(x)) * w2      (the norm sits on the branch's OUTPUT; ff may be absent)
                   x += U(P_l (gelu_tanh(G_l x) * T[token_t, l d : (l + 1) d])) * w_s      (the token's own entry, d wide)
    logits = E (U(x) * w_f)                                         (the table itself, without c_e)

    attention:     q = Wq h, k = Wk h, v = Wv h;  the first r entries of every q and k head turn, pair (2i, 2i + 1) by the
                   angle t * f_i;  f_i = b^(-2i/r), stretched for long contexts: with
                   D(n) = r ln(L / (2 pi n)) / (2 ln b), lo = max(floor(D(fast)), 0), hi = min(ceil(D(slow)), r - 1),
                   m_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1):  f_i <- f_i / F * m_i + f_i * (1 - m_i), and
                   cos, sin are multiplied by 0.1 ln(F) + 1.
                   then every q and k head is divided by its root mean square;  s = c * tanh(scale * (q . k) / c);
                   key j answers query t when 0 <= t - j < W;  softmax;  out = Wo concat(heads).
                   A layer may use the turned, normed keys and the values of an earlier layer instead of its own.
    channel_delta: q, k, v = conv_silu(Wq h), conv_silu(Wk h), conv_silu(Wv h)   (causal per-channel convolution, then silu)
                   q <- q / sqrt(|q|^2 + 1e-6) / sqrt(dim),  k <- k / sqrt(|k|^2 + 1e-6)        per head
                   beta = sg(Wb h);   g = exp(-exp(A_a) * softplus(Wa2 Wa1 h + dt_bias))      (a decay per head and key entry)
                   per head:  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
                   out = Wo (U(o) * w_n * sg(Wg2 Wg1 h))                              (U over each head's value entries)
    lightning:     q, k, v = silu(Wq h), silu(Wk h), silu(Wv h);  per head  S <- lambda_a S + k v^T;  o = S^T q
                   out = Wo (U(concat(o)) * w_n * sg(Wg h))                            (U over all heads at once)
    dense ff:      Wdown (silu(Wgate h) * (Wup h))
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import torch

UNIT_EPS = 1e-6                  # inside the root of the unit vectors of channel_delta


# ---------------------------------------------------------------------------------------------
# files
# ---------------------------------------------------------------------------------------------
def read_safetensors(path: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    kinds = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[b:e]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t.to(dtype) if t.is_floating_point() else t.clone()
    return out


def read_model(model_dir: str, dtype=torch.float64):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"), dtype)


# ---------------------------------------------------------------------------------------------
# mechanisms, one function each
# ---------------------------------------------------------------------------------------------
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


def logistic(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def stretched_frequencies(rot: dict, dtype) -> (torch.Tensor, float):
    """The angle per position of every pair of the turned span, and the factor on cosines and sines."""
    r, base = rot["dims"], float(rot["base"])
    i = torch.arange(r // 2, dtype=dtype)
    f = torch.pow(torch.tensor(base, dtype=dtype), -2.0 * i / r)
    sc = rot.get("scaling")
    if sc is None:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turns_to_index(n: float) -> float:
        return r * math.log(orig / (2.0 * math.pi * n)) / (2.0 * math.log(base))

    lo = max(math.floor(turns_to_index(float(sc["fast"]))), 0)
    hi = min(math.ceil(turns_to_index(float(sc["slow"]))), r - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def turn_pairs(v: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """``v [T, heads, D]``: the first ``rot.dims`` entries of each head turn, pair (2i, 2i + 1)."""
    if rot is None:
        return v
    r = rot["dims"]
    f, mag = stretched_frequencies(rot, v.dtype)
    ang = positions.to(v.dtype)[:, None] * f[None, :]
    cos, sin = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    out = v.clone()
    a, b = v[..., 0:r:2], v[..., 1:r:2]
    out[..., 0:r:2] = a * cos - b * sin
    out[..., 1:r:2] = b * cos + a * sin
    return out


def attention_keys_values(h: torch.Tensor, positions: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float):
    """What the layer's cache holds: keys after turn and norm ``[T, G, dim]`` and values ``[T, G, vdim]``."""
    t = h.shape[0]
    k = (h @ w[p + "k"].T).view(t, m["kv_heads"], m["dim"])
    v = (h @ w[p + "v"].T).view(t, m["kv_heads"], m["vdim"])
    return rms_unit(turn_pairs(k, positions, m.get("rot")), eps), v


def attention_mixer(h: torch.Tensor, positions: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float,
                    k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    t = h.shape[0]
    heads, groups, dim = m["heads"], m["kv_heads"], m["dim"]
    q = rms_unit(turn_pairs((h @ w[p + "q"].T).view(t, heads, dim), positions, m.get("rot")), eps)
    kk = k.repeat_interleave(heads // groups, dim=1)
    vv = v.repeat_interleave(heads // groups, dim=1)
    s = torch.einsum("thd,jhd->htj", q, kk) * float(m["scale"])
    cap = m.get("softcap")
    if cap is not None:
        s = float(cap) * torch.tanh(s / float(cap))
    dist = positions[:, None] - positions[None, :]                        # query minus key
    seen = dist >= 0
    if m.get("mask") is not None:
        seen = seen & (dist < int(m["mask"]["size"]))
    s = s.masked_fill(~seen[None], float("-inf"))
    pr = torch.softmax(s, dim=-1)
    o = torch.einsum("htj,jhd->thd", pr, vv).reshape(t, heads * m["vdim"])
    return o @ w[p + "o"].T


def causal_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """``u [T, C]``, ``taps [C, K]`` with the last column on the present token; zeros before the start."""
    t, k = u.shape[0], taps.shape[1]
    out = torch.zeros_like(u)
    for j in range(k):
        back = k - 1 - j
        if back < t:
            out[back:] += u[:t - back] * taps[:, j][None, :]
    return out


def channel_delta_mixer(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    t = h.shape[0]
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(t, groups, dim)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(t, groups, dim)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(t, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + UNIT_EPS) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + UNIT_EPS)
    q, k = q.repeat_interleave(heads // groups, dim=1), k.repeat_interleave(heads // groups, dim=1)
    beta = logistic(h @ w[p + "b"].T)                                      # [T, heads]
    a = ((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(t, heads, dim)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * softplus(a))
    o = torch.zeros(t, heads, vdim, dtype=h.dtype)
    for a_ in range(heads):
        s = torch.zeros(dim, vdim, dtype=h.dtype)
        for i in range(t):
            s = g[i, a_][:, None] * s
            u = beta[i, a_] * (v[i, a_] - s.T @ k[i, a_])
            s = s + torch.outer(k[i, a_], u)
            o[i, a_] = s.T @ q[i, a_]
    gate = logistic(((h @ w[p + "g1"].T) @ w[p + "g2"].T)).view(t, heads, vdim)
    y = rms_unit(o, eps) * w[p + "norm"][None, None, :] * gate
    return y.reshape(t, heads * vdim) @ w[p + "o"].T


def lightning_mixer(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    t = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(t, heads, dim)
    k = silu(h @ w[p + "k"].T).view(t, heads, dim)
    v = silu(h @ w[p + "v"].T).view(t, heads, vdim)
    o = torch.zeros(t, heads, vdim, dtype=h.dtype)
    for a in range(heads):
        s = torch.zeros(dim, vdim, dtype=h.dtype)
        lam = float(m["decay"][a])
        for i in range(t):
            s = lam * s + torch.outer(k[i, a], v[i, a])
            o[i, a] = s.T @ q[i, a]
    y = rms_unit(o.reshape(t, heads * vdim), eps) * w[p + "norm"] * logistic(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def token_side(x: torch.Tensor, tokens: torch.Tensor, layer: int, d: int, w: Dict[str, torch.Tensor], p: str, eps: float):
    e = w["side.embed"][tokens][:, layer * d:(layer + 1) * d]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return rms_unit(y, eps) * w[p + "norm"]


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], return_layers: bool = False):
    """Logits ``[T, vocab]`` of a whole sequence (and the residual stream after every layer)."""
    dtype = w["embed"].dtype
    ids = torch.tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][ids] * float(cfg.get("embedding", {}).get("scale", 1.0))
    side = cfg.get("token_side")
    kept = {}                                                              # layer -> (keys, values)
    after = []
    for l, layer in enumerate(cfg["layers"]):
        p, m = f"l{l}.", layer["mixer"]
        if layer["type"] == "attention":
            if m.get("kv_from") is None:
                kept[l] = attention_keys_values(x, positions, m, w, p + "mix.", eps)
            k, v = kept[l if m.get("kv_from") is None else int(m["kv_from"])]
            y = attention_mixer(x, positions, m, w, p + "mix.", eps, k, v)
        elif layer["type"] == "channel_delta":
            y = channel_delta_mixer(x, m, w, p + "mix.", eps)
        elif layer["type"] == "lightning":
            y = lightning_mixer(x, m, w, p + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_unit(y, eps) * w[p + "norm1"]
        if layer.get("mlp") is not None:
            x = x + rms_unit(dense_ff(x, w, p + "mlp."), eps) * w[p + "norm2"]
        if side is not None:
            x = x + token_side(x, ids, l, int(side["dim"]), w, p + "side.", eps)
        after.append(x.clone())
    logits = (rms_unit(x, eps) * w["final.norm"]) @ w["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(torch.argmax(forward(cfg, w, seq)[-1])))
    return seq[len(prompt):]
