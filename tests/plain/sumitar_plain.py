"""A plain, slow implementation of the Sumitar forward pass: whole sequences, no cache, one function per mechanism, on the
CPU in float64 (or float32).  It shares no code with ``zedinfer_b200``: it reads ``config.json`` with ``json`` and
``model.safetensors`` with its own few lines.

The design in this file's notation (``x`` the residual stream, ``t`` a token's index in its sequence, ``sg`` the logistic
function, ``U(v) = v / sqrt(mean(v^2) + eps)``, ``T(v; a, w, b) = tanh(a v) * w + b`` the norm of the layers):

    x_t = E[token_t]
    per layer:     x += T1b(mixer(T1(x)));   x += T2b(ff(T2(x)))            (a norm before and one after every sublayer)
    logits = E Tf(x)

    parallel:      two mixers read the same input; the result is (U(left) * w_l + U(right) * w_r) / 2
      left         attention with H query heads on G key/value heads (biases on q, k, v), the first r entries of every q and
                   k head turned, pair (i, i + r/2) by the angle t * base^(-2i/r); score = q . k * scale * temp_head; key j
                   answers query t when 0 <= t - j < W; softmax; Wo on the concatenated heads
      right        q = silu(Wq h), v = Wv h, f = l + (1 - l) sg(Wf h + bf);  per head  S <- diag(f) S + (1 - f) v^T;
                   o = S^T q;  out = Wo concat(U(o) * w_n)                    (U over a head's value entries)
    delta:         q, k, v = silu(conv(Wq h)), silu(conv(Wk h)), silu(conv(Wv h))   (causal per-channel convolution)
                   q <- q / sqrt(|q|^2 + 1e-6) / sqrt(dim),  k <- k / sqrt(|k|^2 + 1e-6)           per head
                   beta = sg(Wb h);  g = exp(-exp(A_head) softplus(Wa h + dt_head))                one decay per head
                   per head:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
                   out = Wo (U(o) * w_n * silu(Wg h))
    dense ff:      Wdown P(Wup h),  P(z) = a U(z) + b U(z^2) + c U(z^3) + e   (powers entry by entry, U over the ff entries)
    routed ff:     s = softmax(Wr h) over all experts, identity ones included;  chosen: the ``top`` largest s + correction;
                   y = sum_chosen s_e expert_e(h)  (an identity expert returns h)  + sg(w_sg . h) shared(h);
                   expert(h) = Wdown (silu(Wgate h) * (Wup h))
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List

import torch

UNIT_EPS = 1e-6                  # inside the root of the delta rule's unit vectors


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


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def tanh_norm(x: torch.Tensor, w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def turn_span(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [tokens, heads, dim]: entry i of the first ``dims`` pairs with entry i + dims / 2."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    lo, hi = x[..., :half], x[..., half:dims]
    return torch.cat([lo * c - hi * s, hi * c + lo * s, x[..., dims:]], dim=-1)


def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(n, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(n, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(n, G, dv)
    pos = torch.arange(n)
    q, k = turn_span(q, pos, m["rot"]["dims"], m["rot"]["base"]), turn_span(k, pos, m["rot"]["dims"], m["rot"]["base"])
    dist = pos[:, None] - pos[None, :]
    seen = (dist >= 0) & (dist < m["mask"]["size"])
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"] * w[p + "temp"][a]
        s = s.masked_fill(~seen, float("-inf"))
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(n, H * dv) @ w[p + "o"].T


def forget_gate_recurrence(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(n, H, d)
    v = (h @ w[p + "v"].T).view(n, H, dv)
    low = w[p + "lower"]
    f = (low + (1.0 - low) * logistic(h @ w[p + "f"].T + w[p + "f.b"])).view(n, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(n, H, dv, dtype=h.dtype)
    for t in range(n):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_unit(o, eps) * w[p + "norm"]
    return o.reshape(n, H * dv) @ w[p + "o"].T


def parallel_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    left = window_attention(h, w, p + "left.", m["left"])
    right = forget_gate_recurrence(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_unit(left, eps) * w[p + "left.out"] + rms_unit(right, eps) * w[p + "right.out"])


def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [tokens, channels], taps [channels, K]: the last column weighs the token itself; zeros before the start."""
    n, K = x.shape[0], taps.shape[1]
    out = torch.zeros_like(x)
    for j in range(K):
        back = K - 1 - j
        if back < n:
            out[back:] += x[:n - back] * taps[:, j]
    return out


def gated_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(n, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(n, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(n, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + UNIT_EPS) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + UNIT_EPS)
    beta = logistic(h @ w[p + "b"].T)                                                       # [n, H]
    g = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))   # [n, H]
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(n, H, dv, dtype=h.dtype)
    for t in range(n):
        for a in range(H):
            kk, qq = k[t, a // (H // G)], q[t, a // (H // G)]
            S[a] = g[t, a] * S[a]
            u = beta[t, a] * (v[t, a] - S[a].T @ kk)
            S[a] = S[a] + kk[:, None] * u[None, :]
            o[t, a] = S[a].T @ qq
    o = rms_unit(o, eps) * w[p + "norm"] * silu(h @ w[p + "g"].T).view(n, H, dv)
    return o.reshape(n, H * dv) @ w[p + "o"].T


def poly_norm_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    z = h @ w[p + "up"].T
    a, b, c, e = [w[p + "act"][i] for i in range(4)]
    act = a * rms_unit(z, eps) + b * rms_unit(z * z, eps) + c * rms_unit(z * z * z, eps) + e
    return act @ w[p + "down"].T


def gated_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def router_choice(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, top: int):
    """(chosen experts [tokens, top], their weights): scores over all experts, the choice by score + correction."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    pick = s + w[p + "correction"]
    order = sorted(range(pick.shape[1]), key=lambda e: e)
    idx = torch.empty(h.shape[0], top, dtype=torch.long)
    for t in range(h.shape[0]):
        ranked = sorted(order, key=lambda e: (-float(pick[t, e]), e))
        idx[t] = torch.tensor(ranked[:top])
    return idx, torch.gather(s, 1, idx)


def routed_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    r = f["router"]
    real = r["experts"]
    idx, wts = router_choice(h, w, p, r["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(idx[t, j])
            y = gated_ff(h[t:t + 1], w, f"{p}e{e}.")[0] if e < real else h[t]
            out[t] += wts[t, j] * y
    if f.get("shared") is not None:
        out = out + logistic(h @ w[p + "shared.sg"].T) * gated_ff(h, w, p + "shared.")
    return out


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], trace: List[torch.Tensor] = None) -> torch.Tensor:
    """Logits [tokens, vocab] of one sequence; ``trace`` collects the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = tanh_norm(x, w, p + "norm1")
        if layer["type"] == "parallel":
            y = parallel_mixer(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "delta":
            y = gated_delta(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        x = x + tanh_norm(y, w, p + "norm1b")
        f = layer.get("mlp")
        if f is not None:
            h = tanh_norm(x, w, p + "norm2")
            y = poly_norm_ff(h, w, p + "mlp.", eps) if f["kind"] == "dense" else routed_ff(h, w, p + "mlp.", f)
            x = x + tanh_norm(y, w, p + "norm2b")
        if trace is not None:
            trace.append(x.clone())
    return tanh_norm(x, w, "final.norm") @ w["embed"].T


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(torch.argmax(forward(cfg, w, seq)[-1])))
    return seq[len(prompt):]
