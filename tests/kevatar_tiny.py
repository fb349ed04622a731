"""Tiny Kevatar configurations for the tests.  They differ in every size and option: the three mixers in several orders,
query heads that share key/value heads and that do not, value heads smaller and larger than the query/key heads, turned
spans from 2 entries to a whole head with and without stretched frequencies (ramps that lie inside the span, below it and
above it), windows from 3 keys to none, layers that read another layer's keys through a window larger and smaller than the
owner's, score caps and none, convolutions of 1 to 4 taps, low ranks that differ from one another and from the per-token
table's width, models without that table, without a feed-forward in some layers, with an embedding scale and without, and
models of recurrent layers alone (no paged cache) and of attention alone (no state slot), and one of ones and extremes."""
import copy
import json
import os


def _rot(dims, base, scaling=None):
    return {"base": base, "dims": dims, "scaling": scaling}


def _stretch(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def _attn(heads, kv, dim, vdim, window, rot, scale, softcap=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": None if window is None else {"size": window},
         "rot": rot, "scale": scale, "softcap": softcap}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def _delta(heads, kv, dim, vdim, conv, decay_rank, gate_rank):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": decay_rank, "gate_rank": gate_rank}}


def _lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def _with(layer, ff):
    out = dict(layer)
    out["mlp"] = None if ff is None else {"kind": "dense", "ff": ff}
    return out


# a lightning layer first; grouped heads; two readers of layer 1's keys, one looking further back than the owner and one
# less far; a stretched span whose ramp lies inside it
_ROT_A = _rot(16, 5000.0, _stretch(8.0, 64, 16.0, 2.0))
KV_A = {
    "architecture": "Kevatar", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.5},
    "token_side": {"dim": 10},
    "layers": [
        _with(_lightning(3, 16, 24, (0.5, 0.9, 0.99)), 80),
        _with(_attn(4, 2, 32, 16, 13, _ROT_A, 0.2, softcap=5.0), 64),
        _with(_delta(4, 2, 16, 24, 3, 6, 14), None),
        _with(_attn(4, 2, 32, 16, 29, _ROT_A, 0.15, softcap=12.0, kv_from=1), 48),
        _with(_attn(4, 2, 32, 16, 5, _ROT_A, 0.3, kv_from=1), 72),
    ],
}
# the tensor-core attention kernels: rows of 64 and 128 with pages of 16; a whole head turned without a stretch, a capped
# and an uncapped layer; no per-token table, no embedding scale
KV_B = {
    "architecture": "Kevatar", "vocab": 500, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        _with(_attn(2, 1, 64, 64, 40, _rot(64, 10000.0), 0.125), 96),
        _with(_delta(2, 2, 32, 64, 4, 8, 8), 160),
        _with(_attn(4, 4, 128, 128, 70, _rot(32, 300.0, _stretch(2.0, 32, 8.0, 0.5)), 0.09, softcap=20.0), None),
        _with(_lightning(2, 64, 32, (0.97, 0.8)), 64),
        _with(_attn(4, 4, 128, 128, 33, _rot(32, 300.0, _stretch(2.0, 32, 8.0, 0.5)), 0.11, softcap=8.0, kv_from=2), 64),
    ],
}
# sizes that fit no vector width: heads of 24 with values of 40 and 2 turned entries, one lightning head, a convolution of
# one tap (no history), a layer that sees every key, a window of 3, a table of 3 columns per layer; a stretch whose ramp
# lies below the span (every frequency divided by the factor)
KV_C = {
    "architecture": "Kevatar", "vocab": 173, "width": 72, "norm": {"eps": 1e-4}, "embedding": {"scale": 0.5},
    "token_side": {"dim": 3},
    "layers": [
        _with(_attn(3, 3, 24, 40, None, _rot(2, 77.0), 0.3, softcap=3.0), 40),
        _with(_delta(2, 2, 72, 8, 1, 5, 3), 24),
        _with(_lightning(1, 40, 20, (0.93,)), None),
        _with(_attn(6, 2, 16, 8, 3, _rot(12, 900.0, _stretch(16.0, 4096, 200000.0, 100000.0)), 0.25), 56),
    ],
}
# recurrent layers alone: no paged cache at all; key sizes on every width of the recurrence kernel (8, 40, 136 entries)
KV_D = {
    "architecture": "Kevatar", "vocab": 150, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0},
    "token_side": {"dim": 16},
    "layers": [
        _with(_delta(3, 1, 136, 12, 2, 4, 20), 48),
        _with(_lightning(4, 8, 136, (0.2, 0.7, 0.95, 0.9995)), 32),
        _with(_delta(6, 3, 40, 20, 4, 16, 2), None),
    ],
}
# attention alone: no state slot; a stretch whose ramp lies above the span (no frequency changes, only the factor on
# cosines and sines), a reader right behind its owner
_ROT_E = _rot(8, 100.0, _stretch(4.0, 8, 0.001, 0.0001))
KV_E = {
    "architecture": "Kevatar", "vocab": 99, "width": 40, "norm": {"eps": 1e-6},
    "layers": [
        _with(_attn(2, 1, 16, 24, 17, _ROT_E, 0.2, softcap=30.0), 32),
        _with(_attn(2, 1, 16, 24, 64, _ROT_E, 0.4, kv_from=0), None),
    ],
}
# ones and extremes: single heads everywhere, a window of one key (a token sees itself alone) read again through a window of
# two, a whole head of 8 turned, a cap of 1 that bends every score, six taps, a key of 256 entries on the widest form of the
# recurrence kernel beside one of 4, low ranks of 1, a table of one column, a decay of 1 (nothing fades) and one of 0
# (nothing is kept)
KV_F = {
    "architecture": "Kevatar", "vocab": 64, "width": 48, "norm": {"eps": 1e-6}, "token_side": {"dim": 1},
    "layers": [
        _with(_attn(1, 1, 8, 8, 1, _rot(8, 10.0), 1.0, softcap=1.0), 8),
        _with(_delta(1, 1, 256, 4, 6, 1, 1), 16),
        _with(_lightning(2, 4, 4, (1.0, 0.0)), None),
        _with(_attn(1, 1, 8, 8, 2, _rot(8, 10.0), 0.7, kv_from=0), 24),
    ],
}
CONFIGS = {"A": (KV_A, 41), "B": (KV_B, 42), "C": (KV_C, 43), "D": (KV_D, 44), "E": (KV_E, 45), "F": (KV_F, 46)}
INIT_SCALE = 5.0


def make_model_dir(tmp_root, name, dtype="bfloat16", strip_ranks=False):
    """Write the folder with the framework's random-weights writer.  ``strip_ranks``: config.json afterwards names no
    low rank of the delta-rule layers, so that a reader has to take them from the tensors' shapes."""
    from zedinfer_b200.weights import write_random_model
    cfg, seed = CONFIGS[name]
    out = os.path.join(str(tmp_root), f"kevatar_{name}_{dtype}" + ("_bare" if strip_ranks else ""))
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        write_random_model(cfg, seed, out, dtype=dtype, init_scale=INIT_SCALE, name_prefix="")
        if strip_ranks:
            bare = copy.deepcopy(cfg)
            for layer in bare["layers"]:
                layer["mixer"].pop("decay_rank", None)
                layer["mixer"].pop("gate_rank", None)
            with open(os.path.join(out, "config.json"), "w", encoding="utf-8") as f:
                json.dump(bare, f, indent=2)
    return out
