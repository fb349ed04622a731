"""Tiny Sumitar configurations for the tests.  They differ in every size and option: both kinds of layer in several orders,
query heads that share key/value heads and that do not, value heads smaller, larger than and equal to the query/key heads,
turned spans from 2 entries to a whole head, windows from one key to more than the prompts hold, forget-gate heads on every
width of the recurrence kernel, delta-rule layers whose heads share query/key heads, convolutions of 1 to 6 taps, dense and
routed feed-forwards and none, routers with and without experts that return their input, with and without a shared expert,
choosing one expert, some and all, and models of one kind of layer alone."""
import copy
import os


def _left(heads, kv, dim, vdim, window, rot_dims, base, scale):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": window}, "rot": {"base": base, "dims": rot_dims},
            "scale": scale}


def _parallel(left, right_heads, right_dim, right_vdim):
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": right_heads, "dim": right_dim, "vdim": right_vdim}}}


def _delta(heads, kv, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, identity, top, ff, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


def _with(layer, mlp):
    out = dict(layer)
    out["mlp"] = mlp
    return out


# grouped heads on both kinds of layer, values smaller than keys, every kind of feed-forward
SM_A = {
    "architecture": "Sumitar", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        _with(_parallel(_left(4, 2, 32, 16, 13, 16, 5000.0, 0.2), 3, 16, 24), _dense(80)),
        _with(_delta(4, 2, 16, 24, 3), _moe(5, 1, 2, 24, shared=40)),
        _with(_parallel(_left(2, 2, 16, 40, 29, 8, 300.0, 0.3), 2, 24, 8), _moe(4, 0, 3, 32)),
        _with(_delta(2, 2, 24, 16, 4), None),
    ],
}
# the tensor-core attention kernels: rows of 64 and 128 with pages of 16, a whole head turned, values equal to keys
SM_B = {
    "architecture": "Sumitar", "vocab": 500, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        _with(_parallel(_left(2, 1, 64, 64, 40, 64, 10000.0, 0.125), 2, 32, 64), _moe(6, 2, 2, 48, shared=64)),
        _with(_delta(2, 2, 32, 64, 4), _dense(160)),
        _with(_parallel(_left(4, 4, 128, 128, 70, 32, 300.0, 0.09), 2, 64, 32), None),
        _with(_parallel(_left(4, 2, 64, 128, 33, 24, 2e5, 0.11), 3, 40, 64), _dense(64)),
    ],
}
# sizes that fit no vector width: heads of 24 with values of 40 and 2 turned entries, a window of 3, one forget-gate head, a
# convolution of one tap (no history), a router that chooses one expert among three and two that return the input
SM_C = {
    "architecture": "Sumitar", "vocab": 173, "width": 72, "norm": {"eps": 1e-4},
    "layers": [
        _with(_parallel(_left(3, 3, 24, 40, 3, 2, 77.0, 0.3), 1, 40, 20), _dense(40)),
        _with(_delta(2, 2, 72, 8, 1), _moe(3, 2, 1, 24)),
        _with(_parallel(_left(6, 2, 16, 8, 500, 12, 900.0, 0.25), 5, 8, 12), _moe(2, 1, 3, 16, shared=8)),
    ],
}
# delta-rule layers alone: no paged cache at all; key sizes on every width of the recurrence kernel (8, 40, 136 entries)
SM_D = {
    "architecture": "Sumitar", "vocab": 150, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        _with(_delta(3, 1, 136, 12, 2), _dense(48)),
        _with(_delta(4, 4, 8, 136, 5), _moe(4, 1, 5, 16, shared=24)),
        _with(_delta(6, 3, 40, 20, 4), None),
    ],
}
# parallel layers alone; a width that is a multiple of 4 only; forget-gate keys of 136 and 256 entries
SM_E = {
    "architecture": "Sumitar", "vocab": 99, "width": 52, "norm": {"eps": 1e-6},
    "layers": [
        _with(_parallel(_left(2, 1, 16, 24, 17, 8, 100.0, 0.2), 1, 136, 4), _dense(36)),
        _with(_parallel(_left(1, 1, 8, 8, 64, 4, 10.0, 0.4), 2, 256, 4), None),
    ],
}
# ones and extremes: single heads, a window of one key (a token sees itself alone), a whole head of 8 turned, six taps, a
# delta-rule key of 256 entries, one expert beside one that returns the input with both chosen, a feed-forward of 8
SM_F = {
    "architecture": "Sumitar", "vocab": 64, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        _with(_parallel(_left(1, 1, 8, 8, 1, 8, 10.0, 1.0), 1, 4, 4), _dense(8)),
        _with(_delta(1, 1, 256, 4, 6), _moe(1, 1, 2, 8)),
        _with(_parallel(_left(1, 1, 8, 8, 2, 8, 10.0, 0.7), 1, 8, 8), _moe(1, 0, 1, 8, shared=8)),
    ],
}
CONFIGS = {"A": (SM_A, 51), "B": (SM_B, 52), "C": (SM_C, 53), "D": (SM_D, 54), "E": (SM_E, 55), "F": (SM_F, 56)}
INIT_SCALE = 5.0


def all_chosen(cfg):
    """The configuration with every router choosing all of its outputs: rounding cannot turn a choice then."""
    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        f = layer.get("mlp")
        if f is not None and f["kind"] == "moe":
            f["router"]["top"] = f["router"]["experts"] + f["router"].get("identity", 0)
    return out


def make_model_dir(tmp_root, name, dtype="bfloat16", choose_all=False):
    """Write the folder with the framework's random-weights writer."""
    from zedinfer_b200.weights import write_random_model
    cfg, seed = CONFIGS[name]
    if choose_all:
        cfg = all_chosen(cfg)
    out = os.path.join(str(tmp_root), f"sumitar_{name}_{dtype}" + ("_all" if choose_all else ""))
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        write_random_model(cfg, seed, out, dtype=dtype, init_scale=INIT_SCALE, name_prefix="")
    return out
