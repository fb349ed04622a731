"""Kevatar on the host: config.json to the model's description, which call reads whose cache, tensor names, cache and state
needs, sizes taken from the tensors' shapes, errors; the plain implementation's own mechanisms against each other."""
import copy
import json
import math
import os

import pytest
import torch

import kevatar_tiny as KT
from plain import kevatar_plain as KP
from zedinfer_b200.cache import CacheManager, StateNeed
from zedinfer_b200.cache.manager import PagedKVNeed
from zedinfer_b200.config.registry import ConfigError, load_model_config, resolve_architecture
from zedinfer_b200.engine.model import Model

F64 = torch.float64


def spec_of(raw):
    arch = resolve_architecture(raw)
    spec = arch.build_spec(arch.parse(raw))
    spec.validate()
    return spec


def test_the_architecture_is_found_by_its_name():
    assert resolve_architecture({"architecture": "Kevatar"}).name == "Kevatar"
    assert resolve_architecture({"model_type": "kevatar"}).name == "Kevatar"
    assert "linrec" in resolve_architecture({"architecture": "Kevatar"}).kernel_libraries


def test_layers_parts_and_whose_cache_a_call_reads():
    spec = spec_of(KT.KV_A)
    assert [l.block for l in spec.layers] == ["branch_norm"] * 5
    kinds = [(l.mixer.kind, l.ffn.kind if l.ffn else None) for l in spec.layers]
    assert kinds == [("lightning", "gated_mlp"), ("attention", "gated_mlp"), ("channel_delta", None), ("attention", "gated_mlp"),
                     ("attention", "gated_mlp")]
    assert [(c.layer, c.cache_of) for c in spec.schedule] == [(0, None), (1, None), (2, None), (3, 1), (4, 1)]
    own, far, near = (spec.layers[i].mixer.params for i in (1, 3, 4))
    assert not own["shared_kv"] and far["shared_kv"] and near["shared_kv"]
    # the owner keeps what its furthest-looking reader sees
    assert (own["window"], own["cache_window"], far["window"], near["window"]) == (13, 29, 29, 5)
    assert (own["scale"], own["softcap"], near["softcap"], own["v_head_dim"]) == (0.2, 5.0, None, 16)
    pos = own["position"]
    assert pos.kind == "rope_span" and pos.params["interleaved"] and pos.params["dims"] == 16 and pos.params["unit_rms_eps"] == 1e-5
    assert pos.params["scaling"] == {"factor": 8.0, "original": 64.0, "fast": 16.0, "slow": 2.0}
    assert sorted(far["names"]) == ["o", "q"] and sorted(own["names"]) == ["k", "o", "q", "v"]
    delta = spec.layers[2].mixer.params
    assert (delta["heads"], delta["kv_heads"], delta["dim"], delta["vdim"], delta["conv"], delta["decay_rank"], delta["gate_rank"]) == (4, 2, 16, 24, 3, 6, 14)
    assert spec.layers[0].mixer.params["decay"] == (0.5, 0.9, 0.99)
    assert spec.tie_word_embeddings and spec.embedding.params["scale"] == 3.5
    assert spec.embedding.params["token_tables"] == {"side": ("side.embed", 50)}
    assert [l.extra["side"][1].params["col0"] for l in spec.layers] == [0, 10, 20, 30, 40]
    # no table, no scale: neither the third branch nor its norm
    bare = spec_of(KT.KV_B)
    assert not bare.layers[0].extra and "norm_side" not in bare.layers[0].norms and bare.embedding.params["scale"] == 1.0
    # a layer that sees every key keeps every key
    assert spec_of(KT.KV_C).layers[0].mixer.params["cache_window"] is None


def test_caches_and_states():
    model = Model(spec_of(KT.KV_A))
    needs = dict(model.cache_needs())
    assert sorted(needs) == [0, 1, 2]                                            # calls 3 and 4 own nothing
    assert needs[1] == PagedKVNeed(2, 32, 29, planes=2)                         # rows as wide as the larger of 32 and 16
    assert needs[0] == StateNeed((3 * 24 * 16,), torch.float32)
    assert needs[2] == StateNeed((4 * 24 * 16 + 2 * (2 * 2 * 16 + 4 * 24),), torch.float32)
    assert model.capture_safe()
    cache = CacheManager(list(needs.items()), 4, max_requests=3)
    assert len(cache.groups) == 1 and cache.slots.num_slots == 3
    c = dict(Model(spec_of(KT.KV_C)).cache_needs())
    assert c[0] == PagedKVNeed(3, 40, None, planes=2) and c[3] == PagedKVNeed(2, 16, 3, planes=2)
    assert c[1] == StateNeed((2 * 8 * 72,), torch.float32)                       # one tap: no history behind the state
    d = Model(spec_of(KT.KV_D))
    assert all(isinstance(n, StateNeed) for _, n in d.cache_needs())
    assert not CacheManager(list(d.cache_needs()), 16, max_requests=2).groups
    e = CacheManager(list(Model(spec_of(KT.KV_E)).cache_needs()), 16, max_requests=2)
    assert len(e.groups) == 1 and e.slots.num_slots == 0


def test_tensor_names_and_shapes():
    names = Model(spec_of(KT.KV_A)).tensor_specs()
    want = {"embed": (211, 96), "side.embed": (211, 50), "final.norm": (96,), "l0.norm1": (96,), "l0.norm2": (96,),
            "l0.mix.q": (48, 96), "l0.mix.v": (72, 96), "l0.mix.g": (72, 96), "l0.mix.norm": (72,), "l0.mix.o": (96, 72),
            "l0.mlp.gate": (80, 96), "l0.mlp.down": (96, 80), "l0.side.gate": (10, 96), "l0.side.proj": (96, 10), "l0.side.norm": (96,),
            "l1.mix.q": (128, 96), "l1.mix.k": (64, 96), "l1.mix.v": (32, 96), "l1.mix.o": (96, 64),
            "l2.mix.q": (32, 96), "l2.mix.q.conv": (32, 3), "l2.mix.v": (96, 96), "l2.mix.v.conv": (96, 3), "l2.mix.b": (4, 96),
            "l2.mix.A_log": (4,), "l2.mix.norm": (24,), "l2.mix.a1": (6, 96), "l2.mix.a2": (64, 6), "l2.mix.dt_bias": (64,),
            "l2.mix.g1": (14, 96), "l2.mix.g2": (96, 14), "l2.mix.o": (96, 96), "l3.mix.q": (128, 96), "l3.mix.o": (96, 64)}
    for k, shape in want.items():
        assert tuple(names[k].shape) == shape, k
    for absent in ("l3.mix.k", "l3.mix.v", "l4.mix.k", "l2.norm2", "l2.mlp.gate", "l1.mix.q.bias", "l1.mix.norm", "pos"):
        assert absent not in names, absent
    assert "side.embed" not in Model(spec_of(KT.KV_B)).tensor_specs()


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="mamba2"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=34), "dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0.0), "scaling"),
    (lambda c: c["layers"][1]["mixer"].update(softcap=-1.0), "softcap"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].update(mask={"size": 0}), "size"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "kv_from"),            # a lightning layer holds no keys
    (lambda c: c["layers"][4]["mixer"].update(kv_from=3), "kv_from"),            # a reader holds none of its own
    (lambda c: c["layers"][3]["mixer"].update(heads=2), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(rot=dict(c["layers"][3]["mixer"]["rot"], base=7.0)), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][2]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][2]["mixer"].pop("gate_rank"), "gate_rank"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.9]), "decay"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c["layers"][0]["mlp"].pop("ff"), "ff"),
    (lambda c: c["token_side"].update(dim=0), "dim"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_a_config_that_cannot_be_used_names_the_key(edit, word):
    raw = copy.deepcopy(KT.KV_A)
    edit(raw)
    with pytest.raises(ConfigError, match=word):
        spec_of(raw)


def test_a_written_folder_reads_back_with_low_ranks_from_the_shapes(tmp_path):
    """config.json that names no low rank: the reader takes them from ``a1`` and ``g1``; the plain implementation runs the
    folder, is causal, and its layers add up."""
    folder = KT.make_model_dir(tmp_path, "A", strip_ranks=True)
    with open(os.path.join(folder, "config.json")) as f:
        assert "decay_rank" not in json.load(f)["layers"][2]["mixer"]
    _, _, spec = load_model_config(folder)
    assert (spec.layers[2].mixer.params["decay_rank"], spec.layers[2].mixer.params["gate_rank"]) == (6, 14)
    cfg, w = KP.read_model(folder)
    assert set(w) == set(Model(spec).tensor_specs()) - {"head"}
    toks = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5, 8, 9, 7, 9, 3, 2, 3, 8, 4]
    out, layers = KP.forward(cfg, w, toks, return_layers=True)
    assert out.shape == (20, 211) and layers.shape == (5, 20, 96) and bool(torch.isfinite(out).all())
    assert torch.allclose(KP.forward(cfg, w, toks[:9]), out[:9], atol=1e-10)
    # the head is the table itself, without the embedding's factor
    x = layers[-1]
    assert torch.allclose(out, (KP.rms_unit(x, 1e-5) * w["final.norm"]) @ w["embed"].T)


def test_plain_mechanisms_agree_with_each_other():
    g = torch.Generator().manual_seed(0)
    # a turn by p and then by q is a turn by p + q, up to the factor on cosines and sines; what lies past the span stays
    rot = {"base": 50.0, "dims": 8, "scaling": None}
    v = torch.randn(5, 2, 12, generator=g, dtype=F64)
    pos = torch.tensor([0, 1, 7, 100, 1000])
    twice = KP.turn_pairs(KP.turn_pairs(v, pos, rot), pos + 3, rot)
    assert torch.allclose(twice, KP.turn_pairs(v, 2 * pos + 3, rot)) and torch.equal(twice[..., 8:], v[..., 8:])
    assert torch.equal(KP.turn_pairs(v, torch.zeros(5, dtype=torch.long), rot), v)
    # pair (0, 1) turns by the position itself
    one = torch.zeros(1, 1, 12, dtype=F64)
    one[0, 0, 0] = 1.0
    t = KP.turn_pairs(one, torch.tensor([2]), rot)[0, 0]
    assert abs(float(t[0]) - math.cos(2.0)) < 1e-12 and abs(float(t[1]) - math.sin(2.0)) < 1e-12
    # stretched frequencies: fast pairs keep theirs, slow pairs are divided by the factor, the ramp lies between
    sc = {"base": 10000.0, "dims": 32, "scaling": {"factor": 4.0, "original": 256, "fast": 16.0, "slow": 1.0}}
    f, mag = KP.stretched_frequencies(sc, F64)
    f0, _ = KP.stretched_frequencies({"base": 10000.0, "dims": 32, "scaling": None}, F64)
    assert abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    assert torch.equal(f[:2], f0[:2]) and torch.allclose(f[-3:], f0[-3:] / 4.0) and bool(((f <= f0) & (f >= f0 / 4.0 - 1e-18)).all())
    assert 0 < int(((f < f0) & (f > f0 / 4.0 + 1e-15)).sum())
    # the convolution's last column meets the current token, the first the oldest
    u = torch.randn(6, 3, generator=g, dtype=F64)
    assert torch.allclose(KP.causal_conv(u, torch.tensor([[0.0, 0.0, 1.0]] * 3, dtype=F64)), u)
    back = KP.causal_conv(u, torch.tensor([[1.0, 0.0, 0.0]] * 3, dtype=F64))
    assert torch.allclose(back[2:], u[:-2]) and bool((back[:2] == 0).all())
    # lightning with decay 1 and one head is a running sum of outer products
    m = {"heads": 1, "dim": 4, "vdim": 3, "decay": [1.0]}
    w = {"q": torch.randn(4, 5, generator=g, dtype=F64), "k": torch.randn(4, 5, generator=g, dtype=F64),
         "v": torch.randn(3, 5, generator=g, dtype=F64), "g": torch.zeros(3, 5, dtype=F64), "norm": torch.ones(3, dtype=F64),
         "o": torch.eye(3, dtype=F64)}
    h = torch.randn(7, 5, generator=g, dtype=F64)
    q, k, vv = KP.silu(h @ w["q"].T), KP.silu(h @ w["k"].T), KP.silu(h @ w["v"].T)
    o = torch.tril(q @ k.T) @ vv
    assert torch.allclose(KP.lightning_mixer(h, m, w, "", 1e-9), KP.rms_unit(o, 1e-9) * 0.5)
    # the delta rule with beta = 1 and no decay stores v under k: reading with the same key returns it
    s = torch.zeros(4, 3, dtype=F64)
    key = torch.tensor([0.6, 0.0, 0.8, 0.0], dtype=F64)
    for val in (torch.tensor([1.0, 2.0, 3.0], dtype=F64), torch.tensor([-1.0, 0.5, 4.0], dtype=F64)):
        s = s + torch.outer(key, val - s.T @ key)
        assert torch.allclose(s.T @ key, val)
    # a window of W keys: the query and the W - 1 before it
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 0.0, "mask": {"size": 3}}
    w = {"q": torch.zeros(2, 2, dtype=F64), "o": torch.eye(2, dtype=F64)}
    vals = torch.arange(10, dtype=F64).view(5, 1, 2)
    out = KP.attention_mixer(torch.zeros(5, 2, dtype=F64), torch.arange(5), m, w, "", 1e-6, torch.zeros(5, 1, 2, dtype=F64), vals)
    assert torch.allclose(out[4], vals[2:5, 0].mean(0)) and torch.allclose(out[1], vals[0:2, 0].mean(0))
