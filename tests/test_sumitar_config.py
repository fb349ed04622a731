"""Sumitar on the host: config.json to the model's description, tensor names, cache and state needs, errors; the plain
implementation's own mechanisms against each other."""
import copy

import pytest
import torch

import sumitar_tiny as ST
from plain import sumitar_plain as SP
from zedinfer_b200.cache import CacheManager, StateNeed
from zedinfer_b200.cache.manager import PagedKVNeed
from zedinfer_b200.config.registry import ConfigError, resolve_architecture
from zedinfer_b200.engine.model import Model

F64 = torch.float64


def spec_of(raw):
    arch = resolve_architecture(raw)
    spec = arch.build_spec(arch.parse(raw))
    spec.validate()
    return spec


def test_the_architecture_is_found_by_its_name():
    assert resolve_architecture({"architecture": "Sumitar"}).name == "Sumitar"
    assert resolve_architecture({"model_type": "sumitar"}).name == "Sumitar"
    libs = resolve_architecture({"architecture": "Sumitar"}).kernel_libraries
    assert "linrec" in libs and "moe" in libs and "rowwise" in libs


def test_layers_and_their_parts():
    spec = spec_of(ST.SM_A)
    assert [l.block for l in spec.layers] == ["sandwich_norm"] * 4
    kinds = [(l.mixer.kind, l.extra["mixer2"][1].kind if "mixer2" in l.extra else None, l.ffn.kind if l.ffn else None) for l in spec.layers]
    assert kinds == [("attention", "forget_gate", "poly_norm_mlp"), ("gated_delta", None, "routed_experts"),
                     ("attention", "forget_gate", "routed_experts"), ("gated_delta", None, None)]
    assert [(c.layer, c.cache_of) for c in spec.schedule] == [(0, None), (1, None), (2, None), (3, None)]
    left = spec.layers[0].mixer.params
    assert (left["num_heads"], left["num_kv_heads"], left["head_dim"], left["v_head_dim"], left["window"], left["scale"]) == (4, 2, 32, 16, 13, 0.2)
    assert left["qkv_bias"] and left["head_scale"] == "temp"
    pos = left["position"]
    assert pos.kind == "rope_span" and not pos.params["interleaved"] and pos.params["dims"] == 16 and pos.params["theta"] == 5000.0
    assert sorted(spec.layers[0].norms) == ["mix2_out", "mix_out", "norm1", "norm1b", "norm2", "norm2b"]
    assert sorted(spec.layers[3].norms) == ["norm1", "norm1b"]
    assert all(n.kind == "tanh_norm" for role, n in spec.layers[0].norms.items() if role.startswith("norm")) and spec.final_norm.kind == "tanh_norm"
    routed = spec.layers[1].ffn.params
    assert (routed["experts"], routed["identity"], routed["top"], routed["score"], routed["choice_bias_name"]) == (5, 1, 2, "softmax_all", "correction")
    assert routed["shared"].params["intermediate_size"] == 40 and routed["shared_gate_name"] == "sg"
    bare = spec.layers[2].ffn.params
    assert bare["shared"] is None and bare["shared_gate_name"] is None and bare["identity"] == 0
    assert spec.tie_word_embeddings
    # without a mask the layer sees, and its cache keeps, every key
    cfg = copy.deepcopy(ST.SM_A)
    cfg["layers"][0]["mixer"]["left"]["mask"] = None
    free = spec_of(cfg).layers[0].mixer.params
    assert free["window"] is None and dict(Model(spec_of(cfg)).cache_needs())[0] == PagedKVNeed(2, 32, None, planes=2)


def test_tensor_names():
    names = Model(spec_of(ST.SM_A)).tensor_specs()
    for n in ("embed", "final.norm", "final.norm.alpha", "final.norm.b", "l0.norm1b.alpha", "l0.mix.left.q.b", "l0.mix.left.temp", "l0.mix.left.out",
              "l0.mix.right.out", "l0.mix.right.f.b", "l0.mix.right.lower", "l0.mix.right.norm", "l0.mlp.act", "l1.mix.q.conv", "l1.mix.A_log",
              "l1.mix.dt_bias", "l1.mix.a", "l1.mix.b", "l1.mix.g", "l1.mlp.router", "l1.mlp.correction", "l1.mlp.e4.gate", "l1.mlp.shared.sg",
              "l1.mlp.shared.down", "l2.mlp.e3.up"):
        assert n in names, n
    assert names["l1.mlp.router"].shape == (6, 96) and names["l1.mlp.correction"].shape == (6,) and "l1.mlp.e5.gate" not in names
    assert names["l0.norm1.alpha"].shape == () and names["l1.mix.dt_bias"].shape == (4,) and names["l1.mlp.shared.sg"].shape == (1, 96)
    assert "l3.norm2" not in names and "l2.mlp.shared.gate" not in names and "l3.mlp.up" not in names


def test_caches_and_states():
    model = Model(spec_of(ST.SM_A))
    needs = dict(model.cache_needs())
    assert sorted(needs, key=str) == [(0, "mixer2"), (2, "mixer2"), 0, 1, 2, 3]
    assert needs[0] == PagedKVNeed(2, 32, 13, planes=2)                          # rows as wide as the larger of 32 and 16
    assert needs[2] == PagedKVNeed(2, 40, 29, planes=2)
    assert needs[(0, "mixer2")] == StateNeed((3 * 24 * 16,), torch.float32)
    assert needs[1] == StateNeed((4 * 24 * 16 + 2 * (2 * 2 * 16 + 4 * 24),), torch.float32)
    assert model.capture_safe()
    cache = CacheManager(list(needs.items()), 4, max_requests=3)
    assert len(cache.groups) == 2 and cache.slots.num_slots == 3
    d = Model(spec_of(ST.SM_D))
    assert all(isinstance(n, StateNeed) for _, n in d.cache_needs())
    assert not CacheManager(list(d.cache_needs()), 16, max_requests=2).groups
    c = dict(Model(spec_of(ST.SM_C)).cache_needs())
    assert c[1] == StateNeed((2 * 8 * 72,), torch.float32)                       # one tap: no history behind the state


@pytest.mark.parametrize("edit,word", [
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=64), "rot"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(mask={"size": 0}), "mask"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][0]["mlp"].update(ff=0), "ff"),
])
def test_errors_name_the_key(edit, word):
    cfg = copy.deepcopy(ST.SM_A)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        spec_of(cfg)
    assert word in str(e.value)


def test_the_plain_mechanisms_agree_with_one_another():
    """The plain implementation against itself: a prefix's logits do not depend on what follows; the forget gate with a lower
    bound of one keeps nothing of the past... and of zero forgets as the logistic says; an identity expert chosen alone with a
    share s returns s times the input."""
    g = torch.Generator().manual_seed(0)
    hidden, H, d, dv = 24, 2, 8, 6
    t = {k: torch.randn(*shape, generator=g, dtype=F64) * 0.4 for k, shape in
         {"q": (H * d, hidden), "f": (H * d, hidden), "f.b": (H * d,), "v": (H * dv, hidden), "norm": (dv,), "o": (hidden, H * dv)}.items()}
    x = torch.randn(9, hidden, generator=g, dtype=F64)
    m = {"heads": H, "dim": d, "vdim": dv}
    # a lower bound of one: the gate is one, nothing is ever written, the read-out is zero
    t["lower"] = torch.ones(H * d, dtype=F64)
    assert float(SP.forget_gate_recurrence(x, t, "", m, 1e-5).abs().max()) == 0.0
    # causality
    t["lower"] = torch.rand(H * d, generator=g, dtype=F64)
    full = SP.forget_gate_recurrence(x, t, "", m, 1e-5)
    assert torch.allclose(SP.forget_gate_recurrence(x[:5], t, "", m, 1e-5), full[:5], atol=1e-12)
    # a router with one expert and one that returns the input: top 1 by the correction alone
    w = {"router": torch.zeros(2, hidden, dtype=F64), "correction": torch.tensor([0.0, 1.0], dtype=F64),
         "e0.gate": torch.randn(4, hidden, generator=g, dtype=F64), "e0.up": torch.randn(4, hidden, generator=g, dtype=F64),
         "e0.down": torch.randn(hidden, 4, generator=g, dtype=F64)}
    f = {"router": {"experts": 1, "identity": 1, "top": 1}, "shared": None}
    assert torch.allclose(SP.routed_ff(x, w, "", f), 0.5 * x, atol=1e-12)
    w["correction"] = torch.tensor([1.0, 0.0], dtype=F64)
    assert torch.allclose(SP.routed_ff(x, w, "", f), 0.5 * SP.gated_ff(x, w, "e0."), atol=1e-12)
    # the whole model: a prefix's logits are what they are in the longer sequence
    cfg = ST.SM_C
    from zedinfer_b200.weights.random_init import random_tensors
    names = Model(spec_of(cfg)).tensor_specs()
    wts = {k: v.double() for k, v in random_tensors({k: s for k, s in names.items() if not s.optional}, 3, torch.float32, init_scale=5.0).items()}
    toks = [5, 17, 3, 99, 140, 2, 2, 60]
    whole = SP.forward(cfg, wts, toks)
    assert torch.allclose(SP.forward(cfg, wts, toks[:5]), whole[:5], atol=1e-9)
