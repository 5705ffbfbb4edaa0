"""The Pisatar decoder's host side: configuration, specification, weight loading, rotary tables, cache needs.  No GPU."""
import copy
import json
import math
import os

import pytest
import torch

from plain import pisatar_plain as plain
from return_b200.cache.storage import CacheStorage
from return_b200.config import registry
from return_b200.config.model_config import ConfigError
from return_b200.config.pisatar_config import PisatarConfig
from return_b200.models.decoder import DecoderModel
from return_b200.parts.base import BuildEnv, CompositeNeed, KVCacheNeed, StateNeed
from return_b200.parts.rope import ScaledRotaryEncoding
from return_b200.weights import loader
from test_pisatar_gpu import config, delta_layer, full_config, parallel_layer, retention_layer


def test_configuration_is_chosen_by_its_architecture_key_and_checked():
    raw = full_config()
    arch = registry.resolve(raw)
    assert arch.name == "Pisatar"
    cfg = arch.config_cls.from_dict(raw)
    assert cfg.vocab == 97 and cfg.width == 48 and cfg.weight_layer(1) == 3 and cfg.weight_layer(4) == 0
    assert PisatarConfig.from_dict(cfg.to_dict()).raw == cfg.raw
    for breakage, text in [
        (lambda r: r.pop("vocab"), "vocab"),
        (lambda r: r["layers"][0].update(type="window"), "type"),
        (lambda r: r["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
        (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=26), "rot.dims"),
        (lambda r: r["layers"][2]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
        (lambda r: r["layers"][2]["mlp"].update(kind="experts"), "dense"),
        (lambda r: r["layers"][4]["mixer"].update(vdim=8), "not shaped like"),
        (lambda r: r["layers"][0].update(weights_of=4), "circle"),
    ]:
        bad = copy.deepcopy(raw)
        breakage(bad)
        with pytest.raises(ConfigError, match=text):
            PisatarConfig.from_dict(bad)


def test_layers_that_borrow_weights_share_a_block_and_own_a_state():
    arch = registry.resolve(full_config())
    spec = arch.decoder_spec(PisatarConfig.from_dict(full_config()), 64)
    assert len(spec.layers) == 4 and [e.layer for e in spec.schedule] == [0, 2, 1, 2, 0, 3]
    assert all(e.cache_of is None for e in spec.schedule)
    assert spec.layers[3].feed_forward is None and spec.embedding_norm.offset == 1.0
    left = spec.layers[1].mixer.mixers[0]
    assert (left.head_dim, left.key_dim, left.value_dim) == (48, 32, 48) and left.position.scaling == (4.0, 1.0, 3.0, 64.0)
    model = DecoderModel(spec, BuildEnv(torch.float32, torch.device("cpu")))
    needs = model.cache_needs()
    assert isinstance(needs[0], StateNeed) and needs[0] == needs[4] and isinstance(needs[2], CompositeNeed)
    storage = CacheStorage(needs, page_size=8, num_pages=16, max_reside=3, env=model.env)
    storage.allocate()
    assert len(storage.states) == 6 and all(t.shape[0] == 4 for t in storage.states.values())
    assert [g.name for g in storage.group_specs] == ["full_h2_d48", "full_h1_d16"]

    class Batch:
        block_tables = [torch.zeros(1, 1, dtype=torch.int32)] * 2
    ctx = storage.layer_context(2, Batch, write=True)
    assert ctx.kv is None and ctx.state is None and set(ctx.children) == {"left", "right"}
    assert ctx.children["left"].kv.k.shape == (16, 2, 8, 48) and ctx.children["right"].state.shape[0] == 4
    assert storage.layer_context(0, Batch, write=True).state is storage.states[(0,)]
    assert storage.layer_context(4, Batch, write=True).state is not storage.states[(0,)]


def test_ranks_of_the_delta_rule_come_from_tensor_shapes(tmp_path):
    raw = config([delta_layer(ranks=(5, 9)), delta_layer(ranks=(5, 9), weights_of=0)])
    d = loader.write_random_model(str(tmp_path / "m"), PisatarConfig(raw), 1, torch.bfloat16)
    with open(os.path.join(d, "config.json")) as f:
        stored = json.load(f)
    for layer in stored["layers"]:
        del layer["mixer"]["decay_rank"], layer["mixer"]["gate_rank"]
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(stored, f)
    arch, cfg = registry.read_config(d)
    assert [(l["mixer"]["decay_rank"], l["mixer"]["gate_rank"]) for l in cfg.layers] == [(5, 9), (5, 9)]
    with pytest.raises(ConfigError, match="ranks"):
        arch.decoder_spec(PisatarConfig.from_dict(stored), 8)


def test_weights_are_fused_and_attention_heads_padded_with_zeros(tmp_path):
    raw = full_config()
    d = loader.write_random_model(str(tmp_path / "m"), PisatarConfig(raw), 2, torch.bfloat16)
    arch, cfg = registry.read_config(d)
    model = DecoderModel(arch.decoder_spec(cfg, 32), BuildEnv(torch.float32, torch.device("cpu")))
    shapes = {n: s for n, (s, _) in loader.checkpoint_shapes(arch, cfg).items()}
    files = plain.read_safetensors(os.path.join(d, "model.safetensors"))
    assert {n: tuple(t.shape) for n, t in files.items()} == shapes
    assert not any(n.startswith(("l1.", "l4.")) for n in files)                     # borrowed layers have no tensors
    p = loader.load_parameters(model.params(), arch.weight_sources(cfg), shapes, d, torch.float32, "cpu",
                               arch.ignorable_tensors(cfg))
    qkv = p["layers.1.mixer.left.qkv"].view(4 + 2 + 2, 48, 48)                       # layer 2 of the file: heads of 48 rows
    assert torch.equal(qkv[:4, :32].reshape(-1, 48), files["l2.mix.left.q"].float()) and not qkv[:6, 32:].any()
    assert torch.equal(qkv[4:6, :32].reshape(-1, 48), files["l2.mix.left.k"].float())
    assert torch.equal(qkv[6:].reshape(-1, 48), files["l2.mix.left.v"].float())
    assert torch.equal(p["layers.1.mixer.left.o"], files["l2.mix.left.o"].float())  # value size 48 is the padded size
    small = p["layers.3.mixer.left.qkv"]
    assert small.shape == ((2 + 1 + 1) * 16, 48)
    assert torch.equal(p["layers.2.mixer.in"], torch.cat([files["l3.mix." + n] for n in ("q", "k", "v", "a1", "g1")]).float())
    assert torch.equal(p["layers.2.mixer.conv"], torch.cat([files["l3.mix." + n + ".conv"] for n in "qkv"]).float())
    assert torch.equal(p["layers.1.mixer.right.gate_bias"], torch.cat([files["l2.mix.right.i.b"], files["l2.mix.right.f.b"]]).float())
    gu = p["layers.0.feed_forward.gate_up"].view(-1, 2, 8, 48)
    assert torch.equal(gu[:, 0].reshape(-1, 48), files["l0.mlp.gate"].float()) and torch.equal(gu[:, 1].reshape(-1, 48), files["l0.mlp.up"].float())
    # a file that lacks a tensor or holds a stranger is refused with every fault named
    with pytest.raises(loader.WeightError, match="missing"):
        loader.load_parameters(model.params(), arch.weight_sources(cfg), dict(shapes, **{"l9.mix.q": (1, 1)}), d,
                               torch.float32, "cpu")


def test_key_and_value_heads_of_unequal_size_are_padded_on_both_sides(tmp_path):
    raw = config([parallel_layer(heads=2, kv_heads=1, dim=40, vdim=24, rot=8)])
    d = loader.write_random_model(str(tmp_path / "m"), PisatarConfig(raw), 2, torch.bfloat16)
    arch, cfg = registry.read_config(d)
    model = DecoderModel(arch.decoder_spec(cfg, 32), BuildEnv(torch.float32, torch.device("cpu")))
    shapes = {n: s for n, (s, _) in loader.checkpoint_shapes(arch, cfg).items()}
    files = plain.read_safetensors(os.path.join(d, "model.safetensors"))
    p = loader.load_parameters(model.params(), arch.weight_sources(cfg), shapes, d, torch.float32, "cpu")
    qkv = p["layers.0.mixer.left.qkv"].view(4, 48, 48)
    assert torch.equal(qkv[3, :24], files["l0.mix.left.v"].float()) and not qkv[3, 24:].any() and not qkv[:3, 40:].any()
    o = p["layers.0.mixer.left.o"].view(48, 2, 48)
    assert torch.equal(o[:, :, :24].reshape(48, 48), files["l0.mix.left.o"].float()) and not o[:, :, 24:].any()


@pytest.mark.parametrize("scaling", [None, (8.0, 1.0, 4.0, 2048.0), (4.0, 1.0, 3.0, 64.0), (2.0, 0.5, 8.0, 300.0)])
def test_rotary_frequencies_with_slowed_long_wavelengths(scaling):
    rot = {"base": 10000.0, "dims": 32}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    want = plain.rotary_frequencies(rot, torch.float64)
    got = ScaledRotaryEncoding.frequencies(32, 10000.0, scaling)
    assert torch.allclose(got, want, rtol=1e-12, atol=0)
    if scaling:
        plainf = ScaledRotaryEncoding.frequencies(32, 10000.0, None)
        lam = 2 * math.pi / plainf
        assert torch.equal(got[lam < scaling[3] / scaling[2]], plainf[lam < scaling[3] / scaling[2]])
        assert torch.allclose(got[lam > scaling[3] / scaling[1]], plainf[lam > scaling[3] / scaling[1]] / scaling[0])


def test_plain_retention_equals_its_closed_form():
    """The plain recurrence against the sum it unrolls to: o_t = sum_s decay^(t-s) (q_t . k_s) v_s."""
    torch.manual_seed(0)
    m = retention_layer(heads=2, dim=6, vdim=5, rot=4)["mixer"]
    W, T = 12, 9
    w = {"x.q": torch.randn(12, W), "x.k": torch.randn(12, W), "x.v": torch.randn(10, W), "x.g": torch.randn(10, W),
         "x.o": torch.eye(10)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, W).double()
    pos = torch.arange(T)
    got = plain.retention(h, m, w, "x.", 1e-5, pos)
    q = plain.rotate((h @ w["x.q"].T).view(T, 2, 6), m["rot"], pos)
    k = plain.rotate((h @ w["x.k"].T).view(T, 2, 6), m["rot"], pos) * 6 ** -0.5
    v = (h @ w["x.v"].T).view(T, 2, 5)
    o = torch.zeros(T, 2, 5).double()
    for t in range(T):
        for s in range(t + 1):
            for hh in range(2):
                o[t, hh] += m["decay"][hh] ** (t - s) * (q[t, hh] @ k[s, hh]) * v[s, hh]
    want = plain.rms(o, 1e-5).reshape(T, 10) * torch.nn.functional.silu(h @ w["x.g"].T)
    assert torch.allclose(got, want, rtol=1e-10, atol=1e-12)


def test_plain_convolution_looks_back_and_starts_from_zeros():
    x = torch.arange(1.0, 7.0).double()[:, None]
    taps = torch.tensor([[100.0, 10.0, 1.0]]).double()                 # the last column weighs the current token
    assert plain.causal_conv(x, taps)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0, 456.0]
