"""Host-side tests of the Gonozen decoder's configuration, specification, weight map, rotary tables and cache layout,
and of the plain implementation against itself (whole sequence against a prefix: causality, the window, the sink)."""
import copy
import math

import pytest
import torch

import helpers  # noqa: F401  (paths)
from plain import gonozen_plain as plain
from return_b200.cache.storage import CacheStorage
from return_b200.config import registry
from return_b200.config.gonozen_config import GonozenConfig
from return_b200.config.model_config import ConfigError
from return_b200.models import gonozen
from return_b200.models.decoder import DecoderModel
from return_b200.parts.base import BuildEnv, KVCacheNeed, LatentCacheNeed
from return_b200.parts.rope import RampedRotaryEncoding
from return_b200.parts.spec import RampedRopeSpec
from return_b200.weights import loader


def raw_config():
    moe = {"kind": "moe", "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}},
           "expert": {"ff": 24, "limit": 1.25}, "shared": {"ff": 40, "limit": 2.0}}
    return {"architecture": "Gonozen", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "logit_softcap": 8.0, "layers": [
        {"type": "latent_attention_2", "mixer": {"heads": 5, "dim": 16, "vdim": 24, "kv_rank": 40, "q_rank": 56, "scale": 0.25,
                                                 "mask": {"size": 19}}, "mlp": moe},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 24, "rot_dim": 16, "vdim": 40, "kv_rank": 48, "scale": 0.2,
                                               "rot": {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "original": 32,
                                                                                                   "fast": 8.0, "slow": 1.0}}},
         "mlp": None}]}


def test_registry_finds_the_architecture_by_its_name():
    arch = registry.resolve({"architecture": "Gonozen"})
    assert arch.config_cls is GonozenConfig and "Gonozen" in registry.architectures()


@pytest.mark.parametrize("path,value", [(("layers", 0, "type"), "attention"), (("layers", 1, "mixer", "rot_dim"), 7),
                                        (("layers", 1, "mixer", "rot", "dims"), 8), (("layers", 0, "mlp", "router", "top"), 5),
                                        (("layers", 0, "mlp", "router", "groups", "count"), 4), (("layers", 0, "mlp", "kind"), "dense"),
                                        (("layers", 0, "mixer", "mask", "size"), 0), (("logit_softcap",), -1.0), (("width",), 0)])
def test_configuration_rejects_what_the_design_does_not_have(path, value):
    raw = raw_config()
    d = raw
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError):
        GonozenConfig(raw)
    missing = raw_config()
    del missing["layers"][0]["mixer"]["q_rank"]
    with pytest.raises(ConfigError):
        GonozenConfig(missing)


def test_specification_follows_the_configuration():
    spec = gonozen.decoder_spec(GonozenConfig(raw_config()), 256)
    assert spec.tie_embeddings and spec.logit_softcap == 8.0 and len(spec.layers) == 2
    a, b = spec.layers[0].mixer, spec.layers[1].mixer
    assert (a.q_rank, a.window, a.sink, a.gate, a.rot_dim, a.position) == (56, 19, True, False, 0, None)
    assert (b.q_rank, b.window, b.sink, b.gate, b.rot_dim) == (None, None, False, True, 16)
    assert b.position.factor == 4.0 and b.position.max_positions == 256
    ff = spec.layers[0].feed_forward
    assert (ff.num_experts, ff.top, ff.groups, ff.keep_groups, ff.expert.limit, ff.shared.intermediate_size) == (6, 2, 3, 2, 1.25, 40)
    assert spec.layers[1].feed_forward is None and spec.layers[1].feed_forward_norm is None
    # optional keys left out: no groups, no shared expert, no window, no stretching, no cap
    raw = raw_config()
    del raw["layers"][0]["mlp"]["router"]["groups"], raw["layers"][0]["mlp"]["shared"], raw["layers"][0]["mixer"]["mask"]
    del raw["layers"][1]["mixer"]["rot"]["scaling"], raw["logit_softcap"]
    spec = gonozen.decoder_spec(GonozenConfig(raw), 64)
    assert spec.layers[0].feed_forward.groups == 1 and spec.layers[0].feed_forward.shared is None
    assert spec.layers[0].mixer.window is None and spec.layers[1].mixer.position.factor is None and spec.logit_softcap is None


def test_a_random_checkpoint_fills_every_parameter(tmp_path):
    cfg = GonozenConfig(raw_config())
    d = loader.write_random_model(str(tmp_path / "m"), cfg, 1, torch.bfloat16)
    arch, cfg2 = registry.read_config(d)
    model = DecoderModel(arch.decoder_spec(cfg2, 64), BuildEnv(torch.float32, torch.device("cpu")))
    expected = {n: shape for n, (shape, _) in loader.checkpoint_shapes(arch, cfg2).items()}
    params = loader.load_parameters(model.params(), arch.weight_sources(cfg2), expected, d, torch.float32, "cpu",
                                    arch.ignorable_tensors(cfg2))
    model.bind(params)
    c, w = plain.read_model(d, torch.float32)
    # the fused parameters hold the checkpoint's tensors in the order the parts read them
    mix = params["layers.1.mixer.in"]
    assert torch.equal(mix[:3 * 40], w["l1.mix.q"]) and torch.equal(mix[120:120 + 64], w["l1.mix.dkv"]) and torch.equal(mix[184:], w["l1.mix.g"])
    gu = params["layers.0.feed_forward.experts.gate_up"].view(6, 48, 48)
    assert torch.equal(gu[4, :24], w["l0.mlp.e4.gate"]) and torch.equal(gu[4, 24:], w["l0.mlp.e4.up"])
    assert torch.equal(params["layers.0.feed_forward.experts.down"].view(6, 48, 24)[5], w["l0.mlp.e5.down"])
    assert model.lm_head is model.embed
    # a checkpoint that lacks a tensor, or holds one of another shape, is refused with one error that names it
    bad = dict(expected)
    bad["l0.mix.sink"] = (6,)
    with pytest.raises(loader.WeightError) as e:
        loader.load_parameters(model.params(), arch.weight_sources(cfg2), bad, d, torch.float32, "cpu")
    assert "l0.mix.sink" in str(e.value)


def test_ramped_rotary_tables_follow_the_plain_frequencies():
    rot = {"base": 5000.0, "dims": 24, "scaling": {"factor": 3.0, "original": 256, "fast": 16.0, "slow": 2.0}}
    spec = RampedRopeSpec(rotary_dim=24, theta=5000.0, max_positions=300, factor=3.0, original=256, fast=16.0, slow=2.0)
    cos, sin, width = RampedRotaryEncoding(spec, BuildEnv(torch.float32, torch.device("cpu"))).rotary_tables()
    f, mag = plain.rotary_frequencies(rot)
    assert width == 24 and mag == pytest.approx(0.1 * math.log(3.0) + 1.0)
    ang = torch.outer(torch.arange(300, dtype=torch.float64), f)
    assert torch.allclose(cos.double(), ang.cos() * mag, atol=1e-6) and torch.allclose(sin.double(), ang.sin() * mag, atol=1e-6)
    # the fast pairs keep their frequency, the slow ones are divided by the factor, and between them lies a ramp
    plain_f = 5000.0 ** (-2.0 * torch.arange(12, dtype=torch.float64) / 24)
    ratio = f / plain_f
    assert ratio[0] == 1.0 and ratio[-1] == pytest.approx(1.0 / 3.0) and (ratio[1:] <= ratio[:-1] + 1e-12).all()
    assert ((ratio > 1.0 / 3.0 + 1e-9) & (ratio < 1.0 - 1e-9)).any()          # some pair lies on the ramp
    # without stretching: plain frequencies and no factor
    spec = RampedRopeSpec(rotary_dim=8, theta=100.0, max_positions=10)
    cos, sin, _ = RampedRotaryEncoding(spec, BuildEnv(torch.float32, torch.device("cpu"))).rotary_tables()
    assert cos[0].tolist() == [1.0] * 4 and sin[1, 0] == pytest.approx(math.sin(1.0))


def test_latents_get_page_groups_of_their_own_by_width_and_window():
    env = BuildEnv(torch.float32, torch.device("cpu"))
    needs = [LatentCacheNeed(80, 50), LatentCacheNeed(144, None), LatentCacheNeed(144, None), LatentCacheNeed(80, 50),
             KVCacheNeed(2, 144, None), None]
    st = CacheStorage(needs, page_size=16, num_pages=40, max_reside=4, env=env, longest_append=64)
    assert [g.name for g in st.group_specs] == ["window50_latent80", "full_latent144", "full_h2_d144"]
    assert st.group_specs[0].num_pages == 4 * ((50 + 64 + 15) // 16 + 1) and st.group_specs[1].num_pages == 40
    st.allocate()
    assert tuple(st.pools[0].shape) == (2, st.group_specs[0].num_pages, 16, 80)        # one tensor: a latent is key and value
    assert tuple(st.pools[1].shape) == (2, 40, 16, 144) and tuple(st.pools[2].shape) == (1, 2, 40, 2, 16, 144)
    assert st.bytes_per_token() == (2 * 80 + 2 * 144 + 2 * 2 * 144) * 4
    manager = st.make_manager()
    manager.add("a")
    manager.append("a", 200)
    manager.append("a", 1)           # room for the next token: first the pages that the window has passed go back

    class Batch:
        block_tables = [torch.zeros((1, 13), dtype=torch.int32)] * 3
    ctx = st.layer_context(3, Batch(), True)
    assert ctx.kv.v is None and tuple(ctx.kv.k.shape) == (st.group_specs[0].num_pages, 16, 80)
    assert ctx.kv.k.data_ptr() == st.pools[0][1].data_ptr()
    # the window gave the first pages back while the full group holds them all
    assert manager.block_table("a", 0)[:10] == [-1] * 9 + [9] and -1 not in manager.block_table("a", 1)


def test_plain_model_is_causal_and_its_window_and_sink_do_what_they_say():
    cfg = raw_config()
    cfg["layers"] = cfg["layers"][:1]
    from return_b200.models.gonozen import checkpoint_shapes
    w = {n: loader.random_tensor(2, n, shp, law, torch.float64) for n, (shp, law) in checkpoint_shapes(GonozenConfig(cfg)).items()}
    ids = list(range(40))
    whole = plain.forward(cfg, w, ids)
    assert torch.allclose(plain.forward(cfg, w, ids[:25]), whole[:25], atol=1e-12)          # causal
    # a token farther back than the window does not reach the logits
    other = [96] + ids[1:]
    assert torch.allclose(plain.forward(cfg, w, other)[19:], whole[19:], atol=1e-12)
    assert not torch.allclose(plain.forward(cfg, w, other)[18], whole[18], atol=1e-6)
    # a sink far below the scores changes nothing; a sink far above them takes the whole weight
    a = plain.masked_softmax(torch.zeros(1, 3, 3, dtype=torch.float64), plain.visible_keys(3), torch.tensor([-50.0], dtype=torch.float64))
    assert torch.allclose(a[0, 2], torch.full((3,), 1 / 3, dtype=torch.float64))
    a = plain.masked_softmax(torch.zeros(1, 3, 3, dtype=torch.float64), plain.visible_keys(3), torch.tensor([0.0], dtype=torch.float64))
    assert torch.allclose(a[0, 2], torch.full((3,), 0.25, dtype=torch.float64)) and a[0, 0, 0] == 0.5


def test_plain_router_keeps_to_the_best_groups():
    z = torch.tensor([[0.0, 5.0, 0.1, 0.2, 4.0, 3.9, 0.3, 4.5]], dtype=torch.float64)
    idx, wt = plain.route(z, {"experts": 8, "top": 3, "groups": {"count": 4, "keep": 2}})
    # groups (0,1) (2,3) (4,5) (6,7): the best two are the first and the last; expert 4 is shut out although it scores high
    assert idx.tolist() == [[1, 7, 6]] and wt.sum().item() == pytest.approx(1.0)
    idx, _ = plain.route(z, {"experts": 8, "top": 3})
    assert idx.tolist() == [[1, 7, 4]]
