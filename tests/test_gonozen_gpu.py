"""The Gonozen decoder through the engine against the plain implementation (tests/plain/gonozen_plain.py).

Every test makes a small configuration of its own with random weights (written as a bfloat16 checkpoint, as a model
folder holds them), replays a trace through the engine's step function and compares every logits row with the plain
implementation's, which walks the whole sequence in float64 with dense masks and expanded keys and values.
float32 path: every row within 1e-4 of its size.  bfloat16 path: every row within a twelfth, their mean within 2 %.
Where random weights would hide a fault (a key just outside a window, a sink, a far key) the scores are made sharp, and
the test first shows that the plain model itself moves by far more than the tolerance when that key is lost.
"""
import json
import os

import pytest
import torch

import helpers
from helpers import collect, mixed, pool_tokens, portions, random_ids, tail_decoded, whole
from plain import gonozen_plain as plain

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 1.0 / 12}


# ------------------------------------------------------------------------------- configurations

def moe(experts=6, top=2, groups=(3, 2), ff=24, limit=1.25, shared=(40, 2.0)):
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "router": router, "expert": {"ff": ff, "limit": limit}}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def rotated_layer(heads=3, dim=24, rot_dim=16, vdim=40, kv_rank=48, scale=None, scaling=True, base=10000.0, mlp="default"):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "rot": rot}
    return {"type": "latent_attention", "mixer": m, "mlp": moe() if mlp == "default" else mlp}


def windowed_layer(heads=5, dim=16, vdim=24, kv_rank=40, q_rank=56, window=19, scale=None, mlp="default"):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": scale if scale is not None else dim ** -0.5, "mask": {"size": window}}
    return {"type": "latent_attention_2", "mixer": m, "mlp": moe() if mlp == "default" else mlp}


def config(layers, vocab=97, width=48, eps=1e-5, softcap=8.0):
    c = {"architecture": "Gonozen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if softcap:
        c["logit_softcap"] = softcap
    return c


def full_config():
    """Both mixers, windows of two sizes (one shorter than a page, one that spans several), one layer without a
    feed-forward, routers with and without groups."""
    return config([windowed_layer(), rotated_layer(), rotated_layer(heads=2, dim=8, rot_dim=8, vdim=16, kv_rank=24, mlp=None),
                   windowed_layer(heads=2, dim=24, vdim=8, kv_rank=16, q_rank=8, window=5, mlp=moe(experts=5, top=3, groups=None, shared=None)),
                   rotated_layer(scaling=False, mlp=moe(experts=8, top=2, groups=(2, 1), ff=16, limit=0.75, shared=(8, 0.5)))])


def other_sizes_config():
    """The values one (one head, one expert chosen, one group kept, a window of one), sizes that fill no whole warp or
    vector, a vocabulary and width that are odd multiples, and no soft cap."""
    return config([rotated_layer(heads=1, dim=40, rot_dim=2, vdim=7, kv_rank=33, mlp=moe(experts=3, top=1, groups=(3, 1), ff=9, shared=(5, 3.0))),
                   windowed_layer(heads=7, dim=8, vdim=8, kv_rank=72, q_rank=3, window=1, mlp=moe(experts=35, top=4, groups=(5, 2), ff=8)),
                   windowed_layer(heads=1, dim=72, vdim=33, kv_rank=8, q_rank=72, window=64, mlp=None),
                   rotated_layer(heads=6, dim=8, rot_dim=24, vdim=8, kv_rank=136, base=300.0,
                                 mlp=moe(experts=2, top=2, groups=None, ff=40, limit=10.0, shared=None))],
                  vocab=61, width=40, eps=1e-6, softcap=None)


_MODELS = {}


def model(tmp_path_factory, name, raw, seed=3):
    """(model folder, (config, float64 weights), memo of plain logits), cached: the plain walk is slow."""
    if name not in _MODELS:
        from return_b200.config.gonozen_config import GonozenConfig
        from return_b200.weights import loader
        d = str(tmp_path_factory.mktemp(name))
        loader.write_random_model(d, GonozenConfig(raw), seed, torch.bfloat16)
        _MODELS[name] = (d, plain.read_model(d), {})
    return _MODELS[name]


def plain_rows(entry, ids):
    d, (c, w), memo = entry
    key = tuple(ids)
    if key not in memo:
        memo[key] = plain.forward(c, w, list(ids)).float()
    return memo[key]


def requests_for(entry, lens, seed=10):
    return {f"r{i}": random_ids(entry[1][0]["vocab"], n, seed + i) for i, n in enumerate(lens)}


def run_trace(model_dir, dtype, steps, page_size=16, max_reside=4, graph=False):
    from return_b200.engine.replay import TraceReplayer
    rp = TraceReplayer(model_dir, dtype, pool_tokens(steps), page_size=page_size, max_reside=max_reside, poison=True,
                       use_cuda_graph=graph)
    outs = []
    for st in steps:
        lg = rp.run_step(st)
        outs.append(None if lg is None else lg.float().cpu())
        rp.runner.manager.check()
    assert rp.runner.manager.num_requests == 0 and rp.runner.manager.pages_used() == [0] * len(rp.runner.manager.groups)
    return collect(steps, outs)


def row_errors(got, want):
    """The error of every row, as a part of the row's size (both with their means taken off: a soft-capped row of
    logits is compared as the softmax sees it)."""
    assert got.shape == want.shape and torch.isfinite(got).all()
    got, want = got - got.mean(1, keepdim=True), want - want.mean(1, keepdim=True)
    return (got - want).norm(dim=1) / want.norm(dim=1)


def worst(got, want):
    return float(row_errors(got, want).max())


def assert_close(got, want, dtype, what=""):
    """float32: every row within 1e-4 of its size.  bfloat16: rounding moves single rows far more than the rest: a
    router whose two best candidates are nearly tied chooses the other one than the float64 walk does, and sharp
    scores multiply the rounding of a query.  So the rows are weighed together: their mean within 3 %, at most one row
    in ten (or two) beyond a twelfth, none beyond six tenths.  A lost key, a wrong window or a stale page moves every
    row behind it, and the tests that aim at single rows compare those rows with what the fault would give."""
    e = row_errors(got, want)
    if dtype == "float32":
        assert float(e.max()) < TOL[dtype], (what, dtype, float(e.max()), int(e.argmax()))
        return
    over = int((e > TOL[dtype]).sum())
    assert over <= max(2, e.numel() // 10) and float(e.max()) < 0.6 and float(e.mean()) < 0.03, \
        (what, dtype, over, float(e.max()), float(e.mean()), int(e.argmax()))


def compare(entry, dtype, steps, requests, **kw):
    got = run_trace(entry[0], dtype, steps, **kw)
    for rid, ids in requests.items():
        assert_close(got[rid], plain_rows(entry, ids), dtype, rid)


# ------------------------------------------------------------------------------- kernels of single mechanisms

@pytest.mark.parametrize("E,top,groups", [(12, 3, (4, 3)), (6, 2, (3, 2)), (40, 5, None), (7, 1, None), (64, 8, (8, 4)),
                                           (35, 4, (5, 2)), (3, 3, (3, 3))])
def test_router_choice(E, top, groups):
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(E * 100 + top)
    z = torch.randn((50, E), generator=g) * 2.0
    router = {"experts": E, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    idx, wt = plain.route(z.double(), router)
    expert_of = torch.empty((50, top), dtype=torch.int32, device="cuda")
    weight = torch.empty((50, top), dtype=torch.float32, device="cuda")
    ops.moe_route(z.cuda(), expert_of, weight, top, groups[0] if groups else 1, groups[1] if groups else 1)
    assert torch.equal(expert_of.cpu().long(), idx)                # in the order of falling score
    assert torch.allclose(weight.cpu().double(), wt, rtol=1e-5, atol=1e-7)
    assert torch.allclose(weight.sum(1).cpu(), torch.ones(50), atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_capped_gated_unit(dtype):
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(5)
    x = (torch.randn((9, 2 * 37), generator=g) * 3.0).to(dtype)
    out = torch.empty((9, 37), dtype=dtype, device="cuda")
    ops.clamped_glu(x.cuda(), out, 1.25, 1.702)
    gate, up = x.double()[:, :37].clamp(max=1.25), x.double()[:, 37:].clamp(-1.25, 1.25)
    want = gate * torch.sigmoid(1.702 * gate) * (up + 1.0)
    assert torch.allclose(out.cpu().double(), want, rtol=1e-5 if dtype == torch.float32 else 1e-2, atol=1e-6 if dtype == torch.float32 else 1e-2)
    assert float(want.max()) > 1.25 * 0.85 * 2.2                   # the cap and the clamp were both reached


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_output_norm_add_input_norm(dtype):
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(6)
    H = 72
    stream, delta = torch.randn((5, H), generator=g), (torch.randn((5, H), generator=g) * 4.0).to(dtype)
    w1, w2 = 1.0 + 0.1 * torch.randn(H, generator=g), 1.0 + 0.1 * torch.randn(H, generator=g)
    s = stream.cuda()
    out = torch.empty((5, H), dtype=dtype, device="cuda")
    ops.postnorm_add_norm(s, delta.cuda(), (w1.cuda(), 1e-5, 0.0), (w2.cuda(), 1e-6, 0.0), out)
    want_s = stream.double() + plain.rms_norm(delta.double(), w1.double(), 1e-5)
    want_o = plain.rms_norm(want_s, w2.double(), 1e-6)
    assert torch.allclose(s.cpu().double(), want_s, rtol=1e-5, atol=1e-5)
    assert torch.allclose(out.cpu().double(), want_o, rtol=1e-5 if dtype == torch.float32 else 1e-2, atol=1e-5 if dtype == torch.float32 else 1e-2)
    s2 = stream.cuda()
    ops.postnorm_add_norm(s2, delta.cuda(), (w1.cuda(), 1e-5, 0.0))          # the add alone
    assert torch.equal(s2, s)


@pytest.mark.parametrize("N,K,counts", [(200, 72, (130, 0, 1, 64, 105)), (128, 32, (64,)), (24, 8, (3, 70, 0, 0, 129, 1))])
def test_experts_products_as_sorted_tiles(N, K, counts):
    """The experts' products over the pairs sorted by expert, on the tensor cores, against float64: experts without a
    pair, runs that end inside a tile, output widths and depths that fill no whole tile; rows gathered through the order."""
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(N)
    E, top = len(counts), 2
    expert_of = torch.cat([torch.full((c,), e, dtype=torch.int32) for e, c in enumerate(counts)])
    expert_of = expert_of[torch.randperm(expert_of.numel(), generator=g)]
    if expert_of.numel() % top:
        expert_of = torch.cat([expert_of, expert_of[:1]])
    pairs = expert_of.numel()
    x = torch.randn((pairs // top, K), generator=g).bfloat16()
    w = (torch.randn((E, N, K), generator=g) * K ** -0.5).bfloat16()
    offsets = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    pair_at, place_of = torch.empty(pairs, dtype=torch.int32, device="cuda"), torch.empty(pairs, dtype=torch.int32, device="cuda")
    ops.moe_sort(expert_of.cuda(), E, offsets, pair_at, place_of)
    assert offsets.cpu().tolist() == [0] + torch.bincount(expert_of.long(), minlength=E).cumsum(0).tolist()
    assert torch.equal(pair_at[place_of.long()].cpu(), torch.arange(pairs, dtype=torch.int32))
    assert torch.equal(expert_of[pair_at.cpu().long()], expert_of.sort().values)
    out = torch.full((pairs, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.moe_grouped_gemm(x.cuda(), pair_at, top, w.cuda(), offsets, out)
    rows = pair_at.cpu().long()
    want = torch.einsum("pk,pnk->pn", x.double()[rows // top], w.double()[expert_of.long()[rows]])
    assert torch.allclose(out.cpu().double(), want, rtol=2e-2, atol=2e-2)
    # the second product reads rows where they lie; and the weighted sum finds a pair's row through the order
    out2 = torch.full((pairs, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    xs = torch.randn((pairs, K), generator=g).bfloat16()
    ops.moe_grouped_gemm(xs.cuda(), None, 1, w.cuda(), offsets, out2)
    want2 = torch.einsum("pk,pnk->pn", xs.double(), w.double()[expert_of.long()[rows]])
    assert torch.allclose(out2.cpu().double(), want2, rtol=2e-2, atol=2e-2)
    weight = torch.rand((pairs // top, top), generator=g)
    y = torch.empty((pairs // top, N), dtype=torch.bfloat16, device="cuda")
    ops.moe_combine(out2, weight.cuda(), None, y, row_of=place_of)
    want_y = (weight.double()[:, :, None] * out2.cpu().double()[place_of.cpu().long()].view(pairs // top, top, N)).sum(1)
    assert torch.allclose(y.cpu().double(), want_y, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("N,K,counts", [(200, 72, (130, 0, 1, 64, 300)), (512, 128, (128, 256)), (24, 8, (3, 70, 0, 0, 129, 1)),
                                        (300, 320, (1,) * 40 + (0,) * 3 + (500,))])
def test_experts_products_on_tcgen05(N, K, counts):
    """The tcgen05 form of the experts' products (rows in the order of the places, operands by TMA) against float64:
    runs that end inside a tile of 128, experts without a pair, many experts of one pair, output widths and depths
    that fill no whole tile or k block, a tile whose box of weight rows reaches past the last expert."""
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(N + K)
    E = len(counts)
    expert_sorted = torch.cat([torch.full((c,), e, dtype=torch.int64) for e, c in enumerate(counts)])
    places = expert_sorted.numel()
    offsets = torch.tensor([0] + torch.bincount(expert_sorted, minlength=E).cumsum(0).tolist(), dtype=torch.int32)
    x = torch.randn((places, K), generator=g).bfloat16()
    w = (torch.randn((E, N, K), generator=g) * K ** -0.5).bfloat16()
    out = torch.full((places, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.moe_tc5_gemm(x.cuda(), w.cuda(), offsets.cuda(), out)
    ops.check_status("cuda:0")
    want = torch.einsum("pk,pnk->pn", x.double(), w.double()[expert_sorted])
    assert torch.allclose(out.cpu().double(), want, rtol=2e-2, atol=2e-2)
    # the gather that feeds it
    pair_at = torch.randperm(places * 1, generator=g).int()
    src = torch.randn((places // 2 + 1, K), generator=g).bfloat16()
    rows = torch.empty((places, K), dtype=torch.bfloat16, device="cuda")
    ops.moe_gather_rows(src.cuda(), pair_at.cuda(), 2, rows)
    assert torch.equal(rows.cpu(), src[pair_at.long() // 2])


def test_soft_cap():
    from return_b200.ext import ops
    x = torch.linspace(-60, 60, 1001)
    y = x.cuda()
    ops.softcap(y, 12.0)
    assert torch.allclose(y.cpu().double(), 12.0 * torch.tanh(x.double() / 12.0), atol=1e-5)


# ------------------------------------------------------------------------------- each mechanism alone in a model

ALONE = {
    "rotated": lambda: config([rotated_layer(mlp=None)]),
    "rotated_plain_frequencies": lambda: config([rotated_layer(scaling=False, mlp=None)], softcap=None),
    "rotated_one_head": lambda: config([rotated_layer(heads=1, dim=16, rot_dim=32, vdim=16, kv_rank=16, mlp=None)]),
    "windowed": lambda: config([windowed_layer(mlp=None)]),
    "windowed_short": lambda: config([windowed_layer(window=3, mlp=None)]),
    "windowed_wider_than_the_prompt": lambda: config([windowed_layer(window=500, mlp=None)]),
    "experts_grouped": lambda: config([windowed_layer(window=500)]),
    "experts_no_groups_no_shared": lambda: config([windowed_layer(window=500, mlp=moe(experts=5, top=2, groups=None, shared=None))]),
    "experts_top_one": lambda: config([windowed_layer(window=500, mlp=moe(experts=4, top=1, groups=(2, 1), limit=0.5))]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(tmp_path_factory, name, dtype):
    entry = model(tmp_path_factory, name, ALONE[name]())
    reqs = requests_for(entry, (70, 1, 33), seed=1)
    compare(entry, dtype, whole(reqs), reqs)


# ------------------------------------------------------------------------------- the whole model under every schedule

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_against_decoding_token_by_token(tmp_path_factory, dtype):
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (90, 47, 16))
    compare(entry, dtype, tail_decoded(reqs, tail=40), reqs)
    first = {"t": reqs["r1"][:24]}                                     # from the very first token on, one by one
    compare(entry, dtype, tail_decoded(first, tail=24), first)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(2, 3, 17, 2, 5, 33, 7), (16, 16, 1, 15, 2, 30, 32, 1), (64, 2)])
def test_portions_of_prompts(tmp_path_factory, dtype, sizes):
    """Portions down to two tokens, cut on page borders and off them, shorter and longer than the windows."""
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (101, 64, 31))
    compare(entry, dtype, portions(reqs, list(sizes)), reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_with_slots_and_pages_used_again(tmp_path_factory, dtype):
    """Seven requests through four slots and a pool that holds four of them: portions of some beside single tokens of
    others, each compared with the request alone (the plain walk).  Pages of 8: the windows give pages back."""
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (60, 33, 80, 17, 49, 2, 71), seed=40)
    for seed in (0, 1):
        compare(entry, dtype, mixed(reqs, max_live=4, portion=13, decode_tail=6, seed=seed), reqs, page_size=8)


def test_one_slot_and_few_pages_taken_again_and_again(tmp_path_factory):
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (40, 9, 40, 23), seed=70)
    compare(entry, "float32", tail_decoded(reqs, tail=5), reqs, max_reside=1, page_size=4)


def test_batching_and_cutting_do_not_change_float32_logits_at_all(tmp_path_factory):
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (60, 33, 45), seed=90)
    a = run_trace(entry[0], "float32", whole(reqs))
    b = run_trace(entry[0], "float32", mixed(reqs, max_live=3, portion=9, decode_tail=8, seed=2))
    for rid in reqs:
        assert torch.equal(a[rid], b[rid]), rid


# ------------------------------------------------------------------------------- faults that random weights would hide

def sharp_config(window=37):
    """Scores eight times larger than usual, so that single keys stand out: a key lost far back, a window that is one
    token off or a sink left out moves the logits by far more than the tolerance."""
    return config([windowed_layer(heads=2, dim=16, vdim=16, kv_rank=24, q_rank=16, window=window, scale=8 * 16 ** -0.5, mlp=None),
                   rotated_layer(heads=2, dim=16, rot_dim=16, vdim=16, kv_rank=24, scale=8 * 32 ** -0.5, mlp=None)], width=32)


def _changed(entry, change):
    """Plain logits of a model whose configuration or weights were changed by ``change(config, weights)``."""
    import copy
    c, w = copy.deepcopy(entry[1][0]), dict(entry[1][1])
    change(c, w)
    return lambda ids: plain.forward(c, w, list(ids)).float()


def _standing_out_pair(c, w):
    """(a, b, fillers): of all pairs of tokens, the one whose score in head 0 of the first layer (which has no positions:
    a token's query and key there depend on the token alone) is the largest, b asking and a answering, and tokens that
    b scores low."""
    m, eps = c["layers"][0]["mixer"], c["norm"]["eps"]
    H, D = m["heads"], m["dim"]
    h = plain.rms_norm(w["embed"], w["l0.norm1"], eps)
    q = (plain.rms_norm(h @ w["l0.mix.dq"].T, w["l0.mix.dq.norm"], eps) @ w["l0.mix.uq"].T).reshape(-1, H, D)
    k = (plain.rms_norm(h @ w["l0.mix.dkv"].T, w["l0.mix.dkv.norm"], eps) @ w["l0.mix.uk"].T).reshape(-1, H, D)
    s0 = torch.einsum("bd,ad->ba", q[:, 0], k[:, 0]) * m["scale"]
    b, a = divmod(int(s0.argmax()), s0.shape[1])
    return a, b, [int(x) for x in s0[b].argsort()[:30] if int(x) not in (a, b)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_just_inside_and_outside_the_window(tmp_path_factory, dtype):
    """A key that one query scores far above all others is put at the window's last place for two queries and one
    place behind it for two more; no other such key is near.  The plain model with a window one shorter (one longer)
    gives other logits there, so an engine whose window is one token off cannot pass."""
    entry = model(tmp_path_factory, "sharp", sharp_config(window=37))
    c, w = entry[1]
    a, b, fill = _standing_out_pair(c, w)
    g = torch.Generator().manual_seed(1)
    ids = [fill[int(i)] for i in torch.randint(0, len(fill), (170,), generator=g)]
    inside, outside = [40, 120], [80, 160]
    for p in inside:
        ids[p], ids[p - 36] = b, a
    for p in outside:
        ids[p], ids[p - 37] = b, a
    want = plain_rows(entry, ids)

    def set_window(n):
        return lambda c, w: c["layers"][0]["mixer"]["mask"].update(size=n)
    shorter = row_errors(_changed(entry, set_window(36))(ids), want)
    longer = row_errors(_changed(entry, set_window(38))(ids), want)
    assert float(shorter[inside].min()) > 2 * TOL[dtype] and float(longer[outside].min()) > 2 * TOL[dtype]
    reqs = {"edge": ids}
    for steps, page in ((whole(reqs), 16), (tail_decoded(reqs, tail=60), 8),          # the window passes over decoded tokens
                        (portions(reqs, [36, 2, 37, 1, 38, 3, 33]), 4),
                        (portions(reqs, [119, 2, 38, 1, 2, 8]), 16)):                  # the asking token first in its portion
        got = run_trace(entry[0], dtype, steps, page_size=page)["edge"]
        assert_close(got, want, dtype, "edge")
        e = row_errors(got, want)                        # at the aimed rows: far nearer the right window than either wrong one
        assert (e[inside] < 0.25 * shorter[inside]).all() and (e[outside] < 0.25 * longer[outside]).all(), (e[inside], e[outside])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_counts(tmp_path_factory, dtype):
    """With a window of three keys the sink holds a good part of the denominator: the plain model without it is
    another model."""
    entry = model(tmp_path_factory, "windowed_short", ALONE["windowed_short"]())
    reqs = requests_for(entry, (70,), seed=1)
    ids = reqs["r0"]
    moved = row_errors(_changed(entry, lambda c, w: w.pop("l0.mix.sink"))(ids), plain_rows(entry, ids))
    assert float(moved.median()) > TOL[dtype]
    compare(entry, dtype, tail_decoded(reqs, tail=30), reqs, page_size=4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_far_back_and_at_page_borders(tmp_path_factory, dtype):
    entry = model(tmp_path_factory, "sharp", sharp_config())
    ids = requests_for(entry, (330,), seed=6)["r0"]
    want = plain_rows(entry, ids)
    c, w = entry[1]
    short = plain.forward(c, w, ids[200:]).float()                     # without the first 200 keys the last rows are others
    assert worst(short[-20:], want[-20:]) > 4 * TOL[dtype]
    lost = row_errors(short[-20:], want[-20:])
    reqs = {"far": ids}
    for steps, page in ((tail_decoded(reqs, tail=36), 16),                           # decoding across two page borders
                        (portions(reqs, [250, 6, 10, 2, 62]), 8)):                   # portions behind a long cached prefix
        got = run_trace(entry[0], dtype, steps, page_size=page)["far"]
        assert_close(got, want, dtype, "far")
        assert float(row_errors(got[-20:], want[-20:]).mean()) < 0.25 * float(lost.mean())


@pytest.mark.parametrize("dtype,graph", [("float32", False), ("bfloat16", True)])
def test_long_decoding(tmp_path_factory, dtype, graph):
    """Up to 160 tokens decoded one by one behind a prompt of three; in bfloat16 through the captured graphs of generation."""
    entry = model(tmp_path_factory, "full", full_config())
    reqs = dict(zip("xy", requests_for(entry, (163, 150), seed=8).values()))
    steps = []
    for k in range(161):
        entries = [{"id": rid, "tokens": ids[:3] if k == 0 else [ids[2 + k]], "want": [2] if k == 0 else [0]}
                   for rid, ids in reqs.items() if 2 + k < len(ids)]
        ended = [rid for rid, ids in reqs.items() if 2 + k == len(ids) - 1]
        steps.append({"step": k, "entries": entries, "end": ended})
    got = run_trace(entry[0], dtype, steps, graph=graph)
    for rid, ids in reqs.items():
        assert_close(got[rid], plain_rows(entry, ids)[2:], dtype, rid)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(tmp_path_factory, dtype):
    entry = model(tmp_path_factory, "other", other_sizes_config(), seed=11)
    reqs = requests_for(entry, (75, 20, 1), seed=20)
    compare(entry, dtype, whole(reqs), reqs)
    compare(entry, dtype, mixed(reqs, max_live=2, portion=11, decode_tail=9, seed=3), reqs, page_size=4, max_reside=2)


def test_a_prompt_of_many_rows(tmp_path_factory):
    """A portion long enough for the tensor-core kernels of prompts (the experts' grouped products, the attention's
    row blocks), beside a short request and followed by decoded tokens."""
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (700, 30), seed=33)
    steps = [{"step": 0, "entries": [{"id": "r1", "tokens": reqs["r1"][:20], "want": list(range(20))}], "end": []},
             {"step": 1, "entries": [{"id": "r0", "tokens": reqs["r0"][:690], "want": list(range(690))},
                                      {"id": "r1", "tokens": reqs["r1"][20:21], "want": [0]}], "end": []}]
    for k in range(9):
        steps.append({"step": 2 + k, "entries": [{"id": "r0", "tokens": [reqs["r0"][690 + k]], "want": [0]},
                                                  {"id": "r1", "tokens": [reqs["r1"][21 + k]], "want": [0]}],
                      "end": ["r0", "r1"] if k == 8 else []})
    for dtype in ("bfloat16", "float32"):
        got = run_trace(entry[0], dtype, steps)
        assert_close(got["r0"][:699], plain_rows(entry, reqs["r0"])[:699], dtype, "long")
        assert_close(got["r1"], plain_rows(entry, reqs["r1"]), dtype, "short")


def kernel_widths_config():
    """Cached vectors of the widths that pick the other attention kernels in bfloat16: 128 and 64 numbers (the tcgen05
    kernel: with a sink and a window wider than the prompt, with a rotated part, with a sink and a short window) and 288
    (wider than a tensor-core head: the CUDA-core kernel)."""
    return config([windowed_layer(heads=4, dim=32, vdim=32, kv_rank=128, q_rank=32, window=2000, mlp=None),
                   rotated_layer(heads=2, dim=32, rot_dim=32, vdim=32, kv_rank=96, mlp=None),
                   windowed_layer(heads=3, dim=16, vdim=16, kv_rank=64, q_rank=24, window=40, mlp=None),
                   rotated_layer(heads=2, dim=16, rot_dim=8, vdim=24, kv_rank=280, mlp=None)], width=64)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_widths_that_pick_the_other_attention_kernels(tmp_path_factory, dtype):
    """Whole prompts, decoded tokens, and a short portion behind a long cached prefix, whose keys the tcgen05 kernel
    shares out over several CTAs and merges (the sink counts once, in the merge)."""
    entry = model(tmp_path_factory, "widths", kernel_widths_config(), seed=5)
    reqs = requests_for(entry, (1200, 300), seed=44)
    ids = reqs["r0"]
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": ids[:1100], "want": [0, 500, 1099]}], "end": []},
             {"step": 1, "entries": [{"id": "r0", "tokens": ids[1100:1190], "want": list(range(90))},
                                      {"id": "r1", "tokens": reqs["r1"][:290], "want": list(range(0, 290, 7))}], "end": []}]
    for k in range(10):
        steps.append({"step": 2 + k, "entries": [{"id": "r0", "tokens": [ids[1190 + k]], "want": [0]},
                                                  {"id": "r1", "tokens": [reqs["r1"][290 + k]], "want": [0]}],
                      "end": ["r0", "r1"] if k == 9 else []})
    got = run_trace(entry[0], dtype, steps)
    want0, want1 = plain_rows(entry, ids), plain_rows(entry, reqs["r1"])
    assert_close(got["r0"], want0[[0, 500, 1099] + list(range(1100, 1200))], dtype, "long")
    assert_close(got["r1"], want1[list(range(0, 290, 7)) + list(range(290, 300))], dtype, "short")
    if dtype == "bfloat16":                            # and through the captured graphs of generation
        graphed = run_trace(entry[0], dtype, steps, graph=True)
        assert_close(graphed["r0"], want0[[0, 500, 1099] + list(range(1100, 1200))], dtype, "long, graphs")


def written_out_config():
    """Heads whose keys and values, written out, are narrower than a cached vector (64 against 96, 128 against 192): in
    bfloat16 portions of prompts then run with keys and values expanded per head while single tokens run over the cached
    vectors themselves, side by side in one step."""
    return config([windowed_layer(heads=3, dim=64, vdim=48, kv_rank=96, q_rank=40, window=50, mlp=None),
                   rotated_layer(heads=2, dim=96, rot_dim=32, vdim=128, kv_rank=160, mlp=None),
                   rotated_layer(heads=4, dim=24, rot_dim=8, vdim=64, kv_rank=80, scaling=False)], width=64)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_with_keys_and_values_written_out(tmp_path_factory, dtype, monkeypatch):
    from return_b200.ext import ops
    entry = model(tmp_path_factory, "written_out", written_out_config(), seed=9)
    reqs = requests_for(entry, (120, 47, 70, 9), seed=60)
    calls, scatter = [], ops.latent_expand_scatter
    monkeypatch.setattr(ops, "latent_expand_scatter", lambda *a, **k: (calls.append(1), scatter(*a, **k))[1])
    compare(entry, dtype, whole(reqs), reqs)
    assert len(calls) == (4 * 3 if dtype == "bfloat16" else 0)     # four prompts, three layers; never in float32
    compare(entry, dtype, tail_decoded(reqs, tail=30), reqs, page_size=8)
    compare(entry, dtype, portions(reqs, [2, 49, 3, 51, 17]), reqs, page_size=4)
    compare(entry, dtype, mixed(reqs, max_live=3, portion=21, decode_tail=7, seed=4), reqs, page_size=16)
    long = requests_for(entry, (1250,), seed=61)
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": long["r0"][:1150], "want": [0, 1149]}], "end": []},
             {"step": 1, "entries": [{"id": "r0", "tokens": long["r0"][1150:], "want": list(range(100))}], "end": ["r0"]}]
    got = run_trace(entry[0], dtype, steps)                        # a short portion behind a long prefix: keys shared out and merged
    assert_close(got["r0"], plain_rows(entry, long["r0"])[[0, 1149] + list(range(1150, 1250))], dtype, "long prefix")


# ------------------------------------------------------------------------------- generation through the engine

def _greedy_plain(entry, prompt, n):
    c, w = entry[1]
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain.forward(c, w, ids)[-1].argmax()))
    return ids[len(prompt):]


@pytest.mark.parametrize("graph", [False, True])
def test_greedy_generation_through_the_scheduler(tmp_path_factory, graph):
    from return_b200.engine.config import EngineConfig
    from return_b200.engine.engine import Engine
    entry = model(tmp_path_factory, "full", full_config())
    prompts = list(requests_for(entry, (5, 29, 1, 40, 12), seed=30).values())
    eng = Engine(entry[0], EngineConfig(max_token=512, max_reside=3, page_size=16, prefill_chunk=24, dtype="float32",
                                        use_cuda_graph=graph))
    got = eng.generate(prompts, max_new_tokens=10, temperature=0.0)
    assert [r.output_ids for r in got] == [_greedy_plain(entry, p, 10) for p in prompts]
    assert eng.runner.manager.pages_used() == [0] * len(eng.runner.manager.groups)


def test_bfloat16_generation_picks_tokens_the_plain_model_rates_highest(tmp_path_factory):
    from return_b200.engine.config import EngineConfig
    from return_b200.engine.engine import Engine
    entry = model(tmp_path_factory, "full", full_config())
    c, w = entry[1]
    prompts = list(requests_for(entry, (7, 33, 20), seed=50).values())
    eng = Engine(entry[0], EngineConfig(max_token=512, max_reside=4, page_size=16, prefill_chunk=32, dtype="bfloat16"))
    for p, r in zip(prompts, eng.generate(prompts, max_new_tokens=8, temperature=0.0)):
        lg = plain.forward(c, w, p + r.output_ids)
        for k, tok in enumerate(r.output_ids):
            row = lg[len(p) - 1 + k]
            assert row[tok] >= row.max() - 0.1 * row.std(), (k, tok)


def test_command_line_generates(tmp_path_factory):
    import subprocess
    import sys
    entry = model(tmp_path_factory, "full", full_config())
    prompt = requests_for(entry, (9,), seed=60)["r0"]
    out = subprocess.run([sys.executable, "-m", "return_b200", "generate", "--model", entry[0], "--prompt-ids",
                          ",".join(map(str, prompt)), "--new", "6", "--temperature", "0", "--dtype", "float32",
                          "--max-token", "256", "--max-reside", "2"], capture_output=True, text=True, timeout=600,
                         cwd=helpers.ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    assert json.loads(out.stdout.strip().splitlines()[0])["output_ids"] == _greedy_plain(entry, prompt, 6)


def test_command_line_replays_a_trace(tmp_path_factory):
    import subprocess
    import sys
    entry = model(tmp_path_factory, "full", full_config())
    out = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "bin", "trace_run"), "--model", entry[0], "--dtype",
                          "float32", "--out", os.path.join(entry[0], "out"), "--max-tokens", "64"],
                         input=json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}], "end": ["a"]}) + "\n",
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "done 0" in out.stdout, out.stderr[-2000:]
    got = torch.frombuffer(bytearray(open(os.path.join(entry[0], "out", "0.f32"), "rb").read()), dtype=torch.float32)
    assert worst(got[None], plain_rows(entry, [1, 2, 3])[2:3]) < TOL["float32"]
