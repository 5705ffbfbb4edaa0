"""The Pisatar decoder through the engine against the plain implementation (tests/plain/pisatar_plain.py).

Every test makes a small configuration of its own with random weights (written as a bfloat16 checkpoint, as a
model folder holds them), replays a trace through the engine's step function and compares every logits row with the
plain implementation's, which walks the whole sequence in float64.  float32 path: every row within 1e-4 of its size.
bfloat16 path: rounding is amplified at single positions (a read-out that is divided by a small root mean square or
a small normaliser), so the rows are weighed together: their mean error below 3 %, at most one row in fifty beyond a
twelfth of its size, none beyond a third.  A lost key, a lost state or a wrong position moves every row behind it.
"""
import json
import os

import pytest
import torch

import helpers
from helpers import collect, mixed, pool_tokens, portions, random_ids, tail_decoded, whole
from plain import pisatar_plain as plain

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 1.0 / 12}


# ------------------------------------------------------------------------------- configurations

def retention_layer(heads=3, dim=24, vdim=40, rot=16, base=5000.0, ff=64, decay=None, **extra):
    decay = decay or [1.0 - 2.0 ** -(3 + i) for i in range(heads)]
    layer = {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay,
                                             "rot": {"base": base, "dims": rot}},
             "mlp": {"kind": "dense", "ff": ff} if ff else None}
    layer.update(extra)
    return layer


def delta_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, ranks=(8, 12), ff=56, **extra):
    layer = {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                                 "decay_rank": ranks[0], "gate_rank": ranks[1]},
             "mlp": {"kind": "dense", "ff": ff} if ff else None}
    layer.update(extra)
    return layer


def parallel_layer(heads=4, kv_heads=2, dim=32, vdim=48, rot=16, scale=None, scaling=True, mem=(2, 40, 16), cap=12.0,
                   scales=(0.7, 1.3), ff=64, **extra):
    rot_d = {"base": 10000.0, "dims": rot}
    if scaling:
        rot_d["scaling"] = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 64}
    layer = {"type": "parallel",
             "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot_d,
                                "scale": scale if scale is not None else dim ** -0.5},
                       "right": {"heads": mem[0], "dim": mem[1], "vdim": mem[2], "gate_cap": cap},
                       "left_scale": scales[0], "right_scale": scales[1]},
             "mlp": {"kind": "dense", "ff": ff} if ff else None}
    layer.update(extra)
    return layer


def config(layers, vocab=97, width=48, eps=1e-5):
    return {"architecture": "Pisatar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def full_config():
    """All three mixers, one layer that runs twice, one without a feed-forward; the layer that lends its weights
    comes after the one that borrows them."""
    return config([retention_layer(), delta_layer(weights_of=3), parallel_layer(), delta_layer(), retention_layer(weights_of=0),
                   parallel_layer(heads=2, kv_heads=1, dim=16, vdim=16, rot=8, scaling=False, mem=(3, 8, 40), ff=0)])


def other_sizes_config():
    """Sizes that take other kernel variants (key sizes of 8, 72 and 136, value sizes that fill no whole tile) and the
    values one: one head, one tap, one layer kind each."""
    return config([retention_layer(heads=1, dim=8, vdim=72, rot=8, ff=40),
                   delta_layer(heads=1, kv_heads=1, dim=72, vdim=8, conv=1, ranks=(1, 3), ff=0),
                   delta_layer(heads=6, kv_heads=3, dim=8, vdim=33, conv=5, ranks=(16, 4), ff=24),
                   parallel_layer(heads=1, kv_heads=1, dim=64, vdim=64, rot=64, mem=(1, 136, 8), scales=(1.0, 1.0)),
                   retention_layer(heads=2, dim=136, vdim=16, rot=0, ff=16)], vocab=61, width=40, eps=1e-6)


_MODELS = {}


def model(tmp_path_factory, name, raw, seed=3):
    """(model folder, plain logits of a request), cached: the plain walk is slow."""
    if name not in _MODELS:
        from return_b200.config.pisatar_config import PisatarConfig
        from return_b200.weights import loader
        d = str(tmp_path_factory.mktemp(name))
        loader.write_random_model(d, PisatarConfig(raw), seed, torch.bfloat16)
        _MODELS[name] = (d, plain.read_model(d), {})
    return _MODELS[name]


def plain_rows(entry, ids):
    d, (c, w), memo = entry
    key = tuple(ids)
    if key not in memo:
        memo[key] = plain.forward(c, w, list(ids))[0].float()
    return memo[key]


def steady_first_token(entry):
    """A token that every test request starts with.  At position 0 a retention head reads out (q . k) v and divides it
    by its root mean square, so the sign of q . k decides the result; for about a fifth of the tokens of these small
    models some head's q . k is so near zero that rounding to bfloat16 turns the sign, and every row behind it moves.
    That is the design's own sensitivity, not an engine's fault, so the requests start with the token whose logits
    move least when the embedding is jittered by bfloat16's rounding step.  Position 0 is still compared."""
    d, (c, w), memo = entry
    if "first" not in memo:
        g = torch.Generator().manual_seed(0)
        vocab = c["vocab"]
        noisy = dict(w)
        moved = torch.zeros(vocab)
        for trial in range(3):
            noisy["embed"] = w["embed"] * (1.0 + 2.0 ** -8 * torch.randn(w["embed"].shape, generator=g, dtype=w["embed"].dtype))
            for t in range(vocab):
                a, b = plain.forward(c, w, [t])[0], plain.forward(c, noisy, [t])[0]
                moved[t] = max(moved[t], float((a - b).norm() / a.norm()))
        memo["first"] = int(moved.argmin())
    return memo["first"]


def requests_for(entry, lens, seed=10):
    first = steady_first_token(entry)
    return {f"r{i}": [first] + random_ids(entry[1][0]["vocab"], n, seed + i)[1:] for i, n in enumerate(lens)}


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
    """The error of every row, as a part of the row's size."""
    assert got.shape == want.shape and torch.isfinite(got).all()
    return (got - want).norm(dim=1) / want.norm(dim=1)


def worst(got, want):
    return float(row_errors(got, want).max())


def assert_close(got, want, dtype, what=""):
    e = row_errors(got, want)
    if dtype == "float32":
        assert float(e.max()) < TOL[dtype], (what, dtype, float(e.max()), int(e.argmax()))
        return
    over = int((e > TOL[dtype]).sum())
    assert float(e.mean()) < 0.03 and over <= max(1, e.numel() // 50) and float(e.max()) < 4 * TOL[dtype], \
        (what, dtype, float(e.mean()), over, float(e.max()), int(e.argmax()))


def compare(entry, dtype, steps, requests, **kw):
    got = run_trace(entry[0], dtype, steps, **kw)
    for rid, ids in requests.items():
        assert_close(got[rid], plain_rows(entry, ids), dtype, rid)


# ------------------------------------------------------------------------------- each mechanism alone

ALONE = {
    "retention": lambda: config([retention_layer()]),
    "retention_whole_rotation": lambda: config([retention_layer(heads=2, dim=16, vdim=32, rot=16, ff=0)]),
    "channel_delta": lambda: config([delta_layer()]),
    "channel_delta_equal_heads": lambda: config([delta_layer(heads=2, kv_heads=2, conv=4, ff=0)]),
    "attention_and_memory": lambda: config([parallel_layer()]),
    "attention_equal_sizes": lambda: config([parallel_layer(dim=32, vdim=32, rot=32, scaling=False, scales=(1.0, 0.0))]),
    "memory_mostly": lambda: config([parallel_layer(scales=(0.0, 1.0), cap=2.0)]),
    "rotary_widths_of_six_and_ten": lambda: config([parallel_layer(rot=6), retention_layer(rot=10)]),
    "layer_run_twice": lambda: config([delta_layer(), delta_layer(weights_of=0), retention_layer(), retention_layer(weights_of=2)]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mixer_alone(tmp_path_factory, name, dtype):
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
    """Portions down to two tokens, cut on page borders and off them, shorter than the convolution reaches."""
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (101, 64, 31))
    compare(entry, dtype, portions(reqs, list(sizes)), reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_with_slots_and_pages_used_again(tmp_path_factory, dtype):
    """Seven requests through four slots and a pool that holds four of them: portions of some beside single tokens of
    others, each compared with the request alone (the plain walk)."""
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (60, 33, 80, 17, 49, 2, 71), seed=40)
    for seed in (0, 1):
        compare(entry, dtype, mixed(reqs, max_live=4, portion=13, decode_tail=6, seed=seed), reqs, page_size=8)


def test_a_slot_taken_again_starts_from_nothing(tmp_path_factory):
    """One slot: every request inherits the slot (and the pages) of the one before it."""
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (40, 9, 40, 23), seed=70)
    compare(entry, "float32", tail_decoded(reqs, tail=5), reqs, max_reside=1)


def test_batching_and_cutting_do_not_change_float32_logits_at_all(tmp_path_factory):
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (60, 33, 45), seed=90)
    a = run_trace(entry[0], "float32", whole(reqs))
    b = run_trace(entry[0], "float32", mixed(reqs, max_live=3, portion=9, decode_tail=8, seed=2))
    for rid in reqs:
        assert torch.equal(a[rid], b[rid]), rid


# ------------------------------------------------------------------------------- faults that random weights would hide

def sharp_config():
    """Attention whose scores are five times larger than usual, so that single keys stand out, beside a retention that
    hardly forgets: a key that is lost far back, or a state that is cut short, moves the logits by far more than the
    tolerance."""
    return config([parallel_layer(heads=2, kv_heads=1, dim=32, vdim=32, rot=32, scale=5 * 32 ** -0.5, scaling=True,
                                  scales=(1.0, 0.2), mem=(1, 16, 16)),
                   retention_layer(heads=2, dim=16, vdim=16, rot=8, decay=[0.999, 0.9999])], width=32)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_far_back_and_at_page_borders(tmp_path_factory, dtype):
    entry = model(tmp_path_factory, "sharp", sharp_config())
    ids = requests_for(entry, (330,), seed=5)["r0"]
    want = plain_rows(entry, ids)
    # the plain attention of the last tokens does lean on single far keys: without the first 200 it is another
    c, w = entry[1]
    short = plain.forward(c, w, ids[200:])[0].float()
    assert worst(short[-20:], want[-20:]) > 4 * TOL[dtype]
    reqs = {"far": ids}
    compare(entry, dtype, tail_decoded(reqs, tail=36), reqs, page_size=16)           # decoding across two page borders
    compare(entry, dtype, portions(reqs, [250, 6, 10, 2, 62]), reqs, page_size=8)    # portions behind a long cached prefix


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


def test_a_long_prompt_scanned_in_pieces_side_by_side(tmp_path_factory):
    """On the bfloat16 path a retention and a matrix memory cut a portion of 1,024 tokens or more into pieces that are
    scanned at the same time, hand the states from piece to piece and scan again.  The outputs of every piece, the state that the tokens
    decoded afterwards start from, and a short request in the same step must all be right; the decays are slow, so a
    state handed on wrongly would show to the end."""
    raw = config([retention_layer(heads=2, dim=24, vdim=40, rot=16, decay=[0.999, 0.9995]),
                  parallel_layer(heads=2, kv_heads=1, dim=16, vdim=16, rot=8, mem=(2, 16, 24), scales=(0.3, 1.0), cap=6.0),
                  retention_layer(heads=3, dim=16, vdim=16, rot=8, decay=[0.99, 0.999, 0.9999], ff=0)], width=32)
    entry = model(tmp_path_factory, "pieces", raw)
    reqs = requests_for(entry, (1300, 40), seed=80)
    long_ids, short_ids = reqs["r0"], reqs["r1"]
    steps = [{"step": 0, "entries": [{"id": "r1", "tokens": short_ids[:30], "want": list(range(30))}], "end": []},
             {"step": 1, "entries": [{"id": "r0", "tokens": long_ids[:100], "want": list(range(100))},
                                      {"id": "r1", "tokens": short_ids[30:31], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "r1", "tokens": short_ids[31:32], "want": [0]},
                                      {"id": "r0", "tokens": long_ids[100:1290], "want": list(range(1190))}], "end": []}]
    for k in range(8):
        steps.append({"step": 3 + k, "entries": [{"id": "r0", "tokens": [long_ids[1290 + k]], "want": [0]},
                                                  {"id": "r1", "tokens": [short_ids[32 + k]], "want": [0]}],
                      "end": ["r0", "r1"] if k == 7 else []})
    got = run_trace(entry[0], "bfloat16", steps)
    assert_close(got["r0"][:1298], plain_rows(entry, long_ids)[:1298], "bfloat16", "long")
    assert_close(got["r1"], plain_rows(entry, short_ids), "bfloat16", "short")
    # the walk token by token and the walk in pieces agree to rounding
    one = run_trace(entry[0], "bfloat16", tail_decoded({"r0": long_ids[:1000]}, tail=8))
    assert_close(got["r0"][:1000], one["r0"], "bfloat16", "pieces against one walk")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(tmp_path_factory, dtype):
    entry = model(tmp_path_factory, "other", other_sizes_config(), seed=11)
    reqs = requests_for(entry, (75, 20, 1), seed=20)
    compare(entry, dtype, whole(reqs), reqs)
    compare(entry, dtype, mixed(reqs, max_live=2, portion=11, decode_tail=9, seed=3), reqs, page_size=4, max_reside=2)


# ------------------------------------------------------------------------------- generation through the engine

def _greedy_plain(entry, prompt, n):
    c, w = entry[1]
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain.forward(c, w, ids)[0][-1].argmax()))
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
        lg = plain.forward(c, w, p + r.output_ids)[0]
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


def test_command_line_runs_the_model(tmp_path_factory):
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
