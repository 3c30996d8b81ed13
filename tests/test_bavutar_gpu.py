"""The Bavutar design in the engine against the plain implementation (tests/plain_bavutar.py):
each mixer alone, whole prompts against token-by-token decoding, portions down to two tokens,
mixed batches with pages and state slots that are used again, far keys and page borders, the
edges of the query temperature's steps, the first tokens of a sequence, long decoding, other
sizes (also values equal to one another or to 1), and greedy generation through ``LLM``."""
import json
import os

import numpy as np
import pytest
import torch

import plain_bavutar as pb
import trace_util as tu

pytestmark = pytest.mark.gpu


def attn(heads, kv, dim, vdim, every=8, coef=0.6, scale=None, kv_from=None, ff=None, temp=True):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if temp:
        m["q_temp"] = {"coef": coef, "every": every}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def ssm(heads, vdim, state, groups, conv, norm_groups, ff=None):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta(heads, kv, dim, vdim, conv, rank, ff=None):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv,
                                               "rank": rank}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(width, vocab, layers, alpha=2.0, scale=6.0, cap=8.0, eps=1e-5):
    return {"architecture": "Bavutar", "vocab": vocab, "width": width, "layers": layers, "postln_alpha": alpha,
            "embedding": {"scale": scale}, "logit_softcap": cap, "norm": {"eps": eps}}


CONFIGS = {
    # every mixer; values of their own size; a layer without feed-forward; a borrowed cache
    "hybrid": config(96, 160, [ssm(4, 16, 24, 1, 3, 1, ff=128), attn(6, 3, 32, 16, every=8), delta(4, 2, 24, 40, 2, 12, ff=64),
                               attn(6, 3, 32, 16, every=5, coef=0.3, kv_from=1, ff=128)]),
    # head sizes the tensor-core attention kernels take in bfloat16 (64), groups of several heads
    "wide": config(128, 200, [attn(4, 1, 64, 64, every=16, ff=192), ssm(4, 32, 64, 2, 4, 4, ff=192),
                              delta(2, 2, 64, 64, 4, 16), attn(4, 1, 64, 64, every=7, kv_from=0, ff=96)], alpha=1.5),
    # head size 128; sizes that are equal or 1; no temperature, no cap
    "ones": config(64, 96, [attn(1, 1, 128, 128, temp=False, ff=64), ssm(1, 64, 128, 1, 2, 1), delta(1, 1, 128, 32, 3, 4, ff=64),
                            ssm(2, 8, 8, 2, 5, 2)], alpha=1.0, scale=1.0, cap=None),
    # sizes that are multiples of nothing in particular
    "odd": config(52, 77, [delta(3, 3, 10, 6, 3, 5, ff=50), attn(3, 1, 20, 12, every=9, ff=30), ssm(5, 10, 12, 5, 4, 1),
                           attn(3, 1, 20, 12, every=11, coef=0.2, kv_from=1)], alpha=3.0, scale=2.0, cap=4.0),
    # no attention at all
    "stateful": config(48, 64, [delta(3, 1, 16, 16, 4, 8, ff=96), ssm(3, 16, 16, 3, 4, 3)]),
}


def write_folder(folder, cfg, seed):
    from safetensors.torch import save_file
    w = pb.random_weights(cfg, seed)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(folder, "model.safetensors"))
    return w


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        d = str(tmp_path_factory.mktemp("bav_" + name))
        out[name] = (d, cfg, write_folder(d, cfg, 11 + i))
    return out


_plain_cache = {}


def plain_logits(name, cfg, w, seqs):
    out = {}
    for sid, toks in seqs.items():
        key = (name, tuple(toks))
        if key not in _plain_cache:
            _plain_cache[key] = pb.forward(cfg, w, toks, torch.float64).float().numpy()
        out[sid] = _plain_cache[key]
    return out


def row_errors(got, ref):
    """Worst difference of a logits row (mean taken off, root mean square) in units of the
    reference rows' root mean square; also where it is."""
    rows = np.stack([ref[sid][p] for sid, p in got])
    rms = float(np.sqrt((rows.astype(np.float64) ** 2).mean()))
    worst, where = 0.0, None
    for (sid, p), row in got.items():
        d = row.astype(np.float64) - ref[sid][p]
        d -= d.mean()
        e = float(np.sqrt((d * d).mean())) / rms
        if not e == e:
            e = float("inf")
        if e > worst:
            worst, where = e, (sid, p)
    return worst, where


# bfloat16: what rounding alone does to these small models (measured up to 4.3e-2); the 32-bit runs carry the sharp bound
BOUND = {"float32": 2e-5, "bfloat16": 6e-2}


def make_runner(folder, dtype, steps, page_size=16, rows=4, **kw):
    from sparseengine_b200.engine.factory import build_runner
    tokens = tu.max_live_tokens(steps, round_to=page_size)
    return build_runner(folder, dtype=dtype, page_size=page_size, num_pages=max(1, tokens // page_size), max_rows=rows,
                        max_seq_len=max(64, tokens), **kw)


def check_trace(folders, name, dtype, steps, seqs, what, bound=None, **kw):
    folder, cfg, w = folders[name]
    runner = make_runner(folder, dtype, steps, **kw)
    got = tu.run_trace_runner(runner, steps)
    from sparseengine_b200.csrc import ops
    ops.error_check(runner.device)
    runner.cache.check()
    assert runner.cache.free_rows == runner.cache.max_rows
    worst, where = row_errors(got, plain_logits(name, cfg, w, seqs))
    assert worst < (bound or BOUND[dtype]), f"{what} ({name}, {dtype}): row error {worst:.3e} at {where}"
    return runner


def prompts(cfg, lengths, seed):
    return {f"s{i}": tu.random_prompt(cfg["vocab"], n, seed + i) for i, n in enumerate(lengths)}


# ---- each mechanism alone ----------------------------------------------------------------------

SINGLE = {
    "attention": [attn(4, 2, 16, 24, every=4, coef=0.9, ff=None)],
    "attention_shared": [attn(2, 2, 32, 32, every=6), attn(2, 2, 32, 32, every=3, kv_from=0)],
    "state_space": [ssm(4, 8, 12, 2, 4, 2)],
    "gated_delta": [delta(4, 2, 12, 20, 4, 6)],
    "feed_forward": [ssm(1, 8, 4, 1, 2, 1, ff=80)],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(SINGLE))
def test_each_mixer_alone(tmp_path, which, dtype):
    cfg = config(40, 50, SINGLE[which], alpha=1.7, scale=3.0, cap=None)
    w = write_folder(str(tmp_path), cfg, 5)
    seqs = prompts(cfg, (37, 1, 18), 3)
    for cut in (tu.trace_whole, lambda s: tu.trace_chunks(s, sizes=(2, 3, 1, 5, 2)), lambda s: tu.trace_tail_decode(s, tail=9)):
        steps = cut(seqs)
        check_trace({which: (str(tmp_path), cfg, w)}, which, dtype, steps, seqs, "alone")


# ---- ways of cutting ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_decode_chunks_mixed(folders, name, dtype):
    cfg = CONFIGS[name]
    seqs = prompts(cfg, (70, 33, 1, 18, 49, 2, 26), 20)
    check_trace(folders, name, dtype, tu.trace_whole(seqs), seqs, "whole")
    check_trace(folders, name, dtype, tu.trace_tail_decode(seqs, tail=20), seqs, "decode")
    check_trace(folders, name, dtype, tu.trace_chunks(seqs), seqs, "portions")
    check_trace(folders, name, dtype, tu.trace_chunks(seqs, sizes=(2,)), seqs, "portions of two")
    # three rows for seven requests, and a pool of the live tokens only: rows, state slots and pages are used again
    runner = check_trace(folders, name, dtype, tu.trace_mixed(seqs, live=3, chunk=6, decode_tail=5), seqs, "mixed", rows=3)
    assert all(g.pool.reused_total > 0 for g in runner.cache.groups)
    check_trace(folders, name, dtype, tu.trace_random(seqs, seed=3, live=4), seqs, "random schedule", page_size=8)


def test_a_state_slot_that_is_used_again_starts_from_zero(folders):
    """One row: every request gets the slot the one before it left; a long request first, so that
    its state is far from zero."""
    name = "stateful"
    cfg = CONFIGS[name]
    seqs = prompts(cfg, (60, 5, 1, 9), 40)
    check_trace(folders, name, "float32", tu.trace_chunks(seqs, sizes=(7, 2)), seqs, "one slot", rows=1)


# ---- places where a fault would sit --------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_and_page_borders(tmp_path, dtype):
    """A sharp softmax (large score scale) makes every query hang on the one or two keys with
    the highest score, which among hundreds of random keys mostly lie far back; a key that is
    missed, or read from the wrong place of a page, changes the row.  Prompts end around page
    borders, and decoding runs across them.  (In bfloat16 the rounding of queries and keys moves
    such sharp weights by themselves, hence the wider bound there; a lost key moves the row by
    its whole size.)"""
    cfg = config(64, 80, [attn(4, 2, 32, 32, every=64, coef=0.5, scale=1.5, ff=64),
                          attn(4, 2, 32, 32, every=50, coef=0.5, scale=1.5, kv_from=0)], cap=None)
    w = write_folder(str(tmp_path), cfg, 9)
    seqs = prompts(cfg, (415, 16, 17, 15, 305), 60)
    fs = {"far": (str(tmp_path), cfg, w)}
    bound = 0.25 if dtype == "bfloat16" else None
    check_trace(fs, "far", dtype, tu.trace_whole(seqs), seqs, "far keys, whole", bound)
    check_trace(fs, "far", dtype, tu.trace_tail_decode(seqs, tail=40), seqs, "far keys, decoded", bound)
    check_trace(fs, "far", dtype, tu.trace_chunks(seqs, sizes=(15, 2, 16, 33, 1, 64)), seqs, "far keys, portions", bound)


def test_sharp_attention_really_looks_far_back():
    """The premise of the test above, on the plain implementation: with that scale a query's
    heaviest key carries a large share of the weight (equal tokens share it: the first layer's keys
    do not know their position) and lies more than 64 positions back."""
    cfg = config(64, 80, [attn(4, 2, 32, 32, every=64, coef=0.5, scale=1.5)], cap=None)
    w = {k: v.double() for k, v in pb.random_weights(cfg, 9).items()}
    toks = torch.tensor(tu.random_prompt(80, 415, 60))
    x = w["embed"][toks] * cfg["embedding"]["scale"]
    m = cfg["layers"][0]["mixer"]
    k, _ = pb.attention_keys_values(x, w, "l0.mix.", m, 1e-5)
    q = (pb.rms(x @ w["l0.mix.q"].T, 1e-5) * w["l0.mix.q.norm"]).view(415, 4, 32)
    s = (q[:, 0] @ k[:, 0].T) * m["scale"]
    s = s.masked_fill(torch.triu(torch.ones(415, 415, dtype=torch.bool), 1), float("-inf"))
    p = torch.softmax(s, -1)
    top = p.argmax(-1)
    late = torch.arange(415) >= 200
    assert float(p.max(-1).values[late].mean()) > 0.2          # of 200 to 415 keys
    assert float(((torch.arange(415) - top)[late] > 64).float().mean()) > 0.9


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_query_temperature_steps(tmp_path, dtype):
    """The temperature changes at positions every-1, 2*every-1, ...; with a large coefficient a
    step taken one position early or late moves the logits far beyond rounding.  Positions on
    both sides of each step are decoded alone and sit in portions that start and end there."""
    cfg = config(48, 64, [attn(3, 3, 16, 16, every=6, coef=2.0, ff=64)], cap=None)
    w = write_folder(str(tmp_path), cfg, 13)
    seqs = prompts(cfg, (40, 12), 80)
    fs = {"temp": (str(tmp_path), cfg, w)}
    check_trace(fs, "temp", dtype, tu.trace_tail_decode(seqs, tail=30), seqs, "temperature, decoded")
    check_trace(fs, "temp", dtype, tu.trace_chunks(seqs, sizes=(5, 1, 6, 6, 7, 4)), seqs, "temperature, portions")
    # the plain implementation itself must be sensitive to the step's place
    other = json.loads(json.dumps(cfg))
    other["layers"][0]["mixer"]["q_temp"]["every"] = 7
    a = pb.forward(cfg, w, seqs["s0"], torch.float64)
    b = pb.forward(other, w, seqs["s0"], torch.float64)
    assert float((a - b).abs().max()) > 1e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_short_portions_under_the_convolution(tmp_path, dtype):
    """Five taps: the first four tokens of a request see zeros, a portion of one or two tokens
    takes its older inputs from the carried ones, which a portion shorter than the taps must
    shift rather than replace."""
    cfg = config(40, 48, [ssm(2, 8, 8, 1, 5, 1), delta(2, 1, 8, 8, 5, 4, ff=48)], cap=None)
    w = write_folder(str(tmp_path), cfg, 17)
    seqs = prompts(cfg, (1, 2, 3, 4, 5, 11), 90)
    fs = {"conv": (str(tmp_path), cfg, w)}
    check_trace(fs, "conv", dtype, tu.trace_whole(seqs), seqs, "first tokens")
    check_trace(fs, "conv", dtype, tu.trace_chunks(seqs, sizes=(1, 2, 1, 1, 3, 2)), seqs, "short portions")
    check_trace(fs, "conv", dtype, tu.trace_mixed(seqs, live=4, chunk=2, decode_tail=3), seqs, "short portions, mixed")


def test_long_decoding_through_replayed_graphs(folders):
    name = "hybrid"
    folder, cfg, w = folders[name]
    seqs = prompts(cfg, (170, 150), 120)
    steps = tu.trace_tail_decode(seqs, tail=140)
    runner = check_trace(folders, name, "float32", steps, seqs, "long decoding")
    assert runner.graph_replays > 200
    check_trace(folders, name, "bfloat16", steps, seqs, "long decoding")


def test_a_batch_does_not_change_a_request(folders):
    """Unequal requests in one step against each alone: equal up to the order of sums in 32-bit."""
    from sparseengine_b200.engine.runner import StepEntry
    name = "hybrid"
    folder, cfg, w = folders[name]
    seqs = prompts(cfg, (29, 3, 11), 140)
    steps = [{"step": 0, "entries": [{"id": sid, "tokens": toks} for sid, toks in seqs.items()], "end": []}]
    runner = make_runner(folder, "float32", steps, rows=4)       # pages for all three at once
    alone = {}
    for sid, toks in seqs.items():
        runner.admit(sid)
        runner.step([StepEntry(sid, toks[:-1], [])])
        alone[sid] = runner.step([StepEntry(sid, toks[-1:], [0])]).clone()
        runner.release(sid)
    for sid in seqs:
        runner.admit(sid)
    runner.step([StepEntry(sid, toks[:-1], []) for sid, toks in seqs.items()])
    together = runner.step([StepEntry(sid, toks[-1:], [0]) for sid, toks in seqs.items()])
    for i, sid in enumerate(seqs):
        assert float((together[i] - alone[sid][0]).abs().max()) < 2e-5 * float(alone[sid][0].abs().max()), sid


# ---- configuration and loading -------------------------------------------------------------------

def test_the_ranks_come_from_the_checkpoint(tmp_path):
    """The low ranks of the decay and gate projections are in no configuration key: the loader
    takes them from the tensors' shapes (here two different ones)."""
    from safetensors.torch import save_file
    from sparseengine_b200.config.registry import load_model_spec
    cfg = config(32, 40, [delta(2, 2, 8, 8, 2, 4)])
    w = pb.random_weights(cfg, 1)
    w["l0.mix.a1"] = torch.randn(6, 32).to(torch.bfloat16) * 0.2
    w["l0.mix.a2"] = torch.randn(16, 6).to(torch.bfloat16) * 0.2
    del cfg["layers"][0]["mixer"]["rank"]
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in w.items()}, str(tmp_path / "model.safetensors"))
    _, spec = load_model_spec(str(tmp_path))
    assert (spec.layers[0].mixer.decay_rank, spec.layers[0].mixer.gate_rank) == (6, 4)
    seqs = prompts(cfg, (9,), 1)
    cfg["layers"][0]["mixer"]["rank"] = 4       # the plain implementation only uses it for shapes
    check_trace({"r": (str(tmp_path), cfg, w)}, "r", "float32", tu.trace_whole(seqs), seqs, "ranks")


# ---- the entry point -----------------------------------------------------------------------------

def plain_greedy(cfg, w, prompt, steps):
    toks, out, margins = list(prompt), [], []
    for _ in range(steps):
        logits = pb.forward(cfg, w, toks, torch.float64)[-1]
        top = torch.topk(logits, 2).values
        margins.append(float(top[0] - top[1]))
        out.append(int(logits.argmax()))
        toks.append(out[-1])
    return out, margins


@pytest.mark.parametrize("name", ["hybrid", "stateful"])
def test_greedy_generation_through_the_entry_point(folders, name):
    from sparseengine_b200 import LLM, SamplingParams
    folder, cfg, w = folders[name]
    llm = LLM(folder, dtype="float32", page_size=8, num_kvcache_slots=512, max_num_batched_tokens=16, max_model_len=128,
              max_num_seqs_in_gpu=3)
    ps = [tu.random_prompt(cfg["vocab"], n, 200 + n) for n in (5, 21, 9, 2, 14)]
    outs = llm.generate(ps, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(ps, outs):
        want, margins = plain_greedy(cfg, w, p, 10)
        if min(margins) > 1e-4:
            assert o["token_ids"] == want
        else:       # a near-tie: the tokens up to it
            k = next(i for i, m in enumerate(margins) if m <= 1e-4)
            assert o["token_ids"][:k] == want[:k]
    assert llm.is_finished() and llm.runner.cache.free_rows == llm.runner.cache.max_rows


def test_trace_program(folders, tmp_path):
    """bin/trace_run as a program on a folder of this design, pages and slots used again."""
    name = "wide"
    folder, cfg, w = folders[name]
    seqs = prompts(cfg, (40, 7, 22, 31, 3), 300)
    steps = tu.trace_mixed(seqs, live=4, chunk=9, decode_tail=4)
    for dtype in ("float32", "bfloat16"):
        out = str(tmp_path / dtype)
        got = tu.run_trace_cli(folder, dtype, steps, out, tu.max_live_tokens(steps))
        worst, where = row_errors(got, plain_logits(name, cfg, w, seqs))
        assert worst < BOUND[dtype], (dtype, worst, where)


def test_temperature_sampling_through_the_entry_point_is_seeded(folders):
    """The engine's sampler on this design's logits: the same seed gives the same tokens, another
    seed others; top-k and top-p keep every token inside what the plain logits allow."""
    from sparseengine_b200 import LLM, SamplingParams
    folder, cfg, w = folders["hybrid"]
    ps = [tu.random_prompt(cfg["vocab"], n, 400 + n) for n in (3, 17, 8)]
    kw = dict(dtype="float32", page_size=8, num_kvcache_slots=512, max_model_len=128)
    sp = SamplingParams(temperature=0.9, top_k=5, max_tokens=8, ignore_eos=True)
    a = [o["token_ids"] for o in LLM(folder, seed=7, **kw).generate(ps, sp)]
    b = [o["token_ids"] for o in LLM(folder, seed=7, **kw).generate(ps, sp)]
    c = [o["token_ids"] for o in LLM(folder, seed=8, **kw).generate(ps, sp)]
    assert a == b and a != c
    for p, out in zip(ps, a):
        toks = list(p)
        for t in out:       # every sampled token is among the five most likely of the plain logits
            top = torch.topk(pb.forward(cfg, w, toks, torch.float64)[-1], 6).indices.tolist()
            assert t in top
            toks.append(t)


def test_command_line(folders, tmp_path):
    import subprocess
    import sys
    folder, cfg, w = folders["stateful"]
    hyper = json.dumps({"dtype": "bfloat16", "page_size": 8, "num_kvcache_slots": 1024, "max_model_len": 256})
    for extra in ([], ["--tiny_random"]):
        r = subprocess.run([sys.executable, "-m", "sparseengine_b200.cli.bench", "--model_path", folder, "--lengths", "24",
                            "--batch_sizes", "3", "--output_len", "6", "--random_prompts", "--generate", "--hyper_params", hyper,
                            *extra], cwd=tu.ROOT, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        assert r.stdout.strip()


def test_a_second_norm_without_a_feed_forward(tmp_path):
    """A layer without feed-forward has no second sublayer; a checkpoint that holds a second norm for
    it all the same gets that norm applied to alpha * x alone."""
    from safetensors.torch import save_file
    cfg = config(40, 48, [ssm(2, 8, 8, 1, 3, 1), attn(2, 1, 16, 16, every=4, ff=48)], cap=None)
    w = pb.random_weights(cfg, 23)
    w["l0.norm2"] = (1.0 + 0.1 * torch.randn(40)).to(torch.bfloat16)
    w["l0.norm2.b"] = (0.1 * torch.randn(40)).to(torch.bfloat16)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in w.items()}, str(tmp_path / "model.safetensors"))
    toks = tu.random_prompt(48, 19, 5)
    # plain: layer 0, then its bare second norm, then the rest
    wd = {k: v.double() for k, v in w.items()}
    x = wd["embed"][torch.tensor(toks)] * cfg["embedding"]["scale"]
    a, eps = cfg["postln_alpha"], cfg["norm"]["eps"]
    x = pb.layer_norm(a * x + pb.mamba2(x, wd, "l0.mix.", cfg["layers"][0]["mixer"], eps), wd["l0.norm1"], wd["l0.norm1.b"], eps)
    x = pb.layer_norm(a * x, wd["l0.norm2"], wd["l0.norm2.b"], eps)
    m = cfg["layers"][1]["mixer"]
    y = pb.attention(x, wd, "l1.mix.", m, eps, *pb.attention_keys_values(x, wd, "l1.mix.", m, eps))
    x = pb.layer_norm(a * x + y, wd["l1.norm1"], wd["l1.norm1.b"], eps)
    x = pb.layer_norm(a * x + pb.feed_forward(x, wd, "l1.mlp."), wd["l1.norm2"], wd["l1.norm2.b"], eps)
    ref = (pb.layer_norm(x, wd["final.norm"], wd["final.norm.b"], eps) @ wd["head"].T).float().numpy()
    seqs = {"s": toks}
    steps = tu.trace_chunks(seqs, sizes=(5, 2, 7))
    runner = make_runner(str(tmp_path), "float32", steps)
    got = tu.run_trace_runner(runner, steps)
    worst, where = row_errors(got, {"s": ref})
    assert worst < BOUND["float32"], (worst, where)
