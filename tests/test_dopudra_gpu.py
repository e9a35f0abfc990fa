"""The Dopudra decoder in the engine against the plain implementation (`plain_dopudra`): every
mechanism alone, every way of cutting requests into steps, slots and pages used again, planted
weights where random ones would hide a fault, and greedy generation through the entry point."""

import copy
import random

import pytest
import torch

import dopudra_helpers as D
import helpers as H
import plain_dopudra as P

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
LENGTHS = {"X": [1, 2, 3, 17, 33, 70, 150], "Y": [2, 5, 31, 64, 65, 200]}


def _requests(name, seed, lengths):
    rng = random.Random(seed)
    vocab = D.CONFIGS[name][0]["vocab"]
    return {f"r{i}": H.random_ids(rng, n, vocab) for i, n in enumerate(lengths)}


# --------------------------------------------------------------------- mechanisms, one at a time

def _one_layer(name, layer, streams, seed, **top):
    cfg = dict(copy.deepcopy(D.CFG_X), layers=[copy.deepcopy(layer)], streams=streams, **top)
    folder = H.tmp_root() / f"dopudra-one-{name}"
    D.register(folder, cfg, D.random_tensors(cfg, 6, 9, seed))
    return folder, cfg


ALONE = {
    "lightning": (D.lightning(3, 16, 24, [0.95, 1.0, 0.2]), 2),
    "lightning_ff": (D.lightning(1, 48, 8, [0.9], ff=56), 1),
    "softmax_branch": (D.parallel(D.left(4, 2, 16, 8, 4, 0.3, 40, 0.5, 5), D.right(1, 8, 8, 2.0), 1.0, 0.0), 4),
    "softmax_branch_equal_heads": (D.parallel(D.left(6, 2, 48, 48, 3, 0.2, 25, 0.4, 9), D.right(1, 8, 8, 2.0), 1.1, 0.0), 2),
    "gated_branch": (D.parallel(D.left(1, 1, 8, 8, 2, 0.3, 40, 0.5, 5), D.right(3, 16, 24, 3.0), 0.0, 1.0), 3),
    "both_branches_ff": (D.parallel(D.left(2, 1, 24, 16, 3, 0.2, 60, 0.2, 3), D.right(2, 8, 16, 8.0), 0.6, 1.4, ff=72), 2),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", sorted(ALONE))
def test_each_mixer_alone(which, dtype):
    layer, streams = ALONE[which]
    folder, cfg = _one_layer(which, layer, streams, 11)
    rng = random.Random(5)
    requests = {"a": H.random_ids(rng, 90, cfg["vocab"]), "b": H.random_ids(rng, 1, cfg["vocab"])}
    steps = H.trace_whole(requests)
    got = H.Replayer(folder, dtype, 16, H.peak_tokens(steps, 16)).run(steps)
    D.check(folder, requests, got, dtype)
    # the same tokens in portions and one by one give the same logits
    steps = H.trace_portions({"a": requests["a"]}, random.Random(1))
    got = H.Replayer(folder, dtype, 16, 96, shuffle_seed=2).run(steps)
    D.check(folder, {"a": requests["a"]}, got, dtype)


@pytest.mark.parametrize("streams", [1, 2, 5])
def test_stream_step_kernel(streams):
    from bare_cuda_4gib_b200.kernels import lib as K, streams as SK
    g = torch.Generator().manual_seed(streams)
    n, width = 7, 40
    xs = torch.randn(streams, n, width, generator=g, dtype=torch.float64)
    y = torch.randn(2, n, width, generator=g, dtype=torch.float64)        # two partial sums
    w = {"l.hc1.in": torch.randn(streams, generator=g, dtype=torch.float64),
         "l.hc1.out": torch.randn(streams, generator=g, dtype=torch.float64),
         "l.hc1.mix": torch.randn(streams, streams, generator=g, dtype=torch.float64),
         "l.ls1": torch.randn(width, generator=g, dtype=torch.float64)}
    norm_w = torch.randn(width, generator=g, dtype=torch.float64)
    read_next = torch.randn(streams, generator=g, dtype=torch.float64)
    want_streams = P.stream_sublayer(xs, w, "l", 1, norm_w, 1e-5, lambda h: y.sum(0))
    want_h = P.rms(torch.einsum("s,stc->tc", read_next, want_streams), 1e-5) * norm_w
    dev = lambda t: t.float().cuda().contiguous()
    buf = dev(xs.permute(1, 0, 2).reshape(n, streams * width))
    out = torch.empty(n, width, device="cuda")
    pending = SK.StreamWrite(K.Partials(dev(y), 2), dev(w["l.ls1"]), dev(w["l.hc1.out"]), dev(w["l.hc1.mix"]))
    SK.stream_step(buf, streams, pending, dev(read_next), dev(norm_w), out, 1e-5, n, width)
    torch.cuda.synchronize()
    assert H.row_error(buf.view(n, streams, width).permute(1, 0, 2), want_streams) < 1e-5
    assert H.row_error(out, want_h) < 1e-5


# ------------------------------------------------------------------ every cutting, two configs

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["X", "Y"])
def test_whole(name, dtype):
    folder, page = D.model_folder(name), D.CONFIGS[name][1]
    requests = _requests(name, 1, LENGTHS[name])
    steps = H.trace_whole(requests)
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page)).run(steps)
    D.check(folder, requests, got, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["X", "Y"])
def test_prefill_then_token_by_token(name, dtype):
    folder, page = D.model_folder(name), D.CONFIGS[name][1]
    requests = _requests(name, 2, LENGTHS[name][3:])
    steps = H.trace_decode_tail(requests, 40)
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page), shuffle_seed=3).run(steps)
    D.check(folder, requests, got, dtype, expect_all=False)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["X", "Y"])
def test_portions_down_to_two_tokens(name, dtype):
    folder, page = D.model_folder(name), D.CONFIGS[name][1]
    requests = _requests(name, 3, LENGTHS[name][2:])
    steps = H.trace_portions(requests, random.Random(5))
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page), shuffle_seed=4).run(steps)
    D.check(folder, requests, got, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["X", "Y"])
def test_mixed_batches_reuse_slots_and_pages(name, dtype):
    """Unequal requests side by side, four slots and a small pool for eleven requests: every logit
    equals the request's alone, whatever slot and pages it got and whoever held them before."""
    folder, page = D.model_folder(name), D.CONFIGS[name][1]
    longest = D.CONFIGS[name][0]["max_positions"]
    rng = random.Random(11)
    requests = _requests(name, 4, [rng.randrange(3, longest // 2) for _ in range(10)] + [longest])
    budget = 2 * longest
    steps = H.trace_mixed(requests, random.Random(6), live=4, budget_tokens=budget, page=page)
    rep = H.Replayer(folder, dtype, page, budget, max_live=4, shuffle_seed=9)
    got = rep.run(steps)
    D.check(folder, requests, got, dtype)
    pool = rep.cache.groups[0].pool
    assert pool.acquired_total > pool.num_pages and pool.pages_in_use == 0
    assert rep.cache.free_slots == 4


@pytest.mark.parametrize("name", ["X", "Y"])
def test_long_decoding_in_graphs(name):
    """Three tokens of prompt, then a hundred and more one by one (captured as CUDA graphs after the
    second step), two requests of different age side by side."""
    folder, page = D.model_folder(name), D.CONFIGS[name][1]
    requests = _requests(name, 8, [140, 120])
    a, b = requests["r0"], requests["r1"]
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": a[:3], "want": [2]}], "end": []}]
    for i in range(3, 140):
        entries = [{"id": "r0", "tokens": [a[i]], "want": [0]}]
        j = i - 20
        if j == 0:
            entries.append({"id": "r1", "tokens": b[:1], "want": [0]})
        elif 0 < j < 120:
            entries.append({"id": "r1", "tokens": [b[j]], "want": [0]})
        steps.append({"step": i, "entries": entries, "end": []})
    rep = H.Replayer(folder, "float32", page, 320, max_live=4)
    got = rep.run(steps)
    assert rep.runner._graphs, "no step was replayed from a CUDA graph"
    D.check(folder, requests, got, "float32", expect_all=False)


# ------------------------------------------------------------------------------ planted weights

def _planted_far_key(seed):
    """One layer, the softmax branch alone.  Token 1's embedding lies along one direction, every
    other token's is orthogonal to it, and the query and key projections read that direction
    strongly: a query at token 1 finds the one earlier token 1, however far back."""
    layer = D.parallel(D.left(2, 1, 64, 64, 2, 0.5, 30, 0.0, 1), D.right(1, 8, 8, 2.0), 1.0, 0.0)
    cfg = dict(copy.deepcopy(D.CFG_X), layers=[layer], streams=2, max_positions=256)
    t = {k: v.float() for k, v in D.random_tensors(cfg, 4, 8, seed).items()}
    d = torch.zeros(cfg["width"])
    d[0] = 1.0
    t["embed"][:, 0] = 0.0
    t["embed"][1] = 8.0 * d
    t["pos"].zero_()
    for name in ("l0.mix.left.q", "l0.mix.left.k"):
        t[name][:, 0] = 3.0
    for name in ("l0.mix.left.q.conv", "l0.mix.left.k.conv"):       # the newest tap passes, the older one barely
        t[name][:, 0] *= 0.1
        t[name][:, 1] = 1.0
    t["l0.mix.left.rel"] *= 0.25
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    folder = H.tmp_root() / f"dopudra-planted-{seed}"
    D.register(folder, cfg, t)
    return folder, cfg


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_key_decides(dtype):
    folder, cfg = _planted_far_key(21)
    rng = random.Random(2)
    filler = lambda n: [rng.randrange(2, cfg["vocab"]) for _ in range(n)]
    ids = filler(9) + [1] + filler(190) + [1] + filler(3)      # the far key is 191 positions back, past a page border
    at = 200
    without = list(ids)
    without[9] = 5
    moved = H.row_error(P.forward(cfg, D._tensors[str(folder)], without)[at], D.plain_logits(folder, ids)[at])
    assert moved > 0.2, f"the planted key moves the logits by only {moved:.3f}"
    # in one prompt, and with the query decoded alone after portions
    requests = {"p": ids}
    got = H.Replayer(folder, dtype, 16, 208).run(H.trace_whole(requests))
    D.check(folder, requests, got, dtype)
    got = H.Replayer(folder, dtype, 16, 208, shuffle_seed=5).run(H.trace_decode_tail(requests, 8))
    D.check(folder, requests, got, dtype, expect_all=False)


@pytest.mark.parametrize("dtype", DTYPES)
def test_undecayed_head_keeps_the_first_token(dtype):
    """A head with decay one: the first token's key and value are in every later output."""
    layer = D.lightning(2, 16, 16, [1.0, 0.5])
    cfg = dict(copy.deepcopy(D.CFG_X), layers=[layer], streams=1, max_positions=256)
    t = {k: v.float() for k, v in D.random_tensors(cfg, 4, 8, 31).items()}
    t["l0.mix.v"][:16] *= 6.0
    t["pos"].zero_()
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    folder = H.tmp_root() / "dopudra-undecayed"
    D.register(folder, cfg, t)
    rng = random.Random(4)
    ids = H.random_ids(rng, 180, cfg["vocab"])
    other = [(ids[0] + 1) % cfg["vocab"]] + ids[1:]
    moved = H.row_error(P.forward(cfg, t, other)[179], D.plain_logits(folder, ids)[179])
    assert moved > 1e-3
    got = H.Replayer(folder, dtype, 16, 192, shuffle_seed=1).run(H.trace_decode_tail({"p": ids}, 30))
    D.check(folder, {"p": ids}, got, dtype, expect_all=False)


# ----------------------------------------------------------------- the entry point and scheduler

@pytest.mark.parametrize("name", ["X", "Y"])
def test_greedy_generation_through_the_engine(name):
    from bare_cuda_4gib_b200.engine.engine import LLMEngine

    folder, page = D.model_folder(name), D.CONFIGS[name][1]
    cfg = D.CONFIGS[name][0]
    rng = random.Random(13)
    prompts = [H.random_ids(rng, n, cfg["vocab"]) for n in (5, 23, 1, 40, 12, 9)]
    engine = LLMEngine(str(folder), max_tokens=96, max_seqs=4, dtype="float32", page_tokens=page, max_step_tokens=24)
    out = engine.generate_batch(prompts, 24)
    alone = engine.generate(prompts[1], 24)
    assert alone == out[1]
    for prompt, new in zip(prompts, out):
        assert len(new) == 24
        logits = D.plain_logits(folder, prompt + new[:-1])
        for i, token in enumerate(new):
            row = logits[len(prompt) - 1 + i]
            best = int(row.argmax())
            if token != best:        # a tie within float32 rounding may go either way
                assert float(row[best] - row[token]) < 1e-4 * float(row.abs().max()), (i, token, best)


# ------------------------------------------------------------------------- command line tools

def _tool(tool, *args, feed=None):
    import os
    import pathlib
    import subprocess
    import sys

    root = pathlib.Path(__file__).resolve().parents[1]
    done = subprocess.run([sys.executable, str(root / "bin" / tool), *map(str, args)], input=feed, capture_output=True,
                          text=True, env=dict(os.environ, PYTHONDONTWRITEBYTECODE="1"), timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    return done.stdout


def test_llm_infer_prints_the_plain_greedy_tokens():
    folder = D.model_folder("Y")
    prompt = [5, 17, 3, 100, 9, 41, 77]
    out = _tool("llm-infer", "--model", folder, "--prompt", ",".join(map(str, prompt)), "--tokens", 10, "--dtype",
                "float32", "--page-tokens", 32)
    generated = [int(t) for t in out.split("generated:")[1].split()]
    assert len(generated) == 10
    logits = D.plain_logits(folder, prompt + generated[:-1])
    assert generated == [int(logits[len(prompt) - 1 + i].argmax()) for i in range(10)]
    assert out.splitlines()[0].startswith("[llm] 3 layers, hidden 96, vocab 130")


def test_llm_infer_runs_a_preset_with_random_weights(tmp_path):
    out = _tool("llm-infer", "--model", tmp_path / "m", "--random", "dopudra-tiny", "--prompt", "1,2,3", "--tokens", 5)
    assert len(out.split("generated:")[1].split()) == 5


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_tool(dtype, tmp_path):
    """bin/trace_run on two requests that share steps; the second takes the first one's slot and pages."""
    import json
    import numpy as np

    folder = D.model_folder("X")
    requests = _requests("X", 17, [40, 19, 33])
    a, b, c = requests["r0"], requests["r1"], requests["r2"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:2], "want": [1]}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [16]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[30:39], "want": []}, {"id": "c", "tokens": c, "want": [32]}], "end": ["c"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[39:], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "out"
    printed = _tool("trace_run", "--model", folder, "--dtype", dtype, "--out", out, "--max-tokens", 128, "--page-tokens", 16,
                    feed="".join(json.dumps(s) + "\n" for s in steps))
    assert [l for l in printed.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    want = {0: [("r0", 0), ("r0", 29), ("r1", 1)], 1: [("r1", 18)], 2: [("r2", 32)], 3: [("r0", 39)]}
    vocab = D.CONFIGS["X"][0]["vocab"]
    for step, rows in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), vocab).copy())
        for i, (rid, p) in enumerate(rows):
            err = H.row_error(got[i], D.plain_logits(folder, requests[rid])[p])
            assert err <= D.TOLERANCE[dtype], (step, rid, p, err)


# ------------------------------------------------------------ long portions walked in stretches

@pytest.mark.parametrize("rank", [8, 5])      # 5: the projection's rows are not 16-byte aligned
def test_long_portions_walked_in_stretches(rank, monkeypatch):
    """A bfloat16 step whose portions are several hundred tokens long walks the linear-attention
    states in stretches side by side and joins them: the same logits as one walk, and the plain
    implementation's; two requests of different length in one step, the second carried on."""
    from bare_cuda_4gib_b200.kernels import linear_attention as LA

    layers = [D.lightning(2, 16, 16, [1.0, 0.9]),
              D.parallel(D.left(2, 1, 16, 16, 3, 0.25, 300, 0.2, 50), D.right(2, 64, 8, 4.0), 0.8, 1.2, ff=48)]
    cfg = dict(copy.deepcopy(D.CFG_Y), layers=layers, streams=2, max_positions=704)
    folder = H.tmp_root() / f"dopudra-stretches-{rank}"
    D.register(folder, cfg, D.random_tensors(cfg, rank, 12, 41))
    rng = random.Random(3)
    a, b = H.random_ids(rng, 700, cfg["vocab"]), H.random_ids(rng, 640, cfg["vocab"])
    tail = lambda n, k=24: list(range(n - k, n))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:650], "want": [0, 127, 128, 129, 255, 256, 400] + tail(650)},
                                     {"id": "b", "tokens": b[:2], "want": [1]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[650:], "want": tail(50, 10)},
                                     {"id": "b", "tokens": b[2:], "want": [0, 125, 126, 127, 300] + tail(638)}], "end": ["a", "b"]}]
    cut = H.Replayer(folder, "bfloat16", 64, 1408).run(steps)
    monkeypatch.setattr(LA, "STRETCHES_FROM", 1 << 30)
    whole = H.Replayer(folder, "bfloat16", 64, 1408).run(steps)
    assert sorted(cut) == sorted(whole)
    for key in cut:
        assert H.row_error(cut[key], whole[key]) < 1e-2, key
    D.check(folder, {"a": a, "b": b}, cut, "bfloat16", expect_all=False)


# ----------------------------------------------------------------- configurations drawn at random

def _random_config(seed):
    rng = random.Random(seed)
    pick = rng.choice
    width = pick([40, 64, 72, 100, 128, 136])
    streams = pick([1, 2, 3, 4, 6])

    def ff():
        return pick([None, pick([24, 50, 96, 160])])

    def light():
        heads = pick([1, 2, 3, 5])
        return D.lightning(heads, pick([4, 8, 12, 16, 32, 40, 64]), pick([4, 8, 10, 16, 24, 64]),
                           [pick([1.0, 0.999, 0.9, 0.5, 0.0]) for _ in range(heads)], ff=ff())

    def both():
        kv = pick([1, 2, 3])
        heads = kv * pick([1, 2, 4])
        dim = pick([8, 12, 16, 32, 48, 64])
        vdim = pick([dim, dim, pick([8, 16, 20, 40])])
        l = D.left(heads, kv, dim, vdim, pick([1, 2, 3, 4, 6]), pick([0.1, 0.3, dim ** -0.5]), pick([6, 30, 64, 500]),
                   pick([0.0, 0.25, 1.0]), pick([1, 3, 16, 64]))
        r = D.right(pick([1, 2, 4]), pick([4, 8, 16, 24, 64]), pick([4, 8, 16, 32]), pick([1.0, 2.0, 16.0]))
        return D.parallel(l, r, pick([0.5, 1.0, 1.2]), pick([0.7, 1.0, 1.1]), ff=ff())

    layers = [pick([light, both])() for _ in range(rng.randrange(1, 5))]
    cfg = {"architecture": "Dopudra", "vocab": pick([50, 97, 301]), "width": width, "max_positions": 128, "streams": streams,
           "embedding": {"scale": pick([0.5, 1.0, 3.0])}, "norm": {"eps": pick([1e-6, 1e-5])}, "layers": layers}
    return cfg, pick([3, 4, 8, 16]), pick([2, 6, 8, 10])        # rank; table rows (half of them below every far distance)


@pytest.mark.parametrize("seed", range(16))
def test_configurations_drawn_at_random(seed):
    cfg, rank, rows = _random_config(100 + seed)
    folder = H.tmp_root() / f"dopudra-random-{seed}"
    D.register(folder, cfg, D.random_tensors(cfg, rank, rows, seed))
    rng = random.Random(seed)
    requests = {"a": H.random_ids(rng, 70, cfg["vocab"]), "b": H.random_ids(rng, 33, cfg["vocab"]),
                "c": H.random_ids(rng, 9, cfg["vocab"])}
    page = rng.choice([16, 32, 64])
    steps = H.trace_mixed(requests, random.Random(seed), live=2, budget_tokens=256, page=page)
    got = H.Replayer(folder, "float32", page, 256, max_live=2, shuffle_seed=seed).run(steps)
    D.check(folder, requests, got, "float32")
    # bfloat16: the fast kernels against the plain ones row by row, and both against the plain implementation
    fast = H.Replayer(folder, "bfloat16", page, 256, max_live=2, shuffle_seed=seed).run(steps)
    slow = H.Replayer(folder, "bfloat16", page, 256, max_live=2, shuffle_seed=seed, use_fast_gemm=False,
                      use_fast_attention=False).run(steps)
    assert sorted(fast) == sorted(slow) and len(fast) == sum(len(ids) for ids in requests.values())
    agree = sorted(H.row_error(fast[key], slow[key]) for key in fast)
    assert agree[int(0.95 * len(agree))] <= 2e-2 and agree[-1] <= 0.3, agree[-3:]
    D.check_most(folder, requests, fast, "bfloat16")


def test_the_other_tools_take_the_design(tmp_path):
    """llm-bench, llm-ppl and llm-batch-check on a preset with random weights: perplexity against the
    plain implementation's, the batch check's verdict, the bench tool's table."""
    import json
    import math

    import numpy as np
    from bare_cuda_4gib_b200.weights.safetensors_io import SafetensorsFile

    folder = tmp_path / "m"
    out = _tool("llm-bench", "--model", folder, "--random", "dopudra-tiny", "--prompt-len", 24, "--tokens", 8, "--runs", 2,
                "--warmup", 1, "--page-tokens", 16)
    assert "TTFT" in out and "TPOT" in out
    rng = random.Random(9)
    ids = np.array([rng.randrange(300) for _ in range(8200)], dtype="<i4")
    ids.tofile(tmp_path / "ids.bin")
    out = _tool("llm-ppl", "--model", folder, "--ids", tmp_path / "ids.bin", "--ctx", 48, "--windows", 2, "--dtype", "float32",
                "--page-tokens", 16)
    got = float([l for l in out.splitlines() if l.startswith("perplexity")][0].split()[1])
    cfg = json.loads((folder / "config.json").read_text())
    with SafetensorsFile(folder / "model.safetensors") as f:
        tensors = {name: f.tensor(name) for name in f.entries}
    nll, n = 0.0, 0
    for w in range(2):
        window = [1] + [int(t) for t in ids[w * 47: (w + 1) * 47]]      # the tool puts id 1 before every window
        logp = torch.log_softmax(P.forward(cfg, tensors, window), -1)
        for t in range(47):
            nll -= float(logp[t, window[t + 1]])
            n += 1
    assert abs(got - math.exp(nll / n)) <= 1e-3 * math.exp(nll / n), (got, math.exp(nll / n))
    out = _tool("llm-batch-check", "--model", folder, "--ids", tmp_path / "ids.bin", "--tokens", 12, "--batch", 4,
                "--page-tokens", 16, "--dtype", "float32")
    assert "PASS" in out
