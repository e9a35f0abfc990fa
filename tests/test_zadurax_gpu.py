"""The Zadurax decoder in the engine against the plain implementation (`plain_zadurax`): every
mechanism alone, every way of cutting requests into steps, slots and pages used again, planted
weights where random ones would hide a fault, and greedy generation through the entry point."""

import copy
import json
import random

import pytest
import torch

import helpers as H
import plain_zadurax as P
import zadurax_helpers as Z

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
LENGTHS = {"P": [1, 2, 3, 17, 33, 70, 150], "Q": [2, 5, 31, 64, 65, 200]}


def _requests(name, seed, lengths):
    rng = random.Random(seed)
    vocab = Z.CONFIGS[name][0]["vocab"]
    return {f"r{i}": H.random_ids(rng, n, vocab) for i, n in enumerate(lengths)}


# --------------------------------------------------------------------- mechanisms, one at a time

def _one_layer(name, layers, seed, width=72, vocab=61, eps=1e-5):
    cfg = {"architecture": "Zadurax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": copy.deepcopy(layers)}
    folder = H.tmp_root() / f"zadurax-one-{name}"
    Z.register(folder, cfg, Z.random_tensors(cfg, seed))
    return folder, cfg


ALONE = {
    "attention": [Z.attention(4, 2, 16, 20, 6)],
    "attention_one_key_head_whole_turn": [Z.attention(3, 1, 48, 7, 48, base=300.0, scale=0.3)],
    "attention_odd_head_size": [Z.attention(2, 2, 10, 33, 4)],          # no tensor-core kernel takes this size
    "attention_head_64": [Z.attention(4, 2, 64, 50, 32, ff=40)],
    "latent": [Z.latent(3, 12, 8, 20, 24, 0.2, scaling=Z.yarn(4.0, 64, 16.0, 2.0))],
    "latent_plain_frequencies": [Z.latent(1, 40, 4, 8, 33, 0.1, base=50.0)],
    "latent_many_heads": [Z.latent(11, 8, 6, 4, 16, 0.4, scaling=Z.yarn(8.0, 32, 8.0, 1.0), ff=56)],
    # sizes the tensor-core kernel takes in bfloat16: fewer heads than a tile has rows; two tiles of heads and
    # key blocks of 64; a cached vector so wide that key blocks are 32
    "latent_tensor_cores": [Z.latent(5, 16, 16, 8, 32, 0.2, scaling=Z.yarn(4.0, 64, 16.0, 2.0))],
    "latent_two_tiles_of_heads": [Z.latent(18, 8, 32, 8, 96, 0.15, base=1000.0)],
    "latent_wide": [Z.latent(2, 8, 32, 8, 256, 0.1, scaling=Z.yarn(2.0, 32, 4.0, 1.0))],
    "first_layer_uses_the_second_ones_tensors": [Z.again([None, Z.latent(2, 8, 8, 8, 16, 0.3)], 1), Z.latent(2, 8, 8, 8, 16, 0.3)],
    "mlstm": [Z.mlstm(3, 8, 20, 15.0)],
    "mlstm_one_head_tight_gates": [Z.mlstm(1, 40, 12, 1.5, ff=48)],
    "mlstm_wide": [Z.mlstm(2, 64, 64, 30.0)],
    "feed_forward_after_a_run_again": [Z.mlstm(2, 16, 16, 10.0, ff=100), Z.again([Z.mlstm(2, 16, 16, 10.0, ff=100)], 0)],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", sorted(ALONE))
def test_each_mixer_alone(which, dtype):
    folder, cfg = _one_layer(which, ALONE[which], 11)
    rng = random.Random(5)
    requests = {"a": H.random_ids(rng, 90, cfg["vocab"]), "b": H.random_ids(rng, 1, cfg["vocab"])}
    steps = H.trace_whole(requests)
    got = H.Replayer(folder, dtype, 16, H.peak_tokens(steps, 16)).run(steps)
    Z.check(folder, requests, got, dtype)
    # the same tokens in portions and one by one give the same logits
    steps = H.trace_portions({"a": requests["a"]}, random.Random(1))
    got = H.Replayer(folder, dtype, 16, 96, shuffle_seed=2).run(steps)
    Z.check(folder, {"a": requests["a"]}, got, dtype)


def test_norm_kernels():
    from bare_cuda_4gib_b200.kernels import lib as K, sandwich as SW
    g = torch.Generator().manual_seed(4)
    n, width = 9, 52
    x = torch.randn(n, width, generator=g, dtype=torch.float64)
    y = torch.randn(3, n, width, generator=g, dtype=torch.float64)       # three partial sums
    wb, wn = torch.randn(width, generator=g, dtype=torch.float64), torch.randn(width, generator=g, dtype=torch.float64)
    want_x = x + P.rms_norm(y.sum(0), wb, 1e-5)
    dev = lambda t: t.float().cuda().contiguous()
    res, out = dev(x), torch.empty(n, width, device="cuda")
    SW.postnorm_add_rmsnorm(res, SW.NormedDelta(K.Partials(dev(y), 3), dev(wb), 1e-5), dev(wn), out, 1e-6, n)
    assert H.row_error(res, want_x) < 1e-6 and H.row_error(out, P.rms_norm(want_x, wn, 1e-6)) < 1e-6
    # wanted rows only: the others stay as they were
    rows = torch.tensor([7, 2], dtype=torch.int32, device="cuda")
    res, out = dev(x), torch.empty(2, width, device="cuda")
    SW.postnorm_add_rmsnorm(res, SW.NormedDelta(K.Partials(dev(y), 3), dev(wb), 1e-5), dev(wn), out, 1e-6, 2, rows)
    assert H.row_error(out, P.rms_norm(want_x[[7, 2]], wn, 1e-6)) < 1e-6
    assert torch.equal(res[0].cpu(), x[0].float()) and H.row_error(res[7], want_x[7]) < 1e-6
    table = torch.randn(30, width, generator=g, dtype=torch.float64)
    ids = torch.tensor([3, 29, 0, 3], dtype=torch.int32, device="cuda")
    emb = torch.empty(4, width, device="cuda")
    SW.embed_rmsnorm(dev(table), ids, dev(wn), emb, 4, 1e-5)
    assert H.row_error(emb, P.rms_norm(table[[3, 29, 0, 3]], wn, 1e-5)) < 1e-6


@pytest.mark.parametrize("n,n_in,n_out,spare", [(70, 19, 66, 5), (150, 24, 72, 8), (9, 40, 13, 0), (200, 64, 8, 0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_matrix_per_head(dtype, n, n_in, n_out, spare):
    """Rows that are and are not 16-byte aligned, few and many tokens: every kernel of the product."""
    from bare_cuda_4gib_b200.kernels import latent as LT

    class Ctx:
        stream = 0

    Ctx.stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(8)
    heads = 3
    x = torch.randn(n, heads, n_in + spare, generator=g).to(dtype).cuda()      # rows wider than what is read
    w_rows = torch.randn(heads * n_in, n_out, generator=g).to(dtype).cuda()
    w_cols = torch.randn(heads * n_out, n_in, generator=g).to(dtype).cuda()
    gate = torch.randn(n, heads * n_out, generator=g).to(dtype).cuda()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    out = torch.zeros(n, heads, n_out + 3, dtype=dtype, device="cuda")
    LT.per_head_linear(Ctx, x, w_rows, True, out, heads, n_in, n_out, n)
    want = torch.einsum("thi,hio->tho", x[..., :n_in].double(), w_rows.double().view(heads, n_in, n_out))
    assert H.row_error(out[..., :n_out], want) < tol and float(out[..., n_out:].abs().max()) == 0.0
    out = torch.zeros(n, heads, n_out, dtype=dtype, device="cuda")
    LT.per_head_linear(Ctx, x, w_cols, False, out, heads, n_in, n_out, n, gate=gate)
    want = torch.einsum("thi,hoi->tho", x[..., :n_in].double(), w_cols.double().view(heads, n_out, n_in))
    want = want * torch.sigmoid(gate.double()).view(n, heads, n_out)
    assert H.row_error(out, want) < tol


# ------------------------------------------------------------------ every cutting, two configs

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_whole(name, dtype):
    folder, page = Z.model_folder(name), Z.CONFIGS[name][1]
    requests = _requests(name, 1, LENGTHS[name])
    steps = H.trace_whole(requests)
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page)).run(steps)
    Z.check(folder, requests, got, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_prefill_then_token_by_token(name, dtype):
    folder, page = Z.model_folder(name), Z.CONFIGS[name][1]
    requests = _requests(name, 2, LENGTHS[name][3:])
    steps = H.trace_decode_tail(requests, 45)          # longer than both windows: they pass over decoded tokens
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page), shuffle_seed=3).run(steps)
    Z.check(folder, requests, got, dtype, expect_all=False)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_portions_down_to_two_tokens(name, dtype):
    folder, page = Z.model_folder(name), Z.CONFIGS[name][1]
    requests = _requests(name, 3, LENGTHS[name][2:])
    steps = H.trace_portions(requests, random.Random(5))
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page), shuffle_seed=4).run(steps)
    Z.check(folder, requests, got, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_mixed_batches_reuse_slots_and_pages(name, dtype):
    """Unequal requests side by side, four slots and a small pool for eleven requests: every logit
    equals the request's alone, whatever slot and pages it got and whoever held them before."""
    folder, page = Z.model_folder(name), Z.CONFIGS[name][1]
    longest = 160
    rng = random.Random(11)
    requests = _requests(name, 4, [rng.randrange(3, longest // 2) for _ in range(10)] + [longest])
    budget = 2 * longest
    steps = H.trace_mixed(requests, random.Random(6), live=4, budget_tokens=budget, page=page)
    rep = H.Replayer(folder, dtype, page, budget, max_live=4, shuffle_seed=9)
    got = rep.run(steps)
    Z.check(folder, requests, got, dtype)
    for group in rep.cache.groups:
        assert group.pool.acquired_total > group.pool.num_pages and group.pool.pages_in_use == 0
    assert rep.cache.free_slots == 4


@pytest.mark.parametrize("name", ["P", "Q"])
def test_long_decoding_in_graphs(name):
    """Three tokens of prompt, then a hundred and more one by one (captured as CUDA graphs after the
    second step), two requests of different age side by side."""
    folder, page = Z.model_folder(name), Z.CONFIGS[name][1]
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
    Z.check(folder, requests, got, "float32", expect_all=False)


# ------------------------------------------------------------------------------ planted weights

def _planted(layer, seed, name, sink=None):
    """One layer whose scores are decided by two tokens.  Token 1's embedding lies along one direction,
    which only the queries read, strongly; token 0's along a second one, which only the keys read,
    strongly; every other token's is orthogonal to both.  A query at a token 1 finds the earlier
    tokens 0 that it may see, however far back, and next to nothing else (its own key is zero)."""
    cfg = {"architecture": "Zadurax", "vocab": 53, "width": 64, "norm": {"eps": 1e-6}, "layers": [layer]}
    t = {k: v.float() for k, v in Z.random_tensors(cfg, seed).items()}
    t["embed"][:, :2] = 0.0
    t["embed"][:2] = 0.0
    t["embed"][1, 0] = 1.0
    t["embed"][0, 1] = 1.0
    m = layer["mixer"]
    if layer["type"] == "attention":
        t["l0.mix.q"][:, 0], t["l0.mix.q"][:, 1] = 2.0, 0.0
        t["l0.mix.k"][:, 0], t["l0.mix.k"][:, 1] = 0.0, 2.0
    else:
        rank, d, r = m["kv_rank"], m["dim"], m["rot_dim"]
        t["l0.mix.dkv"][:, :2] = 0.0
        t["l0.mix.dkv"][:rank, 1] = 2.0
        key = (t["l0.mix.uk"] @ t["l0.mix.dkv.norm"]).view(m["heads"], d)        # a head's plain key for an all-ones latent
        q = t["l0.mix.q"].view(m["heads"], d + r, -1)
        q[:, :, :2] = 0.0
        q[:, :d, 0] = 0.5 * key
        if sink is not None:
            t["l0.mix.sink"][:] = sink
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    folder = H.tmp_root() / f"zadurax-planted-{name}"
    Z.register(folder, cfg, t)
    return folder, cfg


def _moved(folder, cfg, ids, other, at):
    return H.row_error(P.forward(cfg, Z._tensors[str(folder)], other)[at], Z.plain_logits(folder, ids)[at])


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_key_in_the_latent_cache_decides(dtype):
    folder, cfg = _planted(Z.latent(2, 32, 16, 16, 64, 0.25, scaling=Z.yarn(4.0, 64, 16.0, 2.0)), 21, "latent")
    rng = random.Random(2)
    filler = lambda n: [rng.randrange(2, cfg["vocab"]) for _ in range(n)]
    ids = filler(9) + [0] + filler(290) + [1] + filler(3)      # the far key is 291 positions back, pages away
    at = 300
    without = list(ids)
    without[9] = 5
    assert _moved(folder, cfg, ids, without, at) > 0.1
    requests = {"p": ids}
    got = H.Replayer(folder, dtype, 16, 304).run(H.trace_whole(requests))
    Z.check(folder, requests, got, dtype)
    got = H.Replayer(folder, dtype, 16, 304, shuffle_seed=5).run(H.trace_decode_tail(requests, 8))
    Z.check(folder, requests, got, dtype, expect_all=False)
    got = H.Replayer(folder, dtype, 16, 304, shuffle_seed=6).run(H.trace_portions(requests, random.Random(3)))
    Z.check(folder, requests, got, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_takes_its_share(dtype):
    """With a sink far above every score the output all but vanishes; with one far below it changes nothing."""
    rng = random.Random(4)
    ids = H.random_ids(rng, 40, 53)
    logits = {}
    for sink in (-30.0, 2.0, 30.0):
        folder, cfg = _planted(Z.latent(2, 32, 16, 16, 64, 0.25), 22, f"sink{sink}", sink=sink)
        logits[sink] = Z.plain_logits(folder, ids)
        got = H.Replayer(folder, dtype, 16, 48).run(H.trace_whole({"p": ids}))
        Z.check(folder, {"p": ids}, got, dtype)
    assert H.row_error(logits[2.0], logits[-30.0]) > 1e-2 and H.row_error(logits[2.0], logits[30.0]) > 1e-2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim,window", [(64, 37), (16, 16), (32, 64)])
def test_window_edges(head_dim, window, dtype):
    """A planted key just inside the window (window - 1 positions back) and just outside it (window
    back), in a prompt, in a portion that starts between the two, and for a token decoded alone."""
    folder, cfg = _planted(Z.attention(2, 1, head_dim, window, head_dim // 4, scale=0.5), 23, f"window{head_dim}")
    rng = random.Random(6)
    filler = lambda n: [rng.randrange(2, cfg["vocab"]) for _ in range(n)]
    start = 70
    ids = filler(start) + [0] + filler(window - 2) + [1, 1] + filler(5)
    inside, outside = start + window - 1, start + window
    for at in (inside, outside):
        without = list(ids)
        without[start] = 7
        moved = _moved(folder, cfg, ids, without, at)
        assert (moved > 0.05) if at == inside else (moved < 1e-9), (at, moved)
    requests = {"p": ids}
    got = H.Replayer(folder, dtype, 16, 192).run(H.trace_whole(requests))
    Z.check(folder, requests, got, dtype)
    cut = inside - 1
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": ids[:cut], "want": [cut - 1]}], "end": []},
             {"step": 1, "entries": [{"id": "p", "tokens": ids[cut: outside + 3], "want": list(range(outside + 3 - cut))}], "end": ["p"]}]
    got = H.Replayer(folder, dtype, 16, 192, shuffle_seed=3).run(steps)
    Z.check(folder, requests, got, dtype, expect_all=False)
    got = H.Replayer(folder, dtype, 16, 192, shuffle_seed=4).run(H.trace_decode_tail(requests, 9))
    Z.check(folder, requests, got, dtype, expect_all=False)
    assert {("p", inside), ("p", outside)} <= set(got)


@pytest.mark.parametrize("dtype", DTYPES)
def test_matrix_memory_keeps_the_first_token(dtype):
    """Forget gates held open (a large bias): the first token's key and value are in every later output."""
    cfg = {"architecture": "Zadurax", "vocab": 53, "width": 64, "norm": {"eps": 1e-6}, "layers": [Z.mlstm(2, 16, 24, 12.0)]}
    t = {k: v.float() for k, v in Z.random_tensors(cfg, 31).items()}
    t["l0.mix.f.b"][:] = 9.0
    t["l0.mix.i.b"][:] = -1.0
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    folder = H.tmp_root() / "zadurax-first-token"
    Z.register(folder, cfg, t)
    rng = random.Random(4)
    ids = H.random_ids(rng, 180, cfg["vocab"])
    other = [(ids[0] + 1) % cfg["vocab"]] + ids[1:]
    assert _moved(folder, cfg, ids, other, 179) > 1e-3
    got = H.Replayer(folder, dtype, 16, 192, shuffle_seed=1).run(H.trace_decode_tail({"p": ids}, 30))
    Z.check(folder, {"p": ids}, got, dtype, expect_all=False)
    got = H.Replayer(folder, dtype, 16, 192, shuffle_seed=2).run(H.trace_portions({"p": ids}, random.Random(9)))
    Z.check(folder, {"p": ids}, got, dtype)


# ----------------------------------------------------------------- the entry point and scheduler

@pytest.mark.parametrize("name", ["P", "Q"])
def test_greedy_generation_through_the_engine(name):
    from bare_cuda_4gib_b200.engine.engine import LLMEngine

    folder, page = Z.model_folder(name), Z.CONFIGS[name][1]
    cfg = Z.CONFIGS[name][0]
    rng = random.Random(13)
    prompts = [H.random_ids(rng, n, cfg["vocab"]) for n in (5, 23, 1, 40, 12, 9)]
    engine = LLMEngine(str(folder), max_tokens=96, max_seqs=4, dtype="float32", page_tokens=page, max_step_tokens=24)
    out = engine.generate_batch(prompts, 24)
    alone = engine.generate(prompts[1], 24)
    assert alone == out[1]
    for prompt, new in zip(prompts, out):
        assert len(new) == 24
        logits = Z.plain_logits(folder, prompt + new[:-1])
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
    folder = Z.model_folder("Q")
    prompt = [5, 17, 3, 60, 9, 41, 76]
    out = _tool("llm-infer", "--model", folder, "--prompt", ",".join(map(str, prompt)), "--tokens", 10, "--dtype",
                "float32", "--page-tokens", 32)
    generated = [int(t) for t in out.split("generated:")[1].split()]
    assert len(generated) == 10
    logits = Z.plain_logits(folder, prompt + generated[:-1])
    assert generated == [int(logits[len(prompt) - 1 + i].argmax()) for i in range(10)]
    assert out.splitlines()[0].startswith("[llm] 5 layers, hidden 96, vocab 77")


def test_tools_run_a_preset_with_random_weights(tmp_path):
    out = _tool("llm-infer", "--model", tmp_path / "m", "--random", "zadurax-tiny", "--prompt", "1,2,3", "--tokens", 5)
    assert len(out.split("generated:")[1].split()) == 5
    out = _tool("llm-bench", "--model", tmp_path / "m", "--random", "zadurax-tiny", "--prompt-len", 24, "--tokens", 8,
                "--runs", 2, "--warmup", 1, "--page-tokens", 16)
    assert "TTFT" in out and "TPOT" in out


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_tool(dtype, tmp_path):
    """bin/trace_run on requests that share steps; the third takes the second one's slot and pages."""
    import numpy as np

    folder = Z.model_folder("P")
    requests = _requests("P", 17, [40, 19, 33])
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
    vocab = Z.CONFIGS["P"][0]["vocab"]
    for step, rows in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), vocab).copy())
        for i, (rid, p) in enumerate(rows):
            err = H.row_error(got[i], Z.plain_logits(folder, requests[rid])[p])
            assert err <= Z.TOLERANCE[dtype], (step, rid, p, err)


# ----------------------------------------------------------------- configurations drawn at random

def _random_config(seed):
    rng = random.Random(seed)
    pick = rng.choice

    def ff():
        return pick([None, pick([24, 50, 96, 160])])

    def attention():
        kv = pick([1, 2, 3])
        dim = pick([6, 8, 16, 32, 48, 64, 128])
        return Z.attention(kv * pick([1, 2, 4]), kv, dim, pick([1, 2, 5, 16, 31, 64, 500]), pick([2, dim // 2 * 2, dim // 4 * 2 or 2]),
                           base=pick([10.0, 10000.0, 1e6]), scale=pick([0.05, dim ** -0.5, 0.4]), ff=ff())

    def latent():
        rot = pick([2, 4, 8, 16, 32])
        scaling = pick([None, Z.yarn(pick([2.0, 8.0, 40.0]), pick([16, 64, 1000]), pick([4.0, 32.0]), pick([0.5, 1.0, 2.0]))])
        return Z.latent(pick([1, 2, 3, 5, 9, 17]), pick([4, 8, 12, 32, 64]), rot, pick([4, 8, 20, 64]), pick([8, 24, 32, 50, 64, 96]),
                        pick([0.05, 0.11, 0.3]), base=pick([100.0, 30000.0]), scaling=scaling, ff=ff())

    def mlstm():
        return Z.mlstm(pick([1, 2, 3, 6]), pick([4, 8, 12, 16, 32, 40, 64]), pick([4, 8, 10, 16, 24, 64]),
                       pick([1.0, 5.0, 15.0, 40.0]), ff=ff())

    layers = [pick([attention, latent, mlstm])() for _ in range(rng.randrange(1, 4))]
    for _ in range(rng.randrange(0, 3)):
        layers.append(Z.again(layers, rng.randrange(len([l for l in layers if "weights_of" not in l]))))
    own = [l for l in layers if "weights_of" not in l]
    layers = own + [l for l in layers if "weights_of" in l]
    rng.shuffle(layers[len(own):])
    return {"architecture": "Zadurax", "vocab": pick([50, 97, 301]), "width": pick([40, 64, 72, 100, 128, 136]),
            "norm": {"eps": pick([1e-6, 1e-5])}, "layers": layers}


@pytest.mark.parametrize("seed", range(12))
def test_configurations_drawn_at_random(seed):
    cfg = _random_config(200 + seed)
    folder = H.tmp_root() / f"zadurax-random-{seed}"
    Z.register(folder, cfg, Z.random_tensors(cfg, seed))
    rng = random.Random(seed)
    requests = {"a": H.random_ids(rng, 70, cfg["vocab"]), "b": H.random_ids(rng, 33, cfg["vocab"]),
                "c": H.random_ids(rng, 9, cfg["vocab"])}
    page = rng.choice([16, 32, 64])
    steps = H.trace_mixed(requests, random.Random(seed), live=2, budget_tokens=256, page=page)
    got = H.Replayer(folder, "float32", page, 256, max_live=2, shuffle_seed=seed).run(steps)
    Z.check(folder, requests, got, "float32")
    # bfloat16: the fast kernels against the plain ones row by row, and both against the plain implementation
    fast = H.Replayer(folder, "bfloat16", page, 256, max_live=2, shuffle_seed=seed).run(steps)
    slow = H.Replayer(folder, "bfloat16", page, 256, max_live=2, shuffle_seed=seed, use_fast_gemm=False,
                      use_fast_attention=False).run(steps)
    assert sorted(fast) == sorted(slow) and len(fast) == sum(len(ids) for ids in requests.values())
    agree = sorted(H.row_error(fast[key], slow[key]) for key in fast)
    assert agree[int(0.95 * len(agree))] <= 3e-2 and agree[-1] <= 0.3, agree[-3:]
    if not any(layer["type"] == "mlstm" for layer in cfg["layers"]):      # (see zadurax_helpers.TOLERANCE)
        Z.check_most(folder, requests, fast, "bfloat16")
