"""The Ruzunex design on the GPU against its plain statement: whole models under every cutting, batches, slots and
pages used again, replayed steps, the engine's entry points, keys at the edges of windows and far away, and every
new kernel alone."""
from __future__ import annotations

import copy
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_ruzunex as pr
from helpers import cut, random_tokens, rel_err
from ruzunex_cases import CASE_P, CASE_Q, CASE_R, CASES, for_dtype, make_weights

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-4, torch.bfloat16: 5e-2}
SEEDS = {"P": 11, "Q": 12, "R": 13, "S": 14}


def assert_close(got, want, dtype):
    """float32: every row within 2e-4 of its largest value.  bfloat16: rounding is amplified where a head's output is
    nearly zero before it is brought to unit size, so the rows are judged together: their median error and the
    nineteenth of twenty."""
    if isinstance(got, (list, tuple)):                   # several requests: their rows are judged together
        got, want = torch.cat(list(got)), torch.cat(list(want))
    if dtype == torch.float32:
        assert rel_err(got, want) < TOL[dtype]
        return
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape and bool(torch.isfinite(got).all())
    err = (got - want).abs().amax(dim=1) / want.abs().amax(dim=1).clamp_min(1e-30)
    assert float(err.median()) < 2e-2, float(err.median())
    assert float(torch.quantile(err, 0.95)) < TOL[dtype], float(torch.quantile(err, 0.95))


def on_device(w, dtype):
    return {k: v.to(dtype).cuda() for k, v in w.items()}


def make_runner(case, w, dtype, n_pages=24, max_requests=3, page_size=16, use_graphs=False, shapes=None):
    from inferrs_b200.engine.loading import spec_from_config
    from inferrs_b200.engine.runner import ModelRunner
    from inferrs_b200.runtime import Runtime
    spec, _ = spec_from_config(case, tensor_shapes=shapes)
    rt = Runtime.cuda(dtype)
    return ModelRunner(spec, on_device(w, dtype), rt, page_size=page_size, n_pages=n_pages, max_requests=max_requests,
                       use_graphs=use_graphs)


def entry(rid, tokens, want=None):
    from inferrs_b200.engine.batch import StepEntry
    return StepEntry(rid, tokens, list(range(len(tokens))) if want is None else want)


def dev(v, dtype=torch.int32):
    return torch.tensor(v, dtype=dtype, device="cuda")


def act(x, dtype):
    return x.to(dtype).cuda().contiguous()


# ---------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_whole_prompt_and_every_cutting_match_the_plain_statement(name, dtype):
    case = for_dtype(CASES[name], dtype)
    w = make_weights(case, SEEDS[name])
    toks = random_tokens(75, case["vocab"], seed=3)
    want = pr.forward(case, w, toks)
    runner = make_runner(case, w, dtype)
    runner.admit("whole")
    got = runner.step([entry("whole", toks)])
    assert_close(got, want, dtype)
    runner.release("whole")
    # one token a step from an empty cache: the first tokens of a sequence, and decoding through cache and state
    runner.admit("single")
    rows = [runner.step([entry("single", [t])]) for t in toks[:60]]
    assert_close(torch.cat(rows), want[:60], dtype)
    runner.release("single")
    # portions of changing size, down to two tokens and one, another request's portions beside them
    other = random_tokens(40, case["vocab"], seed=4)
    want_other = pr.forward(case, w, other)
    runner.admit("cut")
    runner.admit("other")
    at, o_at, rows, o_rows = 0, 0, [], []
    for n in cut(len(toks), [7, 2, 30, 1, 1, 2, 17, 3]):
        entries = [entry("cut", toks[at:at + n])]
        if o_at < len(other):
            entries.insert(o_at % 2, entry("other", other[o_at:o_at + 6]))
        out = runner.step(entries)
        k = 0
        for e in entries:
            (rows if e.rid == "cut" else o_rows).append(out[k:k + len(e.tokens)])
            k += len(e.tokens)
        o_at += 6
        at += n
    assert_close(torch.cat(rows), want, dtype)
    assert_close(torch.cat(o_rows), want_other[:sum(r.shape[0] for r in o_rows)], dtype)
    runner.manager.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", list(range(16)))
def test_configurations_drawn_at_random(seed, dtype):
    """Sizes, counts, windows, constants and the order of layers drawn from a seed: a whole prompt, then the same
    prompt in portions with its last tokens one by one, in a slot and pages that the first request has used."""
    from ruzunex_cases import random_case
    case = random_case(seed)
    w = make_weights(case, 100 + seed)
    toks = random_tokens(90, case["vocab"], seed=seed)
    want = pr.forward(case, w, toks)
    runner = make_runner(case, w, dtype, n_pages=8, max_requests=1)
    runner.admit("whole")
    assert_close(runner.step([entry("whole", toks)]), want, dtype)
    runner.release("whole")
    runner.admit("cut")
    rows, at = [], 0
    for n in cut(70, [19, 2, 33, 1, 5]):
        rows.append(runner.step([entry("cut", toks[at:at + n])]))
        at += n
    for t in toks[70:]:
        rows.append(runner.step([entry("cut", [t])]))
    assert_close(torch.cat(rows), want, dtype)
    runner.manager.check_invariants()


def test_layer_sums_match_after_every_layer():
    """The sum of the streams after every layer, through the model's own blocks, in float32."""
    from inferrs_b200.engine.batch import build_context
    case, w = CASE_P, make_weights(CASE_P, 17)
    toks = random_tokens(33, case["vocab"], seed=9)
    sums = []
    pr.forward(case, w, toks, layer_sums=sums)
    runner = make_runner(case, w, torch.float32)
    runner.admit(0)
    got = runner.step([entry(0, toks)])
    assert rel_err(got, pr.forward(case, w, toks)) < TOL[torch.float32]
    # the last layer's sum is what the last norm reads: logits = norm(sum) head, so a wrong sum could not pass above;
    # here every earlier layer is looked at too, by running models cut off after it
    for upto in (1, 2, 4):
        short = dict(case, layers=case["layers"][:upto])
        ws = {k: v for k, v in w.items() if not k.startswith("l") or int(k[1:k.index(".")]) < upto}
        r = make_runner(short, ws, torch.float32)
        r.admit(0)
        want = pr.rms_norm(sums[upto - 1], w["final.norm"], case["norm"]["eps"]) @ w["head"].T
        assert rel_err(r.step([entry(0, toks)]), want) < TOL[torch.float32]


def test_a_second_norm_without_a_feed_forward():
    """Weight files that hold a second norm, connection and convolution for a layer without a feed-forward: they are
    read and do nothing."""
    case = CASE_P
    shapes = {"l2.norm2": (case["width"],)}
    w = make_weights(case, 5, bare_second=True)
    assert "l2.canon2" in w and "l2.norm2" in w and "l2.hc2.mix" in w
    toks = random_tokens(30, case["vocab"], seed=6)
    runner = make_runner(case, w, torch.float32, shapes=shapes)
    runner.admit(0)
    assert rel_err(runner.step([entry(0, toks)]), pr.forward(case, w, toks)) < TOL[torch.float32]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_unequal_requests_in_one_batch_slots_and_pages_used_again(name, dtype):
    """Two state slots and pages for two requests; five requests of unequal length take turns, decoding side by side
    with portions of the next ones.  Every request must give what it gives alone (the plain statement knows no
    batches, slots or pages)."""
    case = for_dtype(CASES[name], dtype)
    w = make_weights(case, SEEDS[name])
    lens = {"a": 50, "b": 23, "c": 64, "d": 9, "e": 37}
    toks = {k: random_tokens(n, case["vocab"], seed=ord(k)) for k, n in lens.items()}
    want = {k: pr.forward(case, w, t) for k, t in toks.items()}
    runner = make_runner(case, w, dtype, n_pages=9, max_requests=2)      # 144 cached tokens: no three requests fit
    got = {k: [] for k in lens}
    at = {k: 0 for k in lens}
    live, waiting = [], list(lens)
    sizes = [13, 1, 1, 2, 5, 1, 30, 1]
    i = 0
    while live or waiting:
        while waiting and len(live) < 2:
            k = waiting.pop(0)
            runner.admit(k)
            live.append(k)
        entries = []
        for j, k in enumerate(live):
            n = min(sizes[(i + 3 * j) % len(sizes)], lens[k] - at[k])
            entries.append(entry(k, toks[k][at[k]:at[k] + n]))
        out = runner.step(entries)
        r = 0
        for e in entries:
            got[e.rid].append(out[r:r + len(e.tokens)])
            r += len(e.tokens)
            at[e.rid] += len(e.tokens)
            if at[e.rid] == lens[e.rid]:
                runner.release(e.rid)
                live.remove(e.rid)
        i += 1
    assert_close([torch.cat(got[k]) for k in lens], [want[k] for k in lens], dtype)
    runner.manager.check_invariants()


@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_replayed_steps_give_what_plain_launches_give(name):
    """The same requests through steps captured as CUDA graphs (padding requests, the spare state slot) and through
    steps launched kernel by kernel."""
    case = for_dtype(CASES[name], torch.bfloat16)
    w = make_weights(case, SEEDS[name])
    toks = {k: random_tokens(n, case["vocab"], seed=n) for k, n in (("a", 70), ("b", 45))}
    outs = []
    for graphs in (False, True):
        runner = make_runner(case, w, torch.bfloat16, use_graphs=graphs)
        assert (runner.graphs is not None) == graphs
        runner.admit("a")
        runner.admit("b")
        rows = [runner.step([entry("a", toks["a"][:40]), entry("b", toks["b"][:33])])]
        for i in range(12):
            rows.append(runner.step([entry("a", [toks["a"][40 + i]]), entry("b", [toks["b"][33 + i]])]))
        rows.append(runner.step([entry("a", toks["a"][52:])]))
        outs.append(torch.cat(rows))
    assert_close(outs[1], outs[0], torch.bfloat16)
    want = torch.cat([pr.forward(case, w, toks["a"])[:40], pr.forward(case, w, toks["b"])[:33]])
    assert_close(outs[1][:73], want, torch.bfloat16)


def test_long_decoding_keeps_state_and_keys():
    case, w = CASE_P, make_weights(CASE_P, 21)
    toks = random_tokens(260, case["vocab"], seed=8)
    want = pr.forward(case, w, toks)
    runner = make_runner(case, w, torch.float32, n_pages=20, max_requests=1, use_graphs=True)
    runner.admit(0)
    rows = [runner.step([entry(0, toks[:5])])]
    for t in toks[5:]:
        rows.append(runner.step([entry(0, [t])]))
    assert rel_err(torch.cat(rows), want) < TOL[torch.float32]
    # the early tokens matter to the last logits: without them the states and the far keys are other ones
    late = pr.forward(case, w, toks[100:])
    assert rel_err(late[-1], want[-1]) > 1e-3


# ---------------------------------------------------------------------------------------------------
# through the engine's own entry points
# ---------------------------------------------------------------------------------------------------
def write_folder(path, case, w):
    from inferrs_b200.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(case, f)
    write_safetensors(os.path.join(path, "model.safetensors"), [(k, v.to(torch.bfloat16)) for k, v in w.items()])
    return path


def test_greedy_generation_through_the_engine(tmp_path):
    """More requests than slots and few pages: the scheduler admits, cuts prompts into portions, preempts and computes
    again; every request gets the tokens that the plain statement picks."""
    from inferrs_b200.engine.engine import Engine
    from inferrs_b200.sampling.params import SamplingParams
    case, w = CASE_P, make_weights(CASE_P, 31)
    folder = write_folder(str(tmp_path / "m"), case, w)
    eng = Engine(model_dir=folder, dtype="f32", block_size=16, num_blocks=8, max_batch_size=2, max_tokens_per_step=24)
    prompts = [random_tokens(n, case["vocab"], seed=60 + n) for n in (33, 5, 40, 18)]
    n_new = 14
    want = [pr.greedy(case, w, p, n_new) for p in prompts]
    got = eng.generate(prompts, SamplingParams.greedy(max_tokens=n_new))
    eng.runner.manager.check_invariants()
    assert got == want
    assert eng.generate(prompts[:2], SamplingParams.greedy(max_tokens=n_new)) == want[:2]    # slots used before


def test_command_line_with_random_weights_and_with_a_folder(tmp_path, capsys):
    from inferrs_b200 import cli
    path = str(tmp_path / "config.json")
    with open(path, "w") as f:
        json.dump(dict(CASE_P, eos_token_id=5), f)
    common = [path, "--random-weights", "4", "--max-blocks", "32", "--max-batch-size", "2", "--max-tokens", "7",
              "--ignore-eos", "--seed", "3", "--prefill-chunk", "16", "--random-prompt", "45"]
    outs = []
    for _ in range(2):
        assert cli.main(["run"] + common + ["--temperature", "0.8", "--top-k", "20", "--dtype", "bf16"]) == 0
        cap = capsys.readouterr()
        outs.append([int(t) for t in cap.out.split()])
        assert "45 prompt tokens, 7 generated" in cap.err
    assert outs[0] == outs[1] and len(outs[0]) == 7 and all(0 <= t < CASE_P["vocab"] for t in outs[0])
    folder = write_folder(str(tmp_path / "m"), CASE_Q, make_weights(CASE_Q, 5))
    assert cli.main(["bench", folder, "--prompt-len", "30", "--max-tokens", "6", "--runs", "2", "--warmup", "1",
                     "--max-blocks", "32", "--max-batch-size", "2", "--temperature", "0"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["prompt_len"] == 30 and out["prefill_tok_s"] > 0 and out["decode_tok_s"] > 0


def test_trace_replay_of_a_folder(tmp_path):
    """Four requests at most are live, a later one takes the slot and the pages of one that ended."""
    case, w = CASE_P, make_weights(CASE_P, 41)
    folder = write_folder(str(tmp_path / "m"), case, w)
    toks = {k: random_tokens(n, case["vocab"], seed=n) for k, n in (("a", 70), ("b", 21), ("c", 30))}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks["a"][:50], "want": [0, 49]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks["a"][50:51], "want": [0]},
                                     {"id": "b", "tokens": toks["b"][:19], "want": [18]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": toks["b"][19:], "want": [0, 1]},
                                     {"id": "a", "tokens": toks["a"][51:], "want": [18]}], "end": ["a", "b"]},
             {"step": 3, "entries": [{"id": "c", "tokens": toks["c"][:28], "want": []}], "end": []},
             {"step": 4, "entries": [{"id": "c", "tokens": toks["c"][28:], "want": [0, 1]}], "end": ["c"]}]
    out_dir = str(tmp_path / "out")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", out_dir, "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-800:]
    assert p.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3", "done", "4"]
    wa, wb, wc = (pr.forward(case, w, toks[k]) for k in "abc")
    read = lambda s: torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{s}.f32"), dtype="<f4").reshape(-1, case["vocab"]).copy())
    assert rel_err(read(0), wa[[0, 49]]) < 2e-4
    assert rel_err(read(1), torch.stack([wa[50], wb[18]])) < 2e-4
    assert rel_err(read(2), torch.stack([wb[19], wb[20], wa[69]])) < 2e-4
    assert not os.path.exists(os.path.join(out_dir, "3.f32"))
    assert rel_err(read(4), wc[[28, 29]]) < 2e-4


# ---------------------------------------------------------------------------------------------------
# keys at the edges of windows and far away, in the model: weights under which one token's value stands out
# ---------------------------------------------------------------------------------------------------
W64 = 64


def story_model(layer):
    return {"architecture": "Ruzunex", "vocab": W64, "width": W64, "norm": {"eps": 1e-5}, "streams": 1,
            "canon": {"taps": 1}, "layers": [layer]}


def story_weights(case, seed):
    """Weights under which a token's id is its key: the embedding is the identity times 8, the norms' weights are
    one, the convolution in front of the sub-layer adds nothing, the one stream is read, kept and written as it is,
    the head reads the stream as it is."""
    w = make_weights(case, seed)
    w["embed"] = torch.eye(W64) * 8.0
    w["l0.norm1"], w["final.norm"] = torch.ones(W64), torch.ones(W64)
    w["l0.canon1"] = torch.zeros(W64, 1)
    w["l0.hc1.in"], w["l0.hc1.out"], w["l0.hc1.mix"] = torch.ones(1), torch.ones(1), torch.ones(1, 1)
    w["head"] = torch.eye(W64)
    return w


def ask_and_pick(dim):
    """Key: the first ``dim`` channels of the normed row (a token's id, if below ``dim``, stands out).  Query: the
    same, but token 7 asks for token 9."""
    pick = torch.zeros(dim, W64)
    pick[:min(dim, W64)] = torch.eye(W64)[:min(dim, W64)]
    ask = pick.clone()
    ask[7, 7], ask[9, 7] = 0.0, 1.0
    return ask, pick


def mark_value(dim, gain):
    """Only token 9 has a value (channel 9 minus channel 10, which no token owns)."""
    v = torch.zeros(dim, W64)
    v[0, 9], v[0, 10] = gain, -gain
    return v


def run_whole_and_cut(case, w, dtype, toks, portions, single_from, single_to, max_requests=2):
    """The logits of the whole prompt in one step, and of the same prompt in portions with the tokens
    single_from..single_to decoded one by one (a request after the whole one, in a slot and pages that it used)."""
    runner = make_runner(case, w, dtype, n_pages=60, max_requests=max_requests)
    runner.admit("w")
    got = runner.step([entry("w", toks)])
    runner.release("w")
    runner.admit("c")
    rows, at = [], 0
    for k in cut(single_from, portions):
        rows.append(runner.step([entry("c", toks[at:at + k])]))
        at += k
    for t in toks[single_from:single_to]:
        rows.append(runner.step([entry("c", [t])]))
    if single_to < len(toks):
        rows.append(runner.step([entry("c", toks[single_to:])]))
    return got, torch.cat(rows)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,marked_at,dim,vdim", [(37, 200, 32, 16), (48, 208, 64, 64), (5, 203, 128, 128),
                                                      (64, 192, 64, 24), (1, 150, 16, 16)])
def test_a_marked_token_is_seen_inside_the_window_and_not_beyond(window, marked_at, dim, vdim, dtype):
    """Token 9 stands once in a prompt of other tokens; token 7 asks for it at every distance around the window's
    edge, in a whole prompt, in portions and decoded one by one.  Its value reaches the logits while it is inside the
    window (itself and window - 1 tokens before the asking one) and not one token later."""
    layer = {"type": "attention", "mlp": None,
             "mixer": {"heads": 2, "kv_heads": 1, "dim": dim, "vdim": vdim, "scale": 1.0, "mask": {"size": window}}}
    case = story_model(layer)
    w = story_weights(case, 7)
    ask, pick = ask_and_pick(dim)
    w["l0.mix.q"] = torch.cat([ask, ask]) * 1.0
    w["l0.mix.k"] = pick
    w["l0.mix.q.norm"], w["l0.mix.k.norm"] = torch.ones(dim) * 6.0, torch.ones(dim)
    w["l0.mix.v"] = mark_value(vdim, 1.0)
    w["l0.mix.g"] = torch.zeros(2 * vdim, W64)                        # sigmoid(0): the gate halves every head
    o = torch.zeros(W64, 2 * vdim)
    o[60, 0], o[61, vdim] = 4.0, 4.0                                  # head 0's value to channel 60, head 1's to 61
    w["l0.mix.o"] = o
    n = marked_at + window + 12
    toks = [(11 + 3 * i) % 40 + 12 for i in range(n)]                 # tokens 12..51: never 7 or 9
    toks[marked_at] = 9
    asks = list(range(marked_at + max(window - 4, 1), marked_at + window + 3))
    for a in asks:
        toks[a] = 7
    want = pr.forward(case, w, toks)
    seen = want[:, 60] - want[:, 62]                                  # channel 62: what the norm makes of an empty row
    for a in asks:
        inside = a - marked_at < window
        assert (float(seen[a].abs()) > 0.05) == inside, (a, float(seen[a]))
    got, got_cut = run_whole_and_cut(case, w, dtype, toks, [50, 7, 2, 64, 3], marked_at + max(window - 2, 1), n - 2)
    tol = 2e-4 if dtype == torch.float32 else 3e-2
    assert rel_err(got, want) < tol and rel_err(got_cut, want) < tol


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,marked_at", [(64, 15), (32, 16), (128, 255)])
def test_a_marked_token_far_back_is_found_among_hundreds_and_the_sink_takes_its_share(dim, marked_at, dtype):
    """The left half of a parallel layer: every earlier key is visible, so a marked token hundreds of positions back,
    just before and just after a page's border, is found by the token that asks for it; a sink as large as the
    asking score halves what it gets."""
    left = {"heads": 2, "kv_heads": 1, "dim": dim, "vdim": dim, "scale": 1.0, "conv": 1}
    layer = {"type": "parallel", "mlp": None,
             "mixer": {"left": left, "right": {"heads": 1, "dim": 8, "vdim": 8}, "left_scale": 1.0, "right_scale": 0.0}}
    case = story_model(layer)
    w = story_weights(case, 8)
    ask, pick = ask_and_pick(dim)
    p = "l0.mix.left"
    w[f"{p}.q"], w[f"{p}.k"], w[f"{p}.v"] = torch.cat([ask, ask]), pick, mark_value(dim, 1.0)
    for name, size in (("q", 2 * dim), ("k", dim), ("v", dim)):
        w[f"{p}.{name}.conv"] = torch.ones(size, 1)
    # the whole projections are brought to unit size: one number of sqrt(dim) per head; the weights make the asking
    # score 12, large among hundreds of keys and small enough that float32 rounding does not move its exponential
    w[f"{p}.q.norm"], w[f"{p}.k.norm"] = torch.ones(2 * dim) * 4.0 / dim ** 0.5, torch.ones(dim) * 3.0 / dim ** 0.5
    w[f"{p}.temp"] = torch.tensor([1.0, 1.0])
    o = torch.zeros(W64, 2 * dim)
    o[60, 0], o[61, dim] = 4.0, 4.0
    w[f"{p}.o"] = o
    n = 400
    toks = [(11 + 3 * i) % 40 + 12 for i in range(n)]
    toks[marked_at] = 9
    for a in (marked_at + 1, 300, 399):
        toks[a] = 7
    # the asking score: q . k of the two unit-rms rows times their weights
    qn = pr.rms_norm(torch.eye(W64)[7:8] @ w[f"{p}.q"].T, w[f"{p}.q.norm"], 1e-5)[0, :dim]
    kn = pr.rms_norm(torch.eye(W64)[9:10] @ w[f"{p}.k"].T, w[f"{p}.k.norm"], 1e-5)[0]
    score = float(qn @ kn)
    assert score > 8.0                                               # it stands out among hundreds of keys
    w[f"{p}.sink"] = torch.tensor([-30.0, score])                    # head 1's sink weighs as much as the marked key
    want = pr.forward(case, w, toks)
    h0, h1 = want[:, 60] - want[:, 62], want[:, 61] - want[:, 62]
    for a in (marked_at + 1, 300, 399):
        assert float(h0[a]) > 0.5 and 0.35 < float(h1[a] / h0[a]) < 0.65, (a, float(h0[a]), float(h1[a]))
    got, got_cut = run_whole_and_cut(case, w, dtype, toks, [50, 7, 2, 64, 3], 290, 310)
    tol = 2e-4 if dtype == torch.float32 else 3e-2
    assert rel_err(got, want) < tol and rel_err(got_cut, want) < tol


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_marked_token_far_back_is_kept_by_the_state(dtype):
    """The right half of a parallel layer alone, with a forget gate that forgets nothing on one channel: what a token
    wrote three hundred positions back is still read."""
    layer = {"type": "parallel", "mlp": None,
             "mixer": {"left": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 1.0, "conv": 1},
                       "right": {"heads": 2, "dim": 16, "vdim": 24}, "left_scale": 0.0, "right_scale": 1.0}}
    case = story_model(layer)
    w = story_weights(case, 9)
    p = "l0.mix.right"
    # the gate opens for token 9 on channel 0 of head 0 (f falls to its lower bound, so the value is written) and
    # stays shut for every other token (f = 1 up to rounding: nothing is written, nothing forgotten)
    f = torch.zeros(32, W64)
    f[:, :] = 0.0
    f[0, 9] = -8.0
    w[f"{p}.f"] = f
    w[f"{p}.f.b"] = torch.full((32,), 30.0)
    w[f"{p}.lower"] = torch.full((32,), 0.25)
    q = torch.zeros(32, W64)
    q[0, 7] = 2.0                                                    # token 7 reads channel 0
    w[f"{p}.q"] = q
    w[f"{p}.v"] = torch.cat([mark_value(24, 1.0), torch.zeros(24, W64)])
    w[f"{p}.norm"] = torch.ones(24)
    o = torch.zeros(W64, 48)
    o[60, 0] = 1.0
    w[f"{p}.o"] = o
    n = 330
    toks = [(11 + 3 * i) % 40 + 12 for i in range(n)]
    toks[5], toks[320] = 9, 7
    want = pr.forward(case, w, toks)
    assert float((want[320, 60] - want[320, 62]).abs()) > 0.3
    assert float((want[319, 60] - want[319, 62]).abs()) < 1e-3
    got, got_cut = run_whole_and_cut(case, w, dtype, toks, [50, 7, 2, 64, 3], 310, 325)
    tol = 2e-4 if dtype == torch.float32 else 3e-2
    assert rel_err(got, want) < tol and rel_err(got_cut, want) < tol


# ---------------------------------------------------------------------------------------------------
# the new kernels alone
# ---------------------------------------------------------------------------------------------------
def requests_of(lens):
    q_start = [0]
    for n in lens:
        q_start.append(q_start[-1] + n)
    row_request = [r for r, n in enumerate(lens) for _ in range(n)]
    return q_start, row_request


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,C,add", [(4, 50, True), (1, 8, True), (2, 130, False), (5, 300, True), (4, 256, True),
                                        (3, 1024, False)])
def test_convolution_on_rows_with_its_state(taps, C, add, dtype):
    """Three requests in two steps (portions of 5, 1 and 2 rows after 7, 3 and 1): the second step reads what the
    state keeps of the first; a request shorter than the reach keeps the youngest of what it held."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(taps * 100 + C)
    first, second = [7, 3, 1], [5, 1, 2]
    x = [torch.randn(a + b, C, generator=g).to(torch.bfloat16).float() for a, b in zip(first, second)]
    wt = torch.randn(C, taps, generator=g)
    want = [pr.causal_conv(t, wt) + (t if add else 0.0) for t in x]
    state = torch.zeros(4, 3 + max(taps - 1, 0) * C, device="cuda")
    slots = dev([2, 0, 3])
    got = [[], [], []]
    for step, lens in enumerate((first, second)):
        q_start, row_request = requests_of(lens)
        rows = torch.cat([t[:first[r]] if step == 0 else t[first[r]:] for r, t in enumerate(x)])
        lead = 8 if C % 8 == 0 else 3                               # sixteen bytes at a time where the sizes allow
        pad = torch.randn(rows.shape[0], lead, generator=g)
        wide = act(torch.cat([pad, rows], dim=1), dtype)            # the rows as a slice of a wider tensor
        out = torch.empty(rows.shape[0], C, dtype=dtype, device="cuda")
        kernels.causal_conv_rows(wide, lead, wt.t().contiguous().cuda(), state if taps > 1 else None, 3, dev(q_start),
                                 slots, dev(row_request), out, add)
        kernels.conv_state_shift(wide, lead, C, taps, state, 3, dev(q_start), slots, 3)
        for r in range(3):
            got[r].append(out[q_start[r]:q_start[r + 1]].float().cpu())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for r in range(3):
        assert rel_err(torch.cat(got[r]), want[r]) < tol


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,E,taps,rot,mode", [(6, 2, 24, 20, 3, 12, 2), (1, 1, 16, 64, 1, 0, 2), (4, 4, 16, 40, 2, 16, 2),
                                                  (3, 1, 10, 7, 5, 6, 1), (8, 2, 128, 128, 4, 64, 2), (2, 2, 8, 8, 0, 4, 0),
                                                  (2, 1, 16, 8, 3, 8, 2), (3, 1, 10, 6, 4, 4, 1)])
def test_convolution_norm_rotation_and_store(H, G, D, E, taps, rot, mode, dtype):
    """One pass over q | k | v of two requests in two steps against the plain functions: the convolution (with its
    state), the norm over the whole projection (or per head, or none), the partial rotation, q dense, k and v in
    their pages at the rows' positions."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(H * 1000 + D)
    # the last two cases: more than a thousand rows in a step, where a block takes several rows one after the other
    first, second = ([1100, 30], [10, 1]) if (D, E) in ((16, 8), (10, 6)) else ([21, 3], [14, 1])
    Cq, Ck, Cv = H * D, G * D, G * E
    C = Cq + Ck + Cv
    x = [torch.randn(a + b, C + 5, generator=g).to(torch.bfloat16).float() for a, b in zip(first, second)]
    conv = torch.randn(C, max(taps, 1), generator=g) * 0.5
    wq = 1.0 + 0.2 * torch.randn(Cq if mode == 2 else D, generator=g)
    wk = 1.0 + 0.2 * torch.randn(Ck if mode == 2 else D, generator=g)
    eps, base = 1e-5, 300.0
    want_q, want_k, want_v = [], [], []
    for t in x:
        y = pr.causal_conv(t[:, :C], conv) if taps else t[:, :C]
        q, k, v = y[:, :Cq], y[:, Cq:Cq + Ck], y[:, Cq + Ck:]
        n = t.shape[0]
        if mode == 2:
            q, k = pr.rms_norm(q, wq, eps).view(n, H, D), pr.rms_norm(k, wk, eps).view(n, G, D)
        elif mode == 1:
            q, k = pr.rms_norm(q.view(n, H, D), wq, eps), pr.rms_norm(k.view(n, G, D), wk, eps)
        else:
            q, k = q.reshape(n, H, D), k.reshape(n, G, D)
        if rot:
            q, k = pr.rotate_half(q, torch.arange(n), rot, base), pr.rotate_half(k, torch.arange(n), rot, base)
        want_q.append(q)
        want_k.append(k)
        want_v.append(v.reshape(n, G, E))
    page_size = 16
    need = [(a + b + page_size - 1) // page_size for a, b in zip(first, second)]
    n_pages = sum(need) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    pages = [order[:need[0]], order[need[0]:need[0] + need[1]]]
    k_pages = torch.full((n_pages, G, page_size, D), float("nan"), dtype=dtype, device="cuda")
    v_pages = torch.full((n_pages, G, page_size, E), float("nan"), dtype=dtype, device="cuda")
    table = dev([p + [-1] * (max(need) + 1 - len(p)) for p in pages])
    half = rot // 2
    ang = torch.arange(max(64, sum(first) + sum(second)), dtype=torch.float32)[:, None] * (base ** (-2.0 * torch.arange(max(half, 1), dtype=torch.float64) / max(rot, 1))).float()[None, :]
    cos, sin = torch.cos(ang).cuda().contiguous(), torch.sin(ang).cuda().contiguous()
    state = torch.zeros(3, max(taps - 1, 0) * C + 1, device="cuda")
    slots = dev([1, 0])
    got_q = [[], []]
    for step, lens in enumerate((first, second)):
        q_start, row_request = requests_of(lens)
        rows = act(torch.cat([t[:first[r]] if step == 0 else t[first[r]:] for r, t in enumerate(x)]), dtype)
        positions = [p for r in range(2) for p in (range(first[r]) if step == 0 else range(first[r], first[r] + second[r]))]
        q_out = torch.empty(rows.shape[0], H, D, dtype=dtype, device="cuda")
        kernels.conv_norm_rope_store(rows, H, G, D, conv.t().cuda().contiguous() if taps else None,
                                     state if taps > 1 else None, 0, dev(q_start), slots, dev(row_request), mode,
                                     act(wq, dtype) if mode else None, act(wk, dtype) if mode else None, eps,
                                     cos if rot else None, sin if rot else None, rot, dev(positions), table, k_pages,
                                     v_pages, q_out)
        if taps > 1:
            kernels.conv_state_shift(rows, 0, C, taps, state, 0, dev(q_start), slots, 2)
        for r in range(2):
            got_q[r].append(q_out[q_start[r]:q_start[r + 1]].float().cpu())
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for r in range(2):
        wq_r = want_q[r] if dtype == torch.float32 else want_q[r]
        assert rel_err(torch.cat(got_q[r]).flatten(1), wq_r.flatten(1)) < tol
        n = first[r] + second[r]
        gk = torch.stack([k_pages[pages[r][p // page_size], :, p % page_size].float().cpu() for p in range(n)])
        gv = torch.stack([v_pages[pages[r][p // page_size], :, p % page_size].float().cpu() for p in range(n)])
        assert rel_err(gk.flatten(1), want_k[r].flatten(1)) < tol and rel_err(gv.flatten(1), want_v[r].flatten(1)) < tol
        # behind the request's last value its page holds zeros, not what an earlier owner left
        last = n - 1
        tail = v_pages[pages[r][last // page_size], :, last % page_size + 1:]
        assert bool((tail == 0).all())


@pytest.mark.parametrize("taps,C", [(4, 50), (2, 130), (3, 8)])
def test_steps_of_single_rows_move_the_kept_inputs_themselves(taps, C):
    """After a portion (with the kernel that moves the kept inputs), single rows with ``shift_single``: the
    convolution of every row is what the whole sequence gives."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(taps + C)
    x = [torch.randn(9, C, generator=g), torch.randn(7, C, generator=g)]
    wt = torch.randn(C, taps, generator=g)
    want = [pr.causal_conv(t, wt) for t in x]
    state = torch.zeros(3, (taps - 1) * C, device="cuda")
    slots = dev([2, 0])
    first = [2, 1]
    q_start, row_request = requests_of(first)
    rows = torch.cat([t[:n] for t, n in zip(x, first)]).cuda()
    out = torch.empty(3, C, device="cuda")
    kernels.causal_conv_rows(rows, 0, wt.t().contiguous().cuda(), state, 0, dev(q_start), slots, dev(row_request), out, False)
    kernels.conv_state_shift(rows, 0, C, taps, state, 0, dev(q_start), slots, 2)
    got = [[out[:2].cpu()], [out[2:].cpu()]]
    for i in range(6):
        rows = torch.stack([x[0][2 + i], x[1][1 + i]]).cuda()
        out = torch.empty(2, C, device="cuda")
        kernels.causal_conv_rows(rows, 0, wt.t().contiguous().cuda(), state, 0, dev([0, 1, 2]), slots, dev([0, 1]), out, False,
                                 shift_single=True)
        got[0].append(out[:1].cpu())
        got[1].append(out[1:].cpu())
    assert rel_err(torch.cat(got[0]), want[0][:8]) < 1e-5 and rel_err(torch.cat(got[1]), want[1][:7]) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_blend_of_columns(dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(3)
    x, other = torch.randn(37, 50, generator=g), torch.randn(37, 29, generator=g)
    xd, od = act(x, dtype), act(other, dtype)
    wide = torch.cat([od, od], dim=1)[:, 29:]                         # a view with a row stride of its own
    kernels.blend_columns(xd, 11, wide, torch.tensor([0.3], device="cuda"))
    want = xd.float().cpu() if False else act(x, dtype).float().cpu()
    want[:, 11:40] = 0.7 * want[:, 11:40] + 0.3 * od.float().cpu()
    assert rel_err(xd.float(), want) < (1e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,E", [(3, 20, 12), (1, 128, 64), (2, 36, 20), (2, 250, 33), (4, 32, 64), (1, 16, 130)])
def test_forget_write_scan_against_the_rule(H, D, E, dtype):
    """Prompt portions, single tokens and a request that comes back, against the rule walked token by token."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(H * 100 + D)
    lens = [40, 1, 19]
    steps = ([23, 1, 2], [17, 0, 16], [0, 0, 1])
    hd = H * D
    proj = [torch.randn(n, hd + H * E + 3, generator=g).to(torch.bfloat16).float() for n in lens]
    z = [torch.randn(n, hd, generator=g) * 2 for n in lens]
    bias, low = torch.randn(hd, generator=g), torch.sigmoid(torch.randn(hd, generator=g))
    want = []
    for r, n in enumerate(lens):
        q = pr.silu(proj[r][:, 3:3 + hd]).view(n, H, D)
        v = proj[r][:, 3 + hd:].reshape(n, H, E)
        f = (low + (1 - low) * torch.sigmoid(z[r] + bias)).view(n, H, D)
        want.append(pr.forget_write_rule(q, f, v))
    state = torch.zeros(4, hd * E, device="cuda")
    got = [[] for _ in lens]
    at = [0, 0, 0]
    for step in steps:
        live = [r for r, n in enumerate(step) if n > 0]
        q_start, _ = requests_of([step[r] for r in live])
        rows = torch.cat([proj[r][at[r]:at[r] + step[r]] for r in live])
        zz = torch.cat([z[r][at[r]:at[r] + step[r]] for r in live]).cuda().contiguous()
        out = torch.empty(rows.shape[0], H, E, device="cuda")
        kernels.linear_scan(kernels.SCAN_FORGET_WRITE, act(rows, dtype), 3, 3, 3 + hd, zz,
                            torch.cat([bias, low]).cuda(), 1.0, 1.0, state, dev(q_start), dev([[3, 0, 1][r] for r in live]),
                            len(live), out, D, max_rows=max(step))
        for i, r in enumerate(live):
            got[r].append(out[q_start[i]:q_start[i + 1]].cpu())
            at[r] += step[r]
    for r in range(3):
        assert rel_err(torch.cat(got[r]).flatten(1), want[r].flatten(1)) < 2e-5


def paged(keys, values, page_size, dtype, seed):
    """Keys [T, G, D] and values [T, G, E] of one request scattered over pages in a shuffled order; pages of no
    request hold NaN."""
    T, G, D = keys.shape
    E = values.shape[2]
    n = (T + page_size - 1) // page_size
    order = torch.randperm(n + 3, generator=torch.Generator().manual_seed(seed))[:n].tolist()
    k_pages = torch.full((n + 3, G, page_size, D), float("nan"))
    v_pages = torch.full((n + 3, G, page_size, E), float("nan"))
    for p in range(T):
        k_pages[order[p // page_size], :, p % page_size] = keys[p]
        v_pages[order[p // page_size], :, p % page_size] = values[p]
    tail = T % page_size
    if tail:
        v_pages[order[-1], :, tail:] = 0.0
    return act(k_pages, dtype), act(v_pages, dtype), dev([order])


def plain_scored_attention(q, k, v, positions, scale, window, temp, slopes, sink):
    n, H, D = q.shape
    T, G = k.shape[0], k.shape[1]
    dist = positions[:, None] - torch.arange(T)[None, :]
    see = (dist >= 0) & ((dist < window) if window else True)
    out = torch.zeros(n, H, v.shape[2])
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].T) * scale
        if temp is not None:
            s = s * temp[h]
        if slopes is not None:
            s = s - slopes[h] * dist.clamp(min=0)
        s = s.masked_fill(~see, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h])
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True) + (torch.exp(sink[h] - m) if sink is not None else 0.0)
        out[:, h] = (e / den) @ v[:, h // (H // G)]
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,E,window,opts", [(6, 2, 24, 20, 23, "ts"), (4, 4, 16, 40, 50, "b"), (1, 1, 32, 16, 1, "tbs"),
                                                 (8, 2, 64, 64, None, "tbs"), (3, 3, 10, 7, 7, "s"), (4, 1, 128, 128, 100, "b"),
                                                 (6, 3, 64, 64, 70, "")])
def test_attention_with_a_factor_a_slope_and_a_sink_per_head(H, G, D, E, window, opts, dtype):
    """The dispatching entry (the float32 kernel, or the tensor-core kernel where it takes the sizes) with every
    choice of the three options: a whole prompt, then the last rows as single tokens."""
    from types import SimpleNamespace
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(H * 100 + D)
    T = 150
    q = torch.randn(T, H, D, generator=g).to(torch.bfloat16).float()
    k = torch.randn(T, G, D, generator=g).to(torch.bfloat16).float()
    v = torch.randn(T, G, E, generator=g).to(torch.bfloat16).float()
    temp = (1.0 + 0.3 * torch.randn(H, generator=g)) if "t" in opts else None
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]) if "b" in opts else None
    sink = 2.0 * torch.randn(H, generator=g) if "s" in opts else None
    scale = 1.0 / math.sqrt(D)
    want = plain_scored_attention(q, k, v, torch.arange(T), scale, window, temp, slopes, sink).flatten(1)
    k_pages, v_pages, table = paged(k, v, 16, dtype, 5)
    f = lambda t: None if t is None else t.float().cuda().contiguous()      # noqa: E731
    span = kernels.span_argument(window)
    tol = 2e-5 if dtype == torch.float32 else 2e-2

    def ctx_for(rows, start):
        c = SimpleNamespace(row_request=dev([0] * rows), positions=dev(list(range(start, start + rows))),
                            q_start=dev([0, rows]), n_requests=1, n_rows=rows, max_kv_len=start + rows,
                            decode_only=rows == 1, extra={}, q_lens=[rows], kv_lens=[start + rows],
                            token_ids=dev([0] * rows))
        from inferrs_b200.engine.batch import StepContext
        c.attention_tiles = lambda tokens, portions_only=False: StepContext.attention_tiles(c, tokens, portions_only)
        return c

    out = torch.empty(T, H * E, dtype=dtype, device="cuda")
    kernels.paged_attention(act(q, dtype), k_pages, v_pages, table, ctx_for(T, 0), scale, span, out,
                            head_scale=f(temp), slopes=f(slopes), sinks=f(sink))
    assert rel_err(out.float(), want) < tol
    for p in (0, 1, 15, 16, 17, 99, 149):
        one = torch.empty(1, H * E, dtype=dtype, device="cuda")
        kernels.paged_attention(act(q[p:p + 1], dtype), k_pages, v_pages, table, ctx_for(1, p), scale, span, one,
                                head_scale=f(temp), slopes=f(slopes), sinks=f(sink))
        assert rel_err(one.float(), want[p:p + 1]) < tol, p


@pytest.mark.parametrize("splits", [1, 2, 5])
@pytest.mark.parametrize("H,G,D,window", [(8, 2, 128, 100), (4, 4, 64, None), (6, 1, 64, 37), (3, 3, 256, None)])
def test_tensor_core_decode_form_cut_into_slices_adds_the_sink_once(H, G, D, window, splits):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(H * 10 + splits)
    T = 700
    k = torch.randn(T, G, D, generator=g).to(torch.bfloat16).float()
    v = torch.randn(T, G, D, generator=g).to(torch.bfloat16).float()
    q = torch.randn(1, H, D, generator=g).to(torch.bfloat16).float()
    temp, sink = 1.0 + 0.3 * torch.randn(H, generator=g), 3.0 + torch.randn(H, generator=g)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)])
    scale = 1.0 / math.sqrt(D)
    want = plain_scored_attention(q, k, v, torch.tensor([T - 1]), scale, window, temp, slopes, sink).flatten(1)
    k_pages, v_pages, table = paged(k, v, 16, torch.bfloat16, 6)
    out = torch.empty(1, H * D, dtype=torch.bfloat16, device="cuda")
    kernels.paged_attention_mma(act(q, torch.bfloat16), k_pages, v_pages, table, dev([0]), dev([0, 1]), 1, dev([0, 1]),
                                dev([T - 1]), scale, window, out, True, splits, head_scale=temp.cuda(),
                                slopes=slopes.cuda(), sinks=sink.cuda())
    assert rel_err(out.float(), want) < 2e-2


@pytest.mark.parametrize("H,G,window,opts,start", [(8, 2, 100, "tbs", 0), (4, 4, None, "ts", 0), (6, 1, 37, "b", 0),
                                                   (3, 3, None, "s", 0), (16, 2, 300, "tbs", 0), (8, 2, 129, "tb", 333),
                                                   (5, 5, None, "tbs", 77)])
def test_tcgen05_prefill_form_with_a_factor_a_slope_and_a_sink_per_head(H, G, window, opts, start):
    """The tcgen05 kernel's per-head form alone, head size 128: a prompt from position 0, and a portion behind keys
    that earlier steps left (tiles of the request's later rows; a negative factor among the heads)."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(H * 10 + G)
    D, n = 128, 333
    T = start + n
    q = torch.randn(n, H, D, generator=g).to(torch.bfloat16).float()
    k = torch.randn(T, G, D, generator=g).to(torch.bfloat16).float()
    v = torch.randn(T, G, D, generator=g).to(torch.bfloat16).float()
    temp = (1.0 + 0.3 * torch.randn(H, generator=g)) if "t" in opts else None
    if temp is not None:
        temp[0] = -0.7
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]) if "b" in opts else None
    sink = 2.0 * torch.randn(H, generator=g) if "s" in opts else None
    scale = 1.0 / math.sqrt(D)
    want = plain_scored_attention(q, k, v, torch.arange(start, T), scale, window, temp, slopes, sink).flatten(1)
    k_pages, v_pages, table = paged(k, v, 16, torch.bfloat16, 7)
    tpt = kernels.TC_ROWS // (H // G)
    row0 = list(range(0, n, tpt))
    out = torch.empty(n, H * D, dtype=torch.bfloat16, device="cuda")
    f = lambda t: None if t is None else t.float().cuda().contiguous()      # noqa: E731
    kernels.paged_attention_tcgen05(act(q, torch.bfloat16), k_pages, v_pages, table, dev([0] * len(row0)), dev(row0),
                                    len(row0), dev([0, n]), dev(list(range(start, T))), scale, window, out,
                                    head_scale=f(temp), slopes=f(slopes), sinks=f(sink))
    assert kernels.attention_tcgen05_error() == 0
    assert rel_err(out.float(), want) < 2e-2


@pytest.mark.parametrize("experts,top", [(8, 3), (5, 2), (3, 3), (70, 6), (4, 1), (1, 1)])
def test_router_by_shares_of_the_softmax_over_all(experts, top):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(experts)
    z = torch.randn(33, experts + 2, generator=g) * 2
    z[3, :2] = z[3, 2]                                                # equal scores: the lower index
    idx, wt = pr.route(z[:, :experts], top)
    want = torch.zeros(33, experts).scatter(1, idx, wt)
    got = torch.empty(33, experts, device="cuda")
    kernels.router_topk(z.cuda(), None, experts, top, False, got, torch.float32, mode=kernels.ROUTE_SOFTMAX_SHARE)
    assert rel_err(got, want) < 1e-5 and bool(((got > 0).sum(1) == top).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inner", [24, 50, 1024])
def test_gelu_gate_and_clamped_routed_gate(inner, dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(inner)
    gu = (torch.randn(19, 2 * inner, generator=g) * 2).to(torch.bfloat16).float()
    out = torch.empty(19, inner, dtype=dtype, device="cuda")
    kernels.clamped_gate(act(gu, dtype), out, 0.0, 0.0, activation=kernels.GATE_ACT_GELU_TANH)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert rel_err(out.float(), pr.gelu_tanh(gu[:, :inner]) * gu[:, inner:]) < tol
    experts, ff = (4, inner // 4) if inner % 4 == 0 else (2, inner // 2)
    share = torch.rand(19, experts, generator=g)
    share[:, 1] = 0.0
    limit = 0.8
    gg, uu = gu[:, :inner].clamp(max=limit), gu[:, inner:].clamp(-limit, limit)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1.0) * share.repeat_interleave(ff, dim=1)
    kernels.routed_gate(act(gu, dtype), share.cuda(), experts, ff, out, limit=limit, slope=1.702)
    assert rel_err(out.float(), want) < tol


@pytest.mark.parametrize("dtype", DTYPES)
def test_heads_normed_without_a_gate(dtype):
    from inferrs_b200 import kernels
    o = torch.randn(13, 3, 20, generator=torch.Generator().manual_seed(1))
    wt = 1.0 + 0.2 * torch.randn(20, generator=torch.Generator().manual_seed(2))
    out = torch.empty(13, 60, dtype=dtype, device="cuda")
    kernels.head_norm_gate(o.cuda(), None, act(wt, dtype), True, kernels.GATE_SILU, 1e-5, out)
    want = pr.rms_norm(o, act(wt, dtype).float().cpu(), 1e-5).reshape(13, 60)
    assert rel_err(out.float(), want) < (1e-5 if dtype == torch.float32 else 1e-2)
