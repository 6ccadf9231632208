"""The Sefalorn design in the engine against its plain statement: every kernel alone, whole prompts, every way of
cutting a request into steps, batches, slots and pages used again, keys at the edges of windows and far away, long
decoding, and greedy generation through the engine's own entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_sefalorn as ps
from helpers import cut, random_tokens, rel_err
from sefalorn_cases import CASE_P, CASE_Q, CASE_R, CASES, for_dtype, make_weights

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-4, torch.bfloat16: 5e-2}
SEEDS = {"P": 11, "Q": 12, "R": 13, "S": 14}


def assert_close(got, want, dtype):
    """float32: every row within 2e-4 of its largest value.  bfloat16: rounding is amplified where a head's output is
    nearly zero before it is brought to unit size, so the rows are judged together: their median error and the
    nineteenth of twenty."""
    if dtype == torch.float32:
        if isinstance(got, (list, tuple)):
            got, want = torch.cat(list(got)), torch.cat(list(want))
        assert rel_err(got, want) < TOL[dtype]
        return
    if isinstance(got, (list, tuple)):                   # several requests: their rows are judged together
        got, want = torch.cat(list(got)), torch.cat(list(want))
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
    want = ps.forward(case, w, toks)
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
    want_other = ps.forward(case, w, other)
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


def test_a_second_norm_without_a_feed_forward():
    """Weight files that hold a second norm and gate for a layer without a feed-forward: they are read and do
    nothing."""
    case = CASE_Q
    shapes = {"l2.norm2": (case["width"],)}
    w = make_weights(case, 5, bare_norm2=True)
    assert "l2.rg2" in w and "l2.norm2" in w
    toks = random_tokens(30, case["vocab"], seed=6)
    runner = make_runner(case, w, torch.float32, shapes=shapes)
    runner.admit(0)
    assert rel_err(runner.step([entry(0, toks)]), ps.forward(case, w, toks)) < TOL[torch.float32]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "S"])
def test_unequal_requests_in_one_batch_slots_and_pages_used_again(name, dtype):
    """Two state slots and pages for two requests; five requests of unequal length take turns, decoding side by side
    with portions of the next ones.  Every request must give what it gives alone (the plain statement knows no
    batches, slots or pages)."""
    case = for_dtype(CASES[name], dtype)
    w = make_weights(case, SEEDS[name])
    lens = {"a": 50, "b": 23, "c": 64, "d": 9, "e": 37}
    toks = {k: random_tokens(n, case["vocab"], seed=ord(k)) for k, n in lens.items()}
    want = {k: ps.forward(case, w, t) for k, t in toks.items()}
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
    want = torch.cat([ps.forward(case, w, toks["a"])[:40], ps.forward(case, w, toks["b"])[:33]])
    assert_close(outs[1][:73], want, torch.bfloat16)


def test_long_decoding_keeps_state_and_keys():
    case, w = CASE_P, make_weights(CASE_P, 21)
    toks = random_tokens(260, case["vocab"], seed=8)
    want = ps.forward(case, w, toks)
    runner = make_runner(case, w, torch.float32, n_pages=20, max_requests=1, use_graphs=True)
    runner.admit(0)
    rows = [runner.step([entry(0, toks[:5])])]
    for t in toks[5:]:
        rows.append(runner.step([entry(0, [t])]))
    assert rel_err(torch.cat(rows), want) < TOL[torch.float32]
    # the early tokens matter to the last logits: without them the states are other ones
    late = ps.forward(case, w, toks[100:])
    assert rel_err(late[-1], want[-1]) > 1e-2


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
    want = [ps.greedy(case, w, p, n_new) for p in prompts]
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
    """Four requests at most are live, a fifth takes the slot and the pages of one that ended."""
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
    wa, wb, wc = (ps.forward(case, w, toks[k]) for k in "abc")
    read = lambda s: torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{s}.f32"), dtype="<f4").reshape(-1, case["vocab"]).copy())
    assert rel_err(read(0), wa[[0, 49]]) < 2e-4
    assert rel_err(read(1), torch.stack([wa[50], wb[18]])) < 2e-4
    assert rel_err(read(2), torch.stack([wb[19], wb[20], wa[69]])) < 2e-4
    assert not os.path.exists(os.path.join(out_dir, "3.f32"))
    assert rel_err(read(4), wc[[28, 29]]) < 2e-4


# ---------------------------------------------------------------------------------------------------
# keys at the edges of windows and far away, in the model
# ---------------------------------------------------------------------------------------------------
def one_layer(mixer_type, mixer):
    return {"architecture": "Sefalorn", "vocab": 64, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
            "layers": [{"type": mixer_type, "mlp": None, "mixer": mixer}]}


def story_weights(case, seed):
    """Weights under which a token's id is its key: the embedding is the identity times 8, the norms' weights are
    one, the residual gate is open, the head reads the stream as it is."""
    w = make_weights(case, seed)
    w["embed"] = torch.eye(64, 64) * 8.0
    w["l0.norm1"], w["final.norm"] = torch.ones(64), torch.ones(64)
    w["l0.rg1"], w["l0.rg1.b"] = torch.zeros(64, 64), torch.full((64,), 12.0)
    w["head"] = torch.eye(64, 64)
    return w


def ask_and_pick(dim):
    """Key: the first ``dim`` channels of the normed row (a token's id, if below ``dim``, stands out).  Query: the
    same, but token 7 asks for token 9."""
    pick = torch.zeros(dim, 64)
    pick[:min(dim, 64)] = torch.eye(64)[:min(dim, 64)]
    ask = pick.clone()
    ask[7, 7], ask[9, 7] = 0.0, 1.0
    return ask, pick


def mark_value(dim, gain):
    """Only token 9 has a value (channel 9 minus channel 10, which no token owns: the norm's offset cancels)."""
    v = torch.zeros(dim, 64)
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
@pytest.mark.parametrize("window,marked_at,swap,dim", [(37, 200, False, 32), (48, 208, True, 64), (5, 203, False, 128),
                                                        (64, 192, True, 32), (129, 100, True, 128)])
def test_a_marked_token_is_seen_inside_the_window_and_not_beyond(window, marked_at, swap, dim, dtype):
    """One layer whose left mixer alone speaks (the right one's scale is zero): keys are the tokens' ids, token 7 asks
    for token 9, and only token 9 has a value: the mark.  Token 9 stands once.  A token 7 returns the mark if and only
    if it stands at most window - 1 positions after it: at the window's last position, not one later, not before the
    mark, not far away.  Whole, cut into portions at odd places, decoded one by one across the window's edge; marks
    and edges on page borders too.  ``swap``: the two heads' scores change places before the softmax, so the head
    that owns the marked values must be moved by the other head's query and keys.  Head sizes of 64 and 128 run the
    tensor-core kernel in bfloat16."""
    left = {"heads": 2, "kv_heads": 2, "dim": dim, "vdim": dim, "scale": 0.5, "mask": {"size": window}}
    right = {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 2}
    case = one_layer("parallel", {"left": left, "right": right, "left_scale": 1.0, "right_scale": 0.0})
    w = story_weights(case, 2)
    ask, pick = ask_and_pick(dim)
    zero = torch.zeros(dim, 64)
    # the asking head and its keys: head 1 if the scores are swapped, else head 0; the values are head 0's
    w["l0.mix.left.q"] = torch.cat([zero, ask] if swap else [ask, zero])
    w["l0.mix.left.k"] = torch.cat([zero, pick] if swap else [pick, zero])
    w["l0.mix.left.v"] = torch.cat([mark_value(dim, 4.0), zero])
    for n in ("q", "k", "v", "o"):
        w[f"l0.mix.left.{n}.b"] = torch.zeros_like(w[f"l0.mix.left.{n}.b"])
    w["l0.mix.left.r1"], w["l0.mix.left.r2"] = torch.zeros(2), torch.ones(2)
    w["l0.mix.left.talk"] = torch.tensor([[0.0, 1.0], [1.0, 0.0]]) if swap else torch.eye(2)
    o = torch.zeros(64, 2 * dim)
    o[63, 0] = 2.0                                                # the mark goes to channel 63 of the stream
    w["l0.mix.left.o"] = o
    n = 400
    toks = [(11 + i % 20) for i in range(n)]
    toks[marked_at] = 9
    edge = marked_at + window                                     # the first position that no longer sees the mark
    probes = {marked_at + 1: True, edge - 1: True, edge: False, edge + 1: False, 390: False, marked_at - 1: False,
              10: False}
    if window > 20:
        probes[marked_at + window // 2] = True
    for p in probes:
        toks[p] = 7
    want = ps.forward(case, w, toks)
    assert {p: bool(want[p, 63] > 4.0) for p in probes} == probes       # the plain statement agrees with the story
    got, cut_up = run_whole_and_cut(case, w, dtype, toks, [64, 2, 48, 31, 90], edge - 6, edge + 12)
    for g in (got, cut_up):
        assert_close(g, want, dtype)
        assert {p: bool(g[p, 63] > 4.0) for p in probes} == probes
        assert all(abs(float(g[p, 63])) < 0.5 for p, seen in probes.items() if not seen)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_distance_penalty_decides_between_two_equal_keys(dtype):
    """Two tokens answer the same query equally well; their values differ in sign.  With a penalty on distance the
    nearer one wins, whichever it is; the penalty's size (r1) and how fast it grows (r2) are the head's own."""
    dim = 16
    left = {"heads": 1, "kv_heads": 1, "dim": dim, "vdim": dim, "scale": 0.25}
    right = {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 1}
    case = one_layer("parallel", {"left": left, "right": right, "left_scale": 1.0, "right_scale": 0.0})
    case["max_positions"] = 256
    w = story_weights(case, 3)
    ask, pick = ask_and_pick(dim)
    pick[8, 8], pick[9, 8] = 0.0, 1.0                             # tokens 8 and 9 have the same key ...
    w["l0.mix.left.q"], w["l0.mix.left.k"] = ask, pick
    v = torch.zeros(dim, 64)
    v[0, 9], v[0, 8] = 4.0, -4.0                                  # ... and opposite values
    w["l0.mix.left.v"] = v
    for n in ("q", "k", "v", "o"):
        w[f"l0.mix.left.{n}.b"] = torch.zeros_like(w[f"l0.mix.left.{n}.b"])
    w["l0.mix.left.r1"], w["l0.mix.left.r2"] = torch.tensor([3.0]), torch.tensor([0.5])
    w["l0.mix.left.talk"] = torch.ones(1, 1)
    o = torch.zeros(64, dim)
    o[63, 0] = 2.0
    w["l0.mix.left.o"] = o
    toks = [(11 + i % 20) for i in range(150)]
    toks[20], toks[100] = 9, 8                                    # far: token 9 (+), near: token 8 (-)
    toks[50], toks[120], toks[149] = 7, 7, 7
    want = ps.forward(case, w, toks)
    assert want[50, 63] > 4.0 and want[120, 63] < -4.0 and want[149, 63] < -4.0
    got, cut_up = run_whole_and_cut(case, w, dtype, toks, [33, 2, 70], 118, 125)
    for g in (got, cut_up):
        assert_close(g, want, dtype)
        assert g[50, 63] > 4.0 and g[120, 63] < -4.0 and g[149, 63] < -4.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind,decay", [("lightning", 1.0), ("lightning", 0.99), ("delta", 1.0), ("delta", 0.99)])
def test_a_marked_token_far_back_is_kept_by_the_state(kind, decay, dtype):
    """One layer whose only mixer with a state speaks: keys are the tokens' ids, token 7 asks for token 9, only token
    9 has a value.  Token 9 stands once, at position 5 of 400.  Every token 7 after it returns the mark, hundreds of
    tokens later too (the output is brought to unit size, so a decay only weakens what the norm restores); a token 7
    before it does not, and neither does one in the next request that takes the same state slot."""
    dim = 32
    ask, pick = ask_and_pick(dim)
    if kind == "lightning":
        case = one_layer("lightning", {"heads": 1, "dim": dim, "vdim": dim, "decay": [decay]})
        p = "l0.mix"
    else:
        left = {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.3, "mask": {"size": 4}}
        right = {"heads": 1, "kv_heads": 1, "dim": dim, "vdim": dim, "conv": 2}
        case = one_layer("parallel", {"left": left, "right": right, "left_scale": 0.0, "right_scale": 1.0})
        p = "l0.mix.right"
    w = story_weights(case, 4)
    w[f"{p}.q"], w[f"{p}.k"], w[f"{p}.v"] = ask, pick, mark_value(dim, 4.0)
    gate = torch.zeros_like(w[f"{p}.g"])
    gate[:, 40] = -8.0                                            # the same gate for every token: channel 40 is no
    w[f"{p}.g"] = gate                                            # token's own, the norm leaves it a little below zero
    w[f"{p}.norm"] = torch.ones_like(w[f"{p}.norm"])
    o = torch.zeros(64, dim)
    o[63, 0] = 50.0
    w[f"{p}.o"] = o
    if kind == "delta":
        for n in ("q", "k", "v"):                                 # the convolutions pass the token itself
            w[f"{p}.{n}.conv"] = torch.tensor([[0.0, 1.0]]).repeat(dim, 1)
        w[f"{p}.b"] = torch.zeros(1, 64)                          # beta = 1/2
        w[f"{p}.a"] = torch.zeros(1, 64)
        w[f"{p}.dt_bias"] = torch.zeros(1)                        # softplus(0) = ln 2
        rate = 1e-9 if decay == 1.0 else -float(np.log(decay)) / float(np.log(2.0))
        w[f"{p}.A_log"] = torch.tensor([float(np.log(rate))])
    n, marked_at = 400, 5
    toks = [(11 + i % 20) for i in range(n)]
    toks[marked_at] = 9
    probes = {2: False, 6: True, 17: True, 64: True, 250: True, 399: True}
    for q in probes:
        toks[q] = 7
    want = ps.forward(case, w, toks)
    assert {q: bool(want[q, 63] > 4.0) for q in probes} == probes
    got, cut_up = run_whole_and_cut(case, w, dtype, toks, [3, 2, 1, 64, 30, 2, 90], 300, 400, max_requests=1)
    for g in (got, cut_up):
        assert_close(g, want, dtype)
        assert {q: bool(g[q, 63] > 4.0) for q in probes} == probes
        assert float(g[2, 63]) < 0.5


# ---------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 90, 1024, 2050])
def test_gated_addition_and_layer_norm(width, dtype):
    """x += sigmoid(p + b) * delta, then the norm that takes the mean out; without a gate, without anything to add,
    and on chosen rows (which leaves the stream as it is).  The rows have a mean far from zero."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(width)
    n, eps = 7, 1e-5
    x = torch.randn(n, width, generator=g) * 2 + 5.0
    delta, pre = (torch.randn(n, width, generator=g) * 3).to(dtype), torch.randn(n, width, generator=g).to(dtype)
    bias, wgt = torch.randn(width, generator=g), 1 + 0.3 * torch.randn(width, generator=g)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for with_delta, with_gate in ((True, True), (True, False), (False, False)):
        res = x.clone().cuda()
        out = torch.empty((n, width), dtype=dtype, device="cuda")
        kernels.gated_add_layer_norm(res, delta.cuda() if with_delta else None, pre.cuda() if with_gate else None,
                                     bias.cuda() if with_gate else None, wgt.cuda(), eps, out)
        want_x = x.double()
        if with_delta:
            gate = torch.sigmoid(pre.double() + bias.double()) if with_gate else 1.0
            want_x = want_x + gate * delta.double()
        assert rel_err(res, want_x) < 1e-6
        assert rel_err(out, ps.layer_norm(want_x, wgt.double(), eps)) < tol
    rows = [5, 0, 5, 2]
    res = x.clone().cuda()
    out = torch.empty((len(rows), width), dtype=dtype, device="cuda")
    kernels.gated_add_layer_norm(res, delta.cuda(), pre.cuda(), bias.cuda(), wgt.cuda(), eps, out, dev(rows))
    want_x = x.double() + torch.sigmoid(pre.double() + bias.double()) * delta.double()
    assert rel_err(out, ps.layer_norm(want_x, wgt.double(), eps)[rows]) < tol
    assert torch.equal(res.cpu(), x)
    gated = torch.empty((n, width), dtype=dtype, device="cuda")
    kernels.gated_rows(delta.cuda(), pre.cuda(), bias.cuda(), gated)
    assert rel_err(gated, torch.sigmoid(pre.double() + bias.double()) * delta.double()) < tol


@pytest.mark.parametrize("dtype", DTYPES)
def test_bias_and_scaled_sum(dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(1)
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    a, b = torch.randn(5, 77, generator=g).to(dtype), torch.randn(5, 77, generator=g).to(dtype)
    out = torch.empty((5, 77), dtype=dtype, device="cuda")
    kernels.scaled_sum(a.cuda(), 1.3, b.cuda(), -0.4, out)
    assert rel_err(out, 1.3 * a.double() - 0.4 * b.double()) < tol
    wide = torch.randn(5, 90, generator=g).to(dtype)
    bias = torch.randn(61, generator=g)
    x = wide.clone().cuda()
    kernels.bias_add(x[:, :80], bias.cuda())                      # a view of a wider row, a bias shorter than the view
    want = wide.double()
    want[:, :61] += bias.double()
    assert rel_err(x, want) < tol


def paged(keys, values, page_size, dtype, seed):
    """Pages in a shuffled order for requests' keys [T, G, D] and values [T, G, E]; what no token owns is NaN in the
    keys and zero in the values."""
    g = torch.Generator().manual_seed(seed)
    G, D, E = keys[0].shape[1], keys[0].shape[2], values[0].shape[2]
    pages_per = [(k.shape[0] + page_size - 1) // page_size for k in keys]
    perm = torch.randperm(sum(pages_per) + 2, generator=g).tolist()
    table = torch.full((len(keys), max(pages_per)), -1, dtype=torch.int32)
    k_pages = torch.full((len(perm), G, page_size, D), float("nan"))
    v_pages = torch.zeros((len(perm), G, page_size, E))
    for r, (k, v) in enumerate(zip(keys, values)):
        for p in range(pages_per[r]):
            page = perm.pop()
            table[r, p] = page
            part = slice(p * page_size, min((p + 1) * page_size, k.shape[0]))
            k_pages[page, :, :part.stop - part.start] = k[part].transpose(0, 1)
            v_pages[page, :, :part.stop - part.start] = v[part].transpose(0, 1)
    return table.cuda(), act(k_pages, dtype), act(v_pages, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,E,window", [(6, 2, 24, 20, 23), (4, 4, 16, 40, 50), (1, 1, 32, 16, 1), (8, 2, 64, 64, None),
                                            (3, 1, 10, 7, 7), (5, 5, 6, 14, 33), (4, 2, 128, 128, 72)])
def test_attention_with_mixed_heads_and_a_distance_penalty(H, G, D, E, window, dtype):
    """Queries mixed across heads, then the attention kernel on joint queries with the table of mixed penalties,
    against scores that are penalised and mixed pair by pair.  Three requests: a prompt portion after cached tokens,
    a single token after many, a first token."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(H * 10 + D)
    lens, new = [150, 141, 1], [60, 1, 1]
    ks = [torch.randn(l, G, D, generator=g).to(dtype).float() for l in lens]
    vs = [torch.randn(l, G, E, generator=g).to(dtype).float() for l in lens]
    table, k_pages, v_pages = paged(ks, vs, 16, dtype, D)
    positions = [p for l, t in zip(lens, new) for p in range(l - t, l)]
    row_request = [r for r, t in enumerate(new) for _ in range(t)]
    n = len(positions)
    q = torch.randn(n, H, D, generator=g).to(dtype).float()
    r1, r2 = torch.rand(H, generator=g) + 0.1, torch.rand(H, generator=g) * 0.3 + 0.02
    talk = torch.eye(H) * 0.8 + 0.35 * torch.randn(H, H, generator=g)
    scale = 0.3 * (24.0 / D) ** 0.5
    reach = window or 160
    own = r1.double()[:, None] * torch.log1p(r2.double()[:, None] * torch.arange(reach, dtype=torch.float64)[None, :])
    table_of_penalties = (talk.double() @ own).float().cuda().contiguous()
    mixed = torch.empty((n, H, G * D), dtype=dtype, device="cuda")
    kernels.mix_queries(act(q, dtype), talk.cuda(), G, mixed)
    for h in range(H):                                            # the mixed queries are what their name says
        for c in range(G):
            heads = range(c * (H // G), (c + 1) * (H // G))
            want = sum(talk[h, i].double() * q[:, i].double() for i in heads)
            assert rel_err(mixed[:, h, c * D:(c + 1) * D], want) < (1e-5 if dtype == torch.float32 else 1e-2)
    out = torch.empty((n, H * E), dtype=dtype, device="cuda")
    kernels.paged_attention_generic(mixed, k_pages, v_pages, table, dev(row_request), dev(positions), scale,
                                    kernels.span_argument(window), out, joint=True, dist_bias=table_of_penalties)
    at = 0
    for r, t in enumerate(new):
        want = ps.mixed_score_attention(q[at:at + t].double(), ks[r].double(), vs[r].double(),
                                        torch.tensor(positions[at:at + t]), scale, r1.double(), r2.double(),
                                        talk.double(), window)
        assert rel_err(out[at:at + t], want.reshape(t, -1)) < (2e-5 if dtype == torch.float32 else 3e-2), r
        at += t


@pytest.mark.parametrize("form", ["prefill", "decode", "decode_split"])
@pytest.mark.parametrize("H,G,D,window", [(8, 2, 128, 100), (4, 4, 64, 50), (6, 1, 64, None), (3, 3, 128, 1), (16, 1, 64, 129),
                                          (6, 2, 128, None), (8, 4, 128, 77)])     # the last: one key tile in shared memory
def test_tensor_core_attention_with_mixed_heads_and_a_distance_penalty(H, G, D, window, form):
    """The tensor-core kernel for joint queries (bfloat16, keys and values of 64 or 128 numbers) in its prefill form
    (portions after cached tokens, a single token, a first token, tiles that end inside a request) and its decode
    form, with and without the keys cut into slices; with and without a window; with and without a penalty."""
    from inferrs_b200 import kernels
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(H * 10 + D)
    if form == "prefill":
        lens, new = [333, 141, 1, 90], [150, 1, 1, 90]
    else:
        lens, new = [333, 141, 1, 64, 65], [1, 1, 1, 1, 1]
    ks = [torch.randn(l, G, D, generator=g).to(dtype).float() for l in lens]
    vs = [torch.randn(l, G, D, generator=g).to(dtype).float() for l in lens]
    table, k_pages, v_pages = paged(ks, vs, 16, dtype, D)
    positions = [p for l, t in zip(lens, new) for p in range(l - t, l)]
    n = len(positions)
    q = torch.randn(n, H, D, generator=g).to(dtype).float()
    r1, r2 = torch.rand(H, generator=g) + 0.1, torch.rand(H, generator=g) * 0.3 + 0.02
    talk = torch.eye(H) * 0.8 + 0.35 * torch.randn(H, H, generator=g)
    scale = 0.3 * (24.0 / D) ** 0.5
    reach = window or 340
    own = r1.double()[:, None] * torch.log1p(r2.double()[:, None] * torch.arange(reach, dtype=torch.float64)[None, :])
    penalties = (talk.double() @ own).float().cuda().contiguous()
    mixed = torch.empty((n, H, G * D), dtype=dtype, device="cuda")
    kernels.mix_queries(act(q, dtype), talk.cuda(), G, mixed)
    q_start = [0] + list(np.cumsum(new))
    out = torch.full((n, H * D), float("nan"), dtype=dtype, device="cuda")
    assert kernels.joint_mma_attention_supported(dtype, H, G, D, D, 16, form != "prefill")
    if form == "prefill":
        tpt = kernels.joint_mma_prefill_tokens(H, G, D, 16)      # a tile's tokens
        assert 0 < tpt * (H // G) <= 128
        tiles = [(r, row) for r in range(len(new)) for row in range(q_start[r], q_start[r + 1], tpt)]
        tile_req = dev([t[0] for t in tiles] + [-1, -1])           # places that hold no tile are skipped
        tile_row0 = dev([t[1] for t in tiles] + [0, 0])
        kernels.joint_attention_mma(mixed, k_pages, v_pages, table, tile_req, tile_row0, len(tiles) + 2, dev(q_start),
                                    dev(positions), scale, window, penalties, out, False)
    else:
        kernels.joint_attention_mma(mixed, k_pages, v_pages, table, dev(list(range(n))), dev(q_start), n, dev(q_start),
                                    dev(positions), scale, window, penalties, out, True,
                                    3 if form == "decode_split" else 1)
    mixed_back = mixed.float().cpu()          # the kernel's own input: the mixed queries as bfloat16 rounded them
    at = 0
    for r, t in enumerate(new):
        want = ps.mixed_score_attention(q[at:at + t].double(), ks[r].double(), vs[r].double(),
                                        torch.tensor(positions[at:at + t]), scale, r1.double(), r2.double(),
                                        talk.double(), window)
        assert rel_err(out[at:at + t], want.reshape(t, -1)) < 3e-2, r
        at += t
    assert mixed_back.shape == (n, H, G * D)
    # without a penalty and with the identity as the mixing matrix the plain attention must come out
    eye = torch.eye(H)
    kernels.mix_queries(act(q, dtype), eye.cuda(), G, mixed)
    plain = torch.full((n, H * D), float("nan"), dtype=dtype, device="cuda")
    if form == "prefill":
        kernels.joint_attention_mma(mixed, k_pages, v_pages, table, tile_req, tile_row0, len(tiles) + 2, dev(q_start),
                                    dev(positions), scale, window, None, plain, False)
    else:
        kernels.joint_attention_mma(mixed, k_pages, v_pages, table, dev(list(range(n))), dev(q_start), n, dev(q_start),
                                    dev(positions), scale, window, None, plain, True, 2 if form == "decode_split" else 1)
    at = 0
    for r, t in enumerate(new):
        want = ps.mixed_score_attention(q[at:at + t].double(), ks[r].double(), vs[r].double(),
                                        torch.tensor(positions[at:at + t]), scale, torch.zeros(H, dtype=torch.float64),
                                        torch.ones(H, dtype=torch.float64), eye.double(), window)
        assert rel_err(plain[at:at + t], want.reshape(t, -1)) < 2e-2, r
        at += t


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,E", [(4, 2, 20, 12), (1, 1, 128, 64), (3, 3, 36, 8), (6, 2, 48, 32), (2, 1, 250, 33),
                                     (4, 4, 64, 64), (16, 2, 128, 128), (5, 5, 6, 5), (3, 1, 10, 9)])
@pytest.mark.parametrize("aligned", [False, True])
def test_delta_scan_against_the_rule(H, G, D, E, aligned, dtype):
    """Three requests of unequal length side by side, in three steps (the last one of single tokens), their state
    slots out of order; queries and keys shared by the heads of a group and made unit vectors by the kernel; key
    sizes that are no multiple of 16 and value sizes that are no multiple of 8."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(H * 100 + D)
    slots = [2, 0, 1]
    c0 = 4 if aligned else 1
    ld = (2 * G * D + H * E + c0 + 6) // 4 * 4 + (0 if aligned else 1)
    n_state = H * D * E + 11
    state = torch.zeros((4, n_state), dtype=torch.float32, device="cuda")
    S = [torch.zeros(H, D, E, dtype=torch.float64) for _ in range(3)]
    unit_eps, q_scale = 1e-6, D ** -0.5
    for lens in ([5, 1, 19], [3, 30, 1], [1, 1, 1]):
        n = sum(lens)
        x = torch.randn(n, ld, generator=g)
        fade = torch.rand(n, H, generator=g) * 0.3 + 0.7
        beta = torch.rand(n, H, generator=g)
        gates = torch.cat([fade, beta], dim=1).cuda().contiguous()
        out = torch.empty((n, H, E), dtype=torch.float32, device="cuda")
        kernels.delta_scan(x.cuda(), c0, c0 + G * D, c0 + 2 * G * D, G, gates[:, :H], gates[:, H:], unit_eps, q_scale,
                           state, dev([0] + list(np.cumsum(lens))), dev(slots), 3, out, D, dtype, max_rows=max(lens))
        at = 0
        for r, n_r in enumerate(lens):
            rows = slice(at, at + n_r)
            q = x[rows, c0:c0 + G * D].reshape(n_r, G, D).double()
            k = x[rows, c0 + G * D:c0 + 2 * G * D].reshape(n_r, G, D).double()
            v = x[rows, c0 + 2 * G * D:c0 + 2 * G * D + H * E].reshape(n_r, H, E).double()
            want = ps.delta_rule(ps.unit_vector(q) * q_scale, ps.unit_vector(k), v, beta[rows].double(),
                                 fade[rows].double(), S[r])
            assert rel_err(out[rows], want) < 1e-4, (r, lens)
            at += n_r
    for r, slot in enumerate(slots):
        assert rel_err(state[slot, :H * D * E].reshape(H, D, E), S[r]) < 1e-4
        assert float(state[slot, H * D * E:].abs().max()) == 0.0     # what lies behind the matrices is not touched
    assert float(state[3].abs().max()) == 0.0           # a slot that no request of the step names is not touched


@pytest.mark.parametrize("n", [2, 3, 15, 16, 17, 32, 33, 81])
@pytest.mark.parametrize("H,G,D,E", [(2, 1, 24, 20), (3, 3, 128, 16)])
def test_delta_scan_sixteen_at_once_against_one_by_one(n, H, G, D, E):
    """A prompt portion walked sixteen tokens at once and the same rows as steps of single tokens give the rule's
    result: lengths around the sixteen, a fade of exactly zero (the state is forgotten there, and nothing may divide
    by it), step sizes of zero and one, a state that is not zero at the start."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(n * 7 + D)
    x = torch.randn(n, 2 * G * D + H * E, generator=g)
    fade = torch.rand(n, H, generator=g) * 0.5 + 0.5
    beta = torch.rand(n, H, generator=g)
    if n > 2:
        fade[n // 2, 0] = 0.0
        beta[n // 3, H - 1] = 0.0
        beta[n - 1, 0] = 1.0
    gates = torch.cat([fade, beta], dim=1).cuda().contiguous()
    start = torch.randn(H, D, E, generator=g)
    q = x[:, :G * D].reshape(n, G, D).double()
    k = x[:, G * D:2 * G * D].reshape(n, G, D).double()
    v = x[:, 2 * G * D:].reshape(n, H, E).double()
    S = start.double().clone()
    want = ps.delta_rule(ps.unit_vector(q) * 0.3, ps.unit_vector(k), v, beta.double(), fade.double(), S)
    got = {}
    for form in ("portion", "single"):
        state = torch.zeros((2, H * D * E), dtype=torch.float32, device="cuda")
        state[1] = start.reshape(-1).cuda()
        out = torch.empty((n, H, E), dtype=torch.float32, device="cuda")
        if form == "portion":
            kernels.delta_scan(x.cuda(), 0, G * D, 2 * G * D, G, gates[:, :H], gates[:, H:], 1e-6, 0.3, state,
                               dev([0, n]), dev([1]), 1, out, D, torch.float32, max_rows=n)
        else:
            for t in range(n):
                kernels.delta_scan(x[t:t + 1].cuda(), 0, G * D, 2 * G * D, G, gates[t:t + 1, :H], gates[t:t + 1, H:],
                                   1e-6, 0.3, state, dev([0, 1]), dev([1]), 1, out[t:t + 1], D, torch.float32,
                                   max_rows=1)
        assert rel_err(out, want) < 1e-4, form
        assert rel_err(state[1].reshape(H, D, E), S) < 1e-4, form
        assert float(state[0].abs().max()) == 0.0
        got[form] = out
    assert rel_err(got["portion"], got["single"].double()) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_delta_scan_without_unit_vectors(dtype):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(5)
    H, D, E, n = 2, 12, 20, 9
    x = torch.randn(n, 2 * H * D + H * E, generator=g) * 0.4
    gates = torch.rand(n, 2 * H, generator=g).cuda()
    state = torch.zeros((1, H * D * E), dtype=torch.float32, device="cuda")
    out = torch.empty((n, H, E), dtype=torch.float32, device="cuda")
    kernels.delta_scan(x.cuda(), 0, H * D, 2 * H * D, H, gates[:, :H], gates[:, H:], None, 0.7, state, dev([0, n]),
                       dev([0]), 1, out, D, dtype, max_rows=n)
    xd = x.double()
    want = ps.delta_rule(xd[:, :H * D].reshape(n, H, D) * 0.7, xd[:, H * D:2 * H * D].reshape(n, H, D),
                         xd[:, 2 * H * D:].reshape(n, H, E), gates[:, H:].double().cpu(), gates[:, :H].double().cpu())
    assert rel_err(out, want) < 1e-4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,C,H", [(4, 50, 3), (1, 8, 1), (2, 130, 5), (3, 33, 2)])
def test_convolution_without_a_bias_with_its_state_and_the_rule_s_two_numbers(taps, C, H, dtype):
    """Requests cut into steps, among them steps shorter than the convolution's reach; per head the fade
    exp(-exp(A) softplus(a + b)) and the step size sigmoid(.) of the delta rule."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(taps * 10 + C)
    ld, conv_col, dt_col, beta_col, off = C + 2 * H + 9, 4, 4 + C + 2, 4 + C + 2 + H + 1, 13
    w = torch.randn(C, taps, generator=g)
    dt_bias, a_log = torch.randn(H, generator=g), torch.randn(H, generator=g) * 0.5
    total = {"a": 40, "b": 17}
    proj = {k: torch.randn(n, ld, generator=g).to(dtype) for k, n in total.items()}
    state = torch.zeros((3, off + max(taps - 1, 0) * C + 2), dtype=torch.float32, device="cuda")
    slot = {"a": 2, "b": 0}
    want = {}
    for k, p in proj.items():
        z = ps.short_conv(p.double()[:, conv_col:conv_col + C], w.double())
        fade = torch.exp(-torch.exp(a_log.double()) * ps.softplus(p.double()[:, dt_col:dt_col + H] + dt_bias.double()))
        want[k] = (ps.silu(z), fade, torch.sigmoid(p.double()[:, beta_col:beta_col + H]))
    at = {"a": 0, "b": 0}
    for step in [{"a": 1, "b": 2}, {"a": 1}, {"b": 1, "a": 2}, {"a": 20, "b": 1}, {"b": 13}, {"a": 16}]:
        keys = list(step)
        rows = torch.cat([proj[k][at[k]:at[k] + step[k]] for k in keys]).cuda().contiguous()
        n = rows.shape[0]
        q_start = dev([0] + list(np.cumsum([step[k] for k in keys])))
        slots = dev([slot[k] for k in keys])
        row_request = dev([i for i, k in enumerate(keys) for _ in range(step[k])])
        out = torch.empty((n, C), dtype=torch.float32, device="cuda")
        gates = torch.empty((n, 2 * H), dtype=torch.float32, device="cuda")
        kernels.conv_silu_gates(rows, conv_col, w.cuda(), None, state, off, q_start, slots, row_request, out, dt_col,
                                dt_bias.cuda(), a_log.cuda(), gates, beta_col=beta_col)
        kernels.conv_state_shift(rows, conv_col, C, taps, state, off, q_start, slots, len(keys))
        r0 = 0
        for k in keys:
            sl = slice(at[k], at[k] + step[k])
            assert rel_err(out[r0:r0 + step[k]], want[k][0][sl]) < 1e-5, (k, at[k])
            assert rel_err(gates[r0:r0 + step[k], :H], want[k][1][sl]) < 1e-5
            assert rel_err(gates[r0:r0 + step[k], H:], want[k][2][sl]) < 1e-5
            r0 += step[k]
            at[k] += step[k]
    assert at == total


@pytest.mark.parametrize("experts,top,scale", [(8, 4, 2.0), (5, 2, 1.5), (3, 3, 1.0), (70, 6, 0.5), (4, 1, 2.5), (1, 1, 1.0)])
def test_router_by_sigmoid_shares(experts, top, scale):
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(experts)
    n = 9
    logits = torch.randn(n, experts + 2, generator=g) * 2
    logits[1] = -60.0                                             # scores so small that the 1e-20 beside their sum
    logits[1, :experts] += torch.arange(experts) * 0.5            # decides: the shares no longer add up to the scale
    want = ps.sigmoid_shares(logits[:, :experts].double(), top, scale)
    got = torch.empty((n, experts), dtype=torch.float32, device="cuda")
    kernels.router_topk(logits.cuda(), None, experts, top, False, got, torch.float32, mode=kernels.ROUTE_SIGMOID_SHARE,
                        scale=scale)
    assert rel_err(got, want) < 1e-5
    assert int((got > 0).sum()) == n * top
    others = [r for r in range(n) if r != 1]
    assert rel_err(got.sum(dim=1)[others], torch.full((n - 1,), scale, dtype=torch.float64)) < 1e-5
    assert rel_err(got[1].sum(), want[1].sum()) < 1e-5
    assert experts > 8 or float(got[1].sum()) < 0.01 * scale


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,E", [(3, 40, 24), (1, 10, 7), (6, 32, 64), (5, 16, 120)])    # the last: a block per row
@pytest.mark.parametrize("spare", [3, 4])
def test_silu_on_the_way_in_and_one_norm_over_all_heads(H, D, E, spare, dtype):
    """The pieces that the fixed-decay scan gets for this design: q, k and v through silu as float rows (row lengths
    that are and are not a multiple of four: the kernel's two forms), and after the scan one root mean square over
    the heads side by side, a weight per number and a sigmoid gate."""
    from inferrs_b200 import kernels
    g = torch.Generator().manual_seed(D)
    n, hd, he = 11, H * D, H * E
    proj = torch.randn(n, 2 * hd + 2 * he + spare, generator=g).to(dtype)
    x = torch.empty((n, 2 * hd + he), dtype=torch.float32, device="cuda")
    kernels.heads_to_float(proj.cuda(), ((0, 0, H, D, 0, 1.0, True), (hd, hd, H, D, 0, 1.0, True),
                                         (2 * hd, 2 * hd, H, E, 0, 1.0, True)), x, None, None, 0, None)
    assert rel_err(x, ps.silu(proj.double()[:, :2 * hd + he])) < 1e-6
    decay = torch.rand(H, generator=g) * 0.2 + 0.8
    state = torch.zeros((1, H * D * E), dtype=torch.float32, device="cuda")
    o = torch.empty((n, H, E), dtype=torch.float32, device="cuda")
    kernels.decay_scan(x, 0, hd, 2 * hd, H, decay.cuda(), None, None, state, dev([0, n]), dev([0]), 1, o, D, dtype,
                       max_rows=n)
    xd = x.double().cpu()
    want_o = ps.fixed_decay_rule(xd[:, :hd].reshape(n, H, D), xd[:, hd:2 * hd].reshape(n, H, D),
                                 xd[:, 2 * hd:].reshape(n, H, E), decay.double())
    assert rel_err(o, want_o) < 1e-4
    wgt = (1 + 0.2 * torch.randn(he, generator=g)).to(dtype)
    out = torch.empty((n, he), dtype=dtype, device="cuda")
    kernels.head_norm_gate(o.view(n, 1, he), proj.cuda()[:, 2 * hd + he:2 * hd + 2 * he], wgt.cuda(), True,
                           kernels.GATE_SIGMOID, 1e-5, out)
    want = ps.rms_unit(o.double().cpu().reshape(n, he), 1e-5) * wgt.double() \
        * torch.sigmoid(proj.double()[:, 2 * hd + he:2 * hd + 2 * he])
    assert rel_err(out, want) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_each_mixer_and_feed_forward_alone_in_a_model_of_one_layer(dtype):
    """Every kind of layer as the only layer of a model, against the plain statement."""
    layers = [(CASE_P, 0), (CASE_P, 1), (CASE_P, 3), (CASE_R, 0), (CASE_R, 2), (CASE_Q, 2)]
    for i, (base, which) in enumerate(layers):
        case = {k: v for k, v in for_dtype(base, dtype).items() if k != "layers"}
        case["layers"] = [for_dtype(base, dtype)["layers"][which]]
        w = make_weights(case, 50 + i)
        toks = random_tokens(70, case["vocab"], seed=i)
        runner = make_runner(case, w, dtype)
        runner.admit(0)
        got = runner.step([entry(0, toks[:37])])
        got = torch.cat([got, runner.step([entry(0, toks[37:])])])
        assert_close(got, ps.forward(case, w, toks), dtype)
