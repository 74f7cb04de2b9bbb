"""Pilonex in the engine against the plain implementation: the new kernels alone, every mechanism alone in a model of
one layer, whole prompts, decoding through cache and state, portions, mixed batches, pages and slots that are used
again, window edges, far keys, greedy generation through the scheduler, the command line and the trace program."""
import json
import math
import subprocess
import sys

import pytest
import torch

import plain_pilonex as plain
from pilonex_cases import (CASES, STRETCH, assert_logits, attn, delta, dense, make_folder, mlstm, moe, oracle, parallel, read_folder,
                           bfloat16_noise, float32_noise, router_margin, tokens_for)
from helpers import (ROOT, count_page_handouts, replay_in_process, replay_trace_run, round64, trace_mixed, trace_portions,
                     trace_tail, trace_whole)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: make_folder(str(tmp_path_factory.mktemp(f"plx{n}")), cfg, seed) for n, (cfg, seed) in CASES.items()}


def runner_for(path, dtype, max_tokens=2048, max_requests=4, page_size=16, graphs=True):
    from openinfer_b200.engine.runner import ModelRunner
    r = ModelRunner.from_folder(path, dtype=dtype, max_tokens=max_tokens, max_requests=max_requests, page_size=page_size)
    r.cuda_graph = graphs
    return r


def compare(got, path, toks, dtype, what, rows=slice(None), noise=None):
    assert_logits(got, oracle(path, toks)[rows], dtype, what, margin=router_margin(path, toks)[rows],
                  noise=float32_noise(path, toks) if noise is None else noise, noise16=bfloat16_noise(path, toks))


def check_trace(runner, path, requests, steps, dtype, what):
    got = replay_in_process(runner, steps)
    # what rounding alone does to this model: the largest of its sequences' samples (a short sequence is a poor sample)
    noise = max(float32_noise(path, toks) for toks in requests.values())
    for rid, toks in requests.items():
        compare(got[rid], path, toks, dtype, f"{what}/{rid}", noise=noise)
    runner.cache.check()
    assert runner.cache.min_free_pages() == runner.cache.num_pages and runner.cache.slot_pool.used_count == 0


def _dev(t, dtype=None):
    return t.to(device="cuda", dtype=dtype or t.dtype)


# ---------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("S,W", [(1, 40), (2, 64), (3, 100), (4, 1030), (5, 72), (8, 24), (11, 36), (16, 128)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_stream_kernels(S, W, out_dtype):
    """The kernel that carries a sublayer's result into the streams and reads the next sublayer's normed input off the
    new streams; the same without coefficients (the plain residual); the gathered sum and norm at the end."""
    from openinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(S * 1000 + W)
    T = 7
    X = torch.randn(T, S, W, generator=g)
    y = torch.randn(T, W, generator=g)
    M = (torch.eye(S) + 0.3 * torch.randn(S, S, generator=g)).to(torch.bfloat16)
    b, a = torch.randn(S, generator=g).to(torch.bfloat16), torch.randn(S, generator=g).to(torch.bfloat16)
    w = (0.1 * torch.randn(W, generator=g)).to(torch.bfloat16)
    Xn = torch.einsum("tsw,sr->trw", X.double(), M.double()) + b.double()[None, :, None] * y.double()[:, None, :]
    u = torch.einsum("tsw,s->tw", Xn, a.double())
    ref = plain.rms_one_plus(u, w.double(), 1e-5)
    tol = 2e-5 if out_dtype == torch.float32 else 2e-2
    Xd = _dev(X.clone())
    out = torch.empty(T, W, dtype=out_dtype, device="cuda")
    ops.hyper_step(Xd, y=_dev(y), mix=_dev(M), b_out=_dev(b), a_in=_dev(a), norm_w=_dev(w), eps=1e-5, weight_offset=1.0, out=out)
    assert (Xd.double().cpu() - Xn).abs().max().item() < 1e-5 * max(1.0, Xn.abs().max().item())
    assert (out.double().cpu() - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item())
    # only the first half (no input is read), then only the second half on gathered rows with the plain sum
    Xd = _dev(X.clone())
    ops.hyper_step(Xd, y=_dev(y), mix=_dev(M), b_out=_dev(b))
    assert (Xd.double().cpu() - Xn).abs().max().item() < 1e-5 * max(1.0, Xn.abs().max().item())
    idx = torch.tensor([5, 0, 5], dtype=torch.int32)
    out = torch.empty(3, W, dtype=out_dtype, device="cuda")
    before = Xd.clone()
    ops.hyper_step(Xd, norm_w=_dev(w), eps=1e-5, weight_offset=1.0, out=out, row_idx=_dev(idx))
    ref = plain.rms_one_plus(Xn.sum(1), w.double(), 1e-5)[idx.long()]
    assert (out.double().cpu() - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item()) and torch.equal(Xd, before)
    # two results that come back as a weighted sum
    y2 = torch.randn(T, W, generator=g)
    Xd = _dev(X.clone())
    ops.hyper_step(Xd, y=_dev(y), y2=_dev(y2), c1=1.3, c2=0.6, mix=_dev(M), b_out=_dev(b))
    both = torch.einsum("tsw,sr->trw", X.double(), M.double()) + b.double()[None, :, None] * (1.3 * y.double() + 0.6 * y2.double())[:, None, :]
    assert (Xd.double().cpu() - both).abs().max().item() < 1e-5 * max(1.0, both.abs().max().item())
    # without coefficients: x + y on every stream's own
    Xd = _dev(X.clone())
    ops.hyper_step(Xd, y=_dev(y))
    assert (Xd.double().cpu() - (X.double() + y.double()[:, None, :])).abs().max().item() < 1e-5
    # all streams start as the embedding output
    h = torch.randn(T, W, generator=g)
    ops.hyper_fanout(Xd, _dev(h))
    assert torch.equal(Xd.cpu(), h[:, None, :].expand(T, S, W))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_gate_activation_kernel(dtype):
    from openinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    for rows, inter, limit in ((5, 24, 1.5), (3, 100, 0.7), (9, 64, 7.0)):
        gu = (torch.randn(rows, 2 * inter, generator=g) * 3).to(dtype)
        out = torch.empty(rows, inter, dtype=dtype, device="cuda")
        ops.glu_act(out, _dev(gu), None, "swiglu_clamp", limit)
        gt, up = gu[:, :inter].double().clamp(max=limit), gu[:, inter:].double().clamp(-limit, limit)
        ref = gt * torch.sigmoid(1.702 * gt) * (up + 1)
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert ((out.double().cpu() - ref).abs() <= tol * (1 + ref.abs())).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,W,F,E,top", [(1, 40, 24, 5, 2), (37, 64, 16, 3, 1), (200, 96, 40, 16, 4), (9, 36, 70, 40, 3), (64, 128, 96, 4, 4)])
def test_routed_experts_kernels(dtype, rows, W, F, E, top):
    """Router, grouping and the two grouped products against the plain statement, row by row; the chosen experts are
    the plain implementation's; a row's result does not depend on the rows beside it."""
    from openinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(rows + E)
    x = torch.randn(rows, W, generator=g).to(dtype)
    Wt = {"router": (torch.randn(E, W, generator=g) * 0.5).to(torch.bfloat16)}
    for e in range(E):
        Wt[f"e{e}.gate"] = (torch.randn(F, W, generator=g) * W ** -0.5).to(torch.bfloat16)
        Wt[f"e{e}.up"] = (torch.randn(F, W, generator=g) * W ** -0.5).to(torch.bfloat16)
        Wt[f"e{e}.down"] = (torch.randn(W, F, generator=g) * F ** -0.5).to(torch.bfloat16)
    ref = plain.routed_experts(x.double(), {k: v.double() for k, v in Wt.items()}, "", E, top, 1.25)
    gate_up = torch.stack([torch.cat([Wt[f"e{e}.gate"], Wt[f"e{e}.up"]]) for e in range(E)]).to(dtype)
    down = torch.stack([Wt[f"e{e}.down"] for e in range(E)]).to(dtype)
    routing = ops.moe_route(_dev(x), _dev(Wt["router"]), top)
    z = x.double() @ Wt["router"].double().T
    want_ids = torch.topk(z, top, dim=1).indices
    assert torch.equal(routing[0].cpu().long().sort(dim=1).values, want_ids.sort(dim=1).values)
    assert (routing[1].sum(1) - 1).abs().max().item() < 1e-5
    out = ops.moe_experts(_dev(x), _dev(gate_up), _dev(down), routing, 1.25)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (out.double().cpu() - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item())
    if rows > 100:   # the first rows alone (still a step of tiles): the same bits
        part = ops.moe_experts(_dev(x[:90]), _dev(gate_up), _dev(down), ops.moe_route(_dev(x[:90]), _dev(Wt["router"]), top), 1.25)
        assert torch.equal(part, out[:90])
    if rows > 8:     # a few rows alone go pair by pair: the same result up to the order of the sums
        part = ops.moe_experts(_dev(x[:3]), _dev(gate_up), _dev(down), ops.moe_route(_dev(x[:3]), _dev(Wt["router"]), top), 1.25)
        assert (part.double().cpu() - ref[:3]).abs().max().item() < tol * max(1.0, ref.abs().max().item())


def test_stretched_rotation_tables():
    from openinfer_b200.parts.position import RotaryEncoding
    from openinfer_b200.parts.spec import PositionSpec
    for dims, base, sc in ((8, 10000.0, STRETCH), (64, 200000.0, {"factor": 3.0, "low": 1.0, "high": 5.0, "original": 256}), (6, 100.0, None)):
        spec = PositionSpec(kind="rope", rotary_dim=dims, theta=base, max_positions=700,
                            scaling=(sc["factor"], sc["low"], sc["high"], sc["original"]) if sc else None)
        cos, sin = RotaryEncoding(spec).rotation_tables(torch.device("cuda"))
        f = plain.rotary_frequencies({"dims": dims, "base": base, "scaling": sc}, torch.float64)
        ang = torch.arange(700, dtype=torch.float64)[:, None] * f[None, :]
        assert cos.shape == (700, dims // 2)
        assert (cos.double().cpu() - torch.cos(ang)).abs().max().item() < 1e-4 and (sin.double().cpu() - torch.sin(ang)).abs().max().item() < 1e-4
    if True:   # the three regimes are all present in the first table's frequencies
        f = plain.rotary_frequencies({"dims": 8, "base": 10000.0, "scaling": STRETCH}, torch.float64)
        raw = 10000.0 ** (-2.0 * torch.arange(4, dtype=torch.float64) / 8)
        ratio = (f / raw).tolist()
        assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 8) < 1e-12 and any(1 / 8 < r < 1 for r in ratio)


# ---------------------------------------------------------------------------------------------- mechanisms alone
def _one_layer(layer, streams=None, width=48, vocab=83):
    cfg = {"architecture": "Pilonex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": [layer]}
    if streams:
        cfg["streams"] = streams
    return cfg


MECHANISMS = {
    "matrix memory": _one_layer(mlstm(3, 16, 24, 5.0)),
    "matrix memory, one head, wide keys": _one_layer(mlstm(1, 100, 8, 15.0)),
    "matrix memory with 300 key channels": _one_layer(mlstm(1, 300, 8, 10.0)),
    "window attention alone": _one_layer(parallel(attn(4, 2, 16, 8, 0.5, window=18, rot={"dims": 12, "base": 1000.0, "scaling": STRETCH}),
                                                  delta(2, 1, 8, 8, 2), 1.0, 0.0)),
    "attention with values wider than keys, no rotation, no window": _one_layer(parallel(attn(3, 3, 8, 20, 0.7), delta(1, 1, 8, 8, 1), 1.0, 0.0)),
    "attention with heads wider than 256": _one_layer(parallel(attn(2, 1, 264, 40, 0.08, window=40, rot={"dims": 100, "base": 10000.0}),
                                                               delta(1, 1, 8, 8, 2), 1.0, 0.0)),
    "delta rule alone": _one_layer(parallel(attn(1, 1, 8, 8, 1.0, window=4), delta(4, 2, 12, 20, 4), 0.0, 1.0)),
    "delta rule, one tap": _one_layer(parallel(attn(1, 1, 8, 8, 1.0, window=4), delta(3, 3, 16, 8, 1), 0.0, 1.0)),
    "routed experts": _one_layer(mlstm(1, 8, 8, 5.0, moe(32, 0.9, 7, 3))),
    "dense feed-forward with a small limit": _one_layer(mlstm(2, 8, 8, 5.0, dense(80, 0.6))),
    "three streams": _one_layer(mlstm(2, 8, 8, 5.0, dense(40, 2.0)), streams=3),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(MECHANISMS))
def test_each_mechanism_alone(tmp_path, name, dtype):
    """A model of one layer whose other side is switched off or minimal: a whole prompt, then portions of 2, 1, 5 and 3
    tokens and decoding, two requests in the same steps."""
    cfg = MECHANISMS[name]
    path = make_folder(str(tmp_path / "m"), cfg, 7)
    requests = {"a": tokens_for(cfg, 75, 1), "b": tokens_for(cfg, 40, 2)}
    runner = runner_for(path, dtype, max_tokens=256)
    check_trace(runner, path, requests, trace_whole(requests), dtype, name)
    check_trace(runner, path, requests, trace_portions(requests, sizes=(2, 1, 5, 3, 30, 1, 1, 2)), dtype, name + "/portions")


# ---------------------------------------------------------------------------------------------- the model
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CASES))
def test_whole_prompts_and_decoding_match_plain(folders, name, dtype):
    """Whole prompts in one step (the first tokens of a sequence among them: one and two tokens); then most of a prompt
    in one step and its last 70 tokens one by one through recorded graphs, far enough for every window to pass over
    decoded tokens."""
    cfg = CASES[name][0]
    requests = {f"w{n}": tokens_for(cfg, n, 100 + n) for n in (1, 2, 37, 200)}
    runner = runner_for(folders[name], dtype)
    check_trace(runner, folders[name], requests, trace_whole(requests), dtype, f"{name}/whole")
    del requests["w1"], requests["w2"]
    check_trace(runner, folders[name], requests, trace_tail(requests, tail=70), dtype, f"{name}/decode")


def test_prefill_equals_token_by_token(folders):
    """A prompt fed one token a step from its first token on (state and cache carry everything) against the whole prompt."""
    name = "A"
    toks = tokens_for(CASES[name][0], 60, 5)
    runner = runner_for(folders[name], "float32")
    steps = [{"step": i, "entries": [{"id": "s", "tokens": [t], "want": [0]}], "end": ["s"] if i == len(toks) - 1 else []}
             for i, t in enumerate(toks)]
    compare(replay_in_process(runner, steps)["s"], folders[name], toks, "float32", "token by token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_portions_down_to_two_tokens(folders, name, dtype):
    cfg = CASES[name][0]
    requests = {"p0": tokens_for(cfg, 170, 1), "p1": tokens_for(cfg, 45, 2)}
    runner = runner_for(folders[name], dtype, graphs=False)
    check_trace(runner, folders[name], requests, trace_portions(requests), dtype, f"{name}/portions")
    check_trace(runner, folders[name], requests, trace_portions(requests, sizes=(2, 3, 1, 2, 4)), dtype, f"{name}/small portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("A", 16), ("B", 16), ("C", 8), ("D", 32), ("E", 16)])
def test_mixed_batches_with_pages_and_slots_used_again(folders, name, page, dtype):
    """Up to three live requests of unequal lengths, portions beside single tokens, in a pool that holds less than the
    sum of the requests and has three state slots: every request's logits are those of the request alone."""
    cfg = CASES[name][0]
    lens = [140, 3, 64, 97, 1, 33, 110, 18]
    requests = {f"m{i}": tokens_for(cfg, n, 50 + i) for i, n in enumerate(lens)}
    max_tokens = 384
    runner = runner_for(folders[name], dtype, max_tokens=max_tokens, max_requests=3, page_size=page)
    handed = count_page_handouts(runner.cache) if runner.cache.groups else None
    steps = trace_mixed(requests, max_tokens, seed=3, max_live=3, tail=20)
    check_trace(runner, folders[name], requests, steps, dtype, f"{name}/mixed")
    if handed is not None:
        assert max(handed.values()) >= 2, "no page was used a second time"


def test_a_slot_used_again_starts_from_zero(folders):
    """The same request twice through the same state slot, with another request's state left there in between."""
    name = "B"
    cfg = CASES[name][0]
    runner = runner_for(folders[name], "float32", max_requests=1)
    for seed in (1, 2, 1):
        toks = tokens_for(cfg, 50, seed)
        check_trace(runner, folders[name], {"r": toks}, trace_tail({"r": toks}, tail=10), "float32", f"slot/{seed}")


def test_window_edges_show_in_the_logits(folders):
    """The comparison is sharp enough to see a window that is one key off: the plain implementation with every window
    one longer or one shorter differs from the engine by far more than the bound, at prompt rows and at decoded ones."""
    name = "A"
    cfg, tensors = read_folder(folders[name])
    toks = tokens_for(cfg, 110, 9)
    runner = runner_for(folders[name], "float32")
    got = replay_in_process(runner, trace_tail({"e": toks}, tail=60))["e"].double()
    ref = oracle(folders[name], toks)
    compare(got, folders[name], toks, "float32", "edges")
    scale = ref.pow(2).mean().sqrt().item()
    for d in (-1, 1):
        off = json.loads(json.dumps(cfg))
        off["layers"][0]["mixer"]["left"]["mask"]["size"] += d
        wrong = plain.forward(off, tensors, toks)
        assert (got[30:50] - wrong[30:50]).abs().max().item() > 1e-3 * scale, "a window one key off would not be noticed in a prompt"
        assert (got[60:] - wrong[60:]).abs().max().item() > 1e-3 * scale, "a window one key off would not be noticed while decoding"
        assert (ref[:15] - wrong[:15]).abs().max().item() < 1e-9             # before the window is full the two agree


def test_far_keys_and_old_state_reach_the_last_token(folders):
    """The layer without a window and the recurrences carry the first tokens to the end, also while decoding: with the
    first token changed, the plain implementation's last logits move, and the engine follows the right one."""
    name = "A"
    cfg, tensors = read_folder(folders[name])
    toks = tokens_for(cfg, 300, 21)
    runner = runner_for(folders[name], "float32")
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:200], "want": []}], "end": []}]
    steps += [{"step": 1 + i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": ["x"] if i == 99 else []}
              for i, t in enumerate(toks[200:])]
    got = replay_in_process(runner, steps)["x"].double()
    ref = oracle(folders[name], toks)[200:]
    compare(got, folders[name], toks, "float32", "far keys", rows=slice(200, None))
    other = plain.forward(cfg, tensors, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])[200:]
    assert (ref - other).abs().max().item() > 100 * (got - ref).abs().max().item(), "the first token would not be missed"


def test_a_far_key_among_hundreds_reaches_the_attention(tmp_path):
    """Attention alone (the other side switched off), no window, a sharp softmax: a row's weight sits on the few keys
    that match it best, wherever they are among 300. The engine follows the plain implementation while decoding, and a
    plain implementation that sees only the last 200 keys does not."""
    cfg = _one_layer(parallel(attn(4, 2, 16, 24, 1.2, rot={"dims": 8, "base": 10000.0}), delta(1, 1, 8, 8, 2), 1.0, 0.0, dense(64, 2.0)))
    path = make_folder(str(tmp_path / "far"), cfg, 11)
    raw, tensors = read_folder(path)
    toks = tokens_for(cfg, 300, 5)
    runner = runner_for(path, "float32", max_tokens=512)
    got = replay_in_process(runner, trace_tail({"f": toks}, tail=60))["f"].double()
    ref = oracle(path, toks)
    compare(got, path, toks, "float32", "far key")
    near = json.loads(json.dumps(raw))
    near["layers"][0]["mixer"]["left"]["mask"] = {"size": 200}
    wrong = plain.forward(near, tensors, toks)
    scale = ref.pow(2).mean().sqrt().item()
    assert (ref[240:] - wrong[240:]).abs().max().item() > 1e-2 * scale, "lost far keys would not be noticed"
    assert (got[240:] - ref[240:]).abs().max().item() < 1e-4 * scale


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_scheduler(folders, name):
    from openinfer_b200 import LLM, SamplingParams
    cfg, tensors = read_folder(folders[name])
    prompts = [tokens_for(cfg, n, 70 + n) for n in (1, 9, 33, 70)]
    n_new = 20

    def greedy(prompt):
        toks = list(prompt)
        for _ in range(n_new):
            toks.append(int(plain.forward(cfg, tensors, toks)[-1].argmax()))
        return toks[len(prompt):]

    want = [greedy(p) for p in prompts]
    llm = LLM(folders[name], dtype="float32", max_cache_tokens=512, max_prefill_tokens=13, max_decode_batch=3)
    assert llm.generate(prompts, max_tokens=n_new) == want
    assert llm.runner.cache.min_free_pages() == llm.runner.cache.num_pages
    assert [llm.generate([p], max_tokens=n_new)[0] for p in prompts] == want
    llm16 = LLM(folders[name], dtype="bfloat16", max_cache_tokens=512, max_decode_batch=4)
    sp = SamplingParams(temperature=0.8, top_k=20, top_p=0.9, seed=5)
    a = llm16.generate(prompts, sp, max_tokens=12)
    assert a == llm16.generate(prompts, sp, max_tokens=12) and all(len(t) == 12 for t in a)
    assert llm16.runner.cache.slot_pool.used_count == 0


def test_long_decoding(folders):
    """600 single-token steps behind a short prompt: states, windows and released pages over a long run."""
    name = "D"
    cfg = CASES[name][0]
    toks = tokens_for(cfg, 620, 77)
    runner = runner_for(folders[name], "float32", max_tokens=320)     # the windows give pages back: 320 positions hold 620
    got = replay_in_process(runner, trace_tail({"l": toks}, tail=600))["l"]
    compare(got, folders[name], toks, "float32", "long decoding")


def test_command_line_and_trace_program(folders, tmp_path):
    name = "C"
    cfg, tensors = read_folder(folders[name])
    toks = [7, 8, 9]
    want = []
    for _ in range(5):
        want.append(int(plain.forward(cfg, tensors, toks + want)[-1].argmax()))
    out = subprocess.run([sys.executable, "-m", "openinfer_b200", "--model-path", folders[name], "--dtype", "float32",
                          "--prompt-ids", "7,8,9", "--max-tokens", "5", "--num-pages", "32"],
                         cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["token_ids"] == want and line["finish_reason"] == "length"
    requests = {f"t{i}": tokens_for(cfg, n, 30 + i) for i, n in enumerate([80, 5, 130, 41, 1])}
    max_tokens = round64(130) + round64(80) + 64
    steps = trace_mixed(requests, max_tokens, seed=1, max_live=4, tail=16)
    for dtype in DTYPES:
        got = replay_trace_run(folders[name], dtype, steps, str(tmp_path / dtype), max_tokens, cfg["vocab"])
        for rid, t in requests.items():
            compare(got[rid], folders[name], t, dtype, f"trace_run/{dtype}/{rid}")


@pytest.mark.parametrize("rows", [1, 8, 32, 33, 100, 128, 300, 2100])
def test_clamped_feed_forward_with_the_activation_in_the_products_epilogue(rows):
    """bfloat16 at sizes the tensor-core products take: up to 32 rows the weight stream forms the clamped activation where
    it adds up its K slices, from 128 rows the tcgen05 tiles in their epilogue (pairs of CTAs from 2,048 rows); between
    them, and at sizes they refuse, the plain product and the activation kernel. All against the plain feed-forward."""
    from openinfer_b200.parts.mlp import GatedMlp
    from openinfer_b200.parts.spec import GatedMlpSpec
    from openinfer_b200.kernels import gemm_tcgen05, linear
    g = torch.Generator().manual_seed(rows)
    for hidden, inter, limit in ((256, 768, 1.5), (128, 256, 0.5), (72, 100, 2.0)):
        part = GatedMlp(GatedMlpSpec(hidden_size=hidden, intermediate_size=inter, activation="swiglu_clamp", limit=limit,
                                     gate_name="gate", up_name="up", down_name="down"))
        w = {"gate": torch.randn(inter, hidden, generator=g) * hidden ** -0.5, "up": torch.randn(inter, hidden, generator=g) * hidden ** -0.5,
             "down": torch.randn(hidden, inter, generator=g) * inter ** -0.5}
        w = {k: v.to(torch.bfloat16) for k, v in w.items()}
        part.load({k: _dev(v) for k, v in w.items()})
        x = (torch.randn(rows, hidden, generator=g) * 2.0).to(torch.bfloat16)
        got = part.forward(_dev(x), None, out_dtype=torch.float32)
        assert got.dtype == torch.float32
        ref = plain.clamped_glu(x.double(), w["gate"].double(), w["up"].double(), w["down"].double(), limit)
        err = (got.double().cpu() - ref).abs().max().item() / ref.abs().max().item()
        assert err < 2e-2, f"rows {rows} hidden {hidden}: {err}"
    assert gemm_tcgen05.status() == 0 and linear.stream_status() == 0
