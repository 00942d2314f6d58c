"""The Difavik design in the engine against the plain whole-sequence implementation
(`plain_difavik`): each mechanism alone, whole prompts, token-by-token decoding, portions down to
two tokens, unequal requests in one batch, pages and state slots used again, long decoding, and
greedy generation through the entry point.  Random weights are scaled out of their nearly linear
range, and where a fault would still hide (a far key, a window's edge, the kept first tokens) the
inputs are made so that it shows."""

import json
import math
import os

import pytest
import torch

import difavik_configs as DC
import plain_difavik as PD
import schedules
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu

LENGTHS = [70, 5, 131, 33, 2, 97]


def options(dtype, **kw):
    from ninfer_amd_mi50_b200.config import EngineOptions
    base = dict(dtype=dtype, page_size=16, num_sequences=4, max_context=256, cache_tokens=1024, use_graph=False)
    base.update(kw)
    return EngineOptions(**base)


def run(runner, steps, routing=True):
    """Drive the runner through a schedule -> (logits per request, experts chosen per request: a
    list over the routed layer runs of [tokens, top]).  `routing` false: nothing is recorded (a step
    replayed from a graph runs no Python)."""
    from ninfer_amd_mi50_b200 import kernels
    from ninfer_amd_mi50_b200.engine import StepEntry
    from ninfer_amd_mi50_b200.parts.feedforward import SparseMoeSwiglu
    routed = sum(isinstance(runner.model.blocks[c.layer].feed_forward, SparseMoeSwiglu) for c in runner.model.order)
    got, chosen = {}, {}
    for st in steps:
        entries = []
        for e in st["entries"]:
            if not runner.cache.is_open(e["id"]):
                runner.open(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        SparseMoeSwiglu.record_routing = []
        try:
            out = runner.step(entries)
            record = SparseMoeSwiglu.record_routing
        finally:
            SparseMoeSwiglu.record_routing = None
        if not routing:
            record = []
        assert len(record) == (routed if routing else 0)
        r = row = 0
        for e in st["entries"]:
            n = len(e["want"])
            got.setdefault(e["id"], []).append(out[r:r + n].double().cpu())
            r += n
            per = chosen.setdefault(e["id"], [[] for _ in range(routed)])
            for k, idx in enumerate(record):
                per[k].append(idx[row:row + len(e["tokens"])].long().cpu())
            row += len(e["tokens"])
        for rid in st["end"]:
            runner.close(rid)
        runner.cache.check()
    kernels.check_status("schedule")
    return ({k: torch.cat(v) for k, v in got.items()}, {k: [torch.cat(v) for v in per] for k, per in chosen.items()} if routing else {})


def compare(got, want, dtype, what, bf16_bound=8e-2, touchy=None):
    """float32 is the sharp comparison: 1e-4 of the largest logit for every row.  bfloat16 rounds
    every activation between kernels to 8 bits: every row within 8 %, the median row (of a request
    of 16 rows or more) within 1.5 %.  `touchy` marks rows whose logits hang on a rounding (see
    `touchy_rows`); in bfloat16 they are only asked to be finite, and may be one row in ten."""
    scale = want.abs().max().item()
    err = (got - want).abs().max(dim=1).values / scale
    if dtype == "float32":
        assert err.max().item() <= 1e-4, f"{what}: row {int(err.argmax())} of {len(err)} differs by {err.max().item():.3e} of the scale"
        return err.max().item()
    assert torch.isfinite(got).all(), what
    if touchy is not None and touchy.any():
        assert int(touchy.sum()) <= len(err) // 10 + 1, f"{what}: {int(touchy.sum())} of {len(err)} rows hang on a rounding"
        err = err[~touchy]
        if len(err) == 0:
            return 0.0
    assert err.max().item() <= bf16_bound, f"{what}: row {int(err.argmax())} of {len(err)} differs by {err.max().item():.3e} of the scale"
    if len(err) >= 16:
        assert err.median().item() <= 1.5e-2, f"{what}: the median row differs by {err.median().item():.3e} of the scale"
    return err.max().item()


def touchy_rows(cfg, w, tokens, chosen, want, tries=3):
    """Rows whose logits move by more than 2 % of the scale when every projection's output is
    disturbed by 2^-9 of its size, in any of a few tries.  The design norms every sublayer's OUTPUT
    row by row: where a mixer's output nearly cancels (a request's first token, whose linear
    attention output is sign(q . k) v), the norm blows the rounding up with it."""
    scale = want.abs().max().item()
    out = torch.zeros(want.shape[0], dtype=torch.bool)
    try:
        for i in range(tries):
            PD.NOISE = (torch.Generator().manual_seed(50 + i), 2.0 ** -9)
            noisy = PD.forward(tokens, w, cfg, chosen=chosen)
            out |= (noisy - want).abs().max(dim=1).values / scale > 2e-2
    finally:
        PD.NOISE = None
    return out


def expected(cfg, w, tokens, dtype, chosen):
    """float32: the plain model's own logits.  bfloat16: the plain model with the experts the
    engine chose (a rounding of the router's input flips near-ties, which is no fault)."""
    return PD.forward(tokens, w, cfg, chosen=None if dtype == "float32" else chosen)


@pytest.fixture(scope="module", params=sorted(DC.CONFIGS))
def folder(request, tmp_path_factory):
    cfg, seed = DC.CONFIGS[request.param]
    d = str(tmp_path_factory.mktemp("difavik") / request.param)
    DC.write_folder(cfg, seed, d, scale=DC.LIVELY)
    cfg, w = DC.read_folder(d)
    reqs = {f"r{i}": random_tokens(n, cfg["vocab"], 900 + i) for i, n in enumerate(LENGTHS)}
    return request.param, d, cfg, w, reqs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "tail", "portions", "mixed"])
def test_every_way_of_cutting_matches_the_plain_model(folder, dtype, how):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    make = {"whole": schedules.whole, "tail": lambda r: schedules.tail_decoded(r, tail=40),
            "portions": schedules.portions,
            # a pool of 320 tokens for 338 in all, three slots for six requests: pages and slots come back
            "mixed": lambda r: schedules.mixed(r, max_live=3, page=16, pool_tokens=320, tail=9)}[how]
    pool = 320 if how == "mixed" else 1024
    runner = load_runner(d, options=options(dtype, cache_tokens=pool, num_sequences=3 if how == "mixed" else 4))
    got, chosen = run(runner, make(reqs))
    assert all(n == pool // 16 for n in runner.cache.pages_free())
    for r, toks in reqs.items():
        want = expected(cfg, w, toks, dtype, chosen[r])
        touchy = touchy_rows(cfg, w, toks, chosen[r], want) if dtype == "bfloat16" else None
        compare(got[r], want, dtype, f"{name} {how} {r}", touchy=touchy)


# ---- each mechanism alone ---------------------------------------------------------------------

def model_of(layers, width=96, vocab=113, eps=1e-5, bigram=None):
    c = {"architecture": "Difavik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if bigram:
        c["embedding"] = {"bigram": bigram}
    return c


def run_alone(cfg, d, tokens, dtype, cuts=None, **opt):
    from ninfer_amd_mi50_b200.engine import load_runner
    runner = load_runner(d, options=options(dtype, **opt))
    steps = schedules.whole({"a": tokens}) if cuts is None else schedules.portions({"a": tokens}, cuts=cuts)
    got, chosen = run(runner, steps)
    return got["a"], chosen["a"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("buckets,mul_prev,mul_cur", [(53, 17, 3), (1, 5, 5), (4001, 1000003, 999983)])
def test_the_pair_table_follows_the_previous_token_across_steps(tmp_path, dtype, buckets, mul_prev, mul_cur):
    """A model without layers' feed-forwards would still mix; here the table is large against the
    embedding, so a wrong row (or a first token that does not take the last row) shows at once."""
    cfg = model_of([{"type": "lightning", "mixer": DC.lightning(2, 8, 8, [0.5, 0.9]), "mlp": None}], vocab=1201,
                   bigram={"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur})
    d = DC.write_folder(cfg, 41, str(tmp_path / "m"), scale={"bigram": 40.0, ".ls1": 0.01})
    cfg, w = DC.read_folder(d)
    toks = random_tokens(45, cfg["vocab"], 5)
    rows = PD.pair_rows(toks, buckets, mul_prev, mul_cur)
    assert rows[0] == buckets and all(0 <= r < buckets for r in rows[1:])
    want = PD.forward(toks, w, cfg)
    for cuts in (None, [1], [2, 1, 7]):
        got, _ = run_alone(cfg, d, toks, dtype, cuts=cuts)
        compare(got, want, dtype, f"pair table cuts={cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,vdim,decay", [(3, 16, 24, [0.5, 0.9, 0.999]), (1, 40, 8, [0.97]), (2, 136, 20, [0.8, 1.0]),
                                                  (5, 4, 33, [0.1, 0.3, 0.5, 0.7, 0.9])])
def test_lightning_alone_whole_and_in_portions(tmp_path, dtype, heads, dim, vdim, decay):
    cfg = model_of([{"type": "lightning", "mixer": DC.lightning(heads, dim, vdim, decay), "mlp": None}])
    d = DC.write_folder(cfg, 42, str(tmp_path / "m"), scale={".q": 8.0, ".k": 8.0, ".v": 8.0, ".g": 15.0})
    cfg, w = DC.read_folder(d)
    toks = random_tokens(90, cfg["vocab"], 6)
    want = PD.forward(toks, w, cfg)
    for cuts in (None, [1], [2, 17, 3, 1]):
        got, _ = run_alone(cfg, d, toks, dtype, cuts=cuts)
        compare(got, want, dtype, f"lightning cuts={cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("side", ["left", "right"])
@pytest.mark.parametrize("left,right", [
    (DC.attention(4, 2, 16, 0.5, 7, 2), DC.retention(2, 16, 8, [0.9, 0.99], 100.0, 16)),
    (DC.attention(2, 2, 8, 0.9, 33, 0), DC.retention(3, 12, 20, [0.5, 0.75, 0.95], 10000.0, 4)),
    (DC.attention(6, 1, 24, 0.3, 16, 16), DC.retention(1, 64, 64, [0.9985], 5e5, 64)),
])
def test_each_side_of_the_parallel_mixer_alone(tmp_path, dtype, side, left, right):
    """The other side's weight after its norm is zero, so the mean holds one side only."""
    cfg = model_of([{"type": "parallel", "mixer": DC.parallel(left, right), "mlp": None}])
    other = "right" if side == "left" else "left"
    zero = {f"l0.mix.{other}.out": torch.zeros(cfg["width"])}
    d = DC.write_folder(cfg, 43, str(tmp_path / "m"), replace=zero,
                        scale={".q": 8.0, ".k": 8.0, ".v": 6.0, ".g": 20.0, ".q.b": 40.0, ".k.b": 40.0})
    cfg, w = DC.read_folder(d)
    toks = random_tokens(75, cfg["vocab"], 7)
    want = PD.forward(toks, w, cfg)
    for cuts in (None, [1], [2, 9, 1, 30]):
        got, _ = run_alone(cfg, d, toks, dtype, cuts=cuts)
        compare(got, want, dtype, f"{side} cuts={cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("limit", [0.25, 1.0, 7.0])
def test_dense_feed_forward_caps_and_biases(tmp_path, dtype, limit):
    cfg = model_of([{"type": "lightning", "mixer": DC.lightning(1, 8, 8, [0.9]), "mlp": DC.dense(88, limit)}])
    d = DC.write_folder(cfg, 44, str(tmp_path / "m"),
                        scale={".gate": 10.0, ".up": 10.0, ".gate.b": 50.0, ".up.b": 50.0, ".down.b": 30.0, ".ls1": 0.05})
    cfg, w = DC.read_folder(d)
    toks = random_tokens(40, cfg["vocab"], 8)
    x = PD.embed(toks, w, cfg)
    g = PD.lin(x, w["l0.mlp.gate"], w["l0.mlp.gate.b"])
    assert (g > limit).float().mean() > 0.02 or limit > 5            # the cap is met where it is low
    got, _ = run_alone(cfg, d, toks, dtype)
    compare(got, PD.forward(toks, w, cfg), dtype, f"dense limit={limit}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,rows", [(4, 1, 3), (6, 2, 40), (5, 5, 40), (9, 3, 300)])
def test_routed_experts_take_their_scores_as_they_are(tmp_path, dtype, experts, top, rows):
    """Softmax over all experts, the largest `top`, no renormalisation: with a lively router the
    chosen scores sum to well under one, so a renormalised sum would show."""
    cfg = model_of([{"type": "lightning", "mixer": DC.lightning(1, 8, 8, [0.9]), "mlp": DC.moe(24, 1.5, experts, top)}])
    d = DC.write_folder(cfg, 45, str(tmp_path / "m"), scale={".router": 15.0, ".gate": 8.0, ".up": 8.0, ".ls1": 0.05})
    cfg, w = DC.read_folder(d)
    toks = random_tokens(rows, cfg["vocab"], 9)
    record = []
    want = PD.forward(toks, w, cfg, record=record)
    s, sel = record[0]
    if top < experts:
        assert s.gather(1, sel).sum(dim=1).median() < 0.95
    got, chosen = run_alone(cfg, d, toks, dtype, max_context=512)
    if dtype == "float32":
        assert torch.equal(chosen[0].sort(dim=1).values, sel.sort(dim=1).values)
    compare(got, PD.forward(toks, w, cfg, chosen=None if dtype == "float32" else chosen), dtype, "routed")


# ---- the attention kernel on inputs made so that one key decides ------------------------------

def plain_attention_rows(q, keys, vals, pos, scale, slopes, window, keep_first):
    """q [H, D] at position `pos`; keys, vals [n, G, D] -> [H, D] by the design's rule."""
    H, D = q.shape
    G = keys.shape[1]
    out = torch.zeros((H, D), dtype=torch.float64)
    for h in range(H):
        g = h // (H // G)
        js = [j for j in range(pos + 1) if pos - j < window or j < keep_first]
        s = torch.tensor([float(q[h] @ keys[j, g]) * scale - float(slopes[h]) * (pos - j) for j in js], dtype=torch.float64)
        a = torch.softmax(s, dim=0)
        out[h] = sum(a[i] * vals[j, g] for i, j in enumerate(js))
    return out


@pytest.mark.parametrize("dtype,D,general", [(torch.float32, 16, True), (torch.bfloat16, 16, False), (torch.bfloat16, 64, False),
                                             (torch.bfloat16, 16, True), (torch.bfloat16, 24, True)])
@pytest.mark.parametrize("window,keep_first", [(37, 5), (16, 16), (17, 0), (64, 1), (3, 70)])
def test_one_loud_key_is_heard_just_inside_and_not_just_outside_every_edge(monkeypatch, dtype, D, general, window, keep_first):
    """The cache is filled by hand: every key is faint but one, whose score towers.  Placed just
    inside the window, on a page's border, among the kept first tokens or far back, it must take the
    whole output; placed just outside the window or just after the kept tokens it must not show.
    Rows are served both as a prompt's portion and as single decoded tokens, by the flash kernel
    (bfloat16, head sizes that are multiples of 16) and by the general one."""
    from ninfer_amd_mi50_b200 import kernels
    from ninfer_amd_mi50_b200.parts.base import StepContext
    dev = torch.device("cuda")
    if general and dtype == torch.bfloat16:
        monkeypatch.setitem(kernels.TUNING, "bf16_attention", "generic")      # the general kernel, not the flash one
    H, G, page, n = 4, 2, 16, 150
    gen = torch.Generator().manual_seed(3)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float32)
    pos = n - 1
    places = sorted({pos - window + 1, pos - window, pos - window - 1, keep_first - 1, keep_first, 0, pos, 15, 16, 63, 64, pos - 1}
                    - {-1, -2})
    places = [j for j in places if 0 <= j <= pos]
    for loud in places:
        keys = (torch.randn((n, G, D), generator=gen) * 0.05).to(dtype).double()
        vals = torch.randn((n, G, D), generator=gen).to(dtype).double()
        direction = torch.ones(D, dtype=torch.float64) / math.sqrt(D)
        keys[loud] = (direction * 30.0).to(dtype).double()
        q_all = (direction[None, None, :] * 2.0 + torch.randn((n, H, D), generator=gen).double() * 0.05).to(dtype)
        pages = torch.zeros((n // page + 2, 2, G, page, D), dtype=dtype)
        table = list(range(n // page + 1))[::-1]                       # pages in an order of their own
        for j in range(n):
            pages[table[j // page], 0, :, j % page] = keys[j].to(dtype)
            pages[table[j // page], 1, :, j % page] = vals[j].to(dtype)
        for first_row in (pos, pos - 9):                              # one decoded token; a portion of ten
            rows = list(range(first_row, pos + 1))
            T = len(rows)
            mk = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
            ctx = StepContext(dtype=dtype, device=dev, T=T, S=1, token_ids=mk([0] * T), positions=mk(rows), row_seg=mk([0] * T),
                              seg_row0=mk([0, T]), seg_pos0=mk([first_row]), seg_slot=mk([0]), logit_rows=mk([T - 1]),
                              seg_len_host=[T], seg_pos0_host=[first_row], max_rows_per_seg=T, max_context=n)
            q = q_all[rows].reshape(T, H * D).contiguous().to(dev)
            out = kernels.biased_window_attention(q, H, G, D, pages.to(dev), mk([table]), page, ctx, window, keep_first, 0.7,
                                                  slopes.to(dev)).double().cpu().reshape(T, H, D)
            for i, p in enumerate(rows):
                want = plain_attention_rows(q_all[p].double(), keys, vals, p, 0.7, slopes.double(), window, keep_first)
                tol = 1e-5 if dtype == torch.float32 else 2e-2
                assert (out[i] - want).abs().max() <= tol * max(1.0, want.abs().max()), (loud, p, window, keep_first)
            seen = (pos - loud < window) or loud < keep_first
            share = plain_attention_rows(q_all[pos].double(), keys, vals, pos, 0.7, slopes.double(), window, keep_first)
            if seen and pos - loud < 37:
                # the loud key takes (nearly) the whole output of the heads whose slope leaves it loud
                assert (share[H - 1] - vals[loud, G - 1]).abs().max() < 1e-3


# ---- state, slots, long decoding ----------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_lets_the_window_pass_over_decoded_tokens(folder, dtype):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    toks = random_tokens(236, cfg["vocab"], 77)
    runner = load_runner(d, options=options(dtype))
    got, chosen = run(runner, schedules.tail_decoded({"a": toks}, tail=229))
    want = expected(cfg, w, toks, dtype, chosen["a"])
    touchy = touchy_rows(cfg, w, toks, chosen["a"], want) if dtype == "bfloat16" else None
    compare(got["a"], want, dtype, f"{name} long decoding", touchy=touchy)
    assert all(n == 1024 // 16 for n in runner.cache.pages_free())


def test_a_slot_that_is_used_again_starts_from_nothing(folder):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    runner = load_runner(d, options=options("float32", num_sequences=1, cache_tokens=160))
    a, b = reqs["r0"], reqs["r3"]
    got, _ = run(runner, schedules.whole({"a": a}) + schedules.portions({"b": b}) + schedules.whole({"c": a}))
    compare(got["b"], PD.forward(b, w, cfg), "float32", f"{name} second user of the slot")
    assert torch.equal(got["a"], got["c"])


def test_unequal_requests_in_one_batch_equal_each_alone(folder):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    runner = load_runner(d, options=options("float32"))
    alone, _ = run(runner, schedules.whole(reqs))
    pick = {r: reqs[r] for r in ("r0", "r1", "r3", "r4")}
    step = [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in pick.items()], "end": list(pick)}]
    together, _ = run(runner, step)
    for r in pick:
        assert (together[r] - alone[r]).abs().max() <= 1e-5 * alone[r].abs().max(), r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_replayed_from_graphs_equal_host_driven_ones(folder, dtype):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    pick = {r: reqs[r][:40] for r in ("r0", "r2", "r5")}
    steps = [{"entries": [{"id": r, "tokens": t[:25], "want": [24]} for r, t in pick.items()], "end": []}]
    for i in range(25, 40):
        steps.append({"entries": [{"id": r, "tokens": t[i:i + 1], "want": [0]} for r, t in pick.items()],
                      "end": list(pick) if i == 39 else []})
    plain, _ = run(load_runner(d, options=options(dtype)), steps, routing=False)
    graphs, _ = run(load_runner(d, options=options(dtype, use_graph=True)), steps, routing=False)
    for r in pick:
        assert torch.equal(plain[r], graphs[r]), r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(folder, dtype):
    from ninfer_amd_mi50_b200.api import Ninfer
    name, d, cfg, w, reqs = folder
    prompts = [reqs["r1"], reqs["r3"], reqs["r4"], reqs["r0"][:40]]
    eng = Ninfer(d, max_context=128, prefill_chunk=16, num_sequences=3, dtype=dtype, page_size=16)
    got = eng.generate(prompts, max_new_tokens=10, temperature=0.0)
    for p, out in zip(prompts, got):
        assert len(out) == 10
        seq = list(p)
        for t in out:
            lg = PD.forward(seq, w, cfg)[-1]
            best = float(lg.max())
            # the engine's token is the plain model's, or (bfloat16) one whose logit is as good as ties go
            slack = 1e-4 if dtype == "float32" else 3e-2
            assert float(lg[t]) >= best - slack * float(lg.abs().max()), (name, len(seq), t, int(lg.argmax()))
            seq.append(t)


def test_trace_replay_program_runs_the_design(folder, tmp_path):
    """`bin/trace_run` picks the model class by config.json and gives the in-process logits."""
    import subprocess
    import sys
    import numpy as np
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    small = {r: reqs[r] for r in ("r1", "r3", "r0")}
    steps = schedules.mixed(small, max_live=2, page=64, pool_tokens=192, tail=4)
    lines = "".join(json.dumps({"step": i, **st}) + "\n" for i, st in enumerate(steps))
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "192"], input=lines, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    runner = load_runner(d, options=options("float32", page_size=64, cache_tokens=192, max_context=192))
    got, _ = run(runner, steps)
    rows = {r: 0 for r in small}
    for i, st in enumerate(steps):
        arr = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]).copy()).double()
        at = 0
        for e in st["entries"]:
            n = len(e["want"])
            assert torch.equal(arr[at:at + n], got[e["id"]][rows[e["id"]]:rows[e["id"]] + n]), (i, e["id"])
            at += n
            rows[e["id"]] += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,hidden,k", [(5, 96, 2), (70, 100, 1), (33, 2048, 4)])
def test_the_norm_that_adds_up_the_experts_rows_gives_the_separate_kernels_bits(dtype, rows, hidden, k):
    from ninfer_amd_mi50_b200 import kernels
    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(rows)
    y = torch.randn((rows * k, hidden), generator=gen).to(dtype).to(dev)
    wts = torch.rand((rows, k), generator=gen).to(dev)
    idx = torch.stack([torch.randperm(7, generator=gen)[:k] for _ in range(rows)]).to(torch.int32).to(dev)
    plan = kernels.moe_plan(idx, 7)
    w = (1.0 + 0.1 * torch.randn(hidden, generator=gen)).to(dev)
    ls = torch.randn(hidden, generator=gen).to(dev)
    h0 = torch.randn((rows, hidden), generator=gen).to(dev)
    out_dtype = None if dtype == torch.float32 else dtype
    h1, h2 = h0.clone(), h0.clone()
    x1 = kernels.scaled_norm_add(h1, kernels.moe_combine(y, plan, wts, None, None, dtype), None, w, ls, 1e-5, out_dtype)
    x2 = kernels.routed_scaled_norm_add(h2, y, plan.inv, wts, k, w, ls, 1e-5, out_dtype)
    assert torch.equal(h1, h2)
    if out_dtype is not None:
        assert torch.equal(x1, x2)
    # and against plain arithmetic
    d = torch.zeros((rows, hidden), dtype=torch.float64)
    inv = plan.inv.cpu().long().reshape(rows, k)
    for j in range(k):
        d += wts.cpu().double()[:, j:j + 1] * y.cpu().double()[inv[:, j]]
    d = d.to(dtype).double()
    want = h0.cpu().double() + d / torch.sqrt((d * d).mean(dim=1, keepdim=True) + 1e-5) * w.cpu().double() * ls.cpu().double()
    # (the sum is rounded to the experts' type before the norm: a bfloat16 step where the two sums straddle a rounding)
    assert (h1.cpu().double() - want).abs().max() <= (2e-5 if dtype == torch.float32 else 1e-2) * want.abs().max()


@pytest.mark.parametrize("how", ["folder", "seed"])
def test_the_command_line_generates_from_the_design(tmp_path, how):
    """`bin/ninfer` on a Difavik folder, and on a folder with only config.json and a seed."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg0, seed = DC.CONFIGS["borrowing"]
    d = str(tmp_path / "m")
    DC.write_folder(cfg0, seed, d)
    cfg, w = DC.read_folder(d)
    if how == "seed":
        os.remove(os.path.join(d, "model.safetensors"))
    prompt = random_tokens(30, cfg["vocab"], 12)
    cmd = [sys.executable, os.path.join(root, "bin", "ninfer"), d, "--prompt-ids", ",".join(map(str, prompt)),
           "--temperature", "0", "--max-new", "6", "--dtype", "fp32", "--prefill-chunk", "16", "--repeat-penalty", "1"]
    if how == "seed":
        cmd += ["--random-weights", str(seed)]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    got = [int(x) for x in p.stdout.split()]
    assert len(got) == 6
    seq = list(prompt)
    for t in got:
        lg = PD.forward(seq, w, cfg)[-1]
        assert float(lg[t]) >= float(lg.max()) - 1e-4 * float(lg.abs().max())
        seq.append(t)


def test_sampled_generation_and_a_request_preempted_and_recomputed(folder):
    """Sampling with a temperature through the scheduler, with a pool so small that a request is
    preempted and recomputed: the pair table's previous token and the linear attentions' states
    start again from nothing, and the tokens are those of a roomy pool."""
    from ninfer_amd_mi50_b200.api import Ninfer
    name, d, cfg, w, reqs = folder
    prompts = [reqs["r0"][:50], reqs["r3"], reqs["r5"][:60]]
    roomy = Ninfer(d, max_context=128, prefill_chunk=32, num_sequences=3, dtype="float32", page_size=16)
    want = roomy.generate(prompts, max_new_tokens=24, temperature=0.8, top_k=20, seed=5)
    tight = Ninfer(d, max_context=128, prefill_chunk=32, num_sequences=3, dtype="float32", page_size=16, cache_tokens=160)
    got = tight.generate(prompts, max_new_tokens=24, temperature=0.8, top_k=20, seed=5)
    assert got == want
