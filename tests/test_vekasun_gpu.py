"""The Vekasun design in the engine against the plain whole-sequence implementation
(`plain_vekasun`): each mechanism alone, whole prompts, token-by-token decoding, portions down
to two tokens, unequal requests in one batch, pages and state slots used again, long decoding,
and greedy generation through the entry point.  Random weights are scaled out of their nearly
linear range, and where a fault would still hide (a far key, the sink, the first tokens) the
weights are made so that it shows."""

import json
import math
import os

import pytest
import torch

import plain_vekasun as PV
import schedules
import vekasun_configs as VC
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu

LENGTHS = [70, 5, 131, 33, 2, 97]


def options(dtype, **kw):
    from ninfer_amd_mi50_b200.config import EngineOptions
    base = dict(dtype=dtype, page_size=16, num_sequences=4, max_context=256, cache_tokens=1024, use_graph=False)
    base.update(kw)
    return EngineOptions(**base)


def run(runner, steps):
    """Drive the runner through a schedule -> (logits per request, experts chosen per request and
    layer run [tokens, top])."""
    from ninfer_amd_mi50_b200.engine import StepEntry
    from ninfer_amd_mi50_b200.parts.feedforward import SparseMoeSwiglu
    sparse_runs = [r for r, c in enumerate(runner.model.order)
                   if isinstance(runner.model.blocks[c.layer].feed_forward, SparseMoeSwiglu)]
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
        assert len(record) == len(sparse_runs)
        r = row = 0
        for e in st["entries"]:
            n = len(e["want"])
            got.setdefault(e["id"], []).append(out[r:r + n].double().cpu())
            r += n
            for rn, idx in zip(sparse_runs, record):
                chosen.setdefault(e["id"], {}).setdefault(rn, []).append(idx[row:row + len(e["tokens"])].long().cpu())
            row += len(e["tokens"])
        for rid in st["end"]:
            runner.close(rid)
        runner.cache.check()
    from ninfer_amd_mi50_b200 import kernels
    kernels.check_status("schedule")
    return ({k: torch.cat(v) for k, v in got.items()},
            {k: {rn: torch.cat(v) for rn, v in runs.items()} for k, runs in chosen.items()})


def compare(got, want, dtype, what, bf16_bound=8e-2):
    """float32 is the sharp comparison: 1e-4 of the largest logit for every row (measured: about
    1e-6).  bfloat16 rounds every activation between kernels to 8 bits; with weights scaled out of
    their linear range the worst row of a hundred reaches 3 % here, the typical row 0.3 %: every
    row within 8 %, the median row within 1.5 %."""
    scale = want.abs().max().item()
    err = (got - want).abs().max(dim=1).values / scale
    bound = 1e-4 if dtype == "float32" else bf16_bound
    assert err.max().item() <= bound, f"{what}: row {int(err.argmax())} of {len(err)} differs by {err.max().item():.3e} of the scale"
    if dtype != "float32":
        assert err.median().item() <= 1.5e-2, f"{what}: the median row differs by {err.median().item():.3e} of the scale"
    return err.max().item()


def expected(cfg, w, tokens, dtype, chosen):
    """float32: the plain model's own logits.  bfloat16: the plain model with the experts the
    engine chose (a rounding of the router's input flips near-ties, which is no fault)."""
    return PV.forward(cfg, w, tokens, forced=None if dtype == "float32" else chosen)


@pytest.fixture(scope="module", params=sorted(VC.CONFIGS))
def folder(request, tmp_path_factory):
    cfg, seed = VC.CONFIGS[request.param]
    d = str(tmp_path_factory.mktemp("vekasun") / request.param)
    VC.write_folder(cfg, seed, d, scale=VC.LIVELY)
    cfg, w = VC.read_folder(d)
    reqs = {f"r{i}": random_tokens(n, cfg["vocab"], 700 + i) for i, n in enumerate(LENGTHS)}
    return request.param, d, cfg, w, reqs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "tail", "portions", "mixed"])
def test_every_way_of_cutting_matches_the_plain_model(folder, dtype, how):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    make = {"whole": schedules.whole, "tail": lambda r: schedules.tail_decoded(r, tail=20),
            "portions": schedules.portions,
            # a pool of 320 tokens for 338 in all, three slots for six requests: pages and slots come back
            "mixed": lambda r: schedules.mixed(r, max_live=3, page=16, pool_tokens=320, tail=9)}[how]
    pool = 320 if how == "mixed" else 1024
    runner = load_runner(d, options=options(dtype, cache_tokens=pool, num_sequences=3 if how == "mixed" else 4))
    got, chosen = run(runner, make(reqs))
    assert all(n == pool // 16 for n in runner.cache.pages_free())
    for r, toks in reqs.items():
        compare(got[r], expected(cfg, w, toks, dtype, chosen[r]), dtype, f"{name} {how} {r}")


def test_the_plan_gives_every_run_of_a_layer_its_own_cache_and_state(folder):
    from ninfer_amd_mi50_b200.engine.loading import build_model
    name, d, cfg, w, reqs = folder
    typed, model = build_model(cfg)
    runs = PV.layer_runs(cfg)
    assert [c.layer for c in model.order] == [i for i, _ in runs]
    assert len({c.cache for c in model.order}) == len(runs) and len({c.state_slot() for c in model.order}) == len(runs)
    for c, (i, t) in zip(model.order, runs):
        first = t is not None and i == cfg["loop"]["start"]
        assert c.add_vector == (("loop.step", t) if first else None)
    kinds = [cfg["layers"][i]["type"] for i, _ in runs]
    assert [s is not None for s in model.cache_specs()[:len(runs)]] == [k == "latent_attention" for k in kinds]
    assert [s is not None for s in model.state_specs()[:len(runs)]] == [k == "mamba2" for k in kinds]


# ---- each mechanism alone ---------------------------------------------------------------------

def one_layer(kind, mixer, mlp=None, width=96, vocab=113, eps=1e-5, loop=None):
    c = {"architecture": "Vekasun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": 1.0,
         "layers": [{"type": kind, "mixer": mixer, "mlp": mlp}]}
    if loop:
        c["loop"] = loop
    return c


def run_alone(cfg, d, tokens, dtype, cuts=None, **opt):
    from ninfer_amd_mi50_b200.engine import load_runner
    runner = load_runner(d, options=options(dtype, **opt))
    reqs = {"a": tokens}
    steps = schedules.whole(reqs) if cuts is None else schedules.portions(reqs, cuts=cuts)
    got, chosen = run(runner, steps)
    return got["a"], chosen.get("a", {})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_norm_takes_the_mean_off(dtype):
    from ninfer_amd_mi50_b200 import kernels
    torch.manual_seed(3)
    h = (torch.randn(9, 200) * 3 + 50.0).cuda()          # a large common offset: an RMS norm would show it
    delta = torch.randn(9, 200).cuda().to(getattr(torch, dtype))
    w = (1 + 0.1 * torch.randn(200)).cuda()
    out = torch.empty((9, 200), dtype=getattr(torch, dtype), device="cuda")
    want_h = h.double().cpu() + delta.double().cpu()
    kernels.add_layernorm(h, delta, None, w, 1e-5, out)
    want = PV.layer_norm(want_h, w.double().cpu(), 1e-5)
    assert (h.double().cpu() - want_h).abs().max() < 1e-4
    assert (out.double().cpu() - want).abs().max() < (2e-4 if dtype == "float32" else 3e-2)
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device="cuda")
    out2 = torch.empty((3, 200), dtype=getattr(torch, dtype), device="cuda")
    kernels.add_layernorm(h, None, rows, w, 1e-5, out2)
    assert (out2.double().cpu() - want[[7, 0, 3]]).abs().max() < (2e-4 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("rows", [3, 40, 300])
def test_sigmoid_scores_choose_and_weigh(rows):
    """The chosen experts are those of the largest sigmoid; their weights are the scores as they
    are (no softmax, no division by their sum); every row count's kernel agrees."""
    from ninfer_amd_mi50_b200 import kernels
    torch.manual_seed(rows)
    E, k, H = 7, 3, 64
    x = torch.randn(rows, H).cuda()
    wr = (torch.randn(E, H) * 0.3).cuda()
    idx, wts, _, plan = kernels.route(x, wr, E, k, False, scoring="sigmoid")
    want_idx, want_w = PV.route_sigmoid_top(x.double().cpu(), wr.double().cpu(), k)
    assert torch.equal(idx.long().cpu(), want_idx)
    assert (wts.double().cpu() - want_w).abs().max() < 1e-5
    assert float(wts.sum(dim=1).max()) > 1.05            # sums of sigmoids, not of a softmax


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("top,experts", [(1, 4), (2, 6), (5, 5)])
def test_the_weight_multiplies_the_experts_input(tmp_path, dtype, top, experts):
    """expert(w h), not w expert(h): with scores far from 1 and lively experts the two differ widely."""
    mix = VC.state_space(2, 16, 8, 1, 2, 1)
    cfg = one_layer("mamba2", mix, VC.moe(40, experts, top))
    d = VC.write_folder(cfg, 31, str(tmp_path / "m"), scale={".router": 30.0, ".gate": 12.0, ".up": 12.0, ".down": 12.0})
    cfg, w = VC.read_folder(d)
    toks = random_tokens(50, cfg["vocab"], 1)
    got, chosen = run_alone(cfg, d, toks, dtype)
    compare(got, expected(cfg, w, toks, dtype, chosen), dtype, "input-weighted experts")
    # the other reading is far away
    x = PV.layer_norm(w["embed"][toks] + PV.mamba2(PV.layer_norm(w["embed"][toks], w["l0.norm1"], 1e-5), w, "l0.mix.", mix, 1e-5),
                      w["l0.norm2"], 1e-5)
    idx, wts = PV.route_sigmoid_top(x, w["l0.mlp.router"], top)
    assert float(wts.min()) < 0.5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,groups,norm_groups,state", [(4, 2, 2, 24), (1, 1, 1, 16), (7, 4, 4, 40), (3, 1, 2, 130)])
def test_state_space_mixer_alone_whole_and_in_portions(tmp_path, dtype, taps, groups, norm_groups, state):
    cfg = one_layer("mamba2", VC.state_space(4, 12, state, groups, taps, norm_groups), width=80)
    # decays between about 0.1 and 0.97 a token, step sizes of every size, a skip that matters
    H = 4
    rep = {"l0.mix.A_log": torch.linspace(-2.0, 1.0, H), "l0.mix.dt_bias": torch.linspace(-3.0, 1.5, H),
           "l0.mix.D": torch.linspace(-1.0, 2.0, H)}
    d = VC.write_folder(cfg, 40 + taps, str(tmp_path / "m"), replace=rep, scale={".mix.in": 5.0, ".mix.conv": 12.0, ".mix.o": 5.0})
    cfg, w = VC.read_folder(d)
    toks = random_tokens(90, cfg["vocab"], 2)
    want = PV.forward(cfg, w, toks)
    for cuts in (None, [17, 2, 40, 3, 1, 1, 26], [1] * 90, [2] * 45):
        got, _ = run_alone(cfg, d, toks, dtype, cuts)
        compare(got, want, dtype, f"state-space mixer cut {cuts and cuts[:3]}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,rot_dim,dims,vdim,kv_rank,q_rank", [(3, 16, 16, 16, 24, 32, 40), (1, 8, 24, 6, 8, 20, 12),
                                                                      (6, 32, 8, 8, 16, 64, 48), (2, 24, 0, 0, 40, 48, 16)])
def test_latent_attention_alone_with_a_sink_that_matters(tmp_path, dtype, heads, dim, rot_dim, dims, vdim, kv_rank, q_rank):
    mix = VC.attention(heads, dim, rot_dim, vdim, kv_rank, q_rank, 1.0 / math.sqrt(dim + rot_dim), 900.0, dims)
    cfg = one_layer("latent_attention", mix, width=72)
    # sinks from "takes most of the mass" to "nothing"
    rep = {"l0.mix.sink": torch.linspace(3.0, -4.0, heads) if heads > 1 else torch.tensor([2.0])}
    d = VC.write_folder(cfg, 50 + heads, str(tmp_path / "m"), replace=rep,
                        scale={".mix.uq": 12.0, ".mix.uk": 8.0, ".mix.dkv": 4.0, ".mix.dq": 3.0, ".mix.g": 15.0, ".mix.uv": 5.0, ".mix.o": 5.0})
    cfg, w = VC.read_folder(d)
    toks = random_tokens(77, cfg["vocab"], 3)
    want = PV.forward(cfg, w, toks)
    for cuts in (None, [16, 1, 15, 2, 30, 13], [1] * 77):
        got, _ = run_alone(cfg, d, toks, dtype, cuts)
        compare(got, want, dtype, f"latent attention cut {cuts and cuts[:3]}")
    # and the sink does matter here: without it the first head's output would be several times larger
    no_sink = dict(w)
    no_sink["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -1e4)
    assert (PV.forward(cfg, no_sink, toks) - want).abs().max() > 0.05 * want.abs().max()


@pytest.mark.parametrize("heads,dim,rot_dim,dims,vdim,kv_rank,q_rank", [(3, 16, 16, 16, 24, 64, 40), (40, 8, 32, 16, 8, 128, 24),
                                                                      (16, 32, 0, 0, 16, 192, 32), (5, 24, 48, 48, 32, 256, 48)])
def test_latent_attention_on_tensor_cores(tmp_path, heads, dim, rot_dim, dims, vdim, kv_rank, q_rank):
    """Latent widths that are multiples of 64 take the tensor-core kernel in bfloat16 (tiles of 32
    (token, head) pairs, key blocks of 64, long contexts split and merged): whole, in portions that
    end inside and on key blocks, token by token, and in a batch of unequal requests - against the
    plain model, and against the engine's plain kernel."""
    from ninfer_amd_mi50_b200 import kernels
    from ninfer_amd_mi50_b200.engine import load_runner
    assert kernels.lib.load().nf_latent_attention_mma_fits(kv_rank, rot_dim, dim + rot_dim, dim, heads * (dim + rot_dim))
    mix = VC.attention(heads, dim, rot_dim, vdim, kv_rank, q_rank, 1.5 / math.sqrt(dim + rot_dim), 900.0, dims)
    cfg = one_layer("latent_attention", mix, width=72)
    rep = {"l0.mix.sink": torch.linspace(2.0, -3.0, heads)}
    d = VC.write_folder(cfg, 70 + heads, str(tmp_path / "m"), replace=rep,
                        scale={".mix.uq": 12.0, ".mix.uk": 8.0, ".mix.dkv": 4.0, ".mix.dq": 3.0, ".mix.g": 15.0, ".mix.uv": 5.0, ".mix.o": 5.0})
    cfg, w = VC.read_folder(d)
    toks = random_tokens(330, cfg["vocab"], 5)
    want = PV.forward(cfg, w, toks)
    for cuts in (None, [63, 1, 64, 2, 130, 70], [200] + [1] * 130):
        got, _ = run_alone(cfg, d, toks, "bfloat16", cuts, max_context=384)
        compare(got, want, "bfloat16", f"tensor-core latent attention cut {cuts and cuts[:3]}")
    reqs = {f"r{i}": random_tokens(n, cfg["vocab"], 80 + i) for i, n in enumerate([129, 7, 64, 200])}
    runner = load_runner(d, options=options("bfloat16", max_context=256))
    got, _ = run(runner, schedules.mixed(reqs, max_live=4, page=16, tail=6))
    kernels.TUNING["bf16_attention"] = "generic"
    try:
        plain, _ = run(runner, schedules.mixed(reqs, max_live=4, page=16, tail=6))
    finally:
        kernels.TUNING["bf16_attention"] = "auto"
    for r, t in reqs.items():
        ref = PV.forward(cfg, w, t)
        compare(got[r], ref, "bfloat16", f"tensor-core latent attention, batch, {r}")
        compare(plain[r], ref, "bfloat16", f"plain latent attention, batch, {r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_far_key_among_hundreds_is_found_across_pages_and_portions(tmp_path, dtype):
    """In a one-layer model a token's query and key depend on the token alone (and, in the rotated
    slice, on its place), so the pair of tokens (A, B) whose unrotated score is the largest of all
    can be looked up; with a large scale B's softmax then rests on the one A in the prompt.  A B
    placed right after the only A, a page later and hundreds of positions later must bring A's
    value back, whatever pages lie between and however the prompt is cut."""
    mix = VC.attention(2, 16, 8, 16, 32, 24, 3.0, 1000.0, 8)
    cfg = one_layer("latent_attention", mix, width=64, vocab=64)
    d0 = VC.write_folder(cfg, 61, str(tmp_path / "m0"), scale={".mix.uq": 8.0, ".mix.uk": 8.0, ".mix.dkv": 4.0, ".mix.uv": 6.0, ".mix.o": 6.0})
    cfg, w = VC.read_folder(d0)
    h = PV.layer_norm(w["embed"], w["l0.norm1"], 1e-5)
    q = PV.lin(PV.rms_unit(PV.lin(h, w["l0.mix.dq"]), 1e-5) * w["l0.mix.dq.norm"], w["l0.mix.uq"]).reshape(64, 2, 24)[:, 0, :16]
    c = PV.rms_unit(PV.lin(h, w["l0.mix.dkv"])[:, :32], 1e-5) * w["l0.mix.dkv.norm"]
    k = PV.lin(c, w["l0.mix.uk"]).reshape(64, 2, 16)[:, 0]
    score = q @ k.T
    score.fill_diagonal_(-1e9)
    B, A = divmod(int(score.argmax()), 64)
    filler = [t for t in range(64) if t not in (A, B) and float(score[B, t]) < float(score[B, A]) - 2.0]
    toks = [filler[t % len(filler)] for t in random_tokens(300, 64, 4)]
    for place in (3, 15, 16, 31, 32, 47):                # A at page borders (pages of 16) and inside
        seq = list(toks)
        seq[place] = A
        for b in (place + 1, place + 17, 250, 299):
            seq[b] = B
        want = PV.forward(cfg, w, seq)
        for cuts in (None, [place + 1, 2, 13, 64, 200, 20], [5, 11, 16, 1, 15, 100, 99, 53]):
            got, _ = run_alone(cfg, d0, seq, dtype, cuts, max_context=320)
            compare(got, want, dtype, f"far key at {place}, cut {cuts and cuts[:3]}")
    # the oracle itself rests on the far key: the last B's logits move when A is taken away
    seq2 = list(seq)
    seq2[place] = filler[0]
    assert (PV.forward(cfg, w, seq2)[299] - want[299]).abs().max() > 0.02 * want.abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(folder, dtype):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    toks = random_tokens(230, cfg["vocab"], 9)
    runner = load_runner(d, options=options(dtype, num_sequences=1, cache_tokens=256))
    got, chosen = run(runner, schedules.tail_decoded({"a": toks}, tail=229))     # one token, then 229 one by one
    compare(got["a"], expected(cfg, w, toks, dtype, chosen["a"]), dtype, f"{name}: 229 decoded tokens")


def test_a_slot_that_is_used_again_starts_from_nothing(folder):
    """The same request run a second time in the slot and pages that another, longer request has
    just left gives the same bits."""
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    runner = load_runner(d, options=options("float32", num_sequences=1, cache_tokens=160, max_context=160))
    a, b = reqs["r0"], reqs["r2"]
    first, _ = run(runner, schedules.portions({"a": a}))
    run(runner, schedules.portions({"b": b}))
    again, _ = run(runner, schedules.portions({"a": a}))
    assert torch.equal(first["a"], again["a"])


def test_unequal_requests_in_one_batch_equal_each_alone(folder):
    """float32: a request's logits in a mixed batch are those of the request alone, to rounding."""
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    runner = load_runner(d, options=options("float32"))
    together, _ = run(runner, schedules.mixed(reqs, max_live=4, page=16, tail=5))
    for r, toks in reqs.items():
        alone, _ = run(runner, schedules.whole({r: toks}))
        compare(together[r], alone[r], "float32", f"{name} {r} in a batch")


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
            lg = PV.forward(cfg, w, seq)[-1]
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
            assert torch.equal(arr[at:at + n], got[e["id"]][rows[e["id"]]:rows[e["id"]] + n])
            at += n
            rows[e["id"]] += n


@pytest.mark.parametrize("how", ["folder", "seed"])
def test_the_command_line_generates_from_the_design(tmp_path, how):
    """`bin/ninfer` on a Vekasun folder, and on a folder with only config.json and a seed."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg0, seed = VC.CONFIGS["straight"]
    d = str(tmp_path / "m")
    VC.write_folder(cfg0, seed, d)
    cfg, w = VC.read_folder(d)
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
        lg = PV.forward(cfg, w, seq)[-1]
        assert float(lg[t]) >= float(lg.max()) - 1e-4 * float(lg.abs().max())
        seq.append(t)
