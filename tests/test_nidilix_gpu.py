"""The Nidilix decoder in the engine against the plain float64 implementation (``plain_nidilix``): each mechanism
alone, whole prompts against token-by-token decoding, portions down to two tokens, batches of unequal requests with
pages and state slots that are used again, keys far away and at page borders, the first tokens, long decoding, sizes
unlike one another (single head, one block, one tap, every expert chosen, fewer rotated entries than the rotated
part, no feed-forward, no token input, a borrowed cache), and greedy generation through the engine's scheduler."""

import copy

import pytest
import torch

import nidilix_cases as cases
import plain_nidilix as plain
import trace_modes as modes
from helpers import compare_logits, seeded_tokens, write_model_dir

pytestmark = pytest.mark.gpu
STORED = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def close(got, want, tol):
    got, want = got.double().cpu(), want.double().cpu()
    scale = float(want.abs().max())
    err = float((got - want).abs().max())
    assert err <= tol * scale, f"max abs error {err:.3e} against scale {scale:.3e}"


def rounded(state, dtype):
    return {k: v.to(STORED[dtype]) for k, v in state.items()}


def replay(folder, dtype, steps, want, page, slots, label, poison=True, min_ok=1.0):
    """Runs the steps through a fresh session and compares every wanted row. ``min_ok``: the share of rows that must
    pass (in bfloat16 a router's near-tie may fall the other way than in float64; float32 must pass everywhere)."""
    from stride_b200.engine.trace import TraceSession
    session = TraceSession(folder, dtype, max_tokens=modes.peak_tokens(steps), block_size=page, max_requests=slots)
    if poison:                  # whatever a page or a slot held before must not matter
        for t in session.device_cache.pages:
            t.fill_(float("nan"))
        for t in session.device_cache.states.values():
            t.fill_(float("nan"))
    rows = modes.expected_rows(steps)
    bad, total, first = 0, 0, None
    for s in steps:
        out = session.run_step(s)
        for r, (rid, pos) in enumerate(rows[s["step"]]):
            ok, msg = compare_logits(out[r:r + 1], want[rid][pos:pos + 1], dtype)
            total += 1
            if not ok:
                bad += 1
                first = first or f"{label}: step {s['step']}, request {rid!r}, position {pos}: {msg}"
    assert total and bad <= (1.0 - min_ok) * total, f"{bad} of {total} rows differ; first: {first}"
    stats = session.cache.stats()
    assert stats["live"] == 0 and session.cache.free_slots == session.cache.slot_capacity
    return session


def model_case(tmp_models, name, cfg, dtype, seed, lengths, **weights):
    state = cases.seeded_state(cfg, seed, **weights)
    folder = write_model_dir(str(tmp_models / f"nidilix_{name}_{dtype}_{seed}"), cfg, state, STORED[dtype])
    state = rounded(state, dtype)
    requests = {f"r{i}": seeded_tokens(n, cfg["vocab"], 50 * seed + i) for i, n in enumerate(lengths)}
    want = {rid: plain.forward(cfg, state, toks) for rid, toks in requests.items()}
    return folder, requests, want


# ------------------------------------------------------------------------------------------------ mechanisms
@pytest.mark.parametrize("dtype,tol", [("float32", 3e-6), ("bfloat16", 2e-2)])
def test_dynamic_tanh_with_a_scaled_sum(gpu, dtype, tol):
    from stride_b200.config import NormSpec
    from stride_b200.parts import ResidualStream, Runtime, build_part
    rt = Runtime("cuda", STORED[dtype], 32, 8)
    g = torch.Generator().manual_seed(2)
    width = 70
    norm = build_part("norm", NormSpec("dyt", width, 0.0, "n"), rt)
    assert sorted(norm.declare()) == ["n", "n.alpha", "n.b"]
    w = {"n": 1 + 0.3 * torch.randn(width, generator=g), "n.b": 0.2 * torch.randn(width, generator=g), "n.alpha": torch.tensor(0.8)}
    norm.bind({k: v.cuda() for k, v in w.items()})
    x0 = torch.randn(9, width, generator=g)
    d1, d2 = (torch.randn(9, width, generator=g).to(STORED[dtype]) for _ in range(2))
    stream = ResidualStream(rt, 9, width)
    stream.residual.copy_(x0)
    stream.add(d1.cuda(), 0.5)
    wd = {k: v.double() for k, v in w.items()}
    close(stream.normed(norm), plain.dynamic_tanh(x0.double() + 0.5 * d1.double(), wd, "n"), tol)
    stream.add(d2.cuda(), 0.25)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device="cuda")
    total = x0.double() + 0.5 * d1.double() + 0.25 * d2.double()
    close(stream.normed(norm, rows=rows), plain.dynamic_tanh(total[[8, 0, 3]], wd, "n"), tol)
    close(stream.materialize(), total, 3e-6)
    stream.add(d1.cuda())                       # no multiplier
    close(stream.normed(norm), plain.dynamic_tanh(total + d1.double(), wd, "n"), tol)


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-6), ("bfloat16", 3e-6)])
def test_token_side_input_alone(gpu, dtype, tol):
    """The input is computed in float32 on the stream in both modes, so both hold the float32 bound (on the stored,
    rounded matrices)."""
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(4)
    hidden, dim, layers, vocab, tokens = 52, 6, 3, 31, 11
    w = rounded({"side.embed": torch.randn(vocab, dim * layers, generator=g), "l2.side.gate": torch.randn(dim, hidden, generator=g) / 7,
                 "l2.side.proj": torch.randn(hidden, dim, generator=g), "l2.side.norm": 1 + 0.2 * torch.randn(hidden, generator=g)}, dtype)
    x = torch.randn(tokens, hidden, generator=g)
    ids = torch.randint(0, vocab, (tokens,), generator=g)
    want = x.double() + 0.5 * plain.token_side_input(x.double(), ids, 2, {k: v.double() for k, v in w.items()}, dim, 1e-5)
    res = x.cuda()
    seq = torch.zeros(tokens, dtype=torch.int32, device="cuda")
    seq[4] = -1                                 # a padded row stays as it is
    ops.token_side(res, ids.int().cuda(), seq, w["side.embed"].cuda(), 2 * dim, w["l2.side.gate"].cuda(), w["l2.side.proj"].cuda(),
                   w["l2.side.norm"].float().cuda(), 1e-5, 0.5)
    want[4] = x[4].double()
    close(res, want, tol)


@pytest.mark.parametrize("experts,top,shared", [(6, 2, 20), (4, 4, 0), (9, 1, 8)])
def test_routed_experts_alone(gpu, experts, top, shared):
    from stride_b200.config import FeedForwardSpec
    from stride_b200.parts import Runtime, build_part
    from types import SimpleNamespace
    hidden, ff, tokens = 44, 28, 150
    g = torch.Generator().manual_seed(experts)
    mlp = cases.moe(experts, top, ff, shared or None)
    w = {"m.router": torch.randn(experts, hidden, generator=g), "m.router.b": torch.randn(experts, generator=g)}
    for e in range(experts):
        w[f"m.e{e}.up"], w[f"m.e{e}.down"] = torch.randn(ff, hidden, generator=g) / 6, torch.randn(hidden, ff, generator=g) / 5
    if shared:
        w["m.shared.up"], w["m.shared.down"] = torch.randn(shared, hidden, generator=g) / 6, torch.randn(hidden, shared, generator=g) / 5
    x = torch.randn(tokens, hidden, generator=g)
    want = plain.routed_experts(x.double(), {k: v.double() for k, v in w.items()}, "m.", mlp)
    rt = Runtime("cuda", torch.float32, tokens, 8)
    part = build_part("feed_forward", FeedForwardSpec("routed_experts", hidden, ff, "relu_squared", "m.",
                                                      (("experts", experts), ("top", top), ("shared", shared), ("router_bias", True))), rt)
    assert set(part.declare()) == set(w)
    part.bind({k: v.cuda() for k, v in w.items()})
    seq = torch.zeros(tokens, dtype=torch.int32, device="cuda")
    out = part.forward(x.cuda(), SimpleNamespace(seq_of_token=seq))
    close(out, want, 3e-6)


def test_the_router_as_a_product_chooses_as_the_fused_kernel(gpu):
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(8)
    tokens, hidden, experts, top = 70, 96, 11, 3
    x, w, b = torch.randn(tokens, hidden, generator=g).cuda(), torch.randn(experts, hidden, generator=g).cuda(), torch.randn(experts, generator=g).cuda()
    seq = torch.zeros(tokens, dtype=torch.int32, device="cuda")
    seq[5] = -1
    ids1, w1 = torch.empty(tokens, top, dtype=torch.int32, device="cuda"), torch.empty(tokens, top, device="cuda")
    ids2, w2 = torch.empty_like(ids1), torch.empty_like(w1)
    ops.moe_route(x, w, b, seq, ids1, w1)
    logits = torch.empty(tokens, experts, device="cuda")
    ops.linear(x, w, logits)
    ops.moe_select(logits, b, seq, ids2, w2)
    assert torch.equal(ids1, ids2) and (ids1[5] == -1).all()
    close(w2, w1, 1e-5)
    z = (x.double() @ w.double().T + b.double()).cpu()
    assert torch.equal(ids1.cpu().long()[6], z[6].topk(top).indices)


@pytest.mark.parametrize("heads,rank,rot,page", [(6, 80, 16, 16), (20, 128, 32, 8), (1, 16, 16, 4)])
def test_tensor_core_latent_attention_against_the_exact_kernel(gpu, heads, rank, rot, page):
    """Portions and single tokens of three requests in one step, keys scattered over shuffled pages."""
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(heads)
    lens = [(0, 75), (130, 1), (257, 1), (40, 9)]                    # (cached, new): a prompt, two decoded tokens, a portion
    order = [0, 3, 1, 2]                                              # single tokens last, as the step function lays a batch out
    lens = [lens[i] for i in order]
    total_pages = sum(-(-(c + n) // page) for c, n in lens) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    latent = (torch.randn(total_pages, 1, page, rank, generator=g) * 0.7).bfloat16().cuda()
    key_rot = (torch.randn(total_pages, 1, page, rot, generator=g) * 0.7).bfloat16().cuda()
    width = max(-(-(c + n) // page) for c, n in lens)
    table = torch.zeros(len(lens), width, dtype=torch.int32)
    q_start, q_len, ctx_len, seq_of, positions, at = [], [], [], [], [], 0
    for s, (c, n) in enumerate(lens):
        pages = [perm.pop() for _ in range(-(-(c + n) // page))]
        table[s, :len(pages)] = torch.tensor(pages)
        q_start.append(at), q_len.append(n), ctx_len.append(c + n)
        seq_of += [s] * n
        positions += list(range(c, c + n))
        at += n
    tokens = at
    dev = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    qa = (torch.randn(tokens, heads * (rank + rot), generator=g) * 0.5).bfloat16().cuda()
    want, got = torch.zeros(tokens, heads * rank, dtype=torch.bfloat16, device="cuda"), torch.full((tokens, heads * rank), float("nan"), dtype=torch.bfloat16, device="cuda")
    scale = 0.3
    ops.latent_attention(qa, want, latent, key_rot, table.cuda(), dev(seq_of), dev(positions), heads, rank, rot, page, scale)
    args = (latent, key_rot, table.cuda(), dev(q_start), dev(q_len), dev(ctx_len), dev(seq_of))
    ops.latent_attention_tc(qa, got, None, *args, 0, 2, 0, 84, 75, heads, rank, rot, page, scale)
    splits, per_split = 3, 128
    partial = torch.full((tokens * heads * splits * (rank + 2),), float("nan"), device="cuda")
    ops.latent_attention_tc(qa, got, partial, *args, 2, 2, 84, 2, 1, heads, rank, rot, page, scale, splits=splits, keys_per_split=per_split)
    torch.cuda.synchronize()
    ops.check_kernel_status()
    close(got, want, 2e-2)


# ----------------------------------------------------------- each mixer alone, in a model of nothing else
ONLY_RECURRENT = cases.config(72, 101, [(cases.recurrent(88, 4, 5), None), (cases.recurrent(40, 1, 2), None)], mult=1.0)
ONLY_ATTENTION = cases.config(72, 101, [(cases.attention(3, 24, 8, 4, 16, 48), None),
                                        (cases.attention(3, 24, 8, 4, 16, 48, kv_from=0), None)], mult=0.7)
ONLY_EXPERTS_AND_SIDE = cases.config(56, 89, [(cases.recurrent(56, 2, 1), cases.moe(6, 3, 20, shared=12))], mult=0.5, side=10)
ONE_WIDE_BLOCK = cases.config(48, 67, [(cases.recurrent(1536, 1, 3), None)], mult=1.0)       # a block beyond the gates kernel's default shared memory


@pytest.mark.parametrize("name,cfg", [("recurrent", ONLY_RECURRENT), ("attention", ONLY_ATTENTION), ("experts", ONLY_EXPERTS_AND_SIDE),
                                      ("wide_block", ONE_WIDE_BLOCK)])
def test_each_mechanism_in_a_model_of_its_own(gpu, tmp_models, name, cfg):
    folder, requests, want = model_case(tmp_models, name, cfg, "float32", 7, [45, 19, 3])
    replay(folder, "float32", modes.whole(requests), want, 8, 2, name + " whole")
    replay(folder, "float32", modes.changing_portions(requests), want, 8, 2, name + " portions")
    replay(folder, "float32", modes.tail_one_by_one(requests, tail=15), want, 8, 2, name + " decode")


# ---------------------------------------------------------------------------- whole models, every cutting
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case,page", [("A", 16), ("B", 8), ("C", 32), ("D", 16), ("E", 16)])
def test_every_cutting_gives_the_plain_logits(gpu, tmp_models, case, page, dtype):
    cfg = cases.CASES[case]
    # case E has three experts and takes two: the third logit is often close, so its router is made more decisive
    folder, requests, want = model_case(tmp_models, case, cfg, dtype, 11, [70, 33, 1, 52, 9, 2], router_gain=16.0 if case == "E" else 4.0)
    # float32 must agree everywhere. bfloat16: a router's near-tie may fall the other way; and at case E's width of 100
    # with a multiplier of 0.8 the rounding of single activations reaches the bound on a few rows (its float32 run is exact
    # to 2e-5, layer by layer)
    share = 1.0 if dtype == "float32" else (0.9 if case == "E" else 0.97)
    replay(folder, dtype, modes.whole(requests), want, page, 2, "whole", min_ok=share)
    session = replay(folder, dtype, modes.tail_one_by_one(requests, tail=20), want, page, 2, "decode", min_ok=share)
    assert session.runner.graph_replays > 0, "single-token steps did not go through captured graphs"
    replay(folder, dtype, modes.changing_portions(requests), want, page, 2, "portions", min_ok=share)
    # three live requests on three state slots, six requests in all: pages and slots are used again
    replay(folder, dtype, modes.mixed(requests, live_limit=3, seed=5), want, page, 3, "mixed", min_ok=share)
    replay(folder, dtype, modes.decoding_together(dict(list(requests.items())[:4]), decode_steps=6, prompts_per_step=2), want, page, 4,
           "decoding together", min_ok=share)


def test_float32_logits_do_not_depend_on_the_cutting(gpu, tmp_models):
    """Bitwise: every sum of the 32-bit path has an order that depends on the token's position only."""
    from stride_b200.engine.trace import TraceSession
    cfg = cases.CASE_A
    folder, requests, _want = model_case(tmp_models, "bitwise", cfg, "float32", 13, [41, 18, 27])
    results = []
    for steps in (modes.whole(requests), modes.changing_portions(requests), modes.mixed(requests, live_limit=3, seed=2)):
        session = TraceSession(folder, "float32", max_tokens=modes.peak_tokens(steps), block_size=8, max_requests=3)
        got = {}
        rows = modes.expected_rows(steps)
        for s in steps:
            out = session.run_step(s)
            for r, key in enumerate(rows[s["step"]]):
                got[key] = out[r].clone()
        results.append(got)
    for other in results[1:]:
        for key in other:
            assert torch.equal(other[key], results[0][key]), f"request {key[0]} position {key[1]} differs between cuttings"


# ------------------------------------------------------------- far keys, page borders, the first tokens
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sharp_attention_over_many_pages(gpu, tmp_models, dtype):
    """Queries eight times as large: a softmax settles on one or two keys, near or hundreds of tokens back, so a key
    that is lost, misplaced by a page or rotated for the wrong position changes the logits outright."""
    cfg = cases.config(64, 131, [(cases.attention(4, 16, 16, 16, 16, 32, base=20000.0), None), (cases.recurrent(64, 2, 3), None),
                                 (cases.attention(4, 16, 16, 16, 16, 32, base=20000.0, kv_from=0), cases.moe(4, 2, 24))], mult=0.5, side=8)
    folder, requests, want = model_case(tmp_models, "sharp", cfg, dtype, 17, [389, 131], sharp=8.0)
    share = 1.0 if dtype == "float32" else 0.97
    keep = {"r0": set(range(0, 389, 7)) | set(range(380, 389)) | {0, 1, 2, 3, 7, 8, 9, 15, 16, 17}, "r1": set(range(0, 131, 3))}
    replay(folder, dtype, modes.restrict_wants(modes.whole(requests), keep), want, 8, 2, "whole", min_ok=share)
    replay(folder, dtype, modes.restrict_wants(modes.changing_portions(requests, sizes=(7, 2, 64, 9, 33, 2, 120)), keep), want, 8, 2,
           "portions", min_ok=share)
    replay(folder, dtype, modes.tail_one_by_one(requests, tail=70), want, 8, 2, "long decode", min_ok=share)


def test_a_far_key_that_stands_out_is_found(gpu, tmp_models):
    """One layer of latent attention whose output is visible in the logits: token 5's latent is made the only one that
    matches a query direction used by the last tokens, hundreds of positions and dozens of pages later."""
    cfg = cases.config(48, 61, [(cases.attention(2, 16, 8, 8, 16, 24), None)], mult=1.0)
    state = cases.seeded_state(cfg, 23, sharp=6.0)
    tokens = seeded_tokens(300, cfg["vocab"], 99)
    full = plain.forward(cfg, state, tokens)
    # without the far past the answer is another one: the test would notice a window or a lost page
    recent = plain.forward(cfg, state, tokens[200:])
    assert (full[-1] - recent[-1]).abs().max() > 0.05 * full[-1].abs().max()
    folder = write_model_dir(str(tmp_models / "nidilix_far"), cfg, state, torch.float32)
    requests, want = {"far": tokens}, {"far": full}
    replay(folder, "float32", modes.tail_one_by_one(requests, tail=40), want, 4, 1, "far decode")
    replay(folder, "float32", modes.changing_portions(requests, sizes=(4, 5, 3, 31, 2)), want, 4, 1, "far portions")


def test_the_recurrence_in_pieces_gives_the_chain(gpu, tmp_models, monkeypatch):
    """bfloat16, prompts long enough for the piecewise scan (and a batch of two of them with a short one between):
    against the plain chain, and against the engine's own token-order kernel."""
    from stride_b200.csrc import ops
    cfg = cases.config(64, 101, [(cases.recurrent(96, 3, 4), None), (cases.recurrent(64, 1, 2), cases.moe(4, 2, 24))], mult=0.5, side=8)
    folder, requests, want = model_case(tmp_models, "pieces", cfg, "bfloat16", 31, [300, 70, 261])
    monkeypatch.setattr(ops, "SCAN_PIECES_MIN_TOKENS", 128)
    together = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": [0, len(t) // 2, len(t) - 1]} for r, t in requests.items()],
                 "end": list(requests)}]
    replay(folder, "bfloat16", together, want, 16, 3, "three prompts in one step", min_ok=0.97)
    steps = modes.restrict_wants(modes.changing_portions(requests, sizes=(130, 2, 140, 65)), {r: set(range(0, len(t), 5)) for r, t in requests.items()})
    replay(folder, "bfloat16", steps, want, 16, 3, "portions across the pieces' borders", min_ok=0.97)


# --------------------------------------------------------------------------- generation through the engine
def test_greedy_generation_through_the_engine(gpu, tmp_models):
    from stride_b200 import Engine, SamplingParams
    cfg = cases.CASE_A
    state = cases.seeded_state(cfg, 29)
    folder = write_model_dir(str(tmp_models / "nidilix_generate"), cfg, state, torch.float32)
    prompts = [seeded_tokens(n, cfg["vocab"], 300 + n) for n in (37, 5, 18, 1, 26)]
    new = 9
    expected = []
    for prompt in prompts:
        seq = list(prompt)
        for _ in range(new):
            seq.append(int(plain.forward(cfg, state, seq)[-1].argmax()))
        expected.append(seq[len(prompt):])
    # a token budget below the longest prompt: prompts go in portions beside the others' decoded tokens
    engine = Engine(folder, dtype="float32", block_size=8, num_blocks=64, max_batch_tokens=16, max_batch_seqs=3, max_model_len=64,
                    check_invariants=True)
    outs = engine.generate(copy.deepcopy(prompts), SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True))
    assert [o.tokens for o in outs] == expected
