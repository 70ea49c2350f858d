"""The Migelix decoder in the engine against the plain float64 implementation (``plain_migelix``): each mechanism alone
and in a model of its own, whole prompts against token-by-token decoding, portions down to two tokens, batches of
unequal requests with pages and state slots that are used again, keys just inside and just outside a window, far keys
that a memory must carry, the first tokens, long decoding past a window, sizes unlike one another (shared key heads,
partly rotated heads, no rotation, one tap, values wider than keys, no window, no caps, layers that run twice), the
tensor-core attention kernels against the exact one, and greedy generation through the engine's scheduler."""

import copy
import math

import pytest
import torch

import migelix_cases as cases
import plain_migelix as plain
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


def compare_rows(got, want, dtype):
    """float32: the helpers' bound (cosine and largest difference). bfloat16: what the rounding of activations leaves of
    a row, which is a few per cent of its spread for these small, unnormalised random models; a wrong key, window or
    state changes a row outright, and the float32 runs of the same cuttings hold the tight bound."""
    if dtype == "float32":
        return compare_logits(got, want, dtype)
    a, b = got.double().reshape(-1), want.double().reshape(-1)
    if not torch.isfinite(a).all():
        return False, "non-finite logits"
    cos = float(torch.nn.functional.cosine_similarity(a, b, dim=0))
    rel = float((a - b).norm() / (b - b.mean()).norm())
    return cos >= 0.998 and rel <= 0.06, f"cosine {cos:.6f}, error {rel:.3f} of the row's spread"


def rounded(state, dtype):
    return {k: v.to(STORED[dtype]) for k, v in state.items()}


def replay(folder, dtype, steps, want, page, slots, label, poison=True, min_ok=1.0):
    """Runs the steps through a fresh session and compares every wanted row; pages and state slots start as NaN."""
    from stride_b200.engine.trace import TraceSession
    session = TraceSession(folder, dtype, max_tokens=modes.peak_tokens(steps), block_size=page, max_requests=slots)
    if poison:
        for t in session.device_cache.pages:
            t.fill_(float("nan"))
        for t in session.device_cache.states.values():
            t.fill_(float("nan"))
    rows = modes.expected_rows(steps)
    bad, total, first = 0, 0, None
    for s in steps:
        out = session.run_step(s)
        for r, (rid, pos) in enumerate(rows[s["step"]]):
            ok, msg = compare_rows(out[r:r + 1], want[rid][pos:pos + 1], dtype)
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
    folder = write_model_dir(str(tmp_models / f"migelix_{name}_{dtype}_{seed}"), cfg, state, STORED[dtype])
    state = rounded(state, dtype)
    requests = {f"r{i}": seeded_tokens(n, cfg["vocab"], 50 * seed + i) for i, n in enumerate(lengths)}
    want = {rid: plain.forward(cfg, state, toks) for rid, toks in requests.items()}
    return folder, requests, want


# ------------------------------------------------------------------------------------------- small kernels
@pytest.mark.parametrize("dtype,tol", [("float32", 3e-6), ("bfloat16", 1e-2)])
@pytest.mark.parametrize("tokens,inter,block", [(7, 48, 48), (5, 128, 64), (3, 30, 6)])
def test_gelu_gate_times_up(gpu, dtype, tol, tokens, inter, block):
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(inter)
    gate, up = (torch.randn(tokens, inter, generator=g).to(STORED[dtype]) * 2 for _ in range(2))
    stacked = torch.stack([gate.view(tokens, inter // block, block), up.view(tokens, inter // block, block)], dim=2).reshape(tokens, 2 * inter)
    out = torch.empty(tokens, inter, dtype=STORED[dtype], device="cuda")
    ops.gated_act(stacked.contiguous().cuda(), out, block, "gelu_tanh")
    close(out, plain.gelu_tanh(gate.double()) * up.double(), tol)
    ops.gated_act(stacked.contiguous().cuda(), out, block, "silu")
    close(out, gate.double() * torch.sigmoid(gate.double()) * up.double(), tol)


@pytest.mark.parametrize("tokens,inter,k", [(8, 2752, 1024), (3, 9472, 192), (1, 5504, 2048)])
def test_gelu_in_the_epilogue_of_the_gate_and_up_product(gpu, tokens, inter, k):
    """The product for a few tokens that applies the activation itself, against the product followed by the kernel above."""
    from stride_b200.csrc import ops
    from stride_b200.parts.swiglu import interleave_gate_up
    g = torch.Generator().manual_seed(inter)
    x = torch.randn(tokens, k, generator=g).bfloat16().cuda()
    gate, up = ((torch.randn(inter, k, generator=g) * 0.05).bfloat16() for _ in range(2))
    w = interleave_gate_up(gate, up, ops.GATED_BLOCK).cuda()
    out = torch.full((tokens, inter), 7.0, dtype=torch.bfloat16, device="cuda")
    if not ops.linear_gated_tc(x, w, out, None, "gelu_tanh"):
        pytest.skip("the tcgen05 product does not take these sizes")
    both = torch.empty(tokens, 2 * inter, dtype=torch.bfloat16, device="cuda")
    ops.linear(x, w, both)
    unfused = torch.empty_like(out)
    ops.gated_act(both, unfused, ops.GATED_BLOCK, "gelu_tanh")
    torch.cuda.synchronize()
    ops.check_kernel_status()
    close(out, unfused, 1e-2)
    gx = (x.double().cpu() @ gate.double().T).bfloat16().double()
    ux = (x.double().cpu() @ up.double().T).bfloat16().double()
    close(out, plain.gelu_tanh(gx) * ux, 1e-2)


def test_parallel_branches_are_summed_with_their_weights(gpu):
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(5)
    for n, dtype in ((96, torch.bfloat16), (37, torch.float32)):
        a, b = (torch.randn(4, n, generator=g).to(dtype) for _ in range(2))
        out = a.cuda()
        ops.weighted_sum(out, out, 0.6, b.cuda(), 1.3)
        close(out, 0.6 * a.double() + 1.3 * b.double(), 1e-2 if dtype == torch.bfloat16 else 3e-6)


def test_gates_caps_and_tanh_in_place(gpu):
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(1)
    for n in (64, 37):              # with and without 16-byte packs
        x, gate = torch.randn(3, n, generator=g) * 3, torch.randn(3, n, generator=g) * 3
        a = x.cuda()
        ops.sigmoid_gate(a, gate.cuda())
        close(a, x.double() * torch.sigmoid(gate.double()), 3e-6)
        a = (x * 10).cuda()
        ops.softcap_(a, 7.0)
        close(a, 7.0 * torch.tanh(x.double() * 10 / 7.0), 3e-6)
        a = x.bfloat16().cuda()
        ops.tanh_(a)
        close(a, torch.tanh(x.bfloat16().double()), 1e-2)


def test_norm_whose_factor_is_one_plus_the_weight(gpu):
    from stride_b200.config import NormSpec
    from stride_b200.parts import ResidualStream, Runtime, build_part
    rt = Runtime("cuda", torch.float32, 16, 4)
    g = torch.Generator().manual_seed(3)
    width = 54
    norm = build_part("norm", NormSpec("rmsnorm", width, 1e-3, "unused.", (("tensor", "n"), ("weight_offset", 1.0))), rt)
    assert list(norm.declare()) == ["n"]
    w = 0.3 * torch.randn(width, generator=g)
    norm.bind({"n": w.cuda()})
    assert torch.equal(norm.named_tensors()["n"].cpu(), w)
    x = torch.randn(6, width, generator=g)
    stream = ResidualStream(rt, 6, width)
    stream.residual.copy_(x)
    close(stream.normed(norm), plain.offset_norm(x.double(), w.double(), 1e-3), 3e-6)


@pytest.mark.parametrize("hd,rotated,yarn", [(32, 16, (8.0, 64, 16.0, 2.0)), (16, 16, None), (24, 0, None), (64, 40, (3.0, 256, 32.0, 1.0))])
def test_rotation_tables_and_head_order_give_the_neighbour_pairs(gpu, hd, rotated, yarn):
    """The part's tables in its own head order, applied the kernels' way (entry i with entry i + hd/2), equal the plain
    rotation of neighbouring pairs, YaRN included."""
    from stride_b200.config import PositionSpec, RopeScaling
    from stride_b200.parts import Runtime, build_part
    scaling = RopeScaling("yarn", yarn[0], yarn[3], yarn[2], yarn[1]) if yarn else None
    part = build_part("position", PositionSpec("rope", head_dim=hd, theta=777.0, max_positions=300, scaling=scaling,
                                               params=(("angles", "float64"), ("pairing", "neighbours"), ("rotated", rotated))), Runtime("cuda", torch.float32, 8, 2))
    cos, sin = (t.cpu().double() for t in part.tables())
    perm = part.head_permutation()
    perm = list(range(hd)) if perm is None else perm
    assert sorted(perm) == list(range(hd))
    g = torch.Generator().manual_seed(hd)
    x = torch.randn(300, 1, hd, generator=g).double()
    want = plain.rotate_pairs(x, torch.arange(300), cases.rot(rotated, 777.0, yarn))[:, 0]
    y = x[:, 0, perm]
    a, b = y[:, :hd // 2], y[:, hd // 2:]
    got = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=1)
    assert (got - want[:, perm]).abs().max() < 2e-6


def paged_case(g, lens, page, nkv, hd):
    """Requests of (cached, new) tokens on shuffled pages: index arrays and random keys and values."""
    total_pages = sum(-(-(c + n) // page) for c, n in lens) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
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
    k = (torch.randn(total_pages, nkv, page, hd, generator=g) * 0.8).bfloat16().cuda()
    v = (torch.randn(total_pages, nkv, page, hd, generator=g) * 0.8).bfloat16().cuda()
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    return k, v, table.cuda(), dev(q_start), dev(q_len), dev(ctx_len), dev(seq_of), dev(positions), at


@pytest.mark.parametrize("nq,nkv,hd,page,window,softcap,sinks", [(4, 2, 64, 16, 70, 0.0, True), (6, 2, 128, 16, 33, 30.0, False),
                                                                 (3, 1, 64, 8, 0, 4.0, True), (8, 8, 64, 32, 129, 0.0, False)])
def test_tensor_core_attention_with_caps_and_sinks_against_the_exact_kernel(gpu, nq, nkv, hd, page, window, softcap, sinks):
    """Portions and single tokens of four requests in one step, through the tcgen05 kernel, the mma.sync kernel and the
    split decode kernel; the exact kernel, itself held to the plain formula below, is the reference."""
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(nq * hd)
    lens = [(0, 150), (40, 9), (130, 1), (257, 1)]               # single tokens last, as the step function lays a batch out
    k, v, table, q_start, q_len, ctx_len, seq_of, positions, tokens = paged_case(g, lens, page, nkv, hd)
    q = (torch.randn(tokens, nq * hd, generator=g) * 0.6).bfloat16().cuda()
    sink = (torch.randn(nq, generator=g) * 2).cuda() if sinks else None
    scale = 0.2
    want = torch.zeros(tokens, nq * hd, dtype=torch.bfloat16, device="cuda")
    ops.paged_attention(q, nq * hd, want, k, v, table, seq_of, positions, nq, nkv, hd, page, scale, window, softcap, sink)
    # the exact kernel against the formula, for the last request's token
    t, (cached, _n) = tokens - 1, lens[3]
    first = max(0, cached - window + 1) if window else 0
    pages = table[3].cpu().tolist()
    rows = lambda cache, head: torch.stack([cache[pages[j // page], head, j % page] for j in range(first, cached + 1)]).double().cpu()
    for h in (0, nq - 1):
        s = rows(k, h // (nq // nkv)) @ q[t, h * hd:(h + 1) * hd].double().cpu() * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        e = torch.exp(s - s.max())
        den = e.sum() + (torch.exp(sink[h].double().cpu() - s.max()) if sinks else 0.0)
        close(want[t, h * hd:(h + 1) * hd], (e / den) @ rows(v, h // (nq // nkv)), 1e-2)
    split = 159
    for prefill in (ops.paged_attention_prefill_tc, ops.paged_attention_prefill):
        got = torch.full((tokens, nq * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        done = prefill(q[:split], nq * hd, got[:split], k, v, table, q_start, q_len, ctx_len, 2, nq, nkv, hd, page, scale, window, softcap, sink)
        if done is False:           # the tcgen05 kernel steps aside for pages it does not take
            continue
        scratch = torch.zeros(ops.decode_scratch_floats(2, nq, nkv, hd, 512), device="cuda")
        ops.paged_attention_decode(q[split:], nq * hd, got[split:], k, v, table, seq_of[split:], positions[split:], scratch, nq, nkv, hd, page,
                                   scale, window, 512, softcap, sink)
        torch.cuda.synchronize()
        ops.check_kernel_status()
        close(got, want, 2e-2)


# ------------------------------------------------------------------- each mixer in a model of nothing else
ONLY_DELTA = cases.config(72, 101, [(cases.parallel(cases.attn_sizes(1, 1, 16, cases.rot(4), window=3), cases.delta_sizes(3, 1, 20, 12, 5), 0.0, 1.0), None),
                                    (cases.parallel(cases.attn_sizes(1, 1, 16, cases.rot(4), window=3), cases.delta_sizes(2, 2, 128, 8, 2), 0.0, 1.0), None),
                                    (cases.parallel(cases.attn_sizes(1, 1, 16, cases.rot(4), window=3), cases.delta_sizes(1, 1, 200, 136, 2), 0.0, 1.0), None)])
ONLY_WKV = cases.config(72, 101, [(cases.wkv(2, 36), None), (cases.wkv(5, 8), None), (cases.wkv(1, 128), None), (cases.wkv(1, 160), None)])
ONLY_ATTENTION = cases.config(72, 101, [(cases.attention(3, 1, 24, cases.rot(12, 3000.0, yarn=(4.0, 32, 8.0, 1.0)), window=11, softcap=3.0), None),
                                        (cases.parallel(cases.attn_sizes(2, 2, 8, cases.rot(8), window=40), cases.delta_sizes(1, 1, 4, 4, 1), 1.0, 0.0), None)])
ONLY_FEED_FORWARD = cases.config(56, 89, [(cases.wkv(1, 4), 70)], logit_softcap=3.0)


@pytest.mark.parametrize("name,cfg", [("delta", ONLY_DELTA), ("wkv", ONLY_WKV), ("attention", ONLY_ATTENTION), ("feed_forward", ONLY_FEED_FORWARD)])
def test_each_mechanism_in_a_model_of_its_own(gpu, tmp_models, name, cfg):
    folder, requests, want = model_case(tmp_models, name, cfg, "float32", 7, [45, 19, 3])
    replay(folder, "float32", modes.whole(requests), want, 8, 2, name + " whole")
    replay(folder, "float32", modes.changing_portions(requests), want, 8, 2, name + " portions")
    replay(folder, "float32", modes.tail_one_by_one(requests, tail=15), want, 8, 2, name + " decode")


# ---------------------------------------------------------------------------- whole models, every cutting
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case,page", [("A", 16), ("B", 8), ("C", 16), ("D", 32)])
def test_every_cutting_gives_the_plain_logits(gpu, tmp_models, case, page, dtype):
    cfg = cases.CASES[case]
    folder, requests, want = model_case(tmp_models, case, cfg, dtype, 11, [90, 33, 1, 52, 9, 2])
    share = 1.0 if dtype == "float32" else 0.97
    replay(folder, dtype, modes.whole(requests), want, page, 2, "whole", min_ok=share)
    session = replay(folder, dtype, modes.tail_one_by_one(requests, tail=40), want, page, 2, "decode", min_ok=share)
    assert session.runner.graph_replays > 0, "single-token steps did not go through captured graphs"
    replay(folder, dtype, modes.changing_portions(requests), want, page, 2, "portions", min_ok=share)
    # three live requests on three state slots, six requests in all: pages and slots are used again
    replay(folder, dtype, modes.mixed(requests, live_limit=3, seed=5), want, page, 3, "mixed", min_ok=share)
    replay(folder, dtype, modes.decoding_together(dict(list(requests.items())[:4]), decode_steps=6, prompts_per_step=2), want, page, 4,
           "decoding together", min_ok=share)


def test_float32_logits_do_not_depend_on_the_cutting(gpu, tmp_models):
    """Bitwise: every sum of the 32-bit path has an order that depends on the token's position only."""
    from stride_b200.engine.trace import TraceSession
    folder, requests, _want = model_case(tmp_models, "bitwise", cases.CASE_A, "float32", 13, [41, 18, 27])
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


# --------------------------------------------------------------- window edges, far keys, the first tokens
def one_attention_layer(window, sinks):
    mixer = cases.attn_sizes(2, 1, 16, cases.rot(8, 2000.0), window=window, scale=1.0)
    if sinks:
        return cases.config(48, 61, [(cases.parallel(mixer, cases.delta_sizes(1, 1, 4, 4, 2), 1.0, 0.0), None)])
    return cases.config(48, 61, [({"type": "attention", "mixer": mixer}, None)])


@pytest.mark.parametrize("window,sinks", [(7, False), (37, True), (16, True)])
def test_a_key_at_the_windows_edge_is_seen_and_the_next_one_is_not(gpu, tmp_models, window, sinks):
    """One attention layer whose queries are eight times as large, so single keys decide. Where the key at the window's
    edge (or the first one outside it) is the one a query settles on, the plain logits of a window of W differ outright
    from those of W - 1 (or W + 1); there are such positions in the prompt's part and among the tokens decoded one by
    one, so a window that is one token off, on any page border, cannot pass."""
    cfg = one_attention_layer(window, sinks)
    state = cases.seeded_state(cfg, 23, sharp=8.0)
    tokens = seeded_tokens(150, cfg["vocab"], 99)
    full = plain.forward(cfg, state, tokens)
    for other in (window - 1, window + 1):
        off = plain.forward(one_attention_layer(other, sinks), state, tokens)
        moved = (off - full).abs().amax(dim=1) > 0.05 * full.abs().max()
        assert moved.sum() >= 4 and moved[60:].sum() >= 2, "the edge of the window does not show in these logits"
    if sinks:       # and the sink shows too
        no_sink = dict(state, **{"l0.mix.left.sink": torch.full_like(state["l0.mix.left.sink"], -30.0)})
        assert (plain.forward(cfg, no_sink, tokens) - full).abs().max() > 0.02 * full.abs().max()
    folder = write_model_dir(str(tmp_models / f"migelix_edge_{window}"), cfg, state, torch.float32)
    requests, want = {"edge": tokens}, {"edge": full}
    for page in (4, 16):
        replay(folder, "float32", modes.whole(requests), want, page, 1, "edge whole")
        replay(folder, "float32", modes.tail_one_by_one(requests, tail=90), want, page, 1, "edge decode")
        replay(folder, "float32", modes.changing_portions(requests, sizes=(window - 1, 2, window, 3, window + 1, 2, 5)), want, page, 1, "edge portions")
    folder16 = write_model_dir(str(tmp_models / f"migelix_edge16_{window}"), cfg, state, torch.bfloat16)
    want16 = {"edge": plain.forward(cfg, rounded(state, "bfloat16"), tokens)}
    replay(folder16, "bfloat16", modes.tail_one_by_one(requests, tail=90), want16, 16, 1, "edge decode", min_ok=0.9)


@pytest.mark.parametrize("kind", ["delta", "wkv"])
def test_a_memory_carries_a_far_token(gpu, tmp_models, kind):
    """A model of one recurrent layer with slow decays: the last logits depend on the first tokens, hundreds of steps
    and many state updates back (checked on the plain model), through portions, decoding and a slot used again."""
    if kind == "delta":
        cfg = cases.config(48, 61, [(cases.parallel(cases.attn_sizes(1, 1, 8, cases.rot(8), window=2), cases.delta_sizes(2, 1, 16, 24, 3), 0.0, 1.0), None)])
    else:
        cfg = cases.config(48, 61, [(cases.wkv(2, 16), None)])
    state = cases.seeded_state(cfg, 31)
    for name in state:              # decays close to one
        if name.endswith("dt_bias"):
            state[name] = state[name] - 5.0
        if name.endswith("w0"):
            state[name] = state[name] - 4.0
    tokens = seeded_tokens(400, cfg["vocab"], 5)
    full = plain.forward(cfg, state, tokens)
    recent = plain.forward(cfg, state, tokens[300:])
    assert (full[-1] - recent[-1]).abs().max() > 0.05 * full[-1].abs().max(), "the far past does not show in these logits"
    folder = write_model_dir(str(tmp_models / f"migelix_far_{kind}"), cfg, state, torch.float32)
    requests, want = {"far": tokens, "again": tokens[300:]}, {"far": full, "again": recent}
    replay(folder, "float32", modes.tail_one_by_one(requests, tail=50), want, 8, 1, "far decode")
    replay(folder, "float32", modes.changing_portions(requests, sizes=(4, 5, 3, 31, 2, 17)), want, 8, 1, "far portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sharp_attention_and_long_decoding_past_the_window(gpu, tmp_models, dtype):
    """The tensor-core sizes with queries six times as large and 120 tokens decoded one by one, more than either window."""
    folder, requests, want = model_case(tmp_models, "sharp", cases.CASE_C, dtype, 17, [389, 131], sharp=6.0)
    share = 1.0 if dtype == "float32" else 0.9
    keep = {"r0": set(range(0, 389, 7)) | set(range(260, 389)) | {0, 1, 2, 3, 15, 16, 17, 32, 33, 34, 69, 70, 71}, "r1": set(range(0, 131, 3))}
    replay(folder, dtype, modes.restrict_wants(modes.whole(requests), keep), want, 16, 2, "whole", min_ok=share)
    replay(folder, dtype, modes.restrict_wants(modes.changing_portions(requests, sizes=(7, 2, 64, 9, 33, 2, 120)), keep), want, 16, 2,
           "portions", min_ok=share)
    replay(folder, dtype, modes.tail_one_by_one(requests, tail=120), want, 16, 2, "long decode", min_ok=share)


def test_the_memory_in_pieces_gives_the_chain(gpu, tmp_models, monkeypatch):
    """bfloat16, portions long enough for the recurrence in pieces (and a batch of two of them with a short one between):
    against the plain chain, with portions that end inside pieces and a slot that is used again."""
    from stride_b200.csrc import ops
    cfg = cases.config(64, 101, [(cases.wkv(3, 20), None), (cases.wkv(1, 64), 48), (cases.wkv(2, 128), None),
                                 (cases.parallel(cases.attn_sizes(2, 1, 16, cases.rot(8), window=19), cases.delta_sizes(3, 1, 20, 12, 3), 0.7, 1.0), None),
                                 (cases.parallel(cases.attn_sizes(2, 1, 16, cases.rot(8), window=19), cases.delta_sizes(2, 2, 128, 72, 4), 0.5, 1.2), 48)])
    folder, requests, want = model_case(tmp_models, "pieces", cfg, "bfloat16", 31, [300, 70, 261])
    monkeypatch.setattr(ops, "SCAN_PIECES_MIN_TOKENS", 128)
    monkeypatch.setattr(ops, "DELTA_PIECES_MIN_TOKENS", 128)
    together = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": [0, len(t) // 2, len(t) - 1]} for r, t in requests.items()],
                 "end": list(requests)}]
    replay(folder, "bfloat16", together, want, 16, 3, "three prompts in one step", min_ok=0.97)
    steps = modes.restrict_wants(modes.changing_portions(requests, sizes=(130, 2, 140, 65)), {r: set(range(0, len(t), 5)) for r, t in requests.items()})
    replay(folder, "bfloat16", steps, want, 16, 1, "portions across the pieces' borders", min_ok=0.97)


# --------------------------------------------------------------------------- generation through the engine
def test_greedy_generation_through_the_engine(gpu, tmp_models):
    from stride_b200 import Engine, SamplingParams
    cfg = cases.CASE_A
    state = cases.seeded_state(cfg, 29)
    folder = write_model_dir(str(tmp_models / "migelix_generate"), cfg, state, torch.float32)
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
