"""Vekedra through the engine against the plain implementation (GPU): every mechanism's kernels alone, whole
prompts, portions down to two tokens, token-by-token decoding through captured graphs, batches of unequal requests
beside each alone, pages and request slots used again, window edges, far tokens held only by a recurrent state,
and greedy generation through the scheduler."""
import copy

import pytest
import torch

import plain_vekedra as pv
from vekedra_helpers import (MIXED, ODD, WIDE, assert_close, config, dense, latent, make_engine, make_weights, mamba, moe, plain,
                             run_cut, tokens_of, tolerance)

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(t, dtype):
    return t.to(device="cuda", dtype=DTYPES[dtype]).contiguous()


def step_tables(rows_per_segment, slots):
    cu = [0]
    for n in rows_per_segment:
        cu.append(cu[-1] + n)
    return (torch.tensor(slots, dtype=torch.int32, device="cuda"), torch.tensor(cu, dtype=torch.int32, device="cuda"))


# ---- each mechanism's kernels alone ------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unit_norm_in_parts_with_gate(dtype):
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    for parts, width in ((1, 40), (3, 36), (2, 1024), (5, 4000)):
        y = torch.randn(7, width, generator=g) * 3
        z = torch.randn(7, width + 8, generator=g).to(DTYPES[dtype]).float()
        w = 1 + 0.3 * torch.randn(width, generator=g)
        out = torch.empty(7, width, dtype=DTYPES[dtype], device="cuda")
        zd = dev(z, dtype)
        ops.rms_norm(y.cuda(), w.cuda(), 1e-3, out, parts=parts, gate=zd[:, 4:4 + width], gate_act="silu")
        v = (y.double() * pv.silu(z[:, 4:4 + width].double())).reshape(7, parts, -1)
        ref = (pv.rms_unit(v, 1e-3).reshape(7, width) * w.double())
        tol = 1e-5 if dtype == "float32" else 2e-2
        assert (out.double().cpu() - ref).abs().max() < tol * ref.abs().max()
        x = dev(torch.randn(7, width, generator=g), dtype)
        ops.rms_norm(x, None, 1e-6, out)                              # no gate, no weight, the input in the compute type
        assert (out.double().cpu() - pv.rms_unit(x.double().cpu(), 1e-6)).abs().max() < tol * 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gate_product_and_per_head_products(dtype):
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    buf = dev(torch.randn(9, 50, generator=g), dtype)
    out = torch.empty(9, 20, dtype=DTYPES[dtype], device="cuda")
    ops.gate_mul(buf[:, 3:23], buf[:, 30:50], "silu", out)
    a, b = buf[:, 3:23].double().cpu(), buf[:, 30:50].double().cpu()
    tol = 1e-6 if dtype == "float32" else 1e-2
    assert (out.double().cpu() - pv.silu(a) * b).abs().max() < tol * 10
    ops.gate_mul(buf[:, 3:23], buf[:, 30:50], "sigmoid", out)
    assert (out.double().cpu() - torch.sigmoid(a) * b).abs().max() < tol * 10
    for T in (1, 5, 70):
        x = dev(torch.randn(T, 3 * 12 + 4, generator=g), dtype)
        w = dev(torch.randn(3, 20, 12, generator=g), dtype)
        o = torch.zeros(T, 3 * 20 + 8, dtype=DTYPES[dtype], device="cuda")
        ops.linear_heads(x[:, 4:], w, o[:, 8:])
        ref = torch.einsum("thk,hnk->thn", x[:, 4:].double().cpu().view(T, 3, 12), w.double().cpu()).reshape(T, 60)
        assert (o[:, 8:].double().cpu() - ref).abs().max() < (1e-5 if dtype == "float32" else 0.05) * ref.abs().max()
        assert (o[:, :8] == 0).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps", [1, 2, 4, 5, 8])
def test_causal_convolution_over_steps(dtype, taps):
    """Three requests in three steps of unlike portions (70 rows: several blocks of rows; 1; 2 < taps - 1), each from the
    state the step before left, against the convolution of each whole sequence."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(taps)
    C, c0 = 150, 6
    w = torch.randn(C, taps, generator=g)
    b = torch.randn(C, generator=g)
    seqs = [dev(torch.randn(n, c0 + C + 2, generator=g), dtype) for n in (75, 8, 9)]
    state = torch.zeros(5, (taps - 1) * C + 3, dtype=torch.float32, device="cuda")[:, :max(1, (taps - 1) * C)]
    slots = [3, 0, 4]
    fed = [0, 0, 0]
    got = [[], [], []]
    for portions in ([70, 1, 2], [2, 5, 1], [3, 2, 6]):
        rows = torch.cat([s[f:f + n] for s, f, n in zip(seqs, fed, portions)])
        seg_slot, cu = step_tables(portions, slots)
        out = torch.empty(rows.shape[0], C, dtype=rows.dtype, device="cuda")
        short = max(portions) <= ops.conv_rows_per_block()        # then the convolution may leave the state itself
        ops.causal_conv_act(rows, c0, C, w.cuda(), b.cuda(), state, seg_slot, cu, 3, max(portions), "silu", out,
                            update_state=short)
        if not short:
            ops.conv_state_update(rows, c0, C, taps, state, seg_slot, cu, 3)
        at = 0
        for i, n in enumerate(portions):
            got[i].append(out[at:at + n].double().cpu())
            at += n
            fed[i] += n
    for i, s in enumerate(seqs):
        ref = pv.causal_conv_silu(s[:, c0:c0 + C].double().cpu(), w.double(), b.double())
        tol = 1e-5 if dtype == "float32" else 3e-2
        assert (torch.cat(got[i]) - ref).abs().max() < tol * max(1.0, ref.abs().max())


@pytest.mark.parametrize("pieces", [0, 32])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, P, N, G", [(2, 8, 16, 1), (4, 40, 12, 2), (3, 5, 100, 3), (2, 33, 200, 2), (2, 16, 128, 1)])
def test_state_space_recurrence_over_steps(dtype, H, P, N, G, pieces):
    """Two requests whose rows come in unlike portions; one head decays by less than a thousandth a step, so what the
    first tokens wrote is still most of the state at the end.  Against the recurrence in float64.  ``pieces``: segments
    walked in one piece, or cut into pieces of 32 rows that run side by side (seven of them, the last one short,
    beside a segment of a single row)."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(H * 100 + N)
    inner, lens = H * P, (260, 31)
    a_log = torch.randn(H, generator=g)
    a_log[0] = -5.0
    dt_bias = torch.randn(H, generator=g) - 1.0
    dt_bias[0] = -1.0
    d_skip = torch.randn(H, generator=g)
    seqs = []
    for n in lens:
        xbc = dev(torch.randn(n, inner + 2 * G * N, generator=g), dtype)
        raw = torch.randn(n, 3 + H, generator=g)
        raw[:, 3] = -2.0                                     # head 0: the same small step at every token
        seqs.append((xbc, dev(raw, dtype)))
    state = torch.zeros(4, inner * N, dtype=torch.float32, device="cuda")
    slots, fed, got = [2, 1], [0, 0], [[], []]
    plan = [[200, 1], [1, 2], [2, 27], [57, 1]]
    for portions in plan:
        xs = torch.cat([s[0][f:f + n] for s, f, n in zip(seqs, fed, portions)])
        ps = torch.cat([s[1][f:f + n] for s, f, n in zip(seqs, fed, portions)])
        seg_slot, cu = step_tables(portions, slots)
        y = torch.empty(xs.shape[0], inner, dtype=torch.float32, device="cuda")
        ops.ssm_scan(xs, ps, 3, dt_bias.cuda(), a_log.cuda(), d_skip.cuda(), state, seg_slot, cu, 2, H, P, N, G, y,
                     max_seg_rows=max(portions), piece_rows=pieces)
        at = 0
        for i, n in enumerate(portions):
            got[i].append(y[at:at + n].double().cpu())
            at += n
            fed[i] += n
    for i, (xbc, raw) in enumerate(seqs):
        xbc, raw = xbc.double().cpu(), raw.double().cpu()
        x, B, C = xbc[:, :inner].view(-1, H, P), xbc[:, inner:inner + G * N].view(-1, G, N), xbc[:, inner + G * N:].view(-1, G, N)
        dt = pv.softplus(raw[:, 3:] + dt_bias.double())
        decay = torch.exp(-torch.exp(a_log.double()) * dt)
        S = torch.zeros(H, N, P, dtype=torch.float64)
        ref = torch.zeros(lens[i], H, P, dtype=torch.float64)
        for t in range(lens[i]):
            for h in range(H):
                S[h] = decay[t, h] * S[h] + dt[t, h] * torch.outer(B[t, h // (H // G)], x[t, h])
                ref[t, h] = S[h].T @ C[t, h // (H // G)] + d_skip[h] * x[t, h]
        out = torch.cat(got[i]).view(-1, H, P)
        assert (out - ref).abs().max() < 2e-5 * max(1.0, ref.abs().max())      # the recurrence is 32-bit in both precisions
        if i == 0:
            assert decay[:, 0].min() > 0.999 and S[0].abs().max() > 0.1
    final = state[2].view(H, P, N).double().cpu()
    assert (final - S_of(seqs[0], a_log, dt_bias, H, P, N, G)).abs().max() < 2e-5 * final.abs().max()


def S_of(seq, a_log, dt_bias, H, P, N, G):
    xbc, raw = seq[0].double().cpu(), seq[1].double().cpu()
    inner = H * P
    x, B = xbc[:, :inner].view(-1, H, P), xbc[:, inner:inner + G * N].view(-1, G, N)
    dt = pv.softplus(raw[:, 3:] + dt_bias.double())
    decay = torch.exp(-torch.exp(a_log.double()) * dt)
    S = torch.zeros(H, P, N, dtype=torch.float64)
    for t in range(x.shape[0]):
        for h in range(H):
            S[h] = decay[t, h] * S[h] + dt[t, h] * torch.outer(x[t, h], B[t, h // (H // G)])
    return S


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routing_and_experts(dtype):
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    for W, F, E, top in ((32, 24, 5, 2), (72, 10, 3, 3), (64, 40, 17, 1)):
        h = dev(torch.randn(13, W + 4, generator=g), dtype)[:, 4:]
        router = dev(torch.randn(E, W, generator=g), dtype)
        gate_up = dev(torch.randn(E, 2 * F, W, generator=g) / W ** 0.5, dtype)
        down = dev(torch.randn(E, W, F, generator=g) / F ** 0.5, dtype)
        ids = torch.empty(13, top, dtype=torch.int32, device="cuda")
        wts = torch.empty(13, top, dtype=torch.float32, device="cuda")
        ops.route_topk(h, router, top, "sigmoid", False, ids, wts)
        s = torch.sigmoid(h.double().cpu() @ router.double().cpu().T)
        best = torch.topk(s, top, dim=1)
        assert torch.equal(ids.cpu().long(), best.indices)
        assert (wts.double().cpu() - best.values).abs().max() < 1e-6
        hidden = torch.empty(13 * top, F, dtype=DTYPES[dtype], device="cuda")
        out = torch.empty(13, W, dtype=torch.float32, device="cuda")
        ops.routed_gate_up(h, gate_up, ids, wts, "silu", True, hidden)
        ops.routed_down(hidden, down, ids, wts, True, out)
        experts = [(gate_up[e, :F].double().cpu(), gate_up[e, F:].double().cpu(), down[e].double().cpu()) for e in range(E)]
        ref = pv.routed_experts(h.double().cpu(), router.double().cpu(), experts, top)
        tol = 1e-5 if dtype == "float32" else 3e-2
        assert (out.double().cpu() - ref).abs().max() < tol * max(1.0, ref.abs().max())
        # the other conventions the part offers: softmax scores divided by their sum, the weight on the output
        ops.route_topk(h, router, top, "softmax", True, ids, wts)
        p = torch.softmax(h.double().cpu() @ router.double().cpu().T, 1)
        best = torch.topk(p, top, dim=1)
        assert torch.equal(ids.cpu().long(), best.indices)
        assert (wts.double().cpu() - best.values / best.values.sum(1, keepdim=True)).abs().max() < 1e-6
        ops.routed_gate_up(h, gate_up, ids, wts, "silu", False, hidden)
        ops.routed_down(hidden, down, ids, wts, False, out)
        ref = torch.zeros(13, W, dtype=torch.float64)
        for t in range(13):
            for k in range(top):
                e = int(ids[t, k])
                ref[t] += wts[t, k].double().cpu() * pv.gated_feed_forward(h[t:t + 1].double().cpu(), *experts[e])[0]
        assert (out.double().cpu() - ref).abs().max() < tol * max(1.0, ref.abs().max())


@pytest.mark.parametrize("W, F, E, top, rows", [(64, 40, 5, 2, 200), (72, 16, 3, 1, 70), (32, 24, 9, 3, 333), (128, 96, 4, 2, 64)])
def test_routed_tiles_for_many_rows(W, F, E, top, rows):
    """Rows sorted by expert and run in tiles on the tensor cores (bfloat16): against the plain implementation, and
    the same rows in another order and beside other rows give the same bits (a row's result is its own)."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(rows)
    h = dev(torch.randn(rows, W, generator=g), "bfloat16")
    router = dev(torch.randn(E, W, generator=g), "bfloat16")
    if E == 4:
        router[1:] = 0                                   # nearly every row goes to experts 0 and one more: long runs of tiles
    gate_up = dev(torch.randn(E, 2 * F, W, generator=g) / W ** 0.5, "bfloat16")
    down = dev(torch.randn(E, W, F, generator=g) / F ** 0.5, "bfloat16")

    def run(x, accumulate_into=None):
        n = x.shape[0]
        ids = torch.empty(n, top, dtype=torch.int32, device="cuda")
        wts = torch.empty(n, top, dtype=torch.float32, device="cuda")
        ops.route_topk(x, router, top, "sigmoid", False, ids, wts)
        out = accumulate_into if accumulate_into is not None else torch.empty(n, W, dtype=torch.float32, device="cuda")
        assert ops.routed_tiles_takes(x, gate_up, down)
        ops.routed_tiles(x, gate_up, down, ids, wts, "silu", True, out, accumulate=accumulate_into is not None)
        return out
    out = run(h)
    experts = [(gate_up[e, :F].double().cpu(), gate_up[e, F:].double().cpu(), down[e].double().cpu()) for e in range(E)]
    ref = pv.routed_experts(h.double().cpu(), router.double().cpu(), experts, top)
    assert (out.double().cpu() - ref).abs().max() < 3e-2 * max(1.0, ref.abs().max())
    perm = torch.randperm(rows, generator=g).cuda()
    assert torch.equal(run(h[perm].contiguous()), out[perm])
    more = torch.cat([dev(torch.randn(50, W, generator=g), "bfloat16"), h])
    assert torch.equal(run(more)[50:], out)
    base = torch.randn(rows, W, generator=g).cuda()
    added = run(h, accumulate_into=base.clone())
    assert (added - (base + out)).abs().max() < 1e-5


# ---- single mechanisms and whole models through the engine -----------------------------------------------------
ALONE = {
    "latent": config(32, 50, [latent(2, 8, 12, 16, 6, 0.35, mlp=None)]),
    "latent_shared": config(32, 50, [latent(2, 8, 12, 16, 6, 0.35, mlp=None), latent(1, 16, 8, 16, 9, 0.3, kv_from=0, mlp=None)]),
    "mamba": config(32, 50, [mamba(2, 12, 10, 2, 3, 2, mlp=None)]),
    "dense": config(32, 50, [mamba(1, 8, 8, 1, 2, 1, mlp=dense(44))]),
    "routed": config(32, 50, [mamba(1, 8, 8, 1, 2, 1, mlp=moe(6, 2, 20))]),
    # sizes that are multiples of nothing: no 16-byte load, no tensor-core tile fits
    "ragged": config(36, 37, [latent(3, 10, 6, 20, 7, 0.3, mlp=moe(3, 2, 10)), mamba(3, 6, 5, 1, 4, 3, mlp=dense(22)),
                              latent(1, 7, 9, 20, 5, 0.4, kv_from=0, mlp=None), mamba(1, 9, 3, 1, 3, 1, mlp=moe(2, 2, 7))]),
    # a latent wider than the tiled kernels' and the decode kernel's heads
    "wide_latent": config(64, 50, [latent(2, 16, 16, 320, 12, 0.25, mlp=None), latent(3, 8, 8, 264, 9, 0.3, mlp=dense(24))]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ALONE))
def test_one_mechanism_models(which, dtype):
    cfgd = ALONE[which]
    w = make_weights(cfgd, 21)
    toks = tokens_of(cfgd, 41, 3)
    ref = plain(cfgd, w, toks)
    eng = make_engine(cfgd, w, dtype)
    for sizes in ([41], [2, 5, 1, 1, 3], [1]):
        assert_close(run_cut(eng, toks, sizes), ref, dtype, cfgd, w, toks, (which, sizes))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_whole_portions_and_token_by_token(name, dtype):
    """A whole prompt; portions of several sizes down to two tokens that cross page edges (pages of 8) and window
    edges; and the whole sequence one token at a time (90 decode steps through captured graphs)."""
    cfgd = MIXED if name == "mixed" else ODD
    w = make_weights(cfgd, 7)
    toks = tokens_of(cfgd, 90, 11)
    ref = plain(cfgd, w, toks)
    eng = make_engine(cfgd, w, dtype)
    for sizes in ([90], [2, 7, 2, 16, 3, 2, 9, 2, 25], [13, 1, 1, 1, 2], [1]):
        assert_close(run_cut(eng, toks, sizes), ref, dtype, cfgd, w, toks, sizes)
    assert eng.runner.graph_replays > 80


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wider_sizes_take_the_other_kernels(dtype):
    """Eight layers whose sizes lead to the tensor-core, the tiled and the general attention kernels, long and short
    windows over pages of 16, states of 64 and 128 (16 lanes a column for a single prompt): a prompt of 230 tokens
    whole, in portions, and with its last 50 tokens decoded one by one; and two unequal requests in one batch."""
    from cbis_b200.engine import StepEntry
    cfgd = WIDE
    w = make_weights(cfgd, 17)
    toks = tokens_of(cfgd, 230, 5)
    ref = plain(cfgd, w, toks)
    eng = make_engine(cfgd, w, dtype, page_size=16, num_pages=40, max_batched_tokens=256)
    for sizes in ([230], [100, 3, 64, 2, 61], [180] + [1] * 50):
        assert_close(run_cut(eng, toks, sizes), ref, dtype, cfgd, w, toks, sizes)
    other = tokens_of(cfgd, 75, 6)
    a, b = eng.open_request(0), eng.open_request(1)
    got_a, got_b = [], []
    out = eng.forward_step([StepEntry(a, 0, toks[:120], list(range(120))), StepEntry(b, 0, other[:2], [0, 1])]).double().cpu()
    got_a.append(out[:120]); got_b.append(out[120:])
    out = eng.forward_step([StepEntry(b, 2, other[2:70], list(range(68))), StepEntry(a, 120, toks[120:121], [0])]).double().cpu()
    got_b.append(out[:68]); got_a.append(out[68:])
    for i in range(5):
        out = eng.forward_step([StepEntry(a, 121 + i, toks[121 + i:122 + i], [0]),
                                StepEntry(b, 70 + i, other[70 + i:71 + i], [0])]).double().cpu()
        got_a.append(out[:1]); got_b.append(out[1:])
    assert_close(torch.cat(got_a), ref[:126], dtype, cfgd, w, toks[:126], "a beside b")
    assert_close(torch.cat(got_b), plain(cfgd, w, other), dtype, cfgd, w, other, "b beside a")


def mixed_schedule(eng, cfgd, seqs, plan, order):
    """Runs ``plan`` (request -> list of portion sizes) with up to as many live requests as the engine has slots, a
    request admitted when a slot is free; every step holds the next portion of every live request but one that sits
    it out now and then.  Returns {request: all its logits}."""
    from cbis_b200.engine import StepEntry
    waiting, live, at, fed, slot = list(order), [], {}, {}, {}
    got = {r: [] for r in order}
    turn = 0
    while waiting or live:
        while waiting and len(live) < eng.pool.max_requests:
            r = waiting.pop(0)
            live.append(r)
            at[r], fed[r], slot[r] = 0, 0, eng.open_request(len(slot))
        entries, who, ended = [], [], []
        for i, r in enumerate(list(live)):
            turn += 1
            if len(live) > 1 and turn % 5 == 0:
                continue
            n = plan[r][at[r]]
            entries.append(StepEntry(slot[r], fed[r], seqs[r][fed[r]:fed[r] + n], list(range(n))))
            who.append((r, n))
            fed[r] += n
            at[r] += 1
            if at[r] == len(plan[r]):
                ended.append(r)
                live.remove(r)
        out = eng.forward_step(entries).double().cpu()
        k = 0
        for r, n in who:
            got[r].append(out[k:k + n])
            k += n
        for r in ended:
            eng.close_request(slot[r])
    return {r: torch.cat(v) for r, v in got.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(name, dtype):
    """Six requests through three slots and a pool of 20 pages of 8 tokens (less than the requests together): portions
    of some beside single tokens of others; every logit equals the request's alone (the plain implementation's).
    Freed pages are filled with NaN before they are used again, and a slot's recurrent state starts from zero."""
    cfgd = MIXED if name == "mixed" else ODD
    w = make_weights(cfgd, 9)
    lens = {"a": 70, "b": 33, "c": 58, "d": 2, "e": 47, "f": 64}
    seqs = {r: tokens_of(cfgd, n, 40 + i) for i, (r, n) in enumerate(lens.items())}
    plan = {"a": [30, 2, 1, 1, 1, 1, 1, 33], "b": [2, 20, 1, 1, 1, 8], "c": [50, 1, 1, 2, 1, 1, 1, 1], "d": [2],
            "e": [3, 1, 1, 1, 41], "f": [17, 40, 1, 1, 1, 1, 1, 1, 1]}
    assert all(sum(plan[r]) == lens[r] for r in lens)
    eng = make_engine(cfgd, w, dtype, num_pages=26, max_num_seqs=3, poison_freed_pages=True)
    got = mixed_schedule(eng, cfgd, seqs, plan, list(lens))
    assert eng.pages_poisoned > 10
    for r in lens:
        assert_close(got[r], plain(cfgd, w, seqs[r]), dtype, cfgd, w, seqs[r], r)


# ---- weights made so that a fault shows ------------------------------------------------------------------------
def test_window_edges_in_prompts_and_in_decoding():
    """One latent-attention layer with sharp scores (queries and key projections scaled up): moving the window by one
    token changes the logits by far more than the tolerance, so a window one token off would show; prompts cut at
    and around the window's and the pages' edges, and single tokens, agree with the plain implementation."""
    win = 11
    cfgd = config(32, 40, [latent(2, 8, 8, 16, win, 0.5, mlp=None)], scale=3.0)

    def sharpen(t):
        t["l0.mix.q"].mul_(1.5)
        t["l0.mix.uk"].mul_(1.5)
    w = make_weights(cfgd, 5, tweak=sharpen)
    toks = tokens_of(cfgd, 60, 1)
    ref = plain(cfgd, w, toks)
    for other in (win - 1, win + 1):
        off = copy.deepcopy(cfgd)
        off["layers"][0]["mixer"]["mask"]["size"] = other
        moved = (plain(off, w, toks) - ref).abs().max(1).values
        assert moved[:win - 1].max() < 1e-9 and (moved[win + 5:] > 2e-3).float().mean() > 0.5     # the test can see one token
    eng = make_engine(cfgd, w, "float32")
    for sizes in ([60], [win, 1, 1, 1, win - 1, 2, 3], [win - 1, 2, 8, 1, 1, 16], [8, 8, 8, 3, 1, 1, 1, 1, 1, 7], [1]):
        got = run_cut(eng, toks, sizes)
        assert (got - ref).abs().max() < 2e-4, sizes
    eng16 = make_engine(cfgd, w, "bfloat16")
    for sizes in ([60], [win - 1, 2, 8, 1, 1, 16], [1]):
        assert_close(run_cut(eng16, toks, sizes), ref, "bfloat16", what=sizes)


def test_reader_with_a_wider_window_than_the_layer_it_reads():
    """The layer that keeps the latents sees 4 tokens back, the layer that reads them 23: the pages must stay for the
    reader (pages of 4 tokens: the keeper alone would give them back after two pages)."""
    cfgd = config(32, 40, [latent(2, 8, 8, 16, 4, 0.5, mlp=None), latent(2, 8, 8, 16, 23, 0.5, kv_from=0, mlp=dense(24))])
    w = make_weights(cfgd, 6)
    toks = tokens_of(cfgd, 70, 2)
    ref = plain(cfgd, w, toks)
    eng = make_engine(cfgd, w, "float32", page_size=4, num_pages=12, poison_freed_pages=True, max_model_len=128)
    for sizes in ([9, 2, 1, 1, 1, 5], [1]):
        got = run_cut(eng, toks, sizes)
        assert torch.isfinite(got).all() and (got - ref).abs().max() < 2e-4, sizes
    assert eng.pages_poisoned > 10                      # pages behind the wider window did go back


def test_far_tokens_held_by_the_state():
    """A state-space layer whose first head forgets a few thousandths a step: the logits 300 tokens later still depend
    on the first token (changing it moves them by far more than the tolerance), in a whole prompt, in portions, and
    when the last 120 tokens are decoded one by one."""
    cfgd = config(32, 40, [mamba(2, 8, 16, 1, 4, 1, mlp=None)], scale=3.0)

    def slow(t):
        t["l0.mix.A_log"][0] = -5.5
        t["l0.mix.in"][-2].zero_()                     # head 0's step size does not depend on the token ...
        t["l0.mix.dt_bias"][0] = -0.5                  # ... and is softplus(-0.5) at every step
    w = make_weights(cfgd, 8, tweak=slow)
    toks = tokens_of(cfgd, 300, 4)
    ref = plain(cfgd, w, toks)
    changed = plain(cfgd, w, [(toks[0] + 1) % 40] + toks[1:])
    assert (changed[-1] - ref[-1]).abs().max() > 1e-2
    for dtype in ("float32", "bfloat16"):
        eng = make_engine(cfgd, w, dtype, num_pages=64, max_batched_tokens=512)
        for sizes in ([300], [97, 2, 64, 17], [180] + [1] * 120):
            got = run_cut(eng, toks, sizes)
            err = (got - ref).abs().max(1).values
            if dtype == "float32":
                assert err.max() < 1e-4, (sizes, err.max().item())
            else:
                tol = tolerance(dtype, ref)
                assert err.max() < 2 * tol and err.median() < tol / 4, (sizes, err.max().item(), err.median().item())


def test_long_prompts_cut_into_pieces(monkeypatch):
    """The engine cuts the recurrence of a long prompt into pieces that run side by side (here from 64 rows on, in
    pieces of 48, so that a 300-token prompt is seven pieces): whole, in portions and beside a second request, the
    logits are the plain implementation's, and what the last piece leaves is the state decoding goes on from."""
    from cbis_b200.engine import StepEntry
    from cbis_b200.kernels import ops
    monkeypatch.setattr(ops, "SCAN_PIECES_FROM", 64)
    monkeypatch.setattr(ops, "SCAN_PIECE_ROWS", 48)
    cfgd = config(32, 40, [mamba(2, 8, 16, 1, 4, 1, mlp=None), mamba(4, 4, 64, 2, 2, 2, mlp=dense(24))], scale=3.0)
    w = make_weights(cfgd, 8)
    toks, other = tokens_of(cfgd, 300, 4), tokens_of(cfgd, 131, 5)
    ref, ref_other = plain(cfgd, w, toks), plain(cfgd, w, other)
    for dtype in ("float32", "bfloat16"):
        eng = make_engine(cfgd, w, dtype, num_pages=64, max_batched_tokens=512)
        for sizes in ([300], [97, 2, 150, 51], [280] + [1] * 20):
            assert_close(run_cut(eng, toks, sizes), ref, dtype, what=sizes)
        a, b = eng.open_request(0), eng.open_request(1)
        out = eng.forward_step([StepEntry(a, 0, toks[:200], list(range(200))), StepEntry(b, 0, other[:1], [0])]).double().cpu()
        got_a, got_b = [out[:200]], [out[200:]]
        out = eng.forward_step([StepEntry(b, 1, other[1:], list(range(130))), StepEntry(a, 200, toks[200:201], [0])]).double().cpu()
        got_b.append(out[:130]); got_a.append(out[130:])
        assert_close(torch.cat(got_a), ref[:201], dtype, what="a")
        assert_close(torch.cat(got_b), ref_other, dtype, what="b")


# ---- generation through the scheduler --------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype):
    """Five prompts of unlike lengths through ``Engine.generate`` (three slots, prompts cut into portions of 16, a pool
    that holds less than all of them): the tokens are the plain implementation's greedy choices wherever its two best
    logits are further apart than rounding."""
    import cbis_b200 as cb
    cfgd = MIXED
    w = make_weights(cfgd, 13)
    prompts = [tokens_of(cfgd, n, 70 + n) for n in (3, 40, 1, 25, 33)]
    new = 12
    eng = make_engine(cfgd, w, dtype, num_pages=24, max_num_seqs=3, max_batched_tokens=64, prefill_chunk=16)
    outs = eng.generate(prompts, cb.SamplingParams(max_new_tokens=new))
    gap = 1e-3 if dtype == "float32" else 0.25
    for p, o in zip(prompts, outs):
        assert len(o) == new
        seq = list(p)
        for tok in o:
            logits = plain(cfgd, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if top2[0] - top2[1] < gap:
                break                                   # a close call: from here on the sequences may part
            assert tok == int(logits.argmax()), (len(p), len(seq))
            seq.append(tok)
    assert eng.scheduler.idle()
    again = eng.generate(prompts[:2], cb.SamplingParams(max_new_tokens=new))     # slots, pages and states used again
    assert again == outs[:2]
    # a fresh engine whose decode graphs are captured ahead of serving, with requests of the engine's own that leave
    # their states and pages behind
    warm = make_engine(cfgd, w, dtype, num_pages=24, max_num_seqs=3, max_batched_tokens=64, prefill_chunk=16)
    assert warm.warm_up() > 0
    assert warm.generate(prompts[:2], cb.SamplingParams(max_new_tokens=new)) == outs[:2]


# ---- trace replay through bin/trace_run -------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_a_model_folder(dtype, tmp_path):
    """A Vekedra folder (config.json, model.safetensors) through ``bin/trace_run``: a request whole; one with its last
    20 tokens one by one; one in portions down to two tokens; and four live requests in mixed steps through a pool
    smaller than the requests together, so that pages and state slots are used again."""
    import json
    import os

    import numpy as np

    from cbis_b200.weights.safetensors_io import write_safetensors
    from replay_helpers import Trace, read_logits, run_trace
    cfgd = MIXED
    w = make_weights(cfgd, 23)
    folder = str(tmp_path / "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfgd, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in w.items()})
    lens = {"whole": 70, "tail": 50, "cut": 61, "m0": 40, "m1": 33, "m2": 64, "m3": 9, "m4": 21}
    seqs = {r: tokens_of(cfgd, n, 90 + i) for i, (r, n) in enumerate(lens.items())}
    t = Trace()
    t.step([("whole", seqs["whole"], range(70))], end=["whole"])
    t.step([("tail", seqs["tail"][:30], range(30))])
    for i in range(30, 50):
        t.step([("tail", seqs["tail"][i:i + 1], [0])], end=["tail"] if i == 49 else [])
    pos = 0
    for n in [16, 7, 2, 5, 2, 9, 3, 2, 15]:
        t.step([("cut", seqs["cut"][pos:pos + n], range(n))], end=["cut"] if pos + n == 61 else [])
        pos += n
    plan = {"m0": [30, 2, 1, 1, 6], "m1": [2, 20, 1, 10], "m2": [50, 1, 1, 12], "m3": [9], "m4": [3, 1, 17]}
    waiting, live, at, fed = list(plan), [], {}, {}
    while waiting or live:
        while waiting and len(live) < 4:
            r = waiting.pop(0)
            live.append(r); at[r] = 0; fed[r] = 0
        entries, ended = [], []
        for r in list(live):
            n = plan[r][at[r]]
            entries.append((r, seqs[r][fed[r]:fed[r] + n], range(n)))
            fed[r] += n; at[r] += 1
            if at[r] == len(plan[r]):
                ended.append(r); live.remove(r)
        t.step(entries, end=ended)
    bound = t.live_tokens_bound()
    assert bound < sum(-(-n // 64) * 64 for n in lens.values())
    out = str(tmp_path / "out")
    run_trace(t, folder, dtype, out, max_tokens=bound, page_size=8, env={"CBIS_POISON_FREED_PAGES": "1"})
    got = read_logits(t, out, cfgd["vocab"])
    for r, toks in seqs.items():
        rows = torch.from_numpy(np.stack([got[(r, p)][0] for p in range(len(toks))])).double()
        assert_close(rows, plain(cfgd, w, toks), dtype, cfgd, w, toks, r)
