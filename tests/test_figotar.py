"""Figotar through the engine against the plain implementation (GPU): every mechanism's kernels alone, whole
prompts, portions down to two tokens, token-by-token decoding through captured graphs, batches of unequal requests
beside each alone, pages and request slots used again, window and page edges, far keys, the sink, the first tokens,
long decoding from a recurrent state, and greedy generation through the scheduler."""
import copy

import numpy as np
import pytest
import torch

import plain_figotar as pf
from figotar_helpers import (MIXED, ODD, WIDE, as_numpy, assert_close, assert_same, attn, config, dense, latent, make_engine,
                             make_weights, mixed_schedule, mlstm, plain, run_cut, tokens_of, tolerance)

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(t, dtype):
    return t.to(device="cuda", dtype=DTYPES[dtype]).contiguous()


def rounded(t, dtype):
    return t.to(DTYPES[dtype]).double()


# ---- each mechanism's kernels alone ------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_after_a_part_added_and_norm_before_the_next(dtype):
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    for width, pad in ((40, 3), (40, 4), (321, 3), (1000, 8), (4096, 4), (4100, 4)):     # rows in registers, or staged
        x = torch.randn(9, width, generator=g) * 2
        y = rounded(torch.randn(9, width + pad, generator=g) * 5, dtype)
        bias, wb, w = (0.3 * torch.randn(width, generator=g) for _ in range(3))
        xd, yd = x.cuda(), dev(y.float(), dtype)[:, pad:]
        out = torch.empty(9, width, dtype=DTYPES[dtype], device="cuda")
        ops.add_rmsnorm(xd, yd, bias.cuda(), (wb.cuda(), 1e-3, 1.0), w.cuda(), 1e-4, 1.0, out)
        d = pf.rms_norm((y[:, pad:] + bias.double()).numpy(), wb.numpy(), 1e-3, 1.0)
        x_ref = x.double().numpy() + d
        ref = pf.rms_norm(x_ref, w.numpy(), 1e-4, 1.0)
        assert np.abs(xd.double().cpu().numpy() - x_ref).max() < 1e-5 * np.abs(x_ref).max()     # the stream stays 32-bit
        tol = 1e-5 if dtype == "float32" else 1e-2
        assert np.abs(out.double().cpu().numpy() - ref).max() < tol * np.abs(ref).max()
        # chosen rows only, a plain weight, nothing to add: the stream is left as it is
        rows = torch.tensor([7, 0, 7], dtype=torch.int32, device="cuda")
        before = xd.clone()
        some = torch.empty(3, width, dtype=torch.float32, device="cuda")
        ops.add_rmsnorm(xd, None, None, None, w.cuda(), 1e-4, 0.0, some, rows)
        assert torch.equal(xd, before)
        assert np.abs(some.double().cpu().numpy() - pf.rms_norm(x_ref[[7, 0, 7]], w.numpy(), 1e-4, 0.0)).max() < 1e-5 * np.abs(ref).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rotation_by_position_and_gate_per_head(dtype):
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    T, H, width, dims, base = 6, 3, 10, 6, 77.0
    src = rounded(torch.randn(T, 5 + H * 14, generator=g), dtype)
    pos = torch.tensor([0, 1, 2, 40, 1000, 7], dtype=torch.int32)
    freqs = (base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)).float().cuda()
    dst = torch.zeros(T, 2 + H * 12, dtype=DTYPES[dtype], device="cuda")
    ops.rope_rows(dev(src.float(), dtype), 5 + 4, 14, dst, 2 + 2, 12, pos.cuda(), H, width, dims, freqs)
    for h in range(H):
        ref = pf.rotate_half(src[:, 5 + 4 + 14 * h:5 + 4 + 14 * h + width].numpy(), pos.numpy(), base, dims)
        got = dst[:, 4 + 12 * h:4 + 12 * h + width].double().cpu().numpy()
        assert np.abs(got - ref).max() < (2e-4 if dtype == "float32" else 2e-2)        # angle 1000 in 32-bit: 1e-4
    assert float(dst[:, :4].abs().max()) == 0.0                                         # nothing written before the first head
    x = rounded(torch.randn(T, H * 7, generator=g), dtype)
    gate = torch.randn(T, H, generator=g)
    out = torch.empty(T, H * 7, dtype=DTYPES[dtype], device="cuda")
    ops.head_gate_mul(dev(x.float(), dtype), gate.cuda(), H, out)
    ref = (x.view(T, H, 7) * torch.sigmoid(gate.double())[:, :, None]).view(T, H * 7)
    assert (out.double().cpu() - ref).abs().max() < (1e-6 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unit_norm_per_head_with_the_gate_after_it(dtype):
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    y = torch.randn(5, 3 * 20, generator=g) * 4
    z = rounded(torch.randn(5, 3 * 20, generator=g), dtype)
    w = 1 + 0.3 * torch.randn(60, generator=g)
    out = torch.empty(5, 60, dtype=DTYPES[dtype], device="cuda")
    ops.rms_norm(y.cuda(), w.cuda(), 1e-3, out, parts=3, gate=dev(z.float(), dtype), gate_act="sigmoid", gate_after=True)
    v = y.double().view(5, 3, 20)
    ref = (v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-3)).view(5, 60) * w.double() * torch.sigmoid(z)
    assert (out.double().cpu() - ref).abs().max() < (1e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, D, V", [(2, 16, 24), (1, 12, 44), (3, 48, 48), (2, 100, 36), (1, 300, 20)])
def test_matrix_memory_recurrence_over_steps(H, D, V, dtype):
    """Three requests of unlike lengths: whole, then each cut into steps of other sizes (also single rows) with the
    state carried in its slot; gates that rise above the running maximum and fall below it; a slot used again starts
    from zero."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    lens = [37, 5, 18]
    T = sum(lens)
    qkv = rounded(torch.randn(T, 3 + 2 * H * D + H * V, generator=g), dtype)
    gates = torch.randn(T, 2 * H, generator=g) * 4 + torch.tensor([0.0] * H + [3.0] * H)
    ib, fb = torch.randn(H, generator=g), torch.randn(H, generator=g)
    cap, qs = 5.0, D ** -0.5
    floats = ops.matrix_memory_state_floats(H, D, V)
    refs, at = [], 0
    for n in lens:
        r = slice(at, at + n)
        q = qkv[r, 3:3 + H * D].view(n, H, D).numpy() * qs
        k = qkv[r, 3 + H * D:3 + 2 * H * D].view(n, H, D).numpy()
        v = qkv[r, 3 + 2 * H * D:].view(n, H, V).numpy()
        li, lf = pf.capped_gates((gates[r, :H] + ib).double().numpy(), (gates[r, H:] + fb).double().numpy(), cap)
        refs.append(torch.from_numpy(pf.memory_steps(q, k, v, li, lf)[0]).view(n, H * V))
        at += n
    ref = torch.cat(refs)

    def run(cuts):
        """cuts: per step a list of (request, rows)."""
        state = torch.full((4, floats + 5), float("nan"), device="cuda")
        state[:3].zero_()
        fed = [0, 0, 0]
        first = [0, lens[0], lens[0] + lens[1]]
        y_all = torch.zeros(T, H * V, dtype=torch.float64)
        for step in cuts:
            rows, cu, slots = [], [0], []
            for r, n in step:
                rows += list(range(first[r] + fed[r], first[r] + fed[r] + n))
                fed[r] += n
                cu.append(cu[-1] + n)
                slots.append(r)
            idx = torch.tensor(rows)
            y = torch.empty(len(rows), H * V, dtype=torch.float32, device="cuda")
            ops.matrix_memory(dev(qkv[idx].float(), dtype), 3, 3 + H * D, 3 + 2 * H * D, gates[idx].cuda().contiguous(),
                              ib.cuda(), fb.cuda(), cap, qs, 1e-6, state, torch.tensor(slots, dtype=torch.int32, device="cuda"),
                              torch.tensor(cu, dtype=torch.int32, device="cuda"), len(slots), H, D, V, y,
                              max_seg_rows=max(n for _, n in step))        # steps of short segments take another form
            y_all[idx] = y.double().cpu()
        assert fed == lens
        return y_all

    tol = 2e-4 if dtype == "float32" else 2e-4      # the recurrence is 32-bit in both: only the inputs were rounded
    whole = run([[(0, 37), (1, 5), (2, 18)]])
    assert (whole - ref).abs().max() < tol * max(1.0, ref.abs().max().item())
    cut = run([[(0, 16), (2, 1)], [(2, 1), (1, 2), (0, 1)], [(0, 17), (2, 16)], [(1, 3)], [(0, 1)], [(0, 2)]])
    assert torch.equal(cut, whole)                  # rows walked in order from the state: the same bits however they are cut


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_kernels_with_bias_temperature_sink_and_unlike_widths(dtype):
    """The general kernel and (bfloat16) the tiled one over the same pages: grouped heads, values of another width than
    the keys, values that are the first entries of the keys' rows, a window, a distance bias, a temperature by
    position, a sink; a request that starts at a later position beside one from position 0."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    ps, H, G = 8, 4, 2
    for D, V, shared in ((16, 24, False), (40, 24, True), (48, 80, False), (128, 104, True), (12, 20, False)):
        lens = [70, 33]
        T = sum(lens)
        q = rounded(torch.randn(T, H * D, generator=g), dtype)
        k = rounded(torch.randn(T, G, D, generator=g), dtype)
        v = k[:, :, :V] if shared else rounded(torch.randn(T, G, V, generator=g), dtype)
        slopes, sinks = pf.distance_slopes(H), torch.randn(H, generator=g).double().numpy() + 1
        window, temp, scale = 21, (0.5, 16), 0.3 / D ** 0.5
        n_pages = sum(-(-n // ps) for n in lens)
        perm = torch.randperm(n_pages, generator=g).tolist()
        kp = torch.zeros(n_pages, G, ps, D)
        vp = kp if shared else torch.zeros(n_pages, G, ps, V)
        bt = torch.full((2, 16), -1, dtype=torch.int32)
        refs, at, used = [], 0, 0
        for s, n in enumerate(lens):
            for p in range(n):
                if p % ps == 0:
                    bt[s, p // ps] = perm[used]
                    used += 1
                kp[bt[s, p // ps], :, p % ps] = k[at + p].float()
                if not shared:
                    vp[bt[s, p // ps], :, p % ps] = v[at + p].float()
            temps = [pf.query_temperature(i, *temp) for i in range(n)]
            r = slice(at, at + n)
            refs.append(torch.from_numpy(pf.attention_rows(q[r].view(n, H, D).numpy(), k[r].numpy(), v[r].numpy(), scale, window,
                                                           slopes, temps, sinks)).view(n, H * V))
            at += n
        ref = torch.cat(refs)
        kd = dev(kp, dtype)
        vd = kd if shared else dev(vp, dtype)
        pos = torch.cat([torch.arange(n) for n in lens]).int().cuda()
        row_seq = torch.cat([torch.full((n,), s) for s, n in enumerate(lens)]).int().cuda()
        sl, sk = torch.tensor(slopes).float().cuda(), torch.tensor(sinks).float().cuda()
        out = torch.zeros(T, H * V, dtype=DTYPES[dtype], device="cuda")
        ops.paged_attention_generic(dev(q.float(), dtype), kd, vd, bt.cuda(), row_seq, pos, out, H, G, D, ps, scale, window,
                                    v_head_dim=V, slopes=sl, sinks=sk, q_temp=temp)
        tol = 1e-5 if dtype == "float32" else 2e-2
        assert (out.double().cpu() - ref).abs().max() < tol, (D, V, shared)
        if dtype == "bfloat16" and D % 8 == 0 and V % 8 == 0:
            out2 = torch.zeros_like(out)
            cu = torch.tensor([0, lens[0], T], dtype=torch.int32, device="cuda")
            ops.paged_prefill_bf16(dev(q.float(), dtype), kd, vd, bt.cuda(), cu, torch.zeros(2, dtype=torch.int32, device="cuda"),
                                   out2, 0, 2, max(lens), H, G, D, ps, scale, window, v_head_dim=V, slopes=sl, sinks=sk,
                                   q_temp=temp)
            assert (out2.double().cpu() - ref).abs().max() < tol, (D, V, shared, "tiled")
            # the decode kernel on each request's last row, its keys whole and split three ways
            last = torch.tensor([lens[0] - 1, T - 1])
            qd = dev(q[last].float(), dtype)
            rs = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
            ps_ = torch.tensor([lens[0] - 1, lens[1] - 1], dtype=torch.int32, device="cuda")
            for nsplit in (1, 3):
                out3 = torch.zeros(2, H * V, dtype=DTYPES[dtype], device="cuda")
                scratch = torch.empty(max(1, ops.decode_scratch_floats(2, H, V, nsplit)), device="cuda")
                counters = torch.zeros(2 * H, dtype=torch.int32, device="cuda")
                ops.paged_decode_bf16(qd, -1, -1, kd, vd, bt.cuda(), rs, ps_, ps_, out3, scratch, counters, H, G, D, ps, scale,
                                      window, nsplit, v_head_dim=V, slopes=sl, sinks=sk, q_temp=temp)
                assert (out3.double().cpu() - ref[last]).abs().max() < tol, (D, V, shared, "decode", nsplit)


# ---- each mechanism as a model of one layer, and the mixed models -------------------------------------------
ONE_LAYER = {
    "attention": config(48, 50, [attn(4, 2, 8, 16, 9, 0.3, q_temp=(0.5, 5), mlp=dense(32))]),
    "latent": config(48, 50, [latent(3, 8, 8, 16, 16, 24, 0.25, rot_dims=6, mlp=dense(32))]),
    "memory": config(48, 50, [mlstm(2, 16, 8, cap=4.0, mlp=None)]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["attention", "latent", "memory", "mixed", "odd"])
def test_whole_prompt_portions_and_single_tokens(name, dtype):
    """A whole prompt; portions of several sizes down to two tokens that end inside pages and windows; token by token
    (decode steps, which replay captured graphs): all against the plain implementation."""
    cfgd = {"mixed": MIXED, "odd": ODD}.get(name) or ONE_LAYER[name]
    w = make_weights(cfgd, 7)
    toks = tokens_of(cfgd, 75, 3)
    ref = plain(cfgd, w, toks)
    eng = make_engine(cfgd, w, dtype)
    whole = None
    for sizes in ([75], [13, 2, 9, 3, 16, 2, 30], [40] + [1] * 35, [1]):
        got = run_cut(eng, toks, sizes)
        assert_close(got, ref, dtype, (name, sizes))
        if dtype == "bfloat16":
            whole = got if whole is None else whole
            assert_same(got, whole, (name, sizes))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_of_the_tiled_kernels(dtype):
    cfgd = WIDE
    w = make_weights(cfgd, 17, std=0.12)
    toks = tokens_of(cfgd, 200, 5)
    ref = plain(cfgd, w, toks)
    eng = make_engine(cfgd, w, dtype, page_size=16, num_pages=40, max_batched_tokens=256)
    for sizes in ([200], [100, 3, 64, 2, 31], [170] + [1] * 30):
        # seven layers: a relative change of 1e-7 of the weights alone moves single rows of the plain logits by 1e-4
        assert_close(run_cut(eng, toks, sizes), ref, dtype, sizes, tol32=1e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_widths_beyond_the_tiled_kernels(dtype):
    """Keys of 160 with values of 136, and a cached row of 160 + 32 entries: wider than the tiled kernel's tiles (the
    decode kernel takes them up to 256, prompts go to the general kernel)."""
    cfgd = config(64, 80, [attn(2, 1, 160, 136, 40, 0.08, mlp=dense(32)), latent(2, 32, 32, 32, 160, 48, 0.1, mlp=None)])
    w = make_weights(cfgd, 19, std=0.12)
    toks = tokens_of(cfgd, 90, 7)
    ref = plain(cfgd, w, toks)
    eng = make_engine(cfgd, w, dtype, page_size=16, num_pages=16)
    for sizes in ([90], [33, 2, 40, 15], [60] + [1] * 30):
        assert_close(run_cut(eng, toks, sizes), ref, dtype, sizes)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(name, dtype):
    """Six requests through three slots and a pool smaller than the requests together: portions of some beside single
    tokens of others; every logit equals the request's alone.  Freed pages are filled with NaN before they are used
    again, and a slot's recurrent state starts from zero."""
    cfgd = MIXED if name == "mixed" else ODD
    w = make_weights(cfgd, 9)
    lens = {"a": 70, "b": 33, "c": 58, "d": 2, "e": 47, "f": 64}
    seqs = {r: tokens_of(cfgd, n, 40 + i) for i, (r, n) in enumerate(lens.items())}
    plan = {"a": [30, 2, 1, 1, 1, 1, 1, 33], "b": [2, 20, 1, 1, 1, 8], "c": [50, 1, 1, 2, 1, 1, 1, 1], "d": [2],
            "e": [3, 1, 1, 1, 41], "f": [17, 40, 1, 1, 1, 1, 1, 1, 1]}
    assert all(sum(plan[r]) == lens[r] for r in lens)
    eng = make_engine(cfgd, w, dtype, num_pages=26, max_num_seqs=3, poison_freed_pages=True)
    got = mixed_schedule(eng, seqs, plan, list(lens))
    assert eng.pages_poisoned > 10
    for r in lens:
        assert_close(got[r], plain(cfgd, w, seqs[r]), dtype, r)
        if dtype == "bfloat16":
            assert_same(got[r], run_cut(eng, seqs[r], [lens[r]]), r)


# ---- weights made so that a fault shows ------------------------------------------------------------------------
def sharpen_attention(t):
    t["l0.mix.q"].mul_(2.0)
    t["l0.mix.k"].mul_(2.0)


def test_window_edges_in_prompts_and_in_decoding():
    """One attention layer with sharp scores: moving the window by one token changes the logits by far more than the
    tolerance; prompts cut at and around the window's and the pages' edges, and single tokens, agree with the plain
    implementation in both precisions."""
    win = 11
    cfgd = config(32, 40, [attn(2, 1, 8, 12, win, 0.5, q_temp=(0.5, 16), mlp=None)])
    w = make_weights(cfgd, 5, tweak=sharpen_attention)
    toks = tokens_of(cfgd, 60, 1)
    ref = plain(cfgd, w, toks)
    for other in (win - 1, win + 1):
        off = copy.deepcopy(cfgd)
        off["layers"][0]["mixer"]["mask"]["size"] = other
        moved = (plain(off, w, toks) - ref).abs().max(1).values
        assert moved[:win - 1].max() < 1e-9 and (moved[win + 5:] > 2e-3).float().mean() > 0.2     # the test can see one token
    eng = make_engine(cfgd, w, "float32")
    for sizes in ([60], [win, 1, 1, 1, win - 1, 2, 3], [win - 1, 2, 8, 1, 1, 16], [8, 8, 8, 3, 1, 1, 1, 1, 1, 7], [1]):
        got = run_cut(eng, toks, sizes)
        assert (got - ref).abs().max() < 2e-4, sizes
    eng16 = make_engine(cfgd, w, "bfloat16")
    for sizes in ([60], [win - 1, 2, 8, 1, 1, 16], [1]):
        assert_close(run_cut(eng16, toks, sizes), ref, "bfloat16", sizes)


def test_distance_bias_and_temperature_show():
    """Without the distance bias, or with the temperature's step one token early, the plain logits move by far more
    than the tolerance; the engine agrees with the right ones across the temperature's steps (every 8 tokens)."""
    cfgd = config(32, 40, [attn(2, 2, 8, 8, 40, 0.5, q_temp=(1.0, 8), mlp=None)])
    w = make_weights(cfgd, 6, tweak=sharpen_attention)
    toks = tokens_of(cfgd, 50, 2)
    ref = plain(cfgd, w, toks)
    early = copy.deepcopy(cfgd)
    early["layers"][0]["mixer"]["q_temp"]["every"] = 7
    assert (plain(early, w, toks) - ref).abs().max() > 1e-2
    flat = pf.distance_slopes
    try:
        pf.distance_slopes = lambda heads: np.zeros(heads)
        assert (plain(cfgd, w, toks) - ref).abs().max() > 1e-2
    finally:
        pf.distance_slopes = flat
    for dtype in ("float32", "bfloat16"):
        eng = make_engine(cfgd, w, dtype)
        for sizes in ([50], [7, 1, 1, 7, 2, 6, 10], [1]):
            assert_close(run_cut(eng, toks, sizes), ref, dtype, sizes)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds(dtype):
    """700 keys in pages of 8, no window: the keys at positions 3, 63 and 64 (inside the first page, and on both
    sides of a page's border) are made to stand out for every query (the queries share a direction, these keys lie
    along it), so that they hold most of the softmax's weight hundreds of tokens later; a kernel that loses a far
    key, or takes the page beside it, gives another result altogether."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(6)
    T, H, G, D, V, ps, scale = 700, 2, 1, 16, 24, 8, 0.5
    direction = torch.randn(D, generator=g)
    direction /= direction.norm()
    q = rounded(0.3 * torch.randn(T, H, D, generator=g) + 4.0 * direction, dtype)
    k = 0.3 * torch.randn(T, G, D, generator=g)
    for far in (3, 63, 64):
        k[far, 0] += 4.0 * direction
    k, v = rounded(k, dtype), rounded(torch.randn(T, G, V, generator=g), dtype)
    rows = list(range(600, 700))
    ref = torch.from_numpy(pf.attention_rows(q.numpy(), k.numpy(), v.numpy(), scale))[rows].view(len(rows), H * V)
    alone = pf.softmax_with_sink((k[:700, 0].numpy() @ q[699, 0].numpy()) * scale)
    assert alone[[3, 63, 64]].sum() > 0.8                     # the far keys hold the weight
    pages = -(-T // ps)
    perm = torch.randperm(pages, generator=g)
    kp, vp = torch.zeros(pages, G, ps, D), torch.zeros(pages, G, ps, V)
    for p in range(T):
        kp[perm[p // ps], :, p % ps] = k[p].float()
        vp[perm[p // ps], :, p % ps] = v[p].float()
    bt = perm.int().view(1, pages).cuda()
    qd = dev(q.view(T, H * D).float(), dtype)
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    seq = torch.zeros(T, dtype=torch.int32, device="cuda")
    tol = 1e-5 if dtype == "float32" else 2e-2
    out = torch.zeros(T, H * V, dtype=DTYPES[dtype], device="cuda")
    ops.paged_attention_generic(qd, dev(kp, dtype), dev(vp, dtype), bt, seq, pos, out, H, G, D, ps, scale, 0, v_head_dim=V)
    assert (out[rows].double().cpu() - ref).abs().max() < tol
    # the last 100 rows alone, their keys cut into chunks over more warps (as decoding rows behind a long context are)
    some = torch.zeros(100, H * V, dtype=DTYPES[dtype], device="cuda")
    part = torch.empty(100 * H * 4 * (V + 4), device="cuda")
    ops.paged_attention_generic(qd[600:], dev(kp, dtype), dev(vp, dtype), bt, seq[600:], pos[600:], some, H, G, D, ps, scale, 0,
                                (3, 256), part, v_head_dim=V)
    assert (some.double().cpu() - ref).abs().max() < tol
    if dtype == "bfloat16":
        out2 = torch.zeros_like(out)
        cu = torch.tensor([0, T], dtype=torch.int32, device="cuda")
        ops.paged_prefill_bf16(qd, dev(kp, dtype), dev(vp, dtype), bt, cu, torch.zeros(1, dtype=torch.int32, device="cuda"), out2,
                               0, 1, T, H, G, D, ps, scale, 0, v_head_dim=V)
        assert (out2[rows].double().cpu() - ref).abs().max() < tol


def test_causal_latent_attention_over_many_pages_and_the_sink():
    """Causal attention over a latent, 300 tokens: the sink holds a visible share of the denominator (without it the
    plain logits move by far more than the tolerance).  Whole, in portions across many pages, and decoded one by one."""
    cfgd = config(32, 40, [latent(2, 8, 4, 8, 16, 16, 0.4, base=100.0, mlp=None)])

    def tweak(t):
        t["l0.mix.uk"].mul_(1.5)
        t["l0.mix.uq"].mul_(1.5)
        t["l0.mix.sink"].add_(1.5)
    w = make_weights(cfgd, 8, tweak=tweak)
    toks = tokens_of(cfgd, 300, 4)
    ref = plain(cfgd, w, toks)
    nosink = copy.deepcopy(w)
    nosink["l0.mix.sink"] = nosink["l0.mix.sink"] - 30.0
    assert (plain(cfgd, nosink, toks[:20]) - ref[:20]).abs().max() > 1e-2       # (among hundreds of keys it drowns)
    for dtype in ("float32", "bfloat16"):
        eng = make_engine(cfgd, w, dtype, num_pages=64, max_batched_tokens=512)
        for sizes in ([300], [97, 2, 64, 17], [250] + [1] * 50):
            assert_close(run_cut(eng, toks, sizes), ref, dtype, sizes)


def test_far_tokens_held_by_the_memory_and_long_decoding():
    """A memory whose forget gate stays near one: the logits 300 tokens later still depend on the first token, in a
    whole prompt, in portions, and when the last 150 tokens are decoded one by one."""
    cfgd = config(32, 40, [mlstm(2, 8, 12, cap=15.0, mlp=None)])

    def slow(t):
        t["l0.mix.f"].mul_(0.05)
        t["l0.mix.f.b"].fill_(6.0)
        t["l0.mix.i"].mul_(0.2)
    w = make_weights(cfgd, 8, tweak=slow)
    toks = tokens_of(cfgd, 300, 4)
    ref = plain(cfgd, w, toks)
    changed = plain(cfgd, w, [(toks[0] + 1) % 40] + toks[1:])
    assert (changed[-1] - ref[-1]).abs().max() > 1e-3
    for dtype in ("float32", "bfloat16"):
        eng = make_engine(cfgd, w, dtype, num_pages=64, max_batched_tokens=512)
        for sizes in ([300], [97, 2, 64, 17], [150] + [1] * 150):
            got = run_cut(eng, toks, sizes)
            err = (got - ref).abs().max(1).values
            if dtype == "float32":
                assert err.max() < 2e-4, (sizes, err.max().item())
            else:
                tol = tolerance(dtype, ref)
                assert err.max() < tol and err.median() < tol / 4, (sizes, err.max().item(), err.median().item())


def test_gates_at_their_cap():
    """Raw gates far beyond the cap: the input gate saturates at the cap, the forget gate's logarithm near zero or
    near minus the cap, and the running maximum carries the scale."""
    cfgd = config(32, 40, [mlstm(2, 8, 8, cap=2.0, mlp=dense(16))])

    def wild(t):
        t["l0.mix.i"].mul_(30.0)
        t["l0.mix.f"].mul_(30.0)
    w = make_weights(cfgd, 11, tweak=wild)
    toks = tokens_of(cfgd, 64, 6)
    ref = plain(cfgd, w, toks)
    eng = make_engine(cfgd, w, "float32")
    for sizes in ([64], [5, 2, 1, 30, 26], [1]):
        assert (run_cut(eng, toks, sizes) - ref).abs().max() < 5e-4, sizes


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
    warm = make_engine(cfgd, w, dtype, num_pages=24, max_num_seqs=3, max_batched_tokens=64, prefill_chunk=16)
    assert warm.warm_up() > 0
    assert warm.generate(prompts[:2], cb.SamplingParams(max_new_tokens=new)) == outs[:2]


# ---- trace replay through bin/trace_run -------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_a_model_folder(dtype, tmp_path):
    """A Figotar folder (config.json, model.safetensors) through ``bin/trace_run``: a request whole; one with its last
    20 tokens one by one; one in portions down to two tokens; and four live requests in mixed steps through a pool
    smaller than the requests together, so that pages and state slots are used again."""
    import json
    import os

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
        assert_close(rows, plain(cfgd, w, toks), dtype, r)
