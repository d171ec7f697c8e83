"""Small Figotar configurations with random weights, an engine over them, and the plain implementation's logits."""
import copy

import numpy as np
import torch

import plain_figotar
from vekedra_helpers import make_engine, run_cut, tokens_of, tolerance  # noqa: F401  (the same engine plumbing)


def attn(heads, kv_heads, dim, vdim, window, scale, q_temp=(0.5, 16), mlp=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window},
         "q_temp": {"coef": q_temp[0], "every": q_temp[1]}, "scale": scale, "vdim": vdim}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=1000.0, rot_dims=None, mlp=None):
    m = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank,
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}, "rot_dim": rot_dim, "scale": scale,
         "vdim": vdim}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def mlstm(heads, dim, vdim, cap=15.0, mlp=None):
    return {"type": "mlstm", "mixer": {"dim": dim, "gate_cap": cap, "heads": heads, "vdim": vdim}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(width, vocab, layers, eps=1e-5):
    return {"architecture": "Figotar", "layers": copy.deepcopy(layers), "norm": {"eps": eps}, "vocab": vocab,
            "width": width}


# the three mixers, each once and the memory twice: grouped key/value heads, values wider than keys, a window that ends
# inside a page, a temperature that steps every 16 tokens, a rotated part narrower than the latent, keys and values
# of the memory of unlike widths, a layer without a feed-forward
MIXED = config(64, 96, [
    attn(4, 2, 16, 24, 13, 0.25, mlp=dense(80)),
    mlstm(2, 16, 24, mlp=dense(48)),
    latent(2, 16, 8, 24, 24, 40, 0.2, mlp=None),
    mlstm(4, 8, 8, cap=6.0, mlp=dense(40)),
])
# odd sizes: three heads over one key/value head, widths that are no multiples of 8, a window of one token and one wider
# than any test sequence, a temperature that steps at every token, only part of the rotated entries rotated, one head
# of memory, a memory wider than 32 columns
ODD = config(40, 61, [
    mlstm(1, 12, 20, cap=3.0, mlp=dense(24)),
    attn(3, 1, 12, 20, 1, 0.3, q_temp=(0.25, 1), mlp=None),
    latent(3, 10, 6, 14, 18, 12, 0.3, base=50.0, rot_dims=4, mlp=dense(56)),
    attn(2, 2, 20, 12, 500, 0.2, q_temp=(1.5, 7), mlp=dense(16)),
    mlstm(3, 20, 44, mlp=None),
], eps=1e-4)
# sizes that take the tiled kernels: widths in multiples of 8 and 16 up to 128, several cache groups, a window across
# many pages, memories of 64 and 128 with 48 and 80 columns
WIDE = config(128, 200, [
    attn(4, 2, 48, 80, 70, 0.14, q_temp=(0.5, 32), mlp=dense(192)),
    latent(4, 32, 32, 32, 80, 48, 0.11, base=10000.0, mlp=dense(96)),
    mlstm(2, 64, 48, mlp=dense(128)),
    attn(2, 1, 128, 64, 33, 0.09, q_temp=(0.1, 64), mlp=None),
    latent(2, 64, 16, 64, 48, 80, 0.1, mlp=dense(64)),
    mlstm(1, 128, 80, mlp=None),
    attn(8, 8, 24, 40, 128, 0.2, mlp=dense(64)),
])


def make_weights(cfgd, seed, std=0.25, tweak=None):
    """Random tensors of the configuration, values exact in bfloat16 (both precisions and the plain implementation
    then see the same numbers); ``tweak(tensors)`` may change some before they are rounded."""
    import cbis_b200 as cb
    from cbis_b200.models import Model
    from cbis_b200.weights import InitScheme, random_tensors
    spec = cb.config_from_dict(cfgd).model_spec()
    tensors = random_tensors(Model(spec).declared(), seed, InitScheme(std, 0.3, 0.2, 0.2), torch.float32, draw_on="cpu")
    W = cfgd["width"]
    for name, t in tensors.items():
        if t.dim() == 2 and name != "embed":
            t.mul_((W / t.shape[1]) ** 0.5)         # keep activations of order one
        if name.endswith(".sink"):
            t.add_(1.0)                             # a sink that takes a visible share of the denominator
        if name.endswith(".f.b"):
            t.add_(3.0)                             # a memory that forgets slowly
    if tweak is not None:
        tweak(tensors)
    return {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}


def as_numpy(tensors):
    return {k: v.double().numpy() for k, v in tensors.items()}


def plain(cfgd, tensors, tokens):
    logits, _ = plain_figotar.forward(cfgd, as_numpy(tensors), list(tokens))
    return torch.from_numpy(logits)


def assert_close(got, ref, dtype, what="", tol32=2e-4):
    """32-bit: every row within ``tol32`` and the median row within a quarter of it.  bfloat16: the median row within
    4 % of the largest logit and three rows of four within 8 %.  Single rows may be far off in bfloat16 with random
    weights: where a head of the memory puts out next to nothing (k . q near zero), the unit norm after it blows the
    rounding of the inputs up to the size of the output (the plain implementation itself moves the same rows as far
    when its weights are moved by one bfloat16 rounding).  The 32-bit runs of the same schedules, the kernels' own tests
    in both precisions, and ``assert_same`` against the engine's own run of a request alone are the sharp tests."""
    err = (got - ref).abs().max(1).values
    assert torch.isfinite(got).all(), what
    if dtype == "float32":
        assert err.max() < tol32 and err.median() < tol32 / 4, (what, int(err.argmax()), err.max().item(), err.median().item())
        return
    top = max(1.0, ref.abs().max().item())
    q75 = err.sort().values[min(len(err) - 1, int(0.75 * len(err)))].item() if len(err) >= 8 else err.median().item()
    assert q75 < 0.08 * top and err.median() < 0.04 * top, (what, int(err.argmax()), err.max().item(), q75, err.median().item(), top)


def assert_same(got, alone, what=""):
    """bfloat16: a request's logits from a schedule against the engine's own logits of the request alone and whole:
    the same roundings but for the kernels that differ between prompt portions and single tokens."""
    err = (got - alone).abs().max(1).values
    top = max(1.0, alone.abs().max().item())
    assert torch.isfinite(got).all(), what
    assert err.max() < 0.08 * top and err.median() < 0.01 * top, (what, int(err.argmax()), err.max().item(), err.median().item(), top)


def mixed_schedule(eng, seqs, plan, order):
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
        for r in list(live):
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
