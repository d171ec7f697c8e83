"""Small Vekedra configurations with random weights, an engine over them, and the plain implementation's logits."""
import copy

import torch

import plain_vekedra


def latent(heads, dim, vdim, rank, window, scale, kv_from=None, mlp=None):
    m = {"dim": dim, "heads": heads, "kv_rank": rank, "mask": {"size": window}, "scale": scale, "vdim": vdim}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def mamba(heads, vdim, state, groups, conv, norm_groups, mlp=None):
    return {"type": "mamba2", "mixer": {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups,
                                        "state": state, "vdim": vdim}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(width, vocab, layers, scale=4.0, eps=1e-5):
    return {"architecture": "Vekedra", "embedding": {"scale": scale}, "layers": copy.deepcopy(layers),
            "norm": {"eps": eps}, "vocab": vocab, "width": width}


# four unlike layers: a window narrower than its reader's, two groups, two norm groups, two of five experts, no
# feed-forward at all, a state size that is no power of two, two and three taps
MIXED = config(64, 96, [
    latent(2, 16, 24, 32, 10, 0.3, mlp=dense(80)),
    mamba(4, 8, 16, 2, 3, 2, mlp=moe(5, 2, 24)),
    latent(4, 8, 16, 32, 17, 0.4, kv_from=0, mlp=None),
    mamba(2, 16, 12, 1, 2, 1, mlp=dense(40)),
])
# odd sizes: three heads, a latent of 40 (no multiple of 16), a window of one (a token sees itself only) and one wider
# than any test sequence, one tap (no convolution history), five taps, three of four experts
ODD = config(48, 61, [
    mamba(3, 12, 20, 3, 5, 3, mlp=moe(4, 3, 20)),
    latent(3, 12, 20, 40, 1, 0.25, mlp=moe(3, 1, 16)),
    latent(1, 24, 8, 24, 500, 0.2, mlp=dense(56)),
    mamba(6, 4, 8, 2, 1, 1, mlp=None),
], scale=2.5, eps=1e-4)


# sizes that take other kernels: latents of 64 and 128 (tensor-core attention), 96 (tiled), 192 and 256 (general), a
# reader with another head count and window than the layer it reads, states of 64 and 128, four cache groups
WIDE = config(128, 200, [
    mamba(4, 32, 64, 2, 4, 2, mlp=moe(8, 2, 64)),
    latent(4, 32, 48, 64, 70, 0.18, mlp=dense(192)),
    latent(2, 64, 32, 192, 33, 0.12, mlp=None),
    mamba(2, 64, 128, 1, 3, 1, mlp=dense(128)),
    latent(8, 16, 16, 64, 128, 0.25, kv_from=1, mlp=moe(4, 1, 32)),
    latent(3, 32, 32, 96, 20, 0.18, mlp=dense(96)),
    latent(2, 32, 64, 256, 50, 0.18, mlp=None),
    latent(2, 64, 64, 128, 40, 0.12, mlp=dense(64)),
], scale=6.0)


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
        if t.dim() == 2 and not name.endswith(".conv"):
            t.mul_((W / t.shape[1]) ** 0.5 if name != "embed" else 1.0)     # keep activations of order one
        if name.endswith(".A_log"):
            t.sub_(1.0)
    if tweak is not None:
        tweak(tensors)
    return {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}


def make_engine(cfgd, tensors, dtype, **options):
    import cbis_b200 as cb
    from cbis_b200.models import Model
    model = Model(cb.config_from_dict(cfgd).model_spec()).load(tensors, dtype, "cuda")
    opts = dict(page_size=8, num_pages=64, max_num_seqs=4, max_batched_tokens=256)
    opts.update(options)
    return cb.Engine(model, dtype=dtype, **opts)


def plain(cfgd, tensors, tokens):
    with torch.no_grad():
        return plain_vekedra.forward(cfgd, tensors, list(tokens))


def first_close_call(cfgd, tensors, tokens, gap):
    """The first position at which some routed layer's choice hangs on less than ``gap`` between two router logits
    (the sequence's length if there is none): from there on rounding may send a token to another expert."""
    gaps = []
    with torch.no_grad():
        plain_vekedra.forward(cfgd, tensors, list(tokens), gaps=gaps)
    close = [int(torch.nonzero(g < gap)[0]) for g in gaps if bool((g < gap).any())]
    return min(close, default=len(tokens))


def assert_close(got, ref, dtype, cfgd=None, tensors=None, tokens=None, what=""):
    """32-bit: every row within the tolerance.  bfloat16: every row before the sequence's first routing close call
    within the tolerance, and the median row of the whole sequence too (a flipped expert moves a few rows, a fault
    moves most)."""
    err = (got - ref).abs().max(1).values
    tol = tolerance(dtype, ref)
    assert torch.isfinite(got).all(), what
    if dtype == "float32" or cfgd is None:
        assert err.max() < tol, (what, int(err.argmax()), err.max().item())
        return
    n = first_close_call(cfgd, tensors, tokens, 0.08)
    assert n == 0 or err[:n].max() < tol, (what, int(err[:n].argmax()), err[:n].max().item(), n)
    assert err.median() < tol, (what, err.median().item())


def run_cut(eng, tokens, sizes, slot_id=0):
    """All logits of ``tokens`` fed alone in portions of ``sizes`` (cycled)."""
    from cbis_b200.engine import StepEntry
    slot = eng.open_request(slot_id)
    got, pos, k = [], 0, 0
    while pos < len(tokens):
        n = min(sizes[k % len(sizes)], len(tokens) - pos)
        got.append(eng.forward_step([StepEntry(slot, pos, tokens[pos:pos + n], list(range(n)))]).double().cpu())
        pos += n
        k += 1
    eng.close_request(slot)
    return torch.cat(got)


def tokens_of(cfgd, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfgd["vocab"], (n,), generator=g).tolist()


def tolerance(dtype, ref):
    return 2e-4 if dtype == "float32" else 0.04 * max(1.0, ref.abs().max().item())
