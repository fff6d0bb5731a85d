"""The mechanisms Gukosun brought to the engine, each alone: the kernel (or the part) against the function of
``plain_gukosun`` that states the same mechanism, on hand-made batches whose segments start at position 0,
in the middle of a sequence and on single tokens, over shuffled pages and slots.  Where random numbers
would hide a fault (one key far back, the sink, a window's edge) the inputs are made so that it shows."""
import math

import pytest
import torch

import plain_gukosun as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
F64 = torch.float64
EPS = 1e-5


def dev(t, dtype=None):
    return t.to(device=DEV, dtype=dtype or t.dtype).contiguous()


def close(got, want, rel, what=""):
    got, want = got.detach().cpu().to(F64), want.detach().cpu().to(F64)
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite"
    scale = max(1.0, float(want.abs().max()))
    worst = float((got - want).abs().max())
    assert worst <= rel * scale, f"{what}: max|delta| {worst:.3e} > {rel:.1e} * {scale:.3g}"


def bf16_round(t):
    return t.to(torch.bfloat16).to(F64)


def batch_of(step, done, pages=None):
    """A step's batch: ``step`` is a list of (sequence, new tokens); sequence s sits in slot s."""
    from flyweight_b200.engine import Segment, StepBatch
    segments = [Segment(f"s{s}", s, done[s], [0] * m, []) for s, m in step]
    if pages is None:
        table = [[0]] * len(step)
    else:
        width = max(len(pages[s]) for s, _ in step)
        table = [pages[s] + [-1] * (width - len(pages[s])) for s, _ in step]
    return StepBatch(segments, [table], DEV)


# ------------------------------------------------------------------ the decayed linear recurrence
CUTS_LONG = [[(0, 300), (1, 1), (2, 70)], [(1, 1), (0, 17), (3, 2)], [(0, 1), (1, 1), (2, 1), (3, 1)],
             [(3, 700), (0, 64), (2, 129)], [(2, 256), (3, 257), (1, 16)]]


@pytest.mark.parametrize("form", ["scan", "runs"])
@pytest.mark.parametrize("pad", [5, 8])
@pytest.mark.parametrize("H,d,e", [(2, 16, 8), (3, 24, 40), (1, 128, 128), (2, 64, 32), (1, 1, 1), (2, 18, 10)])
def test_decayed_recurrence_over_portions_pieces_and_single_tokens(form, pad, H, d, e):
    """Four sequences in shuffled slots, fed in portions of 1 to 700 tokens (shorter and longer than a run of
    64 and a piece of 256, and ending on their borders), from a state that is not zero.  ``pad``: unused
    columns behind the projections (5: rows that start off every 16-byte border, so the kernel loads entry by
    entry; 8: rows that 16-byte loads can take where the head sizes allow)."""
    from flyweight_b200.kernels import mixing
    g = torch.Generator().manual_seed(H * 100 + d)
    lengths = [0, 0, 0, 0]
    for step in CUTS_LONG:
        for s, m in step:
            lengths[s] += m
    decay = torch.tensor([1.0 - 2.0 ** (-2 - 3 * j) for j in range(H)], dtype=F64)
    width = 2 * H * d + H * e + pad
    rows = [torch.randn(n, width, generator=g, dtype=F64).float().to(F64) for n in lengths]
    slots = [2, 0, 3, 1]
    start = torch.randn(4, H, d, e, generator=g, dtype=F64).float().to(F64)
    state = torch.full((5, H * d * e + 3), float("nan"), dtype=torch.float32)
    for s in range(4):
        state[slots[s], :H * d * e] = start[s].reshape(-1).float()
    state = dev(state)
    # (the tensor-core form rounds q, k and v to bfloat16: it gets numbers that bfloat16 holds and no
    # activation, so that no rounding of its own can fall the other way; the part's test covers its silu)
    silu_in = form == "scan"
    if not silu_in:
        rows = [bf16_round(r) for r in rows]
    act = P.silu if silu_in else (lambda t: t)
    want, final = [], []
    for s in range(4):
        q = act(rows[s][:, :H * d]).view(-1, H, d)
        k = act(rows[s][:, H * d:2 * H * d]).view(-1, H, d)
        v = act(rows[s][:, 2 * H * d:2 * H * d + H * e]).view(-1, H, e)
        o, S = P.decayed_outer_state(q, k, v, decay, start[s])
        want.append(o.reshape(-1, H * e))
        final.append(S)
    done = [0, 0, 0, 0]
    got = [[] for _ in range(4)]
    kernel = mixing.decay_runs if form == "runs" else mixing.decay_scan
    for step in CUTS_LONG:
        from flyweight_b200.engine import Segment, StepBatch
        batch = StepBatch([Segment(f"s{s}", slots[s], done[s], [0] * m, []) for s, m in step],
                          [[[0]] * len(step)], DEV)
        p = torch.cat([rows[s][done[s]:done[s] + m] for s, m in step]).float()
        o = kernel(dev(p), 0, H * d, 2 * H * d, dev(decay.float()), state, batch, H, d, e, act_silu=silu_in)
        at = 0
        for s, m in step:
            got[s].append(o[at:at + m].cpu())
            at += m
            done[s] += m
    rel = 2e-5 if form == "scan" else 1e-4
    for s in range(4):
        close(torch.cat(got[s]), want[s], rel, f"{form} sequence {s}")
        close(state[slots[s], :H * d * e].cpu().view(H, d, e), final[s], rel, f"{form} state {s}")
    assert torch.isnan(state[4]).all() and torch.isnan(state[:4, H * d * e:]).all()


@pytest.mark.parametrize("form", ["scan", "runs"])
def test_a_key_far_back_still_counts_and_a_decayed_one_does_not(form):
    """Head 0 barely decays and head 1 forgets fast.  Token 3 carries a key and a value far larger than the
    rest; 900 tokens later head 0's read-out is still dominated by it, head 1's holds nothing of it."""
    from flyweight_b200.kernels import mixing
    H, d, e, T = 2, 16, 16, 904
    g = torch.Generator().manual_seed(5)
    decay = torch.tensor([0.9995, 0.5], dtype=F64)
    q = torch.randn(T, H, d, generator=g, dtype=F64).abs() * 0.1
    k = torch.randn(T, H, d, generator=g, dtype=F64).abs() * 0.1
    v = torch.randn(T, H, e, generator=g, dtype=F64) * 0.1
    k[3] = 8.0
    v[3] = torch.linspace(20.0, 50.0, e, dtype=F64)
    q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)
    want, _ = P.decayed_outer_state(q, k, v, decay)
    assert want[-1, 0].abs().min() > 50 * want[-1, 1].abs().max()      # the inputs do what the test is for
    p = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).float()
    kernel = mixing.decay_runs if form == "runs" else mixing.decay_scan
    for cuts in ([T], [600, 300, 4], [2] + [1] * 6 + [896]):
        state = torch.zeros(1, H * d * e, dtype=torch.float32, device=DEV)
        got, done = [], 0
        for m in cuts:
            batch = batch_of([(0, m)], [done])
            got.append(kernel(dev(p[done:done + m]), 0, H * d, 2 * H * d, dev(decay.float()), state, batch, H, d, e,
                              act_silu=False))
            done += m
        close(torch.cat(got).view(T, H, e), want, 1e-4 if form == "runs" else 2e-5, f"{form} cut {cuts}")


# ------------------------------------------------------------------ the mixers as parts
def tiny_config(window=37, heads=4, kv=2, dim=16, vdim=24, width=48, softcap=6.0, rot_dims=8,
                lin=(3, 8, 16), scale=0.3):
    """Three layers: two windowed attentions (the first gives its values to the second) and one pair."""
    att = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window},
           "v_mix": True}
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
            "rot": {"base": 5000.0, "dims": rot_dims,
                    "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}}
    right = {"heads": lin[0], "dim": lin[1], "vdim": lin[2],
             "decay": [round(1.0 - 2.0 ** (-2 - j), 6) for j in range(lin[0])]}
    mlp = {"kind": "dense", "ff": 2 * width}
    return {"architecture": "Gukosun", "vocab": 50, "width": width, "norm": {"eps": EPS}, "logit_scale": 1.0,
            "token_side": {"dim": 8},
            "layers": [{"type": "attention", "mixer": dict(att), "mlp": mlp},
                       {"type": "attention", "mixer": dict(att), "mlp": mlp},
                       {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}]}


def random_weights(raw, seed, dtype):
    """Every tensor the configuration declares, in float64 (rounded to bfloat16 first where that is the dtype)."""
    from flyweight_b200.config import GukosunConfig
    from flyweight_b200.parts import build_arrangement
    g = torch.Generator().manual_seed(seed)
    spec = GukosunConfig.from_dict(raw).model_spec()
    w = {}
    for layer in spec.layers:
        declared = {}
        for part in build_arrangement(layer).parts():
            declared.update(part.declare())
        for name, decl in declared.items():
            t = torch.randn(decl.shape, generator=g, dtype=F64)
            if len(decl.shape) == 2 and ("embed" not in name):
                t = t / math.sqrt(decl.shape[1])
            elif name.endswith("sink"):
                t = t + 1.0
            elif name.endswith("vmix"):
                t = torch.full(decl.shape, 0.3, dtype=F64)
            elif len(decl.shape) == 1:
                t = 1.0 + 0.2 * t
            w[name] = bf16_round(t) if dtype == torch.bfloat16 else t.float().to(F64)
    return spec, w


def run_part(part_spec, w, dtype, h_seqs, cuts, n_pages=24, seed=0, before=None):
    """A mixer over several sequences fed in the portions ``cuts``; pages in shuffled order, slot = 3 - s.
    ``before``: a part that runs first in every step (the layer whose values this one mixes in).
    Returns the outputs by sequence."""
    from flyweight_b200.engine import Segment, StepBatch, StepContext
    from flyweight_b200.parts import Precision, build_mixer
    from flyweight_b200.parts.base import FixedState, PagedKV
    precision = Precision("float32" if dtype == torch.float32 else "bfloat16")
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()

    def made(spec):
        part = build_mixer(spec)
        part.bind(lambda n: w[n].to(dtype), precision, DEV)
        part.prepare(1024, DEV)
        cache = type("Cache", (), {})()
        cache.k_pool = cache.v_pool = cache.state = None
        cache.group = 0
        specs = part.state_spec()
        for one in specs if isinstance(specs, tuple) else (specs,):
            if isinstance(one, PagedKV):
                shape = (n_pages, one.n_kv_heads, 64, one.head_dim)
                cache.k_pool = torch.full(shape, float("nan"), dtype=precision.cache_dtype, device=DEV)
                cache.v_pool = torch.full(shape, float("nan"), dtype=precision.cache_dtype, device=DEV)
            elif isinstance(one, FixedState):
                cache.state = torch.zeros((4,) + tuple(one.shape), dtype=one.dtype, device=DEV)
        return part, cache
    part, cache = made(part_spec)
    first = made(before) if before is not None else None
    pages = {s: [] for s in range(len(h_seqs))}
    done = {s: 0 for s in range(len(h_seqs))}
    outs = {s: [] for s in range(len(h_seqs))}
    for step in cuts:
        segments = []
        for s, m in step:
            while len(pages[s]) * 64 < done[s] + m:
                pages[s].append(order.pop())
            segments.append(Segment(f"s{s}", 3 - s, done[s], [0] * m, []))
        width = max(len(pages[s]) for s, _ in step)
        table = [pages[s] + [-1] * (width - len(pages[s])) for s, _ in step]
        ctx = StepContext(StepBatch(segments, [table], DEV), precision, DEV)
        h = dev(torch.cat([h_seqs[s][done[s]:done[s] + m] for s, m in step]).to(precision.act_dtype))
        if first is not None:
            first[0].forward(ctx, h, first[1])
        out = part.forward(ctx, h, cache)
        at = 0
        for s, m in step:
            outs[s].append(out[at:at + m].float().cpu())
            at += m
            done[s] += m
    return {s: torch.cat(parts) for s, parts in outs.items() if parts}


def inputs_with_partners(lengths, width, pairs, seed, dtype, strength=6.0):
    """Random rows; for every (sequence, key position, query position) in ``pairs`` both rows get a large
    share of one common direction, so that this query's score on this key stands far out."""
    g = torch.Generator().manual_seed(seed)
    seqs = [torch.randn(n, width, generator=g, dtype=F64) for n in lengths]
    for index, (s, j, i) in enumerate(pairs):
        u = torch.randn(width, generator=torch.Generator().manual_seed(1000 + index), dtype=F64)
        seqs[s][j] += strength * u
        seqs[s][i] += strength * u
    return [bf16_round(h) if dtype == torch.bfloat16 else h.float().to(F64) for h in seqs]


def tie_queries_to_keys(w, prefix, heads, kv, dim):
    """Makes every query head's projection its key head's: a row that resembles an earlier one then scores
    high on it, whatever the random weights are."""
    k = w[prefix + "k"].view(kv, dim, -1)
    w[prefix + "q"] = k.repeat_interleave(heads // kv, dim=0).reshape(heads * dim, -1).clone()


CUTS = [[(0, 100), (1, 3)], [(1, 1), (0, 2), (2, 64)], [(0, 1), (1, 1), (2, 1)], [(2, 63), (0, 37), (1, 60)],
        [(0, 1), (2, 2)], [(0, 1)], [(0, 58), (1, 70)]]
LENGTHS = [200, 135, 130]
TOL = {torch.float32: 2e-4, torch.bfloat16: 4e-2}
SHOWS = 20 * TOL[torch.float32]     # what a fault has to change in the plain result for the inputs to count as telling


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,heads,kv,dim,vdim", [(37, 4, 2, 16, 24), (64, 2, 2, 32, 32), (1, 3, 1, 24, 16),
                                                      (129, 4, 1, 16, 16)])
def test_windowed_attention_with_sink_gate_and_mixed_values(dtype, window, heads, kv, dim, vdim):
    """Both roles of the value mix (the layer that gives its values and the one that mixes them in), keys that
    stand out exactly at the window's two sides (in a prompt's portion and for a decoded token), and the
    same with the window one wider or narrower must differ, else the inputs would prove nothing."""
    raw = tiny_config(window=window, heads=heads, kv=kv, dim=dim, vdim=vdim, scale=1.5)
    spec, w = random_weights(raw, 3, dtype)
    for layer in (0, 1):
        tie_queries_to_keys(w, f"l{layer}.mix.", heads, kv, dim)
        w[f"l{layer}.mix.sink"][0] += 1.5 * dim          # (as large as a row's score on itself: head 0 feels it)
    # queries 90 and 150 sit in portions, 102 and 141 are decoded alone (see CUTS); keys just inside, just outside
    pairs = [(0, 90 - window + 1, 90), (0, 150 - window, 150), (0, 102 - window + 1, 102), (0, 141 - window, 141)]
    pairs = [p for p in pairs if p[1] >= 0 and p[1] != p[2]]
    seqs = inputs_with_partners(LENGTHS, raw["width"], pairs, 7, dtype)
    rnd = bf16_round if dtype == torch.bfloat16 else (lambda t: t)
    m = raw["layers"][0]["mixer"]
    source = spec.layers[0].parts["mixer"]
    mixed = spec.layers[1].parts["mixer"]
    got_source = run_part(source, w, dtype, seqs, CUTS)
    got_mixed = run_part(mixed, w, dtype, seqs, CUTS, before=source, seed=1)
    for s, h in enumerate(seqs):
        pos = torch.arange(h.shape[0])
        want, v_first = P.window_attention_mixer(h, w, "l0.mix.", m, EPS, pos, rnd=rnd)
        close(got_source[s], want, TOL[dtype], f"source, sequence {s}")
        want2, _ = P.window_attention_mixer(h, w, "l1.mix.", m, EPS, pos, v_first=v_first, rnd=rnd)
        close(got_mixed[s], want2, TOL[dtype], f"mixed, sequence {s}")
        if s == 0 and window > 1:
            for delta in (-1, 1):
                other = dict(m, mask={"size": window + delta})
                off, _ = P.window_attention_mixer(h, w, "l0.mix.", other, EPS, pos, rnd=rnd)
                rows = [i for _, j, i in pairs if (i - j < window) != (i - j < window + delta)]
                assert all((off[i] - want[i]).abs().max() > SHOWS * max(1.0, want.abs().max())
                                    for i in rows)
    # without the sink, and without mixing, the result would be another: the inputs show both
    h, pos = seqs[1], torch.arange(LENGTHS[1])
    base, v_first = P.window_attention_mixer(h, w, "l0.mix.", m, EPS, pos, rnd=rnd)
    no_sink = dict(w)
    no_sink["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -1e30)
    assert (P.window_attention_mixer(h, no_sink, "l0.mix.", m, EPS, pos, rnd=rnd)[0] - base).abs().max() \
        > SHOWS * base.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,rot_dims,softcap", [(4, 2, 16, 24, 8, 6.0), (2, 1, 32, 32, 32, 2.5),
                                                               (3, 3, 24, 16, 2, 30.0)])
def test_capped_rotated_attention_over_every_earlier_key(dtype, heads, kv, dim, vdim, rot_dims, softcap):
    """The pair's softmax half: a norm over the whole projection, interleaved rotation of the first channels with
    scaled frequencies, capped scores, a sink and a gate per head.  One key far back (position 2, asked for
    from a portion and by decoded tokens 190 later) stands out; uncapped scores would give another result."""
    raw = tiny_config(heads=heads, kv=kv, dim=dim, vdim=vdim, rot_dims=rot_dims, softcap=softcap, scale=2.0)
    spec, w = random_weights(raw, 5, dtype)
    m = raw["layers"][2]["mixer"]["left"]
    pairs = [(0, 2, 95), (0, 2, 102), (0, 2, 199), (1, 0, 134)]
    seqs = inputs_with_partners(LENGTHS, raw["width"], pairs, 9, dtype)
    tie_queries_to_keys(w, "l2.mix.left.", heads, kv, dim)
    w["l2.mix.left.q.norm"] = w["l2.mix.left.k.norm"].view(kv, dim).repeat_interleave(heads // kv, dim=0).reshape(-1)
    rnd = bf16_round if dtype == torch.bfloat16 else (lambda t: t)
    part = spec.layers[2].parts["mixer"].params["left"]
    got = run_part(part, w, dtype, seqs, CUTS)
    for s, h in enumerate(seqs):
        pos = torch.arange(h.shape[0])
        want = P.left_attention_mixer(h, w, "l2.mix.left.", m, EPS, pos, rnd=rnd)
        close(got[s], want, TOL[dtype], f"sequence {s}")
        if s == 0:
            free = P.left_attention_mixer(h, w, "l2.mix.left.", dict(m, softcap=0.0), EPS, pos, rnd=rnd)
            assert (free - want).abs().max() > SHOWS * max(1.0, want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("lin", [(3, 8, 16), (1, 32, 8), (2, 64, 64), (2, 20, 12)])
def test_decayed_linear_attention_part_and_the_pair(dtype, lin):
    """The pair's linear half alone (silu, recurrence in the slot, norm over all heads, gate), then the pair:
    half the sum of the two halves, each normed over the width."""
    raw = tiny_config(lin=lin)
    spec, w = random_weights(raw, 11, dtype)
    seqs = inputs_with_partners(LENGTHS, raw["width"], [], 13, dtype)
    rnd = bf16_round if dtype == torch.bfloat16 else (lambda t: t)
    pair = spec.layers[2].parts["mixer"]
    got_right = run_part(pair.params["right"], w, dtype, seqs, CUTS)
    got_pair = run_part(pair, w, dtype, seqs, CUTS, seed=2)
    m = raw["layers"][2]["mixer"]
    for s, h in enumerate(seqs):
        pos = torch.arange(h.shape[0])
        close(got_right[s], P.right_linear_mixer(h, w, "l2.mix.right.", m["right"], EPS, rnd=rnd), TOL[dtype],
              f"linear half, sequence {s}")
        close(got_pair[s], P.parallel_mixer(h, w, "l2.mix.", m, EPS, pos, rnd=rnd), TOL[dtype], f"pair, sequence {s}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense_feed_forward_and_token_side_input(dtype):
    from flyweight_b200.engine import Segment, StepBatch, StepContext
    from flyweight_b200.parts import Precision
    from flyweight_b200.parts.base import build_feed_forward, build_side_input
    raw = tiny_config()
    spec, w = random_weights(raw, 17, dtype)
    g = torch.Generator().manual_seed(2)
    w["side.embed"] = torch.randn(raw["vocab"], 3 * 8, generator=g, dtype=F64)
    if dtype == torch.bfloat16:
        w["side.embed"] = bf16_round(w["side.embed"])
    precision = Precision("float32" if dtype == torch.float32 else "bfloat16")
    rnd = bf16_round if dtype == torch.bfloat16 else (lambda t: t)
    tokens = [int(t) for t in torch.randint(0, raw["vocab"], (45,), generator=g)]
    batch = StepBatch([Segment("a", 0, 0, tokens[:40], []), Segment("b", 1, 7, tokens[40:], [])], [[[0], [1]]], DEV)
    ctx = StepContext(batch, precision, DEV)
    h = torch.randn(45, raw["width"], generator=g, dtype=F64).float().to(F64)
    ff = build_feed_forward(spec.layers[1].parts["feed_forward"])
    ff.bind(lambda n: w[n].to(dtype), precision, DEV)
    got = ff.forward(ctx, dev(rnd(h).to(precision.act_dtype)))
    close(got, P.dense_feed_forward(h, w, "l1.mlp.", rnd=rnd), TOL[dtype], "feed-forward")
    for index in (0, 2):
        side = build_side_input(spec.layers[index].parts["side"])
        side.bind(lambda n: w[n].to(dtype), precision, DEV)
        x = dev(h.float())
        side.forward(ctx, x)
        want = h + P.token_side_input(h, torch.tensor(tokens), w, f"l{index}.side.", index, 8, EPS, rnd=rnd)
        close(x, want, TOL[dtype], f"side input of layer {index}")
