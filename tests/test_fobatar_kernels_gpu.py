"""The mechanisms Fobatar brought to the engine, each alone: the kernel (or the part) against the function of
``plain_fobatar`` that states the same mechanism, on hand-made batches whose segments start at position 0,
in the middle of a sequence and on single tokens, over shuffled pages and slots.  Where random numbers
would hide a fault (a chunk's edge, the sink, one key far back, a clamp that never acts) the inputs are made
so that it shows."""
import math

import pytest
import torch

import plain_fobatar as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
F64 = torch.float64
EPS = 1e-5
TOL = {torch.float32: 2e-4, torch.bfloat16: 4e-2}
SHOWS = 20 * TOL[torch.float32]     # what a fault has to change in the plain result for the inputs to count as telling


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


def rounding(dtype):
    return bf16_round if dtype == torch.bfloat16 else (lambda t: t)


def ramp(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


# ------------------------------------------------------------------ the causal convolution with its rolling state
CONV_CUTS = [[(0, 9), (1, 1), (2, 70)], [(1, 1), (0, 2), (3, 2)], [(0, 1), (1, 1), (2, 1), (3, 1)],
             [(3, 130), (0, 3), (2, 1)], [(1, 2), (3, 1), (0, 1)], [(0, 64), (1, 5)]]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("channels,taps", [(24, 3), (7, 4), (512, 2), (33, 1), (300, 8)])
def test_causal_convolution_over_portions_single_tokens_and_shuffled_slots(dtype, channels, taps):
    """Four sequences in shuffled slots, fed in portions of 1 to 130 tokens (shorter than the taps reach and far
    longer); a fifth slot nobody owns must stay as it was, and a slot's rows at the end are the sequence's last
    inputs."""
    from flyweight_b200.engine import Segment, StepBatch
    from flyweight_b200.kernels import mixing
    g = torch.Generator().manual_seed(channels + taps)
    lengths = [sum(m for step in CONV_CUTS for s, m in step if s == q) for q in range(4)]
    rnd = rounding(dtype)
    rows = [rnd(torch.randn(n, channels, generator=g, dtype=F64).float().to(F64)) for n in lengths]
    w = torch.randn(channels, taps, generator=g, dtype=F64).float().to(F64)
    want = [P.causal_taps(r, w) for r in rows]
    slots = [2, 0, 3, 1]
    state = None
    if taps > 1:
        state = torch.zeros((5, taps - 1, channels), dtype=torch.float32, device=DEV)
        state[4] = float("nan")
    done = [0, 0, 0, 0]
    got = [[] for _ in range(4)]
    for step in CONV_CUTS:
        batch = StepBatch([Segment(f"s{s}", slots[s], done[s], [0] * m, []) for s, m in step], [[[0]] * len(step)], DEV)
        u = dev(torch.cat([rows[s][done[s]:done[s] + m] for s, m in step]).to(dtype))
        kept = u.clone()
        y = mixing.causal_conv(u, dev(w.float()), state, batch)
        assert torch.equal(u, kept)                       # the input is left as it was
        at = 0
        for s, m in step:
            got[s].append(y[at:at + m].float().cpu())
            at += m
            done[s] += m
    for s in range(4):
        close(torch.cat(got[s]), rnd(want[s]) if dtype == torch.bfloat16 else want[s], 1e-5 if dtype == torch.float32 else 1e-2,
              f"sequence {s}")
        if taps > 1:
            close(state[slots[s]].cpu(), rows[s][-(taps - 1):], 1e-6, f"state of sequence {s}")
    if taps > 1:
        assert torch.isnan(state[4]).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,q,k,v,pad", [(3, 40, 24, 16, 0), (1, 64, 0, 0, 0), (4, 18, 6, 10, 8), (2, 3072, 512, 512, 40)])
def test_convolution_with_the_norm_over_ranges_and_columns_it_leaves_alone(dtype, taps, q, k, v, pad):
    """The convolution that also norms the q range and the k range of its output (the mean over fewer channels
    than a range is wide: the last two of each count as padding), from rows that carry ``pad`` more columns
    behind the convolved ones; two portions of one sequence beside a second sequence."""
    from flyweight_b200.engine import Segment, StepBatch
    from flyweight_b200.kernels import mixing
    g = torch.Generator().manual_seed(q + taps)
    C = q + k + v
    rnd = rounding(dtype)
    rows = [rnd(torch.randn(n, C + pad, generator=g, dtype=F64).float().to(F64)) for n in (70, 9)]
    w = torch.randn(C, taps, generator=g, dtype=F64).float().to(F64)
    wq, wk = (1.0 + 0.2 * torch.randn(q, generator=g, dtype=F64)).float().to(F64), None
    ranges = [(0, dev(wq.float()), q - 2, EPS)]
    if k:
        wk = (1.0 + 0.2 * torch.randn(k, generator=g, dtype=F64)).float().to(F64)
        ranges.append((q, dev(wk.float()), k - 2, EPS))
    want = []
    for r in rows:
        y = P.causal_taps(r[:, :C], w)
        y[:, :q] = y[:, :q] / torch.sqrt((y[:, :q] ** 2).sum(-1, keepdim=True) / (q - 2) + EPS) * wq
        if k:
            y[:, q:q + k] = y[:, q:q + k] / torch.sqrt((y[:, q:q + k] ** 2).sum(-1, keepdim=True) / (k - 2) + EPS) * wk
        want.append(y)
    state = torch.zeros((2, taps - 1, C), dtype=torch.float32, device=DEV) if taps > 1 else None
    got = [[], []]
    done = [0, 0]
    for step in ([(0, 33), (1, 2)], [(1, 7), (0, 37)]):
        batch = StepBatch([Segment(f"s{s}", 1 - s, done[s], [0] * m, []) for s, m in step], [[[0]] * 2], DEV)
        u = dev(torch.cat([rows[s][done[s]:done[s] + m] for s, m in step]).to(dtype))
        y = mixing.causal_conv(u, dev(w.float()), state, batch, norm_ranges=ranges)
        assert tuple(y.shape) == (u.shape[0], C)
        at = 0
        for s, m in step:
            got[s].append(y[at:at + m].float().cpu())
            at += m
            done[s] += m
    for s in range(2):
        close(torch.cat(got[s]), want[s], 1e-5 if dtype == torch.float32 else 1.5e-2, f"sequence {s}")


def test_a_gate_per_head_from_columns_of_another_buffer():
    from flyweight_b200.kernels import mixing
    g = torch.Generator().manual_seed(1)
    T, heads, d = 19, 5, 12
    y = torch.randn(T, heads * d, generator=g, dtype=F64).float().to(F64)
    rows = torch.randn(T, 31, generator=g, dtype=F64).float().to(F64) * 3.0
    want = (y.view(T, heads, d) * torch.sigmoid(rows[:, 20:20 + heads])[:, :, None]).reshape(T, -1)
    for y_dtype, rows_dtype, tol in ((torch.float32, torch.float32, 1e-6), (torch.bfloat16, torch.float32, 1e-2),
                                     (torch.bfloat16, torch.bfloat16, 2e-2)):
        got = mixing.sigmoid_gate_cols_mul_(dev(y.to(y_dtype)), dev(rows.to(rows_dtype)), 20, heads, d)
        close(got, want, tol, f"{y_dtype} rows gated from {rows_dtype} columns")


# ------------------------------------------------------------------ the clamped swish on gate and up
def plain_gated(g, u, limit):
    g = torch.clamp(g, max=limit)
    return g * torch.sigmoid(1.702 * g) * (torch.clamp(u, -limit, limit) + 1.0)


@pytest.mark.parametrize("limit", [0.5, 2.0, 7.0])
def test_clamped_swish_elementwise(limit):
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(int(limit * 10))
    gu = torch.randn(37, 2 * 24, generator=g, dtype=F64) * 4.0
    gu[0, :4] = torch.tensor([limit, -limit, 30.0, -30.0], dtype=F64)
    gu[0, 24:28] = torch.tensor([limit, -limit, 30.0, -30.0], dtype=F64)
    want = plain_gated(gu[:, :24].float().to(F64), gu[:, 24:].float().to(F64), limit)
    assert ((gu[:, :24] > limit).any() and (gu[:, 24:] > limit).any() and (gu[:, 24:] < -limit).any())
    close(ops.gate_act_mul(dev(gu.float()), torch.float32, "swish_clamped", limit), want, 1e-6, "fp32")
    close(ops.gate_act_mul(dev(gu.float()), torch.bfloat16, "swish_clamped", limit), want, 1e-2, "fp32 to bf16")
    rounded = bf16_round(gu)
    close(ops.gate_act_mul(dev(rounded.to(torch.bfloat16)), torch.bfloat16, "swish_clamped", limit),
          plain_gated(rounded[:, :24], rounded[:, 24:], limit), 1e-2, "bf16")
    # the other activations are what they were
    close(ops.gate_act_mul(dev(gu.float()), torch.float32, "silu"), gu[:, :24].float().to(F64) * torch.sigmoid(gu[:, :24].float().to(F64))
          * gu[:, 24:].float().to(F64), 1e-6, "silu")


@pytest.mark.parametrize("tokens", [5, 48, 130, 300])
def test_clamped_swish_in_the_fused_gate_up_product(tokens):
    """The tensor-core product of gate and up with the activation in its epilogue, at every token-tile size."""
    from flyweight_b200.kernels import tensorcore
    g = torch.Generator().manual_seed(tokens)
    K, F, limit = 128, 192, 1.5
    x = bf16_round(torch.randn(tokens, K, generator=g, dtype=F64))
    w = bf16_round(torch.randn(2 * F, K, generator=g, dtype=F64) * (3.0 / math.sqrt(K)))
    gate, up = x @ w[:F].T, x @ w[F:].T
    assert (gate > limit).any() and (up > limit).any() and (up < -limit).any()
    xd, wd = dev(x.to(torch.bfloat16)), dev(w.to(torch.bfloat16))
    if not tensorcore.swiglu_accepts(xd, wd):
        pytest.skip("the tensor-core product does not take this shape")
    got = tensorcore.swiglu_gate_up(xd, wd, activation="swish_clamped", limit=limit)
    close(got, plain_gated(gate, up, limit), 1.5e-2, "fused")
    assert (plain_gated(gate, up, 10 * limit) - plain_gated(gate, up, limit)).abs().max() > 1.0


# ------------------------------------------------------------------ parts from a configuration
def tiny_config(**kw):
    att = {"heads": kw.get("heads", 4), "kv_heads": kw.get("kv", 2), "dim": kw.get("dim", 16), "vdim": kw.get("vdim", 24),
           "scale": kw.get("scale", 0.3), "conv": kw.get("conv", 3)}
    if kw.get("chunk"):
        att["mask"] = {"size": kw["chunk"]}
    if kw.get("rot_dims"):
        att["rot"] = {"base": 10000.0, "dims": kw["rot_dims"]}
        if kw.get("scaling", True):
            att["rot"]["scaling"] = ramp(4.0, 64, 8.0, 1.0)
    heads, dim, rot_dim, vdim, rank = kw.get("latent", (3, 8, 8, 20, 24))
    lat = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": kw.get("scale", 0.3),
           "rot": {"base": 500.0, "dims": rot_dim}}
    if kw.get("scaling", True):
        lat["rot"]["scaling"] = ramp(2.0, 32, 4.0, 0.5)
    ff, limit, experts, top, shared = kw.get("mlp", (32, 1.0, 4, 2, (24, 2.0)))
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    return {"architecture": "Fobatar", "vocab": 61, "width": kw.get("width", 48), "norm": {"eps": EPS},
            "embedding": {"scale": 1.0}, "residual_mult": 1.0,
            "layers": [{"type": "attention", "mixer": att, "mlp": mlp}, {"type": "latent_attention", "mixer": lat, "mlp": None}]}


def random_weights(raw, seed, dtype):
    from flyweight_b200.config.fobatar import FobatarConfig
    from flyweight_b200.parts import build_arrangement
    g = torch.Generator().manual_seed(seed)
    spec = FobatarConfig.from_dict(raw).model_spec()
    w = {}
    for layer in spec.layers:
        declared = {}
        for part in build_arrangement(layer).parts():
            declared.update(part.declare())
        for name, decl in declared.items():
            if decl.role == "table":
                order = torch.rand((decl.shape[0], decl.bound), generator=g).argsort(dim=1)
                w[name] = order[:, :decl.shape[1]].to(torch.int32)
                continue
            t = torch.randn(decl.shape, generator=g, dtype=F64)
            if name.endswith(".conv"):
                t = 0.5 * t + 0.5
            elif len(decl.shape) == 2:
                t = t / math.sqrt(decl.shape[1])
            else:
                t = 1.0 + 0.2 * t
            w[name] = bf16_round(t) if dtype == torch.bfloat16 else t.float().to(F64)
    return spec, w


def run_part(part_spec, w, dtype, h_seqs, cuts, n_pages=24, seed=0):
    """A mixer over several sequences fed in the portions ``cuts``; pages in shuffled order, slot = 3 - s.
    Returns the outputs by sequence."""
    from flyweight_b200.engine import Segment, StepBatch, StepContext
    from flyweight_b200.parts import Precision, build_mixer
    from flyweight_b200.parts.base import FixedState, PagedKV
    precision = Precision("float32" if dtype == torch.float32 else "bfloat16")
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    part = build_mixer(part_spec)
    part.bind(lambda n: w[n].to(dtype) if w[n].is_floating_point() else w[n], precision, DEV)
    part.prepare(1024, DEV)
    cache = type("Cache", (), {})()
    cache.k_pool = cache.v_pool = cache.state = None
    cache.group = 0
    specs = part.state_spec()
    for one in specs if isinstance(specs, tuple) else (specs,):
        if isinstance(one, PagedKV):
            shape = (n_pages, one.n_kv_heads, 64, one.head_dim)
            cache.k_pool = torch.full(shape, float("nan"), dtype=precision.cache_dtype, device=DEV)
            if one.values:
                cache.v_pool = torch.full(shape, float("nan"), dtype=precision.cache_dtype, device=DEV)
        elif isinstance(one, FixedState):
            cache.state = torch.zeros((4,) + tuple(one.shape), dtype=one.dtype, device=DEV)
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
        out = part.forward(ctx, h, cache)
        at = 0
        for s, m in step:
            outs[s].append(out[at:at + m].float().cpu())
            at += m
            done[s] += m
    return {s: torch.cat(parts) for s, parts in outs.items() if parts}


def inputs_with_partners(lengths, width, pairs, seed, dtype, strength=6.0, query_sign=1.0):
    """Random rows; for every (sequence, key position, query position) in ``pairs`` both rows get a large
    share of one common direction (the query's with ``query_sign``), so that this query's score on this key
    stands far out."""
    g = torch.Generator().manual_seed(seed)
    seqs = [torch.randn(n, width, generator=g, dtype=F64) for n in lengths]
    for index, (s, j, i) in enumerate(pairs):
        u = torch.randn(width, generator=torch.Generator().manual_seed(1000 + index), dtype=F64)
        seqs[s][j] += strength * u
        seqs[s][i] += query_sign * strength * u
    return [bf16_round(h) if dtype == torch.bfloat16 else h.float().to(F64) for h in seqs]


def tie_queries_to_keys(w, prefix, heads, kv, dim):
    """Makes every query head's projection minus its key head's, and its taps and norm weight the key head's: a
    row that is the opposite of an earlier one then scores high on it, whatever the random weights are, and
    every row scores far below zero on itself (else a row's own key, which no rotation turns against it,
    would outweigh every partner)."""
    rep = heads // kv
    w[prefix + "q"] = -w[prefix + "k"].view(kv, dim, -1).repeat_interleave(rep, dim=0).reshape(heads * dim, -1).clone()
    w[prefix + "q.norm"] = w[prefix + "k.norm"].view(kv, dim).repeat_interleave(rep, dim=0).reshape(-1).clone()
    if prefix + "k.conv" in w:
        taps = w[prefix + "k.conv"]
        w[prefix + "q.conv"] = taps.view(kv, dim, -1).repeat_interleave(rep, dim=0).reshape(heads * dim, -1).clone()


# sequence 0: positions 0-99, 100-101, 102, 103-139, 140, 141, 142-199 (102, 140 and 141 are decoded alone)
CUTS = [[(0, 100), (1, 3)], [(1, 1), (0, 2), (2, 64)], [(0, 1), (1, 1), (2, 1)], [(2, 63), (0, 37), (1, 60)],
        [(0, 1), (2, 2)], [(0, 1)], [(0, 58), (1, 70)]]
LENGTHS = [200, 135, 130]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunk,heads,kv,dim,vdim,conv,rot_dims", [
    (37, 4, 2, 16, 24, 3, 8), (64, 2, 2, 32, 32, 2, 32), (1, 3, 1, 24, 16, 4, 0), (129, 4, 1, 16, 16, 1, 4),
    (0, 2, 1, 16, 16, 3, 16), (50, 8, 2, 64, 64, 2, 32), (70, 4, 1, 128, 128, 3, 64)])
def test_attention_inside_chunks_with_convolutions_zero_sink_and_gate(dtype, chunk, heads, kv, dim, vdim, conv, rot_dims,
                                                                      monkeypatch):
    """The whole mixer over three sequences in portions and single tokens.  Keys stand out at the first place of
    the query's chunk and at the last place of the chunk before, for queries inside a portion and for tokens
    decoded alone; the plain result with the chunk one longer or shorter, or without the sink, must differ by
    far more than the tolerance, else the inputs would prove nothing."""
    # (a scale that keeps a row's score on its partner near 10 whatever the head size: sharper rows would only
    # magnify the 16-bit rounding of queries and keys)
    raw = tiny_config(chunk=chunk, heads=heads, kv=kv, dim=dim, vdim=vdim, conv=conv, rot_dims=rot_dims, scale=10.0 / dim,
                      width=48 if dim < 64 else 128)
    spec, w = random_weights(raw, 3, dtype)
    tie_queries_to_keys(w, "l0.mix.", heads, kv, dim)
    w["l0.mix.g"] = rounding(dtype)(0.25 * w["l0.mix.g"])      # (so that no gate shuts a partner's head)
    # (sequence, query, inside?, decoded alone?): the partner is the first key of the query's chunk, or the last of
    # the chunk before; every partner row serves one query only
    pairs, kinds = [], {}
    if chunk > 1:
        for s, i, inside, alone in ((0, 102, True, True), (0, 150, False, False), (2, 110, True, False), (2, 64, False, True)):
            first = i - i % chunk
            j = first if inside else first - 1
            if 0 <= j < i:
                pairs.append((s, j, i))
                kinds[(s, i)] = alone
    seqs = inputs_with_partners(LENGTHS, raw["width"], pairs, 7, dtype, query_sign=-1.0)
    rnd = rounding(dtype)
    m = raw["layers"][0]["mixer"]
    got = run_part(spec.layers[0].parts["mixer"], w, dtype, seqs, CUTS)
    shown, flipped = set(), set()
    for s, h in enumerate(seqs):
        pos = torch.arange(h.shape[0])
        want = P.chunked_attention_mixer(h, w, "l0.mix.", m, EPS, pos, rnd=rnd)
        close(got[s], want, TOL[dtype], f"sequence {s}")
        for delta in (-1, 1) if chunk > 1 else ():
            other = dict(m, mask={"size": chunk + delta})
            off = P.chunked_attention_mixer(h, w, "l0.mix.", other, EPS, pos, rnd=rnd)
            for q, j, i in pairs:
                flips = (j // chunk == i // chunk) != (j // (chunk + delta) == i // (chunk + delta))
                if q == s and flips:
                    flipped.add((s, i, delta))
                    if (off[i] - want[i]).abs().max() > SHOWS * max(1.0, want.abs().max()):
                        shown.add((s, i, delta))
    if chunk > 1:
        assert flipped and shown == flipped, "an edge that is one off must show wherever it changes what a query sees"
        if chunk < 100:
            assert {kinds[(s, i)] for s, i, _ in shown} == {True, False}     # in a portion, and decoded alone
    # the sink: a query at its chunk's first place would otherwise weigh its only key by one
    h, pos = seqs[1], torch.arange(LENGTHS[1])
    q_like = P.chunked_attention_mixer(h, w, "l0.mix.", m, EPS, pos, rnd=rnd)
    monkeypatch.setattr(P, "softmax_attention", _no_sink)
    no_sink = P.chunked_attention_mixer(h, w, "l0.mix.", m, EPS, pos, rnd=rnd)
    assert (no_sink - q_like).abs().max() > SHOWS * max(1.0, q_like.abs().max())


_plain_softmax_attention = P.softmax_attention


def _no_sink(q, k, v, q_pos, k_pos, scale, chunk=0, sink_zero=False):
    return _plain_softmax_attention(q, k, v, q_pos, k_pos, scale, chunk, sink_zero=False)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("latent", [(3, 8, 8, 20, 24), (2, 16, 4, 8, 40), (8, 32, 16, 32, 48), (4, 64, 32, 64, 96),
                                    (5, 24, 8, 56, 72), (2, 32, 32, 48, 160), (1, 16, 2, 16, 12)])
@pytest.mark.parametrize("scaling", [True, False])
def test_latent_attention_with_gate_and_scaled_rotation(dtype, latent, scaling):
    """Rows of 32 to 192 entries (the paged tensor-core kernels and the 32-bit kernel), plain softmax, a gate per
    head, the rotated part turned with ramped frequencies and their amplitude.  One key far back (position 2,
    asked for from a portion and by decoded tokens up to 197 later) stands out."""
    raw = tiny_config(latent=latent, scaling=scaling, scale=0.8, width=64)
    spec, w = random_weights(raw, 5, dtype)
    pairs = [(0, 2, 95), (0, 2, 102), (0, 2, 199), (1, 0, 134)]
    seqs = inputs_with_partners(LENGTHS, raw["width"], pairs, 9, dtype, strength=3.0)
    rnd = rounding(dtype)
    m = raw["layers"][1]["mixer"]
    got = run_part(spec.layers[1].parts["mixer"], w, dtype, seqs, CUTS, seed=2)
    for s, h in enumerate(seqs):
        pos = torch.arange(h.shape[0])
        want = P.latent_attention_mixer(h, w, "l1.mix.", m, EPS, pos, rnd=rnd)
        close(got[s], want, TOL[dtype], f"sequence {s}")
    # the gate and the amplitude are felt: the plain result without either is another
    h, pos = seqs[0], torch.arange(LENGTHS[0])
    base = P.latent_attention_mixer(h, w, "l1.mix.", m, EPS, pos, rnd=rnd)
    open_gate = dict(w)
    open_gate["l1.mix.g"] = torch.zeros_like(w["l1.mix.g"])
    assert (P.latent_attention_mixer(h, open_gate, "l1.mix.", m, EPS, pos, rnd=rnd) - base).abs().max() > SHOWS * base.abs().max()
    if scaling:
        flat = dict(m, rot={"base": m["rot"]["base"], "dims": m["rot"]["dims"]})
        assert (P.latent_attention_mixer(h, w, "l1.mix.", flat, EPS, pos, rnd=rnd) - base).abs().max() > SHOWS * base.abs().max()


# ------------------------------------------------------------------ experts chosen by the token's id
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tensor_cores", [True, False])
@pytest.mark.parametrize("mlp,width", [((32, 1.0, 4, 2, (24, 2.0)), 48), ((64, 0.5, 6, 1, None), 64), ((16, 3.0, 3, 3, (8, 0.75)), 40),
                                       ((128, 1.5, 9, 4, (96, 1.0)), 128), ((20, 2.0, 5, 2, (12, 2.0)), 36)])
def test_experts_by_table_with_a_shared_expert(dtype, tensor_cores, mlp, width):
    """Two segments (a prompt's portion and one that starts in mid-sequence), 1 to all experts a token, an expert
    that no token of the step names, both product kernels; limits small enough that the clamps act."""
    from flyweight_b200.engine import Segment, StepBatch, StepContext
    from flyweight_b200.kernels import experts as expert_kernels
    from flyweight_b200.parts import Precision
    from flyweight_b200.parts.base import build_feed_forward
    raw = tiny_config(mlp=mlp, width=width)
    spec, w = random_weights(raw, 17, dtype)
    E, top = mlp[2], mlp[3]
    g = torch.Generator().manual_seed(2)
    tokens = [int(t) for t in torch.randint(0, raw["vocab"], (150,), generator=g)]
    if top < E:
        # nobody names the last expert in this step
        w["l0.mlp.table"] = (w["l0.mlp.table"].to(torch.int64) % (E - 1)).to(torch.int32) if top == 1 else w["l0.mlp.table"]
    precision = Precision("float32" if dtype == torch.float32 else "bfloat16")
    rnd = rounding(dtype)
    batch = StepBatch([Segment("a", 0, 0, tokens[:140], []), Segment("b", 1, 7, tokens[140:], [])], [[[0], [1]]], DEV)
    ctx = StepContext(batch, precision, DEV)
    h = 2.0 * torch.randn(150, width, generator=g, dtype=F64).float().to(F64)
    ff = build_feed_forward(spec.layers[0].parts["feed_forward"])
    ff.bind(lambda n: w[n].to(dtype) if w[n].is_floating_point() else w[n], precision, DEV)
    expert_kernels.set_tensor_cores(tensor_cores)
    try:
        got = ff.forward(ctx, dev(rnd(h).to(precision.act_dtype)))
    finally:
        expert_kernels.set_tensor_cores(True)
    want = P.table_experts(h, tokens, w, "l0.mlp.", raw["layers"][0]["mlp"], rnd=rnd)
    close(got, want, TOL[dtype], "experts")
    # the same with the output norm and the residual sum in the kernel that adds the experts up
    x0 = torch.randn(150, width, generator=g, dtype=F64).float().to(F64)
    norm_w = (1.0 + 0.2 * torch.randn(width, generator=g, dtype=F64)).float().to(F64)
    x = dev(x0.float())
    ff.forward_add_normed(ctx, dev(rnd(h).to(precision.act_dtype)), x, dev(norm_w.float()), EPS)
    close(x, x0 + P.unit(want, EPS) * norm_w, TOL[dtype], "experts, normed and added")
    loose = {"kind": "moe", "expert": {"ff": mlp[0], "limit": 50.0}, "router": raw["layers"][0]["mlp"]["router"]}
    if mlp[4]:
        loose["shared"] = {"ff": mlp[4][0], "limit": 50.0}
    assert (P.table_experts(h, tokens, w, "l0.mlp.", loose, rnd=rnd) - want).abs().max() > SHOWS * max(1.0, want.abs().max())


def test_the_table_router_names_a_row_per_token():
    from flyweight_b200.kernels import experts as expert_kernels
    g = torch.Generator().manual_seed(4)
    table = torch.rand((50, 7), generator=g).argsort(dim=1)[:, :3].to(torch.int32)
    tokens = torch.randint(0, 50, (200,), generator=g).to(torch.int32)
    ids, weights = expert_kernels.route_table(dev(tokens), dev(table), 3)
    assert torch.equal(ids.cpu(), table[tokens.long()])
    assert torch.equal(weights.cpu(), torch.full((200, 3), 1.0 / 3.0, dtype=torch.float32))
