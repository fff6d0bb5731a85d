"""Fobatar without a GPU: the typed configuration (keys, checks, the model in parts, the schedule of repeated
layers, the tensors it declares), the registry, random model folders, the rotation's frequency ramp, and
properties of the plain implementation that the GPU tests lean on."""
import copy
import math

import pytest
import torch

import plain_fobatar as P
from tiny_configs import TINY, make_model_dir

F64 = torch.float64
NAMES = ("FA", "FB", "FC", "FD", "FE")


def typed(raw):
    from flyweight_b200.config.fobatar import FobatarConfig
    return FobatarConfig.from_dict(raw)


def test_the_registry_finds_the_architecture_by_either_key():
    import flyweight_b200.models  # noqa: F401
    from flyweight_b200.config import architecture_name, lookup
    raw = TINY["FA"]
    assert architecture_name(raw) == "Fobatar"
    assert architecture_name({"architectures": ["Fobatar"]}) == "Fobatar"
    assert lookup("Fobatar").config_class.from_dict(raw).to_dict() == typed(raw).to_dict()


@pytest.mark.parametrize("name", NAMES)
def test_the_model_in_parts_follows_the_configuration(name):
    raw = TINY[name]
    config = typed(raw)
    back = config.to_dict()
    assert back["layers"] == raw["layers"] and back["vocab"] == raw["vocab"] and back["width"] == raw["width"]
    assert back["residual_mult"] == raw.get("residual_mult", 1.0)
    assert back["embedding"]["scale"] == (raw.get("embedding") or {}).get("scale", 1.0)
    assert back.get("loop") == raw.get("loop")
    spec = config.model_spec()
    mult, eps = raw.get("residual_mult", 1.0), raw["norm"]["eps"]
    assert spec.vocab_size == raw["vocab"] and spec.hidden_size == raw["width"] and spec.head_tensor is None
    assert spec.embedding_scale == (raw.get("embedding") or {}).get("scale", 1.0)
    for index, (layer, given) in enumerate(zip(spec.layers, raw["layers"])):
        assert layer.arrangement == "sandwich_residual"
        has_ff = given["mlp"] is not None
        assert ("feed_forward" in layer.parts) == has_ff == ("ffn_norm" in layer.parts) == ("ffn_out_norm" in layer.parts)
        # the constant on the residual sums rides on the norm behind a sublayer, never on the one in front
        assert layer.parts["mixer_norm"].params == {"size": raw["width"], "eps": eps}
        assert layer.parts["mixer_out_norm"].params.get("gain", 1.0) == mult
        mixer, m = layer.parts["mixer"], given["mixer"]
        p = mixer.params
        rot = m.get("rot")
        if given["type"] == "attention":
            assert mixer.kind == "gqa_attention"
            assert (p["num_heads"], p["num_kv_heads"], p["head_dim"], p["value_dim"], p["scale"]) == \
                (m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"])
            assert p["chunk"] == (m.get("mask") or {}).get("size", 0) and p["conv"] == m.get("conv", 0)
            assert (p["qk_norm"], p["gate"], p["sink"], p["qk_norm_eps"]) == ("whole", "head", "zero", eps)
            dims = rot["dims"] if rot else 0
        else:
            assert mixer.kind == "latent_attention"
            assert (p["num_heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"], p["scale"]) == \
                (m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"])
            assert (p["gate"], p["sink"], p["eps"]) == ("head", False, eps)
            dims = m["rot_dim"]
        if rot and dims:
            assert p["position"].kind == "rope" and p["position"].params["pairing"] == "interleaved"
            assert p["position"].params["rotary_dim"] == dims and p["position"].params["theta"] == rot["base"]
            assert p["position"].params.get("scaling") == rot.get("scaling")
        else:
            assert p["position"].kind == "no_position"
        if has_ff:
            ff, g = layer.parts["feed_forward"], given["mlp"]
            assert ff.kind == "table_experts"
            assert (ff.params["ffn_dim"], ff.params["limit"], ff.params["experts"], ff.params["top"]) == \
                (g["expert"]["ff"], g["expert"]["limit"], g["router"]["experts"], g["router"]["top"])
            assert ff.params["activation"] == "swish_clamped" and ff.params["vocab_size"] == raw["vocab"]
            assert ("shared_ffn_dim" in ff.params) == ("shared" in g) == ("shared_gate" in ff.tensors)
            if "shared" in g:
                assert (ff.params["shared_ffn_dim"], ff.params["shared_limit"]) == (g["shared"]["ff"], g["shared"]["limit"])
            assert layer.parts["ffn_out_norm"].params.get("gain", 1.0) == mult


@pytest.mark.parametrize("name", NAMES)
def test_the_schedule_repeats_the_looped_layers_with_caches_of_their_own(name):
    raw = TINY[name]
    spec = typed(raw).model_spec()
    n = len(raw["layers"])
    loop = raw.get("loop")
    if loop is None:
        want = [(i, False) for i in range(n)]
    else:
        want = [(i, False) for i in range(loop["start"])]
        for again in range(loop["times"]):
            want += [(i, again > 0 and i == loop["start"]) for i in range(loop["start"], loop["stop"])]
        want += [(i, False) for i in range(loop["stop"], n)]
    assert [(entry.layer, entry.add_embedding) for entry in spec.schedule] == want == P.layer_runs(raw)
    assert all(entry.cache_of is None for entry in spec.schedule)
    # every execution keeps a cache of its own
    from flyweight_b200.cache.manager import CacheManager
    from flyweight_b200.models import FobatarForCausalLM
    from flyweight_b200.parts import Precision
    model = FobatarForCausalLM(typed(raw), Precision("float32"), torch.device("cpu"))
    manager = CacheManager(model.state_specs(), num_pages=4, num_slots=2, device=None)
    assert len(manager.layer_caches) == len(want)
    assert sum(len(group.members) for group in manager.groups) == len(want)


def test_declared_tensors_and_their_shapes():
    from flyweight_b200.models import FobatarForCausalLM
    from flyweight_b200.parts import Precision
    from flyweight_b200.parts.base import FixedState, PagedKV
    raw = TINY["FA"]
    model = FobatarForCausalLM(typed(raw), Precision("float32"), torch.device("cpu"))
    declared = {name: tuple(decl.shape) for name, decl in model.declare().items()}
    W = raw["width"]
    assert declared["embed"] == (raw["vocab"], W) and "head" not in declared and declared["final.norm"] == (W,)
    for i, given in enumerate(raw["layers"]):
        assert declared[f"l{i}.norm1"] == declared[f"l{i}.norm1b"] == (W,)
        assert (f"l{i}.norm2" in declared) == (f"l{i}.norm2b" in declared) == (given["mlp"] is not None)
    a = raw["layers"][0]["mixer"]
    H, G, d, e, taps = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["conv"]
    assert declared["l0.mix.q"] == (H * d, W) and declared["l0.mix.k"] == (G * d, W)
    assert declared["l0.mix.v"] == (G * e, W) and declared["l0.mix.o"] == (W, H * e)
    assert declared["l0.mix.q.norm"] == (H * d,) and declared["l0.mix.k.norm"] == (G * d,)
    assert declared["l0.mix.q.conv"] == (H * d, taps) and declared["l0.mix.k.conv"] == (G * d, taps)
    assert declared["l0.mix.v.conv"] == (G * e, taps) and declared["l0.mix.g"] == (H, W)
    assert "l0.mix.sink" not in declared
    g = raw["layers"][0]["mlp"]
    assert declared["l0.mlp.table"] == (raw["vocab"], g["router"]["top"])
    for j in range(g["router"]["experts"]):
        assert declared[f"l0.mlp.e{j}.gate"] == declared[f"l0.mlp.e{j}.up"] == (g["expert"]["ff"], W)
        assert declared[f"l0.mlp.e{j}.down"] == (W, g["expert"]["ff"])
    assert f"l0.mlp.e{g['router']['experts']}.gate" not in declared
    assert declared["l0.mlp.shared.gate"] == declared["l0.mlp.shared.up"] == (g["shared"]["ff"], W)
    assert declared["l0.mlp.shared.down"] == (W, g["shared"]["ff"])
    assert "l1.mlp.shared.gate" not in declared and "l2.mlp.table" not in declared
    b = raw["layers"][1]["mixer"]
    assert declared["l1.mix.q"] == (b["heads"] * (b["dim"] + b["rot_dim"]), W)
    assert declared["l1.mix.dkv"] == (b["kv_rank"] + b["rot_dim"], W) and declared["l1.mix.dkv.norm"] == (b["kv_rank"],)
    assert declared["l1.mix.uk"] == (b["heads"] * b["dim"], b["kv_rank"])
    assert declared["l1.mix.uv"] == (b["heads"] * b["vdim"], b["kv_rank"])
    assert declared["l1.mix.g"] == (b["heads"], W) and declared["l1.mix.o"] == (W, b["heads"] * b["vdim"])
    # what a request keeps: pages and the convolutions' last inputs for attention, one row pool for a latent layer
    pages, rolling = model.layers[0].state_spec()
    D = -(-max(d, e) // 16) * 16
    assert isinstance(pages, PagedKV) and (pages.n_kv_heads, pages.head_dim, pages.window) == (G, D, 0)
    assert isinstance(rolling, FixedState) and rolling.shape == (taps - 1, (H + 2 * G) * D)
    rows = model.layers[1].state_spec()
    assert isinstance(rows, PagedKV) and rows.values is False and rows.head_dim >= b["kv_rank"] + b["rot_dim"]
    # one tap keeps nothing; no convolution keeps nothing
    for name, index in (("FB", 3), ("FE", 2)):
        other = FobatarForCausalLM(typed(TINY[name]), Precision("float32"), torch.device("cpu"))
        assert isinstance(other.layers[index].state_spec(), PagedKV)


def test_a_random_model_folder_loads_back_and_its_tables_name_different_experts(tmp_path):
    folder = make_model_dir(tmp_path / "m", TINY["FA"], seed=11, dtype=torch.bfloat16)
    cfg, w = P.load_model_dir(folder)
    assert cfg["architecture"] == "Fobatar" and cfg["loop"] == TINY["FA"]["loop"]
    for index, layer in enumerate(cfg["layers"]):
        if layer["mlp"] is None:
            continue
        table = w[f"l{index}.mlp.table"]
        assert not table.is_floating_point() and tuple(table.shape) == (cfg["vocab"], layer["mlp"]["router"]["top"])
        assert int(table.min()) >= 0 and int(table.max()) < layer["mlp"]["router"]["experts"]
        assert all(len(set(row.tolist())) == len(row) for row in table)
        if layer["mlp"]["router"]["experts"] > layer["mlp"]["router"]["top"]:
            assert len({tuple(row.tolist()) for row in table}) > 1
    from flyweight_b200.models import FobatarForCausalLM
    from flyweight_b200.parts import Precision
    from flyweight_b200.weights import load_checkpoint
    model = FobatarForCausalLM(typed(cfg), Precision("bfloat16"), torch.device("cpu"))
    model.load(load_checkpoint(folder, model.declare(), model.spec.unused_tensors))
    assert model.head is model.embedding


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "missing fast"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unknown feed-forward"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top exceeds"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "missing limit"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "missing kv_rank"),
    (lambda c: c["loop"].update(stop=9), "'loop'"),
    (lambda c: c["loop"].update(times=0), "'loop'"),
    (lambda c: c.pop("norm"), "missing norm"),
])
def test_a_configuration_that_does_not_fit_is_refused_with_its_reason(change, message):
    from flyweight_b200.config.lfm2 import ConfigError
    raw = copy.deepcopy(TINY["FA"])
    change(raw)
    with pytest.raises(ConfigError, match=message):
        typed(raw)


@pytest.mark.parametrize("rot", [
    {"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}},
    {"base": 1000000.0, "dims": 32, "scaling": {"factor": 16.0, "original": 256, "fast": 16.0, "slow": 2.0}},
    {"base": 50.0, "dims": 4, "scaling": {"factor": 3.0, "original": 8, "fast": 1.5, "slow": 0.5}},
    {"base": 300.0, "dims": 20},
])
def test_the_rotation_table_follows_the_ramp_and_its_amplitude(rot):
    from flyweight_b200.config.spec import PartSpec
    from flyweight_b200.parts.rope import Rope
    params = {"theta": rot["base"], "rotary_dim": rot["dims"], "pairing": "interleaved"}
    if "scaling" in rot:
        params["scaling"] = rot["scaling"]
    part = Rope(PartSpec("rope", params))
    f, amplitude = P.banded_frequencies(rot)
    assert torch.allclose(part.frequencies(), torch.tensor(f, dtype=F64), rtol=1e-14, atol=0)
    assert part.amplitude() == pytest.approx(amplitude, rel=1e-15)
    table = part.table(300, "cpu").to(F64)
    angle = torch.arange(300, dtype=F64)[:, None] * torch.tensor(f, dtype=F64)[None, :]
    assert torch.allclose(table[..., 0], amplitude * torch.cos(angle), atol=1e-6)
    assert torch.allclose(table[..., 1], amplitude * torch.sin(angle), atol=1e-6)
    if "scaling" in rot:
        plain = [rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)]
        ratios = [a / b for a, b in zip(f, plain)]
        # the fastest pairs keep their frequency or the slowest are divided by the factor (both, when the ramp fits)
        assert all(1.0 / rot["scaling"]["factor"] - 1e-12 <= r <= 1.0 + 1e-12 for r in ratios)
        assert ratios == sorted(ratios, reverse=True) and amplitude > 1.0


# ------------------------------------------------------------------ the plain implementation itself
def test_plain_chunks_sink_and_taps():
    torch.manual_seed(0)
    T, H, G, d, e = 20, 4, 2, 6, 5
    q, k, v = torch.randn(T, H, d, dtype=F64), torch.randn(T, G, d, dtype=F64), torch.randn(T, G, e, dtype=F64)
    pos = torch.arange(T)
    whole = P.softmax_attention(q, k, v, pos, pos, 0.4, chunk=7, sink_zero=True)
    # a query's row changes only with keys of its own chunk at or before it
    k2, v2 = k.clone(), v.clone()
    k2[:7], v2[:7] = 5.0, -3.0
    k2[10:], v2[10:] = 9.0, 2.0
    again = P.softmax_attention(q, k2, v2, pos, pos, 0.4, chunk=7, sink_zero=True)
    assert torch.equal(again[7:10], whole[7:10]) and not torch.allclose(again[10:], whole[10:])
    # the sink: weights sum to less than one, by exactly 1 / (1 + sum exp(s))
    ones = torch.ones(T, G, 1, dtype=F64)
    mass = P.softmax_attention(q, k, ones, pos, pos, 0.4, chunk=7, sink_zero=True)[:, 0, 0]
    for i in (0, 6, 7, 13, 19):
        first = i - i % 7
        s = (q[i, 0] @ k[first:i + 1, 0].T) * 0.4
        assert mass[i].item() == pytest.approx((torch.exp(s).sum() / (1.0 + torch.exp(s).sum())).item(), rel=1e-12)
    # taps: the last tap is on the token itself, history continues a sequence
    u, taps = torch.randn(9, 3, dtype=F64), torch.randn(3, 4, dtype=F64)
    y = P.causal_taps(u, taps)
    assert torch.allclose(y[0], taps[:, 3] * u[0]) and torch.allclose(y[1], taps[:, 3] * u[1] + taps[:, 2] * u[0])
    assert torch.allclose(P.causal_taps(u[5:], taps, history=u[2:5]), y[5:])


def test_plain_expert_clamps_and_the_table_weighs_evenly():
    h = torch.tensor([[1.0, -2.0]], dtype=F64)
    gate, up, down = torch.tensor([[3.0, 0.0]], dtype=F64), torch.tensor([[0.0, 4.0]], dtype=F64), torch.eye(1, dtype=F64)
    # gate h = 3 -> cut to 2; up h = -8 -> held at -2; 2 sigmoid(3.404) (-2 + 1)
    got = P.clamped_gated_expert(h, gate, up, down, 2.0)[0, 0].item()
    assert got == pytest.approx(-2.0 / (1.0 + math.exp(-1.702 * 2.0)), rel=1e-12)
    # a negative gate is not cut
    got = P.clamped_gated_expert(-h, gate, up, down, 2.0)[0, 0].item()
    assert got == pytest.approx(-3.0 / (1.0 + math.exp(1.702 * 3.0)) * 3.0, rel=1e-12)
    for name in NAMES:
        runs = P.layer_runs(TINY[name])
        assert len(runs) >= len(TINY[name]["layers"]) and not runs[0][1]


@pytest.mark.parametrize("name", ("FA", "FB"))
def test_plain_logits_are_causal_and_the_loop_counts(name, tmp_path):
    folder = make_model_dir(tmp_path / "m", TINY[name], seed=5, dtype=torch.float32)
    cfg, w = P.load_model_dir(folder)
    tokens = [int(t) for t in torch.randint(0, cfg["vocab"], (30,), generator=torch.Generator().manual_seed(1))]
    runs = []
    full = P.forward(cfg, w, tokens, layers_out=runs)
    assert len(runs) == len(P.layer_runs(cfg))
    changed = list(tokens)
    changed[20] = (changed[20] + 1) % cfg["vocab"]
    other = P.forward(cfg, w, changed)
    assert torch.equal(other[:20], full[:20]) and not torch.allclose(other[20:], full[20:])
    once = copy.deepcopy(cfg)
    once["loop"]["times"] = 1
    assert not torch.allclose(P.forward(once, w, tokens), full)
