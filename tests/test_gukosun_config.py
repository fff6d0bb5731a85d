"""Gukosun without a GPU: the typed configuration (keys, checks, the model in parts, the tensors it
declares), the registry, random model folders, and properties of the plain implementation that the GPU
tests lean on."""
import copy
import math

import pytest
import torch

import plain_gukosun as P
from tiny_configs import TINY, make_model_dir

F64 = torch.float64
NAMES = ("GA", "GB", "GC", "GD", "GE")


def typed(raw):
    from flyweight_b200.config.gukosun import GukosunConfig
    return GukosunConfig.from_dict(raw)


def test_the_registry_finds_the_architecture_by_either_key():
    import flyweight_b200.models  # noqa: F401
    from flyweight_b200.config import architecture_name, lookup
    raw = TINY["GA"]
    assert architecture_name(raw) == "Gukosun"
    assert architecture_name({"architectures": ["Gukosun"]}) == "Gukosun"
    assert lookup("Gukosun").config_class.from_dict(raw).to_dict() == typed(raw).to_dict()


@pytest.mark.parametrize("name", NAMES)
def test_the_model_in_parts_follows_the_configuration(name):
    raw = TINY[name]
    config = typed(raw)
    back = config.to_dict()
    assert back["layers"] == raw["layers"] and back["vocab"] == raw["vocab"] and back["width"] == raw["width"]
    assert back["logit_scale"] == raw.get("logit_scale", 1.0)
    assert back.get("token_side") == raw.get("token_side")
    spec = config.model_spec()
    assert spec.vocab_size == raw["vocab"] and spec.hidden_size == raw["width"] and spec.head_tensor == "head"
    assert spec.logit_scale == raw.get("logit_scale", 1.0)
    source_seen = False
    for index, (layer, given) in enumerate(zip(spec.layers, raw["layers"])):
        assert layer.arrangement == "parallel_residual"
        assert ("feed_forward" in layer.parts) == (given["mlp"] is not None) == ("ffn_scale" in layer.parts)
        assert ("side" in layer.parts) == bool(raw.get("token_side"))
        if "side" in layer.parts:
            side = layer.parts["side"].params
            assert (side["dim"], side["index"], side["count"]) == (raw["token_side"]["dim"], index, len(raw["layers"]))
        if given["mlp"] is not None:
            assert layer.parts["feed_forward"].params == {"hidden_size": raw["width"], "ffn_dim": given["mlp"]["ff"],
                                                          "activation": "relu_squared"}
        mixer = layer.parts["mixer"]
        if given["type"] == "attention":
            m, p = given["mixer"], mixer.params
            assert mixer.kind == "gqa_attention"
            assert (p["num_heads"], p["num_kv_heads"], p["head_dim"], p["value_dim"], p["scale"]) == \
                (m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"])
            assert p["window"] == (m.get("mask") or {}).get("size", 0)
            assert (p["qk_norm"], p["gate"], p["sink"], p["softcap"]) == ("head", "element", True, 0.0)
            assert p["position"].kind == "no_position"
            role = None
            if m.get("v_mix"):
                role = "mixed" if source_seen else "source"
                source_seen = True
            assert p["value_mix"] == role and ("vmix" in mixer.tensors) == (role == "mixed")
        else:
            assert mixer.kind == "mixer_pair"
            left, right = mixer.params["left"], mixer.params["right"]
            m, p = given["mixer"]["left"], left.params
            assert left.kind == "gqa_attention" and right.kind == "decayed_linear_attention"
            assert (p["num_heads"], p["num_kv_heads"], p["head_dim"], p["value_dim"], p["scale"]) == \
                (m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"])
            assert (p["qk_norm"], p["gate"], p["sink"], p["window"]) == ("whole", "head", True, 0)
            assert p["softcap"] == m.get("softcap", 0.0) and p["value_mix"] is None
            if m.get("rot"):
                assert p["position"].kind == "rope" and p["position"].params["pairing"] == "interleaved"
                assert p["position"].params["rotary_dim"] == m["rot"]["dims"]
                assert ("scaling" in p["position"].params) == ("scaling" in m["rot"])
            else:
                assert p["position"].kind == "no_position"
            r, q = given["mixer"]["right"], right.params
            assert (q["num_heads"], q["dim"], q["vdim"], list(q["decay"])) == (r["heads"], r["dim"], r["vdim"], list(r["decay"]))


def test_declared_tensors_and_their_shapes():
    from flyweight_b200.models import GukosunForCausalLM
    from flyweight_b200.parts import Precision
    raw = TINY["GA"]
    model = GukosunForCausalLM(typed(raw), Precision("float32"), torch.device("cpu"))
    declared = {name: tuple(decl.shape) for name, decl in model.declare().items()}
    W, n_layers, side = raw["width"], len(raw["layers"]), raw["token_side"]["dim"]
    assert declared["embed"] == (raw["vocab"], W) and declared["head"] == (raw["vocab"], W)
    assert declared["final.norm"] == (W,) and declared["side.embed"] == (raw["vocab"], n_layers * side)
    for i in range(n_layers):
        assert declared[f"l{i}.norm1"] == declared[f"l{i}.ls1"] == (W,)
        assert declared[f"l{i}.side.gate"] == (side, W) and declared[f"l{i}.side.proj"] == (W, side)
        assert declared[f"l{i}.side.norm"] == (W,)
    left, right = raw["layers"][0]["mixer"]["left"], raw["layers"][0]["mixer"]["right"]
    H, G, d, e = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
    assert declared["l0.mix.left.q"] == (H * d, W) and declared["l0.mix.left.k"] == (G * d, W)
    assert declared["l0.mix.left.v"] == (G * e, W) and declared["l0.mix.left.o"] == (W, H * e)
    assert declared["l0.mix.left.q.norm"] == (H * d,) and declared["l0.mix.left.k.norm"] == (G * d,)
    assert declared["l0.mix.left.sink"] == (H,) and declared["l0.mix.left.g"] == (H, W)
    assert declared["l0.mix.left.out"] == declared["l0.mix.right.out"] == (W,)
    assert declared["l0.mix.right.q"] == declared["l0.mix.right.k"] == (right["heads"] * right["dim"], W)
    assert declared["l0.mix.right.v"] == declared["l0.mix.right.g"] == (right["heads"] * right["vdim"], W)
    assert declared["l0.mix.right.norm"] == (right["heads"] * right["vdim"],)
    assert declared["l0.mix.right.o"] == (W, right["heads"] * right["vdim"])
    a = raw["layers"][1]["mixer"]
    assert declared["l1.mix.q"] == (a["heads"] * a["dim"], W) and declared["l1.mix.v"] == (a["kv_heads"] * a["vdim"], W)
    assert declared["l1.mix.q.norm"] == declared["l1.mix.k.norm"] == (a["dim"],)
    assert declared["l1.mix.g"] == (a["heads"] * a["vdim"], W) and declared["l1.mix.sink"] == (a["heads"],)
    # the first mixing layer is the source and reads no weight; a layer that does not mix has none; later ones do
    assert "l1.mix.vmix" not in declared and "l2.mix.vmix" not in declared and "l3.mix.vmix" in declared
    assert "l2.mlp.up" not in declared and "l2.ls2" not in declared and declared["l1.mlp.up"] == (raw["layers"][1]["mlp"]["ff"], W)
    # what a request keeps: pages of the left half and the right half's matrices for a pair, pages for a window
    pages, state = model.layers[0].state_spec()
    assert (pages.n_kv_heads, pages.head_dim, pages.window) == (G, -(-max(d, e) // 16) * 16, 0)
    entries = right["heads"] * right["dim"] * right["vdim"]
    assert state.shape == (-(-entries // 4) * 4,)
    pages = model.layers[1].state_spec()
    assert (pages.n_kv_heads, pages.head_dim, pages.window) == (a["kv_heads"], max(a["dim"], a["vdim"]), a["mask"]["size"])


def _broken(edit):
    raw = copy.deepcopy(TINY["GA"])
    edit(raw)
    return raw


@pytest.mark.parametrize("edit,message", [
    (lambda r: r.pop("width"), "missing width"),
    (lambda r: r["norm"].pop("eps"), "missing eps"),
    (lambda r: r["layers"][0].update(type="mamba"), "unknown type"),
    (lambda r: r["layers"][1]["mixer"].pop("scale"), "missing scale"),
    (lambda r: r["layers"][1]["mixer"].update(heads=7), "multiple of kv_heads"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("original"), "missing original"),
    (lambda r: r["layers"][0]["mixer"]["left"].update(softcap=-1.0), "softcap"),
    (lambda r: r["layers"][0]["mixer"].pop("right"), "missing right"),
    (lambda r: r["layers"][0]["mixer"]["right"].update(decay=[0.5]), "one decay per head"),
    (lambda r: r["layers"][3]["mixer"].update(vdim=8), "mixes values"),
    (lambda r: r["layers"][1]["mlp"].update(kind="sparse"), "unknown feed-forward"),
    (lambda r: r["layers"][1]["mixer"]["mask"].update(size=0), "size must be positive"),
    (lambda r: r.update(layers=[]), "at least one layer"),
])
def test_a_configuration_that_does_not_fit_is_refused_with_its_reason(edit, message):
    from flyweight_b200.config import ConfigError
    with pytest.raises(ConfigError, match=message):
        typed(_broken(edit))


def test_a_random_model_folder_loads_and_runs_in_the_plain_implementation(tmp_path):
    make_model_dir(tmp_path / "m", TINY["GB"], seed=1, preset="unit", dtype=torch.bfloat16)
    config, weights = P.load_model_dir(tmp_path / "m")
    assert config["layers"] == TINY["GB"]["layers"]
    logits = P.forward(config, weights, [1, 2, 3, 4, 5])
    assert logits.shape == (5, TINY["GB"]["vocab"]) and torch.isfinite(logits).all()


# ------------------------------------------------------------------ the plain implementation itself
def test_plain_frequency_scaling_has_three_bands():
    rot = {"base": 10000.0, "dims": 32, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}
    plain = P.rotary_frequencies({"base": 10000.0, "dims": 32})
    scaled = P.rotary_frequencies(rot)
    wave = 2 * math.pi / plain
    short, long = wave < 64 / 4.0, wave > 64 / 1.0
    assert short.any() and long.any() and (~short & ~long).any()
    assert torch.equal(scaled[short], plain[short])
    assert torch.allclose(scaled[long], plain[long] / 4.0, rtol=1e-15)
    between = ~short & ~long
    assert ((scaled[between] > plain[between] / 4.0) & (scaled[between] < plain[between])).all()


def test_plain_rotation_turns_neighbouring_channels_and_leaves_the_rest():
    x = torch.zeros(1, 1, 8, dtype=F64)
    x[0, 0, 0] = 1.0
    x[0, 0, 5] = 3.0
    out = P.rotate_pairs(x, torch.tensor([2]), {"base": 100.0, "dims": 4})
    assert torch.allclose(out[0, 0, :2], torch.tensor([math.cos(2.0), math.sin(2.0)], dtype=F64))
    assert out[0, 0, 5] == 3.0 and out[0, 0, 2:5].abs().sum() == 0
    q = torch.randn(6, 2, 8, generator=torch.Generator().manual_seed(0), dtype=F64)
    pos = torch.arange(6)
    rot = {"base": 50.0, "dims": 8}
    a, b = P.rotate_pairs(q, pos, rot), P.rotate_pairs(q, pos + 11, rot)
    # scores depend on the distance of two positions only
    assert torch.allclose((a[4] * a[1]).sum(-1), (b[4] * b[1]).sum(-1), atol=1e-12)


def test_plain_sink_window_and_cap():
    g = torch.Generator().manual_seed(3)
    q = torch.randn(9, 2, 4, generator=g, dtype=F64)
    k = torch.randn(9, 1, 4, generator=g, dtype=F64)
    v = torch.randn(9, 1, 3, generator=g, dtype=F64)
    pos = torch.arange(9)
    far = torch.full((2,), -1e9, dtype=F64)
    # a sink far below every score: ordinary softmax attention; weights then sum to 1
    ones = P.sink_attention(q, k, torch.ones(9, 1, 3, dtype=F64), pos, pos, 0.5, far)
    assert torch.allclose(ones, torch.ones_like(ones))
    # a sink far above: everything goes to the sink, which has no value
    assert P.sink_attention(q, k, v, pos, pos, 0.5, -far).abs().max() < 1e-200
    # position 0 under a sink of 0 and a score s: weight exp(s) / (exp(s) + 1)
    zero = torch.zeros(2, dtype=F64)
    out = P.sink_attention(q, k, v, pos, pos, 0.5, zero)
    s = 0.5 * (q[0, 1] * k[0, 0]).sum()
    assert torch.allclose(out[0, 1], torch.sigmoid(s) * v[0, 0])
    # a window of 3: the output at 8 does not move with the key at 5, and moves with the key at 6
    base = P.sink_attention(q, k, v, pos, pos, 0.5, zero, window=3)
    v2 = v.clone(); v2[5] += 1
    assert torch.equal(P.sink_attention(q, k, v2, pos, pos, 0.5, zero, window=3)[8], base[8])
    v2 = v.clone(); v2[6] += 1
    assert not torch.allclose(P.sink_attention(q, k, v2, pos, pos, 0.5, zero, window=3)[8], base[8])
    # capped scores: a huge score counts as the cap; the sink is not capped
    big = P.sink_attention(q * 1e6, k, v, pos, pos, 1.0, torch.tensor([4.0, 4.0], dtype=F64), softcap=4.0)
    s = (q[0, 0] * k[0, 0]).sum()
    weight = math.exp(math.copysign(4.0, float(s))) / (math.exp(math.copysign(4.0, float(s))) + math.exp(4.0))
    assert torch.allclose(big[0, 0], weight * v[0, 0])


def test_plain_linear_recurrence_cut_anywhere_and_its_closed_form():
    g = torch.Generator().manual_seed(1)
    T, H, d, e = 30, 3, 5, 4
    q, k = torch.randn(T, H, d, generator=g, dtype=F64), torch.randn(T, H, d, generator=g, dtype=F64)
    v = torch.randn(T, H, e, generator=g, dtype=F64)
    decay = torch.tensor([0.5, 0.9, 1.0], dtype=F64)
    whole, last = P.decayed_outer_state(q, k, v, decay)
    state, parts = None, []
    for a, b in ((0, 1), (1, 3), (3, 20), (20, 21), (21, 30)):
        out, state = P.decayed_outer_state(q[a:b], k[a:b], v[a:b], decay, state)
        parts.append(out)
    assert torch.allclose(torch.cat(parts), whole, atol=1e-12) and torch.allclose(state, last, atol=1e-12)
    # o_t = sum_{j <= t} decay^(t-j) (q_t . k_j) v_j
    t, h = 17, 1
    direct = sum(decay[h] ** (t - j) * (q[t, h] * k[j, h]).sum() * v[j, h] for j in range(t + 1))
    assert torch.allclose(whole[t, h], direct, atol=1e-12)


def test_plain_layers_add_what_the_parts_give():
    """The whole model against its parts put together by hand for one pair layer."""
    import tempfile
    raw = {"architecture": "Gukosun", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "token_side": {"dim": 4},
           "layers": [TINY["GD"]["layers"][0] | {"mlp": {"kind": "dense", "ff": 40}}]}
    raw["layers"][0] = copy.deepcopy(raw["layers"][0])
    with tempfile.TemporaryDirectory() as tmp:
        make_model_dir(tmp + "/m", raw, seed=2, preset="unit", dtype=torch.float32)
        config, w = P.load_model_dir(tmp + "/m")
    tokens = [3, 9, 9, 41, 0, 17]
    streams = []
    logits = P.forward(config, w, tokens, layers_out=streams)
    ids, pos, eps = torch.tensor(tokens), torch.arange(len(tokens)), 1e-5
    x = w["embed"][ids]
    h = P.unit(x, eps) * w["l0.norm1"]
    y = P.parallel_mixer(h, w, "l0.mix.", config["layers"][0]["mixer"], eps, pos)
    x = x + y * w["l0.ls1"] + P.dense_feed_forward(h, w, "l0.mlp.") * w["l0.ls2"]
    x = x + P.token_side_input(x, ids, w, "l0.side.", 0, 4, eps)
    assert torch.allclose(streams[0], x, atol=1e-12)
    assert torch.allclose(logits, (P.unit(x, eps) * w["final.norm"]) @ w["head"].T, atol=1e-12)
