"""The Zedirax design without a GPU: configuration reading and refusals, tensor names, what the cache keeps for it, the
package's CPU model against the plain implementation, and the plain implementation's own sensitivity (a key far back, the
distance penalty's two numbers, a temperature step one position early, a depth weight, the candidate's two branches, the
shared expert's gate: each moves the logits by far more than any tolerance and leaves the positions it should not touch as
they were)."""
import numpy as np
import pytest
import torch

import plain_zedirax as plain
import zedirax_helpers as zh


def test_configuration_reading_and_refusals():
    from llaisys_b200.config import ConfigError, config_from_dict
    cfg = config_from_dict(zh.CONFIGS["P"])
    spec = cfg.to_spec()
    assert spec.architecture == "Zedirax" and spec.vocab_size == 211 and spec.hidden_size == 64
    assert [c.cache_of for c in spec.order] == [None] * 6
    assert [l.block for l in spec.layers] == ["depth_averaged_residual"] * 6
    assert [l.params["index"] for l in spec.layers] == list(range(6)) and spec.layers[0].params["mult"] == 0.6
    mixers = [l.sublayers[0].part for l in spec.layers]
    assert [m.kind for m in mixers] == ["min_gru", "latent_attention", "windowed_sink_attention", "min_gru",
                                        "windowed_sink_attention", "latent_attention"]
    assert mixers[1].params["q_rank"] is None and mixers[1].params["gate"] == "elements" and mixers[1].params["window"] is None
    assert mixers[1].params["position"].kind == "rope_leading" and mixers[1].params["position"].params["base"] == 5000.0
    assert mixers[2].params["distance_bias"] and mixers[2].params["q_temp"] == {"coef": 0.4, "every": 16}
    assert mixers[2].params["position"] is None and mixers[2].params["value_dim"] == 24 and mixers[2].params["key_dim"] == 16
    ffs = [l.sublayers[1].part for l in spec.layers]
    assert [f.kind for f in ffs] == ["gated_mlp", "routed_experts", "gated_mlp", "routed_experts", "routed_experts", "gated_mlp"]
    assert ffs[0].params["act"] == "gelu_tanh" and ffs[0].params["bias"]
    assert ffs[1].params["gate"] == "softmax_chosen" and ffs[1].params["act"] == "gelu" and ffs[1].params["shared_gate"]
    assert ffs[4].params["shared_ff"] is None and not ffs[4].params["shared_gate"]
    assert spec.head.params["tied_to"] is None and spec.final_norm.params["offset"] == 1.0
    q = config_from_dict(zh.CONFIGS["Q"]).to_spec()
    assert [len(l.sublayers) for l in q.layers] == [2, 1, 2, 1, 1] and q.layers[0].params["mult"] == 1.0
    assert q.layers[0].sublayers[0].part.params["q_temp"] is None
    assert cfg.to_dict() == zh.CONFIGS["P"]

    def bad(edit, match):
        with pytest.raises(ConfigError, match=match):
            config_from_dict(zh.variant(zh.CONFIGS["P"], edit))

    bad(lambda c: c["layers"][0].__setitem__("type", "gla"), "mixers of this architecture")
    bad(lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu"), "feed-forwards of this architecture")
    bad(lambda c: c["layers"][2]["mixer"].__setitem__("kv_heads", 3), "cannot share")
    bad(lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 7), "even")
    bad(lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 10), "at most")
    bad(lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 7), "cannot use")
    bad(lambda c: c["layers"][0]["mixer"].__setitem__("width", 0), "width")
    bad(lambda c: c["layers"][2]["mixer"]["q_temp"].__setitem__("every", 0), "every")
    bad(lambda c: c.__setitem__("layers", []), "non-empty")


def test_tensor_names_and_shapes(tmp_path):
    from llaisys_b200.config import load_config
    from llaisys_b200.engine.model import DecoderModel
    from llaisys_b200.parts import BuildEnv
    from llaisys_b200.weights import FolderSource, SafetensorsFile, write_safetensors
    from llaisys_b200.weights.loader import WeightsError, check_tensors
    folder = zh.make_folder(tmp_path, zh.CONFIGS["P"], seed=1, gain=1.0)
    model = DecoderModel(load_config(folder).to_spec(), BuildEnv(torch.float32, torch.device("cpu")))
    names = model.expected_tensors()
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.z", "l0.mix.z.b", "l0.mix.x.b", "l0.mix.g", "l0.mix.o",
            "l0.mlp.gate.b", "l0.mlp.down.b", "l0.dwa", "l5.dwa", "l1.mix.q", "l1.mix.dkv", "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv",
            "l1.mix.g", "l1.mlp.router", "l1.mlp.e5.up", "l1.mlp.shared.sg", "l2.mix.r1", "l2.mix.r2", "l2.mix.k"} <= set(names)
    assert "l1.mix.dq" not in names and "l4.mlp.shared.up" not in names and "l1.mlp.e6.up" not in names and "l1.mlp.correction" not in names
    f = SafetensorsFile(folder / "model.safetensors")
    shapes = {n: tuple(f.get(n).shape) for n in f.entries}
    assert set(shapes) == set(names)
    assert shapes["l3.dwa"] == (5,) and shapes["l1.mix.dkv"] == (40 + 8, 64) and shapes["l1.mix.q"] == (3 * 24, 64)
    assert shapes["l1.mix.g"] == (3 * 24, 64) and shapes["l1.mix.o"] == (64, 72) and shapes["l1.mlp.shared.sg"] == (1, 64)
    assert shapes["l2.mix.v"] == (2 * 24, 64) and shapes["l2.mix.o"] == (64, 4 * 24) and shapes["l2.mix.r1"] == (4,)
    check_tensors(model, FolderSource(folder))
    t = {n: f.get(n).clone() for n in f.entries}
    t["l2.mix.r2"] = t["l2.mix.r2"][:-1].clone()
    write_safetensors(folder / "model.safetensors", t)
    with pytest.raises(WeightsError, match="l2.mix.r2"):
        check_tensors(model, FolderSource(folder))


def test_what_the_cache_keeps_for_this_design():
    from llaisys_b200.cache import CacheConfig
    from llaisys_b200.cache.kv import PagedCache
    from llaisys_b200.config import config_from_dict
    from llaisys_b200.engine.model import DecoderModel
    from llaisys_b200.parts import BuildEnv
    model = DecoderModel(config_from_dict(zh.CONFIGS["P"]).to_spec(), BuildEnv(torch.float32, torch.device("cpu")))
    cache = PagedCache(model.kv_needs(), model.cache_of(), model.state_sizes(), CacheConfig(max_tokens=2048, max_seqs=4),
                       torch.float32, "cpu", allocate=False)
    assert cache.rings == [None] * len(cache.rings)                          # nothing is windowed: every row is kept
    assert model.state_sizes() == [40, 0, 0, 72, 0, 0] and model.cache_of() == [None] * 6
    # the latent layers keep one row of kv_rank + rot_dim numbers a token; the attention layers keys and values of their own widths
    needs = model.kv_needs()
    assert needs[0] is None and needs[3] is None and all(needs[i] is not None for i in (1, 2, 4, 5))
    only_gru = zh.config(50, 16, [zh.mingru(8), zh.mingru(24, zh.dense(8))])
    model = DecoderModel(config_from_dict(only_gru).to_spec(), BuildEnv(torch.float32, torch.device("cpu")))
    cache = PagedCache(model.kv_needs(), model.cache_of(), model.state_sizes(), CacheConfig(max_tokens=256, max_seqs=2),
                       torch.float32, "cpu", allocate=False)
    assert cache.group_keys == [] and model.state_sizes() == [8, 24]


@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_cpu_model_against_the_plain_implementation(tmp_path, name):
    from llaisys_b200.models.cpu_model import CpuModel
    folder = zh.make_folder(tmp_path, zh.CONFIGS[name], seed=3, gain=9.0)
    oracle = zh.Oracle(folder)
    toks = zh.random_requests(zh.CONFIGS[name], [90], seed=1)[0]
    m = CpuModel.from_folder(folder)
    got = np.concatenate([m.step(toks[:50])] + [m.step([t]) for t in toks[50:60]] + [m.step(toks[60:])])
    ref = oracle.logits(toks)
    assert np.abs(got - ref).max() < 1e-4 * max(1.0, np.abs(ref).max())
    new = m.generate(toks[:7], 5)
    seq = list(toks[:7])
    for _ in range(5):
        seq.append(int(np.argmax(oracle.logits(seq)[-1])))
    assert new == seq[7:]


def test_the_plain_implementations_own_sensitivity(tmp_path):
    cfg = zh.CONFIGS["P"]
    folder = zh.make_folder(tmp_path, cfg, seed=5, gain=9.0)
    oracle = zh.Oracle(folder)
    toks = zh.random_requests(cfg, [120], seed=2)[0]
    base = oracle.logits(toks)
    tol = 1e-4

    def moved(edit_cfg=None, edit_w=None, tokens=None):
        c = zh.variant(oracle.config, edit_cfg) if edit_cfg else oracle.config
        w = dict(oracle.weights)
        if edit_w:
            edit_w(w)
        return np.abs(plain.forward(c, w, tokens or toks) - base).max(axis=1)

    # the temperature of layer 2 steps at position 15 (every = 16): a step one position later leaves positions < 15 alone
    d = moved(lambda c: c["layers"][2]["mixer"]["q_temp"].__setitem__("every", 17))
    assert d[:15].max() == 0 and d[15] > 10 * tol
    # the penalty grows with distance: position 0 has none, whatever its numbers
    d = moved(edit_w=lambda w: w.__setitem__("l2.mix.r1", w["l2.mix.r1"] * 1.1))
    assert d[0] == 0 and d[1:].max() > 10 * tol
    d = moved(edit_w=lambda w: w.__setitem__("l4.mix.r2", w["l4.mix.r2"] * 0.02))
    assert d[0] == 0 and d[1:].max() > 10 * tol
    # every earlier result enters every later layer
    for name in ("l0.dwa", "l2.dwa", "l5.dwa"):
        def edit(w, name=name):
            a = w[name].copy()
            a[0] += 0.05
            w[name] = a
        assert moved(edit_w=edit).max() > 10 * tol
    assert moved(lambda c: c.__setitem__("residual_mult", 0.7)).max() > 10 * tol
    assert moved(edit_w=lambda w: w.__setitem__("l3.norm2", w["l3.norm2"] - 1.0)).max() > 10 * tol      # the offset of one
    assert moved(edit_w=lambda w: w.__setitem__("l1.mlp.shared.sg", w["l1.mlp.shared.sg"] * 0)).max() > 10 * tol
    assert moved(edit_w=lambda w: w.__setitem__("l1.mix.g", w["l1.mix.g"] * 0)).max() > 10 * tol
    assert moved(edit_w=lambda w: w.__setitem__("l0.mlp.up.b", w["l0.mlp.up.b"] * 0)).max() > 10 * tol
    assert moved(lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("base", 4000.0))[1:].max() > 10 * tol
    # the first token reaches the last one through every kind of mixer alone
    other = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    for i in (0, 1, 2):
        def only(c, i=i):
            c["layers"] = [dict(c["layers"][i], mlp=None)]
        one = zh.variant(oracle.config, only)
        w = {k.replace(f"l{i}.", "l0.", 1) if k.startswith(f"l{i}.") else k: v for k, v in oracle.weights.items()
             if not k.startswith("l0.") or i == 0}
        w["l0.dwa"] = np.array([0.0, 1.0])
        a, b = plain.forward(one, w, toks), plain.forward(one, w, other)
        assert np.abs(a[-1] - b[-1]).max() > 1e-7, i


def test_candidate_of_the_recurrence_and_state_carried():
    u = np.array([-30.0, -1.0, -1e-9, 0.0, 1e-9, 2.0])
    c = plain.mingru_candidate(u)
    assert np.allclose(c, [plain.sigmoid(-30.0), plain.sigmoid(-1.0), 0.5, 0.5, 0.5, 2.5]) and (c > 0).all()
    rng = np.random.default_rng(0)
    W, D = 7, 12
    w = {"p.z": rng.normal(size=(W, D)), "p.z.b": rng.normal(size=W), "p.x": rng.normal(size=(W, D)), "p.x.b": rng.normal(size=W),
         "p.g": rng.normal(size=(W, D)), "p.o": rng.normal(size=(D, W))}
    h = rng.normal(size=(20, D))
    whole, S = plain.mingru_mixer(h, w, "p")
    a, Sa = plain.mingru_mixer(h[:7], w, "p")
    b, Sb = plain.mingru_mixer(h[7:], w, "p", state=Sa)
    assert np.abs(np.concatenate([a, b]) - whole).max() < 1e-12 and np.abs(Sb - S).max() < 1e-12


def test_routing_weights_are_a_softmax_over_the_chosen_logits_only():
    rng = np.random.default_rng(1)
    h = rng.normal(size=(9, 6))
    w = {"p.router": rng.normal(size=(5, 6)) * 3}
    idx, wgt = plain.route(h, w, "p", 2)
    z = h @ w["p.router"].T
    for t in range(9):
        order = np.argsort(-z[t])
        assert list(idx[t]) == list(order[:2])
        e = np.exp(z[t, order[:2]])
        assert np.allclose(wgt[t], e / e.sum())
    idx, wgt = plain.route(h, w, "p", 1)
    assert np.allclose(wgt, 1.0)
    from llaisys_b200 import cpu_ops
    i2, w2 = cpu_ops.route_top_softmax(z.astype(np.float32), None, 3, 1.0)
    i3, w3 = plain.route(h, w, "p", 3)
    assert np.array_equal(i2, i3) and np.abs(w2 - w3).max() < 1e-5
