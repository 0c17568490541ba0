"""The Zetalorn design without a GPU: configuration reading and refusals, tensor names, what the cache keeps, the slot
book's rows per block of tokens, and the plain implementation's own mechanisms and sensitivity."""
import copy

import numpy as np
import pytest
import torch

import plain_zetalorn as plain
import zetalorn_helpers as zh


def _model(cfg):
    from llaisys_b200.config import config_from_dict
    from llaisys_b200.engine.model import DecoderModel
    from llaisys_b200.parts import BuildEnv
    return DecoderModel(config_from_dict(cfg).to_spec(), BuildEnv(torch.float32, torch.device("cpu")))


def test_configuration_is_read_and_turned_into_a_spec():
    from llaisys_b200.config import config_from_dict
    c = config_from_dict(zh.CONFIGS["P"])
    assert (c.vocab, c.width, c.logit_scale, c.loop) == (211, 64, 0.5, (1, 3, 3))
    assert c.order() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    spec = c.to_spec()
    assert [e.layer for e in spec.order] == [0, 1, 2, 1, 2, 1, 2, 3] and [e.opens_pass for e in spec.order] == [None, 0, None, 1, None, 2, None, None]
    assert spec.reentry.params["passes"] == 3 and spec.head.params["scale"] == 0.5
    att = spec.layers[1].sublayers[0].part
    assert att.kind == "differential_attention" and att.params["chunk"] == 40 and att.params["position"].params["factor"] == 2.0
    par = spec.layers[0].sublayers[0].part
    assert par.kind == "parallel_mixers" and [b["part"].kind for b in par.params["branches"]] == ["pooled_window_attention", "lightning_attention"]
    assert spec.layers[0].sublayers[1].part.params["groups"] == {"count": 3, "keep": 2}
    q = config_from_dict(zh.CONFIGS["Q"])
    assert q.loop is None and q.logit_scale == 1.0 and q.to_spec().reentry is None
    assert len(q.to_spec().layers[1].sublayers) == 1 and q.to_spec().layers[1].params["gates"] == ["rg1"]
    assert q.to_dict() == zh.CONFIGS["Q"]
    # what a configuration leaves out does not exist: no pool (a plain window, one user of the cache), one decay for all heads,
    # values as wide as the keys, no limit on the experts' gate and up
    def bare(c):
        c["layers"][0]["mixer"]["left"]["mask"].pop("pool")
        c["layers"][0]["mixer"]["left"].pop("vdim")
        c["layers"][0]["mixer"]["right"].update(decay=0.75)
        c["layers"][0]["mlp"]["expert"].pop("limit")
    b = config_from_dict(zh.variant(zh.CONFIGS["P"], bare))
    assert (b.mixers[0].left.pool, b.mixers[0].left.vdim, b.mixers[0].right.decay, b.ffs[0].limit) == (0, 16, (0.75, 0.75), float("inf"))
    assert len(_model(zh.variant(zh.CONFIGS["P"], bare)).call_all_users[0]) == 2


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "cannot share"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=13), "even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "at most"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5, 1.5]), "decay"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda c: c["layers"][0].update(type="conv"), "mixers"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(start=3), "loop"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(pool=0), "pool"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configurations_that_cannot_be_are_refused(edit, text):
    from llaisys_b200.config import ConfigError, config_from_dict
    with pytest.raises(ConfigError, match=text):
        config_from_dict(zh.variant(zh.CONFIGS["P"], edit))


def test_tensor_names_and_shapes():
    t = _model(zh.CONFIGS["P"]).expected_tensors()
    want = {"embed": (211, 64), "head": (211, 64), "final.norm": (), "loop.step": (3, 64), "l0.norm1": (), "l0.rg1": (64, 64), "l0.rg2.b": (64,),
            "l0.mix.left.q": (64, 64), "l0.mix.left.k": (32, 64), "l0.mix.left.v": (48, 64), "l0.mix.left.o": (64, 96), "l0.mix.left.q.norm": (16,),
            "l0.mix.left.out": (64,), "l0.mix.right.out": (64,), "l0.mix.right.q": (16, 64), "l0.mix.right.v": (32, 64), "l0.mix.right.g": (32, 64),
            "l0.mix.right.norm": (32,), "l0.mix.right.o": (64, 32), "l0.mlp.router": (6, 64), "l0.mlp.e5.gate": (24, 64), "l0.mlp.e0.down": (64, 24),
            "l1.mix.q": (128, 64), "l1.mix.k": (64, 64), "l1.mix.v": (48, 64), "l1.mix.o": (64, 96), "l1.mix.k.norm": (16,), "l1.mix.lq2": (16,)}
    for name, shape in want.items():
        assert tuple(t[name].shape) == shape, name
    assert "l3.norm2" not in t and "l3.rg2" not in t and "l3.mlp.router" not in t          # a layer without a feed-forward
    assert "loop.step" not in _model(zh.CONFIGS["Q"]).expected_tensors()


def test_what_the_cache_keeps():
    from llaisys_b200.cache.kv import CacheConfig, PagedCache
    m = _model(zh.CONFIGS["P"])
    # run order: layer 0, then (1, 2) three times, then 3: eight entries, every pass with users of its own
    assert len(m.call_users) == 8 and [len(u) for u in m.call_all_users] == [3, 1, 3, 1, 3, 1, 3, 1]
    needs, states = m.kv_needs(), m.state_sizes()
    assert (needs[0].window, needs[0].every, needs[1].window, needs[1].every, needs[2]) == (20, 1, None, 8, None)
    assert states[:4] == [0, 0, 2 * 8 * 16, 0] and needs[3].key_dim == 32 and needs[3].window == 40
    assert needs[4].window == 70 and needs[5].every == 4 and states[6] == 3 * 16 * 8
    c = PagedCache(needs, m.cache_of(), states, CacheConfig(max_tokens=64 * 12, max_seqs=2), torch.float32, "cpu", allocate=False)
    assert sorted(c.every) == [1, 1, 1, 1, 4, 8] and [r is None for r in c.rings] == [e > 1 for e in c.every]
    q = _model(zh.CONFIGS["Q"])
    # a pool larger than the window: the ring reaches back over a whole block; blocks of one token are rows per token, all kept
    assert [n.window for n in q.kv_needs() if n is not None and n.window is not None] == [64, 9, 3, 16]
    assert [n.every for n in q.kv_needs() if n is not None and n.window is None] == [1, 3, 16]


def test_slot_book_counts_rows_per_block_of_tokens():
    from llaisys_b200.cache.slots import SlotBook
    book = SlotBook(2, [8, 8], [None, None], 4, [0, 0], [1, 3])
    s = book.acquire()
    for n, want in ((2, (1, 0)), (1, (1, 1)), (8, (3, 1)), (4, (4, 2)), (12, (7, 3))):       # lengths 2, 3, 11, 15, 27
        book.reserve(s, n)
        book.commit(s, n)
        assert (len(book.pages(s, 0)), len(book.pages(s, 1))) == want, book.length(s)
    assert book.audit() == []
    book.release(s)
    assert [p.available for p in book.pools] == [8, 8]


# ----------------------------------------------------------------------------- the plain implementation itself
def test_masks():
    w = plain.window_mask(12, 4)
    assert w[7].tolist() == [False] * 4 + [True] * 4 + [False] * 4
    c = plain.chunk_mask(12, 5)
    assert c[7].tolist() == [False] * 5 + [True] * 3 + [False] * 4 and c[10].tolist() == [False] * 10 + [True, False]
    p = plain.pooled_mask(30, 6, 4)                     # block b is seen from position 4 b + 3 + 6 on
    assert [int(np.argmax(p[:, b])) for b in range(7)] == [9, 13, 17, 21, 25, 29, 0] and not p[:, 6].any()
    assert not p[8, 0] and p[9, 0] and p[29].tolist() == [True] * 6 + [False]


def test_rotation_layouts_and_scaling():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(5, 2, 8))
    pos = np.arange(5) + 3
    a = plain.rotate(x, pos, 4, 100.0, 1.0, "halves")
    b = plain.rotate(x, pos, 4, 100.0, 1.0, "neighbours")
    assert np.array_equal(a[..., 4:], x[..., 4:]) and np.array_equal(b[..., 4:], x[..., 4:])
    ang = 4 * 100.0 ** (-2.0 / 4)                         # position 4, second frequency
    assert np.allclose(a[1, 0, 1], x[1, 0, 1] * np.cos(ang) - x[1, 0, 3] * np.sin(ang))
    assert np.allclose(b[1, 0, 2], x[1, 0, 2] * np.cos(ang) - x[1, 0, 3] * np.sin(ang))
    assert np.allclose(plain.rotate(x, pos * 2, 4, 100.0, 2.0, "halves"), a)            # stretched positions
    assert np.allclose(np.linalg.norm(a, axis=-1), np.linalg.norm(x, axis=-1))


def test_router_groups_and_weights():
    h = np.eye(6)
    z = np.array([[2.0, 1.9, -1.0, 3.0, -5.0, -4.0, 1.0, 0.9]])               # groups of two: sums of sigmoid pairs
    w = np.zeros((8, 6))
    w[:, 0] = z[0]
    idx, wgt = plain.route(h[:1], w, {"experts": 8, "top": 3, "groups": {"count": 4, "keep": 2}})
    s = plain.sigmoid(z[0])
    # the best groups are 0 (2.0, 1.9) and 3 (1.0, 0.9): expert 3 (the largest score) lies in group 1, which is not kept
    assert idx[0].tolist() == [0, 1, 6] and np.allclose(wgt[0], s[[0, 1, 6]] / s[[0, 1, 6]].sum()) and np.isclose(wgt.sum(), 1)
    idx, _ = plain.route(h[:1], w, {"experts": 8, "top": 3})
    assert idx[0].tolist() == [3, 0, 1]


def test_expert_clamps():
    one = np.ones((1, 1))
    e = lambda g, u: plain.expert(np.array([[1.0]]), one * g, one * u, one, 1.5)[0, 0]
    assert np.isclose(e(9.0, 0.0), 1.5 * plain.sigmoid(1.702 * 1.5)) and np.isclose(e(1.0, 7.0), plain.sigmoid(1.702) * 2.5)
    assert np.isclose(e(1.0, -7.0), plain.sigmoid(1.702) * -0.5) and np.isclose(e(-9.0, 0.0), -9.0 * plain.sigmoid(1.702 * -9.0))


def _weights(cfg, seed=3, spread=True):
    """Random float64 weights by the model's own list of tensors (shaped as make_folder shapes them, without files)."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, decl in _model(cfg).expected_tensors().items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("norm1", "norm2", "out") or name == "final.norm" or name.endswith(("q.norm", "k.norm", "right.norm")):
            out[name] = rng.uniform(0.5, 1.5, size=decl.shape) * (2.0 if name.endswith((".q.norm", ".k.norm")) else 1.0)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            out[name] = rng.uniform(-0.4, 0.4, size=decl.shape)
        else:
            out[name] = rng.normal(size=decl.shape) * (0.5 if name.endswith(("rg1", "rg2", "router")) or ".right." in name else 0.2)
    return out


SENSITIVE = [
    ("the window", lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=21), 20),
    ("the pool", lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(pool=7), 26),
    ("the chunk", lambda c: c["layers"][1]["mixer"]["mask"].update(size=41), 40),
    ("the constant of the difference", lambda c: c["layers"][1]["mixer"].update(diff=0.26), 0),
    ("a decay", lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.6, 0.98]), 1),
    ("the rotation's stretch", lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(factor=2.1), 1),
    ("the rotated dimensions", lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=6), 1),
    ("the experts' limit", lambda c: c["layers"][0]["mlp"]["expert"].update(limit=0.9), 0),
    ("the kept groups", lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=3), 0),
    ("the number of passes", lambda c: c["loop"].update(times=2), 0),
    ("the logit scale", lambda c: c.update(logit_scale=0.51), 0),
]


@pytest.mark.parametrize("what, edit, first", SENSITIVE, ids=[s[0] for s in SENSITIVE])
def test_every_constant_moves_the_logits_from_where_it_should(what, edit, first):
    """A constant that is off by one (or by a few per cent) moves the logits by far more than any tolerance of the GPU
    tests, and leaves bit-equal the positions it cannot reach: those before `first`."""
    cfg = zh.CONFIGS["P"]
    w = _weights(cfg)
    toks = np.random.default_rng(1).integers(0, cfg["vocab"], size=60).tolist()
    a = plain.forward(cfg, w, toks)[0]
    other = zh.variant(cfg, edit)
    if what == "the number of passes":
        w = dict(w, **{"loop.step": w["loop.step"][:2]})
    b = plain.forward(other, w, toks)[0]
    moved = np.abs(a - b).max(axis=1)
    assert moved[first:].max() > 1e-2, (what, moved.max())
    assert first == 0 or moved[:first].max() == 0.0, (what, moved[:first].max())


def test_each_tensor_of_a_layer_matters():
    cfg = zh.CONFIGS["P"]
    w = _weights(cfg)
    toks = np.random.default_rng(2).integers(0, cfg["vocab"], size=50).tolist()
    a = plain.forward(cfg, w, toks)[0]
    for name in ("loop.step", "l1.rg1", "l1.rg1.b", "l2.rg2.b", "l0.mix.left.out", "l0.mix.right.out", "l0.mix.right.norm", "l1.mix.lq1",
                 "l1.mix.lk2", "l1.mix.q.norm", "l0.mix.left.k.norm", "l0.norm1", "l3.norm1", "final.norm", "l0.mix.right.g", "l0.mlp.e3.gate"):
        w2 = dict(w)
        w2[name] = w[name] * 1.2 + 0.05
        assert np.abs(plain.forward(cfg, w2, toks)[0] - a).max() > 1e-3, name


def test_the_first_token_reaches_the_last_through_blocks_and_state_only():
    """A parallel layer alone: with the recurrent branch silenced, the first token is seen by a late position only through
    its pooled block; with the attention branch silenced, only through the state."""
    base = zh.config(50, 32, [zh.parallel((2, 1, 8, 8, 6, 4, zh.rot(8)), (2, 4, 8, (0.9, 0.99)))])
    w = _weights(base)
    toks = np.random.default_rng(4).integers(0, 49, size=40).tolist()
    other = [49] + toks[1:]
    for silent, lo in (("l0.mix.right.o", 4 + 6 - 1), ("l0.mix.left.o", 0)):
        w2 = dict(w, **{silent: np.zeros_like(w[silent])})
        moved = np.abs(plain.forward(base, w2, toks)[0] - plain.forward(base, w2, other)[0]).max(axis=1)
        assert moved[-1] > 1e-6, silent
        if silent.endswith("right.o"):
            # positions 6 .. 8: the first token has left the window and its block (positions 0 .. 3) is not seen yet
            assert moved[:6].min() > 0 and moved[6:lo].max() == 0.0 and moved[lo] > 0, moved[:12]


@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_cpu_model_against_the_plain_implementation(tmp_path, name):
    """The package's CPU model (float32 operators, a cache, the prompt and then single tokens) against the plain float64
    evaluation of whole sequences: whole prompts, and the same tokens fed in portions down to single ones."""
    from llaisys_b200.models.cpu_model import CpuModel
    cfg = zh.CONFIGS[name]
    folder = zh.make_folder(tmp_path, cfg, seed=4, gain=4.0)
    oracle = zh.Oracle(folder)
    toks = zh.random_requests(cfg, [90], seed=7)[0]
    ref = oracle.logits(toks)
    model = CpuModel.from_folder(folder)
    assert np.abs(model.step(toks) - ref).max() < 2e-4
    model.reset()
    got = np.concatenate([model.step(toks[:70]), model.step(toks[70:72])] + [model.step([t]) for t in toks[72:]])
    assert np.abs(got - ref).max() < 2e-4
