"""The Zetalorn design on the GPU against its plain implementation: every mechanism alone, then single layers at the
places where a fault would hide (the edges of windows, chunks, pooled blocks and pages, a key far back, the first tokens),
then whole models under every way of cutting requests into steps, then generation and replay through the entry points."""
import json
import subprocess
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_zetalorn as plain
import zetalorn_helpers as zh
from helpers import build_engine, compare, run_batches, run_chunked, run_mixed, run_tail_by_one, run_whole, tolerance
from zetalorn_helpers import compare as compare_zl

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
DTYPES = [torch.float32, torch.bfloat16]
DEV = "cuda:0"


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _bf16_exact(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float64)).to(torch.bfloat16).to(torch.float64).numpy()


def _dev(a, dtype):
    return torch.from_numpy(np.asarray(a)).to(dtype).to(DEV)


def _env(dtype):
    from llaisys_b200.parts import BuildEnv
    return BuildEnv(dtype, torch.device(DEV))


def _close(got, want, dtype, what=""):
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    err = np.abs(np.asarray(got, dtype=np.float64) - want).max()
    assert err <= tol * max(1.0, np.abs(want).max()), (what, err)


# ----------------------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(3, 2, 16, 8, "halves", True), (4, 2, 12, 12, "neighbours", True), (2, 1, 10, 0, "halves", True),
                                   (5, 5, 7, 6, "neighbours", False), (1, 1, 64, 2, "halves", False), (2, 2, 33, 32, "neighbours", True)])
def test_norm_and_rotation_of_heads(dtype, shape):
    """Query and key rows normed over their elements and rotated in their first dimensions, in both layouts, with and
    without the norm, at positions up to the thousands; the values that follow them in the row stay as they are."""
    from llaisys_b200 import kernels
    nq, nk, d, dims, layout, norm = shape
    rng = np.random.default_rng(0)
    T, dv, eps = 9, 5, 1e-5
    pos = np.array([0, 1, 2, 63, 64, 65, 500, 4095, 7])
    x = _bf16_exact(rng.normal(size=(T, (nq + nk) * d + nk * dv)) * 3)
    wq, wk = rng.uniform(0.5, 1.5, size=d), rng.uniform(0.5, 1.5, size=d)
    half = dims // 2
    freq = 300.0 ** (-2.0 * np.arange(half) / max(dims, 1)) / 1.5
    ang = np.arange(4096)[:, None] * freq[None, :]
    tables = (_dev(np.cos(ang), torch.float32).contiguous(), _dev(np.sin(ang), torch.float32).contiguous(), dims) if dims else None
    proj = _dev(x, dtype)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.head_prep(proj, nq, nk, d, kv_heads=nk, dv=dv, q_weight=_dev(wq, torch.float32) if norm else None,
                      k_weight=_dev(wk, torch.float32) if norm else None, eps=eps, tables=tables, layout=layout, tok_pos=_i32(pos), err=err)
    rows = x[:, :(nq + nk) * d].reshape(T, nq + nk, d)
    if norm:
        rows = plain.rms(rows, eps) * np.concatenate([np.tile(wq, (nq, 1)), np.tile(wk, (nk, 1))])[None]
    rows = plain.rotate(rows, pos, dims, 300.0, 1.5, layout)
    got = proj.float().cpu().numpy()
    _close(got[:, :(nq + nk) * d], rows.reshape(T, -1), dtype, "heads")
    assert np.array_equal(got[:, (nq + nk) * d:], x[:, (nq + nk) * d:]) and int(err.item()) == 0


@pytest.mark.parametrize("H", [44, 256, 2050])
def test_gated_join_of_the_stream_and_norm_in_one_pass(H):
    from llaisys_b200 import kernels
    rng = np.random.default_rng(1)
    T = 7
    x, delta, gate, rows = (rng.normal(size=(T, H)) * s for s in (2.0, 1.0, 3.0, 0.5))
    vec, w = rng.normal(size=H), rng.uniform(0.5, 1.5, size=H)
    for dd in DTYPES:
        d_in = _bf16_exact(delta)
        xs = _dev(x, torch.float32)
        h = kernels.stream_join(xs, _dev(d_in, dd), _dev(gate, torch.float32), rows_add=_dev(rows, torch.float32), vec_add=_dev(vec, torch.float32),
                                weight=_dev(w, torch.float32), eps=1e-5, out_dtype=dd)
        want = x + plain.sigmoid(gate.astype(np.float32).astype(np.float64)) * d_in + rows.astype(np.float32) + vec.astype(np.float32)
        _close(xs.cpu().numpy(), want, torch.float32, "stream")
        _close(h.float().cpu().numpy(), plain.rms(want, 1e-5) * w, dd, "normed rows")
    xs = _dev(x, torch.float32)
    assert kernels.stream_join(xs, _dev(delta, torch.float32)) is None                   # ungated, no norm
    _close(xs.cpu().numpy(), x.astype(np.float32).astype(np.float64) + delta.astype(np.float32), torch.float32)
    xs = _dev(x, torch.float32)
    h = kernels.stream_join(xs, weight=_dev(w, torch.float32), eps=1e-6, out_dtype=torch.float32)         # norm alone
    _close(h.cpu().numpy(), plain.rms(x.astype(np.float32).astype(np.float64), 1e-6) * w, torch.float32)
    assert np.array_equal(xs.cpu().numpy(), x.astype(np.float32))


def test_mean_of_normed_branches_and_difference_of_score_maps():
    from llaisys_b200 import kernels
    rng = np.random.default_rng(2)
    T, H = 5, 300
    xs = [rng.normal(size=(T, H)).astype(np.float32) * s for s in (1.0, 30.0, 0.01)]
    xs[2][3] = 0.0                                                                        # a silent branch gives nothing
    ws = [rng.uniform(0.5, 1.5, size=H).astype(np.float32) for _ in xs]
    for n in (1, 2, 3):
        got = kernels.branch_mean([_dev(x, torch.float32) for x in xs[:n]], [_dev(w, torch.float32) for w in ws[:n]], 1e-5, 1.0 / n)
        want = sum(plain.rms(x.astype(np.float64), 1e-5) * w for x, w in zip(xs[:n], ws[:n])) / n
        _close(got.cpu().numpy(), want, torch.float32, n)
    Hh, G, dv, lam = 6, 2, 20, 0.37
    r = Hh // G
    a = rng.normal(size=(T, G, 2, r, dv)).astype(np.float32)
    for dd in DTYPES:
        got = kernels.diff_combine(_dev(a.reshape(T, -1), torch.float32), Hh, r, dv, lam, 1e-5, 0.7, dd).float().cpu().numpy()
        o = a[:, :, 0].astype(np.float64) - lam * a[:, :, 1]
        _close(got, (plain.rms(o, 1e-5) * 0.7).reshape(T, -1), dd)


@pytest.mark.parametrize("shape", [(150, 40, 6, 2, 24, (3, 2), 1.0), (5, 64, 8, 3, 16, (4, 2), 0.4), (33, 48, 4, 4, 16, None, 2.0), (300, 128, 12, 4, 64, (2, 1), 1.5),
                                   (64, 44, 5, 1, 12, None, 0.8), (20, 32, 6, 2, 8, (6, 3), 1.0)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_routed_experts_with_groups_and_the_clamped_gated_activation(dtype, shape):
    """Choice within the best groups, weights divided by their sum, experts with a clamped gate and up, on the tensor-core
    product (bfloat16, widths that it takes) and on the CUDA-core one, against the plain loop over tokens."""
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    T, D, E, top, ff, groups, limit = shape
    rng = np.random.default_rng(T)
    w = {"router": rng.normal(size=(E, D)) * 0.6}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = rng.normal(size=(ff, D)) * 0.3, rng.normal(size=(ff, D)) * 0.3, rng.normal(size=(D, ff)) * 0.2
    w = {n: _bf16_exact(v) for n, v in w.items()}
    router = {"experts": E, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    part = build_part("ffn", PartSpec("routed_experts", {
        "hidden_size": D, "experts": E, "top": top, "expert_ff": ff, "gate": "sigmoid", "act": "swish_clamped", "limit": limit, "alpha": 1.702,
        "renorm": True, "groups": router.get("groups"), "shared_ff": None, "use_bias": False}), _env(dtype))
    part.load({n: _dev(v, dtype) for n, v in w.items()})
    x = _bf16_exact(rng.normal(size=(T, D)))
    got = part.forward(_dev(x, dtype), SimpleNamespace()).cpu().numpy()
    want = plain.moe(x, w, {"router": router, "expert": {"ff": ff, "limit": limit}})
    err = np.abs(got - want).max(axis=1)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    assert (err > tol * max(1.0, np.abs(want).max())).sum() == 0, err.max()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(24, 2, 8, 16, (0.6, 0.99)), (40, 3, 5, 7, (0.0, 1.0, 0.5)), (64, 1, 64, 64, (0.999,)), (32, 4, 32, 4, (0.9, 0.8, 0.7, 0.3))])
def test_constant_decay_linear_attention_with_state_carried_in_slots(dtype, shape):
    """Whole sequences (the long one runs in chunks side by side), then the same sequences in portions down to single
    tokens, interleaved in one batch (long portions in chunks, short ones token by token, in one step), each with its state
    in a slot of its own; the slots hold stale numbers outside the rows that the cache clears."""
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    D, H, dk, dv, decay = shape
    rng = np.random.default_rng(7)
    w = {"q": rng.normal(size=(H * dk, D)) * 0.5, "k": rng.normal(size=(H * dk, D)) * 0.5, "v": rng.normal(size=(H * dv, D)) * 0.5,
         "g": rng.normal(size=(H * dv, D)) * 0.5, "o": rng.normal(size=(D, H * dv)) * 0.3, "norm": rng.uniform(0.5, 1.5, size=H * dv)}
    w = {n: _bf16_exact(v) for n, v in w.items()}
    part = build_part("mixer", PartSpec("lightning_attention", {"hidden_size": D, "num_heads": H, "key_dim": dk, "value_dim": dv,
                                                                 "decay": list(decay), "eps": 1e-5}), _env(dtype))
    part.load({n: _dev(v, dtype if n != "norm" else torch.float32) for n, v in w.items()})
    assert part.state_size() == H * dk * dv
    seqs = [_bf16_exact(rng.normal(size=(n, D))) for n in (700, 1, 23)]
    m = {"heads": H, "dim": dk, "vdim": dv, "decay": list(decay)}
    want = [plain.lightning_attention(s, w, m, 1e-5) for s in seqs]
    state = torch.full((6, H * dk * dv), 7.0, dtype=torch.float32, device=DEV)
    slots = [4, 0, 2]

    def step(who, parts_):
        x = np.concatenate(parts_)
        starts = np.concatenate([[0], np.cumsum([len(p) for p in parts_])])
        ctx = SimpleNamespace(state=lambda call: state, seq_start=_i32(starts), seq_slot=_i32([slots[i] for i in who]), n_seqs=len(who),
                              n_new=[len(p) for p in parts_])
        out = part.forward(_dev(x, dtype), ctx, 0).float().cpu().numpy()
        return [out[starts[j]:starts[j + 1]] for j in range(len(who))]

    for plans in ([[700], [1], [23]], [[3, 1, 1, 301, 2, 328, 64], [0, 1], [1, 2, 17, 1, 2]], [[65, 635], [0, 1], [0, 23]]):
        for s in slots:
            state[s].zero_()
        got, fed = [[] for _ in seqs], [0] * len(seqs)
        for k in range(max(len(p) for p in plans)):
            who = [i for i, p in enumerate(plans) if k < len(p) and p[k] > 0]
            for i, o in zip(who, step(who, [seqs[i][fed[i]:fed[i] + plans[i][k]] for i in who])):
                got[i].append(o)
                fed[i] += plans[i][k]
        for i, (g, y) in enumerate(zip(got, want)):
            _close(np.concatenate(g), y, dtype, (plans, i))
    assert float(state[1].min()) == 7.0 and float(state[5].max()) == 7.0


# ----------------------------------------------------------------------------- single layers at the edges
def _silence(*names):
    def edit(t):
        for n in names:
            t[n] = torch.zeros_like(t[n])
    return edit


EDGE_CUTS = ([63, 2, 65, 1, 64], [2], [1000])


@pytest.mark.parametrize("window, pool", [(1, 1), (9, 4), (64, 8), (65, 64), (72, 8), (130, 3), (5, 100), (20, 7)])
def test_window_with_pooled_blocks_alone_at_every_edge(tmp_path, window, pool):
    """The windowed branch alone (the recurrent one is silenced): every position of sequences that pass several windows,
    blocks and pages, whole, decoded one by one from a short prompt, and in portions down to two tokens."""
    cfg = zh.config(90, 32, [zh.parallel((4, 2, 16, 8, window, pool, zh.rot(8, 1000.0)), (1, 4, 4, (0.9,)))])
    folder = zh.make_folder(tmp_path, cfg, seed=window * 131 + pool, gain=6.0, edit=_silence("l0.mix.right.o"))
    oracle = zh.Oracle(folder)
    toks = zh.random_requests(cfg, [300], seed=pool)
    like = zh.like_config(cfg)
    engine = build_engine(folder, torch.float32, max_tokens=320)
    compare(run_whole(engine, toks), oracle, toks, torch.float32, like, "whole")
    compare(run_tail_by_one(engine, toks, tail=297), oracle, toks, torch.float32, like, "decoded")
    for cuts in EDGE_CUTS[:2]:
        compare(run_chunked(engine, toks, cuts), oracle, toks, torch.float32, like, f"portions {cuts}")
    assert [p.available for p in engine.cache.book.pools] == engine.cache.group_pages


@pytest.mark.parametrize("chunk", [1, 5, 63, 64, 65, 128, 1000])
@pytest.mark.parametrize("heads", [(4, 2), (3, 1)])
def test_two_score_maps_over_chunks_alone_at_every_edge(tmp_path, chunk, heads):
    cfg = zh.config(90, 32, [zh.attention(heads[0], heads[1], 12, 20, chunk, diff=0.35, rotation=zh.rot(6, 500.0, 3.0))])
    folder = zh.make_folder(tmp_path, cfg, seed=chunk, gain=6.0)
    oracle = zh.Oracle(folder)
    toks = zh.random_requests(cfg, [280], seed=chunk + 1)
    like = zh.like_config(cfg)
    engine = build_engine(folder, torch.float32, max_tokens=320)
    compare(run_whole(engine, toks), oracle, toks, torch.float32, like, "whole")
    compare(run_tail_by_one(engine, toks, tail=270), oracle, toks, torch.float32, like, "decoded")
    for cuts in EDGE_CUTS[:2]:
        compare(run_chunked(engine, toks, cuts), oracle, toks, torch.float32, like, f"portions {cuts}")


@pytest.mark.parametrize("layer", [
    zh.parallel((4, 2, 64, 64, 70, 8, zh.rot(32, 1000.0)), (1, 8, 8, (0.9,))),
    zh.parallel((2, 2, 16, 32, 130, 3, zh.rot(16, 1000.0)), (1, 8, 8, (0.9,))),
    zh.parallel((2, 1, 128, 128, 20, 64, None), (1, 8, 8, (0.9,))),
    zh.attention(4, 2, 32, 64, 100, rotation=zh.rot(32, 500.0, 2.0)),
    zh.attention(2, 1, 16, 16, 64, rotation=zh.rot(8, 500.0)),
    zh.attention(3, 3, 64, 64, 1000, diff=0.1),
], ids=["window70", "values_twice_as_wide", "head128", "maps_values_twice_as_wide", "maps16", "maps64"])
def test_prompts_on_the_tensor_cores_against_the_cuda_core_kernel(tmp_path, layer, monkeypatch):
    """bfloat16 prompts and portions with chunks, two score maps, pooled blocks and values twice as wide as the keys run on
    the mma.sync prefill kernel; the same steps with that kernel switched off run on the CUDA-core one.  Both against
    the plain implementation, and against each other row by row."""
    from llaisys_b200.kernels import ops
    cfg = zh.config(90, 64, [layer])
    edit = _silence("l0.mix.right.o") if layer["type"] == "parallel" else None
    folder = zh.make_folder(tmp_path, cfg, seed=3, gain=3.0, edit=edit)
    oracle = zh.Oracle(folder)
    toks = zh.random_requests(cfg, [300, 77], seed=5)
    got = {}
    for on in (True, False):
        monkeypatch.setattr(ops, "MMA_ATTENTION", on)
        engine = build_engine(folder, torch.bfloat16, max_tokens=448, max_seqs=2)
        n0 = ops.launch_count()
        got[on] = (run_whole(engine, toks), run_chunked(engine, toks, [130, 70, 1000]), run_batches(engine, toks, [[0, 1]], [250, 70]))
        for g, what in zip(got[on], ("whole", "portions", "together")):
            compare_zl(g, oracle, toks, torch.bfloat16, cfg, f"{what}, tensor cores {on}")
    for a, b in zip(got[True], got[False]):
        for key, ref in b.items():
            rms = np.sqrt((ref.astype(np.float64) ** 2).mean())
            assert np.sqrt(((a[key] - ref).astype(np.float64) ** 2).mean()) <= 0.05 * rms + 1e-3, key


def _one_direction(cfg, special, gain):
    """Embeddings that share one direction (negative along the first axis, little else), the special token alone on the
    other side of it; queries that ask for that side only, keys that are the stream's leading elements: the special token's
    key, and the block that holds it, get the largest score of every later query that can see them."""
    def edit(t):
        D = cfg["width"]
        e = t["embed"].float()
        e *= 0.1 / e.std()
        e[:, 0] -= 1.0
        e[special] = 0.0
        e[special, 0] = 6.0
        t["embed"] = e.to(t["embed"].dtype)
        for n in [n for n in t if n.endswith((".q", ".k")) and ".right." not in n]:
            d = t[n.rsplit(".", 1)[0] + ".q.norm"].numel()
            eye = torch.zeros((d, D))
            if n.endswith(".q"):
                eye[0, 0] = -1.0
            else:
                eye[:, :d] = torch.eye(d)
            t[n] = eye.repeat(t[n].shape[0] // d, 1).to(t[n].dtype)
        for n in [n for n in t if n.endswith(("q.norm", "k.norm"))]:
            t[n] = torch.full_like(t[n], gain ** 0.5)
    return edit


@pytest.mark.parametrize("at", [0, 37, 63, 64])
def test_one_far_token_that_decides(tmp_path, at):
    """A token hundreds of positions back whose key dominates: through its pooled block in the windowed layer (long after
    it has left the window), and inside a long chunk in the layer with two score maps.  The plain implementation itself
    moves by far more than the tolerance when that token is another one."""
    for layer in (zh.parallel((2, 1, 16, 16, 24, 8, None), (1, 4, 4, (0.5,))), zh.attention(2, 1, 16, 16, 512, diff=0.2)):
        cfg = zh.config(64, 32, [layer])
        sub = tmp_path / layer["type"]
        edits = [_one_direction(cfg, 63, 30.0)] + ([_silence("l0.mix.right.o")] if layer["type"] == "parallel" else [])
        folder = zh.make_folder(sub, cfg, seed=9, gain=1.0, edit=lambda t: [e(t) for e in edits])
        oracle = zh.Oracle(folder)
        toks = np.random.default_rng(1).integers(0, 63, size=400).tolist()
        toks[at] = 63
        other = list(toks)
        other[at] = 5
        like = zh.like_config(cfg)
        moved = np.abs(oracle.logits(toks)[-1] - oracle.logits(other)[-1]).max()
        assert moved > 100 * tolerance(torch.float32, like, None), (layer["type"], moved)
        engine = build_engine(folder, torch.float32, max_tokens=512)
        compare(run_whole(engine, [toks]), oracle, [toks], torch.float32, like, f"far token {at} whole")
        compare(run_tail_by_one(engine, [toks], tail=300), oracle, [toks], torch.float32, like, f"far token {at} decoded")
        compare(run_chunked(engine, [toks], [at + 1, 2, 200, 64]), oracle, [toks], torch.float32, like, f"far token {at} portions")


def test_the_sequences_first_tokens_and_sizes_that_are_one(tmp_path):
    """Sequences of one to ten tokens (nothing has left a window, no block is complete, the state starts at zero), and a
    model whose sizes are all one or equal: one head, one expert, one group, one pass, a pool and a window of one."""
    cfg = zh.CONFIGS["P"]
    folder = zh.make_folder(tmp_path / "p", cfg, seed=5, gain=4.0)
    reqs = zh.random_requests(cfg, [1, 2, 3, 7, 8, 9, 10], seed=1)
    engine = build_engine(folder, torch.float32, max_tokens=64 * 7, max_seqs=7)
    compare_zl(run_whole(engine, reqs), zh.Oracle(folder), reqs, torch.float32, cfg, "first tokens")
    compare_zl(run_batches(engine, reqs, [list(range(7))], [1] * 7), zh.Oracle(folder), reqs, torch.float32, cfg, "first tokens, decoded together")
    ones = zh.config(40, 16, [zh.parallel((1, 1, 16, 16, 1, 1, zh.rot(16)), (1, 16, 16, (1.0,)), zh.moe(1, 1, 16, 1.0, groups=(1, 1))),
                              zh.attention(1, 1, 16, 16, 1, diff=0.0, rotation=zh.rot(16), mlp=zh.moe(2, 2, 16, 1.0, groups=(1, 1)))],
                     loop=(0, 1, 1), logit_scale=1.0)
    folder = zh.make_folder(tmp_path / "ones", ones, seed=6, gain=4.0)
    reqs = zh.random_requests(ones, [70, 3], seed=2)
    engine = build_engine(folder, torch.float32, max_tokens=192)
    compare_zl(run_whole(engine, reqs), zh.Oracle(folder), reqs, torch.float32, ones, "ones whole")
    compare_zl(run_tail_by_one(engine, reqs, tail=60), zh.Oracle(folder), reqs, torch.float32, ones, "ones decoded")


@pytest.mark.parametrize("dtype", DTYPES)
def test_what_a_configuration_leaves_out_does_not_exist(tmp_path, dtype):
    """No pool (a plain window: what has left it is gone), one decay for all heads, values as wide as the keys, no limit on
    the experts, no rotation, no groups, no loop: whole, decoded, in portions and through the CPU model's eyes."""
    left = {"heads": 4, "kv_heads": 2, "dim": 16, "scale": 0.25, "mask": {"size": 40}}
    layer = {"type": "parallel", "mixer": {"left": left, "right": {"heads": 2, "dim": 8, "decay": 0.9}},
             "mlp": {"kind": "moe", "router": {"experts": 4, "top": 4}, "expert": {"ff": 16}}}
    att = {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "scale": 0.25, "diff": 0.2}, "mlp": None}
    cfg = zh.config(70, 32, [layer, att])
    folder = zh.make_folder(tmp_path, cfg, seed=8, gain=3.0)
    oracle = zh.Oracle(folder)
    toks = zh.random_requests(cfg, [150, 20], seed=9)
    engine = build_engine(folder, dtype, max_tokens=256, max_seqs=2)
    assert len(engine.cache.group_keys) == 2 and engine.cache.every == [1, 1]
    compare_zl(run_whole(engine, toks), oracle, toks, dtype, cfg, "whole")
    compare_zl(run_tail_by_one(engine, toks, tail=100), oracle, toks, dtype, cfg, "decoded")
    compare_zl(run_chunked(engine, toks, [63, 2, 65]), oracle, toks, dtype, cfg, "portions")
    from llaisys_b200.models.cpu_model import CpuModel
    assert np.abs(CpuModel.from_folder(folder).step(toks[1]) - oracle.logits(toks[1])).max() < 2e-4


# ----------------------------------------------------------------------------- whole models under every schedule
class Model:
    def __init__(self, name, tmp):
        self.name, self.tmp, self._made = name, tmp, {}

    def at(self, dtype):
        if dtype not in self._made:
            cfg = zh.for_dtype(zh.CONFIGS[self.name], dtype)
            folder = zh.make_folder(self.tmp / str(dtype), cfg, seed=11, gain=zh.GAIN[dtype])
            self._made[dtype] = (cfg, folder, zh.Oracle(folder), zh.random_requests(cfg, [130, 1, 64, 65, 9, 201], seed=3))
        return self._made[dtype]


@pytest.fixture(scope="module", params=["P", "Q", "R"])
def model(request, tmp_path_factory):
    return Model(request.param, tmp_path_factory.mktemp(f"zl{request.param}"))


def _rooms(requests):
    return sum(-(-len(r) // 64) * 64 for r in requests)


def _skip_ill_conditioned(model, dtype):
    """Q norms vectors of five to eight elements (its recurrent heads side by side, its keys): where such a vector is small
    by cancellation, the norm magnifies 16-bit rounding of its inputs by an order of magnitude (the float32 engine is 20
    times further from the float64 evaluation at those positions than elsewhere, and still within its bound).  Against
    the float64 evaluation Q therefore runs in float32 only; in bfloat16 it is compared with itself under other schedules."""
    if model.name == "Q" and dtype == torch.bfloat16:
        pytest.skip("see test_bfloat16_against_the_same_steps_cut_otherwise")


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompts_and_token_by_token(model, dtype):
    _skip_ill_conditioned(model, dtype)
    cfg, folder, oracle, requests = model.at(dtype)
    engine = build_engine(folder, dtype, max_tokens=max(_rooms([r]) for r in requests))
    compare_zl(run_whole(engine, requests), oracle, requests, dtype, cfg, f"{model.name} whole")
    compare_zl(run_tail_by_one(engine, requests, tail=10_000), oracle, requests, dtype, cfg, f"{model.name} token by token")
    compare_zl(run_tail_by_one(engine, requests, tail=32), oracle, requests, dtype, cfg, f"{model.name} tail")
    assert not engine.cache.live_slots


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_with_pages_slots_and_state_rows_used_again(model, dtype):
    _skip_ill_conditioned(model, dtype)
    cfg, folder, oracle, requests = model.at(dtype)
    n = len(requests)
    batches = [list(range(0, n, 2)), list(range(1, n, 2))]
    prompt_lens = [max(1, len(r) - (3 + 5 * i)) for i, r in enumerate(requests)]
    room = max(_rooms([requests[r] for r in b]) for b in batches)
    engine = build_engine(folder, dtype, max_tokens=room, max_seqs=len(batches[0]))
    compare_zl(run_batches(engine, requests, batches, prompt_lens), oracle, requests, dtype, cfg, f"{model.name} batches")
    assert not engine.cache.live_slots
    assert [p.available for p in engine.cache.book.pools] == engine.cache.group_pages
    compare_zl(run_batches(engine, requests, batches[::-1], prompt_lens), oracle, requests, dtype, cfg, f"{model.name} batches again")


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_and_mixed_steps(model, dtype):
    _skip_ill_conditioned(model, dtype)
    cfg, folder, oracle, _ = model.at(dtype)
    requests = zh.random_requests(cfg, [200, 300, 129, 9], seed=41)
    engine = build_engine(folder, dtype, max_tokens=320)
    for cuts in ([70, 60, 1000], [63, 1, 64, 65, 2, 1000], [2, 200, 1000], [64], [2]):
        reqs = requests if cuts != [2] else requests[2:]
        compare_zl(run_chunked(engine, reqs, cuts), oracle, reqs, dtype, cfg, f"{model.name} portions {cuts}")
    requests = zh.random_requests(cfg, [120, 100, 210, 33], seed=43)
    plans = [[50, 1, 1, 1, 40, 1, 0, 1], [0, 0, 90], [70, 60, 0, 40, 1, 1, 30], [1, 1, 1]]
    engine = build_engine(folder, dtype, max_tokens=_rooms(requests), max_seqs=4)
    for turn in range(2):
        compare_zl(run_mixed(engine, requests, plans), oracle, requests, dtype, cfg, f"{model.name} mixed steps, turn {turn}")
        assert not engine.cache.live_slots
        requests, plans = requests[::-1], plans[::-1]


@pytest.mark.parametrize("name, share", [("P", 0.05), ("Q", 0.25)])
def test_bfloat16_against_the_same_steps_cut_otherwise(tmp_path, name, share):
    """bfloat16 with few experts a token (P), and with vectors so short that their norms magnify rounding (Q): which
    experts a token uses, and the last bits of a short vector, may hang on 16-bit rounding against the float64
    implementation, but not on how the request was cut into steps or on what shares its batch.  A lost key, a stale
    state row or a page of another sequence moves every later row by about its own size."""
    cfg = zh.CONFIGS[name]
    folder = zh.make_folder(tmp_path, cfg, seed=12, gain=zh.GAIN[torch.bfloat16])
    requests = zh.random_requests(cfg, [150, 70, 9], seed=2)
    engine = build_engine(folder, torch.bfloat16, max_tokens=_rooms(requests), max_seqs=3)
    whole = run_whole(engine, requests)
    for what, other in (("portions", run_chunked(engine, requests, [63, 2, 65])), ("together", run_batches(engine, requests, [[0, 1, 2]], [100, 64, 1])),
                        ("decoded", run_tail_by_one(engine, requests, tail=40))):
        off = 0
        for key, ref in whole.items():
            rms = np.sqrt((ref.astype(np.float64) ** 2).mean())
            d = np.sqrt(((other[key] - ref).astype(np.float64) ** 2).mean())
            off += d > share * rms + 1e-3
        assert off <= max(2, len(whole) // 25), (what, off, len(whole))


def test_long_decoding_through_captured_steps(tmp_path):
    """Hundreds of single-token steps from a short prompt: pages fill and new ones are taken, rings wrap, blocks complete,
    chunks begin, the state is carried through every step, and the steps are replayed from a captured graph."""
    for dtype in DTYPES:
        cfg = zh.for_dtype(zh.CONFIGS["P"], dtype)
        folder = zh.make_folder(tmp_path / str(dtype), cfg, seed=21, gain=zh.GAIN[dtype])
        oracle = zh.Oracle(folder)
        requests = zh.random_requests(cfg, [330, 290], seed=6)
        engine = build_engine(folder, dtype, max_tokens=_rooms(requests), max_seqs=2)
        assert engine.use_graphs
        compare_zl(run_batches(engine, requests, [[0, 1]], [4, 1]), oracle, requests, dtype, cfg, "long decoding")
        assert engine.graph_replays > 250


# ----------------------------------------------------------------------------- entry points
def _greedy(oracle, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(np.argmax(oracle.logits(seq)[-1])))
    return seq[len(prompt):]


def test_greedy_generation_through_the_entry_point_and_scheduler(tmp_path):
    from llaisys_b200.models import CausalLM, DeviceType
    cfg = zh.CONFIGS["P"]
    folder = zh.make_folder(tmp_path, cfg, seed=31, gain=4.0)
    oracle = zh.Oracle(folder)
    model = CausalLM(folder, DeviceType.NVIDIA, dtype="float32", max_tokens=64 * 4)
    prompts = zh.random_requests(cfg, [5, 9, 2, 70, 1, 17], seed=3)
    # four rooms of 64 tokens for six requests: two batches at least; slots, pages and state rows are used again
    outs = model.generate_batch(prompts, max_new_tokens=12, top_k=1, stop_ids=[])
    for p, new in zip(prompts, outs):
        assert new == _greedy(oracle, p, 12)
    assert model.generate(prompts[0], max_new_tokens=12) == prompts[0] + outs[0]
    assert not model.engine.cache.live_slots


def test_command_line(tmp_path):
    """python -m llaisys_b200.cli on a model folder of this design and on a configuration with random weights; --test
    compares the engine's tokens with those of the package's CPU model."""
    import os
    import sys
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    folder = zh.make_folder(tmp_path / "m", zh.CONFIGS["P"], seed=17, gain=4.0)
    oracle = zh.Oracle(folder)
    (tmp_path / "batch.txt").write_text("5,17,3,200,7,7,7,7,7\n[9, 8]\n1\n")
    out = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--model", str(folder), "--batch-file", str(tmp_path / "batch.txt"),
                          "--max_steps", "6", "--dtype", "float32", "--test"], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.count("Tokens:") == 3 and "Test passed" in out.stdout
    want = [5, 17, 3, 200, 7, 7, 7, 7, 7] + _greedy(oracle, [5, 17, 3, 200, 7, 7, 7, 7, 7], 6)
    assert str(want) in out.stdout or ", ".join(map(str, want)) in out.stdout, out.stdout[-1500:]
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(zh.CONFIGS["Q"]))
    out = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--random-weights", str(cfg), "--seed", "3", "--tokens", "1,2,3",
                          "--max_steps", "4", "--dtype", "float32", "--test"], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "Tokens:" in out.stdout and "Test passed" in out.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_of_a_trace(tmp_path, dtype):
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    cfg = zh.for_dtype(zh.CONFIGS["P"], td)
    folder = zh.make_folder(tmp_path / "m", cfg, seed=13, gain=zh.GAIN[td])
    requests = zh.random_requests(cfg, [1, 7, 90, 20], seed=8)
    lines, rows = [], []
    lines.append({"step": 0, "entries": [{"id": "a", "tokens": requests[0], "want": [0]},
                                         {"id": "c", "tokens": requests[2][:60], "want": list(range(60))}], "end": ["a"]})
    rows.append((0, [(0, 0)] + [(2, p) for p in range(60)]))
    for p in range(60, 90):
        lines.append({"step": p, "entries": [{"id": "c", "tokens": [requests[2][p]], "want": [0]}], "end": ["c"] if p == 89 else []})
        rows.append((p, [(2, p)]))
    lines.append({"step": 500, "entries": [], "end": []})
    lines.append({"step": 501, "entries": [{"id": "b", "tokens": requests[1], "want": list(range(7))},
                                           {"id": "d", "tokens": requests[3], "want": [19]}], "end": ["b", "d"]})
    rows.append((501, [(1, p) for p in range(7)] + [(3, 19)]))
    out_dir = tmp_path / "out"
    proc = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out_dir),
                           "--max-tokens", "128"], input="\n".join(json.dumps(l) for l in lines) + "\n", capture_output=True,
                          text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [int(l.split()[1]) for l in proc.stdout.splitlines() if l.startswith("done ")] == [l["step"] for l in lines]
    oracle = zh.Oracle(folder)
    for step, keys in rows:
        data = np.frombuffer((out_dir / f"{step}.f32").read_bytes(), dtype="<f4").reshape(len(keys), cfg["vocab"])
        for i, (r, p) in enumerate(keys):
            ref = oracle.logits(requests[r])
            assert np.abs(data[i] - ref[p]).max() <= tolerance(td, zh.like_config(cfg), ref) * (1 if dtype == "float32" else 8), (step, r, p)
