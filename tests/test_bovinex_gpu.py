"""The Bovinex family on the layer-list runtime against the plain float64 statement in bovinex_plain.py.

Every test makes its own small configuration and seeded weights.  float32 mode is compared tightly (it shows any wrong
key, a window or kept-first edge that is one token off, a lost state, a wrong expert); bfloat16 mode within bf16 rounding.
Where random weights would hide a fault the scores are sharpened (a large score scale, so that single keys dominate the
softmax) or the router is biased (so that one expert takes every token)."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import bovinex_plain as plain  # noqa: E402

pytestmark = pytest.mark.gpu

from calm_b200 import bovinex, container, registry, serving  # noqa: E402

DENSE = {"ff": 40, "kind": "dense"}
YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}


def moe(experts=6, top=2, ff=12):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def attn(heads=6, kv_heads=2, dim=16, vdim=20, size=7, keep=3, rot=12, base=500.0, scaling=YARN, scale=0.3, mlp=DENSE):
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        mx["mask"] = {"size": size, "keep_first": keep}
    if rot:
        mx["rot"] = {"dims": rot, "base": base}
        if scaling:
            mx["rot"]["scaling"] = scaling
    return {"type": "attention", "mixer": mx, "mlp": mlp}


def gla(heads=3, dim=16, vdim=24, tau=4.0, a_rank=6, mlp=DENSE):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "a_rank": a_rank}, "mlp": mlp}


def config(layers, width=48, vocab=97, eps=1e-5, scale=6.0):
    return {"architecture": "Bovinex", "embedding": {"scale": scale}, "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def weights(cfg, seed=0, favour=None):
    """favour: (expert, bias) -- that expert's router bias, large enough to put it among every token's choices."""
    t = bovinex.random_tensors(cfg, seed)
    if favour:
        for name in t:
            if name.endswith("router.b"):
                t[name][favour[0]] = favour[1]
    return t


def as_f64(t):
    return {k: v.float().numpy().astype(np.float64) for k, v in t.items()}


def tokens(cfg, n, seed=1):
    return [int(x) for x in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]


def rel_err(got, ref):
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    return float(np.sqrt((d * d).mean(-1)).max() / np.sqrt((r * r).mean()))


TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def whole(model, toks):
    s = model.open()
    out = model.step([s], [toks], list(range(len(toks))))
    model.close_seq(s)
    return out


def check_all_ways(cfg, t, toks, dtype="float32", portions=(5, 2, 1), page=4):
    """whole prompt, prompt + token-by-token decoding, and portions: all against the plain statement."""
    ref = plain.forward(cfg, as_f64(t), toks)
    with bovinex.from_tensors(cfg, t, dtype, max_tokens=4 * len(toks) + 64, max_seqs=4, page=page) as m:
        assert rel_err(whole(m, toks), ref) < TOL[dtype]
        for first in {1, max(1, len(toks) // 2)}:
            s = m.open()
            rows = [m.step([s], [toks[:first]], list(range(first)))]
            for p in range(first, len(toks)):
                rows.append(m.step([s], [[toks[p]]], [0]))
            m.close_seq(s)
            assert rel_err(np.concatenate(rows), ref) < TOL[dtype]
        for size in portions:
            s, rows, at = m.open(), [], 0
            while at < len(toks):
                part = toks[at:at + size]
                rows.append(m.step([s], [part], list(range(len(part)))))
                at += len(part)
                size = size + 1 if size > 2 else size  # growing portions: edges fall at ever different places
            m.close_seq(s)
            assert rel_err(np.concatenate(rows), ref) < TOL[dtype]
    return ref


LAYERS = {
    "attention": attn(),
    "attention-noff": attn(mlp=None),
    "attention-mha-norot": attn(heads=3, kv_heads=3, dim=8, vdim=8, rot=0, size=0),
    "attention-fullrot-noscaling": attn(heads=4, kv_heads=1, dim=12, vdim=6, rot=12, scaling=None, size=5, keep=0),
    "attention-window1": attn(heads=2, kv_heads=2, size=1, keep=2, mlp=moe()),
    "attention-keep-beyond-window": attn(size=3, keep=9),
    "gla": gla(),
    "gla-noff": gla(mlp=None),
    "gla-moe": gla(heads=2, dim=32, vdim=16, tau=2.0, mlp=moe()),
    "gla-d24-v20": gla(heads=1, dim=24, vdim=20, tau=16.0, a_rank=3),
    "gla-d64-top1": gla(heads=2, dim=64, vdim=8, mlp=moe(experts=3, top=1)),
    "gla-top-all": gla(mlp=moe(experts=4, top=4, ff=20)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(LAYERS))
def test_each_mechanism_alone(name, dtype):
    cfg = config([LAYERS[name]])
    check_all_ways(cfg, weights(cfg, 3), tokens(cfg, 37), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_align_with_nothing(dtype):
    """Width, head sizes, ranks, expert widths and vocabulary that are multiples of neither 8 nor 4."""
    cfg = config([gla(heads=3, dim=10, vdim=7, a_rank=5, mlp={"ff": 22, "kind": "dense"}),
                  attn(heads=3, kv_heads=3, dim=10, vdim=6, rot=6, size=4, keep=1, mlp=moe(experts=5, top=3, ff=9)),
                  attn(heads=6, kv_heads=2, dim=6, vdim=10, rot=2, size=9, keep=2, mlp=None), gla(heads=1, dim=7, vdim=5, a_rank=1, mlp=moe(experts=2, top=1, ff=3))],
                 width=50, vocab=61, scale=1.0)
    check_all_ways(cfg, weights(cfg, 31), tokens(cfg, 45), dtype, portions=(17, 2))


def test_other_layer_orders():
    for k, order in enumerate(([gla(), gla(mlp=moe()), attn()], [attn(mlp=moe()), attn(size=4, keep=0), gla(mlp=None), attn(mlp=None)])):
        cfg = config(order, width=40)
        check_all_ways(cfg, weights(cfg, 5 + k), tokens(cfg, 41), portions=(6,))


def test_residual_stream_after_every_layer():
    cfg = config([attn(), gla(mlp=moe()), gla(), attn(mlp=moe(top=1))])
    t, toks = weights(cfg, 8), tokens(cfg, 19)
    trace = []
    plain.forward(cfg, as_f64(t), toks, trace)
    with bovinex.from_tensors(cfg, t, "float32", max_tokens=64, max_seqs=2) as m:
        m.set_trace(True)
        whole(m, toks)
        got = m.read_trace(len(toks))
    assert got.shape[0] == len(trace) == 4
    for g, r in zip(got, trace):
        assert np.abs(g - r).max() < 1e-4 * max(1.0, np.abs(r).max())


def test_window_and_kept_first_edges_show():
    """Sharp scores: a window or a kept-first count that is one token off moves the logits far more than the tolerance, in
    prompts, portions and decoding alike (the same check passes for the right values)."""
    cfg = config([attn(size=6, keep=3, scale=1.2)])
    t, toks = weights(cfg, 11), tokens(cfg, 60)
    ref = check_all_ways(cfg, t, toks, portions=(7, 2))
    for key in ("size", "keep_first"):
        for off in (-1, 1):
            wrong = copy.deepcopy(cfg)
            wrong["layers"][0]["mixer"]["mask"][key] += off
            assert rel_err(plain.forward(wrong, as_f64(t), toks), ref) > 100 * TOL["float32"]


def test_rotation_details_show():
    """Partial rotation, the pairing of channels, the rescaled frequencies and the factor on cos and sin all reach the logits."""
    cfg = config([attn(size=0, rot=12, scale=1.0)])
    t, toks = weights(cfg, 12), tokens(cfg, 50)
    ref = check_all_ways(cfg, t, toks, portions=(9,))
    for change in ({"dims": 16}, {"base": 400.0}, {"scaling": None}, {"scaling": dict(YARN, factor=4.5)}, {"scaling": dict(YARN, slow=1.0)}, {"scaling": dict(YARN, fast=2.0)}):
        wrong = copy.deepcopy(cfg)
        wrong["layers"][0]["mixer"]["rot"].update(change)
        assert rel_err(plain.forward(wrong, as_f64(t), toks), ref) > 100 * TOL["float32"]


def test_far_positions_keep_their_angle():
    """Two thousand tokens under a short window: the angles of the fastest pairs reach thousands of radians and still have to
    agree with the float64 statement; the kept first tokens are far behind every later window and pages are crossed all along."""
    cfg = config([attn(heads=2, kv_heads=1, dim=8, vdim=8, size=12, keep=2, rot=8, base=100.0, scaling=None, scale=1.0, mlp=None)], width=24, vocab=31)
    t, toks = weights(cfg, 13), tokens(cfg, 2100)
    ref = plain.forward(cfg, as_f64(t), toks)
    with bovinex.from_tensors(cfg, t, "float32", max_tokens=2304, max_seqs=2, page=16) as m:
        s = m.open()
        rows = [m.step([s], [toks[:2050]], list(range(2050)))]
        for p in range(2050, 2100):
            rows.append(m.step([s], [[toks[p]]], [0]))
        assert rel_err(np.concatenate(rows), ref) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_context_with_shared_out_keys(dtype):
    """Decoding few tokens over a context of several hundred: the attention kernel shares one query's keys (kept first tokens
    and window alike) out over several CTAs and folds the shares; the linear-attention state has 128 key channels."""
    cfg = config([attn(size=200, keep=40, scale=1.0 if dtype == "float32" else 0.3), attn(size=0, keep=0, scale=0.3), gla(heads=1, dim=128, vdim=16, mlp=None)])
    t, toks = weights(cfg, 15), tokens(cfg, 330)
    ref = plain.forward(cfg, as_f64(t), toks)
    with bovinex.from_tensors(cfg, t, dtype, max_tokens=700, max_seqs=2, page=16) as m:
        s = m.open()
        rows = [m.step([s], [toks[:300]], list(range(300)))]
        for p in range(300, 330):
            rows.append(m.step([s], [[toks[p]]], [0]))
        assert rel_err(np.concatenate(rows), ref) < TOL[dtype]
        s2 = m.open()  # the same prompt in two-token portions beside the finished sequence
        rows = [m.step([s2], [toks[a:a + 2]], [0, 1]) for a in range(0, 330, 2)]
        assert rel_err(np.concatenate(rows), ref) < TOL[dtype]


def test_prompt_attention_as_products_matches_the_fused_kernel(monkeypatch):
    """bfloat16 mode computes a long portion's attention as tensor-core products over gathered keys (the kept first tokens in
    front of the window's keys, the per-channel gate in the value product's epilogue), short portions with the fused kernel.
    Both sit within bf16 rounding of the plain statement, also for a portion that continues a cached prefix and for kept tokens
    that reach into the first query's window; an edge that is one token off shows far above that."""
    for size, keep in ((23, 5), (4, 30)):
        cfg = config([attn(size=size, keep=keep, scale=0.8), attn(size=0, heads=4, kv_heads=4, dim=8, vdim=8, rot=4)])
        t, toks = weights(cfg, 16), tokens(cfg, 120)
        ref = plain.forward(cfg, as_f64(t), toks)
        errs = {}
        for products in ("1", "0"):
            monkeypatch.setenv("CALM_B200_SEQ_ATTN_PRODUCTS", products)
            with bovinex.from_tensors(cfg, t, "bfloat16", max_tokens=300, max_seqs=3, page=8) as m:
                s1, s2 = m.open(), m.open()
                a = m.step([s1], [toks[:50]], list(range(50)))
                b = m.step([s1, s2], [toks[50:], toks[:3]], list(range(73)))  # 70 more tokens on the products path beside a 3-token portion
                errs[products] = rel_err(np.concatenate([a, b[:70]]), ref)
                assert rel_err(b[70:], ref[:3]) < TOL["bfloat16"]
        assert errs["1"] < TOL["bfloat16"] and errs["0"] < TOL["bfloat16"] and errs["1"] < 3 * errs["0"] + 1e-3
        for key in ("size", "keep_first"):
            for off in (-1, 1):
                wrong = copy.deepcopy(cfg)
                wrong["layers"][0]["mixer"]["mask"][key] += off
                assert rel_err(plain.forward(wrong, as_f64(t), toks), ref) > 4 * errs["1"]


def test_tensor_core_products_match_the_warp_level_ones(monkeypatch):
    """bfloat16 mode runs products over many tokens on tcgen05 (grouped ones for the experts included) and everything else on
    mma.sync; same bf16 inputs, fp32 sums in another order.  Sizes include edges that do not fill a tile in M, N or K, and
    groups that start and end inside a tile."""
    cfg = config([attn(heads=4, kv_heads=2, dim=32, vdim=24, size=50, keep=4, mlp=moe(experts=5, top=2, ff=40)), gla(heads=2, dim=32, vdim=40, mlp=moe(experts=3, top=1, ff=72))],
                 width=88, vocab=131)
    t, toks = weights(cfg, 17), tokens(cfg, 300)
    outs = {}
    for tc in ("1", "0"):
        monkeypatch.setenv("CALM_B200_SEQ_TC", tc)
        with bovinex.from_tensors(cfg, t, "bfloat16", max_tokens=640, max_seqs=2, page=16) as m:
            s1 = m.open()
            outs[tc] = np.concatenate([m.step([s1], [toks[:237]], list(range(237))), m.step([s1], [toks[237:]], list(range(63)))])
            if tc == "1":
                m.perf(True)
                whole(m, toks)
                stats = m.perf_stats()
                m.perf(False)
                assert stats["gemm_tcgen05"][3] > 0
    assert rel_err(outs["1"], outs["0"]) < 2e-3  # identical inputs; intermediate bf16 roundings may flip on last-bit differences
    assert rel_err(outs["1"], plain.forward(cfg, as_f64(t), toks)) < TOL["bfloat16"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_expert_takes_every_token(dtype):
    """A router bias that puts one expert among every token's choices: its group spans several tiles of the grouped products,
    other groups are short or empty, and the mixing weights stay a softmax restricted to the scores of the experts taken."""
    cfg = config([gla(mlp=moe(experts=7, top=2, ff=16)), attn(mlp=moe(experts=4, top=1, ff=16))])
    t, toks = weights(cfg, 18, favour=(2, 30.0)), tokens(cfg, 200)
    ref = plain.forward(cfg, as_f64(t), toks)
    idx, _ = plain.route(np.random.default_rng(0).normal(size=(50, cfg["width"])), plain.sub(as_f64(t), "l0.mlp."), 2)
    assert (idx[:, 0] == 2).all()
    with bovinex.from_tensors(cfg, t, dtype, max_tokens=512, max_seqs=2, page=16) as m:
        assert rel_err(whole(m, toks), ref) < TOL[dtype]
        s = m.open()
        rows = [m.step([s], [toks[:150]], list(range(150)))] + [m.step([s], [[x]], [0]) for x in toks[150:]]
        assert rel_err(np.concatenate(rows), ref) < TOL[dtype]


def test_long_decoding_keeps_state():
    cfg = config([gla(tau=2.0), attn(size=12, keep=2), gla(mlp=moe())])
    t, toks = weights(cfg, 14), tokens(cfg, 130)
    ref = plain.forward(cfg, as_f64(t), toks)
    with bovinex.from_tensors(cfg, t, "float32", max_tokens=200, max_seqs=2, page=8) as m:
        s = m.open()
        rows = [m.step([s], [[x]], [0]) for x in toks]
        assert rel_err(np.concatenate(rows), ref) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_equals_each_alone(dtype):
    cfg = config([attn(mlp=moe()), gla(), attn(size=4, keep=1, mlp=None), gla(mlp=moe(top=1))])
    t = weights(cfg, 21)
    prompts = [tokens(cfg, n, seed=n) for n in (1, 9, 30, 2)]
    tails = [tokens(cfg, n, seed=50 + n) for n in (6, 3, 0, 6)]
    p = as_f64(t)
    refs = [plain.forward(cfg, p, a + b) for a, b in zip(prompts, tails)]
    with bovinex.from_tensors(cfg, t, dtype, max_tokens=192, max_seqs=5, page=4) as m:
        slots = [m.open() for _ in prompts]
        out = m.step(slots, prompts, list(range(sum(len(a) for a in prompts))))
        got, at = [], 0
        for a in prompts:
            got.append([out[at:at + len(a)]])
            at += len(a)
        for k in range(6):  # decoded together; the shorter ones leave earlier
            live = [i for i, b in enumerate(tails) if k < len(b)]
            o = m.step([slots[i] for i in live], [[tails[i][k]] for i in live], list(range(len(live))))
            for j, i in enumerate(live):
                got[i].append(o[j:j + 1])
        for i, r in enumerate(refs):
            assert rel_err(np.concatenate(got[i]), r) < TOL[dtype]
        if dtype == "float32":  # a row does not depend on what else is in the batch, beyond rounding
            alone = whole(m, prompts[2])
            assert np.abs(alone - np.concatenate(got[2])[:30]).max() < 1e-5 * np.abs(alone).max()


def test_slots_and_pages_are_used_again():
    cfg = config([attn(), gla(mlp=moe()), gla()])
    t = weights(cfg, 22)
    p = as_f64(t)
    with bovinex.from_tensors(cfg, t, "float32", max_tokens=48, max_seqs=2, page=4) as m:
        free0 = m.free_pages()
        for rnd in range(4):  # every pass fills the pool almost completely, with other lengths than the pass before
            a, b = tokens(cfg, 20 + rnd, seed=rnd), tokens(cfg, 23 - rnd, seed=9 + rnd)
            sa, sb = m.open(), m.open()
            out = m.step([sa, sb], [a, b], list(range(len(a) + len(b))))
            assert rel_err(out[:len(a)], plain.forward(cfg, p, a)) < TOL["float32"]
            assert rel_err(out[len(a):], plain.forward(cfg, p, b)) < TOL["float32"]
            m.close_seq(sb if rnd % 2 else sa)
            m.close_seq(sa if rnd % 2 else sb)
            assert m.free_pages() == free0
        s = m.open()
        with pytest.raises(Exception):
            m.step([s], [tokens(cfg, 4 * free0 + 1)], [0])  # more than the pool holds: refused, nothing has run
        assert m.length(s) == 0


def test_greedy_generation_through_the_scheduler():
    cfg = config([attn(), gla(mlp=moe()), attn(size=5, keep=2, mlp=None)])
    t = weights(cfg, 23)
    p = as_f64(t)
    prompts = [tokens(cfg, n, seed=70 + n) for n in (5, 17, 1)]
    with bovinex.from_tensors(cfg, t, "float32", max_tokens=256, max_seqs=2, page=8) as m:
        outs = serving.generate(m, prompts, 12, max_batch=2)  # three requests, two slots: a second batch follows the first
        assert m.free_pages() == 256 // 8 + 2
    for pr, out in zip(prompts, outs):
        assert len(out) == 12
        lg = plain.forward(cfg, p, pr + out)
        for k, tok in enumerate(out):  # each generated token is the plain statement's argmax given the same history
            row = lg[len(pr) + k - 1]
            assert tok == int(row.argmax()) or row.max() - row[tok] < 1e-4 * np.abs(row).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_from_a_model_folder(tmp_path, dtype):
    """bin/trace_run end to end: a model folder written with the container writer and found through the registry, steps on
    standard input (a batch of unequal prompts, decoding together while requests leave, a second batch afterwards), logits
    files compared with the plain statement."""
    cfg = config([gla(heads=2, dim=32, vdim=16, mlp=moe(experts=4, top=2, ff=24)), attn(heads=4, kv_heads=1, dim=16, vdim=8, size=11, keep=2, scale=0.5),
                  attn(heads=2, kv_heads=2, dim=8, vdim=8, size=3, keep=0, rot=4, mlp=None), gla(heads=1, dim=8, vdim=40, tau=1.0)], width=72, vocab=211, eps=1e-6, scale=3.0)
    t = weights(cfg, 41)
    folder, out = tmp_path / "model", tmp_path / "out"
    folder.mkdir(), out.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    container.write_tensors(str(folder / "model.safetensors"), t)
    assert registry.architecture_of(str(folder)) == "Bovinex"
    reqs = {"a": tokens(cfg, 46, 1), "b": tokens(cfg, 9, 2), "c": tokens(cfg, 4, 3), "d": tokens(cfg, 30, 4), "e": tokens(cfg, 2, 5)}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": reqs["a"][:40], "want": [0, 17, 39]}, {"id": "b", "tokens": reqs["b"][:6], "want": [5]},
                                     {"id": "c", "tokens": reqs["c"][:1], "want": [0]}], "end": []}]
    for k in range(3):
        ent = [{"id": "a", "tokens": [reqs["a"][40 + k]], "want": [0]}, {"id": "b", "tokens": [reqs["b"][6 + k]], "want": [0] if k != 1 else []},
               {"id": "c", "tokens": [reqs["c"][1 + k]], "want": [0]}]
        steps.append({"step": 1 + k, "entries": ent, "end": ["b", "c"] if k == 2 else []})
    for k in range(3):
        steps.append({"step": 4 + k, "entries": [{"id": "a", "tokens": [reqs["a"][43 + k]], "want": [0]}], "end": ["a"] if k == 2 else []})
    steps.append({"step": 7, "entries": [{"id": "d", "tokens": reqs["d"][:29], "want": [28]}, {"id": "e", "tokens": reqs["e"][:1], "want": []}], "end": []})
    steps.append({"step": 8, "entries": [{"id": "d", "tokens": reqs["d"][29:], "want": [0]}, {"id": "e", "tokens": reqs["e"][1:], "want": [0]}], "end": ["d", "e"]})
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out), "--max-tokens", "96"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.splitlines() if ln.startswith("done")] == ["done %d" % s["step"] for s in steps]
    ref = {k: plain.forward(cfg, as_f64(t), v) for k, v in reqs.items()}
    at = {k: 0 for k in reqs}
    for s in steps:
        rows = []
        for e in s["entries"]:
            rows += [ref[e["id"]][at[e["id"]] + w] for w in e["want"]]
            at[e["id"]] += len(e["tokens"])
        path = out / ("%d.f32" % s["step"])
        if rows:
            got = np.fromfile(path, "<f4").reshape(len(rows), cfg["vocab"])
            assert rel_err(got, np.stack(rows)) < TOL[dtype]
        else:
            assert not path.exists()
