"""The Vimulorn family on the layer-list runtime against the plain float64 statement in vimulorn_plain.py.

Every test makes its own small configuration and seeded weights.  float32 mode is compared tightly (it shows any wrong
key, window edge, lost state or missing sink); bfloat16 mode within bf16 rounding.  Where random weights would hide a
fault the weights are sharpened (queries and keys scaled up so single keys dominate the softmax, large sinks)."""
import copy
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import vimulorn_plain as plain  # noqa: E402

pytestmark = pytest.mark.gpu

from calm_b200 import serving, vimulorn  # noqa: E402

MLP = {"ff": 40, "kind": "dense", "limit": 1.5}


def latent(heads=4, dim=16, vdim=24, kv_rank=40, q_rank=24, scale=0.3, mlp=MLP):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}, "mlp": mlp}


def delta(heads=4, kv_heads=2, dim=16, vdim=24, conv=4, a_rank=8, g_rank=12, mlp=MLP):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "a_rank": a_rank, "g_rank": g_rank}, "mlp": mlp}


def window(heads=6, kv_heads=2, dim=16, vdim=20, conv=2, size=7, scale=0.4, mlp=MLP):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "mask": {"size": size}, "scale": scale}, "mlp": mlp}


def config(layers, width=48, vocab=97, loop=None, eps=1e-5):
    cfg = {"architecture": "Vimulorn", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def weights(cfg, seed=0, sharpen=0.0, sink=None):
    t = vimulorn.random_tensors(cfg, seed)
    for name in list(t):
        if sharpen and name.endswith((".mix.uq", ".mix.q")) and ".conv" not in name:
            t[name] = (t[name].float() * sharpen).to(torch.bfloat16)
        if sink is not None and name.endswith(".sink"):
            t[name] = torch.full_like(t[name], sink)
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
    with vimulorn.from_tensors(cfg, t, dtype, max_tokens=4 * len(toks) + 64, max_seqs=4, page=page) as m:
        got = whole(m, toks)
        assert rel_err(got, ref) < TOL[dtype]
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", [latent(), delta(), window(), latent(mlp=None), delta(heads=3, kv_heads=3, dim=24, vdim=8, conv=1, mlp=None), window(heads=2, kv_heads=2, size=1),
                                   delta(heads=2, kv_heads=1, dim=32, vdim=20, conv=2), delta(heads=2, kv_heads=2, dim=64, vdim=32, conv=3, mlp=None)],
                         ids=["latent", "delta", "window", "latent-noff", "delta-taps1", "window-size1", "delta-d32-v20", "delta-d64"])
def test_each_mixer_alone(layer, dtype):
    cfg = config([layer])
    check_all_ways(cfg, weights(cfg, 3), tokens(cfg, 37), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_align_with_nothing(dtype):
    """Width, ranks, head sizes and vocabulary that are multiples of neither 8 nor 4: every vector path has to step aside."""
    mlp = {"ff": 22, "kind": "dense", "limit": 0.8}
    cfg = config([latent(heads=3, dim=10, vdim=6, kv_rank=14, q_rank=18, mlp=mlp), delta(heads=3, kv_heads=1, dim=10, vdim=7, conv=5, a_rank=3, g_rank=5, mlp=mlp),
                  window(heads=3, kv_heads=3, dim=6, vdim=10, conv=3, size=4, mlp=mlp)], width=50, vocab=61, loop=(0, 3, 2))
    check_all_ways(cfg, weights(cfg, 31), tokens(cfg, 45), dtype, portions=(17, 2))


def test_latent_wider_than_the_register_tiles():
    """A latent of more than 512 channels: keys no longer fit a lane's registers and values take the one-head-per-CTA path."""
    cfg = config([latent(heads=2, dim=8, vdim=8, kv_rank=528, q_rank=16)])
    check_all_ways(cfg, weights(cfg, 32), tokens(cfg, 70), "float32", portions=(40,))
    check_all_ways(cfg, weights(cfg, 32), tokens(cfg, 70), "bfloat16", portions=(40,))


def test_mixed_stack_with_loop_in_the_middle():
    cfg = config([window(conv=3, size=5), latent(), delta(), window(heads=4, kv_heads=4, dim=8, vdim=8, conv=4, size=9)], width=40, loop=(1, 3, 2))
    assert plain.layer_runs(cfg)[0] == [0, 1, 2, 1, 2, 3]
    check_all_ways(cfg, weights(cfg, 5), tokens(cfg, 41))


def test_residual_stream_after_every_run():
    cfg = config([latent(), delta(), window()], loop=(0, 2, 3))
    t, toks = weights(cfg, 8), tokens(cfg, 19)
    trace = []
    plain.forward(cfg, as_f64(t), toks, trace)
    with vimulorn.from_tensors(cfg, t, "float32", max_tokens=64, max_seqs=2) as m:
        m.set_trace(True)
        whole(m, toks)
        got = m.read_trace(len(toks))
    assert got.shape[0] == len(trace) == 7
    for g, r in zip(got, trace):
        assert np.abs(g - r).max() < 1e-4 * max(1.0, np.abs(r).max())


def test_window_edges_show():
    """Sharp scores and a large window-relative length: a window one token too wide or too narrow moves the logits far more
    than the tolerance, in prompts and in decoding alike."""
    cfg = config([window(size=6, conv=2, scale=1.0)])
    t = weights(cfg, 11, sharpen=6.0)
    toks = tokens(cfg, 60)
    ref = check_all_ways(cfg, t, toks, portions=(7, 2))
    for off in (-1, 1):
        wrong = copy.deepcopy(cfg)
        wrong["layers"][0]["mixer"]["mask"]["size"] += off
        assert rel_err(plain.forward(wrong, as_f64(t), toks), ref) > 100 * TOL["float32"]


def test_sink_shows():
    cfg = config([window(size=8)])
    t = weights(cfg, 12, sink=3.0)
    toks = tokens(cfg, 30)
    ref = check_all_ways(cfg, t, toks)
    none = {k: (torch.full_like(v, -60.0) if k.endswith(".sink") else v) for k, v in t.items()}
    assert rel_err(plain.forward(cfg, as_f64(none), toks), ref) > 100 * TOL["float32"]


def test_far_keys_and_page_borders():
    """Peaked latent attention over a prompt of many pages: single far keys carry the output."""
    cfg = config([latent(scale=1.0), window(size=33, scale=1.0)])
    t = weights(cfg, 13, sharpen=5.0)
    toks = tokens(cfg, 150)
    ref = plain.forward(cfg, as_f64(t), toks)
    with vimulorn.from_tensors(cfg, t, "float32", max_tokens=400, max_seqs=2, page=16) as m:
        assert rel_err(whole(m, toks), ref) < TOL["float32"]
        s = m.open()
        rows = [m.step([s], [toks[:100]], list(range(100)))]
        for p in range(100, 150):  # decoding across the borders of pages 6..9 and with the window's far edge moving through them
            rows.append(m.step([s], [[toks[p]]], [0]))
        assert rel_err(np.concatenate(rows), ref) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_context_with_shared_out_keys(dtype):
    """Decoding few tokens over a context of several hundred: the attention kernels share one query's keys out over
    several CTAs and fold the shares; the delta state sits in registers (dim 128)."""
    cfg = config([latent(scale=1.0), window(size=200, scale=1.0), delta(heads=1, kv_heads=1, dim=128, vdim=16, conv=2, mlp=None)])
    t = weights(cfg, 15, sharpen=3.0 if dtype == "float32" else 0.0, sink=1.0)  # bf16 inputs under sharpened scores: rounding alone passes 4e-2
    toks = tokens(cfg, 330)
    ref = plain.forward(cfg, as_f64(t), toks)
    with vimulorn.from_tensors(cfg, t, dtype, max_tokens=700, max_seqs=2, page=16) as m:
        s = m.open()
        rows = [m.step([s], [toks[:300]], list(range(300)))]
        for p in range(300, 330):
            rows.append(m.step([s], [[toks[p]]], [0]))
        assert rel_err(np.concatenate(rows), ref) < TOL[dtype]
        s2 = m.open()  # the same prompt in two-token portions beside the finished sequence
        rows = [m.step([s2], [toks[a:a + 2]], [0, 1]) for a in range(0, 330, 2)]
        assert rel_err(np.concatenate(rows), ref) < TOL[dtype]


def test_prompt_attention_as_products_matches_the_fused_kernel(monkeypatch):
    """bfloat16 mode computes a long portion's attention as tensor-core products over gathered keys, and short portions
    with the fused kernel.  Both must sit within bf16 rounding of the plain statement, at window edges and with the sink,
    also for a portion that continues a cached prefix; a window that is one token off must show far above that."""
    cfg = config([window(size=23, conv=2, scale=1.0), latent(scale=1.0)])
    t = weights(cfg, 16, sharpen=2.0, sink=2.0)
    toks = tokens(cfg, 120)
    ref = plain.forward(cfg, as_f64(t), toks)
    errs = {}
    for products in ("1", "0"):
        monkeypatch.setenv("CALM_B200_SEQ_ATTN_PRODUCTS", products)
        with vimulorn.from_tensors(cfg, t, "bfloat16", max_tokens=300, max_seqs=3, page=8) as m:
            s1, s2 = m.open(), m.open()
            a = m.step([s1], [toks[:50]], list(range(50)))
            b = m.step([s1, s2], [toks[50:], toks[:3]], list(range(73)))  # 70 more tokens on the products path beside a 3-token portion
            errs[products] = rel_err(np.concatenate([a, b[:70]]), ref)
            assert rel_err(b[70:], ref[:3]) < TOL["bfloat16"]
    assert errs["1"] < TOL["bfloat16"] and errs["0"] < TOL["bfloat16"] and errs["1"] < 3 * errs["0"] + 1e-3
    for off in (-1, 1):
        wrong = copy.deepcopy(cfg)
        wrong["layers"][0]["mixer"]["mask"]["size"] += off
        assert rel_err(plain.forward(wrong, as_f64(t), toks), ref) > 4 * errs["1"]


def test_tensor_core_products_match_the_warp_level_ones(monkeypatch):
    """bfloat16 mode runs products over many tokens on tcgen05 (TMA-fed, TMEM accumulators) and everything else on mma.sync;
    same bf16 inputs, fp32 sums in another order.  Sizes include edges that do not fill a tile in M, N or K."""
    cfg = config([latent(heads=4, dim=32, vdim=24, kv_rank=72, q_rank=40), delta(heads=2, kv_heads=1, dim=32, vdim=40), window(size=50)], width=88, vocab=131)
    t, toks = weights(cfg, 17), tokens(cfg, 200)
    outs = {}
    for tc in ("1", "0"):
        monkeypatch.setenv("CALM_B200_SEQ_TC", tc)
        with vimulorn.from_tensors(cfg, t, "bfloat16", max_tokens=512, max_seqs=2, page=16) as m:
            s1 = m.open()
            outs[tc] = np.concatenate([m.step([s1], [toks[:137]], list(range(137))), m.step([s1], [toks[137:]], list(range(63)))])
            stats = None
            if tc == "1":
                m.perf(True)
                whole(m, toks)
                stats = m.perf_stats()
                m.perf(False)
                assert stats["gemm_tcgen05"][3] > 0
    assert rel_err(outs["1"], outs["0"]) < 2e-3  # identical inputs; intermediate bf16 roundings may flip on last-bit differences
    assert rel_err(outs["1"], plain.forward(cfg, as_f64(t), toks)) < TOL["bfloat16"]


def test_long_decoding_keeps_state():
    cfg = config([delta(conv=3), window(size=12, conv=3)])
    t, toks = weights(cfg, 14), tokens(cfg, 130)
    ref = plain.forward(cfg, as_f64(t), toks)
    with vimulorn.from_tensors(cfg, t, "float32", max_tokens=200, max_seqs=2, page=8) as m:
        s = m.open()
        rows = [m.step([s], [[x]], [0]) for x in toks]
        assert rel_err(np.concatenate(rows), ref) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_equals_each_alone(dtype):
    cfg = config([latent(), delta(), window()], loop=(0, 2, 2))
    t = weights(cfg, 21)
    prompts = [tokens(cfg, n, seed=n) for n in (1, 9, 30, 2)]
    tails = [tokens(cfg, n, seed=50 + n) for n in (6, 3, 0, 6)]
    p = as_f64(t)
    refs = [plain.forward(cfg, p, a + b) for a, b in zip(prompts, tails)]
    with vimulorn.from_tensors(cfg, t, dtype, max_tokens=192, max_seqs=5, page=4) as m:
        slots = [m.open() for _ in prompts]
        want = list(range(sum(len(a) for a in prompts)))
        out = m.step(slots, prompts, want)
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
        if dtype == "float32":  # a row does not depend on what else is in the batch (key shares may be cut differently: rounding only)
            alone = whole(m, prompts[2])
            assert np.abs(alone - np.concatenate(got[2])[:30]).max() < 1e-5 * np.abs(alone).max()


def test_slots_and_pages_are_used_again():
    cfg = config([latent(), delta(), window()])
    t = weights(cfg, 22)
    p = as_f64(t)
    with vimulorn.from_tensors(cfg, t, "float32", max_tokens=48, max_seqs=2, page=4) as m:
        free0 = m.free_pages()
        for rnd in range(4):  # every round fills the pool almost completely, with other lengths than the round before
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
    cfg = config([latent(), delta(), window()], loop=(1, 2, 2))
    t = weights(cfg, 23)
    p = as_f64(t)
    prompts = [tokens(cfg, n, seed=70 + n) for n in (5, 17, 1)]
    with vimulorn.from_tensors(cfg, t, "float32", max_tokens=256, max_seqs=2, page=8) as m:
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
    """bin/trace_run end to end: a model folder written with the container writer, steps on standard input (a batch of unequal
    prompts, decoding together while requests leave, a second batch afterwards), logits files compared with the plain statement."""
    import json
    import subprocess

    from calm_b200 import container

    cfg = config([delta(heads=2, kv_heads=2, dim=32, vdim=16, conv=2), window(heads=4, kv_heads=1, dim=16, vdim=8, conv=4, size=11, scale=0.5),
                  latent(heads=3, dim=8, vdim=16, kv_rank=24, q_rank=16, scale=0.6), window(heads=2, kv_heads=2, dim=8, vdim=8, conv=1, size=3, mlp=None)],
                 width=72, vocab=211, loop=(1, 3, 2), eps=1e-6)
    t = weights(cfg, 41, sink=0.5)
    folder, out = tmp_path / "model", tmp_path / "out"
    folder.mkdir(), out.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    container.write_tensors(str(folder / "model.safetensors"), t)
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


def test_temperature_sampling_through_the_scheduler():
    """Temperature / min-p requests go through the library's device sampler with the scheduler's generator state: the same seed
    gives the same tokens, every token is one the min-p rule allows under the plain statement's distribution."""
    cfg = config([latent(), window()])
    t = weights(cfg, 51)
    p = as_f64(t)
    prompts = [tokens(cfg, 6, 91), tokens(cfg, 11, 92)]
    with vimulorn.from_tensors(cfg, t, "float32", max_tokens=128, max_seqs=2, page=8) as m:
        a = serving.generate(m, prompts, 6, temperature=0.9, minp=0.1, seed=7)
        b = serving.generate(m, prompts, 6, temperature=0.9, minp=0.1, seed=7)
        c = serving.generate(m, prompts, 6, temperature=0.9, minp=0.1, seed=8)
    assert a == b and all(len(o) == 6 for o in a) and a != c
    for pr, out in zip(prompts, a):
        lg = plain.forward(cfg, p, pr + out)
        for k, tok in enumerate(out):
            row = lg[len(pr) + k - 1] / 0.9
            pr_tok = np.exp(row[tok] - row.max())
            assert pr_tok >= 0.1 * (1 - 1e-3)  # min-p: at least minp times the most likely token's probability
