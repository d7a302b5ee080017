"""Host side of the Bovinex family without a GPU: the plan that binds a checkpoint to layer records (stacking order, biases,
experts side by side), the registry, and properties of the plain statement the GPU tests lean on."""
import json
import math
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import bovinex_plain as plain  # noqa: E402

from calm_b200 import bovinex, container, registry, seqlib  # noqa: E402


def small_cfg():
    return {"architecture": "Bovinex", "vocab": 50, "width": 16, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
            "layers": [
                {"type": "gla", "mixer": {"heads": 2, "dim": 4, "vdim": 8, "tau": 8.0, "a_rank": 3},
                 "mlp": {"kind": "moe", "expert": {"ff": 6}, "router": {"experts": 3, "top": 2}}},
                {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 4, "scale": 0.3, "mask": {"size": 5, "keep_first": 2},
                                                "rot": {"dims": 4, "base": 100.0, "scaling": {"factor": 2.0, "original": 32, "fast": 4.0, "slow": 1.0}}},
                 "mlp": {"kind": "dense", "ff": 12}},
                {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 4, "scale": 0.5}, "mlp": None}]}


def test_plan_stacks_inputs_in_kernel_order():
    cfg = small_cfg()
    t = bovinex.random_tensors(cfg, 1)
    head, layers, up = bovinex.plan(cfg, t)
    assert head["norm_kind"] == seqlib.NORM_RMS and head["norm_offset"] == 1.0 and head["block"] == seqlib.BLOCK_PARALLEL and head["embed_scale"] == 4.0
    # what reads the normed input is one matrix per layer: the mixer's rows, then the router's or the dense unit's up rows
    assert torch.equal(up["l0.mix.in"], torch.cat([t["l0.mix." + n] for n in ("q", "k", "v", "g", "a1")] + [t["l0.mlp.router"]]))
    assert torch.equal(up["l0.mix.in.b"], torch.cat([torch.zeros(2 * 8 + 2 * 16 + 3, dtype=torch.bfloat16), t["l0.mlp.router.b"]]))
    assert torch.equal(up["l1.mix.in"], torch.cat([t["l1.mix." + n] for n in ("q", "k", "v", "g")] + [t["l1.mlp.up"]]))
    assert torch.equal(up["l1.mix.in.b"], torch.cat([t["l1.mix.q.b"], t["l1.mix.k.b"], t["l1.mix.v.b"], torch.zeros(16 + 12, dtype=torch.bfloat16)]))
    assert torch.equal(up["l2.mix.in"], torch.cat([t["l2.mix." + n] for n in ("q", "k", "v", "g")])) and up["l2.mix.in.b"].shape == (8 + 8 + 8 + 8,)
    assert up["l0.mlp.gate_up"].shape == (3 * 12, 16) and torch.equal(up["l0.mlp.gate_up"][12:18], t["l0.mlp.e1.gate"]) and torch.equal(up["l0.mlp.gate_up"][18:24], t["l0.mlp.e1.up"])
    assert torch.equal(up["l0.mlp.downs"][32:48], t["l0.mlp.e2.down"])
    g, a, plainattn = layers
    assert g["type"] == seqlib.SEQ_GLA and g["a_rank"] == 3 and g["ff_kind"] == seqlib.FF_MOE and (g["experts"], g["top"], g["ff"], g["in_tail"]) == (3, 2, 6, 3) and g["tau"] == 8.0
    assert a["type"] == seqlib.SEQ_GQA and (a["window"], a["keep_first"], a["rot_dims"], a["rot_factor"], a["rot_original"]) == (5, 2, 4, 2.0, 32.0) and a["ff_kind"] == seqlib.FF_RELU2
    assert a["in_tail"] == a["ff"] == 12 and "w_gate_up" not in a and "w_router" not in g and "l1.mlp.up" not in up and "l0.mlp.router" not in up
    assert (plainattn["window"], plainattn["keep_first"], plainattn["rot_dims"], plainattn["rot_factor"]) == (0, 0, 0, 0.0) and "ff" not in plainattn
    bad = dict(t)
    bad["l1.mix.k.norm"] = bad["l1.mix.k.norm"][:-1]
    with pytest.raises(ValueError):
        bovinex.plan(cfg, bad)
    del bad["l1.mix.k.norm"]
    with pytest.raises(KeyError):
        bovinex.plan(cfg, bad)


def test_registry_picks_the_loader_by_config(tmp_path):
    cfg = small_cfg()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    container.write_tensors(str(tmp_path / "model.safetensors"), bovinex.random_tensors(cfg, 2))
    assert registry.architecture_of(str(tmp_path)) == "Bovinex"
    registry._defaults()
    assert registry.SEQ_LOADERS["Bovinex"] is bovinex.load and "Vimulorn" in registry.SEQ_LOADERS
    back, _ = container.read_tensors(str(tmp_path / "model.safetensors"))
    assert set(back) == set(bovinex.tensor_shapes(cfg))


def test_plain_statement_is_causal_and_sees_what_the_mask_says():
    cfg = small_cfg()
    p = {k: v.float().numpy().astype(np.float64) for k, v in bovinex.random_tensors(cfg, 2).items()}
    toks = [int(x) for x in np.random.default_rng(0).integers(0, 50, 20)]
    full = plain.forward(cfg, p, toks)
    assert np.allclose(full[:11], plain.forward(cfg, p, toks[:11]), atol=1e-12)
    seen = [j for j in range(10) if plain.visible(9, j, 4, 2)]
    assert seen == [0, 1, 6, 7, 8, 9] and not plain.visible(3, 4, 4, 2) and plain.visible(3, 0, 4, 0)


def test_rescaled_frequencies():
    f, mag = plain.yarn_frequencies(8, 100.0, None)
    assert mag == 1.0 and np.allclose(f, [1.0, 100 ** -0.25, 0.1, 100 ** -0.75])
    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    g, mag = plain.yarn_frequencies(8, 100.0, sc)
    assert math.isclose(mag, 0.1 * math.log(4.0) + 1.0)
    lo = max(math.floor(8 * math.log(64 / (2 * math.pi * 8.0)) / (2 * math.log(100.0))), 0)
    hi = min(math.ceil(8 * math.log(64 / (2 * math.pi * 1.0)) / (2 * math.log(100.0))), 7)
    assert (lo, hi) == (0, 3)
    assert np.allclose(g, [f[i] * (1 - i / 3) + f[i] / 4 * (i / 3) for i in range(4)])
    v = np.arange(12.0).reshape(1, 1, 12)
    r = plain.rotate(v, np.array([0]), {"dims": 8, "base": 100.0})
    assert np.allclose(r, v)  # position 0 turns nothing
    r = plain.rotate(v, np.array([3]), {"dims": 8, "base": 100.0})
    assert np.allclose(r[..., 8:], v[..., 8:]) and np.allclose(r[0, 0, 0], 0 * math.cos(3.0) - 4 * math.sin(3.0)) and np.allclose(r[0, 0, 4], 4 * math.cos(3.0) + 0 * math.sin(3.0))


def test_router_keeps_the_largest_and_normalises_over_them():
    W = {"router": np.eye(4), "router.b": np.array([0.0, 0.0, 5.0, 0.0])}
    idx, wt = plain.route(np.array([[1.0, 3.0, -4.0, 2.0], [0.0, 0.0, 0.0, 0.0]]), W, 2)
    assert idx.tolist() == [[1, 3], [2, 0]]  # a tie goes to the lower index
    assert np.allclose(wt[0], np.exp([3.0, 2.0]) / np.exp([3.0, 2.0]).sum()) and np.allclose(wt.sum(-1), 1.0)
