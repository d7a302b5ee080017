"""Host side of the layer-list models without a GPU: the container, the plan that binds a checkpoint to layer records,
the order of layer runs, and the scheduler's batching against a fake model."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import vimulorn_plain as plain  # noqa: E402

from calm_b200 import container, serving, vimulorn  # noqa: E402


def small_cfg():
    return {"architecture": "Vimulorn", "vocab": 50, "width": 16, "norm": {"eps": 1e-5}, "loop": {"start": 1, "stop": 3, "times": 2},
            "layers": [
                {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 4, "conv": 2, "mask": {"size": 5}, "scale": 0.3}, "mlp": None},
                {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "vdim": 4, "kv_rank": 6, "q_rank": 10, "scale": 0.3}, "mlp": {"ff": 12, "kind": "dense", "limit": 2.0}},
                {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 4, "vdim": 8, "conv": 3, "a_rank": 3, "g_rank": 5}, "mlp": {"ff": 12, "kind": "dense", "limit": 2.0}}]}


def test_container_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b.c": torch.arange(7, dtype=torch.int32), "s": torch.tensor(1.5, dtype=torch.bfloat16), "f": torch.randn(2, 2)}
    path = str(tmp_path / "m.safetensors")
    container.write_tensors(path, t, {"k": "v"})
    back, meta = container.read_tensors(path)
    assert meta == {"k": "v"} and set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and back[k].shape == t[k].shape and torch.equal(back[k], t[k])


def test_layer_runs_follow_the_loop():
    cfg = small_cfg()
    assert vimulorn.layer_runs(cfg) == [0, 1, 2, 1, 2] == plain.layer_runs(cfg)[0]
    assert plain.layer_runs(cfg)[1] == [False, False, False, True, False]
    cfg["loop"] = {"start": 0, "stop": 1, "times": 1}
    assert vimulorn.layer_runs(cfg) == [0, 1, 2]


def test_plan_stacks_inputs_in_kernel_order():
    cfg = small_cfg()
    t = vimulorn.random_tensors(cfg, 1)
    head, layers, up = vimulorn.plan(cfg, t)
    assert head["loop_times"] == 2 and len(layers) == 3
    assert torch.equal(up["l0.mix.in"], torch.cat([t["l0.mix.q"], t["l0.mix.k"], t["l0.mix.v"]]))
    assert torch.equal(up["l1.mix.in"], torch.cat([t["l1.mix.dq"], t["l1.mix.dkv"], t["l1.mix.g"]]))
    assert torch.equal(up["l2.mix.in"], torch.cat([t["l2.mix." + n] for n in ("q", "k", "v", "b", "a1", "g1")]))
    assert torch.equal(up["l1.mix.ukT"][1], t["l1.mix.uk"][8:16].T)
    assert layers[2]["a_rank"] == 3 and layers[2]["g_rank"] == 5 and layers[0]["window"] == 5 and layers[0]["ff"] if "ff" in layers[0] else True
    assert up["l2.mix.conv"].shape == (2 * 2 * 4 + 4 * 8, 3)
    bad = dict(t)
    bad["l1.mix.uq"] = bad["l1.mix.uq"][:-1]
    with pytest.raises(ValueError):
        vimulorn.plan(cfg, bad)
    del bad["l1.mix.uq"]
    with pytest.raises(KeyError):
        vimulorn.plan(cfg, bad)


def test_plain_statement_is_causal_and_windowed():
    cfg = small_cfg()
    p = {k: v.float().numpy().astype(np.float64) for k, v in vimulorn.random_tensors(cfg, 2).items()}
    toks = list(np.random.default_rng(0).integers(0, 50, 20))
    full = plain.forward(cfg, p, toks)
    assert np.allclose(full[:11], plain.forward(cfg, p, toks[:11]), atol=1e-12)
    u = np.random.default_rng(1).normal(size=(9, 3))
    w = np.array([[0.0, 0.0, 1.0]] * 3)
    assert np.allclose(plain.short_conv(u, w), u)
    w = np.array([[1.0, 0.0, 0.0]] * 3)
    assert np.allclose(plain.short_conv(u, w)[2:], u[:-2]) and np.all(plain.short_conv(u, w)[:2] == 0)


class FakeModel:
    """Counts pages like the runtime and answers argmax with (last token + 1) % 11."""

    class desc:
        page = 4

    def __init__(self, pages, slots):
        self.pages, self.slots, self.used, self.steps, self.last = pages, slots, {}, [], []

    def free_pages(self):
        return self.pages - sum(-(-n // 4) for n in self.used.values())

    def open(self):
        s = min(set(range(self.slots)) - set(self.used))
        self.used[s] = 0
        return s

    def close_seq(self, s):
        del self.used[s]

    def step(self, slots, toks, want, fetch=True):
        assert len(set(slots)) == len(slots) and all(s in self.used for s in slots)
        for s, t in zip(slots, toks):
            self.used[s] += len(t)
        assert self.free_pages() >= 0
        self.steps.append([len(t) for t in toks])
        self.last = [t[-1] for t in toks]
        return None

    def argmax(self, n):
        return np.array([(x + 1) % 11 for x in self.last[:n]], np.int32)


def test_scheduler_batches_and_returns_pages():
    m = FakeModel(pages=12, slots=3)
    outs = serving.generate(m, [[1, 2, 3], [4], [5, 6, 7, 8, 9, 10, 0], [2, 2]], max_new=5, max_batch=3)
    assert outs[0] == [4, 5, 6, 7, 8] and outs[1] == [5, 6, 7, 8, 9] and outs[3] == [3, 4, 5, 6, 7]
    assert m.steps[0] == [3, 1, 7] and m.steps[1] == [1, 1, 1]          # prompts as one packed step, then one token each
    assert m.steps[5] == [2] and not m.used and m.free_pages() == 12    # the fourth request waited for the next batch
    with pytest.raises(RuntimeError):
        serving.generate(FakeModel(pages=2, slots=2), [[1] * 9], max_new=4)
