"""Vimulorn: a decoder whose config.json lists its layers.  Each layer has one of three token mixers -- latent attention,
a gated delta rule with per-channel decay ("channel_delta"), or windowed attention behind short convolutions with a sink
in the softmax -- Dynamic Tanh norms around every sublayer and a clamped gated feed-forward; a span of layers may be run
several times in a row.  This module is the host side: it reads config.json, names the checkpoint tensors each layer
needs, stacks the input projections of a layer into one matrix (one product per layer input) and binds everything in the
records of seqlib.  The kernels, cache and state live in libcalm_b200_seq.so."""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Tuple

import torch

from . import container, seqlib

ARCHITECTURE = "Vimulorn"
MIXERS = {"latent_attention": seqlib.SEQ_LATENT, "channel_delta": seqlib.SEQ_DELTA, "attention": seqlib.SEQ_WINDOW}


def layer_runs(cfg: dict) -> List[int]:
    """Layer indices in the order they run."""
    n = len(cfg["layers"])
    lp = cfg.get("loop") or {}
    times = int(lp.get("times", 1))
    if times <= 1:
        return list(range(n))
    a, b = int(lp["start"]), int(lp["stop"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def plan(cfg: dict, tensors: Dict[str, torch.Tensor]) -> Tuple[dict, List[dict], Dict[str, torch.Tensor]]:
    """config + checkpoint tensors -> (model head, layer records, tensors to upload)."""
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config")
    width = int(cfg["width"])
    up: Dict[str, torch.Tensor] = {}

    def need(name: str, shape) -> str:
        if name not in tensors:
            raise KeyError(f"checkpoint lacks tensor {name}")
        t = tensors[name]
        if list(t.shape) != list(shape):
            raise ValueError(f"tensor {name} has shape {list(t.shape)}, the config asks for {list(shape)}")
        if t.dtype != torch.bfloat16:
            t = t.to(torch.bfloat16)
        up[name] = t
        return name

    def norm(prefix: str) -> str:
        need(prefix, [width]), need(prefix + ".b", [width]), need(prefix + ".alpha", [])
        return prefix

    def stack(name: str, parts: List[str]) -> str:
        up[name] = torch.cat([up.pop(p) for p in parts], 0).contiguous()
        return name

    layers = []
    for i, lc in enumerate(cfg["layers"]):
        p, mx, kind = f"l{i}.", lc["mixer"], lc["type"]
        if kind not in MIXERS:
            raise ValueError(f"layer {i}: unknown mixer {kind}")
        H, D, Dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
        rec = {"type": MIXERS[kind], "heads": H, "dim": D, "vdim": Dv, "norm1": norm(p + "norm1"), "norm1b": norm(p + "norm1b"), "taps": 1}
        m = p + "mix."
        if kind == "latent_attention":
            Rq, Rk = int(mx["q_rank"]), int(mx["kv_rank"])
            rec.update(q_rank=Rq, kv_rank=Rk, scale=float(mx["scale"]), kv_heads=1)
            rec["w_in"] = stack(m + "in", [need(m + "dq", [Rq, width]), need(m + "dkv", [Rk, width]), need(m + "g", [H, width])])
            rec["dq_norm"], rec["dkv_norm"] = need(m + "dq.norm", [Rq]), need(m + "dkv.norm", [Rk])
            rec["w_uq"], rec["w_uv"] = need(m + "uq", [H * D, Rq]), need(m + "uv", [H * Dv, Rk])
            uk = up.pop(need(m + "uk", [H * D, Rk]))
            up[m + "ukT"] = uk.reshape(H, D, Rk).transpose(1, 2).contiguous()  # per head [kv_rank, dim]: the key side folded into the query
            rec["w_ukT"] = m + "ukT"
        else:
            G, taps = int(mx.get("kv_heads", H)), int(mx.get("conv", 1))
            rec.update(kv_heads=G, taps=taps)
            if kind == "channel_delta":
                cq, cv = G * D, H * Dv
                ra, rg = tensors[m + "a1"].shape[0], tensors[m + "g1"].shape[0]
                rec.update(a_rank=int(ra), g_rank=int(rg))
                rec["w_in"] = stack(m + "in", [need(m + "q", [cq, width]), need(m + "k", [cq, width]), need(m + "v", [cv, width]), need(m + "b", [H, width]),
                                               need(m + "a1", [ra, width]), need(m + "g1", [rg, width])])
                rec["w_a2"], rec["w_g2"] = need(m + "a2", [H * D, ra]), need(m + "g2", [H * Dv, rg])
                rec["a_log"], rec["dt_bias"], rec["out_norm"] = need(m + "A_log", [H]), need(m + "dt_bias", [H * D]), need(m + "norm", [Dv])
                chans = [(m + "q.conv", cq), (m + "k.conv", cq), (m + "v.conv", cv)]
            else:
                cq, ck, cv = H * D, G * D, G * Dv
                mask = mx.get("mask") or {}
                rec.update(scale=float(mx["scale"]), window=int(mask.get("size", 0)))
                rec["w_in"] = stack(m + "in", [need(m + "q", [cq, width]), need(m + "k", [ck, width]), need(m + "v", [cv, width])])
                rec["sink"] = need(m + "sink", [H]) if (m + "sink") in tensors else None
                chans = [(m + "q.conv", cq), (m + "k.conv", ck), (m + "v.conv", cv)]
            if taps > 1:
                rec["conv"] = stack(m + "conv", [need(n, [c, taps]) for n, c in chans])
            else:  # a single tap is a per-channel factor: keep the same kernel
                up[m + "conv"] = torch.cat([tensors[n].to(torch.bfloat16).reshape(c, 1) if n in tensors else torch.ones(c, 1, dtype=torch.bfloat16) for n, c in chans], 0)
                rec["conv"] = m + "conv"
        rec["w_o"] = need(m + "o", [width, H * Dv])
        ml = lc.get("mlp")
        if ml:
            if ml.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: feed-forward kind {ml.get('kind')} is not part of this design")
            ff = int(ml["ff"])
            rec.update(ff=ff, limit=float(ml["limit"]), norm2=norm(p + "norm2"), norm2b=norm(p + "norm2b"))
            rec["w_gate_up"] = stack(p + "mlp.gate_up", [need(p + "mlp.gate", [ff, width]), need(p + "mlp.up", [ff, width])])
            rec["w_down"] = need(p + "mlp.down", [width, ff])
        layers.append(rec)
    lp = cfg.get("loop") or {}
    vocab = int(cfg["vocab"])
    head = {"vocab": vocab, "width": width, "eps": float(cfg["norm"]["eps"]), "loop_start": int(lp.get("start", 0)), "loop_stop": int(lp.get("stop", 0)),
            "loop_times": int(lp.get("times", 1)), "embed": need("embed", [vocab, width]), "head": need("head", [vocab, width]), "final_norm": norm("final.norm")}
    return head, layers, up


def load(folder: str, dtype: str = "bfloat16", max_tokens: int = 4096, max_seqs: int = 64, page: int = 16) -> seqlib.SeqDeviceModel:
    """config.json + model.safetensors of `folder` onto the GPU."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors, _ = container.read_tensors(os.path.join(folder, "model.safetensors"))
    return from_tensors(cfg, tensors, dtype, max_tokens, max_seqs, page)


def from_tensors(cfg: dict, tensors: Dict[str, torch.Tensor], dtype: str = "bfloat16", max_tokens: int = 4096, max_seqs: int = 64, page: int = 16):
    if dtype not in ("bfloat16", "float32"):
        raise ValueError("dtype must be bfloat16 or float32")
    head, layers, up = plan(cfg, tensors)
    return seqlib.SeqDeviceModel(head, layers, up, exact=dtype == "float32", max_tokens=max_tokens, max_seqs=max_seqs, page=page)


# ---------------------------------------------------------------- synthetic checkpoints (tests, bench)

def tensor_shapes(cfg: dict) -> Dict[str, list]:
    W, out = int(cfg["width"]), {}

    def norm(p):
        out[p], out[p + ".b"], out[p + ".alpha"] = [W], [W], []

    out["embed"] = [cfg["vocab"], W]
    for i, lc in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", lc["mixer"]
        H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
        norm(p + "norm1"), norm(p + "norm1b")
        m = p + "mix."
        if lc["type"] == "latent_attention":
            out.update({m + "dq": [mx["q_rank"], W], m + "dq.norm": [mx["q_rank"]], m + "uq": [H * D, mx["q_rank"]], m + "dkv": [mx["kv_rank"], W],
                        m + "dkv.norm": [mx["kv_rank"]], m + "uk": [H * D, mx["kv_rank"]], m + "uv": [H * Dv, mx["kv_rank"]], m + "g": [H, W]})
        elif lc["type"] == "channel_delta":
            G, ra, rg = mx["kv_heads"], mx.get("a_rank", 16), mx.get("g_rank", 16)
            out.update({m + "q": [G * D, W], m + "k": [G * D, W], m + "v": [H * Dv, W], m + "q.conv": [G * D, mx["conv"]], m + "k.conv": [G * D, mx["conv"]],
                        m + "v.conv": [H * Dv, mx["conv"]], m + "b": [H, W], m + "A_log": [H], m + "norm": [Dv], m + "a1": [ra, W], m + "a2": [H * D, ra],
                        m + "dt_bias": [H * D], m + "g1": [rg, W], m + "g2": [H * Dv, rg]})
        else:
            G = mx["kv_heads"]
            out.update({m + "q": [H * D, W], m + "k": [G * D, W], m + "v": [G * Dv, W], m + "q.conv": [H * D, mx["conv"]], m + "k.conv": [G * D, mx["conv"]],
                        m + "v.conv": [G * Dv, mx["conv"]], m + "sink": [H]})
        out[m + "o"] = [W, H * Dv]
        if lc.get("mlp"):
            norm(p + "norm2"), norm(p + "norm2b")
            ff = lc["mlp"]["ff"]
            out.update({p + "mlp.gate": [ff, W], p + "mlp.up": [ff, W], p + "mlp.down": [W, ff]})
    norm("final.norm")
    out["head"] = [cfg["vocab"], W]
    return out


def random_tensors(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Seeded bf16 weights with magnitudes that keep every mechanism active (decays away from 0 and 1, gates open)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf == "alpha":
            t = torch.tensor(0.6 + 0.3 * torch.rand((), generator=g).item())
        elif name.endswith(".b") and len(shape) == 1 and ("norm" in name):
            t = 0.05 * torch.randn(shape, generator=g)
        elif "norm" in leaf or name.endswith(".norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        elif leaf == "A_log":
            t = torch.log(0.5 + 2.0 * torch.rand(shape, generator=g))
        elif leaf in ("dt_bias", "sink"):
            t = torch.randn(shape, generator=g)
        elif leaf == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.5 / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16)
    return out
