"""Bovinex: a decoder whose config.json lists its layers.  Every layer is a parallel block -- one RMS norm (the checkpoint keeps
its weight as the offset from one: applied as 1 + w) whose output feeds both a token mixer and a feed-forward, x <- x + (mixer + feed-forward).
Mixers: grouped-query attention (biased projections, one RMS norm over the whole query / key projection, partial rotation
with frequencies rescaled between two wavelengths, a sliding window that keeps the first tokens, a sigmoid gate per output
channel) and gated linear attention (a decaying [dim x vdim] state per head).  Feed-forward: down(relu(up)^2), or a routed
mixture of SiLU-gated experts.  The embedding is scaled by a constant.

This module is the host side, like vimulorn.py: it reads config.json, checks every tensor's shape, stacks what reads the
same input into one matrix (one product per layer input) and binds everything in the records of seqlib.  The kernels,
cache and state live in libcalm_b200_seq.so; nothing here is specific to one size."""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Tuple

import torch

from . import container, seqlib

ARCHITECTURE = "Bovinex"
MIXERS = {"attention": seqlib.SEQ_GQA, "gla": seqlib.SEQ_GLA}


def plan(cfg: dict, tensors: Dict[str, torch.Tensor]) -> Tuple[dict, List[dict], Dict[str, torch.Tensor]]:
    """config + checkpoint tensors -> (model head, layer records, tensors to upload)."""
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config")
    width, vocab = int(cfg["width"]), int(cfg["vocab"])
    up: Dict[str, torch.Tensor] = {}

    def need(name: str, shape) -> str:
        if name not in tensors:
            raise KeyError(f"checkpoint lacks tensor {name}")
        t = tensors[name]
        if list(t.shape) != list(shape):
            raise ValueError(f"tensor {name} has shape {list(t.shape)}, the config asks for {list(shape)}")
        up[name] = t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)
        return name

    def stack(name: str, parts: List[str]) -> str:
        up[name] = torch.cat([up.pop(p) for p in parts], 0).contiguous()
        return name

    layers = []
    for i, lc in enumerate(cfg["layers"]):
        p, mx, kind = f"l{i}.", lc["mixer"], lc["type"]
        if kind not in MIXERS:
            raise ValueError(f"layer {i}: unknown mixer {kind}")
        H, D, Dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
        rec = {"type": MIXERS[kind], "heads": H, "dim": D, "vdim": Dv, "taps": 1, "norm1": need(p + "norm1", [width])}
        m = p + "mix."
        if kind == "attention":
            G = int(mx.get("kv_heads", H))
            mask, rot = mx.get("mask") or {}, mx.get("rot") or {}
            sc = rot.get("scaling") or {}
            rec.update(kv_heads=G, scale=float(mx["scale"]), window=int(mask.get("size", 0)), keep_first=int(mask.get("keep_first", 0)),
                       rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)), rot_factor=float(sc.get("factor", 0.0)),
                       rot_original=float(sc.get("original", 1.0)), rot_fast=float(sc.get("fast", 1.0)), rot_slow=float(sc.get("slow", 1.0)))
            rows = [("q", H * D), ("k", G * D), ("v", G * Dv), ("g", H * Dv)]
            rec["w_in"] = stack(m + "in", [need(m + n, [r, width]) for n, r in rows])
            # biases of q, k, v in the order of the stacked rows; the gate has none
            up[m + "in.b"] = torch.cat([up.pop(need(m + n + ".b", [r])) for n, r in rows[:3]] + [torch.zeros(H * Dv, dtype=torch.bfloat16)], 0)
            rec["b_in"] = m + "in.b"
            rec["q_norm"], rec["k_norm"] = need(m + "q.norm", [H * D]), need(m + "k.norm", [G * D])
        else:
            ra = int(tensors[m + "a1"].shape[0]) if (m + "a1") in tensors else 0
            rec.update(kv_heads=H, a_rank=ra, tau=float(mx["tau"]))
            rec["w_in"] = stack(m + "in", [need(m + "q", [H * D, width]), need(m + "k", [H * D, width]), need(m + "v", [H * Dv, width]),
                                           need(m + "g", [H * Dv, width]), need(m + "a1", [ra, width])])
            rec["w_a2"], rec["b_a2"], rec["out_norm"] = need(m + "a2", [H * D, ra]), need(m + "a2.b", [H * D]), need(m + "norm", [Dv])
        rec["w_o"] = need(m + "o", [width, H * Dv])
        ml = lc.get("mlp")
        if ml:
            # the block is parallel: what the feed-forward multiplies the normed input with first -- a dense unit's up rows, a
            # router's rows -- rides at the end of the mixer's stacked input matrix (in_tail rows), one product for all of it
            f = p + "mlp."
            n_in = up[rec["w_in"]].shape[0]
            bias = up.pop(rec["b_in"]) if rec.get("b_in") else torch.zeros(n_in, dtype=torch.bfloat16)
            if ml["kind"] == "dense":
                ff = int(ml["ff"])
                tail, tail_b = up.pop(need(f + "up", [ff, width])), torch.zeros(ff, dtype=torch.bfloat16)
                rec.update(ff=ff, ff_kind=seqlib.FF_RELU2, in_tail=ff, w_down=need(f + "down", [width, ff]))
            elif ml["kind"] == "moe":
                ff, E, top = int(ml["expert"]["ff"]), int(ml["router"]["experts"]), int(ml["router"]["top"])
                tail, tail_b = up.pop(need(f + "router", [E, width])), up.pop(need(f + "router.b", [E]))
                rec.update(ff=ff, ff_kind=seqlib.FF_MOE, experts=E, top=top, in_tail=E)
                # experts side by side: [experts][gate | up] and [experts][down], so that one grouped product serves all of them
                rec["w_gate_up"] = stack(f + "gate_up", [x for e in range(E) for x in (need(f + f"e{e}.gate", [ff, width]), need(f + f"e{e}.up", [ff, width]))])
                rec["w_down"] = stack(f + "downs", [need(f + f"e{e}.down", [width, ff]) for e in range(E)])
            else:
                raise ValueError(f"layer {i}: feed-forward kind {ml['kind']} is not part of this design")
            up[rec["w_in"]] = torch.cat([up[rec["w_in"]], tail], 0).contiguous()
            up[m + "in.b"] = torch.cat([bias, tail_b], 0)
            rec["b_in"] = m + "in.b"
        layers.append(rec)
    head = {"vocab": vocab, "width": width, "eps": float(cfg["norm"]["eps"]), "embed": need("embed", [vocab, width]), "head": need("head", [vocab, width]),
            "final_norm": need("final.norm", [width]), "norm_kind": seqlib.NORM_RMS, "norm_offset": 1.0, "block": seqlib.BLOCK_PARALLEL,
            "embed_scale": float((cfg.get("embedding") or {}).get("scale", 1.0))}
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
    out["embed"] = [cfg["vocab"], W]
    for i, lc in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", lc["mixer"]
        H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
        out[p + "norm1"] = [W]
        m = p + "mix."
        if lc["type"] == "attention":
            G = mx.get("kv_heads", H)
            out.update({m + "q": [H * D, W], m + "q.b": [H * D], m + "k": [G * D, W], m + "k.b": [G * D], m + "v": [G * Dv, W], m + "v.b": [G * Dv],
                        m + "q.norm": [H * D], m + "k.norm": [G * D], m + "g": [H * Dv, W]})
        else:
            ra = mx.get("a_rank", 16)
            out.update({m + "q": [H * D, W], m + "k": [H * D, W], m + "v": [H * Dv, W], m + "g": [H * Dv, W], m + "norm": [Dv], m + "a1": [ra, W],
                        m + "a2": [H * D, ra], m + "a2.b": [H * D]})
        out[m + "o"] = [W, H * Dv]
        ml = lc.get("mlp")
        if ml and ml["kind"] == "dense":
            out.update({p + "mlp.up": [ml["ff"], W], p + "mlp.down": [W, ml["ff"]]})
        elif ml:
            ff = ml["expert"]["ff"]
            for e in range(ml["router"]["experts"]):
                out.update({p + f"mlp.e{e}.gate": [ff, W], p + f"mlp.e{e}.up": [ff, W], p + f"mlp.e{e}.down": [W, ff]})
            out.update({p + "mlp.router": [ml["router"]["experts"], W], p + "mlp.router.b": [ml["router"]["experts"]]})
    out["final.norm"] = [W]
    out["head"] = [cfg["vocab"], W]
    return out


def random_tensors(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Seeded bf16 weights with magnitudes that keep every mechanism active (decays away from 0 and 1, gates open, router
    choices spread over the experts)."""
    g = torch.Generator().manual_seed(seed)
    scale = float((cfg.get("embedding") or {}).get("scale", 1.0))
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name.endswith("q.norm") or name.endswith("k.norm") or name.endswith("mix.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf in ("norm1", "norm"):  # the layer norms and final.norm: offsets from one
            t = 0.2 * torch.randn(shape, generator=g)
        elif name.endswith("a2.b"):
            t = 1.5 + 1.5 * torch.randn(shape, generator=g)
        elif name.endswith("router.b"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif leaf == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif leaf == "embed":
            t = torch.randn(shape, generator=g) / scale
        elif leaf == "router":
            t = torch.randn(shape, generator=g) * (3.0 / math.sqrt(shape[-1]))
        else:
            t = torch.randn(shape, generator=g) * (1.2 / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16)
    return out
