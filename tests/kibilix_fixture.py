"""Model folders for the Kibilix tests: small configurations of their own, random weights rounded to bfloat16, written as
config.json + model.safetensors."""
import json
import os

import numpy as np

import kibilix_plain as KP
from safolorn_fixture import bf16_round, close_enough, rel_err, write_safetensors  # noqa: F401  (file format helpers)


def attention(heads=4, kv_heads=2, dim=8, vdim=6, chunk=11, scale=0.3, softcap=4.0, base=50.0, dims=8, scaling=True):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        m["mask"] = {"size": chunk}
    if softcap:
        m["softcap"] = softcap
    if base:
        m["rot"] = {"base": base, "dims": dim if dims is None else dims}
        if scaling:  # with base 50 and 8 dimensions: one frequency kept, two blended, one divided
            m["rot"]["scaling"] = {"factor": 3.0, "low": 1.0, "high": 4.0, "original": 64}
    return m


def delta(heads=4, kv_heads=2, dim=12, vdim=5, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def dense(ff=24):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, identity=2, top=3, ff=9, limit=0.8):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top}}


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(layers, vocab=57, width=40, streams=3, mult=0.7, eps=1e-5, buckets=29, loop=None):
    c = {"architecture": "Kibilix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}
    if streams:
        c["streams"] = streams
    if buckets:
        c["embedding"] = {"bigram": {"buckets": buckets, "mul_prev": 31, "mul_cur": 7}}
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


def small_config(**kw):
    """Both mixers with both kinds of feed-forward and without one; layers 1 and 2 run twice: six layer runs."""
    kw.setdefault("loop", (1, 3, 2))
    return config([layer("attention", attention(), dense()), layer("channel_delta", delta(), moe()),
                   layer("attention", attention(heads=3, kv_heads=3, dim=6, vdim=10, chunk=5, base=0, softcap=0)),
                   layer("channel_delta", delta(heads=2, kv_heads=1, dim=7, vdim=9, conv=2), dense(17))], **kw)


def make_model(tmp, cfg, seed=0, edit=None, rank=6):
    """Writes the folder; returns (folder, weights as float64 of the bfloat16 values)."""
    W = KP.random_weights(cfg, seed, rank)
    if edit:
        edit(W)
    out, vals = {}, {}
    for k, v in W.items():
        vals[k], codes = bf16_round(v)
        out[k] = (codes, np.shape(v))
    os.makedirs(tmp, exist_ok=True)
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(tmp, "model.safetensors"), out, misalign=True)
    return tmp, vals
