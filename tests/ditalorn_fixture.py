"""Model folders for the Ditalorn tests: small configurations of their own, random weights rounded to bfloat16, written
as config.json + model.safetensors."""
import json
import os

import numpy as np

from safolorn_fixture import bf16_round, close_enough, rel_err, write_safetensors  # noqa: F401  (file format helpers)


def close(got, want, dtype):
    """engine against the float64 oracle.  float32: within rounding.  bfloat16: this design adds unnormalised sums over
    every earlier position and norms each sublayer's output, so rounding alone moves a row of logits by about 2 % of
    their scale after five layers and a few hundred positions; a fault of a mechanism moves it by tens of per cent."""
    return close_enough(got, want, dtype, loose=2.0 if dtype == "bfloat16" else 1.0)


def attention(heads=4, kv_heads=2, dim=8, vdim=6, conv=3, scale=0.3, coef=0.4, every=5, mlp="moe"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv:
        m["conv"] = conv
    if every:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": m, "mlp": moe() if mlp == "moe" else mlp}


def latent(heads=3, dim=10, vdim=7, kv_rank=12, q_rank=9, window=11, scale=0.35, mlp="moe"):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": moe() if mlp == "moe" else mlp}


def moe(ff=10, experts=6, top=2, count=3, keep=2):
    r = {"experts": experts, "top": top}
    if count:
        r["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def config(layers, vocab=59, width=40, positions=400, eps=1e-5, scale=3.0):
    return {"architecture": "Ditalorn", "vocab": vocab, "width": width, "max_positions": positions, "norm": {"eps": eps},
            "embedding": {"scale": scale}, "layers": layers}


def small_config(**kw):
    """Both mixers twice in an order of its own; a layer without a feed-forward; grouped and ungrouped routers."""
    return config([latent(), attention(), attention(heads=3, kv_heads=3, dim=5, vdim=9, conv=2, every=0, mlp=None),
                   latent(heads=2, dim=6, vdim=4, kv_rank=20, q_rank=7, window=5, mlp=moe(ff=7, experts=5, top=3, count=0)),
                   attention(heads=6, kv_heads=1, dim=12, vdim=10, conv=0, coef=1.5, every=16, mlp=moe(ff=12, experts=8, top=3, count=4, keep=3))], **kw)


def random_weights(cfg, seed=0):
    """name -> float64 array, sized by the configuration"""
    r = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]
    t = {"embed": r.standard_normal((V, W)) / cfg["embedding"]["scale"], "pos": 0.5 * r.standard_normal((cfg["max_positions"], W)),
         "final.norm": 0.2 * r.standard_normal(W)}

    def lin(n_out, n_in, gain=1.0):
        return gain * r.standard_normal((n_out, n_in)) / np.sqrt(n_in)
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if L.get("mlp") else ()):
            t[p + n] = 0.2 * r.standard_normal(W)
        if L["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                t[p + "mix." + n] = lin(rows, W)
                t[p + "mix." + n + ".b"] = 0.3 * r.standard_normal(rows)
                if m.get("conv"):
                    t[p + "mix." + n + ".conv"] = 0.6 * r.standard_normal((rows, m["conv"]))
            t[p + "mix.r1"] = r.uniform(0.2, 1.0, H)
            t[p + "mix.r2"] = r.uniform(0.1, 1.5, H)
            t[p + "mix.pb"] = r.uniform(-2.5, 0.0, H)
            t[p + "mix.o"] = lin(W, H * Dv)
            t[p + "mix.o.b"] = 0.2 * r.standard_normal(W)
        else:
            H, D, Dv, R, Rq = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            t[p + "mix.dq"] = lin(Rq, W)
            t[p + "mix.dq.norm"] = 1 + 0.2 * r.standard_normal(Rq)
            t[p + "mix.uq"] = lin(H * D, Rq)
            t[p + "mix.dkv"] = lin(R, W)
            t[p + "mix.dkv.norm"] = 1 + 0.2 * r.standard_normal(R)
            t[p + "mix.uk"] = lin(H * D, R)
            t[p + "mix.uv"] = lin(H * Dv, R)
            t[p + "mix.g"] = lin(H, W, 2.0)
            t[p + "mix.o"] = lin(W, H * Dv)
        if L.get("mlp"):
            f = L["mlp"]
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            for e in range(E):
                t[p + "mlp.e%d.gate" % e] = lin(ff, W, 1.5)
                t[p + "mlp.e%d.up" % e] = lin(ff, W, 1.5)
                t[p + "mlp.e%d.down" % e] = lin(W, ff)
            t[p + "mlp.router"] = lin(E, W)
            t[p + "mlp.correction"] = 0.3 * r.standard_normal(E)
    return t


def make_model(tmp, cfg, seed=0, edit=None):
    """Writes the folder; returns (folder, weights as float64 of the bfloat16 values).  edit(W) may change weights before
    they are rounded (tests that make one key stand out)."""
    W = random_weights(cfg, seed)
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
