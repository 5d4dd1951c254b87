"""A plain, slow restatement of the Ditalorn decoder in numpy float64: one function per mechanism, whole sequences, no
cache, no state.  It shares no code with the product; the tests compare the engine with it.

Notation: T tokens, width W, heads H, key/value heads G, query/key size D, value size Dv, latent sizes Rq and R, window
`size`, experts E.  Linear weights are [out, in] and applied as x @ w.T.
"""
import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_plain(x, w, eps):
    return rms_unit(x, eps) * w


def norm_centered(x, w, eps):
    """the layer norms store their weight around zero"""
    return rms_unit(x, eps) * (1.0 + w)


def embed(tokens, table, pos_table, scale, pos0=0):
    tokens = np.asarray(tokens)
    return table[tokens] * scale + pos_table[pos0 + np.arange(len(tokens))]


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start"""
    T, C = u.shape
    taps = w.shape[1]
    pad = np.concatenate([np.zeros((taps - 1, C)), u], axis=0)
    y = np.zeros((T, C))
    for j in range(taps):
        y += pad[j:j + T] * w[:, j]
    return y


def q_temperature(positions, coef, every):
    return 1.0 + coef * np.log(np.floor((np.asarray(positions) + 1) / every) + 1.0)


def sigmoid_attention_core(q, k, v, scale, r1, r2, pb):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv].  Weight of key j for query i (j <= i):
    sigmoid(q.k * scale - r1_h ln(1 + r2_h (i - j)) + pb_h); the weights are not normalised."""
    T, H, D = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    dist = np.arange(T)[:, None] - np.arange(T)[None, :]
    vis = dist >= 0
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * scale
        s = s - r1[h] * np.log1p(r2[h] * np.where(vis, dist, 0)) + pb[h]
        wgt = np.where(vis, sigmoid(s), 0.0)
        out[:, h] = wgt @ v[:, g]
    return out


def attention_mixer(h, w, m, eps, pos0=0):
    """w: dict of the mixer's tensors by their short names; m: the mixer's sizes and constants"""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w["q"].T + w["q.b"]
    k = h @ w["k"].T + w["k.b"]
    v = h @ w["v"].T + w["v.b"]
    if "q.conv" in w:
        q, k, v = causal_conv(q, w["q.conv"]), causal_conv(k, w["k.conv"]), causal_conv(v, w["v.conv"])
    pos = pos0 + np.arange(T)
    if m.get("q_temp"):
        q = q * q_temperature(pos, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None]
    v = rms_unit(v.reshape(T, G, Dv), eps)
    o = sigmoid_attention_core(q.reshape(T, H, D), k.reshape(T, G, D), v, m["scale"], w["r1"], w["r2"], w["pb"])
    return o.reshape(T, H * Dv) @ w["o"].T + w["o.b"]


def window_softmax_core(q, k, v, scale, size):
    """q, k [T, H, D], v [T, H, Dv]: query i sees the keys j with 0 <= i - j < size (size <= 0: every j <= i)"""
    T, H, _ = q.shape
    out = np.zeros((T, H, v.shape[2]))
    dist = np.arange(T)[:, None] - np.arange(T)[None, :]
    vis = (dist >= 0) & ((dist < size) if size > 0 else True)
    for h in range(H):
        s = np.where(vis, q[:, h] @ k[:, h].T * scale, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h] = (p / p.sum(axis=1, keepdims=True)) @ v[:, h]
    return out


def latent_mixer(h, w, m, eps):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    cq = norm_plain(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(T, H, D)
    c = norm_plain(h @ w["dkv"].T, w["dkv.norm"], eps)
    k = (c @ w["uk"].T).reshape(T, H, D)
    v = (c @ w["uv"].T).reshape(T, H, Dv)
    size = (m.get("mask") or {}).get("size", 0)
    o = window_softmax_core(q, k, v, m["scale"], size)
    o = o * sigmoid(h @ w["g"].T)[:, :, None]
    return o.reshape(T, H * Dv) @ w["o"].T


def route(h, router, correction, top, n_groups, keep):
    """-> (chosen [T, top], weights [T, top]).  Scores sigmoid(router h); the choice uses score + correction, inside
    the `keep` groups with the largest sum of their two best choice scores; the weights are the plain scores."""
    s = sigmoid(h @ router.T)
    T, E = s.shape
    choice = s + correction
    gs = E // n_groups
    grouped = choice.reshape(T, n_groups, gs)
    best2 = np.sort(grouped, axis=2)[:, :, -min(2, gs):].sum(axis=2)
    idx = np.zeros((T, top), dtype=np.int64)
    wt = np.zeros((T, top))
    for t in range(T):
        order = sorted(range(n_groups), key=lambda g: (-best2[t, g], g))[:keep]
        allowed = np.full(E, -np.inf)
        for g in order:
            allowed[g * gs:(g + 1) * gs] = choice[t, g * gs:(g + 1) * gs]
        pick = sorted(range(E), key=lambda e: (-allowed[e], e))[:top]
        idx[t] = pick
        wt[t] = s[t, pick]
    return idx, wt


def expert(h, gate, up, down):
    z = h @ gate.T
    return (z * sigmoid(z) * (h @ up.T)) @ down.T


def moe(h, w, f):
    r = f["router"]
    g = r.get("groups") or {"count": 1, "keep": 1}
    idx, wt = route(h, w["router"], w["correction"], r["top"], g["count"], g["keep"])
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, a in zip(idx[t], wt[t]):
            out[t] += a * expert(h[t], w["e%d.gate" % e], w["e%d.up" % e], w["e%d.down" % e])
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, return_layers=False):
    """tensors: name -> float64 array.  Returns the logits [T, vocab] (and the residual stream after every layer)."""
    eps = cfg["norm"]["eps"]
    x = embed(tokens, tensors["embed"], tensors["pos"], cfg["embedding"]["scale"])
    layers = []
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        h = norm_centered(x, tensors[p + "norm1"], eps)
        if L["type"] == "attention":
            y = attention_mixer(h, sub(tensors, p + "mix."), L["mixer"], eps)
        elif L["type"] == "latent_attention":
            y = latent_mixer(h, sub(tensors, p + "mix."), L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + norm_centered(y, tensors[p + "norm1b"], eps)
        if L.get("mlp"):
            h = norm_centered(x, tensors[p + "norm2"], eps)
            x = x + norm_centered(moe(h, sub(tensors, p + "mlp."), L["mlp"]), tensors[p + "norm2b"], eps)
        layers.append(x.copy())
    logits = norm_centered(x, tensors["final.norm"], eps) @ tensors["embed"].T
    return (logits, np.stack(layers)) if return_layers else logits
