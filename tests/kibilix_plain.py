"""The Kibilix design in plain numpy float64: one function per mechanism, whole sequences at once, no cache and no state.
It is the oracle of the Kibilix tests and shares no code with the product.

Notation: T tokens, width W, S residual streams; a mixer has H heads over G key heads of size D with values of size Dv.
Matrices are stored [out, in]; `h @ M.T` applies M to every row of h."""
import numpy as np


# ------------------------------------------------------------------------------------------------ small pieces
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_unit(x, eps):
    """x over the root of (its mean square + eps), along the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def softmax(z):
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


# ------------------------------------------------------------------------------------------------ embedding
def embed(tokens, table, bigram, buckets, mul_prev, mul_cur):
    """Row of the token plus the row of the hashed pair (previous token, token); the first token takes the last row."""
    tokens = np.asarray(tokens, dtype=np.int64)
    x = table[tokens].astype(np.float64)
    if bigram is None:
        return x
    rows = np.empty(len(tokens), dtype=np.int64)
    rows[0] = buckets
    rows[1:] = (tokens[:-1] * mul_prev + tokens[1:] * mul_cur) % buckets
    return x + bigram[rows]


# ------------------------------------------------------------------------------------------------ residual streams
def streams_read(xs, w_in):
    """xs [S, T, W] -> the sublayer's input before its norm: sum_s w_in[s] xs[s]."""
    return np.tensordot(w_in, xs, axes=(0, 0))


def streams_write(xs, y, mix, w_out, m):
    """All streams at once from the old ones: new[t] = sum_s mix[s, t] old[s] + m w_out[t] y."""
    return np.einsum("st,snw->tnw", mix, xs) + m * w_out[:, None, None] * y[None]


# ------------------------------------------------------------------------------------------------ rotary positions
def rot_frequencies(rot):
    d = rot["dims"]
    f = rot["base"] ** (-2.0 * np.arange(d // 2) / d)
    sc = rot.get("scaling")
    if not sc:
        return f
    out = f.copy()
    for i, fi in enumerate(f):
        wave = 2.0 * np.pi / fi
        if wave < sc["original"] / sc["high"]:
            continue
        if wave > sc["original"] / sc["low"]:
            out[i] = fi / sc["factor"]
        else:
            s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
            out[i] = (1.0 - s) * fi / sc["factor"] + s * fi
    return out


def rotate_halves(x, positions, rot):
    """x [T, heads, D]: coordinate i < dims / 2 is paired with i + dims / 2; the pair turns by position * f_i."""
    if not rot or not rot.get("dims"):
        return x
    d = rot["dims"]
    ang = np.asarray(positions, dtype=np.float64)[:, None] * rot_frequencies(rot)[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :d // 2], x[..., d // 2:d]
    return np.concatenate([a * c - b * s, b * c + a * s, x[..., d:]], axis=-1)


# ------------------------------------------------------------------------------------------------ attention
def visible(T, chunk, pos0=0):
    """[T, T] bool: query i sees key j <= i of its own chunk (chunks of `chunk` positions counted from position 0)."""
    i = np.arange(pos0, pos0 + T)[:, None]
    j = np.arange(pos0, pos0 + T)[None, :]
    v = j <= i
    if chunk:
        v &= (i // chunk) == (j // chunk)
    return v


def attention_core(q, k, v, scale, softcap, chunk):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] (already rotated) -> [T, H, Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    vis = visible(T, chunk)
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * np.tanh(s / softcap)
        s = np.where(vis, s, -np.inf)
        out[:, h] = softmax(s) @ v[:, g]
    return out


def attention(h, W, p, m):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    pos = np.arange(T)
    q = rotate_halves((h @ W[p + "q"].T).reshape(T, H, D), pos, m.get("rot"))
    k = rotate_halves((h @ W[p + "k"].T).reshape(T, G, D), pos, m.get("rot"))
    v = (h @ W[p + "v"].T).reshape(T, G, Dv)
    o = attention_core(q, k, v, m["scale"], m.get("softcap", 0.0), (m.get("mask") or {}).get("size", 0))
    return o.reshape(T, H * Dv) @ W[p + "o"].T


# ------------------------------------------------------------------------------------------------ delta rule
def causal_conv(x, w):
    """x [T, C], w [C, taps]: y[t] = sum_j w[:, j] x[t - (taps - 1) + j], zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    xx = np.concatenate([np.zeros((taps - 1, C)), x], axis=0)
    return sum(xx[j:j + T] * w[:, j][None, :] for j in range(taps))


def unit(x):
    return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + 1e-6)


def channel_delta_core(q, k, v, beta, g, S0=None):
    """q, k [T, G, D] (unit, q scaled), v [T, H, Dv], beta [T, H], g [T, H, D] -> (o [T, H, Dv], S [H, D, Dv]).
    Per head and token: rows of S decay by g, then the token's value replaces what its key reads, then the read-out."""
    T, H, Dv = v.shape
    G, D = k.shape[1], k.shape[2]
    S = np.zeros((H, D, Dv)) if S0 is None else S0.copy()
    o = np.zeros((T, H, Dv))
    for t in range(T):
        for h in range(H):
            kh, qh = k[t, h // (H // G)], q[t, h // (H // G)]
            S[h] = g[t, h][:, None] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ kh)
            S[h] = S[h] + np.outer(kh, u)
            o[t, h] = S[h].T @ qh
    return o, S


def channel_delta(h, W, p, m, eps):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, Dv)
    q, k = unit(q) * D ** -0.5, unit(k)
    beta = sigmoid(h @ W[p + "b"].T)
    a = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
    g = np.exp(-np.exp(W[p + "A_log"])[None, :, None] * softplus(a).reshape(T, H, D))
    gate = sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).reshape(T, H, Dv)
    o, _ = channel_delta_core(q, k, v, beta, g)
    o = rms_unit(o, eps) * W[p + "norm"][None, None, :] * gate
    return o.reshape(T, H * Dv) @ W[p + "o"].T


# ------------------------------------------------------------------------------------------------ feed-forward
def dense_ff(h, up, down):
    return np.maximum(h @ up.T, 0.0) ** 2 @ down.T


def expert(h, gate, up, down, limit):
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, router, correction, top):
    """-> (chosen experts [T, top], weights [T, top]): soft-max over all experts, the correction only in the choice."""
    s = softmax(h @ router.T)
    order = np.argsort(-(s + correction[None, :]), axis=-1, kind="stable")[:, :top]
    w = np.take_along_axis(s, order, axis=-1)
    return order, w / (w.sum(axis=-1, keepdims=True) + 1e-20)


def moe_ff(h, W, p, f):
    r = f["router"]
    n_real = r["experts"]
    idx, wt = route(h, W[p + "router"], W[p + "correction"], r["top"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wt[t]):
            if e >= n_real:  # an identity expert
                out[t] += w * h[t]
            else:
                q = p + "e%d." % e
                out[t] += w * expert(h[t], W[q + "gate"], W[q + "up"], W[q + "down"], f["expert"]["limit"])
    return out


# ------------------------------------------------------------------------------------------------ the model
def layer_runs(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))


def forward(tokens, W, cfg, layers_out=None):
    """Logits [T, vocab] of a whole sequence; layers_out collects the sum of the streams after every layer run."""
    eps, m, S = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0), cfg.get("streams", 0)
    bg = (cfg.get("embedding") or {}).get("bigram")
    x = embed(tokens, W["embed"], W["bigram"] if bg else None, *((bg["buckets"], bg["mul_prev"], bg["mul_cur"]) if bg else (0, 0, 0)))
    xs = np.stack([x] * max(S, 1))

    def sublayer(xs, p, q, fn):
        if S:
            y = fn(rms_norm(streams_read(xs, W[p + "hc%d.in" % q]), W[p + "norm%d" % q], eps))
            return streams_write(xs, y, W[p + "hc%d.mix" % q], W[p + "hc%d.out" % q], m)
        return xs + m * fn(rms_norm(xs[0], W[p + "norm%d" % q], eps))[None]

    for li in layer_runs(cfg):
        L, p = cfg["layers"][li], "l%d." % li
        if L["type"] == "attention":
            xs = sublayer(xs, p, 1, lambda h: attention(h, W, p + "mix.", L["mixer"]))
        else:
            xs = sublayer(xs, p, 1, lambda h: channel_delta(h, W, p + "mix.", L["mixer"], eps))
        f = L.get("mlp")
        if f:
            if f["kind"] == "dense":
                xs = sublayer(xs, p, 2, lambda h: dense_ff(h, W[p + "mlp.up"], W[p + "mlp.down"]))
            else:
                xs = sublayer(xs, p, 2, lambda h: moe_ff(h, W, p + "mlp.", f))
        if layers_out is not None:
            layers_out.append(xs.sum(axis=0))
    return rms_norm(xs.sum(axis=0), W["final.norm"], eps) @ W["head"].T


# ------------------------------------------------------------------------------------------------ random weights
def random_weights(cfg, seed=0, rank=6):
    """name -> float64 array, sized so that activations stay of order one through the layers."""
    r = np.random.default_rng(seed)
    Wd, V = cfg["width"], cfg["vocab"]
    S = cfg.get("streams", 0)
    W = {"embed": r.standard_normal((V, Wd)), "head": r.standard_normal((V, Wd)) / np.sqrt(Wd), "final.norm": 1.0 + 0.1 * r.standard_normal(Wd)}
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        W["bigram"] = 0.5 * r.standard_normal((bg["buckets"] + 1, Wd))

    def mat(n_out, n_in, gain=1.0):
        return gain * r.standard_normal((n_out, n_in)) / np.sqrt(n_in)

    for li, L in enumerate(cfg["layers"]):
        p, m = "l%d." % li, L["mixer"]
        H, G, D, Dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
        for q in (1, 2) if L.get("mlp") else (1,):
            W[p + "norm%d" % q] = 1.0 + 0.1 * r.standard_normal(Wd)
            if S:
                W[p + "hc%d.in" % q] = 1.0 / S + 0.2 * r.standard_normal(S)
                W[p + "hc%d.out" % q] = 1.0 + 0.3 * r.standard_normal(S)
                W[p + "hc%d.mix" % q] = np.eye(S) + 0.15 * r.standard_normal((S, S))
        if L["type"] == "attention":
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = mat(H * D, Wd, 2.0), mat(G * D, Wd, 2.0), mat(G * Dv, Wd)
        else:
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = mat(G * D, Wd, 2.0), mat(G * D, Wd, 2.0), mat(H * Dv, Wd, 2.0)
            for n, c in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                W[p + "mix.%s.conv" % n] = 0.6 * r.standard_normal((c, m.get("conv", 1)))
            W[p + "mix.b"] = mat(H, Wd, 2.0)
            W[p + "mix.A_log"] = -1.0 + r.standard_normal(H)
            W[p + "mix.dt_bias"] = r.standard_normal(H * D)
            W[p + "mix.norm"] = 1.0 + 0.1 * r.standard_normal(Dv)
            W[p + "mix.a1"], W[p + "mix.a2"] = mat(rank, Wd), mat(H * D, rank, 2.0)
            W[p + "mix.g1"], W[p + "mix.g2"] = mat(rank + 1, Wd), mat(H * Dv, rank + 1, 2.0)
        W[p + "mix.o"] = mat(Wd, H * Dv)
        f = L.get("mlp")
        if f and f["kind"] == "dense":
            W[p + "mlp.up"], W[p + "mlp.down"] = mat(f["ff"], Wd), mat(Wd, f["ff"])
        elif f:
            E, I = f["router"]["experts"], f["router"].get("identity", 0)
            W[p + "mlp.router"] = mat(E + I, Wd, 2.0)
            W[p + "mlp.correction"] = 0.1 * r.standard_normal(E + I)
            for e in range(E):
                q = p + "mlp.e%d." % e
                W[q + "gate"], W[q + "up"], W[q + "down"] = mat(f["expert"]["ff"], Wd, 1.5), mat(f["expert"]["ff"], Wd, 1.5), mat(Wd, f["expert"]["ff"])
    return W
