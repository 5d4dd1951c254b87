"""The operators that Ditalorn added to the CUDA layer, each alone against the plain float64 functions of
tests/ditalorn_plain.py: learned positions, the norms on both sides of a sublayer, the biased causal convolution, the
grouped sigmoid router, sigmoid attention (store + attention, portions and single tokens, shuffled pages) and the
windowed, gated latent attention.  Where random numbers would hide a fault one key is made to stand out: just inside
and just outside a window, on both sides of a page border, at position 0, hundreds back and at the token itself."""
import numpy as np
import pytest

import ditalorn_fixture as F
import ditalorn_plain as P

pytestmark = pytest.mark.gpu
BF16, F32 = 30, 0
_ALIVE = []


@pytest.fixture(autouse=True)
def _release_buffers():
    yield
    _ALIVE.clear()


def dev(G, a):
    _ALIVE.append(G.DeviceBuffer.from_numpy(np.ascontiguousarray(a)))
    return _ALIVE[-1]


def zeros(G, nbytes):
    b = G.DeviceBuffer(max(int(nbytes), 16))
    b.zero()
    _ALIVE.append(b)
    return b


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def as_dt(dt, a):
    if dt == BF16:
        return F.bf16_round(a)
    a32 = f32(a)
    return a32.astype(np.float64), a32


def from_dt(dt, buf, shape):
    n = int(np.prod(shape))
    if dt == BF16:
        return (buf.download(np.uint16, n).astype(np.uint32) << 16).view(np.float32).reshape(shape).astype(np.float64)
    return buf.download(np.float32, n).reshape(shape).astype(np.float64)


def ptr(b):
    return b.ptr if b is not None else None


# ------------------------------------------------------------------------------------------------ dense.cu
@pytest.mark.parametrize("dt", [F32, BF16])
def test_embedding_with_learned_positions(gpu, dt):
    r = np.random.default_rng(1)
    V, E, n_pos, T, p0 = 23, 37, 50, 9, 17
    tv, tu = as_dt(dt, r.standard_normal((V, E)))
    pv, pu = as_dt(dt, r.standard_normal((n_pos, E)))
    ids = r.integers(0, V, T).astype(np.int32)
    wn = f32(0.3 * r.standard_normal(E))
    y, yn = zeros(gpu, T * E * 4), zeros(gpu, T * E * 4)
    gpu.check(gpu.cuda_lib().ggb_op_embed_pos(dt, dev(gpu, tu).ptr, dev(gpu, pu).ptr, dev(gpu, ids).ptr, dev(gpu, np.array([p0], dtype=np.int32)).ptr,
                                              T, E, 2.5, y.ptr, dev(gpu, f32(1 + wn)).ptr, 1e-3, yn.ptr), "embed_pos")
    want = P.embed(ids, tv, pv, 2.5, p0)
    assert F.rel_err(y.download(np.float32, T * E).reshape(T, E), want) < 1e-6
    assert F.rel_err(from_dt(dt, yn, (T, E)), P.norm_centered(want, wn.astype(np.float64), 1e-3)) < (5e-3 if dt == BF16 else 1e-6)
    gpu.check(gpu.cuda_lib().ggb_op_embed_pos(dt, dev(gpu, tu).ptr, None, dev(gpu, ids).ptr, None, T, E, 1.0, y.ptr, None, 0.0, None), "embed_pos")
    assert F.rel_err(y.download(np.float32, T * E).reshape(T, E), tv[ids]) < 1e-6


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("E", [5, 256, 1100])
def test_norms_on_both_sides_of_a_sublayer(gpu, dt, E):
    r = np.random.default_rng(E)
    T, eps = 7, 1e-4
    a, x, bias = f32(3 * r.standard_normal((T, E))), f32(r.standard_normal((T, E))), f32(r.standard_normal(E))
    wa, wy = f32(0.2 * r.standard_normal(E)), f32(0.2 * r.standard_normal(E))
    es = 2 if dt == BF16 else 4
    for use_bias, use_y in ((True, True), (False, True), (True, False)):
        xd, y = dev(gpu, x), zeros(gpu, T * E * es)
        gpu.check(gpu.cuda_lib().ggb_op_norm_add_norm(dt, dev(gpu, a).ptr, ptr(dev(gpu, bias)) if use_bias else None, dev(gpu, f32(1 + wa)).ptr, eps, E, T, xd.ptr,
                                                      ptr(dev(gpu, f32(1 + wy))) if use_y else None, y.ptr if use_y else None), "norm_add_norm")
        v = a.astype(np.float64) + (bias if use_bias else 0)
        x2 = x + P.norm_centered(v, wa.astype(np.float64), eps)
        assert F.rel_err(xd.download(np.float32, T * E).reshape(T, E), x2) < 1e-6
        if use_y:
            assert F.rel_err(from_dt(dt, y, (T, E)), P.norm_centered(x2, wy.astype(np.float64), eps)) < (5e-3 if dt == BF16 else 1e-6)


# ------------------------------------------------------------------------------------------------ recurrent.cu
@pytest.mark.parametrize("taps", [1, 2, 4, 8])
def test_biased_convolution_continues_over_portions(gpu, taps):
    r = np.random.default_rng(taps)
    T, C, ld = 75, 45, 51
    x, w, b = f32(r.standard_normal((T, ld))), f32(r.standard_normal((C, taps))), f32(r.standard_normal(C))
    want = P.causal_conv(x[:, :C].astype(np.float64) + b, w.astype(np.float64))
    for cuts in ([T], [1] * 10 + [2, 3, 33, 27], [40, 1, 1, 1, 32]):
        tail = zeros(gpu, max(taps - 1, 1) * C * 4)
        lo, got = 0, []
        for c in cuts:
            y = zeros(gpu, c * (C + 2) * 4)
            gpu.check(gpu.cuda_lib().ggb_op_causal_conv_bias(F32, dev(gpu, x[lo:lo + c]).ptr, ld, c, C, dev(gpu, w).ptr, dev(gpu, b).ptr, taps, 0, 0,
                                                             tail.ptr if taps > 1 else None, y.ptr, C + 2, None), "causal_conv_bias")
            got.append(y.download(np.float32, c * (C + 2)).reshape(c, C + 2)[:, :C])
            lo += c
        assert F.rel_err(np.concatenate(got), want) < 1e-6, cuts


# ------------------------------------------------------------------------------------------------ moe.cu
def run_route(gpu, dt, h, router, corr, top, n_groups, keep):
    T, W = h.shape
    E = router.shape[0]
    _, hu = as_dt(dt, h)
    z, idx, wt = zeros(gpu, T * E * 4), zeros(gpu, T * top * 4), zeros(gpu, T * top * 4)
    gpu.check(gpu.cuda_lib().ggb_op_moe_route_sigmoid(dt, dev(gpu, hu).ptr, W, T, dev(gpu, f32(router)).ptr, ptr(dev(gpu, f32(corr))) if corr is not None else None,
                                                      E, top, n_groups, keep, z.ptr, idx.ptr, wt.ptr, None), "route")
    return idx.download(np.int32, T * top).reshape(T, top), wt.download(np.float32, T * top).reshape(T, top)


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("E,top,n_groups,keep", [(12, 4, 3, 2), (6, 2, 1, 1), (8, 8, 4, 4), (40, 5, 8, 3), (7, 1, 7, 1), (9, 3, 3, 1), (64, 6, 4, 2)])
def test_router_sigmoid_groups_and_correction(gpu, dt, E, top, n_groups, keep):
    r = np.random.default_rng(E * 10 + top)
    T, W = 70, 24
    hv, _ = as_dt(dt, r.standard_normal((T, W)))
    router = f32(r.standard_normal((E, W)) * 0.8).astype(np.float64)
    corr = f32(r.standard_normal(E) * 0.6).astype(np.float64)  # large enough to change the choice and to make choice scores negative
    idx, wt = run_route(gpu, dt, hv, router, corr, top, n_groups, keep)
    want_i, want_w = P.route(hv, router, corr, top, n_groups, keep)
    assert (idx == want_i).all()
    assert np.abs(wt - want_w).max() < 1e-6
    plain_i, _ = P.route(hv, router, np.zeros(E), top, n_groups, keep)
    assert (plain_i != want_i).any()  # the correction did matter, and the weights above are the uncorrected scores
    idx, wt = run_route(gpu, dt, hv[:5], router, corr, top, n_groups, keep)  # few tokens: logits and choice in one launch
    assert (idx == want_i[:5]).all() and np.abs(wt - want_w[:5]).max() < 1e-6


def test_router_group_of_negative_scores_beats_an_excluded_one(gpu):
    """every choice score negative: an expert of a group that was dropped must not come back because 'minus infinity'
    was written as zero"""
    E, W = 8, 4
    h = np.array([[1.0, 0, 0, 0]])
    router = np.zeros((E, W)); router[:, 0] = [3, 3, -1, -1, 2, 2, -2, -2]
    corr = np.full(E, -2.0)  # sigmoid < 1: every choice score below -1
    with pytest.raises(gpu.GgbError):  # one group stays and holds 2 experts: 3 cannot be chosen
        run_route(gpu, F32, h, router, corr, 3, 4, 1)
    idx, wt = run_route(gpu, F32, h, router, corr, 2, 4, 1)
    assert sorted(idx[0]) == [0, 1] and np.allclose(wt[0], P.sigmoid(3.0))
    idx, wt = run_route(gpu, F32, h, router, corr, 4, 4, 2)
    assert sorted(idx[0]) == [0, 1, 4, 5]


# ------------------------------------------------------------------------------------------------ sigmoid_attention.cu
def run_sigmoid(gpu, dt, q, k, v, H, G, scale, r1, r2, pb, cuts, page, coef=0.0, every=0, eps=1e-5, seed=0, scratch=True):
    """feeds q, k, v rows in portions through qkv_store + sigmoid_attn over shuffled pages; returns [T, H Dv]"""
    T = q.shape[0]
    D, Dv = q.shape[1] // H, v.shape[1] // G
    lib = gpu.cuda_lib()
    ld = int(lib.ggb_window_cache_ld(G, D, Dv))
    n_pages = (T + page - 1) // page + 3
    table = np.random.default_rng(seed).permutation(n_pages).astype(np.int32)
    es = 2 if dt == BF16 else 4
    cache, tb = zeros(gpu, n_pages * page * ld * es), dev(gpu, table)
    rows = f32(np.concatenate([q, k, v], 1))
    ldr = rows.shape[1]
    ws = zeros(gpu, lib.ggb_sigmoid_attn_scratch_bytes(H)) if scratch else None
    r1d, r2d, pbd = (dev(gpu, f32(a)) if a is not None else None for a in (r1, r2, pb))
    lo, got = 0, []
    for c in cuts:
        xr, qo, out = dev(gpu, rows[lo:lo + c]), zeros(gpu, c * H * D * 4), zeros(gpu, c * H * Dv * es)
        pos0 = dev(gpu, np.array([lo], dtype=np.int32))
        b = xr.ptr.value
        gpu.check(lib.ggb_op_sigmoid_qkv_store(dt, b, b + 4 * H * D, b + 4 * (H + G) * D, ldr, c, H, G, D, Dv, coef, every, eps, scale, pos0.ptr, tb.ptr, page,
                                               cache.ptr, qo.ptr), "sigmoid_qkv_store")
        gpu.check(lib.ggb_op_sigmoid_attn(dt, qo.ptr, cache.ptr, tb.ptr, page, pos0.ptr, c, H, G, D, Dv, 0, ptr(r1d), ptr(r2d), ptr(pbd), out.ptr, ptr(ws)),
                  "sigmoid_attn")
        got.append(from_dt(dt, out, (c, H * Dv)))
        lo += c
    assert lo == T
    return np.concatenate(got)


def sigmoid_want(q, k, v, H, G, scale, r1, r2, pb, coef, every, eps):
    T = q.shape[0]
    D, Dv = q.shape[1] // H, v.shape[1] // G
    if every:
        q = q * P.q_temperature(np.arange(T), coef, every)[:, None]
    z = np.zeros(H)
    o = P.sigmoid_attention_core(q.reshape(T, H, D), k.reshape(T, G, D), P.rms_unit(v.reshape(T, G, Dv), eps), scale,
                                 z if r1 is None else r1, z if r2 is None else r2, z if pb is None else pb)
    return o.reshape(T, H * Dv)


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("H,Gk,D,Dv,page", [(4, 2, 8, 6, 8), (3, 3, 16, 16, 16), (6, 1, 6, 34, 7), (2, 2, 64, 128, 64), (8, 2, 32, 48, 64), (2, 1, 23, 9, 16),
                                           (1, 1, 5, 255, 4)])
def test_sigmoid_attention_portions_and_single_tokens(gpu, dt, H, Gk, D, Dv, page):
    G = Gk
    r = np.random.default_rng(H * 100 + D)
    T = 150
    q, k, v = r.standard_normal((T, H * D)), r.standard_normal((T, G * D)), 3 * r.standard_normal((T, G * Dv))
    r1, r2, pb = r.uniform(0.2, 1.0, H), r.uniform(0.1, 2.0, H), r.uniform(-3, 0, H)
    want = sigmoid_want(q, k, v, H, G, 0.3, r1, r2, pb, 0.7, 11, 1e-5)
    for cuts in ([T], [40] + [1] * 30 + [2, 3, 33, 42], [1] * 20 + [130]):
        got = run_sigmoid(gpu, dt, q, k, v, H, G, 0.3, r1, r2, pb, cuts, page, 0.7, 11, scratch=len(cuts) != 21)
        assert F.rel_err(got, want) < (2e-2 if dt == BF16 else 5e-6), cuts
    if dt == F32:  # without penalty, offset, temperature: the bare mechanism
        got = run_sigmoid(gpu, dt, q, k, v, H, G, 0.3, None, None, None, [64, 1, 85], page)
        assert F.rel_err(got, sigmoid_want(q, k, v, H, G, 0.3, None, None, None, 0, 0, 1e-5)) < 5e-6


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("steps", ["portion", "single"])
def test_sigmoid_attention_one_key_standing_out_far_back_and_at_page_borders(gpu, dt, steps):
    """A large negative offset silences every key but the one the query points at: the head returns that key's unit
    value times its weight, wherever it lies (position 0, hundreds back, either side of a page border, the token itself)
    and nothing of a key one place after the token."""
    H, G, D, Dv, page = 2, 1, 8, 6, 16
    T = 300
    r = np.random.default_rng(9)
    r1, r2, pb = np.array([0.5, 0.5]), np.array([1.0, 1.0]), np.array([-25.0, -25.0])
    for i, j in ((299, 0), (299, 1), (250, 15), (250, 16), (250, 17), (199, 168), (64, 63), (64, 64), (63, 64), (5, 0), (0, 0), (31, 32), (280, 31)):
        q, k, v = 0.05 * r.standard_normal((T, H * D)), 0.05 * r.standard_normal((T, G * D)), r.standard_normal((T, G * Dv))
        u = r.standard_normal(D); u /= np.linalg.norm(u)
        q[i, :D] = 6.0 * u
        k[j] = 6.0 * u
        want = sigmoid_want(q, k, v, H, G, 1.0, r1, r2, pb, 0, 0, 1e-5)
        unit = P.rms_unit(v[j], 1e-5)
        wgt = P.sigmoid(36.0 - 0.5 * np.log1p(float(max(i - j, 0))) - 25.0)
        assert (np.abs(want[i, :Dv] - wgt * unit).max() < 1e-4) == (j <= i)  # the oracle itself tells seen from unseen
        if j > i:
            assert np.abs(want[i]).max() < 1e-6
        cuts = [T] if steps == "portion" else ([i - 3] if i > 3 else []) + [1] * (T - max(i - 3, 0))
        got = run_sigmoid(gpu, dt, q, k, v, H, G, 1.0, r1, r2, pb, cuts, page, seed=i)
        assert np.abs(got[i] - want[i]).max() < (2e-2 if dt == BF16 else 1e-5), (i, j)
        assert np.abs(got - want).max() < (2e-2 if dt == BF16 else 1e-5), (i, j)


# ------------------------------------------------------------------------------------------------ latent_attention.cu
def run_latent(gpu, dt, d, q, wuk, wuv, gate, nw, H, D, Dv, window, scale, cuts, page, n_split, eps=1e-5, seed=0):
    """d [T, R] raw latents, q [T, H D], gate [T, H] raw: kv_store + q_absorb + windowed attention + gated output"""
    T, R = d.shape
    lib = gpu.cuda_lib()
    ld = int(lib.ggb_latent_cache_ld(R, 0))
    n_pages = (T + page - 1) // page + 3
    table = np.random.default_rng(seed).permutation(n_pages).astype(np.int32)
    es = 2 if dt == BF16 else 4
    cache, tb = zeros(gpu, n_pages * page * ld * es), dev(gpu, table)
    _, uk = as_dt(dt, wuk)
    _, uv = as_dt(dt, wuv)
    ukd, uvd, nwd = dev(gpu, uk), dev(gpu, uv), dev(gpu, f32(nw))
    lo, got = 0, []
    for c in cuts:
        pos0 = dev(gpu, np.array([lo], dtype=np.int32))
        qa, out = zeros(gpu, c * H * R * 4), zeros(gpu, c * H * Dv * es)
        part = zeros(gpu, lib.ggb_latent_attn_scratch_bytes(c, H, R, n_split))
        gpu.check(lib.ggb_op_latent_kv_store(dt, dev(gpu, f32(d[lo:lo + c])).ptr, R, c, R, 0, 0, nwd.ptr, eps, None, pos0.ptr, tb.ptr, page, cache.ptr), "kv_store")
        gpu.check(lib.ggb_op_latent_q_absorb(dt, dev(gpu, f32(q[lo:lo + c])).ptr, H * D, c, H, D, 0, 0, None, pos0.ptr, ukd.ptr, R, scale, qa.ptr), "q_absorb")
        gpu.check(lib.ggb_op_latent_attn_window(dt, qa.ptr, cache.ptr, tb.ptr, page, pos0.ptr, c, H, R, 0, window or 0, n_split, part.ptr), "latent_attn_window")
        gpu.check(lib.ggb_op_latent_attn_out_gated(dt, part.ptr, n_split, None, uvd.ptr, c, H, R, Dv, ptr(dev(gpu, f32(gate[lo:lo + c]))) if gate is not None else None,
                                                   H, out.ptr), "latent_attn_out_gated")
        got.append(from_dt(dt, out, (c, H * Dv)))
        lo += c
    assert lo == T
    return np.concatenate(got)


def latent_want(dt, d, q, wuk, wuv, gate, nw, H, D, Dv, window, scale, eps=1e-5):
    T = d.shape[0]
    ukv, _ = as_dt(dt, wuk)
    uvv, _ = as_dt(dt, wuv)
    c, _ = as_dt(dt, P.norm_plain(f32(d).astype(np.float64), f32(nw).astype(np.float64), eps))  # the cache keeps the latent in the storage type
    o = P.window_softmax_core(f32(q).astype(np.float64).reshape(T, H, D), (c @ ukv.T).reshape(T, H, D), (c @ uvv.T).reshape(T, H, Dv), scale, window or 0)
    if gate is not None:
        o = o * P.sigmoid(f32(gate).astype(np.float64))[:, :, None]
    return o.reshape(T, H * Dv)


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("H,D,Dv,R,window,page", [(3, 10, 7, 12, 11, 8), (8, 32, 64, 96, 70, 64), (2, 6, 4, 20, 5, 4), (1, 16, 16, 64, None, 16), (5, 8, 9, 33, 1, 16),
                                                  (19, 4, 3, 136, 40, 16)])
def test_latent_attention_window_gate_portions_and_single_tokens(gpu, dt, H, D, Dv, R, window, page):
    r = np.random.default_rng(H * 100 + R)
    T = 150
    d, q, gate = r.standard_normal((T, R)), r.standard_normal((T, H * D)), 2 * r.standard_normal((T, H))
    wuk, wuv, nw = r.standard_normal((H * D, R)) / np.sqrt(R), r.standard_normal((H * Dv, R)) / np.sqrt(R), 1 + 0.2 * r.standard_normal(R)
    want = latent_want(dt, d, q, wuk, wuv, gate, nw, H, D, Dv, window, 0.5)
    for cuts, ns in (([T], 1), ([T], 3), ([40] + [1] * 30 + [2, 3, 33, 42], 2), ([1] * 20 + [130], 1), ([7, 64, 79], 5)):
        got = run_latent(gpu, dt, d, q, wuk, wuv, gate, nw, H, D, Dv, window, 0.5, cuts, page, ns)
        assert F.rel_err(got, want) < (2e-2 if dt == BF16 else 5e-6), (cuts[:3], ns)
    got = run_latent(gpu, dt, d, q, wuk, wuv, None, nw, H, D, Dv, window, 0.5, [T], page, 2)
    assert F.rel_err(got, latent_want(dt, d, q, wuk, wuv, None, nw, H, D, Dv, window, 0.5)) < (2e-2 if dt == BF16 else 5e-6)


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("steps", ["portion", "single"])
def test_latent_window_edge_with_one_key_standing_out(gpu, dt, steps):
    """Head 0 of token i points at the latent of position j: at the window's last place the head returns j's value, one
    place outside nothing of it; j walks over page and tile borders, the first positions and the token itself."""
    H, D, Dv, R, page = 2, 8, 6, 16, 16
    T = 200
    r = np.random.default_rng(4)
    wuk = np.concatenate([np.eye(D, R), r.standard_normal((D, R)) / 3])  # head 0 reads the latent's first coordinates as they are
    wuv = r.standard_normal((H * Dv, R))
    nw = np.ones(R)
    for window, i, j in ((32, 199, 168), (32, 199, 167), (17, 63, 47), (17, 64, 47), (17, 64, 48), (70, 199, 130), (70, 199, 129), (200, 199, 0), (5, 4, 0),
                         (5, 5, 0), (1, 77, 77), (1, 77, 76), (33, 96, 64), (33, 96, 63), (None, 199, 0)):
        d, q = 0.3 * r.standard_normal((T, R)), 0.05 * r.standard_normal((T, H * D))
        d[:, R - 1] += 4.0               # every latent lies mostly along a coordinate that head 0 does not read ...
        u = np.zeros(R); u[j % D] = 1.0
        d[j] = 50.0 * u                  # ... but this one: sqrt(R) along u after the norm
        q[i, :D] = 12.0 * u[:D]
        want = latent_want(dt, d, q, wuk, wuv, None, nw, H, D, Dv, window, 1.0)
        cj, _ = as_dt(dt, P.norm_plain(f32(d[j]).astype(np.float64), nw, 1e-5))
        vj = (cj @ as_dt(dt, wuv)[0].T)[:Dv]
        visible = j <= i and (window is None or i - j < window)
        assert (np.abs(want[i, :Dv] - vj).max() < 1e-3) == visible
        cuts = [T] if steps == "portion" else ([i - 3] if i > 3 else []) + [1] * (T - max(i - 3, 0))
        got = run_latent(gpu, dt, d, q, wuk, wuv, None, nw, H, D, Dv, window, 1.0, cuts, page, 2 if steps == "portion" else 4, seed=i)
        assert np.abs(got[i] - want[i]).max() < (5e-2 if dt == BF16 else 2e-5), (window, i, j)
        assert F.rel_err(got, want) < (2e-2 if dt == BF16 else 5e-6), (window, i, j)


# ------------------------------------------------------------------------------------------------ experts end to end
@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("T", [1, 3, 8, 40])
def test_experts_in_step_form_and_in_portion_form(gpu, dt, T):
    """router -> slots -> gated experts -> weighted sum -> norms on both sides, as the model chains them: a step of few
    slots (the router lists the slots, gate and up in one mat-vec) and a portion (sorted slots, tiles) give the oracle's sum"""
    lib = gpu.cuda_lib()
    r = np.random.default_rng(T)
    W, E, ff, top, n_groups, keep, eps = 24, 6, 10, 2, 3, 2, 1e-5
    f = {"router": {"experts": E, "top": top, "groups": {"count": n_groups, "keep": keep}}}
    w = {"router": f32(r.standard_normal((E, W)) / 4).astype(np.float64), "correction": f32(0.3 * r.standard_normal(E)).astype(np.float64)}
    gu, dn = [], []
    for e in range(E):
        for n, shape in (("gate", (ff, W)), ("up", (ff, W)), ("down", (W, ff))):
            w["e%d.%s" % (e, n)], _ = as_dt(dt, r.standard_normal(shape) / np.sqrt(shape[1]))
        gu += [w["e%d.gate" % e], w["e%d.up" % e]]
        dn.append(w["e%d.down" % e])
    hv, hu = as_dt(dt, r.standard_normal((T, W)))
    x0, wa, wy = f32(r.standard_normal((T, W))), f32(0.2 * r.standard_normal(W)), f32(0.2 * r.standard_normal(W))
    n, es = T * top, 2 if dt == BF16 else 4
    z, idx, wt = zeros(gpu, T * E * 4), zeros(gpu, n * 4), zeros(gpu, n * 4)
    ws = zeros(gpu, lib.ggb_moe_group_ints(n, E) * 4)
    guw, dnw, hd = dev(gpu, as_dt(dt, np.concatenate(gu))[1]), dev(gpu, as_dt(dt, np.concatenate(dn))[1]), dev(gpu, hu)
    act, y2, x, out = zeros(gpu, n * ff * es), zeros(gpu, n * W * 4), dev(gpu, x0), zeros(gpu, T * W * es)
    gpu.check(lib.ggb_op_moe_route_sigmoid(dt, hd.ptr, W, T, dev(gpu, f32(w["router"])).ptr, dev(gpu, f32(w["correction"])).ptr, E, top, n_groups, keep, z.ptr,
                                           idx.ptr, wt.ptr, ws.ptr), "route")
    if lib.ggb_moe_step_form(n):
        assert n <= 16
        gpu.check(lib.ggb_op_moe_linear(dt, guw.ptr, ff, W, hd.ptr, W, 1, T, top, E, ws.ptr, 2, act.ptr, ff), "gate_up")
    else:
        gbuf = zeros(gpu, n * 2 * ff * 4)
        gpu.check(lib.ggb_op_moe_group(idx.ptr, T, top, E, ws.ptr), "group")
        gpu.check(lib.ggb_op_moe_linear(dt, guw.ptr, 2 * ff, W, hd.ptr, W, 1, T, top, E, ws.ptr, 0, gbuf.ptr, 2 * ff), "gate_up")
        gpu.check(lib.ggb_op_glu_bias(dt, gbuf.ptr, ff, n, None, None, 1, act.ptr), "glu")
    gpu.check(lib.ggb_op_moe_linear(dt, dnw.ptr, W, ff, act.ptr, ff, 0, T, top, E, ws.ptr, 0, y2.ptr, W), "down")
    gpu.check(lib.ggb_op_moe_combine_norm(dt, y2.ptr, ws.ptr, wt.ptr, T, top, E, W, dev(gpu, f32(1 + wa)).ptr, eps, x.ptr, dev(gpu, f32(1 + wy)).ptr, out.ptr), "combine_norm")
    x2 = x0 + P.norm_centered(P.moe(hv, w, f), wa.astype(np.float64), eps)
    tol = 2e-2 if dt == BF16 else 5e-6
    assert F.rel_err(x.download(np.float32, T * W).reshape(T, W), x2) < tol
    assert F.rel_err(from_dt(dt, out, (T, W)), P.norm_centered(x2, wy.astype(np.float64), eps)) < tol


# ------------------------------------------------------------------------------------------------ latent attention, materialised form
def run_latent_materialised(gpu, dt, d, q, wuk, wuv, gate, nw, H, D, Dv, window, scale, cuts, page, eps=1e-5, seed=0):
    """the portion form: kv_store, then per portion the visible latents expanded to keys | values by one product and read by
    the window attention kernel through an identity page table, positions counted from the first visible one"""
    T, R = d.shape
    lib = gpu.cuda_lib()
    ld = int(lib.ggb_latent_cache_ld(R, 0))
    ldkv = int(lib.ggb_window_cache_ld(H, D, Dv))
    n_pages = (T + page - 1) // page + 3
    table = np.random.default_rng(seed).permutation(n_pages).astype(np.int32)
    es = 2 if dt == BF16 else 4
    cache, tb = zeros(gpu, n_pages * page * ld * es), dev(gpu, table)
    ukv = dev(gpu, as_dt(dt, np.concatenate([wuk, wuv]))[1])
    nwd, ident = dev(gpu, f32(nw)), dev(gpu, np.arange(T // page + 2, dtype=np.int32))
    lo, got = 0, []
    for c in cuts:
        first = max(0, lo - window + 1) if window else 0
        n = lo + c - first
        pos0, rel = dev(gpu, np.array([lo], dtype=np.int32)), dev(gpu, np.array([lo - first], dtype=np.int32))
        crows, kvf, kv, out = zeros(gpu, n * R * es), zeros(gpu, n * ldkv * 4), zeros(gpu, n * ldkv * es), zeros(gpu, c * H * Dv * es)
        gpu.check(lib.ggb_op_latent_kv_store(dt, dev(gpu, f32(d[lo:lo + c])).ptr, R, c, R, 0, 0, nwd.ptr, eps, None, pos0.ptr, tb.ptr, page, cache.ptr), "kv_store")
        gpu.check(lib.ggb_op_latent_expand(dt, cache.ptr, tb.ptr, page, first, n, R, 0, ukv.ptr, H * (D + Dv), crows.ptr, kvf.ptr, kv.ptr, ldkv), "expand")
        qs = dev(gpu, f32(q[lo:lo + c] * scale))
        gpu.check(lib.ggb_op_window_attn(dt, qs.ptr, kv.ptr, ident.ptr, page, rel.ptr, c, H, H, D, Dv, window or 0, None, out.ptr, None), "window_attn")
        if gate is not None:
            gpu.check(lib.ggb_op_head_gate(dt, out.ptr, c, H, Dv, dev(gpu, f32(gate[lo:lo + c])).ptr, H), "head_gate")
        got.append(from_dt(dt, out, (c, H * Dv)))
        lo += c
    return np.concatenate(got)


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("H,D,Dv,R,window,page", [(2, 6, 4, 20, 5, 4), (4, 32, 32, 64, 70, 16), (3, 8, 6, 40, None, 16), (1, 4, 2, 9, 1, 8)])
def test_latent_attention_materialised_form_equals_the_oracle(gpu, dt, H, D, Dv, R, window, page):
    r = np.random.default_rng(H * 10 + R)
    T = 150
    d, q, gate = r.standard_normal((T, R)), r.standard_normal((T, H * D)), 2 * r.standard_normal((T, H))
    wuk, wuv, nw = r.standard_normal((H * D, R)) / np.sqrt(R), r.standard_normal((H * Dv, R)) / np.sqrt(R), 1 + 0.2 * r.standard_normal(R)
    want = latent_want(dt, d, q, wuk, wuv, gate, nw, H, D, Dv, window, 0.5)
    for cuts in ([T], [40, 33, 77], [32, 32, 32, 54]):
        got = run_latent_materialised(gpu, dt, d, q, wuk, wuv, gate, nw, H, D, Dv, window, 0.5, cuts, page)
        assert F.rel_err(got, want) < (3e-2 if dt == BF16 else 5e-6), cuts


@pytest.mark.parametrize("dt", [F32, BF16])
def test_latent_materialised_window_edge_with_one_key_standing_out(gpu, dt):
    H, D, Dv, R, page = 2, 8, 6, 16, 16
    T = 200
    r = np.random.default_rng(6)
    wuk = np.concatenate([np.eye(D, R), r.standard_normal((D, R)) / 3])
    wuv, nw = r.standard_normal((H * Dv, R)), np.ones(R)
    for window, i, j in ((32, 199, 168), (32, 199, 167), (17, 64, 48), (17, 64, 47), (70, 199, 130), (70, 199, 129), (200, 199, 0), (33, 96, 64), (33, 96, 63),
                         (None, 199, 0), (40, 130, 100), (40, 140, 100)):
        d, q = 0.3 * r.standard_normal((T, R)), 0.05 * r.standard_normal((T, H * D))
        d[:, R - 1] += 4.0
        u = np.zeros(R); u[j % D] = 1.0
        d[j] = 50.0 * u
        q[i, :D] = 12.0 * u[:D]
        want = latent_want(dt, d, q, wuk, wuv, None, nw, H, D, Dv, window, 1.0)
        for cuts in ([T], [100, 100], [64, 36, 100]):  # the key and the query in one portion, and in two
            got = run_latent_materialised(gpu, dt, d, q, wuk, wuv, None, nw, H, D, Dv, window, 1.0, cuts, page, seed=i)
            assert np.abs(got[i] - want[i]).max() < (5e-2 if dt == BF16 else 2e-5), (window, i, j, cuts)
            assert F.rel_err(got, want) < (3e-2 if dt == BF16 else 5e-6), (window, i, j, cuts)
