"""The operators that Kibilix added to the CUDA layer, each alone against the plain float64 functions of
tests/kibilix_plain.py: several residual streams (dense.cu), the chunk mask, the soft cap and the halves layout of the
rotary pairs (window_attention.cu), the delta rule with one decay per key channel (recurrent.cu), the soft-max router
with identity experts and the clamped gate folded into the experts' mat-vec (moe.cu).  Recurrent operators are fed in
portions that continue from the state they left; chunks get one key made to stand out just inside and just outside the
edge, at page borders and at the first positions, in portions and in single-token steps."""
import numpy as np
import pytest

import kibilix_fixture as F
import kibilix_plain as KP

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


def i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


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


# ------------------------------------------------------------------------------------------------ residual streams
@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("S,W", [(1, 40), (2, 33), (3, 40), (4, 256), (5, 12), (8, 64), (11, 20), (16, 7)])
def test_streams_start_renew_read_out_and_rows(gpu, dt, S, W):
    r = np.random.default_rng(S * 100 + W)
    T, eps, m = 9, 1e-5, 0.7
    lib = gpu.cuda_lib()
    x0, y1, y2 = r.standard_normal((T, W)), r.standard_normal((T, W)), r.standard_normal((T, W))
    w_in, w_out, mix, nw = r.standard_normal((3, S)), r.standard_normal((2, S)), r.standard_normal((2, S, S)), 1 + 0.2 * r.standard_normal((3, W))
    xs = zeros(gpu, T * S * W * 4)
    xs.upload(f32(np.full(T * S * W, 77.0)))  # what an earlier portion left: the start ignores it
    h = zeros(gpu, T * W * 4)
    tol = 1e-2 if dt == BF16 else 5e-6

    def call(x0_, y_, k, in_, nw_, rows=None, u=None, n=T):
        coef = dev(gpu, f32(m * w_out[k])) if y_ is not None else None
        gpu.check(lib.ggb_op_hyper_mix(dt, xs.ptr, ptr(dev(gpu, f32(x0_)) if x0_ is not None else None), ptr(dev(gpu, f32(y_)) if y_ is not None else None),
                                       ptr(dev(gpu, f32(mix[k])) if y_ is not None else None), ptr(coef), S, ptr(dev(gpu, f32(in_)) if in_ is not None else None),
                                       ptr(dev(gpu, f32(nw_)) if nw_ is not None else None), eps, W, n, ptr(dev(gpu, i32(rows)) if rows is not None else None),
                                       ptr(u), h.ptr if nw_ is not None else None), "hyper_mix")
    # every stream starts as the embedding row; the first sublayer's input is read out in the same pass
    ref = np.stack([x0] * S)
    call(x0, None, 0, w_in[0], nw[0])
    assert F.rel_err(from_dt(dt, h, (T, W)), KP.rms_norm(KP.streams_read(ref, w_in[0]), nw[0], eps)) < tol
    assert F.rel_err(xs.download(np.float32, T * S * W).reshape(T, S, W).transpose(1, 0, 2), ref) < 1e-6
    # a sublayer's output enters, the next input is read out
    ref = KP.streams_write(ref, y1, mix[0], w_out[0], m)
    call(None, y1, 0, w_in[1], nw[1])
    assert F.rel_err(from_dt(dt, h, (T, W)), KP.rms_norm(KP.streams_read(ref, w_in[1]), nw[1], eps)) < tol
    assert F.rel_err(xs.download(np.float32, T * S * W).reshape(T, S, W).transpose(1, 0, 2), ref) < 2e-6
    # a few rows at the end: the last output enters on the way, nothing is written back, the plain sum comes out too
    last = KP.streams_write(ref, y2, mix[1], w_out[1], m)
    rows = [T - 1, 0, 4]
    u = zeros(gpu, 3 * W * 4)
    call(None, y2, 1, np.ones(S), nw[2], rows=rows, u=u, n=3)
    assert F.rel_err(u.download(np.float32, 3 * W).reshape(3, W), last.sum(0)[rows]) < 2e-6
    assert F.rel_err(from_dt(dt, h, (3, W)), KP.rms_norm(last.sum(0)[rows], nw[2], eps)) < tol
    assert F.rel_err(xs.download(np.float32, T * S * W).reshape(T, S, W).transpose(1, 0, 2), ref) < 2e-6


def test_one_stream_with_unit_weights_is_the_plain_residual_sum(gpu):
    r = np.random.default_rng(3)
    T, W = 5, 24
    x0, y = f32(r.standard_normal((T, W))), f32(r.standard_normal((T, W)))
    xs, one, coef = zeros(gpu, T * W * 4), dev(gpu, f32([1.0])), dev(gpu, f32([0.5]))
    lib = gpu.cuda_lib()
    gpu.check(lib.ggb_op_hyper_mix(F32, xs.ptr, dev(gpu, x0).ptr, dev(gpu, y).ptr, one.ptr, coef.ptr, 1, None, None, 0.0, W, T, None, None, None), "hyper_mix")
    assert np.array_equal(xs.download(np.float32, T * W).reshape(T, W), x0 + np.float32(0.5) * y)


@pytest.mark.parametrize("dt", [F32, BF16])
def test_act_rows_square_of_relu_and_strided_copy(gpu, dt):
    r = np.random.default_rng(1)
    x = f32(r.standard_normal((7, 50)))
    lib = gpu.cuda_lib()
    for act, want in ((1, np.maximum(x[:, 3:40], 0) ** 2), (0, x[:, 3:40])):
        y = zeros(gpu, 7 * 37 * 4)
        gpu.check(lib.ggb_op_act_rows(dt, dev(gpu, x).ptr.value + 12, 50, 7, 37, act, y.ptr), "act_rows")
        assert F.rel_err(from_dt(dt, y, (7, 37)), want) < (5e-3 if dt == BF16 else 1e-7)


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("T,N,K", [(1, 24, 40), (3, 17, 33), (8, 64, 128), (9, 24, 40), (70, 50, 22), (128, 256, 128)])
def test_first_product_of_the_dense_feed_forward_with_its_activation(gpu, dt, T, N, K):
    r = np.random.default_rng(T + N)
    (wv, wu), (av, au) = as_dt(dt, r.standard_normal((N, K)) / np.sqrt(K)), as_dt(dt, r.standard_normal((T, K)))
    y, scratch = zeros(gpu, T * N * 4), zeros(gpu, T * N * 4)
    gpu.check(gpu.cuda_lib().ggb_op_linear_relu2(dt, dev(gpu, wu).ptr, N, K, dev(gpu, au).ptr, K, T, scratch.ptr, y.ptr), "linear_relu2")
    assert F.rel_err(from_dt(dt, y, (T, N)), np.maximum(av @ wv.T, 0) ** 2) < (6e-3 if dt == BF16 else 3e-6)


# ------------------------------------------------------------------------------------------------ chunked attention
def cos_sin(freqs, n):
    a = np.arange(n)[:, None] * np.asarray(freqs)[None, :]
    return f32(np.stack([np.cos(a), np.sin(a)], -1))


def run_chunked(gpu, dt, q, k, v, H, G, chunk, scale, softcap, rot, cuts, page, seed=0, scratch=True):
    """feeds q, k, v rows in portions through masked_qkv_store (halves layout) + masked_attn over shuffled pages; returns [T, H Dv]"""
    T = q.shape[0]
    D, Dv = q.shape[1] // H, v.shape[1] // G
    lib = gpu.cuda_lib()
    ld = int(lib.ggb_window_cache_ld(G, D, Dv))
    n_pages = (T + page - 1) // page + 3
    table = np.random.default_rng(seed).permutation(n_pages).astype(np.int32)
    es = 2 if dt == BF16 else 4
    cache = zeros(gpu, n_pages * page * ld * es)
    tb = dev(gpu, table)
    ck = dev(gpu, cos_sin(KP.rot_frequencies(rot), T + 1)) if rot else None
    rows = f32(np.concatenate([q, k, v], 1))
    ldr = rows.shape[1]
    ws = zeros(gpu, lib.ggb_window_attn_scratch_bytes(H)) if scratch else None
    lo, got = 0, []
    for c in cuts:
        xr, qo, out = dev(gpu, rows[lo:lo + c]), zeros(gpu, c * H * D * 4), zeros(gpu, c * H * Dv * es)
        pos0 = dev(gpu, np.array([lo], dtype=np.int32))
        b = xr.ptr.value
        gpu.check(lib.ggb_op_masked_qkv_store(dt, b, b + 4 * H * D, b + 4 * (H + G) * D, ldr, c, H, G, D, Dv, None, None, 0.0, rot["dims"] if rot else 0, 1, ptr(ck),
                                              None, scale, pos0.ptr, tb.ptr, page, cache.ptr, qo.ptr), "masked_qkv_store")
        gpu.check(lib.ggb_op_masked_attn(dt, qo.ptr, cache.ptr, tb.ptr, page, pos0.ptr, c, H, G, D, Dv, chunk or 0, 1, softcap, None, out.ptr, ptr(ws)), "masked_attn")
        got.append(from_dt(dt, out, (c, H * Dv)))
        lo += c
    assert lo == T
    return np.concatenate(got)


def chunked_want(q, k, v, H, G, chunk, scale, softcap, rot):
    T = q.shape[0]
    D, Dv = q.shape[1] // H, v.shape[1] // G
    pos = np.arange(T)
    qq, kk = KP.rotate_halves(q.reshape(T, H, D), pos, rot), KP.rotate_halves(k.reshape(T, G, D), pos, rot)
    return KP.attention_core(qq, kk, v.reshape(T, G, Dv), scale, softcap, chunk).reshape(T, H * Dv)


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("H,Gk,D,Dv,chunk,page,dims,cap", [(4, 2, 8, 6, 11, 8, 4, 2.0), (3, 3, 16, 16, 64, 16, 16, 0.0), (6, 1, 6, 34, 5, 7, 2, 1.5), (2, 2, 64, 128, 33, 64, 32, 30.0),
                                                          (2, 1, 24, 10, None, 16, 0, 0.7), (1, 1, 10, 4, 1, 4, 10, 0.0)])
def test_chunked_attention_portions_and_single_tokens(gpu, dt, H, Gk, D, Dv, chunk, page, dims, cap):
    G = Gk
    r = np.random.default_rng(H * 100 + D)
    T = 150
    q, k, v = r.standard_normal((T, H * D)), r.standard_normal((T, G * D)), r.standard_normal((T, G * Dv))
    rot = {"dims": dims, "base": 40.0, "scaling": {"factor": 5.0, "low": 1.0, "high": 3.0, "original": 40}} if dims else None
    want = chunked_want(q, k, v, H, G, chunk, 0.4, cap, rot)
    for cuts in ([T], [40] + [1] * 30 + [2, 3, 33, 42], [1] * 20 + [130]):
        got = run_chunked(gpu, dt, q, k, v, H, G, chunk, 0.4, cap, rot, cuts, page, scratch=len(cuts) != 21)
        assert F.rel_err(got, want) < (2e-2 if dt == BF16 else 5e-6), cuts


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("steps", ["portion", "single"])
def test_chunk_edges_page_borders_and_first_positions_with_one_key_standing_out(gpu, dt, steps):
    """Query i points at key j: in i's chunk the head returns j's value, in the chunk before nothing of it.  j walks over the
    first and last place of a chunk, page borders and position 0; chunks are counted from position 0 wherever a portion starts."""
    H, G, D, Dv, page = 2, 1, 8, 6, 16
    T = 200
    r = np.random.default_rng(9)
    for chunk, i, j in ((32, 199, 192), (32, 199, 191), (32, 192, 192), (32, 191, 160), (32, 191, 159), (17, 67, 51), (17, 68, 67), (17, 68, 68), (None, 199, 0),
                        (None, 150, 15), (None, 150, 16), (200, 199, 0), (5, 4, 0), (5, 5, 4), (5, 5, 5), (1, 77, 77), (1, 77, 76), (48, 100, 96), (48, 100, 95)):
        q, k, v = 0.05 * r.standard_normal((T, H * D)), 0.05 * r.standard_normal((T, G * D)), r.standard_normal((T, G * Dv))
        u = r.standard_normal(D); u /= np.linalg.norm(u)
        q[i, :D] = 30.0 * u      # head 0 of token i
        k[j] = 30.0 * u
        want = chunked_want(q, k, v, H, G, chunk, 1.0, 0.0, None)
        visible = j <= i and (chunk is None or i // chunk == j // chunk)
        assert (np.abs(want[i, :Dv] - v[j]).max() < 1e-6) == visible  # the oracle itself tells inside from outside
        cuts = [T] if steps == "portion" else [i - 3] + [1] * (T - i + 3) if i > 3 else [1] * T
        got = run_chunked(gpu, dt, q, k, v, H, G, chunk, 1.0, 0.0, None, cuts, page, seed=i)
        assert np.abs(got[i] - want[i]).max() < (3e-2 if dt == BF16 else 1e-5), (chunk, i, j)
        assert F.rel_err(got, want) < (2e-2 if dt == BF16 else 5e-6), (chunk, i, j)


def test_soft_cap_bounds_a_score_that_would_take_all_the_weight(gpu):
    """Two keys, one with a score of 900: without the cap it takes everything, with cap 2 the weights are e^2 : e^s."""
    H = G = 1
    D, Dv, T = 4, 2, 2
    q, k, v = np.zeros((T, D)), np.zeros((T, D)), np.array([[1.0, 0.0], [0.0, 1.0]])
    q[1] = [30, 0, 0, 0]; k[0] = [30, 0, 0, 0]; k[1] = [0.01, 0, 0, 0]
    capped = run_chunked(gpu, F32, q, k, v, H, G, None, 1.0, 2.0, None, [T], 4)
    plain = run_chunked(gpu, F32, q, k, v, H, G, None, 1.0, 0.0, None, [T], 4)
    s = 2.0 * np.tanh(np.array([900.0, 0.3]) / 2.0)
    w = np.exp(s) / np.exp(s).sum()
    assert np.abs(capped[1] - w).max() < 1e-6 and np.abs(plain[1] - [1.0, 0.0]).max() < 1e-6
    assert F.rel_err(capped, chunked_want(q, k, v, H, G, None, 1.0, 2.0, None)) < 1e-6


def test_halves_layout_differs_from_neighbour_pairs_and_leaves_the_rest(gpu):
    r = np.random.default_rng(4)
    H, G, D, Dv, T = 2, 1, 12, 4, 20
    q, k, v = r.standard_normal((T, H * D)), r.standard_normal((T, G * D)), r.standard_normal((T, G * Dv))
    rot = {"dims": 8, "base": 10.0}
    got = run_chunked(gpu, F32, q, k, v, H, G, None, 0.5, 0.0, rot, [7, 1, 12], 8)
    assert F.rel_err(got, chunked_want(q, k, v, H, G, None, 0.5, 0.0, rot)) < 5e-6
    # the same numbers read as neighbour pairs give another answer: the layout is not a matter of taste
    perm = np.array([0, 4, 1, 5, 2, 6, 3, 7, 8, 9, 10, 11])
    other = chunked_want(q.reshape(T, H, D)[:, :, perm].reshape(T, -1), k.reshape(T, G, D)[:, :, perm].reshape(T, -1), v, H, G, None, 0.5, 0.0, rot)
    assert F.rel_err(got, other) > 1e-2


# ------------------------------------------------------------------------------------------------ delta rule, one decay per channel
def delta_inputs(r, T, H, G, D, Dv):
    q, k, v = r.standard_normal((T, G * D)), r.standard_normal((T, G * D)), r.standard_normal((T, H * Dv))
    b, a = r.standard_normal((T, H)), 2.0 * r.standard_normal((T, H * D))
    return q, k, v, b, a, -1.0 + r.standard_normal(H), r.standard_normal(H * D)


def delta_want(q, k, v, b, a, A_log, dt_bias, H, G, D, Dv):
    T = q.shape[0]
    qq, kk = KP.unit(q.reshape(T, G, D)) * D ** -0.5, KP.unit(k.reshape(T, G, D))
    g = np.exp(-np.exp(A_log)[None, :, None] * KP.softplus(a + dt_bias).reshape(T, H, D))
    return KP.channel_delta_core(qq, kk, v.reshape(T, H, Dv), KP.sigmoid(b), g)


def run_delta(gpu, q, k, v, b, a, A_log, dt_bias, H, G, D, Dv, cuts, ld_extra=3, decays=0):
    lib = gpu.cuda_lib()
    T = q.shape[0]
    rows = f32(np.concatenate([q, k, v, np.zeros((T, ld_extra))], 1))   # a row stride of its own
    ld = rows.shape[1]
    state = zeros(gpu, H * D * Dv * 4)
    Al, db = dev(gpu, f32(A_log)), dev(gpu, f32(dt_bias))
    lo, got = 0, []
    for c in cuts:
        xr, bb, aa, o = dev(gpu, rows[lo:lo + c]), dev(gpu, f32(b[lo:lo + c])), dev(gpu, f32(a[lo:lo + c])), zeros(gpu, c * H * Dv * 4)
        p = xr.ptr.value
        gpu.check(lib.ggb_op_channel_delta(p, p + 4 * G * D, p + 8 * G * D, ld, bb.ptr, H, aa.ptr, H * D, decays, c, H, G, D, Dv, Al.ptr, db.ptr, state.ptr, o.ptr, H * Dv),
                  "channel_delta")
        got.append(o.download(np.float32, c * H * Dv).reshape(c, H, Dv))
        lo += c
    return np.concatenate(got), state.download(np.float32, H * D * Dv).reshape(H, D, Dv)


@pytest.mark.parametrize("H,Gk,D,Dv", [(4, 2, 12, 5), (1, 1, 7, 9), (2, 2, 32, 40), (3, 1, 64, 16), (2, 1, 100, 33), (1, 1, 256, 20), (4, 4, 128, 128)])
def test_channel_delta_in_portions_continues_from_its_state(gpu, H, Gk, D, Dv):
    G = Gk
    r = np.random.default_rng(D * 7 + Dv)
    T = 70
    args = delta_inputs(r, T, H, G, D, Dv)
    want, S = delta_want(*args, H, G, D, Dv)
    for cuts in ([T], [1] * 5 + [2, 3, 16, 17, 27], [33, 1, 1, 35]):
        got, state = run_delta(gpu, *args, H, G, D, Dv, cuts)
        assert F.rel_err(got, want) < 5e-6 and F.rel_err(state, S) < 5e-6, cuts


def test_a_channel_that_forgets_at_once_keeps_nothing_and_its_neighbours_keep_all(gpu):
    """dt_bias makes channel 2 of head 0 decay to nothing every token and every other channel not at all: the state row of
    channel 2 holds the last token's write only; with one decay per head (the other rule) this cannot be told apart."""
    H, G, D, Dv, T = 2, 1, 6, 3, 12
    r = np.random.default_rng(5)
    q, k, v, b, a, A_log, dt_bias = delta_inputs(r, T, H, G, D, Dv)
    a[:] = 0.0
    A_log[:] = 0.0
    dt_bias[:] = -40.0         # softplus -> 0: g = 1
    dt_bias[2] = 40.0          # g = e^-40
    want, S = delta_want(q, k, v, b, a, A_log, dt_bias, H, G, D, Dv)
    got, state = run_delta(gpu, q, k, v, b, a, A_log, dt_bias, H, G, D, Dv, [5, 1, 6])
    assert F.rel_err(got, want) < 5e-6 and F.rel_err(state, S) < 5e-6
    kk = KP.unit(k.reshape(T, G, D))[-1, 0]
    assert np.abs(state[0, 2]).max() <= np.abs(kk[2]) * np.abs(v).max() * 4 and np.abs(state[0, 1]).max() > 0


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("Ka,Kg,H,D,Dv,T", [(6, 7, 4, 12, 5, 5), (24, 24, 4, 64, 64, 37), (64, 64, 2, 128, 128, 1), (9, 130, 3, 7, 9, 16), (8, 16, 5, 40, 52, 17)])
def test_low_rank_pair_gives_the_decays_and_the_gate_rows(gpu, dt, Ka, Kg, H, D, Dv, T):
    r = np.random.default_rng(Ka + T)
    lib = gpu.cuda_lib()
    x = f32(r.standard_normal((T, Ka + Kg + 3)))
    (wav, wau), (wgv, wgu) = as_dt(dt, r.standard_normal((H * D, Ka))), as_dt(dt, r.standard_normal((H * Dv, Kg)) / np.sqrt(Kg))
    A_log, dt_bias = -1.0 + r.standard_normal(H), r.standard_normal(H * D)
    xa, xg = as_dt(dt, x[:, :Ka])[0], as_dt(dt, x[:, Ka:Ka + Kg])[0]
    want_a = np.exp(-np.exp(A_log)[None, :, None] * KP.softplus(xa @ wav.T + dt_bias).reshape(T, H, D)).reshape(T, H * D)
    want_g = xg @ wgv.T
    assert lib.ggb_lowrank_pair_fits(dt, Ka, Kg) == 1 and lib.ggb_lowrank_pair_fits(dt, 4000, Kg) == 0
    a, g = zeros(gpu, T * H * D * 4), zeros(gpu, T * H * Dv * 4)
    gpu.check(lib.ggb_op_lowrank_pair(dt, dev(gpu, x).ptr, x.shape[1], T, dev(gpu, wau).ptr, H * D, Ka, dev(gpu, wgu).ptr, H * Dv, Kg, dev(gpu, f32(A_log)).ptr,
                                      dev(gpu, f32(dt_bias)).ptr, D, a.ptr, g.ptr), "lowrank_pair")
    assert F.rel_err(a.download(np.float32, T * H * D).reshape(T, -1), want_a) < 5e-6
    assert F.rel_err(g.download(np.float32, T * H * Dv).reshape(T, -1), want_g) < 5e-6
    # without the decay's constants both outputs are plain products
    gpu.check(lib.ggb_op_lowrank_pair(dt, dev(gpu, x).ptr, x.shape[1], T, dev(gpu, wau).ptr, H * D, Ka, dev(gpu, wgu).ptr, H * Dv, Kg, None, None, 0, a.ptr, g.ptr),
              "lowrank_pair")
    assert F.rel_err(a.download(np.float32, T * H * D).reshape(T, -1), xa @ wav.T) < 5e-6


def test_the_recurrence_takes_ready_decays_as_well_as_raw_rows(gpu):
    H, G, D, Dv, T = 3, 1, 20, 6, 40
    q, k, v, b, a, A_log, dt_bias = delta_inputs(np.random.default_rng(6), T, H, G, D, Dv)
    want, S = delta_want(q, k, v, b, a, A_log, dt_bias, H, G, D, Dv)
    g = np.exp(-np.exp(A_log)[None, :, None] * KP.softplus(a + dt_bias).reshape(T, H, D)).reshape(T, H * D)
    got, state = run_delta(gpu, q, k, v, b, g, A_log * 0 + 99, dt_bias * 0 + 99, H, G, D, Dv, [7, 1, 32], decays=1)
    assert F.rel_err(got, want) < 5e-6 and F.rel_err(state, S) < 5e-6


# ------------------------------------------------------------------------------------------------ router and identity experts
def run_moe(gpu, dt, h, W, p, f, T, streams=None):
    """router -> groups -> gate | up -> clamped gate -> down -> weighted sum with identity slots, as the model calls them"""
    lib = gpu.cuda_lib()
    r = f["router"]
    E, I, top, FF, lim = r["experts"], r["identity"], r["top"], f["expert"]["ff"], f["expert"]["limit"]
    Wd = h.shape[1]
    es = 2 if dt == BF16 else 4
    hv, hu = as_dt(dt, h)
    gu = np.concatenate([np.concatenate([W[p + "e%d.gate" % e], W[p + "e%d.up" % e]]) for e in range(E)])
    dn = np.concatenate([W[p + "e%d.down" % e] for e in range(E)])
    (guv, guu), (dnv, dnu) = as_dt(dt, gu), as_dt(dt, dn)
    Wq = dict(W)
    for e in range(E):
        Wq[p + "e%d.gate" % e], Wq[p + "e%d.up" % e] = guv[2 * e * FF:(2 * e + 1) * FF], guv[(2 * e + 1) * FF:(2 * e + 2) * FF]
        Wq[p + "e%d.down" % e] = dnv[e * Wd:(e + 1) * Wd]
    hd, gud, dnd = dev(gpu, hu), dev(gpu, guu), dev(gpu, dnu)
    n = T * top
    z, idx, wt = zeros(gpu, T * (E + I) * 4), zeros(gpu, n * 4), zeros(gpu, n * 4)
    ws = zeros(gpu, int(lib.ggb_moe_group_ints(n, E + I)) * 4)
    gu_o, act, y2, out = zeros(gpu, n * 2 * FF * 4), zeros(gpu, n * FF * es), zeros(gpu, n * Wd * 4), zeros(gpu, T * Wd * 4)
    y2.upload(f32(np.full(n * Wd, np.nan)))  # rows of identity slots are never written and never read
    gpu.check(lib.ggb_op_moe_route_softmax(dt, hd.ptr, Wd, T, dev(gpu, f32(W[p + "router"])).ptr, dev(gpu, f32(W[p + "correction"])).ptr, E + I, top, z.ptr, idx.ptr,
                                           wt.ptr, ws.ptr), "route")
    if lib.ggb_moe_step_form(n):
        gpu.check(lib.ggb_op_moe_linear_identity(dt, gud.ptr, FF, Wd, hd.ptr, Wd, 1, T, top, E + I, I, ws.ptr, 3, lim, 1.702, act.ptr, FF), "gate|up")
    else:
        gpu.check(lib.ggb_op_moe_group_identity(idx.ptr, T, top, E + I, I, ws.ptr), "group")
        gpu.check(lib.ggb_op_moe_linear_identity(dt, gud.ptr, 2 * FF, Wd, hd.ptr, Wd, 1, T, top, E + I, I, ws.ptr, 0, 0.0, 0.0, gu_o.ptr, 2 * FF), "gate|up")
        gpu.check(lib.ggb_op_glu_clamp(dt, gu_o.ptr, FF, n, lim, 1.702, act.ptr), "glu")
    gpu.check(lib.ggb_op_moe_linear_identity(dt, dnd.ptr, Wd, FF, act.ptr, FF, 0, T, top, E + I, I, ws.ptr, 0, 0.0, 0.0, y2.ptr, Wd), "down")
    gpu.check(lib.ggb_op_moe_combine_identity(dt, y2.ptr, ws.ptr, wt.ptr, idx.ptr, T, top, E + I, I, Wd, hd.ptr, out.ptr), "combine")
    if streams is not None:  # the weighted sum taken inside the pass over the residual streams instead, h written over the experts' input
        S, xs0, mix, coef, w_in, nw = streams
        xs = dev(gpu, f32(xs0.transpose(1, 0, 2)))
        gpu.check(lib.ggb_op_hyper_mix_moe(dt, xs.ptr, y2.ptr, ws.ptr, wt.ptr, idx.ptr, T, top, E + I, I, hd.ptr, dev(gpu, f32(mix)).ptr, dev(gpu, f32(coef)).ptr, S,
                                           dev(gpu, f32(w_in)).ptr, dev(gpu, f32(nw)).ptr, 1e-5, Wd, T, None, None, hd.ptr), "hyper_mix_moe")
        streams.append(xs.download(np.float32, T * S * Wd).reshape(T, S, Wd).transpose(1, 0, 2))
        streams.append(from_dt(dt, hd, (T, Wd)))
    return (out.download(np.float32, T * Wd).reshape(T, Wd), idx.download(np.int32, n).reshape(T, top), wt.download(np.float32, n).reshape(T, top),
            KP.moe_ff(hv, Wq, p, f), hv)


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("E,I,top,FF,Wd,T", [(5, 2, 3, 9, 40, 4), (5, 2, 3, 9, 40, 70), (1, 0, 1, 5, 22, 3), (2, 3, 5, 7, 22, 40), (3, 1, 2, 16, 33, 1), (8, 1, 2, 64, 128, 300),
                                             (40, 3, 4, 8, 24, 33)])
def test_router_experts_and_identity_experts(gpu, dt, E, I, top, FF, Wd, T):
    r = np.random.default_rng(E * 10 + T)
    f = F.moe(experts=E, identity=I, top=top, ff=FF, limit=0.8)
    cfg = F.config([F.layer("attention", F.attention(), f)], width=Wd, streams=0)
    W = KP.random_weights(cfg, seed=T)
    h = r.standard_normal((T, Wd))
    S = 1 + E % 4
    st = [S, r.standard_normal((S, T, Wd)), np.eye(S) + 0.2 * r.standard_normal((S, S)), r.standard_normal(S), r.standard_normal(S), 1 + 0.1 * r.standard_normal(Wd)]
    got, idx, wt, want, hv = run_moe(gpu, dt, h, W, "l0.mlp.", f, T, streams=st)
    widx, wwt = KP.route(hv, W["l0.mlp.router"].astype(np.float32).astype(np.float64), W["l0.mlp.correction"].astype(np.float32).astype(np.float64), top)
    same = (idx == widx).all(-1)
    assert same.mean() > 0.95  # a close call of two choice scores may fall the other way in fp32
    assert np.abs(wt[same] - wwt[same]).max() < 1e-5 and np.abs(wt.sum(-1) - 1).max() < 1e-5
    assert (idx >= E).any() == (I > 0 and top * T > 8) or I == 0 or top * T <= 8
    assert F.rel_err(got[same], want[same]) < (1.5e-2 if dt == BF16 else 1e-5)
    # the same sum folded into the pass over the streams: the streams renewed from the separate sum, and the next input read out
    new = KP.streams_write(st[1], got.astype(np.float64), st[2], st[3], 1.0)
    assert F.rel_err(st[6], new) < 5e-6
    assert F.rel_err(st[7], KP.rms_norm(KP.streams_read(new, st[4]), st[5], 1e-5)) < (1e-2 if dt == BF16 else 1e-5)


def test_the_correction_changes_the_choice_and_not_the_weights_and_identity_hands_the_input_through(gpu):
    """Router rows make expert 0 the favourite by score; a correction lifts the identity expert over it.  With top 1 the one
    weight is 1 whatever the correction, and the output is the input itself."""
    Wd, T = 16, 3
    f = F.moe(experts=2, identity=1, top=1, ff=4)
    cfg = F.config([F.layer("attention", F.attention(), f)], width=Wd, streams=0)
    W = KP.random_weights(cfg, seed=2)
    h = np.abs(np.random.default_rng(0).standard_normal((T, Wd))) + 0.5
    W["l0.mlp.router"] = np.stack([np.full(Wd, 0.3), np.zeros(Wd), np.full(Wd, 0.1)])
    W["l0.mlp.correction"] = np.zeros(3)
    got, idx, wt, want, hv = run_moe(gpu, F32, h, W, "l0.mlp.", f, T)
    assert (idx == 0).all() and np.abs(wt - 1).max() < 1e-6 and F.rel_err(got, want) < 1e-5
    W["l0.mlp.correction"] = np.array([0.0, 0.0, 5.0])
    got, idx, wt, want, hv = run_moe(gpu, F32, h, W, "l0.mlp.", f, T)
    assert (idx == 2).all() and np.abs(wt - 1).max() < 1e-6 and np.abs(got - h).max() < 1e-6
    # with top 2 the weights are the two scores over their sum: the correction is not in them
    f2 = F.moe(experts=2, identity=1, top=2, ff=4)
    got, idx, wt, want, hv = run_moe(gpu, F32, h, W, "l0.mlp.", f2, T)
    s = KP.softmax(hv @ W["l0.mlp.router"].T)
    assert (idx == [2, 0]).all() and np.abs(wt - s[:, [2, 0]] / s[:, [2, 0]].sum(-1, keepdims=True)).max() < 1e-6
    assert F.rel_err(got, want) < 1e-5


def test_experts_on_the_tensor_cores_skip_the_identity_slots(gpu):
    """600 slots of width 128: the grouped tcgen05 product runs over the experts that have matrices only."""
    E, I, top, FF, Wd, T = 4, 2, 2, 64, 128, 300
    f = F.moe(experts=E, identity=I, top=top, ff=FF, limit=0.9)
    cfg = F.config([F.layer("attention", F.attention(), f)], width=Wd, streams=0)
    W = KP.random_weights(cfg, seed=1)
    h = np.random.default_rng(1).standard_normal((T, Wd))
    got, idx, wt, want, hv = run_moe(gpu, BF16, h, W, "l0.mlp.", f, T)
    assert (idx >= E).any() and np.isfinite(got).all() and F.rel_err(got, want) < 2e-2
