"""Host-side pieces of the Ditalorn path that need no GPU: registry, configuration reader and its refusals, and the plain
oracle's own consistency (a window as long as the prompt hides nothing, the window's edge with one huge key, the distance
penalty, the convolution's start, the router's groups)."""
import ctypes as C
import json

import numpy as np
import pytest

import ditalorn_fixture as F
import ditalorn_plain as P


def probe(G, cfg):
    out = (C.c_int64 * 8)()
    rc = G.host_lib().dl_config_probe(json.dumps(cfg).encode(), out)
    return rc, list(out), G.host_lib().gm_last_error().decode()


def test_registry_knows_the_architecture(G):
    assert {"Ditalorn", "Begupel", "Safolorn"} <= set(G.architectures())


def test_config_reader_takes_every_size_from_the_file(G):
    rc, out, _ = probe(G, F.small_config())
    assert rc == 0 and out == [5, 3, 2, 4, 59, 40, 400, 0]
    rc, out, _ = probe(G, F.config([F.latent(window=9, mlp=None), F.latent(window=33)], vocab=7, width=16, positions=50))
    assert rc == 0 and out == [2, 0, 2, 1, 7, 16, 50, 33]
    rc, out, _ = probe(G, F.config([F.latent(window=9), F.latent(window=0)]))
    assert rc == 0 and out[7] == 0  # one layer without a window keeps every page


@pytest.mark.parametrize("breaker, word", [
    (lambda c: c["layers"][0].update(type="other_mixer"), "unknown mixer"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads must divide"),
    (lambda c: c["layers"][1]["mixer"].update(conv=12), "conv"),
    (lambda c: c["layers"][1]["mixer"].update(conv=-1), "conv"),
    (lambda c: c["layers"][1]["mixer"]["q_temp"].update(every=0), "q_temp.every"),
    (lambda c: c["layers"][0]["mixer"].update(kv_rank=0), "positive"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unknown mlp"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=1, count=6), "groups"),
    (lambda c: c["layers"][0]["mlp"].pop("router"), "router"),
    (lambda c: c.update(max_positions=0), "max_positions"),
    (lambda c: c.update(width=0), "positive"),
])
def test_config_reader_refuses_what_the_design_does_not_have(G, breaker, word):
    cfg = F.small_config()
    breaker(cfg)
    rc, _, msg = probe(G, cfg)
    assert rc != 0 and word in msg, msg


def test_plain_window_and_its_edge():
    r = np.random.default_rng(0)
    T, H, D, Dv = 40, 2, 6, 5
    q, k, v = r.standard_normal((T, H, D)), r.standard_normal((T, H, D)), r.standard_normal((T, H, Dv))
    assert np.allclose(P.window_softmax_core(q, k, v, 0.4, T), P.window_softmax_core(q, k, v, 0.4, 0))
    assert np.allclose(P.window_softmax_core(q, k, v, 0.4, 1), v)  # a window of one: the token's own value
    u = np.ones(D) / np.sqrt(D)
    for size, i, j, seen in ((8, 30, 23, True), (8, 30, 22, False), (8, 7, 0, True), (8, 8, 0, False)):
        qq, kk = 0.01 * q, 0.01 * k
        qq[i, 0], kk[j, 0] = 40 * u, 40 * u
        o = P.window_softmax_core(qq, kk, v, 1.0, size)
        assert (np.abs(o[i, 0] - v[j, 0]).max() < 1e-6) == seen


def test_plain_sigmoid_attention_penalty_and_causality():
    T, H, D, Dv = 12, 2, 4, 3
    q, k = np.zeros((T, H, D)), np.zeros((T, 1, D))
    v = np.random.default_rng(1).standard_normal((T, 1, Dv))
    r1, r2, pb = np.array([0.7, 0.0]), np.array([2.0, 5.0]), np.array([0.3, -1.0])
    o = P.sigmoid_attention_core(q, k, v, 1.0, r1, r2, pb)
    for i in (0, 5, 11):
        w0 = P.sigmoid(-0.7 * np.log(1 + 2.0 * (i - np.arange(i + 1))) + 0.3)
        assert np.allclose(o[i, 0], w0 @ v[:i + 1, 0])                                 # weights fall with the distance, no normalisation
        assert np.allclose(o[i, 1], P.sigmoid(-1.0) * v[:i + 1, 0].sum(0))               # r1 = 0: every visible key the same weight
    v2 = v.copy(); v2[6:] += 100.0
    assert np.allclose(P.sigmoid_attention_core(q, k, v2, 1.0, r1, r2, pb)[:6], o[:6])   # nothing of a later key
    assert np.allclose(P.q_temperature([0, 3, 4, 8, 9], 0.5, 5), 1 + 0.5 * np.log([1, 1, 2, 2, 3]))


def test_plain_convolution_starts_from_zeros_and_weighs_the_current_token_last():
    u = np.arange(1.0, 7.0)[:, None] * np.ones((1, 2))
    w = np.array([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]])
    y = P.causal_conv(u, w)
    assert np.allclose(y[:, 0], u[:, 0]) and np.allclose(y[:, 1], [0, 0, 1, 2, 3, 4])


def test_plain_router_groups():
    h = np.eye(4)[:1]
    router = np.zeros((6, 4)); router[:, 0] = [2.0, -3.0, 1.0, 1.1, 0.5, 0.4]
    zero = np.zeros(6)
    idx, wt = P.route(h, router, zero, 2, 3, 1)  # groups {0,1} {2,3} {4,5}: the pair (1.0, 1.1) beats (2.0, -3.0)
    assert sorted(idx[0]) == [2, 3] and np.allclose(sorted(wt[0]), P.sigmoid(np.array([1.0, 1.1])))
    idx, _ = P.route(h, router, zero, 2, 3, 3)
    assert sorted(idx[0]) == [0, 3]
    corr = np.array([-5.0, 0, 0, 0, 0, 0])
    idx, wt = P.route(h, router, corr, 2, 3, 3)    # the correction moves the choice, not the weight
    assert sorted(idx[0]) == [2, 3]
    idx, wt = P.route(h, router, -corr, 1, 3, 1)
    assert idx[0, 0] == 0 and np.allclose(wt[0, 0], P.sigmoid(2.0))


def test_plain_forward_runs_and_depends_on_the_past_only():
    cfg = F.small_config()
    W = {k: F.bf16_round(v)[0] for k, v in F.random_weights(cfg, 3).items()}
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 30)
    a = P.forward(cfg, W, toks)
    b = P.forward(cfg, W, toks[:17])
    assert a.shape == (30, cfg["vocab"]) and np.isfinite(a).all() and np.allclose(a[:17], b)
