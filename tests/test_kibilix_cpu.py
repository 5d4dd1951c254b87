"""Host-side pieces of the Kibilix path that need no GPU: registry, configuration reader, the order of layer runs and the
refusals, and the plain oracle's own consistency (streams, chunks, rotary bands, the delta rule continued from a state,
identity experts)."""
import ctypes as C
import json

import numpy as np
import pytest

import kibilix_fixture as F
import kibilix_plain as KP


def probe(G, cfg):
    out = (C.c_int64 * 8)()
    rc = G.host_lib().kb_config_probe(json.dumps(cfg).encode(), out)
    return rc, list(out), G.host_lib().gm_last_error().decode()


def test_registry_knows_the_architecture(G):
    assert "Kibilix" in G.architectures() and "Begupel" in G.architectures()


def test_config_reader_takes_every_size_and_the_order_of_runs_from_the_file(G):
    rc, out, _ = probe(G, F.small_config())   # layers 1 and 2 twice: 0 1 2 1 2 3
    assert rc == 0 and out == [4, 6, 3, 3, 1, 57, 40, 3]
    rc, out, _ = probe(G, F.config([F.layer("channel_delta", F.delta())], vocab=7, width=16, streams=0, buckets=0))
    assert rc == 0 and out == [1, 1, 0, 1, 0, 7, 16, 0]
    rc, out, _ = probe(G, F.small_config(loop=(0, 4, 3)))
    assert rc == 0 and out[:4] == [4, 12, 6, 6]
    rc, out, _ = probe(G, F.small_config(loop=(2, 2, 5)))  # an empty block runs nothing, however often
    assert rc == 0 and out[:2] == [4, 4]
    assert KP.layer_runs(F.small_config()) == [0, 1, 2, 1, 2, 3] and KP.layer_runs(F.small_config(loop=(2, 2, 5))) == [0, 1, 2, 3]


@pytest.mark.parametrize("breaker, word", [
    (lambda c: c["layers"][0].update(type="other_mixer"), "unknown mixer"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads must divide"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(high=0.5), "high > low"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=5), "even"),
    (lambda c: c["layers"][1]["mixer"].update(conv=12), "conv"),
    (lambda c: c["layers"][1]["mixer"].update(dim=300), "256"),
    (lambda c: c["layers"][1]["mlp"].update(kind="other"), "unknown mlp"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top at most"),
    (lambda c: c["layers"][1]["mlp"]["expert"].update(limit=0), "limit"),
    (lambda c: c["loop"].update(stop=7), "loop"),
    (lambda c: c.update(streams=40), "streams"),
    (lambda c: c.update(width=0), "positive"),
])
def test_config_reader_refuses_what_the_design_does_not_have(G, breaker, word):
    cfg = F.small_config()
    breaker(cfg)
    rc, _, msg = probe(G, cfg)
    assert rc != 0 and word in msg, msg


def test_one_stream_with_unit_weights_is_the_plain_residual():
    r = np.random.default_rng(0)
    x, y = r.standard_normal((1, 5, 8)), r.standard_normal((5, 8))
    assert np.allclose(KP.streams_write(x, y, np.eye(1), np.ones(1), 0.5)[0], x[0] + 0.5 * y)
    assert np.allclose(KP.streams_read(x, np.ones(1)), x[0])
    # mix is indexed [from, to]: stream 0 copied into stream 1
    xs = r.standard_normal((2, 3, 4))
    out = KP.streams_write(xs, np.zeros((3, 4)), np.array([[1.0, 1.0], [0.0, 0.0]]), np.zeros(2), 1.0)
    assert np.allclose(out[0], xs[0]) and np.allclose(out[1], xs[0])


def test_chunks_are_counted_from_position_zero():
    v = KP.visible(12, 5)
    assert v[4, 0] and not v[5, 4] and v[9, 5] and not v[10, 9] and v[11, 10] and not v[3, 4]
    assert (KP.visible(7, 0) == np.tril(np.ones((7, 7), dtype=bool))).all()
    assert (KP.visible(6, 5, pos0=3)[:, 0] == [True, True, False, False, False, False]).all()  # positions 3..8: the edge is at 5


def test_rotary_bands_keep_blend_and_divide():
    rot = {"dims": 8, "base": 50.0, "scaling": {"factor": 3.0, "low": 1.0, "high": 4.0, "original": 64}}
    f, plain = KP.rot_frequencies(rot), KP.rot_frequencies({"dims": 8, "base": 50.0})
    assert f[0] == plain[0] and np.isclose(f[3], plain[3] / 3.0)
    assert plain[1] / 3.0 < f[1] < plain[1] and plain[2] / 3.0 < f[2] < plain[2]
    # position 0 turns nothing; a turn keeps lengths; the coordinates behind `dims` pass
    x = np.random.default_rng(1).standard_normal((3, 2, 12))
    y = KP.rotate_halves(x, [0, 5, 9], rot)
    assert np.allclose(y[0], x[0]) and np.allclose(y[..., 8:], x[..., 8:])
    assert np.allclose((y[..., :8] ** 2).sum(-1), (x[..., :8] ** 2).sum(-1))
    assert np.allclose(y[1, 0, 0], x[1, 0, 0] * np.cos(5 * f[0]) - x[1, 0, 4] * np.sin(5 * f[0]))


def test_plain_delta_rule_continues_from_its_state_and_a_key_seen_twice_is_replaced():
    r = np.random.default_rng(0)
    T, H, G, D, Dv = 9, 4, 2, 5, 3
    q, k, v = r.standard_normal((T, G, D)), KP.unit(r.standard_normal((T, G, D))), r.standard_normal((T, H, Dv))
    beta, g = r.uniform(0, 1, (T, H)), r.uniform(0.5, 1, (T, H, D))
    o, S = KP.channel_delta_core(q, k, v, beta, g)
    o1, S1 = KP.channel_delta_core(q[:4], k[:4], v[:4], beta[:4], g[:4])
    o2, S2 = KP.channel_delta_core(q[4:], k[4:], v[4:], beta[4:], g[4:], S1)
    assert np.allclose(np.concatenate([o1, o2]), o) and np.allclose(S2, S)
    kk = np.zeros((2, 1, D)); kk[:, 0, 1] = 1.0
    vv = r.standard_normal((2, 1, Dv))
    o, S = KP.channel_delta_core(kk, kk, vv, np.ones((2, 1)), np.ones((2, 1, D)))
    assert np.allclose(o[1, 0], vv[1, 0]) and np.allclose(S[0, 1], vv[1, 0])
    # a channel whose decay is 0 forgets: only the last write is in its row
    g0 = np.ones((2, 1, D)); g0[:, 0, 1] = 0.0
    k2 = KP.unit(np.ones((2, 1, D)))
    o, S = KP.channel_delta_core(k2, k2, vv, np.full((2, 1), 0.5), g0)
    assert np.allclose(S[0, 1], k2[1, 0, 1] * 0.5 * (vv[1, 0] - (g0[1, 0][:, None] * np.outer(k2[0, 0], 0.5 * vv[0, 0])).T @ k2[1, 0]))


def test_convolution_ends_on_the_current_token():
    x = np.arange(1.0, 6.0)[:, None]
    assert np.allclose(KP.causal_conv(x, np.array([[0.0, 0.0, 1.0]])), x)
    assert np.allclose(KP.causal_conv(x, np.array([[1.0, 0.0, 0.0]]))[:, 0], [0, 0, 1, 2, 3])


def test_router_scores_choice_and_identity_experts():
    r = np.random.default_rng(2)
    h = r.standard_normal((6, 10))
    router, corr = r.standard_normal((5, 10)), np.array([0.0, 0.0, 0.0, 0.0, 9.0])
    idx, wt = KP.route(h, router, corr, 2)
    s = KP.softmax(h @ router.T)
    assert (idx[:, 0] == 4).all() and np.allclose(wt.sum(-1), 1.0)
    assert np.allclose(wt[:, 0], s[:, 4] / (s[:, 4] + s[np.arange(6), idx[:, 1]]))
    f = F.moe(experts=4, identity=1, top=1, ff=3)
    W = {"m.router": router, "m.correction": corr}
    assert np.allclose(KP.moe_ff(h, W, "m.", f), h)  # only the identity expert is ever chosen: the input comes back
    # the clamp: a gate far above the limit counts as the limit, an up value far below as its negative
    y = KP.expert(np.array([[1.0]]), np.array([[50.0]]), np.array([[-50.0]]), np.array([[1.0]]), 2.0)
    assert np.allclose(y, 2.0 * KP.sigmoid(1.702 * 2.0) * (-2.0 + 1.0))
