"""Ditalorn through the serving engine against the plain numpy oracle (tests/ditalorn_plain.py): whole prompts and every
layer, portions down to two tokens, token-by-token decoding, several live sequences of unequal length, slots and pages
that are freed and used again (a dirty convolution tail, a window's pages given back while the sequence lives), the
first tokens of a sequence, long decoding, other sizes and optional parts, and greedy generation through the engine's
own entry point."""
import numpy as np
import pytest

import ditalorn_fixture as F
import ditalorn_plain as P

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def small(gpu, tmp_path_factory):
    cfg = F.small_config()
    d, W = F.make_model(str(tmp_path_factory.mktemp("dl") / "m"), cfg, seed=11)
    toks = np.random.default_rng(5).integers(0, cfg["vocab"], 150)
    return cfg, d, W, toks, P.forward(cfg, W, toks)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_and_every_layer(gpu, small, dtype):
    cfg, d, W, toks, want = small
    eng = gpu.Engine(d, dtype=dtype, max_tokens=256, page_size=16)
    assert eng.architecture == "Ditalorn"
    eng.capture(True)
    got = eng.step([("a", toks, np.arange(len(toks)))], ["a"])
    assert F.close(got, want, dtype)
    _, layers = P.forward(cfg, W, toks, return_layers=True)
    for i, x in enumerate(layers):
        assert F.close(eng.captured(i, len(toks), cfg["width"]), x, dtype), i
    assert eng.stats()["live_seqs"] == 0 and eng.stats()["free_pages"] == eng.stats()["pages"]
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_and_decoding_equal_the_whole_prompt(gpu, small, dtype):
    cfg, d, W, toks, want = small
    for cuts, page, portion in (([1] * 40, 16, 0), ([2] * 20 + [3, 5, 2, 31, 17, 2, 1, 1, 48], 16, 0), ([150], 8, 7), ([63, 1, 1, 1, 64, 2, 18], 64, 32),
                                ([2, 1, 2, 4, 3, 33, 1, 1, 2, 60], 4, 0), ([64, 64] + [1] * 22, 32, 0)):
        eng = gpu.Engine(d, dtype=dtype, max_tokens=200, page_size=page, max_portion=portion)
        lo, rows = 0, []
        for c in cuts:
            rows.append(eng.step([("s", toks[lo:lo + c], np.arange(c))]))
            lo += c
        got = np.concatenate(rows)
        assert F.close(got, want[:lo], dtype), cuts[:3]
        eng.end("s")
        whole = eng.step([("w", toks[:lo], np.arange(lo))], ["w"])
        assert F.close_enough(got, whole, dtype), cuts[:3]
        eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_several_sequences_reused_slots_and_first_tokens(gpu, small, dtype):
    cfg, d, W, toks, want = small
    r = np.random.default_rng(8)
    seqs = {k: r.integers(0, cfg["vocab"], n) for k, n in (("a", 70), ("b", 9), ("c", 33), ("d", 50), ("e", 1), ("f", 3))}
    alone = {k: P.forward(cfg, W, v) for k, v in seqs.items()}
    eng = gpu.Engine(d, dtype=dtype, max_tokens=140, page_size=8, max_seqs=3)
    got = {k: [] for k in seqs}
    at = {k: 0 for k in seqs}

    def feed(*items, end=()):
        entries = [(k, seqs[k][at[k]:at[k] + n], np.arange(n)) for k, n in items]
        out = eng.step(entries, end)
        lo = 0
        for k, n in items:
            got[k].append(out[lo:lo + n])
            lo += n
            at[k] += n
    feed(("a", 30), ("b", 2))
    feed(("c", 20), ("a", 1), ("b", 5))
    feed(("b", 2), ("a", 2), ("c", 13), end=["b", "c"])   # two slots and their pages come back
    free_mid = eng.stats()["free_pages"]
    feed(("d", 1), ("e", 1), end=["e"])                    # d and e start in slots that b and c used: the convolutions' tails must be clean
    feed(("a", 37), ("d", 2), ("f", 3), end=["a", "f"])
    feed(("d", 47), end=["d"])
    for k in seqs:
        assert at[k] == len(seqs[k]) and F.close(np.concatenate(got[k]), alone[k], dtype), k
    st = eng.stats()
    assert st["live_seqs"] == 0 and st["free_pages"] == st["pages"] and free_mid < st["pages"]
    with pytest.raises(gpu.GgbError):  # a fourth live sequence has no slot
        eng.step([(k, [1], []) for k in "wxyz"])
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_behind_every_window_are_used_again_and_positions_end(gpu, small, dtype):
    cfg, d, W, toks, want = small
    # latent layers only, windows of 11 and 5: two prompts of 150 tokens live together in a cache sized for 150
    cfg2 = F.config([F.latent(), F.latent(heads=2, dim=6, vdim=4, kv_rank=20, q_rank=7, window=5, mlp=None)], positions=160)
    d2, W2 = F.make_model(d + "_windows", cfg2, seed=2)
    other = toks[::-1].copy()
    want2, want_other = P.forward(cfg2, W2, toks), P.forward(cfg2, W2, other)
    eng = gpu.Engine(d2, dtype=dtype, max_tokens=150, page_size=4, max_seqs=2)
    lo, rows, rows_o = 0, [], []
    for c in [9, 1, 1, 7, 16, 2, 2, 1, 16, 13, 1, 1, 1, 16, 3, 16, 16, 12, 2, 14]:
        out = eng.step([("s", toks[lo:lo + c], np.arange(c)), ("o", other[lo:lo + c], np.arange(c))])
        rows.append(out[:c]); rows_o.append(out[c:])
        lo += c
        assert eng.seq_live_pages("s") <= 11 // 4 + 2 and eng.seq_live_pages("o") <= 11 // 4 + 2
    assert lo == 150 and F.close(np.concatenate(rows), want2, dtype) and F.close(np.concatenate(rows_o), want_other, dtype)
    eng.end("s", "o")
    assert eng.stats()["free_pages"] == eng.stats()["pages"]
    eng.close()
    # the learned positions end at max_positions: loudly
    eng = gpu.Engine(d2, dtype=dtype, max_tokens=400, page_size=16)
    eng.step([("s", np.resize(toks, 160), [159])])
    with pytest.raises(gpu.GgbError, match="positions"):
        eng.step([("s", toks[:1], [0])])
    eng.close()
    # an attention layer sees everything: nothing is trimmed and a cache that is too small runs out, loudly
    eng = gpu.Engine(small[1], dtype=dtype, max_tokens=16, page_size=4, max_seqs=2)
    eng.step([("s", toks[:20], [19])])
    assert eng.seq_live_pages("s") == 5
    with pytest.raises(gpu.GgbError, match="out of pages"):
        eng.step([("t", toks[:8], [])])
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(gpu, small, dtype):
    cfg, d, W, _, _ = small
    toks = np.random.default_rng(3).integers(0, cfg["vocab"], 340)
    want = P.forward(cfg, W, toks)
    eng = gpu.Engine(d, dtype=dtype, max_tokens=700, page_size=16)
    rows = [eng.step([("s", toks[:20], np.arange(20))])]
    for p in range(20, 340):
        rows.append(eng.step([("s", toks[p:p + 1], [0])]))
    assert F.close(np.concatenate(rows), want, dtype)
    whole = eng.step([("w", toks, np.arange(340))], ["s", "w"])  # the same numbers from one portion, up to the order of the sums
    assert F.close_enough(np.concatenate(rows), whole, dtype)
    eng.close()


OTHER = {
    "one head, one key head, window 1, eight taps, one expert of one": F.config(
        [F.attention(heads=1, kv_heads=1, dim=4, vdim=4, conv=8, every=1, mlp=F.moe(ff=4, experts=1, top=1, count=1, keep=1)),
         F.latent(heads=1, dim=4, vdim=4, kv_rank=4, q_rank=4, window=1, mlp=F.moe(ff=4, experts=4, top=4, count=4, keep=4))], vocab=7, width=4, scale=1.0),
    "attention only, as many key heads as heads, odd sizes": F.config(
        [F.attention(heads=5, kv_heads=5, dim=7, vdim=3, conv=2, mlp=None), F.attention(heads=2, kv_heads=1, dim=9, vdim=33, conv=5, every=3, mlp=F.moe(experts=9, top=2, count=3, keep=1)),
         F.attention(heads=3, kv_heads=1, dim=4, vdim=6, conv=1, every=0, mlp=None)],
        vocab=31, width=22),
    "latent only, a window longer than the prompt and none": F.config(
        [F.latent(heads=4, dim=6, vdim=5, kv_rank=9, q_rank=17, window=300), F.latent(heads=2, dim=16, vdim=16, kv_rank=40, q_rank=8, window=0, mlp=None)], vocab=40, width=24),
    "tensor-core sizes": F.config(
        [F.latent(heads=4, dim=32, vdim=32, kv_rank=64, q_rank=64, window=70, mlp=F.moe(ff=64, experts=8, top=2, count=4, keep=2)),
         F.attention(heads=4, kv_heads=2, dim=32, vdim=32, conv=4, every=64, mlp=F.moe(ff=32, experts=4, top=3, count=2, keep=2))], vocab=128, width=128, positions=700),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(OTHER))
def test_other_sizes_and_optional_parts(gpu, tmp_path, name, dtype):
    cfg = OTHER[name]
    d, W = F.make_model(str(tmp_path / "m"), cfg, seed=len(name))
    n = 600 if name.startswith("tensor") else 90
    toks = np.random.default_rng(1).integers(0, cfg["vocab"], n)
    want = P.forward(cfg, W, toks)
    eng = gpu.Engine(d, dtype=dtype, max_tokens=n + 40, page_size=16)
    got = eng.step([("a", toks, np.arange(n))], ["a"])
    assert F.close_enough(got, want, dtype, loose=2.0 if name.startswith("one head") else 1.0)
    lo, rows = 0, []
    for c in [n - 60, 2, 2, 1, 1, 33, 1, 1, 1] + [1] * 18:
        rows.append(eng.step([("s", toks[lo:lo + c], np.arange(c))]))
        lo += c
    assert lo == n and F.close_enough(np.concatenate(rows), want, dtype, loose=2.0 if name.startswith("one head") else 1.0)
    eng.close()


def test_a_size_the_configuration_leaves_out_comes_from_the_tensor(gpu, small, tmp_path):
    cfg, d, W, toks, want = small
    import copy
    import json
    import os
    import shutil
    cfg2 = copy.deepcopy(cfg)
    for L in cfg2["layers"]:
        L["mixer"].pop("q_rank", None)
        L["mixer"].pop("vdim", None)
    os.makedirs(tmp_path / "m")
    shutil.copy(os.path.join(d, "model.safetensors"), tmp_path / "m" / "model.safetensors")
    with open(tmp_path / "m" / "config.json", "w") as f:
        json.dump(cfg2, f)
    eng = gpu.Engine(str(tmp_path / "m"), dtype="float32", max_tokens=200, page_size=16)
    assert F.close_enough(eng.step([("a", toks, np.arange(len(toks)))], ["a"]), want, "float32")
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_weight_engines_and_greedy_generation(gpu, small, dtype):
    cfg, d, W, toks, _ = small
    eng = gpu.Engine(d, dtype=dtype, max_tokens=256, page_size=16)
    prompt = toks[:37]
    out = eng.generate("g", prompt, 24)
    # the oracle follows the same tokens; where its two best logits are not close the engine must have picked its first
    seq = np.concatenate([prompt, out])
    logits = P.forward(cfg, W, seq)
    checked = 0
    for i in range(24):
        row = logits[len(prompt) - 1 + i]
        best = np.sort(row)[-2:]
        if best[1] - best[0] > (0.2 if dtype == "bfloat16" else 1e-3):
            assert int(np.argmax(row)) == int(out[i]), i
            checked += 1
    assert checked >= 12 and eng.seq_len("g") == len(prompt) + 23
    eng.close()
    # an engine from a configuration and a seed alone (no file): same logits from any cut, in both ways of stepping
    cfg3 = OTHER["tensor-core sizes"]
    eng = gpu.Engine(config=cfg3, seed=7, dtype=dtype, max_tokens=300, page_size=32)
    t3 = np.random.default_rng(2).integers(0, cfg3["vocab"], 200)
    whole = eng.step([("a", t3, np.arange(200))], ["a"])
    parts = np.concatenate([eng.step([("b", t3[:130], np.arange(130))]), eng.step([("b", t3[130:190], np.arange(60))])] +
                           [eng.step([("b", t3[p:p + 1], [0])]) for p in range(190, 200)])
    assert F.close_enough(parts, whole, dtype) and np.isfinite(whole).all() and whole.std() > 1e-3
    eng.close()
