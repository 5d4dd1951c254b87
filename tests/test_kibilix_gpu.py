"""Kibilix through the serving engine against the plain numpy oracle (tests/kibilix_plain.py): whole prompts and every
layer run, portions down to two tokens, token-by-token decoding, several live sequences of unequal length, slots and
pages that are freed and used again (also by the same sequence, behind its chunks), the first tokens of a sequence, long
decoding, other sizes and optional parts, and greedy generation through the engine's own entry point."""
import numpy as np
import pytest

import kibilix_fixture as F
import kibilix_plain as KP

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def small(gpu, tmp_path_factory):
    cfg = F.small_config()
    d, W = F.make_model(str(tmp_path_factory.mktemp("kb") / "m"), cfg, seed=11)
    toks = np.random.default_rng(5).integers(0, cfg["vocab"], 150)
    return cfg, d, W, toks, KP.forward(toks, W, cfg)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_and_every_layer_run(gpu, small, dtype):
    cfg, d, W, toks, want = small
    eng = gpu.Engine(d, dtype=dtype, max_tokens=256, page_size=16)
    assert eng.architecture == "Kibilix"
    eng.capture(True)
    got = eng.step([("a", toks, np.arange(len(toks)))], ["a"])
    assert F.close_enough(got, want, dtype)
    runs = []
    KP.forward(toks, W, cfg, runs)
    assert len(runs) == 6
    for i, x in enumerate(runs):
        assert F.close_enough(eng.captured(i, len(toks), cfg["width"]), x, dtype), i
    assert eng.stats()["live_seqs"] == 0 and eng.stats()["free_pages"] == eng.stats()["pages"]
    eng.capture(False)  # the same numbers when nothing is captured (a sublayer's output then enters on the next pass)
    again = eng.step([("b", toks, np.arange(len(toks)))], ["b"])
    assert F.close_enough(again, got, dtype) and np.abs(again - got).max() < 1e-3
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_and_decoding_equal_the_whole_prompt(gpu, small, dtype):
    cfg, d, W, toks, want = small
    for cuts, page, portion in (([1] * 40, 16, 0), ([2] * 20 + [3, 5, 2, 31, 17, 2, 1, 1, 48], 16, 0), ([150], 8, 7), ([63, 1, 1, 1, 64, 2, 18], 64, 32),
                                ([2, 1, 2, 4, 3, 33, 1, 1, 2, 60], 4, 0), ([10, 1, 11, 11, 1, 10, 5, 6, 22], 2, 0)):
        eng = gpu.Engine(d, dtype=dtype, max_tokens=200, page_size=page, max_portion=portion)
        lo, rows = 0, []
        for c in cuts:
            rows.append(eng.step([("s", toks[lo:lo + c], np.arange(c))]))
            lo += c
        got = np.concatenate(rows)
        assert F.close_enough(got, want[:lo], dtype), cuts[:3]
        eng.end("s")
        whole = eng.step([("w", toks[:lo], np.arange(lo))], ["w"])
        assert F.close_enough(got, whole, dtype), cuts[:3]
        eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_several_sequences_reused_slots_and_first_tokens(gpu, small, dtype):
    cfg, d, W, toks, want = small
    r = np.random.default_rng(8)
    seqs = {k: r.integers(0, cfg["vocab"], n) for k, n in (("a", 70), ("b", 9), ("c", 33), ("d", 50), ("e", 1), ("f", 3))}
    alone = {k: KP.forward(v, W, cfg) for k, v in seqs.items()}
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
    feed(("d", 1), ("e", 1), end=["e"])                    # d and e start in slots that b and c used: state must be clean
    feed(("a", 37), ("d", 2), ("f", 3), end=["a", "f"])
    feed(("d", 47), end=["d"])
    for k in seqs:
        assert at[k] == len(seqs[k]) and F.close_enough(np.concatenate(got[k]), alone[k], dtype), k
    st = eng.stats()
    assert st["live_seqs"] == 0 and st["free_pages"] == st["pages"] and free_mid < st["pages"]
    with pytest.raises(gpu.GgbError):  # a fourth live sequence has no slot
        eng.step([(k, [1], []) for k in "wxyz"])
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_behind_every_chunk_are_used_again_while_the_sequence_lives(gpu, small, dtype):
    cfg, d, W, toks, want = small   # chunks of 11 and 5 positions
    other = toks[::-1].copy()
    want_other = KP.forward(other, W, cfg)
    # two prompts of 150 tokens live together in a cache sized for 150: only the rows of the running chunks keep their pages
    eng = gpu.Engine(d, dtype=dtype, max_tokens=150, page_size=4, max_seqs=2)
    lo, rows, rows_o = 0, [], []
    cuts = [9, 1, 1, 7, 16, 2, 2, 1, 16, 13, 1, 1, 1, 16, 3, 16, 16, 12, 2, 14]
    for c in cuts:
        out = eng.step([("s", toks[lo:lo + c], np.arange(c)), ("o", other[lo:lo + c], np.arange(c))])
        rows.append(out[:c]); rows_o.append(out[c:])
        lo += c
        assert eng.seq_live_pages("s") <= 11 // 4 + 2 and eng.seq_live_pages("o") <= 11 // 4 + 2
    assert lo == 150 and F.close_enough(np.concatenate(rows), want, dtype) and F.close_enough(np.concatenate(rows_o), want_other, dtype)
    assert len(eng.seq_pages("s")) == (150 + 3) // 4 and (eng.seq_pages("s") >= 0).sum() == eng.seq_live_pages("s")
    with pytest.raises(gpu.GgbError, match="positions"):  # trimming frees pages, not positions
        eng.step([("s", toks[:20], [])])
    eng.end("s", "o")
    assert eng.stats()["free_pages"] == eng.stats()["pages"]
    # one attention layer that sees everything: nothing is trimmed and the same cache runs out, loudly
    cfg2 = F.config([F.layer("attention", F.attention(chunk=0)), F.layer("attention", F.attention(chunk=4))])
    d2, _ = F.make_model(d + "_unbounded", cfg2, seed=1)
    eng2 = gpu.Engine(d2, dtype=dtype, max_tokens=16, page_size=4, max_seqs=2)
    eng2.step([("s", toks[:20], [19])])
    assert eng2.seq_live_pages("s") == 5
    with pytest.raises(gpu.GgbError, match="out of pages"):
        eng2.step([("t", toks[:8], [])])
    eng.close(); eng2.close()


def test_long_decoding(gpu, small):
    cfg, d, W, toks, _ = small
    long = np.random.default_rng(2).integers(0, cfg["vocab"], 330)
    want = KP.forward(long, W, cfg)
    for dtype in ("float32", "bfloat16"):
        eng = gpu.Engine(d, dtype=dtype, max_tokens=400, page_size=32)
        rows = [eng.step([("s", long[:10], np.arange(10))])] + [eng.step([("s", long[i:i + 1], [0])]) for i in range(10, 330)]
        assert F.close_enough(np.concatenate(rows), want, dtype)
        eng.close()


OTHER = {
    # what the small configuration has unequal, equal or 1; what it has, absent
    "equal_and_absent": lambda: F.config([F.layer("attention", F.attention(heads=2, kv_heads=2, dim=8, vdim=8, chunk=0, softcap=0, base=0)),
                                          F.layer("channel_delta", F.delta(heads=2, kv_heads=2, dim=8, vdim=8, conv=1), F.dense(16))],
                                         vocab=17, width=16, streams=0, mult=1.0, buckets=0),
    "one_stream_one_expert": lambda: F.config([F.layer("channel_delta", F.delta(heads=1, kv_heads=1, dim=9, vdim=11, conv=8), F.moe(experts=1, identity=0, top=1, ff=5)),
                                               F.layer("attention", F.attention(heads=6, kv_heads=1, dim=10, vdim=4, chunk=1, dims=4, scaling=False), F.moe(experts=2, identity=3, top=5, ff=7))],
                                              vocab=30, width=22, streams=1, buckets=1, loop=(0, 2, 3)),
    "only_attention": lambda: F.config([F.layer("attention", F.attention(), F.moe()), F.layer("attention", F.attention(heads=1, kv_heads=1, dim=4, vdim=2, chunk=200, dims=2), F.dense(9))],
                                       vocab=64, width=12, streams=5, loop=(1, 2, 2)),
    "only_delta": lambda: F.config([F.layer("channel_delta", F.delta(), F.moe(experts=3, identity=1, top=2)), F.layer("channel_delta", F.delta(heads=3, kv_heads=3, dim=5, vdim=3, conv=4))],
                                   vocab=19, width=20, streams=2, buckets=3, loop=(0, 1, 1)),
    # seven streams (the scalar form of the stream kernel), low-rank projections too wide for the fused pair (rank 800, 801)
    "seven_streams_wide_rank": lambda: F.config([F.layer("channel_delta", F.delta(heads=2, kv_heads=1, dim=8, vdim=6, conv=2), F.moe(experts=3, identity=2, top=2, ff=6)),
                                                 F.layer("attention", F.attention(heads=2, kv_heads=1, dim=8, vdim=4, chunk=7), F.dense(12))],
                                                vocab=23, width=24, streams=7, buckets=5),
    "sixteen_streams": lambda: F.config([F.layer("attention", F.attention(heads=2, kv_heads=2, dim=6, vdim=6, chunk=0, dims=None), F.dense(10)),
                                         F.layer("channel_delta", F.delta(heads=2, kv_heads=2, dim=6, vdim=4, conv=3))], vocab=29, width=18, streams=16, loop=(0, 2, 2)),
    "wide": lambda: F.config([F.layer("channel_delta", F.delta(heads=4, kv_heads=2, dim=128, vdim=48, conv=4), F.moe(experts=6, identity=1, top=2, ff=40, limit=1.1)),
                              F.layer("attention", F.attention(heads=4, kv_heads=2, dim=32, vdim=64, chunk=70, dims=16), F.dense(160)),
                              F.layer("attention", F.attention(heads=2, kv_heads=1, dim=64, vdim=34, chunk=9, dims=None, scaling=False)),
                              F.layer("channel_delta", F.delta(heads=1, kv_heads=1, dim=20, vdim=70, conv=2), F.dense(96))],
                             vocab=200, width=128, streams=4, buckets=251, loop=(1, 4, 2)),
}


@pytest.mark.parametrize("name", sorted(OTHER))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes_and_optional_parts(gpu, tmp_path, name, dtype):
    cfg = OTHER[name]()
    d, W = F.make_model(str(tmp_path / name), cfg, seed=3, rank={"wide": 24, "seven_streams_wide_rank": 800}.get(name, 4))
    toks = np.random.default_rng(4).integers(0, cfg["vocab"], 140)
    want = KP.forward(toks, W, cfg)
    eng = gpu.Engine(d, dtype=dtype, max_tokens=300, page_size=16)
    whole = eng.step([("w", toks, np.arange(140))], ["w"])
    assert F.close_enough(whole, want, dtype)
    lo, rows = 0, []
    for c in [2, 2, 65, 1, 1, 3, 64, 2]:
        rows.append(eng.step([("s", toks[lo:lo + c], np.arange(c))]))
        lo += c
    assert F.close_enough(np.concatenate(rows), want, dtype)
    eng.close()


def test_a_far_token_reaches_the_end_through_the_delta_rule_only(gpu, tmp_path):
    """Attention sees its own chunk only; what a token 120 positions back changes in the last logits went through the
    recurrent state.  Changing token 3 moves the last row, in the oracle and in the engine alike."""
    cfg = F.config([F.layer("attention", F.attention(chunk=16), F.dense()), F.layer("channel_delta", F.delta(heads=2, kv_heads=1, dim=64, vdim=8), F.dense())], buckets=0)

    def remember(W):  # hardly any decay, and wide keys: a write is still there after 120 others
        W["l1.mix.A_log"][:] = -9.0
    d, W = F.make_model(str(tmp_path / "far"), cfg, seed=9, edit=remember)
    toks = np.random.default_rng(1).integers(0, cfg["vocab"], 124)
    other = toks.copy()
    other[3] = (other[3] + 1) % cfg["vocab"]
    za, zb = KP.forward(toks, W, cfg)[-1], KP.forward(other, W, cfg)[-1]
    assert np.abs(za - zb).max() > 1e-3
    eng = gpu.Engine(d, dtype="float32", max_tokens=300, page_size=16)
    for seq, want in ((toks, za), (other, zb)):
        eng.step([("s", seq[:100], [])])
        rows = [eng.step([("s", seq[i:i + 1], [0])]) for i in range(100, 124)]
        assert F.rel_err(rows[-1][0], want) < 3e-5
        eng.end("s")
    eng.close()


def test_random_weight_engine_portions_agree_at_sizes_that_reach_the_tensor_cores(gpu):
    cfg = F.config([F.layer("channel_delta", F.delta(heads=6, kv_heads=2, dim=64, vdim=32, conv=3), F.moe(experts=6, identity=1, top=2, ff=128, limit=7.0)),
                    F.layer("attention", F.attention(heads=8, kv_heads=2, dim=64, vdim=64, chunk=100, dims=32), F.dense(512))],
                   vocab=500, width=384, streams=3, buckets=251, loop=(0, 2, 2))
    toks = np.random.default_rng(0).integers(0, 500, 400)
    for dtype in ("bfloat16", "float32"):
        eng = gpu.Engine(config=cfg, seed=7, dtype=dtype, max_tokens=1024)
        whole = eng.step([("w", toks, np.arange(400))], ["w"])
        lo, rows = 0, []
        for c in [130, 2, 1, 1, 64, 200, 2]:
            rows.append(eng.step([("s", toks[lo:lo + c], np.arange(c))]))
            lo += c
        assert np.isfinite(whole).all() and F.close_enough(np.concatenate(rows), whole, dtype, loose=2.0)
        eng.close()


def test_greedy_generation_through_the_engine(gpu, small):
    cfg, d, W, toks, _ = small
    eng = gpu.Engine(d, dtype="float32", max_tokens=128)
    prompt = toks[:12]
    out = eng.generate("g", prompt, 25)
    assert len(out) == 25 and eng.seq_len("g") == 12 + 24
    z = KP.forward(np.concatenate([prompt, out]), W, cfg)
    for i, t in enumerate(out):  # every chosen token is the oracle's maximum at its place (up to rounding between near-equal logits)
        row = z[len(prompt) - 1 + i]
        assert row[t] >= row.max() - 1e-4, i
    eng.end("g")
    assert eng.stats()["live_seqs"] == 0
    eng.close()


def test_the_command_line_programs_replay_a_trace_and_generate(gpu, small, tmp_path):
    """bin/trace_run as its user starts it: steps on standard input, logits in files, a line per step; two requests one after the
    other with the second one's id used again; bin/lm_generate gives the ids Engine.generate gives."""
    import json
    import os
    import subprocess
    import sys
    cfg, d, W, toks, want = small
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "out")
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:40].tolist(), "want": [0, 39]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[40:42].tolist(), "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[42:43].tolist(), "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "a", "tokens": toks[:5].tolist(), "want": [4]}], "end": ["a"]}]
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [line for line in p.stdout.split("\n") if line.startswith("done")] == ["done %d" % i for i in range(4)]
    assert not os.path.exists(os.path.join(out, "1.f32"))
    got = {i: np.fromfile(os.path.join(out, "%d.f32" % i), dtype="<f4").reshape(-1, cfg["vocab"]) for i in (0, 2, 3)}
    assert F.close_enough(got[0], want[[0, 39]], "float32") and F.close_enough(got[2], want[[42]], "float32") and F.close_enough(got[3], want[[4]], "float32")
    g = subprocess.run([sys.executable, os.path.join(root, "bin", "lm_generate"), "--model", d, "--dtype", "float32", "--prompt", ",".join(map(str, toks[:12])), "--new", "9"],
                       capture_output=True, text=True, timeout=600)
    assert g.returncode == 0, g.stderr[-2000:]
    eng = gpu.Engine(d, dtype="float32", max_tokens=128)
    assert [int(t) for t in g.stdout.strip().split("\n")[-1].split(",")] == eng.generate("g", toks[:12], 9).tolist()
    eng.close()
