#!/usr/bin/env python
"""bench.py — the headline measurement: decode tokens/s of the Gemma quantized hot path on B200,
with the mat-vec kernels' HBM roofline fraction and the reference's CPU path timed beside it.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode token through the whole path (embedding row -> L layers -> logits -> greedy
token) at a pinned context length n_kv = ctx (BASELINE.json config 2: Gemma-2B, Q4_0, batch 1,
ctx 2048).  Weights (1.41 GB) are larger than the 126 MB L2, so every step re-streams them from HBM;
no L2 flush is needed.  One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            j = json.load(open(p))
            return float(j["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return 6650.0, "fallback (B200_PROFILING.md)"


class ClockSampler:
    """SM clock / throttle reasons sampled DURING the timed region (pynvml, every 100 ms)."""

    def __init__(self, index=0):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        if self.nv:
            self._t = threading.Thread(target=self._loop, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._t:
            self._t.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "note": "nvml unavailable"}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


MODELS = {"2b": "GEMMA_2B", "7b": "GEMMA_7B"}
WTYPES = {"q4_0": 2, "q8_0": 8}


def workload_name(args):
    return f"gemma-{args.model} {args.wtype} batch-1 decode, n_kv={args.ctx} pinned"


def matvec_bytes_per_step(dims, wtype):
    """algorithmic bytes of the mat-vec launches of one token: weights at 18|34 B per 32
    + Q8_0 activations read + fp32 outputs written."""
    bpb = 18 if wtype == 2 else 34
    E, L, H, Hkv, d, F, V = (dims[k] for k in ("n_embd", "n_layer", "n_head", "n_head_kv", "head_dim", "n_ff", "n_vocab"))
    QD, KD = H * d, Hkv * d
    mats = [(QD + 2 * KD, E), (E, QD), (2 * F, E), (E, F)]
    per_layer = sum(n * (k // 32) * bpb + (k // 32) * 34 + 4 * n for n, k in mats)
    per_layer -= 4 * 2 * F - (F // 32) * 34  # gate/up write Q8_0 blocks, not fp32
    return L * per_layer + V * (E // 32) * bpb + (E // 32) * 34 + 4 * V


def cpu_reference_tokens_per_s(args, n_tokens, warm=1, budget_s=None):
    """The reference's CPU path restated by the oracle (thread_pool row split, scalar vec_dot), on the
    same workload; ORACLE USE: this is the oracle timed as a baseline, never the product.
    budget_s bounds the timed region: tokens stop early once it is spent (the count actually timed is
    returned), so the run ends within minutes whatever the host's core count."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    import gemma_ggml_b200 as G
    dims = dict(getattr(G, MODELS[args.model]), n_ctx=args.ctx)
    threads = os.cpu_count() or 1
    m = O.Model(wtype=WTYPES[args.wtype], n_threads=threads, **dims)
    m.fill_kv_synth(99)
    tok = np.array([4242], dtype=np.int32)
    for _ in range(warm):
        m.forward(tok, args.ctx - 1, O.REF)
    t0 = time.perf_counter()
    done = 0
    for _ in range(n_tokens):
        logits = m.forward(tok, args.ctx - 1, O.REF)
        tok[0] = O.argmax(logits)
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    m.close()
    return done / dt, threads, dt, done


def bench_config(args, world, lowering, kernels_per_step):
    """the `config` object of a line: the SAME keys for both arms (the driver compares them)"""
    return {"workload": workload_name(args), "parallelism": f"tp{world}" if world > 1 else "single",
            "l2": "weights (1.41 GB for 2B Q4_0) > 126 MB L2: re-streamed from HBM every step, no flush needed",
            "lowering": lowering, "graph": "one CUDA graph per token", "kernels_per_step": kernels_per_step}


def run_reference(args):
    """--impl reference: the reference's own CPU implementation of the path.  The reference cannot be compiled
    (un-vendored ggml), so this is the oracle's restatement of its thread_pool mul_mat path
    with all host threads (kind "port": scalar vec_dot, not ggml's hand-written SIMD).  One step = one full decode
    token of the same workload; the timed region is capped at ~150 s."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t_all0 = time.perf_counter()
    warm = max(1, args.warmup)
    # warm-up tokens are bounded in time as well (a token takes ~1 s on 16 cores): the count actually run is reported
    tps_w, threads, dt_w, warm_done = cpu_reference_tokens_per_s(args, warm, warm=0, budget_s=20.0)
    tps, threads, dt, done = cpu_reference_tokens_per_s(args, args.steps, warm=0, budget_s=150.0)
    line = {
        "impl": "reference", "metric": "decode tokens/s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "steps_timed": done, "warmup_run": warm_done,
        "ms_per_step": 1000.0 * dt / done,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 dot (dp4a), fp32 accumulate",
        "data": "synthetic (seeded random-init Gemma-architecture weights in ggml quant format, synthetic KV)",
        "config": bench_config(args, args.gpus, "fused persistent decode kernel", 1),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{done} full decode tokens (of {args.steps} requested; timed region capped at 150 s), "
                                   f"oracle restatement of src/hpc.cpp thread_pool path (scalar ggml vec_dot, "
                                   f"gcc -O3 AVX2 autovec; upstream hand-written SIMD kernels not reproduced)"},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t_all0,
    }
    print(json.dumps(line), flush=True)


def time_decode(G, L, m, steps, warmup, pos, barrier, dist):
    """K graph-replayed steps, inputs resident, CUDA events on the launching stream; max over ranks"""
    m.set_state(4242, pos, 0)
    m.run_steps(warmup)
    barrier()
    L.ggb_prof_enable(1)
    G.prof_reset()
    barrier()
    L.ggb_prof_start(b"bench_timed_region")
    m.run_steps(steps)
    L.ggb_prof_stop(b"bench_timed_region")
    barrier()
    ms, _ = G.prof_get("bench_timed_region")
    L.ggb_prof_enable(0)
    if dist is not None:
        import torch
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def rank_bytes(m, dims, ctx, world):
    """algorithmic bytes THIS GPU streams per token: its weight pass streams (row shards + replicated phases; 18 | 34 B
    per 32 weights, the same figure as SURVEY 8d for one GPU) + the KV rows of the heads whose cache it holds"""
    kv = dims["n_layer"] * 2 * m.rank_kv_heads * dims["head_dim"] * 2 * ctx
    return m.rank_stream_bytes + kv


def sub_record_7b(G, L, args, dist, rank, world, barrier, peak):
    """BASELINE config 4 on the same run: Gemma-7B Q4_0, n_kv 2048, tensor parallel over the same ranks"""
    dims = dict(G.GEMMA_7B, n_ctx=2048)
    m = G.GemmaModel(G.make_config(wtype=2, **dims))
    if world > 1:
        m.init_tensor_parallel(dist, rank, world)
    m.init_synthetic_weights(); m.init_kv_cache(); m.fill_kv_cache_synthetic(99)
    m.build_compute_graph(capture_acts=False, fused=True)
    steps = max(16, min(args.steps, 128))
    ms = time_decode(G, L, m, steps, max(3, min(args.warmup, 8)), 2047, barrier, dist)
    rb = rank_bytes(m, dims, 2048, world)
    step_s = ms / steps / 1000.0
    rec = {"workload": "gemma-7b q4_0 batch-1 decode, n_kv=2048 pinned", "value": steps / (ms / 1000.0), "unit": "tokens/s",
           "ms_per_step": ms / steps, "steps": steps, "parallelism": f"tp{world}" if world > 1 else "single",
           "per_gpu_bytes_per_step": rb, "per_gpu_gbs": rb / step_s / 1e9, "per_gpu_frac_of_peak": rb / step_s / 1e9 / peak}
    m.close()
    return rec


def sub_record_prefill(G, L, args):
    """BASELINE config 3 on the same run (1 GPU): Gemma-2B Q8_0, prefill of 512 tokens through the tcgen05 GEMMs"""
    T = 512
    dims = dict(G.GEMMA_2B, n_ctx=T)
    m = G.GemmaModel(G.make_config(wtype=8, **dims))
    m.init_synthetic_weights(); m.init_kv_cache(); m.build_compute_graph(capture_acts=False, fused=True)
    prompt = ((1 + 7919 * np.arange(T)) % dims["n_vocab"]).astype(np.int32)
    for _ in range(3):
        m.prefill(prompt, 0)
    G.sync()
    steps = 5
    t0 = time.perf_counter()            # the step as a user runs it: no profiling probes
    for _ in range(steps):
        m.prefill(prompt, 0)
    G.sync()
    wall = time.perf_counter() - t0
    L.ggb_prof_enable(1)                # then the same steps with cudaEvent probes around every operator: GEMM time
    G.prof_reset()
    for _ in range(steps):
        m.prefill(prompt, 0)
    G.sync()
    gemm_ms, _ = G.prof_get("op_mul_mat")
    L.ggb_prof_enable(0)
    peak_tf = 1396.9
    try:
        peak_tf = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"])
    except Exception:
        pass
    ach = m.prefill_gemm_flops / (gemm_ms / steps / 1000.0) / 1e12 if gemm_ms > 0 else 0.0
    rec = {"workload": "gemma-2b q8_0 prefill of 512 tokens (host call: H2D ids, per-op launches, D2H token)",
           "value": T * steps / wall, "unit": "tokens/s", "ms_per_step": 1000.0 * wall / steps,
           "gemm_tflops": ach, "gemm_frac_of_tensor_peak": ach / peak_tf, "gemm_ms_per_step": gemm_ms / steps,
           "tensor_peak_tflops": peak_tf, "kernel": "gemm_bf16w_kernel (tcgen05.mma kind::f16, TMEM accumulators)"}
    m.close()
    return rec


def mul_mat_dropin_us(G):
    """the plugin boundary itself: the reference's mul_mat entry (host buffers in, host buffer out, src/hpc.h:22-32)
    per Gemma-2B Q4_0 shape, one column: us per call after the weight is resident (H2D of the Q8_0 row + kernel + D2H)"""
    import ctypes as C
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    out = {}
    L = G.cuda_lib()
    rng = np.random.default_rng(5)
    for name, (K, N) in {"q/o 2048x2048": (2048, 2048), "gate/up 2048x16384": (2048, 16384), "down 16384x2048": (16384, 2048)}.items():
        nb = K // 32
        w = rng.integers(0, 256, size=(N, nb * 18), dtype=np.uint8)
        w[:, 0::18] = 0; w[:, 1::18] = 0x1c  # fp16 scales ~ 0.004
        act = rng.integers(0, 256, size=(nb * 34,), dtype=np.uint8)
        act[0::34] = 0; act[1::34] = 0x20
        dst = np.zeros(N, dtype=np.float32)
        call = lambda: L.ggb_mul_mat(N, 1, 1, nb * 18, 1, N * 4, N * 4, nb * 34, K, w.ctypes.data_as(C.c_void_p),
                                     dst.ctypes.data_as(C.c_void_p), 2, act.ctypes.data_as(C.c_char_p))
        if call() != 0:
            out[name] = None
            continue
        for _ in range(5):
            call()
        t0 = time.perf_counter()
        for _ in range(50):
            call()
        out[name] = (time.perf_counter() - t0) / 50 * 1e6
        L.ggb_mul_mat_forget(w.ctypes.data_as(C.c_void_p))
    return out


def kquant_matvec_record(G, peak_gbs):
    """SURVEY.md 8f-2 on the record: the resident (packed) K-quant mat-vecs on the tied-embedding shape of Gemma-2B
    (256000 x 2048, one Q8_K activation row), device-timed; algorithmic bytes = ggml's block bytes (144 / 210 per 256)."""
    L = G.cuda_lib()
    rng = np.random.default_rng(11)
    n, k = 256000, 2048
    nb = k // 256
    out = {}
    x = rng.standard_normal((1, k)).astype(np.float32)
    act = G.quantize_q8_K(x)
    ad = G.DeviceBuffer.from_numpy(act)
    dst = G.DeviceBuffer(4 * n)
    for name, size, d_off in (("q4_K", 144, 0), ("q6_K", 210, 208)):
        w = rng.integers(0, 256, size=(n, nb, size), dtype=np.uint8)
        w[:, :, d_off] = 0
        w[:, :, d_off + 1] = 0x1c            # fp16 super-scale ~ 0.004
        if name == "q4_K":
            w[:, :, 2] = 0
            w[:, :, 3] = 0x1c
        w = np.ascontiguousarray(w.reshape(n, nb * size))
        wd = G.DeviceBuffer.from_numpy(w)
        if name == "q4_K":
            packed = G.DeviceBuffer(w.nbytes)
            G.check(L.ggb_op_q4k_repack(wd.ptr, n, w.shape[1], k, packed.ptr), "repack")
            call = lambda: L.ggb_op_mul_mat_q4k_packed(packed.ptr, n, k, ad.ptr, act.shape[1], 1, dst.ptr, n)
        else:
            packed = G.DeviceBuffer(L.ggb_q6k_packed_bytes(n, k))
            G.check(L.ggb_op_q6k_repack(wd.ptr, n, w.shape[1], k, packed.ptr), "repack")
            call = lambda: L.ggb_op_mul_mat_q6k_packed(packed.ptr, n, k, ad.ptr, act.shape[1], 1, dst.ptr, n)
        for _ in range(5):
            G.check(call(), "kquant mat-vec")
        G.sync()
        L.ggb_prof_enable(1); G.prof_reset()
        L.ggb_prof_start(b"kq")
        for _ in range(40):
            call()
        L.ggb_prof_stop(b"kq")
        G.sync()
        ms, _ = G.prof_get("kq")
        L.ggb_prof_enable(0)
        us = ms * 1e3 / 40
        gbs = w.nbytes / (us * 1e-6) / 1e9
        out[name] = {"shape": "256000 x 2048 (resident, packed form)", "us_per_launch": us, "algorithmic_gbs": gbs,
                     "frac_of_hbm_peak": gbs / peak_gbs}
        del wd, packed
    return out


def run_ours(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    import gemma_ggml_b200 as G

    dist = None
    if world > 1:
        # NCCL prints its version banner to stdout at NCCL_DEBUG=VERSION: the line rank 0 prints must stay the only one
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        import torch
        import torch.distributed as dist_mod
        torch.cuda.set_device(local_rank)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    G.init(local_rank)
    L = G.cuda_lib()

    def barrier():
        G.sync()
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()

    # ---- multi-GPU: parity first (tiny MQA + MHA models, both quant types, fused lowering, against the oracle, bit for
    # bit) - ORACLE USE: the oracle, before and outside every timed region
    tp_parity = None
    if world > 1:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as O
        import tp_worker
        try:
            n = tp_worker.check(G, O, dist, rank, world, lowerings=(True,))
            tp_parity = f"ok ({n} cases: small mqa / mha / thin models x q4_0/q8_0, tokens and logits bit-identical to the oracle)"
        except AssertionError as e:
            tp_parity = f"FAILED: {e}"
        barrier()

    wtype = WTYPES[args.wtype]
    dims = dict(getattr(G, MODELS[args.model]), n_ctx=args.ctx)
    cfg = G.make_config(wtype=wtype, **dims)
    m = G.GemmaModel(cfg)
    if world > 1:
        m.init_tensor_parallel(dist, rank, world)
    m.init_synthetic_weights()
    m.init_kv_cache()
    m.fill_kv_cache_synthetic(99)
    m.build_compute_graph(capture_acts=False, fused=(args.mode == "fused"))
    fused = m.is_fused
    kernels_per_step = m.kernels_per_step
    pos = args.ctx - 1

    # ---- value: K graph-replayed steps, inputs resident, CUDA events on the launching stream
    with ClockSampler(local_rank) as clocks:
        ms = time_decode(G, L, m, args.steps, args.warmup, pos, barrier, dist)
    tok_s = args.steps / (ms / 1000.0)

    # ---- e2e: the host-buffer call a user makes (pinned H2D of token+pos, graph, D2H of the token)
    e2e_steps = max(8, min(args.steps, 128))
    for _ in range(3):
        m.decode_step(4242, pos)
    barrier()
    t0 = time.perf_counter()
    tok = 4242
    for _ in range(e2e_steps):
        tok = m.decode_step(tok, pos)
    G.sync()
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        import torch
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_tok_s = e2e_steps / e2e_s

    # ---- roofline of the dominant kernel: PER GPU (what this GPU streams per launch / its launch time / its peak)
    peak, peak_src = load_peaks()
    kv_bytes = dims["n_layer"] * 2 * dims["n_head_kv"] * dims["head_dim"] * 2 * args.ctx
    step_s = ms / args.steps / 1000.0
    per_class = {}
    wname = "Q4_0" if wtype == 2 else "Q8_0"
    if fused:
        # one persistent kernel per token: algorithmic bytes per launch = weights + KV this GPU reads,
        # duration = the CUDA-event time of the timed region / launches
        step_bytes = (m.weight_bytes + kv_bytes) if world == 1 else rank_bytes(m, dims, args.ctx, world)
        achieved = step_bytes / step_s / 1e9
        quad = "true" if args.model == "7b" else "false"
        roof_kernel = f"decoder_kernel<{wname}, QUAD={quad}, PROF=false> (persistent, one cooperative launch per token)"
        roof_bytes, roof_launches, roof_us = step_bytes, 1.0, step_s * 1e6
    else:
        # per-operator lowering: cudaEvent probes around every launch of an eager pass, mat-vec class
        prof_steps = 8
        m.set_state(4242, pos, 0)
        m.run_steps_profiled(2)
        G.prof_reset()
        m.run_steps_profiled(prof_steps)
        for name in ("op_mul_mat", "op_attn", "op_rms_norm", "op_rope", "op_get_rows", "op_argmax"):
            tms, calls = G.prof_get(name)
            per_class[name] = {"ms_per_step": tms / prof_steps, "launches_per_step": calls / prof_steps}
        step_bytes = (m.weight_bytes + kv_bytes) / world
        roof_bytes = matvec_bytes_per_step(dims, wtype) / world
        mv_ms = per_class["op_mul_mat"]["ms_per_step"]
        roof_launches = per_class["op_mul_mat"]["launches_per_step"]
        achieved = roof_bytes / (mv_ms / 1000.0) / 1e9 if mv_ms > 0 else 0.0
        roof_kernel = f"matvec_kernel<{wname}> / gate_up_kernel<{wname}> (all weight mat-vecs of a step, eager + cudaEvent probes)"
        roof_us = 1000.0 * mv_ms / roof_launches if roof_launches else None
    traffic = None
    if world == 1:  # one ncu --set full capture of this kernel on this workload (profiles/traffic.json); not valid for shards
        tpath = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(tpath) and args.model == "2b" and args.wtype == "q4_0" and args.ctx == 2048:
            try:
                traffic = json.load(open(tpath)).get("fused" if fused else "ops")
            except Exception:
                traffic = None
    exp_mode = int(L.ggb_decoder_exp_computed(m.H.gm_decoder(m.h))) if fused else None
    m.close()

    # ---- sub-records measured in the same run
    extra = {}
    if fused and args.model == "2b" and not args.no_sub_records:
        try:
            extra["config4_7b_q4_0"] = sub_record_7b(G, L, args, dist, rank, world, barrier, peak)
        except Exception as e:
            extra["config4_7b_q4_0"] = {"failed": str(e)}
        if world == 1:
            try:
                extra["config3_prefill_2b_q8_0"] = sub_record_prefill(G, L, args)
            except Exception as e:
                extra["config3_prefill_2b_q8_0"] = {"failed": str(e)}
            try:
                extra["mul_mat_dropin_us_per_call"] = mul_mat_dropin_us(G)
            except Exception as e:
                extra["mul_mat_dropin_us_per_call"] = {"failed": str(e)}
            try:
                extra["kquant_matvec"] = kquant_matvec_record(G, peak)
            except Exception as e:  # noqa: BLE001
                extra["kquant_matvec"] = {"failed": str(e)}
    if rank != 0:
        return
    line = {
        "metric": "decode tokens/s", "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 dot (dp4a), fp32 accumulate",
        "data": "synthetic (seeded random-init Gemma-architecture weights in ggml quant format, synthetic KV)",
        "config": bench_config(args, world, "fused persistent decode kernel" if fused else "per-operator kernels", kernels_per_step),
        "clocks": clocks.summary(),
        "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 16, "d2h_bytes_per_step": 4,
                "steps": e2e_steps},
        "gpu_launches": kernels_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak if peak else None, "traffic": traffic, "peak_source": peak_src,
                     "kernel": roof_kernel, "algorithmic_bytes_per_launch": roof_bytes / roof_launches,
                     "launches_per_step": roof_launches, "avg_launch_us": roof_us,
                     "scope": "per GPU: bytes this GPU streams per launch / its launch time / its measured peak",
                     "step_frac_of_8tbs": step_bytes / step_s / 1e9 / 8000.0},
        "parity": "tokens and logits bit-identical to the oracle's scalar ggml order (tests/test_model_gpu.py; config 1 "
                  "at full size from tests/golden/)",
        "softmax_exp": {2: "computed (fp32 expf, proved equal to the fp16 table)", 1: "computed (double exp, proved equal)",
                        0: "fp16 table lookup", None: None}[exp_mode],
        "op_classes": per_class,
    }
    if tp_parity is not None:
        line["tp_parity"] = tp_parity
    line.update(extra)
    if world == 1 and not args.no_cpu_baseline:
        try:
            tps, threads, dt, done = cpu_reference_tokens_per_s(args, args.cpu_tokens, budget_s=30.0)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                                    "sample": f"{done} full decode tokens of the same workload in {dt:.1f} s "
                                              f"(oracle restatement of the reference thread_pool path, scalar vec_dot; "
                                              f"upstream ggml's hand-written SIMD kernels are not reproduced)"}
        except Exception as e:  # the baseline must not take the GPU number down with it
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                                    "sample": f"failed: {e}"}
    print(json.dumps(line), flush=True)


def run_prefill(args):
    """Secondary workload (BASELINE.json config 3): batched prefill of T tokens through the dequant -> bf16
    tcgen05 GEMMs.  value = prompt tokens/s; roofline = tensor pipe (GEMM flops / cudaEvent time of the GEMM
    launches vs the measured dense bf16 peak)."""
    import gemma_ggml_b200 as G
    G.init(0)
    L = G.cuda_lib()
    T = args.prefill_tokens
    dims = dict(getattr(G, MODELS[args.model]), n_ctx=max(args.ctx, T))
    m = G.GemmaModel(G.make_config(wtype=WTYPES[args.wtype], **dims))
    m.init_synthetic_weights(); m.init_kv_cache(); m.build_compute_graph(capture_acts=False, fused=True)
    prompt = ((1 + 7919 * np.arange(T)) % dims["n_vocab"]).astype(np.int32)
    for _ in range(max(3, args.warmup if args.warmup < 8 else 3)):
        m.prefill(prompt, 0)
    G.sync()
    steps = max(1, min(args.steps, 20))
    with ClockSampler(0) as clocks:       # the step as a user runs it: no profiling probes
        t0 = time.perf_counter()
        for _ in range(steps):
            m.prefill(prompt, 0)
        G.sync()
        wall = time.perf_counter() - t0
    L.ggb_prof_enable(1)                  # then the same steps with cudaEvent probes around every operator
    G.prof_reset()
    for _ in range(steps):
        m.prefill(prompt, 0)
    G.sync()
    gemm_ms, gemm_calls = G.prof_get("op_mul_mat")
    classes = {}
    for name in ("op_mul_mat", "op_attn", "op_rms_norm", "op_rope", "op_cvt", "op_gelu", "op_cpy", "op_get_rows", "op_argmax"):
        tms, calls = G.prof_get(name)
        classes[name] = {"ms_per_step": tms / steps, "launches_per_step": calls / steps}
    L.ggb_prof_enable(0)
    flops = m.prefill_gemm_flops
    peak_tf = 1396.9
    try:
        peak_tf = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"])
    except Exception:
        pass
    ach = flops / (gemm_ms / steps / 1000.0) / 1e12 if gemm_ms > 0 else 0.0
    line = {
        "metric": "prefill tokens/s", "value": T * steps / wall, "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": 3, "ms_per_step": 1000.0 * wall / steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 x bf16 -> fp32 (weights dequantised from " + args.wtype + ")",
        "data": "synthetic (seeded random-init Gemma-architecture weights in ggml quant format)",
        "config": {"workload": f"gemma-{args.model} {args.wtype} prefill of {T} tokens (host call: H2D ids, per-op launches, D2H token)",
                   "timing": "value / ms_per_step: eager per-op launches, no probes; roofline and op_classes: a second pass of the same steps with cudaEvent probes per operator (the probes add ~1 ms of launch gaps per step)"},
        "clocks": clocks.summary(),
        "roofline": {"bound": "tensor", "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s", "frac": ach / peak_tf,
                     "traffic": None, "kernel": "gemm_bf16w_kernel (tcgen05.mma kind::f16, TMEM accumulators)",
                     "algorithmic_flops_per_step": flops, "gemm_ms_per_step": gemm_ms / steps,
                     "launches_per_step": gemm_calls / steps, "peak_source": "MEASURED_PEAKS.json bf16_tflops_sustained"},
        "op_classes": classes,
    }
    m.close()
    print(json.dumps(line), flush=True)


SAFOLORN_SIZES = {
    # width, layers, heads, dim, rot_dim, vdim, kv_rank, dense ff, experts, top, expert ff, vocab
    "s": (1024, 8, 8, 64, 32, 64, 256, 4096, 16, 2, 1024, 32000),
    "m": (2048, 8, 16, 128, 64, 128, 512, 8192, 32, 4, 1408, 32000),
    "l": (4096, 4, 32, 128, 64, 128, 512, 12288, 16, 2, 2048, 32000),
}


def safolorn_config(size):
    """Layers in the pattern own-cache/dense, own-cache/experts, borrowed-cache/dense, borrowed-cache/experts."""
    W, L, H, D, Dr, Dv, R, ff, E, top, eff, V = SAFOLORN_SIZES[size]
    rot = {"base": 10000.0, "dims": Dr, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    layers = []
    for i in range(L):
        mx = {"heads": H, "dim": D, "rot_dim": Dr, "vdim": Dv, "kv_rank": R, "scale": 1.0 / (D + Dr) ** 0.5, "rot": rot}
        if i % 4 >= 2:
            mx["kv_from"] = i - 2
        mlp = {"kind": "dense", "ff": ff, "limit": 7.0} if i % 2 == 0 else \
            {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "top": top}}
        layers.append({"type": "latent_attention", "mixer": mx, "mlp": mlp})
    return {"architecture": "Safolorn", "vocab": V, "width": W, "norm": {"eps": 1e-5}, "token_side": {"dim": 64}, "layers": layers}


def run_safolorn(args):
    """--arch safolorn: prefill and decode throughput of the Safolorn design (random bf16 weights) at layer sizes of real
    models, through the serving engine (host call: H2D token ids, operator launches / graph replay, D2H result), with
    cudaEvent time per operator class and roofline fractions of the matrix and attention operators; beside it the
    Gemma path (Q8_0 weights) at the same width, depth, heads and feed-forward size."""
    import gemma_ggml_b200 as G
    G.init(0)
    L = G.cuda_lib()
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    try:
        pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        peaks = {"hbm_gbs": float(pk["hbm_gbs"]), "bf16_tflops_sustained": float(pk["bf16_tflops_sustained"]), "source": "MEASURED_PEAKS.json"}
    except Exception:
        pass
    T, ctx, n_dec = args.prefill_tokens if args.prefill_tokens != 512 else 2048, args.ctx, min(args.steps, 128)
    records = {}
    for size in args.sizes.split(","):
        cfg = safolorn_config(size)
        W, nl, H, D, Dr, Dv, R, ff, E, top, eff, V = SAFOLORN_SIZES[size]
        eng = G.Engine(config=cfg, seed=7, dtype="bfloat16", max_tokens=ctx + n_dec + 64, page_size=64, max_portion=1024)
        r = np.random.default_rng(0)
        prompt = r.integers(0, V, T).astype(np.int32)

        def prefill():
            eng.step([("p", prompt, [T - 1])], ["p"])
        for _ in range(3):
            prefill()
        reps = 5
        with ClockSampler(0) as clocks:
            t0 = time.perf_counter()
            for _ in range(reps):
                prefill()
            pf = (time.perf_counter() - t0) / reps
        L.ggb_prof_enable(1)
        G.prof_reset()
        prefill()
        G.sync()
        pf_ops = {k: G.prof_get(k)[0] for k in ("op_linear", "op_attn", "op_attn_prep", "op_attn_out", "op_moe", "op_moe_linear", "op_norm", "op_act", "op_residual", "op_rows")}
        L.ggb_prof_enable(0)
        # algorithmic work of one prefill
        lin_flops = moe_flops = attn_flops = 0.0
        lin_bytes = moe_bytes = 0.0
        for i, Ly in enumerate(cfg["layers"]):
            own = "kv_from" not in Ly["mixer"]
            n_lin = H * (D + Dr) * W + (own and (R + Dr) * W or 0) + W * H * Dv
            if Ly["mlp"]["kind"] == "dense":
                n_lin += 3 * ff * W
            else:
                moe_flops += 2.0 * T * top * 2 * eff * W
                moe_bytes += 2.0 * top * 2 * eff * W  # decode: the chosen experts only
            lin_flops += 2.0 * T * n_lin
            lin_bytes += 2.0 * n_lin
            attn_flops += 2.0 * H * (2 * R + Dr) * T * (T + 1) / 2
        lin_flops += 2.0 * V * W  # one row of logits
        lin_bytes += 2.0 * V * W
        # decode at n_kv ~ ctx: fill the cache with a prompt, then greedy tokens through the captured one-token step
        eng.step([("d", r.integers(0, V, ctx - 1).astype(np.int32), [])])
        eng.generate("d", [1], 8)
        t0 = time.perf_counter()
        eng.generate("d", [2], n_dec)
        dec = (time.perf_counter() - t0) / n_dec
        kernels = eng.stats()["kernels_last_forward"]
        eng.use_graphs(False)
        eng.generate("d", [3], 4)
        L.ggb_prof_enable(1)
        G.prof_reset()
        eng.generate("d", [4], 8)
        G.sync()
        dc_ops = {k: G.prof_get(k)[0] / 8 for k in pf_ops}
        L.ggb_prof_enable(0)
        eng.end("d")
        n_cache = sum("kv_from" not in Ly["mixer"] for Ly in cfg["layers"])
        cache_bytes = 2.0 * nl * ctx * (R + Dr)  # every layer reads a cache (its own or a borrowed one)
        wbytes = eng.stats()["weight_bytes"]
        eng.close()
        rec = {
            "config": {"width": W, "layers": nl, "heads": H, "dim": D, "rot_dim": Dr, "vdim": Dv, "kv_rank": R, "ff": ff, "experts": E, "top": top,
                       "expert_ff": eff, "vocab": V, "caching_layers": n_cache, "weight_bytes": wbytes},
            "prefill": {"tokens": T, "tokens_per_s": T / pf, "ms": 1e3 * pf, "op_ms": pf_ops, "clocks": clocks.summary(),
                        "linear_tflops": lin_flops / (pf_ops["op_linear"] / 1e3) / 1e12,
                        "linear_frac_of_tensor_peak": lin_flops / (pf_ops["op_linear"] / 1e3) / 1e12 / peaks["bf16_tflops_sustained"],
                        "moe_linear_tflops": moe_flops / (pf_ops["op_moe_linear"] / 1e3) / 1e12,
                        "attn_tflops_cuda_cores": attn_flops / (pf_ops["op_attn"] / 1e3) / 1e12},
            "decode": {"n_kv": ctx, "tokens_per_s": 1.0 / dec, "us_per_token": 1e6 * dec, "kernels_per_token": kernels, "op_us": {k: 1e3 * v for k, v in dc_ops.items()},
                       "linear_gbs": lin_bytes / (dc_ops["op_linear"] / 1e3) / 1e9, "linear_frac_of_hbm_peak": lin_bytes / (dc_ops["op_linear"] / 1e3) / 1e9 / peaks["hbm_gbs"],
                       "moe_linear_gbs": moe_bytes / (dc_ops["op_moe_linear"] / 1e3) / 1e9,
                       "attn_gbs": cache_bytes / (dc_ops["op_attn"] / 1e3) / 1e9,
                       "token_frac_of_hbm_roofline": ((lin_bytes + moe_bytes + cache_bytes) / (peaks["hbm_gbs"] * 1e9)) / dec},
        }
        # the closest existing model at equal size: the Gemma path, Q8_0, same width / depth / heads / feed-forward
        if not args.no_sub_records:
            dims = dict(n_embd=W, n_layer=nl, n_head=H, n_head_kv=H, head_dim=D + Dr if (D + Dr) % 64 == 0 else 128, n_ff=ff, n_vocab=V, n_ctx=ctx + 8)
            m = G.GemmaModel(G.make_config(wtype=8, **dims))
            m.init_synthetic_weights(); m.init_kv_cache(); m.fill_kv_cache_synthetic(99); m.build_compute_graph(capture_acts=False, fused=False)
            gp = ((1 + 7919 * np.arange(T)) % V).astype(np.int32)
            for _ in range(3):
                m.prefill(gp, 0)
            G.sync()
            t0 = time.perf_counter()
            for _ in range(reps):
                m.prefill(gp, 0)
            G.sync()
            gpf = (time.perf_counter() - t0) / reps
            L.ggb_prof_enable(1)
            G.prof_reset()
            m.prefill(gp, 0)
            G.sync()
            g_gemm, g_attn = G.prof_get("op_mul_mat")[0], G.prof_get("op_attn")[0]
            L.ggb_prof_enable(0)
            g_flops = m.prefill_gemm_flops
            m.fill_kv_cache_synthetic(99)
            m.set_state(1, ctx - 1, 0); m.run_steps(8); G.sync()
            t0 = time.perf_counter()
            m.run_steps(n_dec); G.sync()
            gdec = (time.perf_counter() - t0) / n_dec
            G.prof_reset()
            m.run_steps_profiled(8)
            G.sync()
            g_mv, g_at = G.prof_get("op_mul_mat")[0] / 8, G.prof_get("op_attn")[0] / 8
            gbytes = m.weight_bytes
            rec["gemma_equal_size"] = {
                "config": dict(dims, wtype="q8_0", lowering="per-operator graph"),
                "prefill": {"tokens_per_s": T / gpf, "ms": 1e3 * gpf, "gemm_ms": g_gemm, "attn_ms": g_attn, "gemm_tflops": g_flops / (g_gemm / 1e3) / 1e12,
                            "gemm_frac_of_tensor_peak": g_flops / (g_gemm / 1e3) / 1e12 / peaks["bf16_tflops_sustained"],
                            "attn_tflops_cuda_cores": 4.0 * nl * H * dims["head_dim"] * T * (T + 1) / 2 / (g_attn / 1e3) / 1e12},
                "decode": {"tokens_per_s": 1.0 / gdec, "us_per_token": 1e6 * gdec, "matvec_us": 1e3 * g_mv, "attn_us": 1e3 * g_at,
                           "matvec_gbs": gbytes / (g_mv / 1e3) / 1e9, "matvec_frac_of_hbm_peak": gbytes / (g_mv / 1e3) / 1e9 / peaks["hbm_gbs"],
                           "attn_gbs": 2.0 * 2 * nl * ctx * H * dims["head_dim"] / (g_at / 1e3) / 1e9},
            }
            m.close()
        records[size] = rec
    first = records[args.sizes.split(",")[0]]
    print(json.dumps({"metric": "safolorn decode tokens/s", "value": first["decode"]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
                      "steps": n_dec, "warmup": 8, "ms_per_step": first["decode"]["us_per_token"] / 1e3, "higher_is_better": True,
                      "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random bf16 weights of the configured sizes)",
                      "config": {"workload": "Safolorn sizes " + args.sizes + ": prefill of %d tokens, greedy decode at n_kv %d, through the serving engine" % (T, ctx),
                                 "l2": "weights of every size exceed the 126 MB L2"},
                      "peaks": peaks, "sizes": records}), flush=True)


BEGUPEL_SIZES = {  # width, layers, heads, kv heads, head size, window, delta heads, delta kv heads, lightning heads, ff, vocab
    "s": (1024, 8, 8, 2, 128, 1024, 8, 4, 8, 4096, 32000),
    "m": (2048, 8, 16, 4, 128, 1024, 16, 8, 16, 8192, 32000),
    "l": (4096, 4, 32, 8, 128, 2048, 32, 16, 32, 12288, 32000),
}


def begupel_config(size):
    """Layers alternate: window attention beside a gated delta rule, then lightning attention; each with a dense feed-forward."""
    W, L, H, G, D, win, Hr, Gr, Hl, ff, V = BEGUPEL_SIZES[size] if isinstance(size, str) else size
    layers = []
    for i in range(L):
        if i % 2 == 0:
            mx = {"left": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "mask": {"size": win},
                           "rot": {"base": 1000000.0, "dims": D, "scaling": {"factor": 4.0}}},
                  "right": {"heads": Hr, "kv_heads": Gr, "dim": D, "vdim": D, "conv": 4}, "left_scale": 1.0, "right_scale": 1.0}
            layers.append({"type": "parallel", "mixer": mx, "mlp": {"kind": "dense", "ff": ff}})
        else:
            mx = {"heads": Hl, "dim": D, "vdim": D, "decay": [float(np.exp(-1.0 / (2.0 * 2.0 ** (10.0 * h / Hl)))) for h in range(Hl)]}
            layers.append({"type": "lightning", "mixer": mx, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Begupel", "vocab": V, "width": W, "norm": {"eps": 1e-5, "groups": 4}, "canon": {"taps": 4},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 131, "mul_cur": 31}}, "logit_softcap": 30.0, "layers": layers}


BG_OPS = ("op_linear", "op_attn", "op_attn_prep", "op_attn_out", "op_recurrence", "op_conv", "op_norm", "op_act", "op_residual", "op_rows")


def _engine_times(G, eng, V, T, ctx, n_dec, ops):
    """prefill of T tokens and greedy decode at n_kv ~ ctx through an engine: host-timed seconds, cudaEvent ms per operator class"""
    L = G.cuda_lib()
    r = np.random.default_rng(0)
    prompt = r.integers(0, V, T).astype(np.int32)

    def prefill():
        eng.step([("p", prompt, [T - 1])], ["p"])
    for _ in range(3):
        prefill()
    reps = 5
    with ClockSampler(0) as clocks:
        t0 = time.perf_counter()
        for _ in range(reps):
            prefill()
        pf = (time.perf_counter() - t0) / reps
    L.ggb_prof_enable(1)
    G.prof_reset()
    prefill()
    G.sync()
    pf_ops = {k: G.prof_get(k)[0] for k in ops}
    L.ggb_prof_enable(0)
    eng.step([("d", r.integers(0, V, ctx - 1).astype(np.int32), [])])
    eng.generate("d", [1], 8)
    t0 = time.perf_counter()
    eng.generate("d", [2], n_dec)
    dec = (time.perf_counter() - t0) / n_dec
    kernels = eng.stats()["kernels_last_forward"]
    eng.use_graphs(False)
    eng.generate("d", [3], 4)
    L.ggb_prof_enable(1)
    G.prof_reset()
    eng.generate("d", [4], 8)
    G.sync()
    dc_ops = {k: G.prof_get(k)[0] / 8 for k in ops}
    L.ggb_prof_enable(0)
    eng.end("d")
    return pf, pf_ops, dec, dc_ops, kernels, clocks.summary()


def _begupel_record(G, peaks, dims, T, ctx, n_dec):
    """prefill and decode of the Begupel design at the sizes `dims` (a row of BEGUPEL_SIZES) with its roofline fractions"""
    cfg = begupel_config(dims)
    W, nl, H, Gk, D, win, Hr, Gr, Hl, ff, V = dims
    eng = G.Engine(config=cfg, seed=7, dtype="bfloat16", max_tokens=ctx + n_dec + 64, page_size=64, max_portion=1024)
    pf, pf_ops, dec, dc_ops, kernels, clocks = _engine_times(G, eng, V, T, ctx, n_dec, BG_OPS)
    wbytes = eng.stats()["weight_bytes"]
    eng.close()
    lin_params = attn_flops = rec_flops = 0.0
    cache_bytes = state_bytes = 0.0
    visible = float(sum(min(i + 1, win) for i in range(T)))
    for Ly in cfg["layers"]:
        if Ly["type"] == "parallel":
            lin_params += W * (H * D + 2 * Gk * D) + W * H * D + W * (2 * Gr * D + 2 * Hr * D + 2 * Hr) + W * Hr * D
            attn_flops += 4.0 * H * D * visible
            rec_flops += 7.0 * Hr * D * D * T
            cache_bytes += 2.0 * min(ctx, win) * 2 * Gk * D
            state_bytes += 8.0 * Hr * D * D
        else:
            lin_params += W * 4 * Hl * D + W * Hl * D
            rec_flops += 4.0 * Hl * D * D * T
            state_bytes += 8.0 * Hl * D * D
        lin_params += 3.0 * ff * W
    lin_flops = 2.0 * T * lin_params + 2.0 * V * W
    lin_bytes = 2.0 * (lin_params + V * W)
    rec = {
        "config": {"width": W, "layers": nl, "heads": H, "kv_heads": Gk, "dim": D, "window": win, "delta_heads": Hr, "delta_kv_heads": Gr,
                   "lightning_heads": Hl, "ff": ff, "vocab": V, "weight_bytes": wbytes},
        "prefill": {"tokens": T, "tokens_per_s": T / pf, "ms": 1e3 * pf, "op_ms": pf_ops, "clocks": clocks,
                    "linear_tflops": lin_flops / (pf_ops["op_linear"] / 1e3) / 1e12,
                    "linear_frac_of_tensor_peak": lin_flops / (pf_ops["op_linear"] / 1e3) / 1e12 / peaks["bf16_tflops_sustained"],
                    "attn_tflops_cuda_cores": attn_flops / (pf_ops["op_attn"] / 1e3) / 1e12,
                    "recurrence_tflops_cuda_cores": rec_flops / (pf_ops["op_recurrence"] / 1e3) / 1e12},
        "decode": {"n_kv": ctx, "tokens_per_s": 1.0 / dec, "us_per_token": 1e6 * dec, "kernels_per_token": kernels, "op_us": {k: 1e3 * v for k, v in dc_ops.items()},
                   "linear_gbs": lin_bytes / (dc_ops["op_linear"] / 1e3) / 1e9, "linear_frac_of_hbm_peak": lin_bytes / (dc_ops["op_linear"] / 1e3) / 1e9 / peaks["hbm_gbs"],
                   "attn_gbs": cache_bytes / (dc_ops["op_attn"] / 1e3) / 1e9, "recurrence_gbs": state_bytes / (dc_ops["op_recurrence"] / 1e3) / 1e9,
                   "token_frac_of_hbm_roofline": ((lin_bytes + cache_bytes + state_bytes) / (peaks["hbm_gbs"] * 1e9)) / dec},
    }
    return rec


def run_begupel(args):
    """--arch begupel: prefill and decode throughput of the Begupel design (random bf16 weights) at layer sizes of real
    models, through the serving engine (host call: H2D token ids, operator launches / graph replay, D2H result), with
    cudaEvent time per operator class and roofline fractions; beside it Safolorn, the closest model of the framework
    (same engine, same plain bf16 products), at the same width, depth, heads and feed-forward size, all layers dense."""
    import gemma_ggml_b200 as G
    G.init(0)
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    try:
        pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        peaks = {"hbm_gbs": float(pk["hbm_gbs"]), "bf16_tflops_sustained": float(pk["bf16_tflops_sustained"]), "source": "MEASURED_PEAKS.json"}
    except Exception:
        pass
    T, ctx, n_dec = args.prefill_tokens if args.prefill_tokens != 512 else 2048, args.ctx, min(args.steps, 128)
    records = {}
    for size in args.sizes.split(","):
        W, nl, H, Gk, D, win, Hr, Gr, Hl, ff, V = BEGUPEL_SIZES[size]
        rec = _begupel_record(G, peaks, BEGUPEL_SIZES[size], T, ctx, n_dec)
        if not args.no_sub_records:  # Safolorn at equal size: latent attention with heads of the same size, dense feed-forward everywhere
            R = 512 if W >= 2048 else 256
            mx = {"heads": H, "dim": D, "rot_dim": 64, "vdim": D, "kv_rank": R, "scale": (D + 64) ** -0.5,
                  "rot": {"base": 10000.0, "dims": 64, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
            scfg = {"architecture": "Safolorn", "vocab": V, "width": W, "norm": {"eps": 1e-5},
                    "layers": [{"type": "latent_attention", "mixer": mx, "mlp": {"kind": "dense", "ff": ff, "limit": 7.0}} for _ in range(nl)]}
            seng = G.Engine(config=scfg, seed=7, dtype="bfloat16", max_tokens=ctx + n_dec + 64, page_size=64, max_portion=1024)
            spf, spf_ops, sdec, sdc_ops, skernels, _ = _engine_times(G, seng, V, T, ctx, n_dec, BG_OPS)
            s_params = nl * (W * (H * (D + 64) + R + 64) + W * H * D + 3.0 * ff * W)
            s_flops, s_bytes = 2.0 * T * s_params + 2.0 * V * W, 2.0 * (s_params + V * W)
            s_attn = 2.0 * nl * H * (2 * R + 64) * T * (T + 1) / 2
            s_cache = 2.0 * nl * ctx * (R + 64)
            rec["safolorn_equal_size"] = {
                "config": {"kv_rank": R, "rot_dim": 64, "weight_bytes": seng.stats()["weight_bytes"]},
                "prefill": {"tokens_per_s": T / spf, "ms": 1e3 * spf, "op_ms": spf_ops, "linear_tflops": s_flops / (spf_ops["op_linear"] / 1e3) / 1e12,
                            "linear_frac_of_tensor_peak": s_flops / (spf_ops["op_linear"] / 1e3) / 1e12 / peaks["bf16_tflops_sustained"],
                            "attn_tflops_cuda_cores": s_attn / (spf_ops["op_attn"] / 1e3) / 1e12},
                "decode": {"tokens_per_s": 1.0 / sdec, "us_per_token": 1e6 * sdec, "kernels_per_token": skernels, "op_us": {k: 1e3 * v for k, v in sdc_ops.items()},
                           "linear_gbs": s_bytes / (sdc_ops["op_linear"] / 1e3) / 1e9, "linear_frac_of_hbm_peak": s_bytes / (sdc_ops["op_linear"] / 1e3) / 1e9 / peaks["hbm_gbs"],
                           "attn_gbs": s_cache / (sdc_ops["op_attn"] / 1e3) / 1e9,
                           "token_frac_of_hbm_roofline": ((s_bytes + s_cache) / (peaks["hbm_gbs"] * 1e9)) / sdec},
            }
            seng.close()
        records[size] = rec
    first = records[args.sizes.split(",")[0]]
    print(json.dumps({"metric": "begupel decode tokens/s", "value": first["decode"]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
                      "steps": n_dec, "warmup": 8, "ms_per_step": first["decode"]["us_per_token"] / 1e3, "higher_is_better": True,
                      "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random bf16 weights of the configured sizes)",
                      "config": {"workload": "Begupel sizes " + args.sizes + ": prefill of %d tokens, greedy decode at n_kv %d, through the serving engine" % (T, ctx),
                                 "l2": "weights of every size exceed the 126 MB L2"},
                      "peaks": peaks, "sizes": records}), flush=True)


DITALORN_SIZES = {  # width, layers, heads, kv_heads, dim, q_rank, kv_rank, window, experts, top, groups, keep, expert ff, vocab
    "s": (1024, 8, 8, 2, 128, 384, 256, 1024, 16, 2, 4, 2, 1024, 32000),
    "m": (2048, 8, 16, 4, 128, 768, 512, 1024, 32, 4, 8, 4, 1408, 32000),
    "l": (4096, 4, 32, 8, 128, 1536, 512, 2048, 16, 2, 4, 2, 2048, 32000),
}
DL_OPS = ("op_linear", "op_sigmoid_attn", "op_attn", "op_attn_prep", "op_attn_out", "op_conv", "op_moe", "op_moe_linear", "op_norm", "op_act",
          "op_residual", "op_rows")


def ditalorn_config(size, positions):
    """Layers alternate: sigmoid attention over every earlier position, then latent attention over a window; experts everywhere."""
    W, L, H, Gk, D, Rq, R, win, E, top, groups, keep, eff, V = DITALORN_SIZES[size]
    mlp = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}}}
    layers = []
    for i in range(L):
        if i % 2 == 0:
            mx = {"heads": H, "kv_heads": Gk, "dim": D, "vdim": D, "conv": 4, "scale": D ** -0.5, "q_temp": {"coef": 0.1, "every": 256}}
            layers.append({"type": "attention", "mixer": mx, "mlp": mlp})
        else:
            mx = {"heads": H, "dim": D, "vdim": D, "q_rank": Rq, "kv_rank": R, "scale": D ** -0.5, "mask": {"size": win}}
            layers.append({"type": "latent_attention", "mixer": mx, "mlp": mlp})
    return {"architecture": "Ditalorn", "vocab": V, "width": W, "max_positions": positions, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0}, "layers": layers}


def run_ditalorn(args):
    """--arch ditalorn: prefill and decode throughput of the Ditalorn design (random bf16 weights) at layer sizes of real
    models, through the serving engine (host call: H2D token ids, operator launches / graph replay, D2H result), with
    cudaEvent time per operator class and roofline fractions; beside it Safolorn, the closest model of the framework (latent
    attention and experts through the same operators), at the same width, depth, heads, latent and expert sizes."""
    import gemma_ggml_b200 as G
    G.init(0)
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    try:
        pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        peaks = {"hbm_gbs": float(pk["hbm_gbs"]), "bf16_tflops_sustained": float(pk["bf16_tflops_sustained"]), "source": "MEASURED_PEAKS.json"}
    except Exception:
        pass
    T, ctx, n_dec = args.prefill_tokens if args.prefill_tokens != 512 else 2048, args.ctx, min(args.steps, 128)
    records = {}
    for size in args.sizes.split(","):
        W, nl, H, Gk, D, Rq, R, win, E, top, groups, keep, eff, V = DITALORN_SIZES[size]
        cfg = ditalorn_config(size, ctx + n_dec + 64)
        eng = G.Engine(config=cfg, seed=7, dtype="bfloat16", max_tokens=ctx + n_dec + 64, page_size=64, max_portion=1024)
        pf, pf_ops, dec, dc_ops, kernels, clocks = _engine_times(G, eng, V, T, ctx, n_dec, DL_OPS)
        wbytes = eng.stats()["weight_bytes"]
        eng.close()
        n_att, n_lat = (nl + 1) // 2, nl // 2
        vis_all = T * (T + 1) / 2.0
        vis_win = float(sum(min(i + 1, win) for i in range(T)))
        lin_params = n_att * (W * (H * D + 2 * Gk * D) + W * H * D) + n_lat * (W * (Rq + R + H) + Rq * H * D + W * H * D)
        lin_flops, lin_bytes = 2.0 * T * lin_params + 2.0 * V * W, 2.0 * (lin_params + V * W)
        sig_flops = 4.0 * n_att * H * D * vis_all                # q.k and p.v
        # portions take the materialised form when heads are short beside the latent (q.k and p.v over D numbers each, after
        # one product [visible][R] x [H 2D][R]^T per portion); else the absorbed form (qa.c and p.c, R numbers each)
        materialised = 4 * 2 * D <= 5 * R
        vis_rows = sum(min(p0 + 1024, win + 1024 - 1) for p0 in range(0, T, 1024))
        lat_flops = n_lat * (4.0 * H * D * vis_win + 2.0 * vis_rows * R * 2 * H * D) if materialised else 4.0 * n_lat * H * R * vis_win
        moe_flops = 2.0 * T * top * 3 * eff * W * nl
        moe_bytes = 2.0 * top * 3 * eff * W * nl
        sig_cache, lat_cache = 2.0 * n_att * ctx * 2 * Gk * D, 2.0 * n_lat * min(ctx, win) * R
        rec = {
            "config": {"width": W, "layers": nl, "heads": H, "kv_heads": Gk, "dim": D, "q_rank": Rq, "kv_rank": R, "window": win, "experts": E, "top": top,
                       "groups": [groups, keep], "expert_ff": eff, "vocab": V, "weight_bytes": wbytes},
            "prefill": {"tokens": T, "tokens_per_s": T / pf, "ms": 1e3 * pf, "op_ms": pf_ops, "clocks": clocks,
                        "linear_tflops": lin_flops / (pf_ops["op_linear"] / 1e3) / 1e12,
                        "linear_frac_of_tensor_peak": lin_flops / (pf_ops["op_linear"] / 1e3) / 1e12 / peaks["bf16_tflops_sustained"],
                        "moe_linear_tflops": moe_flops / (pf_ops["op_moe_linear"] / 1e3) / 1e12,
                        "sigmoid_attn_tflops_cuda_cores": sig_flops / (pf_ops["op_sigmoid_attn"] / 1e3) / 1e12,
                        "latent_attn_form": "materialised" if materialised else "absorbed",
                        "latent_attn_tflops": lat_flops / ((pf_ops["op_attn"] + (pf_ops["op_attn_prep"] if materialised else 0.0)) / 1e3) / 1e12},
            "decode": {"n_kv": ctx, "tokens_per_s": 1.0 / dec, "us_per_token": 1e6 * dec, "kernels_per_token": kernels, "op_us": {k: 1e3 * v for k, v in dc_ops.items()},
                       "linear_gbs": lin_bytes / (dc_ops["op_linear"] / 1e3) / 1e9, "linear_frac_of_hbm_peak": lin_bytes / (dc_ops["op_linear"] / 1e3) / 1e9 / peaks["hbm_gbs"],
                       "moe_linear_gbs": moe_bytes / (dc_ops["op_moe_linear"] / 1e3) / 1e9,
                       "sigmoid_attn_gbs": sig_cache / (dc_ops["op_sigmoid_attn"] / 1e3) / 1e9, "latent_attn_gbs": lat_cache / (dc_ops["op_attn"] / 1e3) / 1e9,
                       "token_frac_of_hbm_roofline": ((lin_bytes + moe_bytes + sig_cache + lat_cache) / (peaks["hbm_gbs"] * 1e9)) / dec},
        }
        if not args.no_sub_records:  # Safolorn at equal size: latent attention in every layer, the same experts
            mx = {"heads": H, "dim": D, "rot_dim": 64, "vdim": D, "kv_rank": R, "scale": (D + 64) ** -0.5,
                  "rot": {"base": 10000.0, "dims": 64, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
            scfg = {"architecture": "Safolorn", "vocab": V, "width": W, "norm": {"eps": 1e-5},
                    "layers": [{"type": "latent_attention", "mixer": mx, "mlp": {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "top": top}}} for _ in range(nl)]}
            seng = G.Engine(config=scfg, seed=7, dtype="bfloat16", max_tokens=ctx + n_dec + 64, page_size=64, max_portion=1024)
            spf, spf_ops, sdec, sdc_ops, skernels, _ = _engine_times(G, seng, V, T, ctx, n_dec, DL_OPS)
            s_params = nl * (W * (H * (D + 64) + R + 64) + W * H * D)
            s_flops, s_bytes = 2.0 * T * s_params + 2.0 * V * W, 2.0 * (s_params + V * W)
            s_attn = 2.0 * nl * H * (2 * R + 64) * vis_all
            s_moe_flops, s_moe_bytes = 2.0 * T * top * 2 * eff * W * nl, 2.0 * top * 2 * eff * W * nl  # experts without a gate: up and down
            s_cache = 2.0 * nl * ctx * (R + 64)
            rec["safolorn_equal_size"] = {
                "config": {"weight_bytes": seng.stats()["weight_bytes"]},
                "prefill": {"tokens_per_s": T / spf, "ms": 1e3 * spf, "op_ms": spf_ops, "linear_tflops": s_flops / (spf_ops["op_linear"] / 1e3) / 1e12,
                            "linear_frac_of_tensor_peak": s_flops / (spf_ops["op_linear"] / 1e3) / 1e12 / peaks["bf16_tflops_sustained"],
                            "moe_linear_tflops": s_moe_flops / (spf_ops["op_moe_linear"] / 1e3) / 1e12,
                            "latent_attn_tflops_cuda_cores": s_attn / (spf_ops["op_attn"] / 1e3) / 1e12},
                "decode": {"tokens_per_s": 1.0 / sdec, "us_per_token": 1e6 * sdec, "kernels_per_token": skernels, "op_us": {k: 1e3 * v for k, v in sdc_ops.items()},
                           "linear_gbs": s_bytes / (sdc_ops["op_linear"] / 1e3) / 1e9, "linear_frac_of_hbm_peak": s_bytes / (sdc_ops["op_linear"] / 1e3) / 1e9 / peaks["hbm_gbs"],
                           "moe_linear_gbs": s_moe_bytes / (sdc_ops["op_moe_linear"] / 1e3) / 1e9,
                           "latent_attn_gbs": s_cache / (sdc_ops["op_attn"] / 1e3) / 1e9,
                           "token_frac_of_hbm_roofline": ((s_bytes + s_moe_bytes + s_cache) / (peaks["hbm_gbs"] * 1e9)) / sdec},
            }
            seng.close()
        records[size] = rec
    first = records[args.sizes.split(",")[0]]
    print(json.dumps({"metric": "ditalorn decode tokens/s", "value": first["decode"]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
                      "steps": n_dec, "warmup": 8, "ms_per_step": first["decode"]["us_per_token"] / 1e3, "higher_is_better": True,
                      "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random bf16 weights of the configured sizes)",
                      "config": {"workload": "Ditalorn sizes " + args.sizes + ": prefill of %d tokens, greedy decode at n_kv %d, through the serving engine" % (T, ctx),
                                 "l2": "weights of every size exceed the 126 MB L2"},
                      "peaks": peaks, "sizes": records}), flush=True)


KIBILIX_SIZES = {  # width, layers, heads, kv heads, head size, chunk, delta heads, delta kv heads, dense ff, experts, identity, top, expert ff, vocab
    "s": (1024, 8, 8, 2, 128, 1024, 8, 4, 4096, 16, 2, 2, 1024, 32000),
    "m": (2048, 8, 16, 4, 128, 1024, 16, 8, 8192, 32, 2, 4, 1408, 32000),
    "l": (4096, 4, 32, 8, 128, 2048, 32, 16, 12288, 16, 2, 2, 2048, 32000),
}
KB_OPS = ("op_linear", "op_attn", "op_attn_prep", "op_recurrence", "op_conv", "op_norm", "op_act", "op_residual", "op_rows", "op_moe", "op_moe_linear")
KB_RANK, KB_STREAMS = 64, 4


def kibilix_config(size):
    """Layers alternate: a delta rule with per-channel decay, then chunked attention; the feed-forward is dense in the first
    layer of every four and a mixture of experts with identity experts in the third; four residual streams."""
    W, L, H, G, D, chunk, Hr, Gr, ff, E, I, top, eff, V = KIBILIX_SIZES[size]
    layers = []
    for i in range(L):
        if i % 2 == 0:
            mx = {"heads": Hr, "kv_heads": Gr, "dim": D, "vdim": D, "conv": 4, "rank": KB_RANK}
            kind = "channel_delta"
        else:
            mx = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "softcap": 30.0, "mask": {"size": chunk},
                  "rot": {"base": 500000.0, "dims": D // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
            kind = "attention"
        mlp = {"kind": "dense", "ff": ff} if i % 4 < 2 else {"kind": "moe", "expert": {"ff": eff, "limit": 7.0}, "router": {"experts": E, "identity": I, "top": top}}
        layers.append({"type": kind, "mixer": mx, "mlp": mlp})
    return {"architecture": "Kibilix", "vocab": V, "width": W, "norm": {"eps": 1e-5}, "residual_mult": 0.7, "streams": KB_STREAMS,
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 131, "mul_cur": 31}}, "layers": layers}


def run_kibilix(args):
    """--arch kibilix: prefill and decode throughput of the Kibilix design (random bf16 weights) at layer sizes of real
    models, through the serving engine (host call: H2D token ids, operator launches / graph replay, D2H result), with
    cudaEvent time per operator class and roofline fractions; beside it Begupel, the closest model of the framework
    (the same engine, products, cache and state blocks; window attention and a delta rule with one decay per head), at the
    same width, depth, heads and dense feed-forward size."""
    import gemma_ggml_b200 as G
    G.init(0)
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    try:
        pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        peaks = {"hbm_gbs": float(pk["hbm_gbs"]), "bf16_tflops_sustained": float(pk["bf16_tflops_sustained"]), "source": "MEASURED_PEAKS.json"}
    except Exception:
        pass
    T, ctx, n_dec = args.prefill_tokens if args.prefill_tokens != 512 else 2048, args.ctx, min(args.steps, 128)
    records = {}
    for size in args.sizes.split(","):
        cfg = kibilix_config(size)
        W, nl, H, Gk, D, chunk, Hr, Gr, ff, E, I, top, eff, V = KIBILIX_SIZES[size]
        eng = G.Engine(config=cfg, seed=7, dtype="bfloat16", max_tokens=ctx + n_dec + 64, page_size=64, max_portion=1024)
        pf, pf_ops, dec, dc_ops, kernels, clocks = _engine_times(G, eng, V, T, ctx, n_dec, KB_OPS)
        wbytes = eng.stats()["weight_bytes"]
        eng.close()
        lin_params = attn_flops = rec_flops = exp_params = 0.0
        cache_bytes = state_bytes = stream_bytes = 0.0
        visible = float(sum(i % chunk + 1 for i in range(T)))
        real = top * E / float(E + I)  # slots of a token that reach an expert with matrices, if the router chose evenly
        for Ly in cfg["layers"]:
            if Ly["type"] == "attention":
                lin_params += W * (H * D + 2 * Gk * D) + W * H * D
                attn_flops += 4.0 * H * D * visible
                cache_bytes += 2.0 * ((ctx - 1) % chunk + 1) * 2 * Gk * D
            else:
                lin_params += W * (2 * Gr * D + Hr * D + Hr + 2 * KB_RANK) + 2.0 * KB_RANK * Hr * D + W * Hr * D
                rec_flops += 7.0 * Hr * D * D * T
                state_bytes += 8.0 * Hr * D * D
            if Ly["mlp"]["kind"] == "dense":
                lin_params += 2.0 * ff * W
            else:
                exp_params += real * 3.0 * eff * W
            stream_bytes += 2 * (2 * KB_STREAMS + 1) * W * 4.0   # two passes over the streams per layer: read, write, one output
        lin_flops = 2.0 * T * lin_params + 2.0 * V * W
        lin_bytes = 2.0 * (lin_params + V * W)
        exp_flops, exp_bytes = 2.0 * T * exp_params, 2.0 * exp_params
        rec = {
            "config": {"width": W, "layers": nl, "heads": H, "kv_heads": Gk, "dim": D, "chunk": chunk, "delta_heads": Hr, "delta_kv_heads": Gr, "rank": KB_RANK,
                       "streams": KB_STREAMS, "ff": ff, "experts": E, "identity": I, "top": top, "expert_ff": eff, "vocab": V, "weight_bytes": wbytes},
            "prefill": {"tokens": T, "tokens_per_s": T / pf, "ms": 1e3 * pf, "op_ms": pf_ops, "clocks": clocks,
                        "linear_tflops": lin_flops / (pf_ops["op_linear"] / 1e3) / 1e12,
                        "linear_frac_of_tensor_peak": lin_flops / (pf_ops["op_linear"] / 1e3) / 1e12 / peaks["bf16_tflops_sustained"],
                        "experts_tflops": exp_flops / (pf_ops["op_moe_linear"] / 1e3) / 1e12,
                        "attn_tflops_cuda_cores": attn_flops / (pf_ops["op_attn"] / 1e3) / 1e12,
                        "recurrence_tflops_cuda_cores": rec_flops / (pf_ops["op_recurrence"] / 1e3) / 1e12,
                        "streams_gbs": T * stream_bytes / (pf_ops["op_residual"] / 1e3) / 1e9},
            "decode": {"n_kv": ctx, "tokens_per_s": 1.0 / dec, "us_per_token": 1e6 * dec, "kernels_per_token": kernels, "op_us": {k: 1e3 * v for k, v in dc_ops.items()},
                       "linear_gbs": lin_bytes / (dc_ops["op_linear"] / 1e3) / 1e9, "linear_frac_of_hbm_peak": lin_bytes / (dc_ops["op_linear"] / 1e3) / 1e9 / peaks["hbm_gbs"],
                       "experts_gbs": exp_bytes / (dc_ops["op_moe_linear"] / 1e3) / 1e9,
                       "attn_gbs": cache_bytes / (dc_ops["op_attn"] / 1e3) / 1e9, "recurrence_gbs": state_bytes / (dc_ops["op_recurrence"] / 1e3) / 1e9,
                       "token_frac_of_hbm_roofline": ((lin_bytes + exp_bytes + cache_bytes + state_bytes) / (peaks["hbm_gbs"] * 1e9)) / dec},
        }
        if not args.no_sub_records:  # Begupel at equal size: window = chunk, the same delta heads, as many lightning heads as attention heads
            rec["begupel_equal_size"] = _begupel_record(G, peaks, (W, nl, H, Gk, D, chunk, Hr, Gr, H, ff, V), T, ctx, n_dec)
        records[size] = rec
    first = records[args.sizes.split(",")[0]]
    print(json.dumps({"metric": "kibilix decode tokens/s", "value": first["decode"]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
                      "steps": n_dec, "warmup": 8, "ms_per_step": first["decode"]["us_per_token"] / 1e3, "higher_is_better": True,
                      "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random bf16 weights of the configured sizes)",
                      "config": {"workload": "Kibilix sizes " + args.sizes + ": prefill of %d tokens, greedy decode at n_kv %d, through the serving engine" % (T, ctx),
                                 "l2": "weights of every size exceed the 126 MB L2"},
                      "peaks": peaks, "sizes": records}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", default="gemma", choices=["gemma", "safolorn", "begupel", "ditalorn", "kibilix"],
                    help="gemma: the headline workload (default); safolorn: throughput of the Safolorn design beside Gemma at equal size; "
                         "begupel: throughput of the Begupel design beside Safolorn at equal size; ditalorn: the Ditalorn design beside Safolorn at equal size; kibilix: the Kibilix design beside Begupel at equal size")
    ap.add_argument("--sizes", default="s,m,l", help="--arch safolorn / begupel / ditalorn / kibilix: which of the sizes s, m, l to run")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="2b", choices=list(MODELS))
    ap.add_argument("--wtype", default="q4_0", choices=list(WTYPES))
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--mode", default="fused", choices=["fused", "ops", "prefill"])
    ap.add_argument("--prefill-tokens", type=int, default=512)
    ap.add_argument("--cpu-tokens", type=int, default=16)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sub-records", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.arch == "safolorn":
        run_safolorn(args)
    elif args.arch == "begupel":
        run_begupel(args)
    elif args.arch == "ditalorn":
        run_ditalorn(args)
    elif args.arch == "kibilix":
        run_kibilix(args)
    elif args.mode == "prefill":
        run_prefill(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
