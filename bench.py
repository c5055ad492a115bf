#!/usr/bin/env python
"""Benchmark of the batched paged-KV decode step: Llama-2-7B-shaped Q4_0, B=64 per GPU.

    python bench.py --gpus N --steps K --warmup W            (N>1: launched with torch.distributed.run)
    python bench.py --impl reference ...                     (the CPU port of the reference path, bounded sample)

A step = one decode step of the whole ragged batch (one new token per sequence).  Every GPU holds a full
model replica and its own block pool and serves its own B sequences (request sharding, no collective on the
data path), so per-GPU work is fixed as N grows: weak scaling.  Inputs are synthetic: seeded random Q4_0
weights of the named shape generated on the device, KV pages pre-filled with fp16 noise on shuffled physical
blocks, context lengths ~U[128, 2048].  One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from vexel_b200 import capi, gguf_synth as gs, replicas  # noqa: E402

NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one paged_flash_kernel launch divided by its algorithmic bytes,
# from the ncu capture summarised in profiles/ (None until a capture has been taken)
ATTN_TRAFFIC_RATIO = 1.0137   # profiles/paged_flash_kernel_llama2-7b_B64.md: 1.2256 GB DRAM traffic / 1.2090 GB algorithmic (traffic grows with the KV bytes)

WORKLOADS = {
    "llama2-7b-q4_0": gs.C2_LLAMA2_7B,
    "tinyllama-1.1b-q4_0": gs.C1_TINYLLAMA,
    "llama3-8b-q4_k_m": gs.C3_LLAMA3_8B,
    "gemma2-9b-q6_k": gs.C4_GEMMA2_9B,
    "llama3-70b-q4_k_m": gs.C5_LLAMA3_70B,
}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                                       "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.p is None:
            return out
        time.sleep(0.15)
        self.p.terminate()          # the exact process started above
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush(); self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.f.close()
        try:
            os.unlink(self.f.name)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm))
        return out


def cpu_baseline(spec, seconds_target=15.0, sample_layers=2, sample_seqs=4, ctx=1088, threads=None):
    """The CPU port of the reference's decode path (oracle/), timed on this host's cores on a bounded sample:
    `sample_layers` layers + the output head of the named shape, `sample_seqs` sequences at context `ctx`, decoded one
    sequence at a time as the reference's batched path does (runtime/decode.go:623-654).  Layer time is scaled to the
    full depth.  Random Q4_0 bytes stand in for the weights (timing does not depend on the values)."""
    from oracle import oracle as O
    threads = threads or os.cpu_count() or 1
    O.lib().vo_set_threads(threads)
    rng = np.random.default_rng(0)
    small = gs.scaled(spec, sample_layers, spec.hidden, spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.ffn, spec.vocab)
    max_blocks = sample_seqs * ((ctx + 64) // 16 + 2)
    cfg = O.Config(n_layers=small.n_layers, hidden=small.hidden, n_heads=small.n_heads, n_kv_heads=small.n_kv_heads,
                   head_dim=small.head_dim, ffn=small.ffn, vocab=small.vocab, rms_eps=small.rms_eps, rope_theta=small.rope_theta,
                   rope_neox=0, geglu=0, post_norms=0, embed_scale=0.0, attn_softcap=0.0, final_softcap=0.0, sliding_window=0,
                   window_alternating=0, max_blocks=max_blocks, kv_f16=1)
    om = O.Model(cfg)

    def rand_q4(n, k):
        raw = rng.integers(0, 256, (n, k // 32, 18), dtype=np.uint8)
        raw[:, :, 0:2] = np.array([0.0045], np.float16).view(np.uint8)     # d ~ 0.02 * 1.8 / 8
        return raw

    ones = np.ones(spec.hidden, np.float32)
    om.set_global(O.G_EMBED, O.Q4_0, rand_q4(spec.vocab, spec.hidden))
    om.set_global(O.G_OUTPUT, O.Q4_0, rand_q4(spec.vocab, spec.hidden))
    om.set_global(O.G_FINAL_NORM, O.F32, ones)
    slots = {O.T_WQ: capi.W_WQ, O.T_WK: capi.W_WK, O.T_WV: capi.W_WV, O.T_WO: capi.W_WO, O.T_W1: capi.W_W1, O.T_W3: capi.W_W3, O.T_W2: capi.W_W2}
    for layer in range(sample_layers):
        om.set_layer(layer, O.T_ATTN_NORM, O.F32, ones); om.set_layer(layer, O.T_FFN_NORM, O.F32, ones)
        for oslot, gslot in slots.items():
            n, k = gs.slot_shape(spec, gslot)
            om.set_layer(layer, oslot, O.Q4_0, rand_q4(n, k))
    kvd = spec.n_kv_heads * spec.head_dim
    kv = (rng.random((ctx, kvd), dtype=np.float32) - 0.5) * 0.2
    for s in range(sample_seqs):
        om.pool.create_seq(s + 1)
        for layer in range(sample_layers):
            om.pool.store_kv(layer, s + 1, 0, kv, kv, ctx)
    import ctypes as C
    L = O.lib()
    tok = np.int32([7])
    logits = np.empty((1, spec.vocab), np.float32)

    def run(with_head, pos):
        t0 = time.perf_counter()
        for s in range(sample_seqs):
            L.vo_model_forward(om.h, s + 1, tok.ctypes.data_as(C.c_void_p), 1, pos, 0,
                               logits.ctypes.data_as(C.c_void_p) if with_head else None, None)
        return time.perf_counter() - t0

    t_layers, t_total, steps, pos = [], [], 0, ctx
    t_begin = time.perf_counter()
    while steps < 1 or (time.perf_counter() - t_begin) < seconds_target * 0.6:
        t_layers.append(run(False, pos)); pos += 1
        t_total.append(run(True, pos)); pos += 1
        steps += 1
        if steps >= 8:
            break
    tl, tt = min(t_layers), min(t_total)
    t_head = max(tt - tl, 0.0)
    per_token = (tl / sample_layers * spec.n_layers + t_head) / sample_seqs
    return {"value": 1.0 / per_token, "unit": "tok/s", "cores": threads, "kind": "port",
            "sample": f"{sample_layers} of {spec.n_layers} layers + output head of the {spec.name} shape, {sample_seqs} sequences at context {ctx}, "
                      f"{steps} timed decode steps, layer time scaled to {spec.n_layers} layers; C port of the reference CPU path "
                      f"(inference/backend/cpu/cpu.go arithmetic, sequences decoded one at a time), OpenMP over output elements"}


def dist_setup(n_gpus):
    world, rank, local = replicas.rank_env()
    return world, rank, local, replicas.init("nccl", local)


def reference_arm(args):
    """Times the CPU port of the reference's path with all host threads, on a bounded sample of the same workload."""
    world, rank, _ = replicas.rank_env()
    if rank != 0:
        return
    spec = WORKLOADS[args.workload]
    vals = []
    base = None
    for _ in range(max(1, min(args.steps, 3))):
        base = cpu_baseline(spec, seconds_target=20.0)
        vals.append(base["value"])
    v = float(np.median(vals))
    base["value"] = v
    line = {"impl": "reference", "metric": "decode tok/s", "value": v, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": args.batch / v * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": f"{spec.name} batched decode B={args.batch}, ctx~U[128,2048], 16-token pages"},
            "cpu_baseline": base, "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def trace_arm(args):
    """Continuous batching under staggered arrivals: a synthetic Poisson trace (prompt lengths log-normal around 512, outputs
    U[32,512], random token ids) replayed through the scheduler with max batch 256 on one GPU; prints one JSON line."""
    from vexel_b200 import trace as tr
    spec = WORKLOADS[args.workload]
    if args.layers > 0:
        spec = gs.scaled(spec, args.layers, spec.hidden, spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.ffn, spec.vocab)
    max_ctx = args.trace_max_prompt + 512 + 16
    arrivals, prompts, olen = tr.make_trace(args.trace, args.trace_rate, spec.vocab, seed=4, prompt_clip=(16, args.trace_max_prompt))
    be = capi.Backend(0)
    kv_block_bytes = spec.kv_bytes_per_token() * 16
    max_blocks = int(min(120e9 // kv_block_bytes, 256 * (max_ctx // 16 + 2)))         # as much pool as ~120 GB allows; admission handles the rest
    model = capi.Model(be, gs.model_config(spec, max_blocks, max_seqs=256, max_batch_tokens=256, max_blocks_per_seq=max_ctx // 16 + 2))
    gs.synth_weights_on_device(be, model, spec, seed=0)
    res = tr.replay(model, arrivals, prompts, olen, max_batch=256)
    line = {"metric": "trace decode tok/s", "value": res["tok_per_s"], "unit": "tok/s", "n_gpus": 1, "higher_is_better": True, "data": "synthetic",
            "config": {"workload": f"{spec.name}: {args.trace} requests, Poisson {args.trace_rate}/s, prompts lognormal(ln 512, 0.8) clipped to "
                                   f"[16,{args.trace_max_prompt}], outputs U[32,512], max batch 256, pool {max_blocks} blocks"},
            "trace": res}
    emit(line)
    model.close(); be.close()


_RESULT_FD = None


def claim_stdout():
    """Keeps the process's stdout for the one result line: everything else that writes to file descriptor 1 (libraries that
    print a banner from native code, child processes) is sent to stderr from here on."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode()); sys.stdout.flush()
    else:
        sys.stdout.flush()
        os.write(_RESULT_FD, data)


def main():
    claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="llama2-7b-q4_0", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=64, help="sequences per GPU")
    ap.add_argument("--ctx-min", type=int, default=128)
    ap.add_argument("--ctx-max", type=int, default=2048)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiling on a small case)")
    ap.add_argument("--trace", type=int, default=0, help="replay a Poisson arrival trace of this many requests through the scheduler instead of the fixed-batch steps")
    ap.add_argument("--trace-rate", type=float, default=40.0, help="trace arrivals per second")
    ap.add_argument("--trace-max-prompt", type=int, default=8192)
    ap.add_argument("--no-dependent-launch", action="store_true", help="experiment: projections in plain stream order instead of as programmatic dependents")
    ap.add_argument("--no-graphs", action="store_true", help="experiment: launch every kernel individually instead of replaying CUDA graphs")
    ap.add_argument("--tc-min-rows", type=int, default=-1, help="experiment: batch size from which projections use the tcgen05 kernel")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    if args.trace > 0:
        return trace_arm(args)
    world, rank, local, dist = dist_setup(args.gpus)
    spec = WORKLOADS[args.workload]
    if args.layers > 0:
        spec = gs.scaled(spec, args.layers, spec.hidden, spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.ffn, spec.vocab)
    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    seeds = replicas.rank_seeds(rank)
    rng = np.random.default_rng(seeds["workload"])
    ctx = rng.integers(args.ctx_min, args.ctx_max + 1, B)
    total_new = W + 2 * K + 16                      # warm-up + device-resident leg + projection leg (the end-to-end leg rolls back)
    blocks_per_seq = int((args.ctx_max + total_new) // 16 + 2)
    max_blocks = int(sum((c + total_new) // 16 + 2 for c in ctx) + 64)

    be = capi.Backend(local)
    if args.tc_min_rows >= 0:
        be.lib.vx_set_tc_min_rows(args.tc_min_rows)
    if args.no_dependent_launch:
        be.lib.vx_set_dependent_launch(0)
    if args.no_graphs:
        be.lib.vx_set_graphs(0)
    model = capi.Model(be, gs.model_config(spec, max_blocks, max_seqs=B, max_batch_tokens=max(B, 8), max_blocks_per_seq=blocks_per_seq))
    gs.synth_weights_on_device(be, model, spec, seed=seeds["weights"])
    model.shuffle_free_list(seeds["free_list"])               # physical blocks shuffled randomly in the pool
    seqs = np.arange(1, B + 1, dtype=np.int64)
    for i, s in enumerate(seqs):
        model.seq_fill_synthetic(int(s), int(ctx[i]), seed=seeds["kv_fill"] + i)
    tokens = rng.integers(0, spec.vocab, B).astype(np.int32)
    pos = ctx.astype(np.int32).copy()

    # ---- warm-up (W >= 3 steps), then K timed steps with the tokens fed back on the device
    out, _ = model.decode_run(seqs, tokens, pos, W)
    tokens = out[-1].copy(); pos += W
    replicas.barrier(dist)
    sampler = ClockSampler(local) if rank == 0 else None
    l0, s0 = model.counters()
    # CUDA events around every launch of the dominant kernel (paged attention) during the timed steps; the projections are
    # timed in a short leg of their own afterwards, because five more event pairs per layer cost the step ~6 %
    model.kernel_time(0, 1); model.kernel_time(1, 0)
    # sum over the K timed steps and the sequences of the attended length, for global layers and for sliding-window layers
    kv_tokens_global = float(sum(int(p) * K + K * (K + 1) // 2 for p in pos))
    n_slide = spec.n_layers // 2 if (spec.window_alternating and spec.sliding_window > 0) else 0   # odd layers slide
    kv_tokens_slide = float(sum(min(int(p) + j, spec.sliding_window) for p in pos for j in range(1, K + 1))) if n_slide else 0.0
    kv_tokens_timed = ((spec.n_layers - n_slide) * kv_tokens_global + n_slide * kv_tokens_slide) / spec.n_layers   # per-layer mean
    pos_timed, tokens_timed = pos.copy(), tokens.copy()       # where the timed leg starts: the end-to-end leg starts there again
    out, dev_ms = model.decode_run(seqs, tokens, pos, K)
    attn_ms, attn_n = model.kernel_time(0, 0)
    l1, s1 = model.counters()
    clocks = sampler.stop() if sampler else None
    tokens = out[-1].copy(); pos += K
    Kg = min(K, 8)
    model.kernel_time(1, 1)
    out, _ = model.decode_run(seqs, tokens, pos, Kg)
    gemm_ms, gemm_n = model.kernel_time(1, 0)
    gemm_ms = gemm_ms / Kg * K            # scaled to the K timed steps for the shares below
    tokens = out[-1].copy(); pos += Kg
    replicas.barrier(dist)
    value, max_s = replicas.job_throughput(dist, B * K, dev_ms / 1e3, local)
    max_ms = max_s * 1e3

    # ---- end to end through vx_decode_step: host token ids in, host tokens out, every step
    e2e = None
    if not args.no_e2e:
        # the same K steps over the same contexts as the device-timed leg: the sequences are rolled back to where it began
        # (TruncateSequence, gpu_block_pool.go:162-190) and fed the same first tokens
        for i, sq in enumerate(seqs):
            model.seq_truncate(int(sq), int(pos_timed[i]))
        pos = pos_timed.copy(); tokens = tokens_timed
        replicas.barrier(dist)
        be.Sync()
        t0 = time.perf_counter()
        cur = tokens
        for _ in range(K):
            cur = model.decode_step(seqs, cur, pos)
            pos += 1
        be.Sync()
        e2e_v, e2e_s = replicas.job_throughput(dist, B * K, time.perf_counter() - t0, local)
        e2e = {"value": e2e_v, "unit": "tok/s", "h2d_bytes_per_step": int(4 * B * 4), "d2h_bytes_per_step": int(4 * B + 4),
               "ms_per_step": e2e_s / K * 1e3}

    if rank != 0:
        model.close(); be.close()
        replicas.shutdown(dist)
        return

    # ---- roofline of the dominant kernel (paged attention) and of the whole step
    peak, peak_kind = measured_peak()
    kv_bytes_per_token_layer = 2 * spec.n_kv_heads * spec.head_dim * 2             # K and V, fp16
    attn_bytes_per_launch = kv_tokens_timed * kv_bytes_per_token_layer / K         # one launch = one layer of one step
    attn_launch_ms = attn_ms / max(attn_n, 1)
    attn_gbs = attn_bytes_per_launch / (attn_launch_ms * 1e-3) / 1e9 if attn_n else None
    W_bytes = model.weight_bytes()
    bytes_step = W_bytes + kv_tokens_timed / K * kv_bytes_per_token_layer * spec.n_layers + B * spec.n_layers * kv_bytes_per_token_layer
    step_gbs = bytes_step / (max_ms / K * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "paged_flash_kernel (+merge), one launch per layer", "achieved": attn_gbs, "peak": peak, "unit": "GB/s",
                "frac": (attn_gbs / peak) if attn_gbs else None, "peak_source": f"{peak_kind} copy bandwidth",
                "traffic": (ATTN_TRAFFIC_RATIO * attn_bytes_per_launch) if ATTN_TRAFFIC_RATIO else None,
                "algorithmic_bytes_per_launch": attn_bytes_per_launch, "launch_ms": attn_launch_ms,
                "share_of_step": attn_ms / dev_ms if dev_ms else None,
                "projections": {"timed_in": "a separate leg of %d steps right after the timed region" % Kg, "launch_ms_total_per_step": gemm_ms / K, "share_of_step": gemm_ms / dev_ms if dev_ms else None,
                                "weight_bytes": W_bytes, "achieved_GBs": W_bytes / (gemm_ms / K * 1e-3) / 1e9 if gemm_ms else None}}
    line = {"metric": "decode tok/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": max_ms / K,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 activations, %s weights, f16 kv" % spec.quant,
            "data": "synthetic",
            "config": {"workload": f"{spec.name} batched decode, B={B} per GPU, ctx~U[{args.ctx_min},{args.ctx_max}] + generated, 16-token pages, shuffled blocks",
                       "global_batch": world * B, "parallelism": f"replicas x{world} (request sharding, no collective)",
                       "l2": "inputs larger than L2: each step streams %.1f GB of weights+KV" % (bytes_step / 1e9),
                       "timing": "CUDA events on the launching stream around K steps with on-device token feedback; max over ranks"},
            "roofline": roofline,
            "step_roofline": {"bytes_per_step": bytes_step, "achieved_GBs": step_gbs, "frac_of_measured": step_gbs / peak,
                              "frac_of_nominal_8TBs": step_gbs / NOMINAL_HBM_GBS,
                              "roofline_tok_s_measured": B / (bytes_step / (peak * 1e9)), "roofline_tok_s_nominal": B / (bytes_step / (NOMINAL_HBM_GBS * 1e9))},
            "clocks": clocks, "gpu_launches": int(l1 - l0), "e2e": e2e}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(spec)
    emit(line)
    model.close(); be.close()
    replicas.shutdown(dist)


if __name__ == "__main__":
    main()
