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
# dram__bytes_read.sum + dram__bytes_write.sum of one paged attention launch divided by its algorithmic bytes, from one ncu
# capture of a smaller case of the same kernel (1.2256 GB of DRAM traffic for 1.2090 GB of KV); the traffic grows in
# proportion to the KV bytes, so the figure reported per run is this ratio times the launch's algorithmic bytes
ATTN_TRAFFIC_RATIO = 1.0137

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


class CpuPort:
    """The CPU port of the reference's decode path (oracle/) set up for timing: the named shape at FULL depth when its
    weights are Q4_0 (the reference multiplies those straight from the blocks, backend/cpu/cpu.go:842-911), `n_seqs`
    sequences with contexts drawn like the benchmark's, decoded one sequence at a time as the reference's batched path does
    (runtime/decode.go:623-654) -- so its tok/s does not depend on how many sequences share a step.  K-quant shapes would need
    their float32 expansion (the reference's CPU route for them, runtime/loader.go:214-271), which for the larger models does
    not fit a host: those keep a `layers`-deep slice and scale its layer time.  Random block bytes stand in for the weights
    and a repeated noise pattern for the KV pages: timing does not depend on the values."""

    def __init__(self, spec, n_seqs, ctx_min, ctx_max, threads=None, slice_layers=2):
        from oracle import oracle as O
        self.O, self.spec = O, spec
        self.threads = threads or os.cpu_count() or 1
        O.lib().vo_set_threads(self.threads)
        rng = np.random.default_rng(0)
        self.full_depth = spec.quant == "q4_0"
        self.layers = spec.n_layers if self.full_depth else min(slice_layers, spec.n_layers)
        self.ctx = np.random.default_rng(replicas.GLOBAL_WORKLOAD_SEED).integers(ctx_min, ctx_max + 1, n_seqs)
        max_blocks = int(sum((int(c) + 4096) // 16 + 2 for c in self.ctx))
        cfg = O.Config(n_layers=self.layers, hidden=spec.hidden, n_heads=spec.n_heads, n_kv_heads=spec.n_kv_heads,
                       head_dim=spec.head_dim, ffn=spec.ffn, vocab=spec.vocab, rms_eps=spec.rms_eps, rope_theta=spec.rope_theta,
                       rope_neox=0, geglu=int(spec.geglu), post_norms=int(spec.post_norms), embed_scale=spec.embed_scale,
                       attn_softcap=spec.attn_softcap, final_softcap=spec.final_softcap, sliding_window=spec.sliding_window,
                       window_alternating=int(spec.window_alternating), max_blocks=max_blocks, kv_f16=1)
        self.om = om = O.Model(cfg)
        proj_types, _, out_type = gs.tensor_types(spec)
        blk = {capi.T_Q4_0: (32, 18), capi.T_Q4_K: (256, 144), capi.T_Q6_K: (256, 210)}

        def rand_blocks(n, k, t):
            per, nbytes = blk[t]
            raw = rng.integers(0, 256, (n, k // per, nbytes), dtype=np.uint8)
            d = np.array([0.0045 if t == capi.T_Q4_0 else 0.0003], np.float16).view(np.uint8)     # block scales of N(0, 0.02) weights
            if t == capi.T_Q6_K: raw[:, :, 208:210] = d
            else: raw[:, :, 0:2] = d
            if t == capi.T_Q4_K: raw[:, :, 2:4] = d
            return raw

        ones = np.ones(spec.hidden, np.float32)
        om.set_global(capi.G_EMBED, capi.T_Q4_0, rand_blocks(spec.vocab, spec.hidden, capi.T_Q4_0))
        om.set_global(capi.G_OUTPUT, out_type, rand_blocks(spec.vocab, spec.hidden, out_type))
        om.set_global(capi.G_FINAL_NORM, capi.T_F32, ones)
        for layer in range(self.layers):
            for slot in (capi.W_ATTN_NORM, capi.W_FFN_NORM) + ((capi.W_POST_ATTN_NORM, capi.W_POST_FFN_NORM) if spec.post_norms else ()):
                om.set_layer(layer, slot, capi.T_F32, ones)
            for slot in (capi.W_WQ, capi.W_WK, capi.W_WV, capi.W_WO, capi.W_W1, capi.W_W3, capi.W_W2):
                n, k = gs.slot_shape(spec, slot)
                om.set_layer(layer, slot, proj_types[slot], rand_blocks(n, k, proj_types[slot]))
        pattern = ((rng.random(1 << 16, dtype=np.float32) - 0.5) * 0.2).astype(np.float16).view(np.uint16)
        for layer in range(self.layers):
            data = om.pool.layer_data(layer)
            whole = data.size // pattern.size * pattern.size
            data[:whole].reshape(-1, pattern.size)[:] = pattern
            data[whole:] = pattern[:data.size - whole]
            for i in range(n_seqs):
                if layer == 0: om.pool.create_seq(i + 1)
                om.pool.store_kv(layer, i + 1, 0, None, None, int(self.ctx[i]))       # pages allocated, contents = the pattern
        self.pos = self.ctx.astype(np.int64).copy()
        self.logits = np.empty((1, spec.vocab), np.float32)
        self.tok = np.int32([7])
        self.next_seq = 0

    def decode(self, n_tokens):
        """One new token for each of the next n_tokens sequences (round robin); returns the seconds it took."""
        import ctypes as C
        L = self.O.lib()
        t0 = time.perf_counter()
        for _ in range(n_tokens):
            i = self.next_seq; self.next_seq = (i + 1) % len(self.ctx)
            rc = L.vo_model_forward(self.om.h, i + 1, self.tok.ctypes.data_as(C.c_void_p), 1, int(self.pos[i]), 0,
                                    self.logits.ctypes.data_as(C.c_void_p), None)
            assert rc == 0, rc
            self.pos[i] += 1
        return time.perf_counter() - t0

    def scale(self):
        """tokens/s of the whole model per tokens/s measured: 1 at full depth, otherwise the slice's share of the layers (the head
        is counted as part of the slice, which flatters the CPU a little)."""
        return 1.0 if self.full_depth else self.layers / self.spec.n_layers

    def describe(self, what):
        depth = (f"all {self.spec.n_layers} layers + output head" if self.full_depth
                 else f"{self.layers} of {self.spec.n_layers} layers + output head, layer time scaled to full depth")
        return (f"{what}; {self.spec.name} shape, {depth}, contexts ~U[{int(self.ctx.min())},{int(self.ctx.max())}] drawn like the benchmark's; "
                f"C port of the reference CPU path (inference/backend/cpu/cpu.go arithmetic, sequences decoded one at a time as "
                f"runtime/decode.go:623-654 does), OpenMP over output elements")


def cpu_baseline(spec, ctx_min, ctx_max, seconds_target=15.0):
    """Bounded CPU sample timed beside the GPU number: a few sequences of the workload, one token each, until the time is up."""
    port = CpuPort(spec, n_seqs=4, ctx_min=ctx_min, ctx_max=ctx_max)
    port.decode(1)                                         # warm the caches and the thread pool
    n, secs = 0, 0.0
    while n < 4 or (secs < seconds_target and n < 64):
        secs += port.decode(1); n += 1
    return {"value": n / secs * port.scale(), "unit": "tok/s", "cores": port.threads, "kind": "port",
            "sample": port.describe(f"{n} tokens decoded over 4 sequences in {secs:.1f} s")}


def dist_setup(n_gpus):
    world, rank, local = replicas.rank_env()
    return world, rank, local, replicas.init("nccl", local)


def reference_arm(args):
    """Times the CPU port of the reference's path with all host threads.  A step = one new token for each sequence of a bounded
    sample of the batch (the reference loops over the sequences of a batch, so its tok/s is the same for any batch size); the
    sample is sized from the first token's time so that W + K steps end within a few minutes."""
    world, rank, _ = replicas.rank_env()
    if rank != 0:
        return
    spec = WORKLOADS[args.workload]
    K, W = args.steps, max(args.warmup, 1)
    n_max = min(args.batch, 8)
    port = CpuPort(spec, n_seqs=n_max, ctx_min=args.ctx_min, ctx_max=args.ctx_max)
    t_tok = min(port.decode(1), port.decode(1))
    n_s = int(max(1, min(n_max, 150.0 / ((K + W) * t_tok))))
    for _ in range(W):
        port.decode(n_s)
    secs = [port.decode(n_s) for _ in range(K)]
    step_s = float(np.mean(secs))
    v = n_s / step_s * port.scale()
    base = {"value": v, "unit": "tok/s", "cores": port.threads, "kind": "port",
            "sample": port.describe(f"{K} timed steps of {n_s} of the batch's {args.batch} sequences each, {step_s * 1e3:.0f} ms per step")}
    line = {"impl": "reference", "metric": "decode tok/s", "value": v, "unit": "tok/s", "n_gpus": args.gpus, "steps": K,
            "warmup": W, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": f"{spec.name} batched decode B={args.batch}, ctx~U[{args.ctx_min},{args.ctx_max}], 16-token pages"},
            "sequences_per_step": n_s, "same_config": n_s == args.batch and port.full_depth, "extrapolated": not port.full_depth,
            "note": "value = sampled sequences per step / measured step time; the reference decodes a batch one sequence at a time, so tok/s does not depend on the batch size",
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
    # a step packs the decode rows of up to 256 sequences plus prompt chunks up to this row budget
    model = capi.Model(be, gs.model_config(spec, max_blocks, max_seqs=256, max_batch_tokens=args.trace_step_tokens, max_blocks_per_seq=max_ctx // 16 + 2))
    gs.synth_weights_on_device(be, model, spec, seed=0)
    res = tr.replay(model, arrivals, prompts, olen, max_batch=256)
    line = {"metric": "trace decode tok/s", "value": res["tok_per_s"], "unit": "tok/s", "n_gpus": 1, "higher_is_better": True, "data": "synthetic",
            "config": {"workload": f"{spec.name}: {args.trace} requests, Poisson {args.trace_rate}/s, prompts lognormal(ln 512, 0.8) clipped to "
                                   f"[16,{args.trace_max_prompt}], outputs U[32,512], max batch 256, {args.trace_step_tokens} rows per step (decode rows + prompt chunks), pool {max_blocks} blocks"},
            "trace": res}
    emit(line)
    model.close(); be.close()


_RESULT_FD = None


def tp_arm(args):
    """One model split over all the ranks (tensor parallelism over NCCL) instead of one replica per rank: the configuration for
    a model that one GPU cannot hold next to its KV cache.  Every rank keeps 1/world of each projection and of the KV heads of
    ALL --batch sequences, runs the same greedy step and meets the others in two all-reduces per layer.  Total work is fixed as
    the ranks grow, so the line reports strong scaling; value = batch * K / the slowest rank's device time."""
    from vexel_b200 import tp
    world, rank, local, dist = dist_setup(args.gpus)
    spec = WORKLOADS[args.workload]
    if args.layers > 0:
        spec = gs.scaled(spec, args.layers, spec.hidden, spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.ffn, spec.vocab)
    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    loc = tp.local_spec(spec, world)
    rng = np.random.default_rng(replicas.GLOBAL_WORKLOAD_SEED)
    ctx = rng.integers(args.ctx_min, args.ctx_max + 1, B)
    tokens = rng.integers(0, spec.vocab, B).astype(np.int32)
    total_new = W + 2 * K + 16
    blocks_per_seq = int((args.ctx_max + total_new) // 16 + 2)
    max_blocks = int(sum((c + total_new) // 16 + 2 for c in ctx) + 64)
    be = capi.Backend(local)
    if args.no_graphs:
        be.lib.vx_set_graphs(0)
    if world > 1:
        tp.init_from_torch(be, dist)
    else:
        tp.init(be, tp.unique_id(be), 0, 1)
    model = tp.create_model(be, spec, world, max_blocks=max_blocks, max_seqs=B, max_batch_tokens=max(B, 8), max_blocks_per_seq=blocks_per_seq)
    gs.synth_weights_on_device(be, model, loc, seed=1000, embed_vocab=spec.vocab)   # (the same draws on every rank: the embedding is replicated)
    model.shuffle_free_list(7)                                # the same block order on every rank: one set of block tables
    seqs = np.arange(1, B + 1, dtype=np.int64)
    for i, s in enumerate(seqs):
        model.seq_fill_synthetic(int(s), int(ctx[i]), seed=100 + i)
    pos = ctx.astype(np.int32).copy()
    out, _ = model.decode_run(seqs, tokens, pos, W)
    tokens = out[-1].copy(); pos += W
    replicas.barrier(dist)
    sampler = ClockSampler(local)
    l0, _ = model.counters()
    pos_timed, tokens_timed = pos.copy(), tokens.copy()
    out, dev_ms = model.decode_run(seqs, tokens, pos, K)
    l1, _ = model.counters()
    clocks = sampler.stop()
    replicas.barrier(dist)
    slowest = replicas.max_over_ranks(dist, dev_ms / 1e3, local)
    same = replicas.gather_objects(dist, int(np.asarray(out[-1], np.int64).sum()))
    e2e = None
    if not args.no_e2e:
        for i, sq in enumerate(seqs):
            model.seq_truncate(int(sq), int(pos_timed[i]))
        pos = pos_timed.copy(); cur = tokens_timed
        replicas.barrier(dist)
        be.Sync()
        t0 = time.perf_counter()
        for _ in range(K):
            cur = model.decode_step(seqs, cur, pos)
            pos += 1
        be.Sync()
        e2e_s = replicas.max_over_ranks(dist, time.perf_counter() - t0, local)
        e2e = {"value": B * K / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": int(5 * B * 4), "d2h_bytes_per_step": int(4 * B + 4),
               "ms_per_step": e2e_s / K * 1e3}
    per_rank = replicas.gather_objects(dist, {"rank": rank, "ms_per_step": dev_ms / K, "sm_mhz_median": clocks.get("sm_mhz"),
                                              "clock_reasons": clocks.get("reasons")})
    if rank == 0:
        peak, peak_kind = measured_peak()
        kvb = 2 * loc.n_kv_heads * loc.head_dim * 2
        kv_tokens = float(sum(int(p) * K + K * (K + 1) // 2 for p in pos_timed)) / K
        bytes_step = model.weight_bytes() + kv_tokens * kvb * spec.n_layers + B * spec.n_layers * kvb      # this rank's share
        ar_bytes = 2 * spec.n_layers * B * spec.hidden * 4                                                # two f32 all-reduces per layer
        step_ms = slowest / K * 1e3
        emit({"metric": "decode tok/s", "value": B * K / slowest, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
              "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
              "dtype": "f32 activations, %s weights, f16 kv" % spec.quant, "data": "synthetic",
              "config": {"workload": f"{spec.name} batched decode, B={B} over the whole group, ctx~U[{args.ctx_min},{args.ctx_max}] + generated, 16-token pages, shuffled blocks",
                         "global_batch": B, "parallelism": f"tp{world} (NCCL all-reduce after Wo and W2, vocabulary-split head)",
                         "l2": "inputs larger than L2: each step streams %.1f GB of weights+KV per rank" % (bytes_step / 1e9),
                         "timing": "CUDA events on the launching stream around K steps with on-device token feedback; max over ranks"},
              "step_roofline": {"bytes_per_step_per_rank": bytes_step, "achieved_GBs_per_rank": bytes_step / (step_ms * 1e-3) / 1e9,
                                "frac_of_measured": bytes_step / (step_ms * 1e-3) / 1e9 / peak, "peak_source": f"{peak_kind} copy bandwidth",
                                "allreduce_bytes_per_step": ar_bytes},
              "ranks_agree_on_tokens": len(set(same)) == 1, "clocks": clocks, "gpu_launches": int(l1 - l0), "e2e": e2e, "per_rank": per_rank})
    model.close(); be.close()
    replicas.shutdown(dist)


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
    ap.add_argument("--tp", action="store_true", help="one model split over all the ranks (tensor parallelism) instead of one replica per rank")
    ap.add_argument("--trace-rate", type=float, default=40.0, help="trace arrivals per second")
    ap.add_argument("--trace-max-prompt", type=int, default=8192)
    ap.add_argument("--trace-step-tokens", type=int, default=1024, help="rows per scheduler step in the trace replay: decode rows plus prompt chunks")
    ap.add_argument("--no-dependent-launch", action="store_true", help="experiment: projections in plain stream order instead of as programmatic dependents")
    ap.add_argument("--chain-launch", action="store_true", help="experiment: every kernel of a layer launched as a programmatic dependent of the one before it, not only the projections")
    ap.add_argument("--no-graphs", action="store_true", help="experiment: launch every kernel individually instead of replaying CUDA graphs")
    ap.add_argument("--no-persistent", action="store_true", help="experiment: Q4_0 decode projections on the one-CTA-per-tile tcgen05 kernel instead of the persistent one")
    ap.add_argument("--aligned-split", action="store_true", help="experiment: persistent projections with tile-aligned split-K only (no stream mode)")
    ap.add_argument("--no-thin", action="store_true", help="experiment: 1-4 row Q4_0 projections on the staged mma.sync kernel instead of the weight-streaming one")
    ap.add_argument("--tc-min-rows", type=int, default=-1, help="experiment: batch size from which projections use the tcgen05 kernel")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    if args.trace > 0:
        return trace_arm(args)
    if args.tp:
        return tp_arm(args)
    world, rank, local, dist = dist_setup(args.gpus)
    spec = WORKLOADS[args.workload]
    if args.layers > 0:
        spec = gs.scaled(spec, args.layers, spec.hidden, spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.ffn, spec.vocab)
    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    Ka = Kg = min(K, 8)                             # short legs that time the attention and the projection launches
    seeds = replicas.rank_seeds(rank)
    # ONE arrival stream for the whole job: B * world contexts, placed by the dispatcher on the replica with the most free
    # blocks.  Every rank replays the same stream and keeps its own share (no communication: the placement is a pure function
    # of the stream).  At one GPU this is the plain draw of B contexts.
    rng = np.random.default_rng(replicas.GLOBAL_WORKLOAD_SEED)
    ctx_all = rng.integers(args.ctx_min, args.ctx_max + 1, B * world)
    tokens_all = rng.integers(0, spec.vocab, B * world).astype(np.int32)
    total_new = W + 2 * K + Ka + Kg + 16            # warm-up + device-resident leg + the two kernel legs (the end-to-end leg rolls back)
    seq_cap = B                                     # a replica's batch limit: the projections' fast path covers 64 rows, the 65th would cost more than it balances
    router = replicas.Dispatcher(world, blocks_per_replica=10 ** 9, max_seqs_per_replica=seq_cap)
    owner = np.array([router.place(i, int(c) + total_new) for i, c in enumerate(ctx_all)])
    mine = np.nonzero(owner == rank)[0]
    ctx = ctx_all[mine]
    Bl = int(len(mine))                             # this replica's sequences
    blocks_per_seq = int((args.ctx_max + total_new) // 16 + 2)
    max_blocks = int(sum((c + total_new) // 16 + 2 for c in ctx) + 64)

    be = capi.Backend(local)
    if args.tc_min_rows >= 0:
        be.lib.vx_set_tc_min_rows(args.tc_min_rows)
    if args.no_dependent_launch:
        be.lib.vx_set_dependent_launch(0)
    if args.chain_launch:
        be.lib.vx_set_dependent_launch(2)
    if args.no_graphs:
        be.lib.vx_set_graphs(0)
    if args.no_persistent:
        be.lib.vx_set_persistent_projections(0)
    if args.aligned_split:
        be.lib.vx_set_persistent_projections(1)
    if args.no_thin:
        be.lib.vx_set_thin_batch_projections(0)
    model = capi.Model(be, gs.model_config(spec, max_blocks, max_seqs=seq_cap, max_batch_tokens=max(seq_cap, 8), max_blocks_per_seq=blocks_per_seq))
    gs.synth_weights_on_device(be, model, spec, seed=seeds["weights"])
    model.shuffle_free_list(seeds["free_list"])               # physical blocks shuffled randomly in the pool
    seqs = np.arange(1, Bl + 1, dtype=np.int64)
    for i, s in enumerate(seqs):
        model.seq_fill_synthetic(int(s), int(ctx[i]), seed=seeds["kv_fill"] + i)
    tokens = tokens_all[mine].copy()
    pos = ctx.astype(np.int32).copy()

    def kv_tokens_over(pos0, n_steps):
        """Sum over n_steps steps and the sequences of the attended length, as a per-layer mean (windowed layers attend less)."""
        g = float(sum(int(p) * n_steps + n_steps * (n_steps + 1) // 2 for p in pos0))
        n_slide = spec.n_layers // 2 if (spec.window_alternating and spec.sliding_window > 0) else 0   # odd layers slide
        sl = float(sum(min(int(p) + j, spec.sliding_window) for p in pos0 for j in range(1, n_steps + 1))) if n_slide else 0.0
        return ((spec.n_layers - n_slide) * g + n_slide * sl) / spec.n_layers

    # ---- warm-up (W >= 3 steps; it also captures the step graphs), then K timed steps with the tokens fed back on the device.
    # No per-kernel events in the timed steps: they replay from CUDA graphs exactly like the end-to-end leg.
    out, _ = model.decode_run(seqs, tokens, pos, W)
    tokens = out[-1].copy(); pos += W
    replicas.barrier(dist)
    sampler = ClockSampler(local)
    l0, s0 = model.counters()
    g0 = model.graph_stats()[0]
    kv_tokens_timed = kv_tokens_over(pos, K)
    pos_timed, tokens_timed = pos.copy(), tokens.copy()       # where the timed leg starts: the end-to-end leg starts there again
    out, dev_ms = model.decode_run(seqs, tokens, pos, K)
    l1, s1 = model.counters()
    replayed = model.graph_stats()[0] - g0
    clocks = sampler.stop()
    tokens = out[-1].copy(); pos += K
    replicas.barrier(dist)
    value, max_s = replicas.job_throughput(dist, Bl * K, dev_ms / 1e3, local)
    max_ms = max_s * 1e3
    # ---- CUDA events around every launch of the dominant kernel (paged attention), in a leg of its own right after the timed
    # region (events inside the timed steps would keep them out of graph replay); then the same for the projections
    model.kernel_time(0, 1); model.kernel_time(1, 0)
    kv_tokens_attn = kv_tokens_over(pos, Ka)
    out, attn_leg_ms = model.decode_run(seqs, tokens, pos, Ka)
    attn_ms, attn_n = model.kernel_time(0, 0)
    tokens = out[-1].copy(); pos += Ka
    model.kernel_time(1, 1)
    out, _ = model.decode_run(seqs, tokens, pos, Kg)
    gemm_ms, gemm_n = model.kernel_time(1, 0)
    gemm_ms_per_step = gemm_ms / Kg
    tokens = out[-1].copy(); pos += Kg

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
        e2e_v, e2e_s = replicas.job_throughput(dist, Bl * K, time.perf_counter() - t0, local)
        e2e = {"value": e2e_v, "unit": "tok/s", "h2d_bytes_per_step": int(5 * Bl * 4), "d2h_bytes_per_step": int(4 * Bl + 4),
               "ms_per_step": e2e_s / K * 1e3}

    kv_bytes_per_token_layer = 2 * spec.n_kv_heads * spec.head_dim * 2             # K and V, fp16
    per_rank = replicas.gather_objects(dist, {
        "rank": rank, "sequences": Bl, "ms_per_step": dev_ms / K, "kv_GB_per_step": kv_tokens_timed / K * kv_bytes_per_token_layer * spec.n_layers / 1e9,
        "sm_mhz_median": clocks.get("sm_mhz"), "clock_reasons": clocks.get("reasons"), "graph_replayed_steps": int(replayed),
        "attn_launch_ms": attn_ms / max(attn_n, 1)})

    if rank != 0:
        model.close(); be.close()
        replicas.shutdown(dist)
        return

    # ---- roofline of the dominant kernel (paged attention) and of the whole step (rank 0's replica)
    peak, peak_kind = measured_peak()
    attn_bytes_per_launch = kv_tokens_attn * kv_bytes_per_token_layer / Ka         # one launch = one layer of one step
    attn_launch_ms = attn_ms / max(attn_n, 1)
    attn_gbs = attn_bytes_per_launch / (attn_launch_ms * 1e-3) / 1e9 if attn_n else None
    W_bytes = model.weight_bytes()
    bytes_step = W_bytes + kv_tokens_timed / K * kv_bytes_per_token_layer * spec.n_layers + Bl * spec.n_layers * kv_bytes_per_token_layer
    step_ms = dev_ms / K                                                           # rank 0's own step time for rank 0's own bytes
    step_gbs = bytes_step / (step_ms * 1e-3) / 1e9
    attn_ms_per_step = attn_launch_ms * spec.n_layers
    roofline = {"bound": "hbm", "kernel": "paged attention (flash kernel + merge/split), one launch pair per layer", "achieved": attn_gbs, "peak": peak, "unit": "GB/s",
                "frac": (attn_gbs / peak) if attn_gbs else None, "peak_source": f"{peak_kind} copy bandwidth",
                "traffic": (ATTN_TRAFFIC_RATIO * attn_bytes_per_launch) if ATTN_TRAFFIC_RATIO else None,
                "traffic_note": "DRAM bytes of one ncu capture of a smaller case, scaled by the algorithmic bytes of this launch",
                "algorithmic_bytes_per_launch": attn_bytes_per_launch, "launch_ms": attn_launch_ms,
                "timed_in": "a leg of %d steps right after the timed region, CUDA events around every launch" % Ka,
                "share_of_step": attn_ms_per_step / step_ms if step_ms else None,
                "projections": {"timed_in": "a leg of %d steps after the attention leg" % Kg, "launch_ms_total_per_step": gemm_ms_per_step,
                                "share_of_step": gemm_ms_per_step / step_ms if step_ms else None,
                                "weight_bytes": W_bytes, "achieved_GBs": W_bytes / (gemm_ms_per_step * 1e-3) / 1e9 if gemm_ms else None}}
    line = {"metric": "decode tok/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": max_ms / K,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 activations, %s weights, f16 kv" % spec.quant,
            "data": "synthetic",
            "config": {"workload": f"{spec.name} batched decode, B={B} per GPU ({B * world} sequences placed by free blocks), ctx~U[{args.ctx_min},{args.ctx_max}] + generated, 16-token pages, shuffled blocks",
                       "global_batch": world * B, "parallelism": f"replicas x{world} (request sharding, no collective)",
                       "l2": "inputs larger than L2: each step streams %.1f GB of weights+KV" % (bytes_step / 1e9),
                       "timing": "CUDA events on the launching stream around K graph-replayed steps with on-device token feedback; max over ranks"},
            "roofline": roofline,
            "step_roofline": {"bytes_per_step": bytes_step, "achieved_GBs": step_gbs, "frac_of_measured": step_gbs / peak,
                              "frac_of_nominal_8TBs": step_gbs / NOMINAL_HBM_GBS,
                              "roofline_tok_s_measured": B / (bytes_step / (peak * 1e9)), "roofline_tok_s_nominal": B / (bytes_step / (NOMINAL_HBM_GBS * 1e9))},
            "clocks": clocks, "gpu_launches": int(l1 - l0), "e2e": e2e, "per_rank": per_rank}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(spec, args.ctx_min, args.ctx_max)
    emit(line)
    model.close(); be.close()
    replicas.shutdown(dist)


if __name__ == "__main__":
    main()
