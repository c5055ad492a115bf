"""Replay of a synthetic request trace through the continuous-batching scheduler (vx_sched_*).

Requests arrive as a Poisson process, prompts are log-normal, output lengths uniform — the shape of a serving trace, with
random token ids.  The clock is virtual and deterministic in its inputs: it advances by the measured duration of every
scheduler step, and jumps to the next arrival when nothing is in flight, so a trace replays the same admission order on
any machine while the reported throughput is that of the machine it ran on.
"""
import time

import numpy as np

from . import capi


def make_trace(n_requests, rate_per_s, vocab, seed=4, prompt_mu=np.log(512.0), prompt_sigma=0.8, prompt_clip=(16, 8192),
               out_range=(32, 512)):
    """Returns (arrival seconds [n], prompts list of int32 arrays, output lengths [n])."""
    rng = np.random.default_rng(seed)
    arrivals = np.cumsum(rng.exponential(1.0 / rate_per_s, n_requests))
    plen = np.clip(np.rint(rng.lognormal(prompt_mu, prompt_sigma, n_requests)), prompt_clip[0], prompt_clip[1]).astype(np.int64)
    olen = rng.integers(out_range[0], out_range[1] + 1, n_requests)
    prompts = [rng.integers(0, vocab, int(n)).astype(np.int32) for n in plen]
    return arrivals, prompts, olen


def replay(model: capi.Model, arrivals, prompts, out_lens, max_batch=256, max_sequences=0, temperature=0.0, top_k=0, top_p=0.0, seed=0):
    """Runs the trace to completion.  Returns a dict of totals and latencies (seconds of virtual time)."""
    n = len(prompts)
    sched = capi.Scheduler(model, max_batch_size=max_batch, max_sequences=max_sequences, temperature=temperature, top_k=top_k, top_p=top_p, seed=seed)
    now, nxt = 0.0, 0
    first_tok = np.full(n, np.nan); done_at = np.full(n, np.nan); got = np.zeros(n, np.int64)
    live = set()
    steps = 0; busy = 0.0
    while nxt < n or live:
        while nxt < n and arrivals[nxt] <= now:
            sched.AddSequence(1000 + nxt, prompts[nxt], max_tokens=int(out_lens[nxt])); live.add(nxt); nxt += 1
        if not live:
            now = float(arrivals[nxt]); continue
        t0 = time.perf_counter()
        sched.step()
        dt = time.perf_counter() - t0
        now += dt; busy += dt; steps += 1
        for i in list(live):
            toks, fin = sched.poll(1000 + i)
            if toks.size:
                if got[i] == 0: first_tok[i] = now
                got[i] += toks.size
            if fin:
                done_at[i] = now; live.discard(i)
    met = sched.Metrics()
    preemptions, refused = sched.pressure()
    sched.close()
    gen = int(got.sum())
    return {"requests": n, "generated_tokens": gen, "prompt_tokens": int(sum(len(p) for p in prompts)), "makespan_s": now, "busy_s": busy,
            "steps": steps, "tok_per_s": gen / busy if busy > 0 else 0.0, "tok_per_s_makespan": gen / now if now > 0 else 0.0,
            "ttft_mean_s": float(np.nanmean(first_tok - arrivals[:n])), "ttft_p95_s": float(np.nanpercentile(first_tok - arrivals[:n], 95)),
            "latency_mean_s": float(np.nanmean(done_at - arrivals[:n])),
            "sched_prefill_s": met.prefill_seconds, "sched_decode_s": met.decode_seconds, "sched_decode_tokens": met.decode_tokens,
            "sched_prefill_tokens": met.prefill_tokens, "completed": int(np.isfinite(done_at).sum()), "preemptions": int(preemptions),
            "refused": int(refused)}
