// Continuous-batching scheduler over the batched decode fast path: the host logic of inference/scheduler
// (scheduler.go:168-483, sequence.go) restated in C++ because no Go toolchain exists where this library is built.
// Same state machine (Pending -> Decoding -> Finished), same step order (prefill the pending sequences of the batch,
// sample their first token, then one decode step for every decoding sequence of the batch), same metrics.  Differences,
// all deliberate: the batch is taken in arrival order (the reference iterates a Go map), the whole batch is ONE
// vx_decode_step instead of a per-sequence loop, and a pending prompt that does not fit the free blocks waits
// instead of stopping the scheduler loop (scheduler.go:134-136).  Temperature 0 is greedy (first maximum); otherwise
// tokens are drawn on the device by the sampler's rules with uniform draws from a generator seeded by the config
// (the reference copies the logits to the host and draws from math/rand, scheduler.go:783-820).
#include <chrono>
#include <deque>

#include "vx_common.cuh"

namespace {
enum SeqState { kPending = 0, kPrefill = 1, kDecoding = 2, kFinished = 3 };   // sequence.go:15-20
struct Seq {
    int64_t id; SeqState state = kPending;
    std::vector<int32_t> prompt, generated; std::deque<int32_t> chan;           // chan = tokenChan (sequence.go:70-80)
    int position = 0, max_tokens = 0; size_t drained = 0;
};
}  // namespace

struct vx_sched {
    vx_model *m = nullptr; vx_ctx *c = nullptr;
    vx_sched_config cfg{};
    std::vector<Seq> seqs;            // arrival order
    vx_sched_metrics met{};
    std::mutex mu;
    uint64_t rng = 0;
    // splitmix64; the top 24 bits make a float in [0, 1) like rand.Float32
    float uniform() {
        uint64_t z = (rng += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; z ^= z >> 31;
        return (float)(z >> 40) * (1.0f / 16777216.0f);
    }
    vx_sample_params draw() { return vx_sample_params{cfg.temperature, cfg.top_k, cfg.top_p, uniform()}; }
};

extern "C" {

int vx_sched_create(vx_model *m, const vx_sched_config *cfg, vx_sched **out) {
    if (!m || !cfg || !out || cfg->max_batch_size <= 0) return VX_E_BAD_ARG;
    vx_sched *s = new vx_sched();
    s->m = m; s->cfg = *cfg; s->rng = cfg->seed;
    *out = s;
    return VX_OK;
}
int vx_sched_destroy(vx_sched *s) { if (!s) return VX_E_BAD_ARG; delete s; return VX_OK; }

// Scheduler.AddSequence (scheduler.go:645-676): registers the request; its KV sequence is created on first use
int vx_sched_add_sequence(vx_sched *s, int64_t id, const int32_t *prompt, int n_prompt, int max_tokens) {
    if (!s || !prompt || n_prompt <= 0) return VX_E_BAD_ARG;
    std::lock_guard<std::mutex> g(s->mu);
    for (auto &q : s->seqs) if (q.id == id && q.state != kFinished) return VX_E_BAD_ARG;
    int live = 0;
    for (auto &q : s->seqs) live += q.state != kFinished;
    if (s->cfg.max_sequences > 0 && live >= s->cfg.max_sequences) return VX_E_OOM;   // the reference stores MaxSequences but never enforces it
    Seq q; q.id = id; q.prompt.assign(prompt, prompt + n_prompt); q.max_tokens = max_tokens;
    s->seqs.push_back(std::move(q));
    return VX_OK;
}

// Scheduler.RemoveSequence (scheduler.go:690-698)
int vx_sched_remove_sequence(vx_sched *s, int64_t id) {
    if (!s) return VX_E_BAD_ARG;
    std::lock_guard<std::mutex> g(s->mu);
    for (size_t i = 0; i < s->seqs.size(); i++)
        if (s->seqs[i].id == id) {
            if (s->seqs[i].state != kFinished) vx_seq_delete(s->m, id);
            s->seqs.erase(s->seqs.begin() + (long)i);
            return VX_OK;
        }
    return VX_OK;
}

static bool finish_if_done(vx_sched *s, Seq &q, int32_t tok) {
    int limit = q.max_tokens > 0 ? q.max_tokens : s->cfg.max_tokens;                  // sequence.go ReachedMaxTokens
    bool stop = (s->cfg.eos_token >= 0 && tok == s->cfg.eos_token);                   // isStopToken
    if (!stop) q.chan.push_back(tok);                                                 // PushToken
    if (stop || (limit > 0 && (int)q.generated.size() >= limit)) {
        q.state = kFinished;
        vx_seq_delete(s->m, q.id);
        s->met.completed_sequences++;
        return true;
    }
    return false;
}

// Scheduler.step (scheduler.go:168-203) + runDecodeStep (:245-483)
int vx_sched_step(vx_sched *s, int *n_active_out) {
    if (!s) return VX_E_BAD_ARG;
    std::lock_guard<std::mutex> g(s->mu);
    using clk = std::chrono::steady_clock;
    std::vector<Seq *> batch;                                                          // collectReady + formBatches
    for (auto &q : s->seqs) {
        if (q.state == kFinished) continue;
        if ((int)batch.size() < s->cfg.max_batch_size) batch.push_back(&q);
    }
    int active = 0;
    for (auto &q : s->seqs) active += q.state != kFinished;
    s->met.active_sequences = active;
    if (n_active_out) *n_active_out = active;
    if (batch.empty()) return VX_OK;
    // 1. prefill the pending sequences of the batch (runBatchedPrefill, scheduler.go:486-550)
    for (Seq *q : batch) {
        if (q->state != kPending) continue;
        int total = 0, free_blocks = 0;
        VX_TRY(vx_pool_stats(s->m, &total, &free_blocks, nullptr));
        int per_layer_free = free_blocks / std::max(1, total / std::max(1, vx_model_max_blocks(s->m)));
        int need = ((int)q->prompt.size() + 16) / 16 + 1;
        if (need > per_layer_free) continue;                                           // block-aware admission: wait for blocks
        auto t0 = clk::now();
        int32_t tok = 0;
        vx_sample_params sp = s->draw();
        int rc = s->cfg.temperature == 0.f ? vx_prefill(s->m, q->id, q->prompt.data(), (int)q->prompt.size(), 0, &tok, nullptr)
                                           : vx_prefill_sampled(s->m, q->id, q->prompt.data(), (int)q->prompt.size(), 0, &sp, &tok, nullptr);
        if (rc != VX_OK) return rc;
        q->position = (int)q->prompt.size();
        q->generated.push_back(tok);
        s->met.total_tokens += (int)q->prompt.size(); s->met.prefill_tokens += (int)q->prompt.size();
        s->met.prefill_seconds += std::chrono::duration<double>(clk::now() - t0).count();
        q->state = kDecoding;
        finish_if_done(s, *q, tok);
    }
    // 2. one decode step for every decoding sequence of the batch
    std::vector<int64_t> ids; std::vector<int32_t> toks, pos; std::vector<Seq *> dec;
    for (Seq *q : batch)
        if (q->state == kDecoding) { dec.push_back(q); ids.push_back(q->id); toks.push_back(q->generated.back()); pos.push_back(q->position); }
    if (dec.empty()) return VX_OK;
    auto t0 = clk::now();
    std::vector<int32_t> out(dec.size());
    int rc;
    if (s->cfg.temperature == 0.f) rc = vx_decode_step(s->m, (int)dec.size(), ids.data(), toks.data(), pos.data(), nullptr, out.data(), nullptr);
    else {
        std::vector<vx_sample_params> sp(dec.size());
        for (auto &p : sp) p = s->draw();
        rc = vx_decode_step_sampled(s->m, (int)dec.size(), ids.data(), toks.data(), pos.data(), nullptr, sp.data(), out.data(), nullptr);
    }
    if (rc != VX_OK) return rc;
    for (size_t i = 0; i < dec.size(); i++) {
        Seq &q = *dec[i];
        q.position++;                                                                   // AdvancePosition
        q.generated.push_back(out[i]);                                                  // AddGeneratedToken
        finish_if_done(s, q, out[i]);
    }
    s->met.total_tokens += (int)dec.size(); s->met.decode_tokens += (int)dec.size();
    s->met.decode_seconds += std::chrono::duration<double>(clk::now() - t0).count();
    return VX_OK;
}

// drains the sequence's token channel (Sequence.TokenChan); *finished is set once the sequence has ended
int vx_sched_poll(vx_sched *s, int64_t id, int32_t *out, int cap, int *n_out, int *finished) {
    if (!s || !n_out) return VX_E_BAD_ARG;
    std::lock_guard<std::mutex> g(s->mu);
    for (auto &q : s->seqs)
        if (q.id == id) {
            int n = 0;
            while (n < cap && !q.chan.empty()) { if (out) out[n] = q.chan.front(); q.chan.pop_front(); n++; }
            *n_out = n;
            if (finished) *finished = q.state == kFinished && q.chan.empty();
            return VX_OK;
        }
    return VX_E_NO_SEQ;
}

// Scheduler.Metrics (scheduler.go:475-481)
int vx_sched_get_metrics(vx_sched *s, vx_sched_metrics *out) {
    if (!s || !out) return VX_E_BAD_ARG;
    std::lock_guard<std::mutex> g(s->mu);
    *out = s->met;
    return VX_OK;
}

}  // extern "C"
