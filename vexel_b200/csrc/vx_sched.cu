// Continuous-batching scheduler over the batched decode fast path: the host logic of inference/scheduler
// (scheduler.go:168-483, sequence.go) restated in C++ because no Go toolchain exists where this library is built.
// Same state machine (Pending -> Prefill -> Decoding -> Finished) and the same metrics.  Where it differs, on purpose:
//   * one packed step per iteration: the decoding sequences (one row each) and the next chunk of every prompt that is being
//     read share ONE vx_decode_step_ex call, so a long prompt no longer stalls the sequences that are generating (the
//     reference prefills each pending sequence with a call of its own, then decodes, scheduler.go:245-303, 486-550);
//   * block-aware admission: a request enters the batch only when the pool can hold its prompt plus everything it may
//     generate (its token limit), so a step can never run out of blocks half way; a request that could never fit is ended
//     with an error instead of waiting for ever, and requests that wait take no batch slot (the reference stops its loop on
//     the first allocation error, scheduler.go:134-136);
//   * requests without a token limit reserve their prompt only; if the pool then runs dry the youngest sequence is
//     preempted (its blocks freed, its prompt + generated tokens re-read later) so that the others keep going;
//   * the batch is taken in arrival order (the reference iterates a Go map).
// Temperature 0 is greedy (first maximum); otherwise tokens are drawn on the device by the sampler's rules with uniform
// draws from a generator seeded by the config (the reference copies the logits to the host and draws from math/rand,
// scheduler.go:783-820).
#include <algorithm>
#include <chrono>
#include <deque>

#include "vx_common.cuh"

namespace {
constexpr int BS = 16;
enum SeqState { kPending = 0, kPrefill = 1, kDecoding = 2, kFinished = 3 };   // sequence.go:15-20
struct Seq {
    int64_t id; SeqState state = kPending;
    std::vector<int32_t> feed, generated; std::deque<int32_t> chan;           // chan = tokenChan (sequence.go:70-80)
    size_t n_prompt = 0;              // the request's own prompt; feed grows by the generated tokens when it is preempted
    int position = 0;                 // tokens in the KV cache
    int fed = 0;                      // tokens of `feed` already in the cache
    int max_tokens = 0;
    bool admitted = false; int reserved = 0;       // blocks set aside for this sequence (held + still to come)
    int fail_code = 0; bool reported = false;
};
int blocks_for(int tokens) { return (tokens + BS - 1) / BS; }
}  // namespace

struct vx_sched {
    vx_model *m = nullptr; vx_ctx *c = nullptr;
    vx_sched_config cfg{};
    vx_model_config mc{};
    std::deque<Seq> seqs;             // arrival order
    vx_sched_metrics met{};
    std::mutex mu;
    uint64_t rng = 0;
    uint64_t preemptions = 0, refused = 0;
    // splitmix64; the top 24 bits make a float in [0, 1) like rand.Float32
    float uniform() {
        uint64_t z = (rng += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; z ^= z >> 31;
        return (float)(z >> 40) * (1.0f / 16777216.0f);
    }
    vx_sample_params draw() { return vx_sample_params{cfg.temperature, cfg.top_k, cfg.top_p, uniform()}; }
    int limit_of(const Seq &q) const { return q.max_tokens > 0 ? q.max_tokens : cfg.max_tokens; }
    // Entries whose end the caller has seen stay pollable for a while (a client may ask again), but not for ever: beyond
    // KEEP_REPORTED of them the oldest go, so the scans above stay short however many requests a server has seen.
    static constexpr size_t KEEP_REPORTED = 256;
    void purge() {
        size_t n = 0;
        for (auto &q : seqs) n += q.state == kFinished && q.reported && q.chan.empty();
        for (size_t i = 0; i < seqs.size() && n > KEEP_REPORTED;)
            if (seqs[i].state == kFinished && seqs[i].reported && seqs[i].chan.empty()) { seqs.erase(seqs.begin() + (long)i); n--; } else i++;
    }
};

extern "C" {

int vx_sched_create(vx_model *m, const vx_sched_config *cfg, vx_sched **out) {
    if (!m || !cfg || !out || cfg->max_batch_size <= 0) return VX_E_BAD_ARG;
    vx_sched *s = new vx_sched();
    s->m = m; s->c = vx_model_ctx(m); s->cfg = *cfg; s->rng = cfg->seed;
    if (vx_model_get_config(m, &s->mc) != VX_OK) { delete s; return VX_E_BAD_ARG; }
    *out = s;
    return VX_OK;
}
int vx_sched_destroy(vx_sched *s) { if (!s) return VX_E_BAD_ARG; delete s; return VX_OK; }

// Scheduler.AddSequence (scheduler.go:645-676): registers the request; its KV sequence is created on first use
int vx_sched_add_sequence(vx_sched *s, int64_t id, const int32_t *prompt, int n_prompt, int max_tokens) {
    if (!s || !prompt || n_prompt <= 0) return VX_E_BAD_ARG;
    std::lock_guard<std::mutex> g(s->mu);
    s->purge();
    int live = 0;
    for (size_t i = 0; i < s->seqs.size();) {
        Seq &q = s->seqs[i];
        if (q.id == id) {
            if (q.state != kFinished) return VX_E_BAD_ARG;
            s->seqs.erase(s->seqs.begin() + (long)i);       // a finished request of the same id makes room for the new one
            continue;
        }
        live += q.state != kFinished;
        i++;
    }
    if (s->cfg.max_sequences > 0 && live >= s->cfg.max_sequences) return VX_E_OOM;   // the reference stores MaxSequences but never enforces it
    Seq q; q.id = id; q.feed.assign(prompt, prompt + n_prompt); q.n_prompt = (size_t)n_prompt; q.max_tokens = max_tokens;
    s->seqs.push_back(std::move(q));
    return VX_OK;
}

// Scheduler.RemoveSequence (scheduler.go:690-698)
int vx_sched_remove_sequence(vx_sched *s, int64_t id) {
    if (!s) return VX_E_BAD_ARG;
    std::lock_guard<std::mutex> g(s->mu);
    for (size_t i = 0; i < s->seqs.size(); i++)
        if (s->seqs[i].id == id) {
            if (s->seqs[i].state != kFinished && s->seqs[i].position > 0) vx_seq_delete(s->m, id);
            s->seqs.erase(s->seqs.begin() + (long)i);
            return VX_OK;
        }
    return VX_OK;
}

static void finish(vx_sched *s, Seq &q) {
    q.state = kFinished; q.admitted = false; q.reserved = 0;
    if (q.position > 0) vx_seq_delete(s->m, q.id);
    q.position = 0;
}
static bool finish_if_done(vx_sched *s, Seq &q, int32_t tok) {
    int limit = s->limit_of(q);                                                       // sequence.go ReachedMaxTokens
    bool stop = (s->cfg.eos_token >= 0 && tok == s->cfg.eos_token);                   // isStopToken
    if (!stop) q.chan.push_back(tok);                                                 // PushToken
    if (stop || (limit > 0 && (int)q.generated.size() >= limit)) {
        finish(s, q);
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
    s->purge();
    int active = 0;
    for (auto &q : s->seqs) active += q.state != kFinished;
    s->met.active_sequences = active;
    if (n_active_out) *n_active_out = active;
    if (active == 0) return VX_OK;

    int total = 0, free_blocks = 0;
    VX_TRY(vx_pool_stats(s->m, &total, &free_blocks, nullptr));
    const int n_layers = std::max(1, s->mc.n_layers);
    int pool_free = free_blocks / n_layers;                     // every layer's pool evolves alike
    // ---- admission, in arrival order: blocks still owed to the admitted sequences are not available to newcomers
    int owed = 0, admitted_live = 0;
    for (auto &q : s->seqs)
        if (q.state != kFinished && q.admitted) { owed += std::max(0, q.reserved - blocks_for(q.position)); admitted_live++; }
    for (auto &q : s->seqs) {
        if (q.state == kFinished || q.admitted) continue;
        const int limit = s->limit_of(q);
        const int remaining = limit > 0 ? std::max(1, limit - (int)q.generated.size()) : 0;
        // the cache ends up holding the fed tokens plus every generated token but the last
        const int need = limit > 0 ? blocks_for((int)q.feed.size() + remaining) : blocks_for((int)q.feed.size()) + 1;
        if (need > s->mc.max_blocks || need > s->mc.max_blocks_per_seq) {
            // never: not with an empty pool either.  End the request with an error the caller can read (vx_sched_poll).
            q.fail_code = VX_E_OOM_BLOCKS; finish(s, q); s->refused++;
            continue;
        }
        if (admitted_live >= s->mc.max_seqs || need > pool_free - owed) break;     // wait; later arrivals do not jump the queue
        q.admitted = true; q.reserved = need; owed += need; admitted_live++;
    }

    // ---- the batch: decoding sequences first, then prompt chunks up to the step's token budget
    const int T = s->mc.max_batch_tokens;
    std::vector<Seq *> dec, pre; std::vector<int> chunk;
    for (;;) {
        dec.clear(); pre.clear(); chunk.clear();
        for (auto &q : s->seqs)
            if (q.state == kDecoding && q.admitted && (int)dec.size() < std::min(s->cfg.max_batch_size, T)) dec.push_back(&q);
        int budget = T - (int)dec.size();
        for (auto &q : s->seqs) {
            if ((q.state != kPending && q.state != kPrefill) || !q.admitted) continue;
            if ((int)(dec.size() + pre.size()) >= s->cfg.max_batch_size || budget <= 0) break;
            int n = std::min(budget, (int)q.feed.size() - q.fed);
            pre.push_back(&q); chunk.push_back(n); budget -= n;
        }
        // blocks this step takes; sequences admitted with a token limit are covered by their reservation, the others may not be
        long need = 0;
        for (Seq *q : dec) need += blocks_for(q->position + 1) - blocks_for(q->position);
        for (size_t i = 0; i < pre.size(); i++) need += blocks_for(pre[i]->fed + chunk[i]) - blocks_for(pre[i]->fed);
        if (need <= pool_free) break;
        // preempt the youngest sequence that holds blocks: free them, and read its prompt + generated tokens again later
        Seq *victim = nullptr;
        for (auto it = s->seqs.rbegin(); it != s->seqs.rend(); ++it)
            if (it->state != kFinished && it->admitted && it->position > 0) { victim = &*it; break; }
        int holders = 0;
        for (auto &q : s->seqs) holders += q.state != kFinished && q.admitted && q.position > 0;
        if (!victim || holders <= 1) {
            // a single sequence outgrew the pool: end it rather than spin
            Seq *last = victim ? victim : (dec.empty() ? (pre.empty() ? nullptr : pre[0]) : dec[0]);
            if (!last) return vx_fail(s->c, VX_E_OOM_BLOCKS, "scheduler: the pool cannot hold a single step");
            last->fail_code = VX_E_OOM_BLOCKS; finish(s, *last); s->refused++;
        } else {
            pool_free += blocks_for(victim->position);
            vx_seq_delete(s->m, victim->id);
            if (victim->state == kDecoding) victim->feed.insert(victim->feed.end(), victim->generated.begin() + (long)(victim->feed.size() - victim->n_prompt), victim->generated.end());
            victim->state = kPending; victim->admitted = false; victim->reserved = 0; victim->position = 0; victim->fed = 0;
            s->preemptions++;
        }
        VX_TRY(vx_pool_stats(s->m, &total, &free_blocks, nullptr));
        pool_free = free_blocks / n_layers;
    }
    if (dec.empty() && pre.empty()) return VX_OK;

    // ---- one packed step (scheduler.go:245-303 and 486-550 in one call)
    const size_t n = dec.size() + pre.size();
    std::vector<int64_t> ids; std::vector<int32_t> toks, pos, qlens;
    ids.reserve(n); pos.reserve(n); qlens.reserve(n);
    for (Seq *q : dec) { ids.push_back(q->id); toks.push_back(q->generated.back()); pos.push_back(q->position); qlens.push_back(1); }
    for (size_t i = 0; i < pre.size(); i++) {
        Seq *q = pre[i];
        ids.push_back(q->id); pos.push_back(q->fed); qlens.push_back(chunk[i]);
        toks.insert(toks.end(), q->feed.begin() + q->fed, q->feed.begin() + q->fed + chunk[i]);
        q->state = kPrefill;
    }
    auto t0 = clk::now();
    std::vector<int32_t> out(n);
    std::vector<vx_sample_params> sp;
    if (s->cfg.temperature != 0.f) { sp.resize(n); for (auto &p : sp) p = s->draw(); }
    int rc = vx_decode_step_ex(s->m, (int)n, ids.data(), toks.data(), pos.data(), qlens.data(), VX_STEP_LAST_ROWS | VX_STEP_PROMPT_ROWS,
                               sp.empty() ? nullptr : sp.data(), out.data(), nullptr, nullptr);
    if (rc != VX_OK) return rc;
    const double dt = std::chrono::duration<double>(clk::now() - t0).count();
    int prefill_rows = 0;
    for (size_t i = 0; i < dec.size(); i++) {
        Seq &q = *dec[i];
        q.position++;                                                                   // AdvancePosition
        q.generated.push_back(out[i]);                                                  // AddGeneratedToken
        finish_if_done(s, q, out[i]);
    }
    for (size_t i = 0; i < pre.size(); i++) {
        Seq &q = *pre[i];
        q.fed += chunk[i]; q.position = q.fed; prefill_rows += chunk[i];
        if (q.fed == (int)q.feed.size()) {                                              // the prompt is in: its last row gave the next token
            q.state = kDecoding;
            q.generated.push_back(out[dec.size() + i]);
            finish_if_done(s, q, out[dec.size() + i]);
        }
    }
    const int rows = (int)dec.size() + prefill_rows;
    s->met.total_tokens += rows; s->met.decode_tokens += (int)dec.size(); s->met.prefill_tokens += prefill_rows;
    s->met.decode_seconds += dt * (double)dec.size() / rows;
    s->met.prefill_seconds += dt * (double)prefill_rows / rows;
    return VX_OK;
}

// drains the sequence's token channel (Sequence.TokenChan).  *finished: 0 = running, 1 = ended and drained, 2 = ended
// because it was refused (it could never fit the block pool); ended sequences whose end was reported are forgotten once
// more than a few hundred of them have piled up
int vx_sched_poll(vx_sched *s, int64_t id, int32_t *out, int cap, int *n_out, int *finished) {
    if (!s || !n_out) return VX_E_BAD_ARG;
    std::lock_guard<std::mutex> g(s->mu);
    for (auto it = s->seqs.rbegin(); it != s->seqs.rend(); ++it) {
        Seq &q = *it;
        if (q.id != id) continue;
        int n = 0;
        while (n < cap && !q.chan.empty()) { if (out) out[n] = q.chan.front(); q.chan.pop_front(); n++; }
        *n_out = n;
        const bool done = q.state == kFinished && q.chan.empty();
        if (finished) *finished = done ? (q.fail_code ? 2 : 1) : 0;
        if (done) q.reported = true;
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

// how often a sequence was preempted to free blocks, and how many requests were refused because they could never fit
int vx_sched_get_pressure(vx_sched *s, uint64_t *preemptions, uint64_t *refused) {
    if (!s) return VX_E_BAD_ARG;
    std::lock_guard<std::mutex> g(s->mu);
    if (preemptions) *preemptions = s->preemptions;
    if (refused) *refused = s->refused;
    return VX_OK;
}

}  // extern "C"
