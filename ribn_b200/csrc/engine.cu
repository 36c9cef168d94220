// The host engine behind include/ribn_b200_engine.h: the scheduling, negotiation, validation and fault rules of
// the reference's runtime engine (crates/runtime/src/engine.rs, engine/scheduling.rs, engine/preparation.rs,
// engine/completion.rs) over a table of executor functions.  Host code only: nothing here touches the device.
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/ribn_b200_engine.h"

namespace {

struct Slot {
    uint64_t request = 0, sequence = 0;
    std::vector<uint32_t> prompt, stop, output;
    std::vector<uint64_t> token_ns;   // when each output token was committed
    uint32_t max_output = 0;
    float temperature = 0.0f;
    uint32_t prefix = 0, generated = 0;
    uint32_t state = RIBN_B200_REQUEST_QUEUED, finish = RIBN_B200_FINISH_NONE;
    std::string reason;
    uint64_t enqueue_ns = 0, first_token_ns = 0, last_token_ns = 0;
    uint64_t parked_epoch = 0;
    uint32_t prompt_tokens() const { return (uint32_t)prompt.size(); }
};

uint64_t now_ns() {
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

}  // namespace

struct ribn_b200_engine {
    ribn_b200_executor_table ex{};
    ribn_b200_engine_config config{};
    ribn_b200_schedule_policy policy{};
    std::deque<uint64_t> waiting, prefill, decode, parked;
    std::unordered_map<uint64_t, Slot> slots;  // every request ever queued; `state` says where it is
    uint64_t resource_epoch = 0, next_id = 1, steps = 0;
    uint32_t decode_only_steps = 0;
    bool faulted = false;
    // the batch in flight
    bool in_flight = false;
    uint64_t submission = 0;
    std::vector<ribn_b200_batch_item> flight_items;
    std::vector<uint64_t> flight_keys;
    std::string error;

    int fail(const char* fmt, ...) {
        char buf[4096];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof(buf), fmt, ap);
        va_end(ap);
        error = buf;
        return RIBN_B200_ERROR;
    }
    // An executor call failed: keep its diagnostic.
    int executor_failed(const char* what) {
        char buf[4096] = {0};
        if (ex.last_error != nullptr) ex.last_error(ex.self, buf, sizeof(buf));
        return fail("%s: %s", what, buf[0] ? buf : "executor error");
    }

    size_t active() const { return prefill.size() + decode.size() + parked.size() + (in_flight ? flight_keys.size() : 0); }
    bool idle() const { return waiting.empty() && prefill.empty() && decode.empty() && parked.empty() && !in_flight; }

    // A request ends: its sequence goes back to the executor, and whoever waits on resources may try again.
    int finish(uint64_t rid, uint32_t how, const std::string& reason) {
        Slot& s = slots[rid];
        s.finish = how;
        s.reason = reason;
        s.state = RIBN_B200_REQUEST_FINISHED;
        if (ex.release(ex.self, s.sequence) != RIBN_B200_OK) return executor_failed("release");
        ++resource_epoch;
        return RIBN_B200_OK;
    }

    // reactivate_parked (engine/preparation.rs:118-140): a parked row returns to its queue once the resource it
    // waits for has changed (any release since it was parked).
    void reactivate_parked() {
        for (size_t n = parked.size(); n > 0; --n) {
            const uint64_t rid = parked.front();
            parked.pop_front();
            Slot& s = slots[rid];
            if (s.parked_epoch == resource_epoch) { parked.push_back(rid); continue; }
            (s.prefix < s.prompt_tokens() ? prefill : decode).push_back(rid);
        }
    }

    int admit_waiters() {
        for (size_t n = waiting.size(); n > 0; --n) {
            if (active() >= config.max_active_requests) break;
            const uint64_t rid = waiting.front();
            Slot& s = slots[rid];
            ribn_b200_sampling sampling{};
            sampling.temperature = s.temperature;
            sampling.top_p = 1.0f;
            const int rc = ex.admit(ex.self, rid, s.sequence, s.prompt.data(), s.prompt_tokens(), s.max_output, &sampling,
                                    s.stop.empty() ? nullptr : s.stop.data(), (uint32_t)s.stop.size());
            if (rc == RIBN_B200_DEFERRED) break;
            if (rc != RIBN_B200_OK && rc != RIBN_B200_REJECTED) return executor_failed("admit");
            waiting.pop_front();
            if (rc == RIBN_B200_REJECTED) {
                char buf[1024] = {0};
                if (ex.last_error != nullptr) ex.last_error(ex.self, buf, sizeof(buf));
                s.finish = RIBN_B200_FINISH_REJECTED;
                s.reason = std::string("rejected: ") + buf;
                s.state = RIBN_B200_REQUEST_FINISHED;
                continue;
            }
            s.state = RIBN_B200_REQUEST_ACTIVE;
            prefill.push_back(rid);
        }
        return RIBN_B200_OK;
    }

    // schedule_kind (engine/scheduling.rs:39-96): rows of one kind, oldest first, while budget and row slots last.
    uint32_t schedule(uint32_t kind, uint32_t budget, uint32_t limit, std::vector<ribn_b200_batch_item>& batch,
                      std::vector<uint64_t>& keys) {
        std::deque<uint64_t>& queue = kind == RIBN_B200_PREFILL ? prefill : decode;
        uint32_t selected = 0;
        for (size_t n = queue.size(); n > 0; --n) {
            if (selected >= limit || batch.size() >= config.max_active_requests || budget == 0) break;
            const uint64_t rid = queue.front();
            queue.pop_front();
            const Slot& s = slots[rid];
            uint32_t tokens, outputs;
            if (kind == RIBN_B200_PREFILL) {
                tokens = std::min(std::min(s.prompt_tokens() - s.prefix, policy.prefill_chunk_tokens), budget);
                outputs = s.prefix + tokens == s.prompt_tokens() ? 1u : 0u;
            } else {
                tokens = std::min(std::min(policy.decode_tokens, s.max_output - s.generated), budget);
                outputs = tokens;
            }
            if (tokens == 0) { queue.push_back(rid); continue; }
            batch.push_back(ribn_b200_batch_item{s.sequence, kind, s.prefix, tokens, outputs});
            keys.push_back(rid);
            budget -= tokens;
            ++selected;
        }
        return budget;
    }

    // build_batch (engine/scheduling.rs:6-37): a forced prefill row when decode-only steps have starved the
    // prefill queue, then decode rows, then prefill chunks with what is left of the budget.
    void build_batch(std::vector<ribn_b200_batch_item>& batch, std::vector<uint64_t>& keys) {
        uint32_t budget = policy.max_batch_tokens;
        if (!prefill.empty() && decode_only_steps >= policy.max_decode_only_steps) {
            budget = schedule(RIBN_B200_PREFILL, budget, 1, batch, keys);
        }
        budget = schedule(RIBN_B200_DECODE, budget, 0xffffffffu, batch, keys);
        schedule(RIBN_B200_PREFILL, budget, 0xffffffffu, batch, keys);
    }

    // prepare_batch (engine/preparation.rs:5-86): Ready keeps the batch; Selected keeps its ready rows with the
    // granted budgets, parks the deferred ones and fails the rejected ones.
    int prepare(std::vector<ribn_b200_batch_item>& batch, std::vector<uint64_t>& keys) {
        std::vector<ribn_b200_prepared_row> rows(batch.size());
        const int rc = ex.prepare_rows(ex.self, batch.data(), (uint32_t)batch.size(), rows.data());
        if (rc == RIBN_B200_OK) return RIBN_B200_OK;
        if (rc != RIBN_B200_SELECTED) return executor_failed("prepare");
        std::vector<ribn_b200_batch_item> kept;
        std::vector<uint64_t> kept_keys;
        for (size_t i = 0; i < batch.size(); ++i) {
            const ribn_b200_batch_item& offered = batch[i];
            const uint64_t rid = keys[i];
            Slot& s = slots[rid];
            if (rows[i].state == RIBN_B200_ROW_READY) {
                const uint32_t tokens = rows[i].token_budget, outputs = rows[i].output_budget;
                bool ok = tokens > 0 && tokens <= offered.token_budget && outputs <= offered.output_budget;
                if (offered.kind == RIBN_B200_PREFILL) {
                    const uint32_t end = offered.prefix + tokens;
                    ok = ok && end <= s.prompt_tokens() && outputs == (end == s.prompt_tokens() ? 1u : 0u);
                } else {
                    ok = ok && outputs == tokens;
                }
                if (!ok) {
                    ex.abandon_preparation(ex.self);
                    return fail("preparation does not match its offered rows or budgets");
                }
                kept.push_back(ribn_b200_batch_item{offered.sequence, offered.kind, offered.prefix, tokens, outputs});
                kept_keys.push_back(rid);
            } else if (rows[i].state == RIBN_B200_ROW_DEFERRED) {
                s.parked_epoch = resource_epoch;
                parked.push_back(rid);
            } else if (rows[i].state == RIBN_B200_ROW_REJECTED) {
                // the preparation still names the row: the executor lets go of it when the batch is abandoned or run
                pending_failures.push_back(rid);
            } else {
                ex.abandon_preparation(ex.self);
                return fail("preparation does not match its offered rows or budgets");
            }
        }
        if (kept.empty() && ex.abandon_preparation(ex.self) != RIBN_B200_OK) return executor_failed("abandon_preparation");
        batch.swap(kept);
        keys.swap(kept_keys);
        return RIBN_B200_OK;
    }
    std::vector<uint64_t> pending_failures;   // rows rejected at preparation, finished once no preparation names them

    int flush_failures() {
        for (uint64_t rid : pending_failures) {
            const int rc = finish(rid, RIBN_B200_FINISH_FAILED, "failed: rejected at preparation");
            if (rc != RIBN_B200_OK) return rc;
        }
        pending_failures.clear();
        return RIBN_B200_OK;
    }

    // complete_step (engine/completion.rs:45-131): every row is checked against what was submitted before any
    // of them is committed.
    int commit(const std::vector<ribn_b200_completion>& rows) {
        if (rows.size() != flight_items.size()) return fail("malformed completion: row count");
        for (size_t i = 0; i < rows.size(); ++i) {
            const ribn_b200_completion& row = rows[i];
            const ribn_b200_batch_item& item = flight_items[i];
            const Slot& s = slots[flight_keys[i]];
            const int64_t advance = (int64_t)row.prefix - (int64_t)item.prefix;
            bool ok = row.sequence == item.sequence && s.prefix == item.prefix && advance > 0 && advance <= (int64_t)item.token_budget;
            if (item.kind == RIBN_B200_PREFILL) {
                ok = ok && row.n_tokens == (row.prefix == s.prompt_tokens() ? 1u : 0u);
            } else {
                ok = ok && (int64_t)row.n_tokens == advance && row.n_tokens <= item.output_budget;
            }
            if (!ok) return fail("malformed completion");
        }
        const uint64_t now = now_ns();
        const std::vector<uint64_t> keys = flight_keys;
        in_flight = false;
        flight_items.clear();
        flight_keys.clear();
        for (size_t i = 0; i < rows.size(); ++i) {
            const uint64_t rid = keys[i];
            Slot& s = slots[rid];
            s.prefix = rows[i].prefix;
            uint32_t how = RIBN_B200_FINISH_NONE;
            if (rows[i].n_tokens > 0) {   // max_decode_tokens is 1: a row carries at most one token
                const uint32_t token = rows[i].token;
                ++s.generated;
                bool stop = false;
                for (uint32_t t : s.stop) stop = stop || t == token;
                if (stop) {
                    how = RIBN_B200_FINISH_STOP;
                } else {
                    s.output.push_back(token);
                    s.token_ns.push_back(now);
                    if (s.first_token_ns == 0) s.first_token_ns = now;
                    s.last_token_ns = now;
                    if (s.generated == s.max_output) how = RIBN_B200_FINISH_LENGTH;
                }
            }
            if (how != RIBN_B200_FINISH_NONE) {
                const int rc = finish(rid, how, how == RIBN_B200_FINISH_STOP ? "stop" : "length");
                if (rc != RIBN_B200_OK) return rc;
            } else if (s.prefix < s.prompt_tokens()) {
                prefill.push_back(rid);
            } else {
                decode.push_back(rid);
            }
        }
        return RIBN_B200_OK;
    }

    int step_inner(int32_t* progressed) {
        *progressed = 0;
        if (in_flight) {
            std::vector<ribn_b200_completion> rows(flight_items.size() + 1);
            uint32_t count = 0;
            const int rc = ex.poll(ex.self, submission, rows.data(), (uint32_t)rows.size(), &count);
            if (rc == RIBN_B200_PENDING) return RIBN_B200_OK;
            if (rc != RIBN_B200_OK) return executor_failed("poll");
            rows.resize(std::min<size_t>(count, rows.size()));
            const int done = commit(rows);
            if (done != RIBN_B200_OK) return done;
            *progressed = 1;
        }
        reactivate_parked();
        int rc = admit_waiters();
        if (rc != RIBN_B200_OK) return rc;
        std::vector<ribn_b200_batch_item> batch;
        std::vector<uint64_t> keys;
        build_batch(batch, keys);
        if (!batch.empty()) {
            rc = prepare(batch, keys);
            if (rc != RIBN_B200_OK) return rc;
        }
        if (!batch.empty()) {
            uint64_t sid = 0;
            if (ex.submit(ex.self, batch.data(), (uint32_t)batch.size(), &sid) != RIBN_B200_OK) return executor_failed("submit");
            in_flight = true;
            submission = sid;
            flight_items = batch;
            flight_keys = keys;
            // record_batch (engine/scheduling.rs:98-110)
            bool any_prefill = false;
            for (const ribn_b200_batch_item& it : batch) any_prefill = any_prefill || it.kind == RIBN_B200_PREFILL;
            if (any_prefill) decode_only_steps = 0;
            else if (!prefill.empty()) ++decode_only_steps;
            ++steps;
            *progressed = 1;
        }
        // rows rejected at preparation: no preparation names them any more
        rc = flush_failures();
        if (rc != RIBN_B200_OK) return rc;
        if (batch.empty() && !parked.empty() && !in_flight && prefill.empty() && decode.empty()) {
            // Every live sequence is parked and nothing is in flight, so no release can come: the most recently
            // admitted one gives its pages back and the others are offered again.  (The reference leaves this
            // policy to the executor's ReadinessWait source.)
            uint64_t victim = 0;
            for (uint64_t rid : parked) victim = std::max(victim, rid);
            for (auto it = parked.begin(); it != parked.end(); ++it) {
                if (*it == victim) { parked.erase(it); break; }
            }
            rc = finish(victim, RIBN_B200_FINISH_FAILED, "failed: KV arena exhausted");
            if (rc != RIBN_B200_OK) return rc;
            *progressed = 1;
        }
        return RIBN_B200_OK;
    }
};

namespace {

int report(char* error, size_t capacity, const char* message) {
    if (error != nullptr && capacity > 0) snprintf(error, capacity, "%s", message);
    return RIBN_B200_ERROR;
}

// The table over this library's CUDA executor.
int ex_info(void* self, ribn_b200_limits* out) { return ribn_b200_info((ribn_b200_executor*)self, out); }
int ex_admit(void* self, uint64_t request_id, uint64_t sequence, const uint32_t* tokens, uint32_t token_count,
             uint32_t max_output_tokens, const ribn_b200_sampling* sampling, const uint32_t* stop_tokens, uint32_t stop_count) {
    return ribn_b200_admit((ribn_b200_executor*)self, request_id, sequence, tokens, token_count, max_output_tokens, sampling,
                           stop_tokens, stop_count);
}
int ex_prepare_rows(void* self, const ribn_b200_batch_item* items, uint32_t count, ribn_b200_prepared_row* rows) {
    return ribn_b200_prepare_rows((ribn_b200_executor*)self, items, count, rows);
}
int ex_abandon(void* self) { return ribn_b200_abandon_preparation((ribn_b200_executor*)self); }
int ex_submit(void* self, const ribn_b200_batch_item* items, uint32_t count, uint64_t* submission) {
    return ribn_b200_submit((ribn_b200_executor*)self, items, count, submission);
}
int ex_poll(void* self, uint64_t submission, ribn_b200_completion* rows, uint32_t capacity, uint32_t* count) {
    return ribn_b200_poll((ribn_b200_executor*)self, submission, rows, capacity, count);
}
int ex_release(void* self, uint64_t sequence) { return ribn_b200_release((ribn_b200_executor*)self, sequence); }
size_t ex_last_error(void* self, char* buffer, size_t capacity) {
    return ribn_b200_last_error((ribn_b200_executor*)self, buffer, capacity);
}

}  // namespace

extern "C" {

int ribn_b200_engine_create(const ribn_b200_executor_table* executor, const ribn_b200_engine_config* config,
                            const ribn_b200_schedule_policy* policy, ribn_b200_engine** out, char* error,
                            size_t error_capacity) {
    if (executor == nullptr || config == nullptr || policy == nullptr || out == nullptr) return report(error, error_capacity, "null argument");
    if (executor->info == nullptr || executor->admit == nullptr || executor->prepare_rows == nullptr ||
        executor->abandon_preparation == nullptr || executor->submit == nullptr || executor->poll == nullptr ||
        executor->release == nullptr) {
        return report(error, error_capacity, "the executor table is incomplete");
    }
    ribn_b200_limits limits{};
    if (executor->info(executor->self, &limits) != RIBN_B200_OK) return report(error, error_capacity, "the executor does not answer info()");
    if (policy->max_batch_tokens == 0 || policy->prefill_chunk_tokens == 0 || policy->decode_tokens == 0 ||
        policy->max_decode_only_steps == 0 || policy->max_batch_tokens > limits.max_batch_tokens ||
        policy->decode_tokens > limits.max_decode_tokens || config->max_active_requests == 0 ||
        config->max_active_requests > limits.max_sequences) {
        return report(error, error_capacity, "invalid engine configuration for this executor");
    }
    ribn_b200_engine* e = new ribn_b200_engine();
    e->ex = *executor;
    e->config = *config;
    e->policy = *policy;
    *out = e;
    return RIBN_B200_OK;
}

int ribn_b200_engine_create_for(ribn_b200_executor* executor, const ribn_b200_engine_config* config,
                                const ribn_b200_schedule_policy* policy, ribn_b200_engine** out, char* error,
                                size_t error_capacity) {
    if (executor == nullptr) return report(error, error_capacity, "null argument");
    ribn_b200_executor_table table{};
    table.self = executor;
    table.info = ex_info;
    table.admit = ex_admit;
    table.prepare_rows = ex_prepare_rows;
    table.abandon_preparation = ex_abandon;
    table.submit = ex_submit;
    table.poll = ex_poll;
    table.release = ex_release;
    table.last_error = ex_last_error;
    return ribn_b200_engine_create(&table, config, policy, out, error, error_capacity);
}

int ribn_b200_engine_destroy(ribn_b200_engine* engine) {
    delete engine;
    return RIBN_B200_OK;
}

int ribn_b200_engine_enqueue(ribn_b200_engine* engine, const uint32_t* tokens, uint32_t token_count, uint32_t max_output_tokens,
                             const uint32_t* stop_tokens, uint32_t stop_count, float temperature, uint64_t* request) {
    if (engine == nullptr) return RIBN_B200_ERROR;
    if (tokens == nullptr || token_count == 0 || request == nullptr || (stop_count > 0 && stop_tokens == nullptr)) {
        return engine->fail("enqueue: a request needs tokens and a place for its id");
    }
    if (engine->waiting.size() >= engine->config.max_queued_requests) {
        engine->error = "queue full";
        return RIBN_B200_REJECTED;
    }
    const uint64_t rid = engine->next_id++;
    Slot& s = engine->slots[rid];
    s.request = s.sequence = rid;
    s.prompt.assign(tokens, tokens + token_count);
    if (stop_count > 0) s.stop.assign(stop_tokens, stop_tokens + stop_count);
    s.max_output = max_output_tokens;
    s.temperature = temperature;
    s.enqueue_ns = now_ns();
    engine->waiting.push_back(rid);
    *request = rid;
    return RIBN_B200_OK;
}

int ribn_b200_engine_step(ribn_b200_engine* engine, int32_t* progressed) {
    if (engine == nullptr) return RIBN_B200_ERROR;
    int32_t local = 0;
    if (progressed == nullptr) progressed = &local;
    *progressed = 0;
    if (engine->faulted) return engine->fail("engine is faulted");
    const int rc = engine->step_inner(progressed);
    if (rc != RIBN_B200_OK) engine->faulted = true;   // fault_all (crates/runtime/src/engine.rs:578-594)
    return rc;
}

int ribn_b200_engine_idle(ribn_b200_engine* engine) { return engine != nullptr && engine->idle() ? 1 : 0; }

int ribn_b200_engine_status(ribn_b200_engine* engine, uint64_t request, ribn_b200_request_status* out) {
    if (engine == nullptr || out == nullptr) return RIBN_B200_ERROR;
    const auto it = engine->slots.find(request);
    if (it == engine->slots.end()) return engine->fail("unknown request %llu", (unsigned long long)request);
    const Slot& s = it->second;
    *out = ribn_b200_request_status{s.state, s.finish, s.prompt_tokens(), s.prefix, s.generated, (uint32_t)s.output.size(),
                                    s.enqueue_ns, s.first_token_ns, s.last_token_ns};
    return RIBN_B200_OK;
}

int ribn_b200_engine_output(ribn_b200_engine* engine, uint64_t request, uint32_t* tokens, uint32_t capacity, uint32_t* count) {
    if (engine == nullptr) return RIBN_B200_ERROR;
    const auto it = engine->slots.find(request);
    if (it == engine->slots.end()) return engine->fail("unknown request %llu", (unsigned long long)request);
    const std::vector<uint32_t>& out = it->second.output;
    if (count != nullptr) *count = (uint32_t)out.size();
    if (tokens != nullptr && capacity > 0 && !out.empty()) {
        memcpy(tokens, out.data(), std::min<size_t>(capacity, out.size()) * sizeof(uint32_t));
    }
    return RIBN_B200_OK;
}

int ribn_b200_engine_token_times(ribn_b200_engine* engine, uint64_t request, uint64_t* stamps, uint32_t capacity, uint32_t* count) {
    if (engine == nullptr) return RIBN_B200_ERROR;
    const auto it = engine->slots.find(request);
    if (it == engine->slots.end()) return engine->fail("unknown request %llu", (unsigned long long)request);
    const std::vector<uint64_t>& ns = it->second.token_ns;
    if (count != nullptr) *count = (uint32_t)ns.size();
    if (stamps != nullptr && capacity > 0 && !ns.empty()) {
        memcpy(stamps, ns.data(), std::min<size_t>(capacity, ns.size()) * sizeof(uint64_t));
    }
    return RIBN_B200_OK;
}

size_t ribn_b200_engine_finish_reason(ribn_b200_engine* engine, uint64_t request, char* buffer, size_t capacity) {
    if (engine == nullptr) return 0;
    const auto it = engine->slots.find(request);
    if (it == engine->slots.end()) return 0;
    if (buffer != nullptr && capacity > 0) snprintf(buffer, capacity, "%s", it->second.reason.c_str());
    return it->second.reason.size();
}

int ribn_b200_engine_counters(ribn_b200_engine* engine, ribn_b200_engine_counts* out) {
    if (engine == nullptr || out == nullptr) return RIBN_B200_ERROR;
    *out = ribn_b200_engine_counts{engine->steps, engine->decode_only_steps, (uint32_t)engine->waiting.size(),
                                     (uint32_t)engine->prefill.size(), (uint32_t)engine->decode.size(),
                                     (uint32_t)engine->parked.size(), engine->in_flight ? (uint32_t)engine->flight_keys.size() : 0u,
                                     engine->resource_epoch, engine->faulted ? 1u : 0u, 0u};
    return RIBN_B200_OK;
}

size_t ribn_b200_engine_last_error(ribn_b200_engine* engine, char* buffer, size_t capacity) {
    if (engine == nullptr) return 0;
    if (buffer != nullptr && capacity > 0) snprintf(buffer, capacity, "%s", engine->error.c_str());
    return engine->error.size();
}

}  // extern "C"
