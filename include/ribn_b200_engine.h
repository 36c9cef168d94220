/* ribn_b200_engine.h -- the host engine that drives a GenerationExecutor the way ribn's `Engine` does.
 *
 * The reference's runtime (crates/runtime) owns the rules that decide which batch shapes an executor
 * sees: decode rows first, then prefill chunks, under a token budget, with a forced prefill after
 * `max_decode_only_steps` decode-only steps (crates/runtime/src/engine/scheduling.rs:6-96); one batch in
 * flight (crates/runtime/src/engine.rs:344-398); whole-batch validation of a completion before any of it
 * is committed (crates/runtime/src/engine/completion.rs:45-131); the pre-submit negotiation over the
 * offered rows, with deferred rows parked until a resource changes (crates/runtime/src/engine/preparation.rs:5-140);
 * and a fault that is final (crates/runtime/src/engine.rs:578-594).  This is that part of the runtime as
 * native code over the C ABI of ribn_b200.h -- no mailboxes, credits, cancellation or driver thread.
 *
 * The engine talks to its executor through a table of functions with the signatures of ribn_b200.h, so the
 * same engine drives the CUDA executor (ribn_b200_engine_create_for) or a test double.
 */
#ifndef RIBN_B200_ENGINE_H
#define RIBN_B200_ENGINE_H

#include "ribn_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* The GenerationExecutor trait (crates/runtime/src/executor.rs:171-254) as the engine uses it.  Every entry
 * has the meaning and return codes of the ribn_b200_* function of the same name, with `self` in place of the
 * executor handle.  `prepare_rows` may answer RIBN_B200_OK (Ready) or RIBN_B200_SELECTED with `rows` filled. */
typedef struct {
    void* self;
    int (*info)(void* self, ribn_b200_limits* out);
    int (*admit)(void* self, uint64_t request_id, uint64_t sequence, const uint32_t* tokens, uint32_t token_count,
                 uint32_t max_output_tokens, const ribn_b200_sampling* sampling, const uint32_t* stop_tokens,
                 uint32_t stop_count);
    int (*prepare_rows)(void* self, const ribn_b200_batch_item* items, uint32_t count, ribn_b200_prepared_row* rows);
    int (*abandon_preparation)(void* self);
    int (*submit)(void* self, const ribn_b200_batch_item* items, uint32_t count, uint64_t* submission);
    int (*poll)(void* self, uint64_t submission, ribn_b200_completion* rows, uint32_t capacity, uint32_t* count);
    int (*release)(void* self, uint64_t sequence);
    size_t (*last_error)(void* self, char* buffer, size_t capacity);
} ribn_b200_executor_table;

/* EngineConfig (crates/runtime/src/config.rs:5-30). */
typedef struct {
    uint32_t max_active_requests;
    uint32_t max_queued_requests;
} ribn_b200_engine_config;

/* SchedulePolicy (crates/runtime/src/config.rs:32-56). */
typedef struct {
    uint32_t max_batch_tokens;
    uint32_t prefill_chunk_tokens;
    uint32_t decode_tokens;
    uint32_t max_decode_only_steps;
} ribn_b200_schedule_policy;

typedef struct ribn_b200_engine ribn_b200_engine;

/* Where a request is, and how it ended. */
enum { RIBN_B200_REQUEST_QUEUED = 0, RIBN_B200_REQUEST_ACTIVE = 1, RIBN_B200_REQUEST_FINISHED = 2 };
enum {
    RIBN_B200_FINISH_NONE = 0,
    RIBN_B200_FINISH_STOP = 1,      /* a stop token was sampled (it is not part of the output) */
    RIBN_B200_FINISH_LENGTH = 2,    /* max_output_tokens reached */
    RIBN_B200_FINISH_REJECTED = 3,  /* Admission::Rejected */
    RIBN_B200_FINISH_FAILED = 4     /* rejected at preparation, or the KV arena can never serve it */
};
typedef struct {
    uint32_t state;          /* RIBN_B200_REQUEST_* */
    uint32_t finish;         /* RIBN_B200_FINISH_* */
    uint32_t prompt_tokens;
    uint32_t prefix;         /* committed prefix */
    uint32_t generated;      /* sampled tokens, a stop token included */
    uint32_t output_tokens;  /* tokens in the output */
    uint64_t enqueue_ns;     /* steady clock, nanoseconds */
    uint64_t first_token_ns; /* 0 until the first output token is committed */
    uint64_t last_token_ns;
} ribn_b200_request_status;

typedef struct {
    uint64_t steps;              /* batches submitted */
    uint32_t decode_only_steps;  /* since the last batch with a prefill row, while prefill rows wait */
    uint32_t waiting, prefill, decode, parked, in_flight_rows;
    uint64_t resource_epoch;     /* releases so far: what a parked row waits on */
    uint32_t faulted;
    uint32_t reserved;
} ribn_b200_engine_counts;

/* Engine::new (crates/runtime/src/engine.rs:100-148) with validate_policy (crates/runtime/src/config.rs:58-72):
 * every policy field positive, max_batch_tokens and decode_tokens within the executor's limits,
 * max_active_requests within its max_sequences.  The table is copied; `self` must outlive the engine. */
RIBN_B200_API int ribn_b200_engine_create(const ribn_b200_executor_table* executor, const ribn_b200_engine_config* config,
                                          const ribn_b200_schedule_policy* policy, ribn_b200_engine** out, char* error,
                                          size_t error_capacity);
/* The same over a CUDA executor of this library (finalized, not tensor-parallel). */
RIBN_B200_API int ribn_b200_engine_create_for(ribn_b200_executor* executor, const ribn_b200_engine_config* config,
                                              const ribn_b200_schedule_policy* policy, ribn_b200_engine** out,
                                              char* error, size_t error_capacity);
RIBN_B200_API int ribn_b200_engine_destroy(ribn_b200_engine* engine);

/* Queue a request (its sequence id is its request id).  OK with `*request` set, REJECTED when the queue holds
 * max_queued_requests already, ERROR on a bad argument. */
RIBN_B200_API int ribn_b200_engine_enqueue(ribn_b200_engine* engine, const uint32_t* tokens, uint32_t token_count,
                                           uint32_t max_output_tokens, const uint32_t* stop_tokens, uint32_t stop_count,
                                           float temperature, uint64_t* request);
/* Engine::step: poll the batch in flight (PENDING: nothing else happens), commit it, release what ended, offer
 * parked rows again, admit waiters, build the next batch, negotiate it, submit it.  OK with `*progressed` 0 / 1,
 * or ERROR: the engine is faulted for good and every later step returns ERROR. */
RIBN_B200_API int ribn_b200_engine_step(ribn_b200_engine* engine, int32_t* progressed);
/* 1 when nothing is queued, active, parked or in flight. */
RIBN_B200_API int ribn_b200_engine_idle(ribn_b200_engine* engine);
RIBN_B200_API int ribn_b200_engine_status(ribn_b200_engine* engine, uint64_t request, ribn_b200_request_status* out);
/* The request's output tokens so far: copies at most `capacity`, reports how many there are. */
RIBN_B200_API int ribn_b200_engine_output(ribn_b200_engine* engine, uint64_t request, uint32_t* tokens,
                                          uint32_t capacity, uint32_t* count);
/* When each output token was committed (steady clock, nanoseconds; the clock of enqueue_ns): copies at most
 * `capacity` stamps, reports how many there are. */
RIBN_B200_API int ribn_b200_engine_token_times(ribn_b200_engine* engine, uint64_t request, uint64_t* stamps,
                                               uint32_t capacity, uint32_t* count);
/* Why the request ended, as text ("length", "stop", "rejected: ...", "failed: ..."); returns the length. */
RIBN_B200_API size_t ribn_b200_engine_finish_reason(ribn_b200_engine* engine, uint64_t request, char* buffer,
                                                    size_t capacity);
RIBN_B200_API int ribn_b200_engine_counters(ribn_b200_engine* engine, ribn_b200_engine_counts* out);
RIBN_B200_API size_t ribn_b200_engine_last_error(ribn_b200_engine* engine, char* buffer, size_t capacity);

#ifdef __cplusplus
}
#endif
#endif /* RIBN_B200_ENGINE_H */
