/* C interface of the celeg_b200 engine: one model folder on one B200, requests in as token ids, tokens
 * out. The calls and their meanings follow celsowm/celeg's engine API (include/celeg/api.h:142-179:
 * celeg_engine_create / _submit / _poll / _status / _cancel / _step / _destroy / _last_error); names carry
 * the prefix celeg_b200_ so that both libraries can live in one process. Option structs carry their own
 * size in `struct_size` and are filled with defaults by their *_init function; a struct that is smaller
 * than the library's is refused (celeg: src/api/api_common.cpp require_size).
 *
 * The library (libceleg_b200_api.so, built by `python -m celeg_b200.capi.build`) hosts the engine's Python
 * host side in an embedded interpreter when the process has none, or uses the running one; every call may
 * come from any thread. Token ids are int32; request ids are positive. The engine does not run by itself
 * unless celeg_b200_engine_start is called: celeg_b200_engine_step runs one scheduler step.
 */
#ifndef CELEG_B200_API_H
#define CELEG_B200_API_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define CELEG_B200_API __attribute__((visibility("default")))
#else
#define CELEG_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum celeg_b200_status {
    CELEG_B200_STATUS_OK = 0,
    CELEG_B200_STATUS_INVALID_ARGUMENT = 1,
    CELEG_B200_STATUS_ERROR = 2,
    CELEG_B200_STATUS_BUFFER_TOO_SMALL = 3,
    CELEG_B200_STATUS_NOT_FOUND = 4,
    CELEG_B200_STATUS_BACKEND_UNAVAILABLE = 5
} celeg_b200_status;

typedef enum celeg_b200_request_status {
    CELEG_B200_REQUEST_QUEUED = 0, CELEG_B200_REQUEST_PREFILLING = 1, CELEG_B200_REQUEST_DECODING = 2,
    CELEG_B200_REQUEST_COMPLETED = 3, CELEG_B200_REQUEST_CANCELLED = 4, CELEG_B200_REQUEST_FAILED = 5
} celeg_b200_request_status;

typedef struct celeg_b200_engine celeg_b200_engine;
typedef uint64_t celeg_b200_request_id;

typedef struct celeg_b200_generation_options {
    uint32_t struct_size;
    float temperature;            /* <= 0: greedy */
    int32_t top_k;                /* 1: greedy; at most 128 */
    float top_p;                  /* (0, 1] */
    float repetition_penalty;     /* >= 1 */
    uint64_t seed;                /* non-zero */
} celeg_b200_generation_options;

typedef struct celeg_b200_engine_options {
    uint32_t struct_size;
    int32_t max_context;          /* 0: the model's own limit */
    int32_t dtype;                /* 0: bfloat16 (serving), 1: float32 (everything in true 32-bit) */
    int32_t device;               /* CUDA device index */
    int32_t cuda_graph;           /* 1: decode steps and repeated prompt steps replay captured graphs */
    int32_t max_active_requests;  /* celeg's ConcurrentEngineOptions, same names and defaults: 8 */
    int32_t max_batched_tokens;   /* 512 */
    int32_t prefill_chunk_tokens; /* 256 */
    int32_t page_tokens;          /* 16 */
    uint64_t logical_kv_pages;    /* 0: ceil(max_context / page_tokens) * max_active_requests */
    int32_t scheduler_policy;     /* 0: guaranteed-no-evict, 1: max-utilization */
} celeg_b200_engine_options;

typedef struct celeg_b200_request_options {
    uint32_t struct_size;
    uint32_t max_new_tokens;      /* 128 */
    int32_t eos_token_id;         /* -1: the stop ids of the model's configuration; -2: none */
    int32_t priority;
    celeg_b200_generation_options generation;
} celeg_b200_request_options;

typedef struct celeg_b200_metrics {
    uint32_t struct_size;
    uint64_t submitted, completed, cancelled, failed, preempted, steps, prefill_tokens, decode_tokens;
    uint64_t active_requests, queued_requests, pages_used, pages_total, pages_high_water;
    double ttft_ms_sum;
    uint64_t ttft_samples;
    double itl_ms_sum;
    uint64_t itl_samples;
    double host_ms_sum;           /* plan + launch + commit, summed over steps */
    double gpu_ms_sum;            /* device time of the steps */
} celeg_b200_metrics;

CELEG_B200_API void celeg_b200_engine_options_init(celeg_b200_engine_options* options);
CELEG_B200_API void celeg_b200_request_options_init(celeg_b200_request_options* options);

/* NULL on failure; celeg_b200_engine_last_error(NULL) then says why. */
CELEG_B200_API celeg_b200_engine* celeg_b200_engine_create(const char* model_path,
                                                           const celeg_b200_engine_options* options);
CELEG_B200_API void celeg_b200_engine_destroy(celeg_b200_engine* engine);
CELEG_B200_API celeg_b200_status celeg_b200_engine_submit(celeg_b200_engine* engine, const int32_t* tokens,
                                                          size_t count, const celeg_b200_request_options* options,
                                                          celeg_b200_request_id* request_id);
/* Pops up to `capacity` tokens produced since the last poll; *finished once the request is terminal and
 * nothing is left to pop. */
CELEG_B200_API celeg_b200_status celeg_b200_engine_poll(celeg_b200_engine* engine, celeg_b200_request_id request_id,
                                                        int32_t* output, size_t capacity, size_t* count,
                                                        int* finished);
CELEG_B200_API celeg_b200_status celeg_b200_engine_status(celeg_b200_engine* engine, celeg_b200_request_id request_id,
                                                          celeg_b200_request_status* status);
CELEG_B200_API celeg_b200_status celeg_b200_engine_cancel(celeg_b200_engine* engine, celeg_b200_request_id request_id);
/* Forget a terminal request. */
CELEG_B200_API celeg_b200_status celeg_b200_engine_release(celeg_b200_engine* engine, celeg_b200_request_id request_id);
CELEG_B200_API celeg_b200_status celeg_b200_engine_step(celeg_b200_engine* engine, int* progressed);
/* Steps on a worker thread until _stop (celeg's engine does that by default; here it is a choice). */
CELEG_B200_API celeg_b200_status celeg_b200_engine_start(celeg_b200_engine* engine);
CELEG_B200_API celeg_b200_status celeg_b200_engine_stop(celeg_b200_engine* engine);
CELEG_B200_API celeg_b200_status celeg_b200_engine_get_metrics(celeg_b200_engine* engine, celeg_b200_metrics* metrics);
/* 64 hexadecimal digits and a terminating zero: the hash of the resolved configuration and the tensor table. */
CELEG_B200_API celeg_b200_status celeg_b200_engine_fingerprint(celeg_b200_engine* engine, char* output, size_t capacity);
/* The message of the last failed call on this engine (or, with NULL, of the last failed create). */
CELEG_B200_API const char* celeg_b200_engine_last_error(const celeg_b200_engine* engine);

#ifdef __cplusplus
}
#endif

#endif
