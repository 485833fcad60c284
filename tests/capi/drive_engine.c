/* Drives the engine through include/celeg_b200/api.h alone: loads the model folder given as the first
 * argument, submits the prompt given as further arguments (token ids), steps until the request is finished and
 * prints "tokens: a b c ...", "fingerprint: <hex>" and "steps: n". dtype: second argument, 0 = bfloat16,
 * 1 = float32. Exit code 0 on success; on failure the library's message goes to stderr. */
#include <stdio.h>
#include <stdlib.h>

#include "celeg_b200/api.h"

int main(int argc, char** argv) {
    if (argc < 5) {
        fprintf(stderr, "usage: %s MODEL_DIR DTYPE MAX_NEW TOKEN [TOKEN ...]\n", argv[0]);
        return 2;
    }
    celeg_b200_engine_options options;
    celeg_b200_engine_options_init(&options);
    options.dtype = atoi(argv[2]);
    options.max_active_requests = 2;
    options.max_batched_tokens = 64;
    options.prefill_chunk_tokens = 7;
    celeg_b200_engine* engine = celeg_b200_engine_create(argv[1], &options);
    if (engine == NULL) {
        fprintf(stderr, "create failed: %s\n", celeg_b200_engine_last_error(NULL));
        return 1;
    }
    int32_t prompt[256];
    size_t count = 0;
    for (int i = 4; i < argc && count < 256; ++i) prompt[count++] = (int32_t)atoi(argv[i]);
    celeg_b200_request_options request;
    celeg_b200_request_options_init(&request);
    request.max_new_tokens = (uint32_t)atoi(argv[3]);
    request.eos_token_id = -2;
    request.generation.temperature = 0.0f;
    request.generation.top_k = 1;
    request.generation.repetition_penalty = 1.0f;
    celeg_b200_request_id id = 0;
    if (celeg_b200_engine_submit(engine, prompt, count, &request, &id) != CELEG_B200_STATUS_OK) {
        fprintf(stderr, "submit failed: %s\n", celeg_b200_engine_last_error(engine));
        return 1;
    }
    int32_t out[64];
    int finished = 0, steps = 0;
    printf("tokens:");
    while (!finished && steps < 10000) {
        int progressed = 0;
        if (celeg_b200_engine_step(engine, &progressed) != CELEG_B200_STATUS_OK) {
            fprintf(stderr, "step failed: %s\n", celeg_b200_engine_last_error(engine));
            return 1;
        }
        ++steps;
        size_t got = 0;
        if (celeg_b200_engine_poll(engine, id, out, 64, &got, &finished) != CELEG_B200_STATUS_OK) {
            fprintf(stderr, "poll failed: %s\n", celeg_b200_engine_last_error(engine));
            return 1;
        }
        for (size_t i = 0; i < got; ++i) printf(" %d", out[i]);
    }
    printf("\n");
    char fingerprint[80];
    if (celeg_b200_engine_fingerprint(engine, fingerprint, sizeof(fingerprint)) == CELEG_B200_STATUS_OK)
        printf("fingerprint: %s\n", fingerprint);
    celeg_b200_metrics metrics;
    metrics.struct_size = sizeof(metrics);
    if (celeg_b200_engine_get_metrics(engine, &metrics) == CELEG_B200_STATUS_OK)
        printf("steps: %llu completed: %llu\n", (unsigned long long)metrics.steps, (unsigned long long)metrics.completed);
    celeg_b200_engine_destroy(engine);
    return finished ? 0 : 1;
}
