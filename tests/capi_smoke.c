/* A plain C program over libqengine: it includes inference.h, links nothing but the library, loads a model folder
 * and prints tokens.  The test that builds and runs it (tests/test_gpu_capi.py) compares what it prints with the
 * plain implementation.  (The reference has a program of the same purpose, tests/capi_smoke.c there.)
 *
 *   capi_smoke MODEL_DIR DTYPE N_NEW TOKEN_ID [TOKEN_ID ...]
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "inference.h"

#define CHECK(call)                                                                                     \
    do {                                                                                                \
        int rc_ = (call);                                                                               \
        if (rc_ < 0) {                                                                                  \
            fprintf(stderr, "%s failed: %s: %s\n", #call, inference_strerror((inference_error_t)rc_),   \
                    inference_get_last_error());                                                        \
            return 1;                                                                                   \
        }                                                                                               \
    } while (0)

static int seen_tokens = 0;
static int count_token(void* user, int32_t token, const char* text, int text_len) {
    (void)user; (void)token;
    if (text == NULL || text_len != 0) return 1;      /* no tokenizer: the text is always "" */
    seen_tokens++;
    return 0;
}

static void print_ids(const char* label, const int32_t* ids, int n) {
    printf("%s", label);
    for (int i = 0; i < n; i++) printf(" %d", ids[i]);
    printf("\n");
}

int main(int argc, char** argv) {
    if (argc < 5) {
        fprintf(stderr, "usage: %s MODEL_DIR DTYPE N_NEW TOKEN_ID...\n", argv[0]);
        return 2;
    }
    const char* dir = argv[1];
    const char* dtype = argv[2];
    const int n_new = atoi(argv[3]);
    const int n_prompt = argc - 4;
    int32_t* prompt = (int32_t*)malloc(sizeof(int32_t) * (size_t)n_prompt);
    int32_t* out = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n_new + 1));
    for (int i = 0; i < n_prompt; i++) prompt[i] = atoi(argv[4 + i]);

    /* a folder that is not there: NULL and a message, not a crash */
    if (inference_load_model("/nonexistent/model") != NULL || strlen(inference_get_last_error()) == 0) {
        fprintf(stderr, "loading a missing folder did not fail with a message\n");
        return 1;
    }
    printf("missing: %s\n", inference_strerror(INFERENCE_ERR_MODEL_LOAD));

    inference_model_t* m = inference_load_model_ex(dir, dtype, NULL);
    if (!m) {
        fprintf(stderr, "load failed: %s\n", inference_get_last_error());
        return 1;
    }
    if (inference_prefill(m, prompt, n_prompt) != INFERENCE_ERR_INVALID_STATE) {
        fprintf(stderr, "a prefill before inference_kv_cache_init was not refused\n");
        return 1;
    }
    const int n_ctx = inference_max_position(m) < 256 ? inference_max_position(m) : 256;
    CHECK(inference_kv_cache_init(m, n_ctx));
    printf("facts: vocab %d hidden %d n_ctx %d sequences %d name %s\n", inference_vocab_size(m), inference_hidden_size(m),
           inference_n_ctx(m), inference_batch_size(m), inference_model_name(m));

    /* 1. generate: new sequence, prefill, greedy */
    int n_out = 0;
    CHECK(inference_generate_ex(m, prompt, n_prompt, n_new, NULL, out, &n_out));
    print_ids("generate_ex:", out, n_out);

    /* 2. the same by hand: prefill, logits, decode one token at a time */
    inference_reset(m);
    CHECK(inference_prefill(m, prompt, n_prompt));
    const int V = inference_vocab_size(m);
    float* logits = (float*)malloc(sizeof(float) * (size_t)V);
    CHECK(inference_get_logits(m, NULL, logits));
    int best = 0;
    for (int i = 1; i < V; i++) if (logits[i] > logits[best]) best = i;
    out[0] = best;
    for (int i = 1; i < n_new; i++) {
        int next = -1;
        CHECK(inference_decode_token(m, out[i - 1], &next));
        out[i] = next;
    }
    print_ids("decode_token:", out, n_new);
    printf("n_past: %d\n", inference_n_past(m));

    /* 3. a stream with a callback, on a second sequence */
    int seq = inference_seq_new(m);
    CHECK(seq);
    CHECK(inference_seq_select(m, seq));
    inference_gen_options o = inference_gen_default_options();
    o.sampler.temperature = 0.0f;
    o.max_new_tokens = n_new;
    o.ignore_eog = 1;
    o.on_token = count_token;
    inference_stop_reason reason = INFERENCE_STOP_NONE;
    CHECK(inference_generate_stream(m, prompt, n_prompt, &o, out, n_new, &n_out, &reason));
    print_ids("generate_stream:", out, n_out);
    printf("callback saw %d tokens, stop reason %d\n", seen_tokens, (int)reason);

    /* 4. the request queue: the prompt twice, side by side */
    inference_request_options ro;
    ro.sampler = sampler_default_params();
    ro.sampler.temperature = 0.0f;
    ro.max_new_tokens = n_new;
    ro.ignore_eog = 1;
    long long a = inference_request_add(m, prompt, n_prompt, &ro), b = inference_request_add(m, prompt, n_prompt > 1 ? n_prompt - 1 : 1, &ro);
    if (a < 0 || b < 0) { fprintf(stderr, "request_add: %s\n", inference_get_last_error()); return 1; }
    int left;
    while ((left = inference_step(m)) > 0) {}
    CHECK(left);
    int finished = 0;
    CHECK(inference_request_poll(m, a, out, n_new, &n_out, &finished, &reason));
    print_ids("request:", out, n_out);
    printf("finished %d reason %d\n", finished, (int)reason);
    CHECK(inference_request_free(m, a));
    CHECK(inference_request_free(m, b));

    /* 5. the step function itself: the prompt in two portions, logits of the last place */
    engine_step_entry e;
    engine_step_batch batch;
    engine_step_output so;
    static const int32_t last_place[1] = {0};
    memset(&so, 0, sizeof so);
    so.logits = logits;
    so.logits_capacity = V;
    CHECK(engine_request_add(m, 1000));
    batch.entries = &e; batch.n_entries = 1;
    e.request = 1000;
    if (n_prompt > 1) {
        e.tokens = prompt; e.n_tokens = n_prompt - 1; e.want = NULL; e.n_want = 0;
        CHECK(engine_step(m, &batch, &so));
    }
    e.tokens = prompt + n_prompt - 1; e.n_tokens = 1; e.want = last_place; e.n_want = 1;
    CHECK(engine_step(m, &batch, &so));
    best = 0;
    for (int i = 1; i < V; i++) if (logits[i] > logits[best]) best = i;
    printf("engine_step: rows %d vocab %d length %d argmax %d\n", so.n_rows, so.vocab_size, engine_request_length(m, 1000), best);
    CHECK(engine_request_release(m, 1000));

    inference_free_model(m);
    free(logits); free(out); free(prompt);
    printf("ok\n");
    return 0;
}
