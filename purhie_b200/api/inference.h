/* inference.h -- the C interface of libqengine, a B200 inference engine for Qwen3-dense models.
 *
 * Plain C, opaque handles, no C++ or CUDA types.  The names and meanings of the functions follow the C API of
 * aardbeiplantje/PURHIE (src/inference.h there) wherever that API has the function: load a model, make its cache,
 * prefill, decode, generate with a sampler chain, several sequences on one model, step-wise streams.  There is no
 * tokenizer here: prompts and results are token ids, and the `text` a token callback receives is always empty.
 * Beyond that API: models are folders (config.json + safetensors) or seeded random weights; a request queue over
 * the scheduler (inference_request_*); and engine_step, the one step function itself, for tools that bring their
 * own tokens and want logits back (the trace replay tool is built on it).
 *
 * Errors: functions return 0 or a negative inference_error_t (or NULL), and inference_get_last_error() has the
 * text, per thread.  Nothing here computes on the host: without a CUDA device every call that needs one fails
 * with a message, and a missing kernel library is an error that says how to build it.
 */
#ifndef PURHIE_B200_INFERENCE_H
#define PURHIE_B200_INFERENCE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    INFERENCE_OK = 0,
    INFERENCE_ERR_INVALID_ARG = -1,
    INFERENCE_ERR_OUT_OF_MEMORY = -2,
    INFERENCE_ERR_MODEL_LOAD = -3,
    INFERENCE_ERR_KV_CACHE = -4,
    INFERENCE_ERR_TOKENIZER = -5,      /* never returned: there is no tokenizer */
    INFERENCE_ERR_KERNEL_LAUNCH = -6,
    INFERENCE_ERR_INVALID_STATE = -7,
    INFERENCE_ERR_NOT_IMPLEMENTED = -8,
    INFERENCE_ERR_CONTEXT_FULL = -9,
    INFERENCE_ERR_CANCELLED = -10
} inference_error_t;

const char* inference_strerror(inference_error_t err);
/* The text of the last error on this thread ("" when none). */
const char* inference_get_last_error(void);

typedef struct inference_model inference_model_t;

/* ---- sampler (the chain: penalties -> top-k -> top-p -> min-p -> temperature -> one draw) ---------------------- */
typedef struct sampler_params {
    float temperature;      /* <= 0: greedy (argmax after the penalties, lowest id on ties) */
    int top_k;              /* keep the k most likely tokens; <= 0: off */
    float top_p;            /* smallest set with cumulative probability >= top_p; >= 1: off */
    float min_p;            /* keep tokens with p >= min_p * p_max; <= 0: off */
    float repeat_penalty;   /* positive logits / r, negative * r, for recent tokens; 1: off */
    int repeat_last_n;      /* how many accepted tokens the penalties look back over */
    uint64_t seed;          /* equal seeds and inputs give equal tokens */
    float presence_penalty; /* subtracted from the logit of each recent token, after repeat_penalty; 0: off */
} sampler_params;

typedef struct sampler sampler_t;
/* temperature 0.8, top_k 40, top_p 0.95, min_p 0.05, repeat_penalty 1, repeat_last_n 64, seed 0, presence 0 */
sampler_params sampler_default_params(void);
sampler_t* sampler_create(const sampler_params* params);
void sampler_free(sampler_t* s);
int sampler_sample(sampler_t* s, const float* logits, int n_vocab);   /* does not record the token */
void sampler_accept(sampler_t* s, int token);
void sampler_reset(sampler_t* s);

/* ---- models ------------------------------------------------------------------------------------------------------ */
/* A folder with config.json and model.safetensors (or a shard index); bfloat16 compute.  NULL on failure. */
inference_model_t* inference_load_model(const char* model_dir);
/* dtype: "bfloat16" or "float32" (a true 32-bit path: float32 weights, activations, cache and products).
 * options_json: NULL or {"gemm": "auto|tcgen05|simple", "attention": "auto|flash|generic"}. */
inference_model_t* inference_load_model_ex(const char* model_dir, const char* dtype, const char* options_json);
/* Seeded random weights made on the device for the configuration in config_json (the text of a config.json):
 * matrices N(0, 0.02), norm weights 1.  The values are those inference_write_random_model stores. */
inference_model_t* inference_load_model_random(const char* config_json, uint64_t seed, const char* dtype);
inference_model_t* inference_load_model_random_ex(const char* config_json, uint64_t seed, const char* dtype, double std,
                                                  double scale_low, double scale_high, const char* options_json);
/* Write config.json and model.safetensors for config_json into model_dir (no device needed).  stored_dtype:
 * "bfloat16" or "float32" for the matrices; vectors are stored as float32. */
int inference_write_random_model(const char* model_dir, const char* config_json, uint64_t seed, double std,
                                 double scale_low, double scale_high, const char* stored_dtype);
void inference_free_model(inference_model_t* model);

/* The cache: room for sequences of up to n_ctx tokens.  The plain call makes four sequences' worth of pages of 16
 * tokens; _ex chooses the number of sequences, the page size and the pool (kv_tokens tokens in all, 0: every
 * sequence a full context) and takes n_ctx 0 for "as long as the model allows".  engine_options_json: NULL or {"poison_cache": bool, "cuda_graphs": bool,
 * "num_pages": n | [n per group], "max_batch_tokens": n, "prefill_chunk": n, "step": {kernel choices}}. */
int inference_kv_cache_init(inference_model_t* model, int n_ctx);
int inference_kv_cache_init_ex(inference_model_t* model, int n_ctx, int max_sequences, int page_size, long long kv_tokens,
                               const char* engine_options_json);
void inference_kv_cache_free(inference_model_t* model);

/* Wait until everything the model has launched is done; reports a kernel that gave up on a wait. */
int inference_synchronize(inference_model_t* model);

/* The end-of-generation token ids (by default config.json's or generation_config.json's eos_token_id). */
int inference_set_eog_tokens(inference_model_t* model, const int32_t* ids, int n);

void inference_set_seed(inference_model_t* model, unsigned int seed);      /* for inference_generate_ex without params */
void inference_set_prefill_batch(inference_model_t* model, int n_tokens); /* most tokens per pass of a prefill (default 1024) */

/* The model holds sequences of tokens at positions 0, 1, 2, ...; everything below works on the current one
 * (sequence 0 until another is selected).  inference_reset starts the current sequence anew. */
void inference_reset(inference_model_t* model);
int inference_n_past(const inference_model_t* model);

/* n tokens of the current sequence at positions n_past .. n_past + n - 1, in passes of at most the prefill batch.
 * Afterwards the logits are those of the last token.  INFERENCE_ERR_CONTEXT_FULL if they do not fit. */
int inference_prefill(inference_model_t* model, const int32_t* tokens, int n);
/* The same, and the logits after every one of the n tokens into logits ([n][vocab_size] floats). */
int inference_prefill_logits(inference_model_t* model, const int32_t* tokens, int n, float* logits);
/* One token at position n_past; *next_token_out is the greedy next token. */
int inference_decode_token(inference_model_t* model, int token_id, int* next_token_out);
/* The logits of the last token of the current sequence, copied to the host (no forward pass when they are at
 * hand).  vocab_ids (optional) is filled with 0 .. vocab_size - 1. */
int inference_get_logits(inference_model_t* model, int* vocab_ids, float* logits);

/* New sequence, prefill, then sample up to max_new_tokens (params NULL: greedy with the model's seed).  Stops early
 * at an end-of-generation token (not written) or when the context is full. */
int inference_generate_ex(inference_model_t* model, const int32_t* prompt_ids, int prompt_len, int max_new_tokens,
                          const sampler_params* params, int32_t* out_ids, int* out_len);

typedef enum {
    INFERENCE_STOP_NONE = 0,
    INFERENCE_STOP_EOG = 1,           /* an end-of-generation token (config.json's eos_token_id) */
    INFERENCE_STOP_MAX_TOKENS = 2,
    INFERENCE_STOP_STRING = 3,        /* never: there is no text */
    INFERENCE_STOP_CALLBACK = 4,      /* on_token returned nonzero */
    INFERENCE_STOP_CONTEXT_FULL = 5,
    INFERENCE_STOP_CANCELLED = 6      /* inference_request_cancel */
} inference_stop_reason;

/* Called once per generated token; text is "" and text_len 0.  Return nonzero to stop after this token. */
typedef int (*inference_token_cb)(void* user, int32_t token, const char* text, int text_len);

typedef struct inference_gen_options {
    sampler_params sampler;
    int max_new_tokens;               /* default 256 */
    const char* const* stop_strings;  /* ignored (no text) */
    int n_stop_strings;
    int ignore_eog;                   /* 1: do not stop at end-of-generation tokens */
    int reuse_prefix;                 /* 1: prompt_ids is the whole sequence; the prefix it shares with the current one is kept */
    int checkpoint_tail;              /* ignored (no recurrent state to checkpoint) */
    inference_token_cb on_token;
    void* user;
    int prefill_chunk;                /* streams: prefill the prompt in steps of at most this many tokens (0: all at begin) */
} inference_gen_options;
inference_gen_options inference_gen_default_options(void);

/* Continue the current sequence with n_prompt tokens (0: from the last token's logits) and generate.  out_ids
 * (optional, max_out entries) receives the emitted tokens, *n_out counts all of them, *reason says why it stopped.
 * The end-of-generation token that stops it is neither emitted nor kept in the sequence. */
int inference_generate_stream(inference_model_t* model, const int32_t* prompt_ids, int n_prompt,
                              const inference_gen_options* options, int32_t* out_ids, int max_out, int* n_out,
                              inference_stop_reason* reason);
int inference_last_prompt_stats(const inference_model_t* model, int* reused, int* prefilled);

/* Several sequences on one model, each with its own block table in the shared page pool. */
int inference_seq_new(inference_model_t* model);          /* its number, or -1 when every slot is taken */
int inference_seq_select(inference_model_t* model, int seq);
int inference_seq_current(const inference_model_t* model);
int inference_seq_free(inference_model_t* model, int seq); /* not sequence 0 */

/* Step-wise generation, so that a caller can interleave sequences. */
typedef struct inference_stream inference_stream_t;
inference_stream_t* inference_stream_begin(inference_model_t* model, const int32_t* prompt_ids, int n_prompt,
                                           const inference_gen_options* options);
/* 1 while generation goes on, 0 when it has stopped (the last step may still emit a token), negative on error.
 * *token: the emitted token (-1: none, e.g. a step that only prefilled). */
int inference_stream_step(inference_stream_t* stream, int32_t* token, const char** text, int* text_len,
                          inference_stop_reason* reason);
int inference_stream_tokens(const inference_stream_t* stream);
int inference_stream_seq(const inference_stream_t* stream);
void inference_stream_free(inference_stream_t* stream);
typedef struct {
    int32_t token;
    const char* text;
    int text_len;
    inference_stop_reason reason;
    int rc;                           /* as inference_stream_step returns */
} inference_step_result;
/* One step of each of n streams with ONE pass for all: prompt portions and decode rows share the batch. */
int inference_stream_step_batch(inference_stream_t* const* streams, int n, inference_step_result* results);
/* Up to n_steps steps of every stream; results[step * n + i] is what inference_stream_step_batch would have given
 * streams[i] in that step.  While all streams are decoding with device samplers a step is launched with the
 * token ids the step before left on the device, so the host's work overlaps the device's.  Returns the number of
 * steps taken (fewer when every stream ends earlier), negative on error. */
int inference_stream_run(inference_stream_t* const* streams, int n, int n_steps, inference_step_result* results);

/* ---- the request queue (over the scheduler: admission, chunked prompts, preemption when pages run out) ----------- */
typedef struct inference_request_options {
    sampler_params sampler;
    int max_new_tokens;
    int ignore_eog;
} inference_request_options;
long long inference_request_add(inference_model_t* model, const int32_t* tokens, int n, const inference_request_options* options);
/* One scheduler step (or a run of decode steps launched ahead of the host).  Returns the number of requests still
 * waiting or running, negative on error. */
int inference_step(inference_model_t* model);
/* Tokens generated so far into out (optional, max_out entries); *n_out counts all of them; *finished and *reason
 * say whether and why it ended.  A finished request stays until inference_request_free. */
int inference_request_poll(inference_model_t* model, long long request, int32_t* out, int max_out, int* n_out,
                           int* finished, inference_stop_reason* reason);
int inference_request_cancel(inference_model_t* model, long long request);
int inference_request_free(inference_model_t* model, long long request);

/* ---- the step function itself ------------------------------------------------------------------------------------ */
typedef struct engine_step_entry {
    long long request;        /* made live with engine_request_add */
    const int32_t* tokens;    /* its next tokens: a portion of a prompt, or one decoded token */
    int n_tokens;
    const int32_t* want;      /* places among these tokens whose logits are returned */
    int n_want;
} engine_step_entry;
typedef struct engine_step_batch {
    const engine_step_entry* entries;
    int n_entries;
} engine_step_batch;
typedef struct engine_step_output {
    float* logits;            /* in: room for logits_capacity floats (may be NULL when nothing is wanted) */
    long long logits_capacity;
    int n_rows;               /* out: wanted places, in the order of the entries and of each want */
    int vocab_size;
    int tokens, prompt_rows, decode_rows, replayed_graph;    /* out: what the step ran */
} engine_step_output;
int engine_request_add(inference_model_t* model, long long request);
int engine_request_release(inference_model_t* model, long long request);
int engine_request_length(const inference_model_t* model, long long request);   /* tokens in the cache; -1: not live */
/* Run one batch: only the tokens it brings, against the cache earlier steps left.  INFERENCE_ERR_CONTEXT_FULL,
 * with nothing changed, when the cache cannot hold it. */
int engine_step(inference_model_t* model, const engine_step_batch* batch, engine_step_output* out);

/* ---- facts ------------------------------------------------------------------------------------------------------- */
int inference_n_ctx(const inference_model_t* model);
int inference_batch_size(const inference_model_t* model);     /* most sequences (state slots) */
const char* inference_model_name(const inference_model_t* model);
int inference_vocab_size(const inference_model_t* model);
int inference_hidden_size(const inference_model_t* model);
int inference_max_position(const inference_model_t* model);   /* the longest sequence the model's configuration allows */

#ifdef __cplusplus
}
#endif
#endif
