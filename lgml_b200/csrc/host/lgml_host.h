/* The host side of lgml_b200 that mischief/lgml has in C as well: the safetensors reader
 * (src/safetensors.c) and the sampler (src/sample.c).  Plain C11, no dependencies but libc and
 * libm; built with the system compiler into one shared object and loaded with ctypes.
 *
 * Every function that can fail returns a negative number (or NULL) and leaves a message that
 * lgml_host_last_error() gives, per thread.  Nothing here touches the GPU.
 */
#ifndef LGML_HOST_H
#define LGML_HOST_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LGML_HOST_API __attribute__((visibility("default")))

LGML_HOST_API const char *lgml_host_last_error(void);

/* ---- safetensors ------------------------------------------------------------------------- */

enum { LGML_ST_MAX_NAME = 63, LGML_ST_MAX_RANK = 4, LGML_ST_MAX_TENSORS = 65536 };
#define LGML_ST_MAX_HEADER ((uint64_t)100 << 20)

/* element types in the order of lgml_st_dtype_name() */
enum { LGML_ST_F64, LGML_ST_F32, LGML_ST_F16, LGML_ST_BF16, LGML_ST_I64, LGML_ST_I32, LGML_ST_I16, LGML_ST_I8, LGML_ST_N_DTYPES };

typedef struct {
    char name[LGML_ST_MAX_NAME + 1];
    int32_t dtype;                      /* LGML_ST_* */
    int32_t rank;
    int64_t shape[LGML_ST_MAX_RANK];
    int64_t begin, end;                 /* absolute offsets in the file */
} lgml_st_entry;

typedef struct lgml_st_index lgml_st_index;

/* The tensors of one file, every size and offset checked; reads the header only. */
LGML_HOST_API lgml_st_index *lgml_st_open(const char *path);
LGML_HOST_API int lgml_st_count(const lgml_st_index *ix);
LGML_HOST_API const lgml_st_entry *lgml_st_get(const lgml_st_index *ix, int i);   /* in the order of the header */
LGML_HOST_API void lgml_st_close(lgml_st_index *ix);
LGML_HOST_API const char *lgml_st_dtype_name(int dtype);
LGML_HOST_API int lgml_st_dtype_size(int dtype);
/* `nbytes` bytes from offset `begin` of the file into dst (pageable or pinned memory); 0 or -1. */
LGML_HOST_API int lgml_st_read(const char *path, int64_t begin, int64_t nbytes, void *dst);

/* ---- sampler ------------------------------------------------------------------------------ */

typedef struct {
    float temperature;                  /* <= 0: the argmax, ties to the lowest id */
    int32_t top_k;                      /* <= 0: off */
    float top_p;                        /* >= 1: off */
    float min_p;                        /* <= 0: off */
    float repeat_penalty, frequency_penalty, presence_penalty;
    int32_t repeat_last_n;
} lgml_sampler_params;

typedef struct lgml_sampler lgml_sampler;

LGML_HOST_API lgml_sampler *lgml_sampler_new(const lgml_sampler_params *p, uint64_t seed);
LGML_HOST_API void lgml_sampler_free(lgml_sampler *s);
/* id -> bias pairs added to the logits before everything else; replaces earlier ones */
LGML_HOST_API int lgml_sampler_set_bias(lgml_sampler *s, const int32_t *ids, const float *bias, int n);
LGML_HOST_API int lgml_sampler_accept(lgml_sampler *s, int32_t token);
LGML_HOST_API void lgml_sampler_reset(lgml_sampler *s);
/* the history, oldest first; returns its length (at most repeat_last_n) */
LGML_HOST_API int lgml_sampler_history(const lgml_sampler *s, int32_t *out, int max);
/* the generator: its four words of state, its next 64 bits, its next double in [0, 1) */
LGML_HOST_API void lgml_sampler_state(const lgml_sampler *s, uint64_t out[4]);
LGML_HOST_API uint64_t lgml_sampler_next_u64(lgml_sampler *s);
LGML_HOST_API double lgml_sampler_uniform(lgml_sampler *s);
/* ln(min_p) in the chain's own arithmetic (float32), so that a copy of the chain elsewhere draws the same bound */
LGML_HOST_API float lgml_log_min_p(float min_p);
/* One id from a row of n float32 logits.  The row after bias and penalties is kept for
 * lgml_sampler_logprobs; `edited` (n floats, may be NULL) receives a copy of it. */
LGML_HOST_API int lgml_sampler_sample(lgml_sampler *s, const float *logits, int n, float *edited);
/* The chain from top_p on for k candidates that top_k has already chosen and sorted (logit
 * descending, id ascending). */
LGML_HOST_API int lgml_sampler_sample_candidates(lgml_sampler *s, const int64_t *ids, const float *vals, int k);
/* log-softmax of `token` in the last sampled row (after bias and penalties), and of the k best:
 * top_ids / top_lp receive k entries (logit descending, id ascending). */
LGML_HOST_API int lgml_sampler_logprobs(const lgml_sampler *s, int32_t token, int k, double *lp, int32_t *top_ids, double *top_lp);

#ifdef __cplusplus
}
#endif
#endif
