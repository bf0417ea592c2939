/* See lgml_host.h.  Part 1: errors, a strict JSON reader for headers, the safetensors index.
 *
 * The format and every check follow mischief/lgml's reader (src/safetensors.c): an 8-byte
 * little-endian header length, a JSON header, raw little-endian data (st_read, :278-332); the
 * header length is bounded and must lie inside the file (:101); a tensor has at most four
 * dimensions, each at least one (:173-188); begin <= end <= data size and end - begin equals the
 * element count times the element size (check_entry, :229-244); names are 1..63 bytes
 * (:313-315); at most 65536 tensors (:31, :316).
 */
#define _FILE_OFFSET_BITS 64
#define _POSIX_C_SOURCE 200809L
#include "lgml_host.h"

#include <errno.h>
#include <fcntl.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

static _Thread_local char err_buf[768];

static void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err_buf, sizeof(err_buf), fmt, ap);
    va_end(ap);
}

const char *lgml_host_last_error(void) { return err_buf; }

/* ---- JSON ------------------------------------------------------------------------------------
 * A reader over a byte range that knows what a header needs: objects, arrays, strings (with
 * escapes), integers; any other value can be skipped.  Depth is bounded. */
typedef struct {
    const char *p, *end;
    const char *why;                    /* first fault */
} json;

enum { JSON_MAX_DEPTH = 32 };

static void json_ws(json *j) {
    while (j->p < j->end && (*j->p == ' ' || *j->p == '\t' || *j->p == '\n' || *j->p == '\r')) ++j->p;
}
static int json_fail(json *j, const char *why) {
    if (!j->why) j->why = why;
    return -1;
}
static int json_eat(json *j, char c) {
    json_ws(j);
    if (j->p < j->end && *j->p == c) {
        ++j->p;
        return 1;
    }
    return 0;
}
static int json_peek(json *j) {
    json_ws(j);
    return j->p < j->end ? (unsigned char)*j->p : -1;
}
static int hex4(const char *p) {
    int v = 0;
    for (int i = 0; i < 4; ++i) {
        const char c = p[i];
        int d = (c >= '0' && c <= '9') ? c - '0' : (c >= 'a' && c <= 'f') ? c - 'a' + 10 : (c >= 'A' && c <= 'F') ? c - 'A' + 10 : -1;
        if (d < 0) return -1;
        v = v * 16 + d;
    }
    return v;
}
static size_t put_utf8(char *out, size_t cap, size_t n, uint32_t cp) {
    char b[4];
    int len;
    if (cp < 0x80) { b[0] = (char)cp; len = 1; }
    else if (cp < 0x800) { b[0] = (char)(0xC0 | (cp >> 6)); b[1] = (char)(0x80 | (cp & 0x3F)); len = 2; }
    else if (cp < 0x10000) { b[0] = (char)(0xE0 | (cp >> 12)); b[1] = (char)(0x80 | ((cp >> 6) & 0x3F)); b[2] = (char)(0x80 | (cp & 0x3F)); len = 3; }
    else { b[0] = (char)(0xF0 | (cp >> 18)); b[1] = (char)(0x80 | ((cp >> 12) & 0x3F)); b[2] = (char)(0x80 | ((cp >> 6) & 0x3F)); b[3] = (char)(0x80 | (cp & 0x3F)); len = 4; }
    for (int i = 0; i < len; ++i)
        if (n + i < cap) out[n + i] = b[i];
    return n + len;
}
/* A string into out (cap bytes, always NUL-terminated); *len receives the decoded length, which
 * may exceed cap - 1 (the caller decides whether that is an error).  out may be NULL. */
static int json_string(json *j, char *out, size_t cap, size_t *len) {
    size_t n = 0;
    if (!json_eat(j, '"')) return json_fail(j, "a string was expected");
    while (1) {
        if (j->p >= j->end) return json_fail(j, "a string does not end");
        unsigned char c = (unsigned char)*j->p++;
        if (c == '"') break;
        if (c < 0x20) return json_fail(j, "a control character in a string");
        if (c != '\\') {
            if (out && n < cap) out[n] = (char)c;
            ++n;
            continue;
        }
        if (j->p >= j->end) return json_fail(j, "a string does not end");
        c = (unsigned char)*j->p++;
        uint32_t cp;
        switch (c) {
            case '"': cp = '"'; break;
            case '\\': cp = '\\'; break;
            case '/': cp = '/'; break;
            case 'b': cp = '\b'; break;
            case 'f': cp = '\f'; break;
            case 'n': cp = '\n'; break;
            case 'r': cp = '\r'; break;
            case 't': cp = '\t'; break;
            case 'u': {
                if (j->end - j->p < 4) return json_fail(j, "a short \\u escape");
                int h = hex4(j->p);
                if (h < 0) return json_fail(j, "a bad \\u escape");
                j->p += 4;
                cp = (uint32_t)h;
                if (cp >= 0xD800 && cp < 0xDC00) {       /* a surrogate pair */
                    if (j->end - j->p < 6 || j->p[0] != '\\' || j->p[1] != 'u') return json_fail(j, "half a surrogate pair");
                    int lo = hex4(j->p + 2);
                    if (lo < 0xDC00 || lo > 0xDFFF) return json_fail(j, "half a surrogate pair");
                    j->p += 6;
                    cp = 0x10000 + ((cp - 0xD800) << 10) + ((uint32_t)lo - 0xDC00);
                } else if (cp >= 0xDC00 && cp < 0xE000) {
                    return json_fail(j, "half a surrogate pair");
                }
                break;
            }
            default: return json_fail(j, "an unknown escape");
        }
        n = put_utf8(out, out ? cap : 0, n, cp);
    }
    if (out && cap) out[n < cap ? n : cap - 1] = 0;
    if (len) *len = n;
    return 0;
}
/* An integer that fits int64 (no fraction, no exponent). */
static int json_int(json *j, int64_t *v) {
    json_ws(j);
    const char *p = j->p;
    int neg = 0;
    if (p < j->end && *p == '-') { neg = 1; ++p; }
    if (p >= j->end || *p < '0' || *p > '9') return json_fail(j, "an integer was expected");
    if (*p == '0' && p + 1 < j->end && p[1] >= '0' && p[1] <= '9') return json_fail(j, "a number with a leading zero");
    uint64_t u = 0;
    while (p < j->end && *p >= '0' && *p <= '9') {
        if (u > (UINT64_MAX - 9) / 10) return json_fail(j, "an integer too large");
        u = u * 10 + (uint64_t)(*p - '0');
        ++p;
    }
    if (p < j->end && (*p == '.' || *p == 'e' || *p == 'E')) return json_fail(j, "an integer was expected");
    if (u > (uint64_t)INT64_MAX) return json_fail(j, "an integer too large");
    *v = neg ? -(int64_t)u : (int64_t)u;
    j->p = p;
    return 0;
}
static int json_skip(json *j, int depth);
static int json_skip_number(json *j) {
    const char *p = j->p;
    if (p < j->end && *p == '-') ++p;
    const char *digits = p;
    while (p < j->end && *p >= '0' && *p <= '9') ++p;
    if (p == digits) return json_fail(j, "a value was expected");
    if (p < j->end && *p == '.') {
        ++p;
        const char *f = p;
        while (p < j->end && *p >= '0' && *p <= '9') ++p;
        if (p == f) return json_fail(j, "a bad number");
    }
    if (p < j->end && (*p == 'e' || *p == 'E')) {
        ++p;
        if (p < j->end && (*p == '+' || *p == '-')) ++p;
        const char *x = p;
        while (p < j->end && *p >= '0' && *p <= '9') ++p;
        if (p == x) return json_fail(j, "a bad number");
    }
    j->p = p;
    return 0;
}
static int json_skip(json *j, int depth) {
    if (depth > JSON_MAX_DEPTH) return json_fail(j, "nested too deeply");
    int c = json_peek(j);
    if (c == '"') return json_string(j, NULL, 0, NULL);
    if (c == '{' || c == '[') {
        const char close = c == '{' ? '}' : ']';
        ++j->p;
        if (json_eat(j, close)) return 0;
        do {
            if (c == '{') {
                if (json_string(j, NULL, 0, NULL)) return -1;
                if (!json_eat(j, ':')) return json_fail(j, "':' was expected");
            }
            if (json_skip(j, depth + 1)) return -1;
        } while (json_eat(j, ','));
        if (!json_eat(j, close)) return json_fail(j, "',' or a closing bracket was expected");
        return 0;
    }
    if (c == 't' && j->end - j->p >= 4 && !memcmp(j->p, "true", 4)) { j->p += 4; return 0; }
    if (c == 'f' && j->end - j->p >= 5 && !memcmp(j->p, "false", 5)) { j->p += 5; return 0; }
    if (c == 'n' && j->end - j->p >= 4 && !memcmp(j->p, "null", 4)) { j->p += 4; return 0; }
    return json_skip_number(j);
}

/* Is the byte range well-formed UTF-8 (no overlong forms, no surrogates, nothing past U+10FFFF)? */
static int utf8_ok(const unsigned char *p, size_t n) {
    size_t i = 0;
    while (i < n) {
        const unsigned char c = p[i];
        size_t len;
        uint32_t cp;
        if (c < 0x80) { ++i; continue; }
        else if ((c & 0xE0) == 0xC0) { len = 2; cp = c & 0x1F; }
        else if ((c & 0xF0) == 0xE0) { len = 3; cp = c & 0x0F; }
        else if ((c & 0xF8) == 0xF0) { len = 4; cp = c & 0x07; }
        else return 0;
        if (i + len > n) return 0;
        for (size_t k = 1; k < len; ++k) {
            if ((p[i + k] & 0xC0) != 0x80) return 0;
            cp = (cp << 6) | (p[i + k] & 0x3F);
        }
        if ((len == 2 && cp < 0x80) || (len == 3 && cp < 0x800) || (len == 4 && cp < 0x10000) || cp > 0x10FFFF || (cp >= 0xD800 && cp < 0xE000)) return 0;
        i += len;
    }
    return 1;
}

/* ---- safetensors ------------------------------------------------------------------------------ */

static const char *const st_names[LGML_ST_N_DTYPES] = {"F64", "F32", "F16", "BF16", "I64", "I32", "I16", "I8"};
static const int st_sizes[LGML_ST_N_DTYPES] = {8, 4, 2, 2, 8, 4, 2, 1};

const char *lgml_st_dtype_name(int dtype) { return dtype >= 0 && dtype < LGML_ST_N_DTYPES ? st_names[dtype] : "?"; }
int lgml_st_dtype_size(int dtype) { return dtype >= 0 && dtype < LGML_ST_N_DTYPES ? st_sizes[dtype] : 0; }

struct lgml_st_index {
    int n, cap;
    lgml_st_entry *e;
};

/* An integer element of an array, or any other value skipped (then *ok = 0). */
static int int_or_skip(json *j, int64_t *v, int *ok) {
    const char *at = j->p;
    if (json_int(j, v) == 0) return 0;
    j->p = at;
    j->why = NULL;
    *ok = 0;
    return json_skip(j, 2);
}

/* One entry {"dtype": .., "shape": [..], "data_offsets": [b, e]} checked against the data size. */
static int st_entry(json *j, const char *path, const char *name, int64_t data_start, int64_t data_size, lgml_st_entry *out) {
    char dtype[16] = "";
    int have_dtype = 0, shape_ok = 0, offs_ok = 0, rank = 0, n_offs = 0;
    int64_t shape[LGML_ST_MAX_RANK] = {0}, offs[2] = {0, 0};
    if (!json_eat(j, '{')) {
        if (json_skip(j, 1)) return -2;
        set_error("%s: entry of '%s' must be an object", path, name);
        return -1;
    }
    if (!json_eat(j, '}')) {
        do {
            char key[32];
            size_t klen;
            if (json_string(j, key, sizeof(key), &klen)) return -2;
            if (!json_eat(j, ':')) return json_fail(j, "':' was expected"), -2;
            if (klen == 5 && !strcmp(key, "dtype") && json_peek(j) == '"') {
                size_t dl;
                if (json_string(j, dtype, sizeof(dtype), &dl)) return -2;
                have_dtype = dl < sizeof(dtype);
            } else if (klen == 5 && !strcmp(key, "shape") && json_peek(j) == '[') {
                ++j->p;
                shape_ok = 1;
                rank = 0;
                if (!json_eat(j, ']')) {
                    do {
                        int64_t d = 0;
                        int ok = 1;
                        if (int_or_skip(j, &d, &ok)) return -2;
                        if (!ok || d < 1 || rank >= LGML_ST_MAX_RANK) shape_ok = 0;
                        else shape[rank] = d;
                        ++rank;
                    } while (json_eat(j, ','));
                    if (!json_eat(j, ']')) return json_fail(j, "',' or ']' was expected"), -2;
                }
                if (rank > LGML_ST_MAX_RANK) shape_ok = 0;
            } else if (klen == 12 && !strcmp(key, "data_offsets") && json_peek(j) == '[') {
                ++j->p;
                offs_ok = 1;
                n_offs = 0;
                if (!json_eat(j, ']')) {
                    do {
                        int64_t d = 0;
                        int ok = 1;
                        if (int_or_skip(j, &d, &ok)) return -2;
                        if (!ok || n_offs >= 2) offs_ok = 0;
                        else offs[n_offs] = d;
                        ++n_offs;
                    } while (json_eat(j, ','));
                    if (!json_eat(j, ']')) return json_fail(j, "',' or ']' was expected"), -2;
                }
                if (n_offs != 2) offs_ok = 0;
            } else if (json_skip(j, 1)) {
                return -2;
            }
        } while (json_eat(j, ','));
        if (!json_eat(j, '}')) return json_fail(j, "',' or '}' was expected"), -2;
    }
    int dt = -1;
    for (int i = 0; have_dtype && i < LGML_ST_N_DTYPES; ++i)
        if (!strcmp(dtype, st_names[i])) dt = i;
    if (dt < 0) {
        set_error("%s: tensor '%s' has unsupported dtype '%s'", path, name, have_dtype ? dtype : "(none)");
        return -1;
    }
    if (!shape_ok) {
        set_error("%s: tensor '%s' has bad shape (at most %d dimensions, each an integer >= 1)", path, name, LGML_ST_MAX_RANK);
        return -1;
    }
    if (!offs_ok) {
        set_error("%s: tensor '%s' has bad data_offsets (two integers)", path, name);
        return -1;
    }
    /* the element count times the element size, without overflow */
    int64_t numel = 1;
    int fits = 1;
    for (int i = 0; i < rank; ++i) {
        if (shape[i] > INT64_MAX / 16 / numel) fits = 0;
        else numel *= shape[i];
    }
    if (!fits || !(0 <= offs[0] && offs[0] <= offs[1] && offs[1] <= data_size) || offs[1] - offs[0] != numel * st_sizes[dt]) {
        set_error("%s: tensor '%s' offsets [%lld, %lld) do not fit %lld x %s in %lld data bytes", path, name, (long long)offs[0], (long long)offs[1],
                  (long long)numel, st_names[dt], (long long)data_size);
        return -1;
    }
    memset(out, 0, sizeof(*out));
    memcpy(out->name, name, strnlen(name, LGML_ST_MAX_NAME));
    out->dtype = dt;
    out->rank = rank;
    for (int i = 0; i < rank; ++i) out->shape[i] = shape[i];
    out->begin = data_start + offs[0];
    out->end = data_start + offs[1];
    return 0;
}

static int read_fully(int fd, void *dst, int64_t n, int64_t off) {
    char *p = (char *)dst;
    while (n > 0) {
        ssize_t r = pread(fd, p, (size_t)(n > (1 << 30) ? (1 << 30) : n), (off_t)off);
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) return -1;
        p += r;
        off += r;
        n -= r;
    }
    return 0;
}

lgml_st_index *lgml_st_open(const char *path) {
    int fd = open(path, O_RDONLY);
    if (fd < 0) {
        set_error("%s: %s", path, strerror(errno));
        return NULL;
    }
    struct stat sb;
    char *raw = NULL;
    lgml_st_index *ix = NULL;
    if (fstat(fd, &sb)) {
        set_error("%s: %s", path, strerror(errno));
        goto fail;
    }
    const int64_t size = (int64_t)sb.st_size;
    unsigned char head[8];
    if (size < 8 || read_fully(fd, head, 8, 0)) {
        set_error("%s: shorter than its 8-byte header length", path);
        goto fail;
    }
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | head[i];
    if (hlen < 2 || hlen > LGML_ST_MAX_HEADER || 8 + hlen > (uint64_t)size) {
        set_error("%s: bad header length %llu (file has %lld bytes)", path, (unsigned long long)hlen, (long long)size);
        goto fail;
    }
    raw = (char *)malloc((size_t)hlen);
    if (!raw || read_fully(fd, raw, (int64_t)hlen, 8)) {
        set_error("%s: short read of the header", path);
        goto fail;
    }
    ix = (lgml_st_index *)calloc(1, sizeof(*ix));
    if (!ix) {
        set_error("%s: out of memory", path);
        goto fail;
    }
    const int64_t data_start = 8 + (int64_t)hlen, data_size = size - data_start;
    json j = {raw, raw + hlen, NULL};
    if (!utf8_ok((const unsigned char *)raw, (size_t)hlen)) {
        json_fail(&j, "the header is not UTF-8");
        goto syntax;
    }
    if (!json_eat(&j, '{')) {
        json_fail(&j, "the header must be an object");
        goto syntax;
    }
    if (!json_eat(&j, '}')) {
        do {
            char name[LGML_ST_MAX_NAME + 2];
            size_t nlen;
            if (json_string(&j, name, sizeof(name), &nlen)) goto syntax;
            if (!json_eat(&j, ':')) {
                json_fail(&j, "':' was expected");
                goto syntax;
            }
            if (!strcmp(name, "__metadata__")) {
                if (json_skip(&j, 1)) goto syntax;
                continue;
            }
            if (nlen < 1 || nlen > LGML_ST_MAX_NAME || strlen(name) != nlen) {
                set_error("%s: bad tensor name '%.80s' (1..%d bytes, no NUL)", path, name, LGML_ST_MAX_NAME);
                goto fail;
            }
            for (int i = 0; i < ix->n; ++i)
                if (!strcmp(ix->e[i].name, name)) {
                    set_error("%s: tensor '%s' is in the header twice", path, name);
                    goto fail;
                }
            if (ix->n >= LGML_ST_MAX_TENSORS) {
                set_error("%s: more than %d tensors", path, LGML_ST_MAX_TENSORS);
                goto fail;
            }
            if (ix->n == ix->cap) {
                const int cap = ix->cap ? 2 * ix->cap : 256;
                lgml_st_entry *e = (lgml_st_entry *)realloc(ix->e, (size_t)cap * sizeof(*e));
                if (!e) {
                    set_error("%s: out of memory", path);
                    goto fail;
                }
                ix->e = e;
                ix->cap = cap;
            }
            const int rc = st_entry(&j, path, name, data_start, data_size, &ix->e[ix->n]);
            if (rc == -2) goto syntax;
            if (rc) goto fail;
            ++ix->n;
        } while (json_eat(&j, ','));
        if (!json_eat(&j, '}')) {
            json_fail(&j, "',' or '}' was expected");
            goto syntax;
        }
    }
    json_ws(&j);
    if (j.p != j.end) {
        json_fail(&j, "text behind the header's object");
        goto syntax;
    }
    free(raw);
    close(fd);
    return ix;
syntax:
    set_error("%s: header is not JSON: %s at byte %lld", path, j.why ? j.why : "fault", (long long)(j.p - raw));
fail:
    free(raw);
    if (ix) {
        free(ix->e);
        free(ix);
    }
    close(fd);
    return NULL;
}

int lgml_st_count(const lgml_st_index *ix) { return ix ? ix->n : 0; }
const lgml_st_entry *lgml_st_get(const lgml_st_index *ix, int i) { return ix && i >= 0 && i < ix->n ? &ix->e[i] : NULL; }
void lgml_st_close(lgml_st_index *ix) {
    if (ix) {
        free(ix->e);
        free(ix);
    }
}

int lgml_st_read(const char *path, int64_t begin, int64_t nbytes, void *dst) {
    int fd = open(path, O_RDONLY);
    if (fd < 0) {
        set_error("%s: %s", path, strerror(errno));
        return -1;
    }
    const int rc = read_fully(fd, dst, nbytes, begin);
    close(fd);
    if (rc) set_error("%s: short read of %lld bytes at %lld", path, (long long)nbytes, (long long)begin);
    return rc;
}

/* ---- sampler ------------------------------------------------------------------------------------
 * One per request, with mischief/lgml's options, order and arithmetic (src/sample.c): the chain
 * is bias -> penalties -> top_k -> top_p -> min_p -> temperature -> draw (:1050-1055, chain
 * :929-962); temperature <= 0 is the argmax with ties to the lowest index (:937-940, :913-926).
 * The generator is xoshiro256** seeded by splitmix64 (:93-139) and a draw uses one double
 * (next() >> 11) * 2^-53 (:126-130).  Weights are float32, their sums in a draw float64. */

typedef struct {
    int64_t id;
    float v;
} cand;

struct lgml_sampler {
    lgml_sampler_params p;
    uint64_t s[4];
    int32_t *hist;                      /* ring of the last repeat_last_n ids */
    int hist_n, hist_at;                /* entries, index of the oldest */
    int32_t *bias_ids;
    float *bias;
    int n_bias;
    float *last;                        /* the last sampled row after bias and penalties */
    int last_n, last_cap;
    cand *c;                            /* work space of the chain */
    int c_cap;
};

static uint64_t rotl64(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }

uint64_t lgml_sampler_next_u64(lgml_sampler *sm) {
    uint64_t *s = sm->s;
    const uint64_t r = rotl64(s[1] * 5, 7) * 9, t = s[1] << 17;
    s[2] ^= s[0];
    s[3] ^= s[1];
    s[1] ^= s[2];
    s[0] ^= s[3];
    s[2] ^= t;
    s[3] = rotl64(s[3], 45);
    return r;
}
/* ln(min_p) as the chain computes it (float32 logf), for the device's copy of the chain. */
float lgml_log_min_p(float min_p) { return logf(min_p); }

double lgml_sampler_uniform(lgml_sampler *sm) { return (double)(lgml_sampler_next_u64(sm) >> 11) * 0x1.0p-53; }

lgml_sampler *lgml_sampler_new(const lgml_sampler_params *p, uint64_t seed) {
    if (p->repeat_last_n < 0 || !(p->repeat_penalty > 0.f)) {
        set_error("sampler: repeat_last_n must be >= 0 and repeat_penalty > 0");
        return NULL;
    }
    lgml_sampler *sm = (lgml_sampler *)calloc(1, sizeof(*sm));
    if (!sm) {
        set_error("sampler: out of memory");
        return NULL;
    }
    sm->p = *p;
    uint64_t x = seed;
    for (int i = 0; i < 4; ++i) {       /* splitmix64 */
        x += 0x9E3779B97F4A7C15ull;
        uint64_t z = x;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        sm->s[i] = z ^ (z >> 31);
    }
    if (p->repeat_last_n > 0) {
        sm->hist = (int32_t *)malloc((size_t)p->repeat_last_n * sizeof(int32_t));
        if (!sm->hist) {
            free(sm);
            set_error("sampler: out of memory");
            return NULL;
        }
    }
    return sm;
}

void lgml_sampler_free(lgml_sampler *sm) {
    if (!sm) return;
    free(sm->hist);
    free(sm->bias_ids);
    free(sm->bias);
    free(sm->last);
    free(sm->c);
    free(sm);
}

int lgml_sampler_set_bias(lgml_sampler *sm, const int32_t *ids, const float *bias, int n) {
    free(sm->bias_ids);
    free(sm->bias);
    sm->bias_ids = NULL;
    sm->bias = NULL;
    sm->n_bias = 0;
    if (n <= 0) return 0;
    sm->bias_ids = (int32_t *)malloc((size_t)n * sizeof(int32_t));
    sm->bias = (float *)malloc((size_t)n * sizeof(float));
    if (!sm->bias_ids || !sm->bias) {
        set_error("sampler: out of memory");
        return -1;
    }
    memcpy(sm->bias_ids, ids, (size_t)n * sizeof(int32_t));
    memcpy(sm->bias, bias, (size_t)n * sizeof(float));
    sm->n_bias = n;
    return 0;
}

/* the history (src/sample.c:603-650) */
int lgml_sampler_accept(lgml_sampler *sm, int32_t token) {
    if (token < 0) {
        set_error("sampler: bad token id %d", token);
        return -1;
    }
    const int cap = sm->p.repeat_last_n;
    if (cap == 0) return 0;
    if (sm->hist_n < cap) {
        sm->hist[(sm->hist_at + sm->hist_n) % cap] = token;
        ++sm->hist_n;
    } else {
        sm->hist[sm->hist_at] = token;
        sm->hist_at = (sm->hist_at + 1) % cap;
    }
    return 0;
}
void lgml_sampler_reset(lgml_sampler *sm) { sm->hist_n = sm->hist_at = 0; }
int lgml_sampler_history(const lgml_sampler *sm, int32_t *out, int max) {
    const int n = sm->hist_n < max ? sm->hist_n : max;
    for (int i = 0; i < n; ++i) out[i] = sm->hist[(sm->hist_at + i) % sm->p.repeat_last_n];
    return sm->hist_n;
}

static int by_id(const void *a, const void *b) {
    const int32_t x = *(const int32_t *)a, y = *(const int32_t *)b;
    return (x > y) - (x < y);
}
/* Each distinct id of the history once (apply_penalties, src/sample.c:652-677). */
static int apply_penalties(lgml_sampler *sm, float *l, int n) {
    const lgml_sampler_params *p = &sm->p;
    if (sm->hist_n == 0 || (p->repeat_penalty == 1.f && p->frequency_penalty == 0.f && p->presence_penalty == 0.f)) return 0;
    int32_t *ids = (int32_t *)malloc((size_t)sm->hist_n * sizeof(int32_t));
    if (!ids) {
        set_error("sampler: out of memory");
        return -1;
    }
    lgml_sampler_history(sm, ids, sm->hist_n);
    qsort(ids, (size_t)sm->hist_n, sizeof(int32_t), by_id);
    for (int i = 0; i < sm->hist_n;) {
        int k = i;
        while (k < sm->hist_n && ids[k] == ids[i]) ++k;
        const int32_t t = ids[i];
        if (t < n) {
            float v = l[t];
            v = v <= 0.f ? v * p->repeat_penalty : v / p->repeat_penalty;
            l[t] = v - ((float)(k - i) * p->frequency_penalty + p->presence_penalty);
        }
        i = k;
    }
    free(ids);
    return 0;
}

/* logit descending, id ascending */
static int by_logit(const void *a, const void *b) {
    const cand *x = (const cand *)a, *y = (const cand *)b;
    if (x->v != y->v) return x->v > y->v ? -1 : 1;
    return (x->id > y->id) - (x->id < y->id);
}
static int better(const cand *x, const cand *y) { return x->v > y->v || (x->v == y->v && x->id < y->id); }

/* The k best of c[0..n) in order at the front (a heap of the k best so far whose root is the
 * worst of them, then a sort of the k). */
static void top_k_first(cand *c, int n, int k) {
    /* heap over c[0..k): parent is worse than its children */
    for (int i = 1; i < k; ++i)
        for (int j = i; j > 0 && better(&c[(j - 1) / 2], &c[j]); j = (j - 1) / 2) {
            cand t = c[j];
            c[j] = c[(j - 1) / 2];
            c[(j - 1) / 2] = t;
        }
    for (int i = k; i < n; ++i) {
        if (!better(&c[i], &c[0])) continue;
        c[0] = c[i];
        for (int j = 0;;) {
            int w = j;
            const int a = 2 * j + 1, b = a + 1;
            if (a < k && better(&c[w], &c[a])) w = a;
            if (b < k && better(&c[w], &c[b])) w = b;
            if (w == j) break;
            cand t = c[j];
            c[j] = c[w];
            c[w] = t;
            j = w;
        }
    }
    qsort(c, (size_t)k, sizeof(cand), by_logit);
}

/* draw (src/sample.c:855-877): float32 weights, float64 sums, the first candidate whose running
 * sum reaches sum * u; a zero weight never wins. */
static int64_t draw(lgml_sampler *sm, const cand *c, int n) {
    float m = c[0].v;
    for (int i = 1; i < n; ++i)
        if (c[i].v > m) m = c[i].v;
    double total = 0.0;
    for (int i = 0; i < n; ++i) total += (double)expf(c[i].v - m);
    const double tgt = total * lgml_sampler_uniform(sm);
    double run = 0.0;
    int64_t last_nz = c[0].id;
    int any = 0;
    for (int i = 0; i < n; ++i) {
        const double w = (double)expf(c[i].v - m);
        run += w;
        if (w > 0.0) {
            if (run >= tgt) return c[i].id;
            last_nz = c[i].id;
            any = 1;
        }
    }
    return any ? last_nz : c[0].id;
}

/* top_p (apply_top_p, :808-831; float32 running sums), min_p (apply_min_p, :834-852),
 * temperature, draw.  c is sorted iff `sorted`. */
static int64_t after_top_k(lgml_sampler *sm, cand *c, int n, int sorted) {
    const lgml_sampler_params *p = &sm->p;
    if (p->top_p < 1.f) {
        if (!sorted) qsort(c, (size_t)n, sizeof(cand), by_logit);
        float total = 0.f;
        for (int i = 0; i < n; ++i) total += expf(c[i].v - c[0].v);
        float cum = 0.f;
        int keep = n;
        for (int i = 0; i < n; ++i) {
            cum += expf(c[i].v - c[0].v) / total;
            if (cum >= p->top_p) {
                keep = i + 1;
                break;
            }
        }
        n = keep;
    }
    if (p->min_p > 0.f) {
        float m = c[0].v;
        for (int i = 1; i < n; ++i)
            if (c[i].v > m) m = c[i].v;
        const float thr = m + logf(p->min_p);          /* float32 as the reference's (src/sample.c:841, :847) */
        int k = 0;
        for (int i = 0; i < n; ++i)
            if (c[i].v >= thr) c[k++] = c[i];
        n = k;
    }
    if (p->temperature != 1.f)
        for (int i = 0; i < n; ++i) c[i].v = c[i].v / p->temperature;
    return draw(sm, c, n);
}

static int need_cands(lgml_sampler *sm, int n) {
    if (n <= sm->c_cap) return 0;
    cand *c = (cand *)realloc(sm->c, (size_t)n * sizeof(cand));
    if (!c) {
        set_error("sampler: out of memory");
        return -1;
    }
    sm->c = c;
    sm->c_cap = n;
    return 0;
}

int lgml_sampler_sample(lgml_sampler *sm, const float *logits, int n, float *edited) {
    if (n <= 0) {
        set_error("sampler: an empty row");
        return -1;
    }
    if (n > sm->last_cap) {
        float *l = (float *)realloc(sm->last, (size_t)n * sizeof(float));
        if (!l) {
            set_error("sampler: out of memory");
            return -1;
        }
        sm->last = l;
        sm->last_cap = n;
    }
    float *l = sm->last;
    sm->last_n = n;
    memcpy(l, logits, (size_t)n * sizeof(float));
    for (int i = 0; i < sm->n_bias; ++i)
        if (sm->bias_ids[i] >= 0 && sm->bias_ids[i] < n) l[sm->bias_ids[i]] += sm->bias[i];
    if (apply_penalties(sm, l, n)) return -1;
    if (edited) memcpy(edited, l, (size_t)n * sizeof(float));
    const lgml_sampler_params *p = &sm->p;
    if (!(p->temperature > 0.f)) {      /* the first maximum: the lowest index wins a tie */
        int best = 0;
        for (int i = 1; i < n; ++i)
            if (l[i] > l[best]) best = i;
        return best;
    }
    if (need_cands(sm, n)) return -1;
    for (int i = 0; i < n; ++i) {
        sm->c[i].id = i;
        sm->c[i].v = l[i];
    }
    int sorted = 0, m = n;
    if (p->top_k > 0 && p->top_k < n) {
        top_k_first(sm->c, n, p->top_k);
        m = p->top_k;
        sorted = 1;
    }
    return (int)after_top_k(sm, sm->c, m, sorted);
}

int lgml_sampler_sample_candidates(lgml_sampler *sm, const int64_t *ids, const float *vals, int k) {
    if (!(sm->p.temperature > 0.f)) {
        set_error("sampler: candidates are for temperature > 0 (the argmax needs none)");
        return -1;
    }
    if (k <= 0) {
        set_error("sampler: no candidates");
        return -1;
    }
    if (need_cands(sm, k)) return -1;
    for (int i = 0; i < k; ++i) {
        sm->c[i].id = ids[i];
        sm->c[i].v = vals[i];
    }
    sm->last_n = 0;
    return (int)after_top_k(sm, sm->c, k, 1);
}

/* sampler_logprobs (src/sample.c:1075-1110): log-softmax of the last sampled row after bias and
 * penalties, before temperature and truncation. */
int lgml_sampler_logprobs(const lgml_sampler *sm, int32_t token, int k, double *lp, int32_t *top_ids, double *top_lp) {
    const int n = sm->last_n;
    if (n <= 0) {
        set_error("sampler: no logits: sample first");
        return -1;
    }
    if (token < 0 || token >= n || k < 0 || k > n) {
        set_error("sampler: bad token id or count");
        return -1;
    }
    const float *l = sm->last;
    float m = l[0];
    for (int i = 1; i < n; ++i)
        if (l[i] > m) m = l[i];
    double sum = 0.0;
    for (int i = 0; i < n; ++i) sum += exp((double)l[i] - (double)m);
    const double lse = (double)m + log(sum);
    *lp = (double)l[token] - lse;
    if (k > 0) {
        cand *c = (cand *)malloc((size_t)n * sizeof(cand));
        if (!c) {
            set_error("sampler: out of memory");
            return -1;
        }
        for (int i = 0; i < n; ++i) {
            c[i].id = i;
            c[i].v = l[i];
        }
        if (k < n) top_k_first(c, n, k);
        else qsort(c, (size_t)n, sizeof(cand), by_logit);
        for (int i = 0; i < k; ++i) {
            top_ids[i] = (int32_t)c[i].id;
            top_lp[i] = (double)c[i].v - lse;
        }
        free(c);
    }
    return 0;
}

void lgml_sampler_state(const lgml_sampler *sm, uint64_t out[4]) { memcpy(out, sm->s, sizeof(sm->s)); }
