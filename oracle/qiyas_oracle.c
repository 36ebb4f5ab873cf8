/*
 * qiyas_oracle.c -- TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C restatement, on the CPU, of the arithmetic of Qiyas's block-scaled
 * quantized product path.  Only the tests, the smoke check and the bench's
 * cpu_baseline / reference arm may load this library; the CUDA library never
 * links or calls it.
 *
 * Parity status: the reference is C# (.NET 10) and cannot be executed where
 * this is built, so the oracle is pinned against the reference's own
 * known-answer blocks (src/Checks.cs:264-355, reproduced as formulas over
 * indices in tests/) and its round-trip gate (src/Checks.cs:198-207).  The
 * reference holds no stored golden outputs for the products; the f32-lane
 * products are therefore "parity unpinned" beyond what those gates fix: the
 * restatement follows the cited source line by line instead.
 *
 * Every function names the reference lines it follows.  Build with
 * -ffp-contract=off so that no multiply-add is fused unless written as fmaf().
 */
#define _GNU_SOURCE
#include <immintrin.h>
#include <math.h>
#include <pthread.h>
#include <sched.h>
#include <stdatomic.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#define QO_Q8_0 0
#define QO_Q4_0 1
#define QO_Q4_K 2
#define QO_Q6_K 3
#define QO_F32 100

#define QO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ half */

/* (float)Half: exact widening, subnormals included (src/Blocks.cs:27). */
QO_API float qo_half_to_float(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 31u, man = h & 1023u, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 1024u));
            bits = sign | (uint32_t)(127 - 15 - e) << 23 | (man & 1023u) << 13;
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | man << 13;
    else bits = sign | (exp + 112u) << 23 | man << 13;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* (Half)float: round to nearest, ties to even, subnormals and overflow to infinity (src/Blocks.cs:28). */
QO_API uint16_t qo_float_to_half(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u, abs = x & 0x7FFFFFFFu;
    if (abs >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (abs > 0x7F800000u ? 0x200u | ((abs >> 13) & 1023u) : 0));
    if (abs >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);           /* rounds to or past 65520 */
    if (abs < 0x33000001u) return (uint16_t)sign;                        /* at most half the least subnormal */
    int exp = (int)(abs >> 23) - 127;
    uint32_t man = (abs & 0x7FFFFFu) | 0x800000u;
    int shift = exp < -14 ? 13 + (-14 - exp) : 13;
    uint32_t kept = man >> shift, rest = man & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
    if (rest > halfway || (rest == halfway && (kept & 1u))) kept++;
    uint32_t out = exp < -14 ? kept : ((uint32_t)(exp + 15) << 10) + (kept - 1024u);
    return (uint16_t)(sign | out);
}

static float half_at(const uint8_t *p) { return qo_half_to_float((uint16_t)(p[0] | p[1] << 8)); }
static void half_put(float v, uint8_t *p) { uint16_t h = qo_float_to_half(v); p[0] = (uint8_t)h; p[1] = (uint8_t)(h >> 8); }

QO_API int qo_block_values(int fmt) { return fmt == QO_Q8_0 || fmt == QO_Q4_0 ? 32 : fmt == QO_Q4_K || fmt == QO_Q6_K ? 256 : 0; }
QO_API int qo_block_bytes(int fmt) { return fmt == QO_Q8_0 ? 34 : fmt == QO_Q4_0 ? 18 : fmt == QO_Q4_K ? 144 : fmt == QO_Q6_K ? 210 : 0; }
/* TN.Bytes(values): whole blocks (src/Blocks.cs:269,287,305,323). */
QO_API int64_t qo_bytes(int fmt, int64_t values)
{
    int bv = qo_block_values(fmt);
    return bv ? (values + bv - 1) / bv * qo_block_bytes(fmt) : 0;
}

/* ------------------------------------------------------------------ decoders */

/* DecodeQ8_0 (src/Blocks.cs:31-35). */
static void dec_q8_0(const uint8_t *b, float *v)
{
    float d = half_at(b);
    for (int i = 0; i < 32; i++) v[i] = d * (float)(int8_t)b[2 + i];
}

/* DecodeQ4_0 (src/Blocks.cs:48-56). */
static void dec_q4_0(const uint8_t *b, float *v)
{
    float d = half_at(b);
    for (int i = 0; i < 16; i++) {
        v[i] = d * (float)((b[2 + i] & 15) - 8);
        v[i + 16] = d * (float)((b[2 + i] >> 4) - 8);
    }
}

/* ScaleMin (src/Blocks.cs:73-77). */
static void scale_min(const uint8_t *sc, int j, int *scale, int *min)
{
    if (j < 4) { *scale = sc[j] & 63; *min = sc[j + 4] & 63; }
    else { *scale = (sc[j + 4] & 15) | ((sc[j - 4] >> 6) << 4); *min = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
}

/* DecodeQ4_K (src/Blocks.cs:79-96): both products rounded to f32 before the subtraction. */
static void dec_q4_k(const uint8_t *b, float *v)
{
    float d = half_at(b), dmin = half_at(b + 2);
    const uint8_t *sc = b + 4, *qs = b + 16;
    for (int pair = 0; pair < 4; pair++) {
        int s0, m0, s1, m1;
        scale_min(sc, 2 * pair, &s0, &m0);
        scale_min(sc, 2 * pair + 1, &s1, &m1);
        float d0 = d * (float)s0, dm0 = dmin * (float)m0, d1 = d * (float)s1, dm1 = dmin * (float)m1;
        for (int i = 0; i < 32; i++) {
            uint8_t q = qs[pair * 32 + i];
            v[pair * 64 + i] = d0 * (float)(q & 15) - dm0;
            v[pair * 64 + 32 + i] = d1 * (float)(q >> 4) - dm1;
        }
    }
}

/* DecodeQ6_K (src/Blocks.cs:151-173): d * scale * q, left to right in f32. */
static void dec_q6_k(const uint8_t *b, float *v)
{
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t *sc = (const int8_t *)(b + 192);
    float d = half_at(b + 208);
    for (int half = 0; half < 2; half++) {
        const uint8_t *l = ql + half * 64, *h = qh + half * 32;
        const int8_t *s = sc + half * 8;
        float *o = v + half * 128;
        for (int i = 0; i < 32; i++) {
            int g = i / 16;
            int q1 = ((l[i] & 15) | (((h[i] >> 0) & 3) << 4)) - 32;
            int q2 = ((l[i + 32] & 15) | (((h[i] >> 2) & 3) << 4)) - 32;
            int q3 = ((l[i] >> 4) | (((h[i] >> 4) & 3) << 4)) - 32;
            int q4 = ((l[i + 32] >> 4) | (((h[i] >> 6) & 3) << 4)) - 32;
            o[i] = d * (float)s[g] * (float)q1;
            o[i + 32] = d * (float)s[g + 2] * (float)q2;
            o[i + 64] = d * (float)s[g + 4] * (float)q3;
            o[i + 96] = d * (float)s[g + 6] * (float)q4;
        }
    }
}

static void dec_block(int fmt, const uint8_t *b, float *v)
{
    switch (fmt) {
    case QO_Q8_0: dec_q8_0(b, v); break;
    case QO_Q4_0: dec_q4_0(b, v); break;
    case QO_Q4_K: dec_q4_k(b, v); break;
    default: dec_q6_k(b, v); break;
    }
}

/* TN.Load over whole blocks (src/Blocks.cs:218-230): values [0, count) of a block array as f32. */
QO_API int qo_decode(int fmt, const uint8_t *blocks, int64_t count, float *out)
{
    int bv = qo_block_values(fmt), bb = qo_block_bytes(fmt);
    if (!bv) return -1;
    float tmp[256];
    for (int64_t at = 0; at < count; at += bv) {
        dec_block(fmt, blocks + at / bv * bb, tmp);
        int64_t n = count - at < bv ? count - at : bv;
        memcpy(out + at, tmp, (size_t)n * 4);
    }
    return 0;
}

/* ------------------------------------------------------------------ encoders */

static float clampf(float v, float lo, float hi) { return v < lo ? lo : v > hi ? hi : v; }
static int clampi(int v, int lo, int hi) { return v < lo ? lo : v > hi ? hi : v; }

/* EncodeQ8_0 (src/Blocks.cs:37-45); device twin src/Ptx.Blocks.cs:54-73 (div.rn, cvt.rni: the same roundings).
 * MathF.Round is ties-to-even = rintf under the default rounding mode. */
static void enc_q8_0(const float *v, uint8_t *b)
{
    float amax = 0;
    for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(v[i]));
    float d = amax / 127;
    half_put(d, b);
    d = half_at(b);
    float id = d == 0 ? 0 : 1 / d;
    for (int i = 0; i < 32; i++) b[2 + i] = (uint8_t)(int8_t)clampf(rintf(v[i] * id), -127, 127);
}

/* EncodeQ4_0 (src/Blocks.cs:58-70).  fused = 0: the CPU's v*id + 8.5f in two roundings, truncated;
 * fused = 1: the device's fma.rn then cvt.rmi (src/Ptx.Blocks.cs:80-85). */
static void enc_q4_0(const float *v, uint8_t *b, int fused)
{
    float amax = 0, max = 0;
    for (int i = 0; i < 32; i++) if (fabsf(v[i]) > amax) { amax = fabsf(v[i]); max = v[i]; }
    float d = max / -8;
    half_put(d, b);
    d = half_at(b);
    float id = d == 0 ? 0 : 1 / d;
    for (int i = 0; i < 16; i++) {
        float tl, th;
        int lo, hi;
        if (fused) {
            tl = fmaf(v[i], id, 8.5f); th = fmaf(v[i + 16], id, 8.5f);
            lo = (int)floorf(clampf(tl, -64.f, 64.f)); hi = (int)floorf(clampf(th, -64.f, 64.f));
        } else {
            tl = v[i] * id; tl = tl + 8.5f; th = v[i + 16] * id; th = th + 8.5f;
            lo = (int)clampf(tl, -64.f, 64.f); hi = (int)clampf(th, -64.f, 64.f);
        }
        lo = clampi(lo, 0, 15); hi = clampi(hi, 0, 15);
        b[2 + i] = (uint8_t)(lo | hi << 4);
    }
}

static int round_clamp(float x, int lo, int hi) { return clampi((int)clampf(rintf(x), -1e6f, 1e6f), lo, hi); }

/* EncodeQ4_K (src/Blocks.cs:98-148). */
static void enc_q4_k(const float *v, uint8_t *b)
{
    float scales[8], mins[8], max_scale = 0, max_min = 0;
    for (int j = 0; j < 8; j++) {
        float lo = 3.40282347e38f, hi = -3.40282347e38f;
        for (int i = 0; i < 32; i++) { float x = v[j * 32 + i]; lo = fminf(lo, x); hi = fmaxf(hi, x); }
        lo = fminf(lo, 0);
        scales[j] = (hi - lo) / 15; mins[j] = -lo;
        max_scale = fmaxf(max_scale, scales[j]); max_min = fmaxf(max_min, mins[j]);
    }
    float d = max_scale / 63, dmin = max_min / 63;
    half_put(d, b); half_put(dmin, b + 2);
    d = half_at(b); dmin = half_at(b + 2);
    uint8_t *sc = b + 4;
    memset(sc, 0, 12);
    int ls[8], lm[8];
    for (int j = 0; j < 8; j++) {
        ls[j] = d == 0 ? 0 : round_clamp(scales[j] / d, 0, 63);
        lm[j] = dmin == 0 ? 0 : round_clamp(mins[j] / dmin, 0, 63);
    }
    for (int j = 0; j < 8; j++) {
        if (j < 4) { sc[j] = (uint8_t)ls[j]; sc[j + 4] = (uint8_t)lm[j]; }
        else {
            sc[j + 4] = (uint8_t)((ls[j] & 15) | ((lm[j] & 15) << 4));
            sc[j - 4] |= (uint8_t)((ls[j] >> 4) << 6);
            sc[j] |= (uint8_t)((lm[j] >> 4) << 6);
        }
    }
    uint8_t *qs = b + 16;
    for (int j = 0; j < 8; j++) {
        float dj = d * (float)ls[j], mj = dmin * (float)lm[j];
        for (int i = 0; i < 32; i++) {
            int q = dj == 0 ? 0 : round_clamp((v[j * 32 + i] + mj) / dj, 0, 15);
            int at = j / 2 * 32 + i;
            if (j % 2 == 0) qs[at] = (uint8_t)((qs[at] & 0xF0) | q); else qs[at] = (uint8_t)((qs[at] & 0x0F) | q << 4);
        }
    }
}

/* EncodeQ6_K (src/Blocks.cs:175-215). */
static void enc_q6_k(const float *v, uint8_t *b)
{
    float scales[16], max_scale = 0;
    for (int j = 0; j < 16; j++) {
        float amax = 0;
        for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(v[j * 16 + i]));
        scales[j] = amax / 31;
        max_scale = fmaxf(max_scale, scales[j]);
    }
    float d = max_scale / 127;
    half_put(d, b + 208);
    d = half_at(b + 208);
    int ls[16], q[256];
    for (int j = 0; j < 16; j++) {
        ls[j] = d == 0 ? 0 : round_clamp(scales[j] / d, -127, 127);
        b[192 + j] = (uint8_t)(int8_t)ls[j];
    }
    for (int j = 0; j < 16; j++) {
        float dj = d * (float)ls[j];
        for (int i = 0; i < 16; i++) q[j * 16 + i] = (dj == 0 ? 0 : round_clamp(v[j * 16 + i] / dj, -32, 31)) + 32;
    }
    memset(b, 0, 192);
    for (int half = 0; half < 2; half++) {
        uint8_t *l = b + half * 64, *h = b + 128 + half * 32;
        const int *p = q + half * 128;
        for (int i = 0; i < 32; i++) {
            int q1 = p[i], q2 = p[i + 32], q3 = p[i + 64], q4 = p[i + 96];
            l[i] = (uint8_t)((q1 & 15) | ((q3 & 15) << 4));
            l[i + 32] = (uint8_t)((q2 & 15) | ((q4 & 15) << 4));
            h[i] = (uint8_t)(((q1 >> 4) & 3) | (((q2 >> 4) & 3) << 2) | (((q3 >> 4) & 3) << 4) | (((q4 >> 4) & 3) << 6));
        }
    }
}

/* TN.Store of `count` values into a fresh buffer (src/Blocks.cs:235-249): a last partial block is encoded with
 * zeros past the count, which is also what the device encoder reads (src/Ptx.Blocks.cs:36-44).
 * variant 0 = the CPU encoders, 1 = the device's Q4_0 rounding (fma, floor). */
QO_API int qo_encode(int fmt, const float *values, int64_t count, uint8_t *blocks, int variant)
{
    int bv = qo_block_values(fmt), bb = qo_block_bytes(fmt);
    if (!bv) return -1;
    float tmp[256];
    for (int64_t at = 0; at < count; at += bv) {
        int64_t n = count - at < bv ? count - at : bv;
        memset(tmp, 0, sizeof tmp);
        memcpy(tmp, values + at, (size_t)n * 4);
        uint8_t *b = blocks + at / bv * bb;
        switch (fmt) {
        case QO_Q8_0: enc_q8_0(tmp, b); break;
        case QO_Q4_0: enc_q4_0(tmp, b, variant); break;
        case QO_Q4_K: enc_q4_k(tmp, b); break;
        default: enc_q6_k(tmp, b); break;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ the thread team */

/* Team.For (src/Team.cs:46-94): the caller and size-1 kept workers take chunks from one counter; a job of one chunk,
 * or of fewer than 2^15 work units, runs on the caller. */
typedef void (*qo_body)(void *ctx, int first, int last);

static struct {
    pthread_mutex_t gate, lock;
    pthread_cond_t wake;
    pthread_t *threads;
    int size, started;
    qo_body body;
    void *ctx;
    int count, chunk, chunks;
    atomic_int next, done;
    int generation;
} team = { PTHREAD_MUTEX_INITIALIZER, PTHREAD_MUTEX_INITIALIZER, PTHREAD_COND_INITIALIZER, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0 };

static void team_take(void)
{
    for (;;) {
        int c = atomic_fetch_add(&team.next, 1);
        if (c >= team.chunks) return;
        int first = c * team.chunk, last = first + team.chunk < team.count ? first + team.chunk : team.count;
        team.body(team.ctx, first, last);
        atomic_fetch_add(&team.done, 1);
    }
}

static void *team_worker(void *arg)
{
    (void)arg;
    int seen = 0;
    for (;;) {
        pthread_mutex_lock(&team.lock);
        while (team.generation == seen) pthread_cond_wait(&team.wake, &team.lock);
        seen = team.generation;
        pthread_mutex_unlock(&team.lock);
        if (seen < 0) return 0;
        team_take();
    }
}

QO_API int qo_team_size(void)
{
    if (!team.size) {
        long n = sysconf(_SC_NPROCESSORS_ONLN);
        const char *env = getenv("QIYAS_ORACLE_THREADS");
        if (env && atoi(env) > 0) n = atoi(env);
        team.size = n < 1 ? 1 : (int)n;
    }
    return team.size;
}

QO_API void qo_team_set_size(int threads)
{
    if (!team.started && threads > 0) team.size = threads;
}

static void team_for(int count, int chunk, int64_t work, qo_body body, void *ctx)
{
    int size = qo_team_size(), chunks = (count + chunk - 1) / chunk;
    if (chunks <= 1 || work < (1 << 15) || size == 1) { body(ctx, 0, count); return; }
    pthread_mutex_lock(&team.gate);
    if (!team.started) {
        team.threads = (pthread_t *)calloc((size_t)size, sizeof(pthread_t));
        for (int i = 0; i < size - 1; i++) pthread_create(&team.threads[i], 0, team_worker, 0);
        team.started = 1;
    }
    team.body = body; team.ctx = ctx; team.count = count; team.chunk = chunk; team.chunks = chunks;
    atomic_store(&team.done, 0);
    atomic_store(&team.next, 0);
    pthread_mutex_lock(&team.lock);
    team.generation++;
    pthread_cond_broadcast(&team.wake);
    pthread_mutex_unlock(&team.lock);
    team_take();
    while (atomic_load(&team.done) < chunks) sched_yield();
    atomic_store(&team.next, 1 << 30);          /* the job is closed: a late worker finds no chunk */
    pthread_mutex_unlock(&team.gate);
}

/* ------------------------------------------------------------------ integer rows */

/* Kernels.UnpackBlock (src/BlockProducts.cs:30-35): scale and 32 int8 (Q4_0: q - 8). */
static void unpack_block(int fmt, const uint8_t *b, float *scale, int8_t *q)
{
    *scale = half_at(b);
    if (fmt == QO_Q8_0) { memcpy(q, b + 2, 32); return; }
    for (int i = 0; i < 16; i++) { q[i] = (int8_t)((b[2 + i] & 15) - 8); q[i + 16] = (int8_t)((b[2 + i] >> 4) - 8); }
}

/* Dot32 (src/BlockProducts.cs:58-70).  Variant 0 is its plain-integer branch (:66-69, the lane the reference calls
 * "s32 blocks"); variant 1 stands in for its vector branch (:60-64: one 256-bit S8Dot.Fma and a horizontal sum, the
 * lane "s8dp blocks", which needs AVX-VNNI-INT8): the same exact integer from AVX2's widening multiply-adds, |p| times
 * q with p's sign (pairs of products fit 16 bits: 2 * 127 * 128 < 2^15), then pairs of 16-bit sums into 32 bits.
 * Variant 1 also unpacks Q4_0 nibbles 16 at a time.  Both give bit-identical results; the bench times both. */
static int g_dot_variant = 0;
QO_API void qo_set_dot_variant(int v) { g_dot_variant = v; }
QO_API int qo_dot_variant_available(int v) { return v == 0 || (v == 1 && __builtin_cpu_supports("avx2") && __builtin_cpu_supports("f16c")); }
/* the block's f16 scale by the F16C instruction (bit-identical to qo_half_to_float: the conversion is exact) */
__attribute__((target("avx2,f16c"))) static float half_at_f16c(const uint8_t *p) { return _cvtsh_ss((unsigned short)(p[0] | p[1] << 8)); }

static int dot32_scalar(const int8_t *p, const int8_t *q)
{
    int sum = 0;
    for (int i = 0; i < 32; i++) sum += p[i] * q[i];
    return sum;
}

__attribute__((target("avx2"))) static int dot32_avx2(const int8_t *p, const int8_t *q)
{
    const __m256i a = _mm256_loadu_si256((const __m256i *)p), b = _mm256_loadu_si256((const __m256i *)q);
    const __m256i pairs = _mm256_maddubs_epi16(_mm256_abs_epi8(a), _mm256_sign_epi8(b, a));
    const __m256i quads = _mm256_madd_epi16(pairs, _mm256_set1_epi16(1));
    __m128i s = _mm_add_epi32(_mm256_castsi256_si128(quads), _mm256_extracti128_si256(quads, 1));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4E));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xB1));
    return _mm_cvtsi128_si32(s);
}

/* UnpackBlock for Q4_0 with 128-bit operations: low nibbles are values 0..15, high nibbles values 16..31, each minus 8. */
__attribute__((target("avx2,f16c"))) static void unpack_q4_0_avx2(const uint8_t *b, float *scale, int8_t *q)
{
    *scale = half_at_f16c(b);
    const __m128i raw = _mm_loadu_si128((const __m128i *)(b + 2)), m = _mm_set1_epi8(15), eight = _mm_set1_epi8(8);
    _mm_storeu_si128((__m128i *)q, _mm_sub_epi8(_mm_and_si128(raw, m), eight));
    _mm_storeu_si128((__m128i *)(q + 16), _mm_sub_epi8(_mm_and_si128(_mm_srli_epi16(raw, 4), m), eight));
}

static int dot32(const int8_t *p, const int8_t *q) { return g_dot_variant == 1 ? dot32_avx2(p, q) : dot32_scalar(p, q); }

struct gemv_job {
    int fmt_a, order, cols, bb;
    const uint8_t *a;
    const float *xs;
    const int8_t *xq;
    float *y;
    int32_t *sums;
    double *abs_sum;
};

/* GemvBlockBody.Run (src/BlockProducts.cs:39-55) for order 0: acc += d * xs[b] * dot, every operation rounded to
 * f32 on its own.  Order 1 is the device kernel's (src/BlockProducts.cs:158-161): scale = dA*dX, then
 * acc = fma(scale, float(dot), acc).  Both walk the blocks in ascending order. */
static void gemv_body(void *p, int first, int last)
{
    struct gemv_job *j = (struct gemv_job *)p;
    int blocks = j->cols / 32;
    int8_t q[32];
    const int fast = g_dot_variant == 1;
    for (int r = first; r < last; r++) {
        float acc = 0;
        double mag = 0;
        for (int b = 0; b < blocks; b++) {
            float d;
            const uint8_t *blk = j->a + ((int64_t)r * blocks + b) * j->bb;
            int dot;
            if (fast && j->fmt_a == QO_Q8_0) { d = half_at_f16c(blk); dot = dot32_avx2((const int8_t *)blk + 2, j->xq + b * 32); }
            else if (fast) { unpack_q4_0_avx2(blk, &d, q); dot = dot32_avx2(q, j->xq + b * 32); }
            else { unpack_block(j->fmt_a, blk, &d, q); dot = dot32_scalar(q, j->xq + b * 32); }
            if (j->sums) j->sums[(int64_t)r * blocks + b] = dot;
            if (j->order == 0) { float s = d * j->xs[b]; float t = s * (float)dot; acc = acc + t; }
            else { float s = d * j->xs[b]; acc = fmaf(s, (float)dot, acc); }
            if (j->abs_sum) mag += fabs((double)d * (double)j->xs[b] * (double)dot);      /* test-only: not in the timed path */
        }
        j->y[r] = acc;
        if (j->abs_sum) j->abs_sum[r] = mag;
    }
}

/* x as (scale, int8 values) per block of 32: Q8_0 / Q4_0 blocks unpacked (src/BlockProducts.cs:22-24), or f32 values
 * first encoded to Q8_0 as the reference encodes activations (src/Blocks.cs:37-45). */
static int unpack_x(int fmt_x, const void *x, int cols, float *xs, int8_t *xq)
{
    int blocks = cols / 32;
    if (fmt_x == QO_F32) {
        uint8_t blk[34];
        for (int b = 0; b < blocks; b++) { enc_q8_0((const float *)x + b * 32, blk); unpack_block(QO_Q8_0, blk, &xs[b], xq + b * 32); }
        return 0;
    }
    if (fmt_x != QO_Q8_0 && fmt_x != QO_Q4_0) return -1;
    int bb = qo_block_bytes(fmt_x);
    for (int b = 0; b < blocks; b++) unpack_block(fmt_x, (const uint8_t *)x + (int64_t)b * bb, &xs[b], xq + b * 32);
    return 0;
}

/* Kernels.GemvBlocks (src/BlockProducts.cs:17-27), widened to a second operand format: y = A.x for A in Q8_0 or Q4_0
 * and x in Q8_0, Q4_0 or f32 (quantized to Q8_0 first).  order 0 = CPU rounding order, 1 = device rounding order.
 * sums (rows*blocks s32) and abs_sum (rows f64, sum of |term|) are optional outputs for the tests. */
QO_API int qo_gemv_blocks(int fmt_a, int fmt_x, const uint8_t *a, const void *x, float *y, int rows, int cols, int order,
                          int32_t *sums, double *abs_sum)
{
    if ((fmt_a != QO_Q8_0 && fmt_a != QO_Q4_0) || cols % 32 != 0 || cols <= 0 || rows < 0) return -1;
    int blocks = cols / 32;
    float *xs = (float *)malloc((size_t)blocks * 4);
    int8_t *xq = (int8_t *)malloc((size_t)cols);
    if (unpack_x(fmt_x, x, cols, xs, xq)) { free(xs); free(xq); return -1; }
    struct gemv_job job = { fmt_a, order, cols, qo_block_bytes(fmt_a), a, xs, xq, y, sums, abs_sum };
    int chunk = rows / (qo_team_size() * 4);
    team_for(rows, chunk < 1 ? 1 : chunk, (int64_t)rows * cols, gemv_body, &job);
    free(xs); free(xq);
    return 0;
}

/* ------------------------------------------------------------------ K-quant rows against Q8_0 activations */

/* The reference has no integer product for Q4_K / Q6_K (its gemv decodes them, src/GpuOps.cs:287-300).  These are
 * the exact integer sums the block formulation rests on, from the byte layouts of src/Blocks.cs:73-96,151-173:
 *   Q4_K sub-block j (32 values):  S_j = sum q*qx  and  X_j = sum qx   (value = (d*sc_j)*q - dmin*m_j)
 *   Q6_K 32 values = two 16-value sub-blocks:  T = sc_a*sum (q-32)*qx + sc_b*sum (q-32)*qx  (value = d*sc*(q-32))
 * sums gets one s32 per 32 values (Q4_K: S_j; Q6_K: T). */
QO_API int qo_k_block_sums(int fmt_a, const uint8_t *a, const int8_t *xq, int rows, int cols, int32_t *sums)
{
    if ((fmt_a != QO_Q4_K && fmt_a != QO_Q6_K) || cols % 256 != 0) return -1;
    int sbs = cols / 256, bb = qo_block_bytes(fmt_a);
    for (int r = 0; r < rows; r++) {
        for (int s = 0; s < sbs; s++) {
            const uint8_t *b = a + ((int64_t)r * sbs + s) * bb;
            const int8_t *x = xq + s * 256;
            int32_t *out = sums + ((int64_t)r * sbs + s) * 8;
            if (fmt_a == QO_Q4_K) {
                for (int j = 0; j < 8; j++) {
                    int acc = 0;
                    for (int i = 0; i < 32; i++) {
                        uint8_t q = b[16 + j / 2 * 32 + i];
                        acc += (j % 2 ? q >> 4 : q & 15) * x[j * 32 + i];
                    }
                    out[j] = acc;
                }
            } else {
                int q[256];
                for (int half = 0; half < 2; half++) {
                    const uint8_t *l = b + half * 64, *h = b + 128 + half * 32;
                    for (int i = 0; i < 32; i++) {
                        q[half * 128 + i] = ((l[i] & 15) | (((h[i] >> 0) & 3) << 4)) - 32;
                        q[half * 128 + i + 32] = ((l[i + 32] & 15) | (((h[i] >> 2) & 3) << 4)) - 32;
                        q[half * 128 + i + 64] = ((l[i] >> 4) | (((h[i] >> 4) & 3) << 4)) - 32;
                        q[half * 128 + i + 96] = ((l[i + 32] >> 4) | (((h[i] >> 6) & 3) << 4)) - 32;
                    }
                }
                const int8_t *sc = (const int8_t *)(b + 192);
                for (int j = 0; j < 8; j++) {
                    int lo = 0, hi = 0;
                    for (int i = 0; i < 16; i++) { lo += q[j * 32 + i] * x[j * 32 + i]; hi += q[j * 32 + 16 + i] * x[j * 32 + 16 + i]; }
                    out[j] = sc[2 * j] * lo + sc[2 * j + 1] * hi;
                }
            }
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ float64 references */

/* References.Gemv (Program.cs:946-952): y[i] = sum_j a[i,j]*x[j] in float64 over the decoded stored values
 * (Registry.Values widens the f32 decode to double, src/Bench/Registry.cs:170-180). */
QO_API int qo_gemv_f64(int fmt_a, const uint8_t *a, const float *x, double *y, int rows, int cols)
{
    int bv = qo_block_values(fmt_a), bb = qo_block_bytes(fmt_a);
    if (!bv || cols % bv) return -1;
    int blocks = cols / bv;
    float v[256];
    for (int r = 0; r < rows; r++) {
        double s = 0;
        for (int b = 0; b < blocks; b++) {
            dec_block(fmt_a, a + ((int64_t)r * blocks + b) * bb, v);
            for (int i = 0; i < bv; i++) s += (double)v[i] * (double)x[b * bv + i];
        }
        y[r] = s;
    }
    return 0;
}

/* What the reference runs today for Q4_K / Q6_K (and any block type off the block path): Widen to f32
 * (src/Ptx.Attention.cs:202-219), then gemv_rows: a warp a row, lane l takes columns l, l+32, ... with one fma each,
 * then a shuffle tree (src/Ptx.Reduce.cs:554-592). */
QO_API int qo_gemv_decoded_f32(int fmt_a, const uint8_t *a, const float *x, float *y, int rows, int cols)
{
    int bv = qo_block_values(fmt_a), bb = qo_block_bytes(fmt_a);
    if (!bv || cols % bv) return -1;
    int blocks = cols / bv;
    float *row = (float *)malloc((size_t)cols * 4);
    for (int r = 0; r < rows; r++) {
        for (int b = 0; b < blocks; b++) dec_block(fmt_a, a + ((int64_t)r * blocks + b) * bb, row + b * bv);
        float lane[32];
        for (int l = 0; l < 32; l++) {
            float acc = 0;
            for (int c = l; c < cols; c += 32) acc = fmaf(row[c], x[c], acc);
            lane[l] = acc;
        }
        for (int off = 16; off > 0; off >>= 1) for (int l = 0; l < off; l++) lane[l] = lane[l] + lane[l + off];
        y[r] = lane[0];
    }
    free(row);
    return 0;
}

/* ------------------------------------------------------------------ A.B^T */

struct mm_job {
    int m, n, k, order;
    const int8_t *qa, *qb;
    const float *sa, *sb;           /* one scale per block (k/32 per row) */
    float *c;
    int32_t *sums;
};

/* UnpackRows (src/MatMulBlocks.cs:84-110), with one scale kept per block instead of one per 4 bytes (equal values). */
static void unpack_rows(int fmt, const uint8_t *x, int rows, int k, int8_t *q, float *s)
{
    int blocks = k / 32, bb = qo_block_bytes(fmt);
    for (int64_t at = 0; at < (int64_t)rows * blocks; at++) unpack_block(fmt, x + at * bb, &s[at], q + at * 32);
}

static int dot4(const int8_t *p, const int8_t *q) { return p[0] * q[0] + p[1] * q[1] + p[2] * q[2] + p[3] * q[3]; }

/* order 0, MatMulBlocksBody (src/MatMulBlocks.cs:115-168) at Vector<int>.Count = 8: eight float lanes per C element;
 * lane l adds, for every 4-byte group g = l (mod 8) in ascending order, float(dot4) * (sA*sB); the lanes are then
 * summed.  Vector.Sum's order is the runtime's; pairwise halves are taken here.
 * order 1, the device tile (src/MatMulBlocks.cs:339-347): per block, acc = fma(float(D), sA*sB, acc), ascending. */
static void mm_body(void *p, int first, int last)
{
    struct mm_job *j = (struct mm_job *)p;
    int blocks = j->k / 32, k4 = j->k / 4;
    for (int i = first; i < last; i++) {
        for (int c = 0; c < j->n; c++) {
            const int8_t *a = j->qa + (int64_t)i * j->k, *b = j->qb + (int64_t)c * j->k;
            const float *sa = j->sa + (int64_t)i * blocks, *sb = j->sb + (int64_t)c * blocks;
            float out;
            if (j->order == 0) {
                float lane[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
                int v = 0;
                for (; v + 8 <= k4; v += 8)
                    for (int l = 0; l < 8; l++) {
                        int g = v + l;
                        float s = sa[g / 8] * sb[g / 8];
                        float t = (float)dot4(a + g * 4, b + g * 4) * s;
                        lane[l] = lane[l] + t;
                    }
                out = ((lane[0] + lane[4]) + (lane[2] + lane[6])) + ((lane[1] + lane[5]) + (lane[3] + lane[7]));
                for (; v < k4; v++) { float s = sa[v / 8] * sb[v / 8]; float t = (float)dot4(a + v * 4, b + v * 4) * s; out = out + t; }
            } else {
                float acc = 0;
                for (int kb = 0; kb < blocks; kb++) {
                    int d = dot32(a + kb * 32, b + kb * 32);
                    if (j->sums) j->sums[((int64_t)i * j->n + c) * blocks + kb] = d;
                    float s = sa[kb] * sb[kb];
                    acc = fmaf((float)d, s, acc);
                }
                out = acc;
            }
            j->c[(int64_t)i * j->n + c] = out;
        }
    }
}

/* Kernels.MatMulBlocks (src/MatMulBlocks.cs:28-36), widened to two operand formats: C (m x n) = A.B^T for A (m x k)
 * and B (n x k) each Q8_0 or Q4_0.  sums (optional, order 1 only): m*n*(k/32) exact block sums. */
QO_API int qo_matmul_blocks(int fmt_a, int fmt_b, const uint8_t *a, const uint8_t *b, float *c, int m, int n, int k, int order,
                            int32_t *sums)
{
    if ((fmt_a != QO_Q8_0 && fmt_a != QO_Q4_0) || (fmt_b != QO_Q8_0 && fmt_b != QO_Q4_0) || k % 32 != 0 || k <= 0) return -1;
    int blocks = k / 32;
    int8_t *qa = (int8_t *)malloc((size_t)m * k), *qb = (int8_t *)malloc((size_t)n * k);
    float *sa = (float *)malloc((size_t)m * blocks * 4), *sb = (float *)malloc((size_t)n * blocks * 4);
    unpack_rows(fmt_a, a, m, k, qa, sa);
    unpack_rows(fmt_b, b, n, k, qb, sb);
    struct mm_job job = { m, n, k, order, qa, qb, sa, sb, c, sums };
    team_for(m, 1, (int64_t)m * n * k, mm_body, &job);
    free(qa); free(qb); free(sa); free(sb);
    return 0;
}

/* The block product against Q4_K rows.  The reference has no such kernel (its Q4_K products decode to f32 first,
 * src/GpuOps.Products.cs:28-42); this restates the arithmetic this repo's device kernel defines for it, built from the
 * reference's pieces: DecodeQ4_K's value (d*sc)*q - dmin*m with both products rounded to f32 (src/Blocks.cs:88-93) and
 * the device tile's per-block fma (src/MatMulBlocks.cs:339-347).  Per 32-value sub-block, ascending:
 *     acc = fma(float(sum qA*q), sA * (d*sc), acc);   acc = fma(dmin*m, -(sA * float(sum qA)), acc).
 * sums (optional): the m*n*(k/32) exact sums of qA*q. */
struct mmk_job { int m, n, k; const int8_t *qa; const float *sa; const uint8_t *b; float *c; int32_t *sums; };

static void mmk_body(void *p, int first, int last)
{
    struct mmk_job *j = (struct mmk_job *)p;
    int blocks = j->k / 32, supers = j->k / 256;
    for (int i = first; i < last; i++)
        for (int c = 0; c < j->n; c++) {
            const int8_t *a = j->qa + (int64_t)i * j->k;
            const float *sa = j->sa + (int64_t)i * blocks;
            float acc = 0;
            for (int sb = 0; sb < supers; sb++) {
                const uint8_t *blk = j->b + ((int64_t)c * supers + sb) * 144;
                float d = half_at(blk), dmin = half_at(blk + 2);
                for (int sub = 0; sub < 8; sub++) {
                    int sc, mn, kb = sb * 8 + sub, dot = 0, sum = 0;
                    scale_min(blk + 4, sub, &sc, &mn);
                    const uint8_t *qs = blk + 16 + (sub / 2) * 32;
                    for (int t = 0; t < 32; t++) {
                        int q = (sub & 1) ? qs[t] >> 4 : qs[t] & 15;
                        dot += a[kb * 32 + t] * q;
                        sum += a[kb * 32 + t];
                    }
                    if (j->sums) j->sums[((int64_t)i * j->n + c) * blocks + kb] = dot;
                    float scale = d * (float)sc, min = dmin * (float)mn;
                    float s = sa[kb] * scale;
                    acc = fmaf((float)dot, s, acc);
                    float u = sa[kb] * (float)sum;
                    acc = fmaf(min, -u, acc);
                }
            }
            j->c[(int64_t)i * j->n + c] = acc;
        }
}

QO_API int qo_matmul_q4_k(int fmt_a, const uint8_t *a, const uint8_t *b, float *c, int m, int n, int k, int32_t *sums)
{
    if ((fmt_a != QO_Q8_0 && fmt_a != QO_Q4_0) || k % 256 != 0 || k <= 0) return -1;
    int blocks = k / 32;
    int8_t *qa = (int8_t *)malloc((size_t)m * k);
    float *sa = (float *)malloc((size_t)m * blocks * 4);
    unpack_rows(fmt_a, a, m, k, qa, sa);
    struct mmk_job job = { m, n, k, qa, sa, b, c, sums };
    team_for(m, 1, (int64_t)m * n * k, mmk_body, &job);
    free(qa); free(sa);
    return 0;
}

/* The block product against Q6_K rows (again no counterpart kernel in the reference).  DecodeQ6_K's value is
 * d * sc * q evaluated left to right (src/Blocks.cs:167-170), i.e. (d*sc) rounded, then times the code q - 32; a scale
 * covers 16 values.  Per 16-value sub-block s, ascending (A's block s / 2 supplies sA):
 *     acc = fma(float(sum of qA*(q-32) over the 16), sA * (d*sc[s]), acc).
 * sums (optional): the m*n*(k/16) exact sums. */
static void mm6_body(void *p, int first, int last)
{
    struct mmk_job *j = (struct mmk_job *)p;
    int blocks = j->k / 32, subs = j->k / 16, supers = j->k / 256;
    for (int i = first; i < last; i++)
        for (int c = 0; c < j->n; c++) {
            const int8_t *a = j->qa + (int64_t)i * j->k;
            const float *sa = j->sa + (int64_t)i * blocks;
            float acc = 0;
            for (int sb = 0; sb < supers; sb++) {
                const uint8_t *blk = j->b + ((int64_t)c * supers + sb) * 210;
                const uint8_t *ql = blk, *qh = blk + 128;
                const int8_t *sc = (const int8_t *)(blk + 192);
                float d = half_at(blk + 208);
                for (int s = 0; s < 16; s++) {
                    int half = s >> 3, g = (s >> 1) & 3, l0 = (s & 1) * 16, dot = 0, at = sb * 256 + half * 128 + g * 32 + l0;
                    for (int t = 0; t < 16; t++) {
                        int l = l0 + t;
                        int byte = ql[64 * half + 32 * (g & 1) + l];
                        int nib = g >= 2 ? byte >> 4 : byte & 15;
                        int q = (nib | (((qh[32 * half + l] >> (2 * g)) & 3) << 4)) - 32;
                        dot += a[at + t] * q;
                    }
                    if (j->sums) j->sums[((int64_t)i * j->n + c) * subs + sb * 16 + s] = dot;
                    float scale = d * (float)sc[s];
                    float w = sa[at / 32] * scale;
                    acc = fmaf((float)dot, w, acc);
                }
            }
            j->c[(int64_t)i * j->n + c] = acc;
        }
}

QO_API int qo_matmul_q6_k(int fmt_a, const uint8_t *a, const uint8_t *b, float *c, int m, int n, int k, int32_t *sums)
{
    if ((fmt_a != QO_Q8_0 && fmt_a != QO_Q4_0) || k % 256 != 0 || k <= 0) return -1;
    int blocks = k / 32;
    int8_t *qa = (int8_t *)malloc((size_t)m * k);
    float *sa = (float *)malloc((size_t)m * blocks * 4);
    unpack_rows(fmt_a, a, m, k, qa, sa);
    struct mmk_job job = { m, n, k, qa, sa, b, c, sums };
    team_for(m, 1, (int64_t)m * n * k, mm6_body, &job);
    free(qa); free(sa);
    return 0;
}

/* References.MatMul through ProductView.Reference for B^T (Program.cs:995-1019, src/Products.cs:32-47): float64
 * products made exact by fma, accumulated as a double-double. */
struct ref_job { int fmt_a, fmt_b, n, k; const float *va, *vb; double *c; };

static void ref_body(void *p, int first, int last)
{
    struct ref_job *j = (struct ref_job *)p;
    for (int i = first; i < last; i++)
        for (int c = 0; c < j->n; c++) {
            double hi = 0, lo = 0;
            for (int t = 0; t < j->k; t++) {
                double x = j->va[(int64_t)i * j->k + t], y = j->vb[(int64_t)c * j->k + t];
                double ph = x * y, pl = fma(x, y, -ph);
                double h = hi, sum = h + ph, bv = sum - h, err = (h - (sum - bv)) + (ph - bv);
                hi = sum;
                lo += err + pl;
            }
            j->c[(int64_t)i * j->n + c] = hi + lo;
        }
}

QO_API int qo_matmul_f64(int fmt_a, int fmt_b, const uint8_t *a, const uint8_t *b, double *c, int m, int n, int k)
{
    if (!qo_block_values(fmt_a) || !qo_block_values(fmt_b) || k % qo_block_values(fmt_a) || k % qo_block_values(fmt_b)) return -1;
    float *va = (float *)malloc((size_t)m * k * 4), *vb = (float *)malloc((size_t)n * k * 4);
    for (int i = 0; i < m; i++) qo_decode(fmt_a, a + (int64_t)i * qo_bytes(fmt_a, k), k, va + (int64_t)i * k);
    for (int i = 0; i < n; i++) qo_decode(fmt_b, b + (int64_t)i * qo_bytes(fmt_b, k), k, vb + (int64_t)i * k);
    struct ref_job job = { fmt_a, fmt_b, n, k, va, vb, c };
    team_for(m, 1, (int64_t)m * n * k, ref_body, &job);
    free(va); free(vb);
    return 0;
}

/* ------------------------------------------------------------------ timing for the CPU baseline */

QO_API double qo_now(void)
{
    struct timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return (double)t.tv_sec + 1e-9 * (double)t.tv_nsec;
}

/* `reps` back-to-back calls of the CPU block gemv (order 0), returning seconds per call. */
QO_API double qo_time_gemv_blocks(int fmt_a, int fmt_x, const uint8_t *a, const void *x, float *y, int rows, int cols, int reps)
{
    double t0 = qo_now();
    for (int i = 0; i < reps; i++) if (qo_gemv_blocks(fmt_a, fmt_x, a, x, y, rows, cols, 0, 0, 0)) return -1;
    return (qo_now() - t0) / (reps > 0 ? reps : 1);
}
