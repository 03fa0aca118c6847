/*
 * CPU oracle (TEST INFRASTRUCTURE ONLY - never linked or called by the product
 * path) for the serialization stage of Point Transformer V3.
 *
 * Plain-C restatement of the reference algorithm; every function names the
 * reference lines it follows.  The restatement is pinned by tests that compare
 * it with the reference package imported directly (when it is present) and with
 * committed golden vectors generated from that import.
 *
 *   serialization/default.py:8-24    encode(): order dispatch, x/y swap for the
 *                                    "-trans" orders, batch << 3*depth | code
 *   serialization/z_order.py:40-50   bit placement of the Morton key
 *   serialization/z_order.py:87-95   only the low `depth` bits of a coordinate
 *                                    take part (LUT masks)
 *   serialization/hilbert.py:143-196 Skilling transform on the low `depth`
 *                                    bits, dim 0 most significant in the
 *                                    interleave, Gray decode by prefix XOR
 *   model.py:118-126                 argsort of every code row + inverse
 *                                    permutation by scatter
 *   serialization/default.py:27-38   decode(): batch = code >> 3*depth, curve
 *                                    inverse of the low bits
 *   serialization/z_order.py:52-60   inverse Morton bit placement
 *   serialization/hilbert.py:201-303 binary -> Gray, de-interleave, the
 *                                    transform undone from the lowest level up
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { ORDER_Z = 0, ORDER_Z_TRANS = 1, ORDER_HILBERT = 2, ORDER_HILBERT_TRANS = 3 };

/* z_order.py:40-50 : x -> bit 3i+2, y -> bit 3i+1, z -> bit 3i. */
static uint64_t interleave3(uint64_t a, uint64_t b, uint64_t c, int depth)
{
    uint64_t key = 0;
    for (int i = 0; i < depth; ++i) {
        key |= ((a >> i) & 1ull) << (3 * i + 2);
        key |= ((b >> i) & 1ull) << (3 * i + 1);
        key |= ((c >> i) & 1ull) << (3 * i + 0);
    }
    return key;
}

/* hilbert.py:156-196, written on integers instead of a bit tensor. */
static uint64_t hilbert3(uint64_t x0, uint64_t x1, uint64_t x2, int depth)
{
    uint64_t X[3] = { x0, x1, x2 };
    for (int bit = 0; bit < depth; ++bit) {           /* hilbert.py:156 */
        uint64_t Q = 1ull << (depth - 1 - bit);
        uint64_t P = Q - 1;                            /* the bits below Q */
        for (int dim = 0; dim < 3; ++dim) {            /* hilbert.py:158 */
            if (X[dim] & Q) {
                X[0] ^= P;                             /* hilbert.py:163-165 */
            } else {
                uint64_t t = (X[0] ^ X[dim]) & P;      /* hilbert.py:168-175 */
                X[0] ^= t;
                X[dim] ^= t;
            }
        }
    }
    uint64_t g = interleave3(X[0], X[1], X[2], depth); /* hilbert.py:178 */
    /* hilbert.py:84-88 : Gray -> binary, prefix XOR from the top bit. */
    for (int s = 1; s < 64; s <<= 1) g ^= g >> s;
    return g;
}

/*
 * grid: n x 3 int32 row-major.  batch: n int64 or NULL.  out: n int64.
 * Returns 0, or -1 on a bad argument.
 */
int oracle_encode(const int32_t *grid, const int64_t *batch, int64_t n,
                  int depth, int order, int64_t *out)
{
    if (depth < 1 || depth > 21 || order < 0 || order > 3) return -1;
    const uint64_t mask = (1ull << depth) - 1;
    for (int64_t i = 0; i < n; ++i) {
        /* two's-complement low bits, as `.long() & mask` / the bit unpacking do */
        uint64_t a = (uint64_t)(int64_t)grid[3 * i + 0] & mask;
        uint64_t b = (uint64_t)(int64_t)grid[3 * i + 1] & mask;
        uint64_t c = (uint64_t)(int64_t)grid[3 * i + 2] & mask;
        if (order == ORDER_Z_TRANS || order == ORDER_HILBERT_TRANS) {
            uint64_t t = a; a = b; b = t;              /* default.py:14,18 */
        }
        uint64_t code = (order == ORDER_Z || order == ORDER_Z_TRANS)
                            ? interleave3(a, b, c, depth)
                            : hilbert3(a, b, c, depth);
        if (batch) code |= (uint64_t)batch[i] << (3 * depth); /* default.py:21-23 */
        out[i] = (int64_t)code;
    }
    return 0;
}

/* Stable argsort (ties keep the original index order) by bottom-up merge sort. */
int oracle_argsort_stable(const int64_t *code, int64_t n, int64_t *order)
{
    if (n == 0) return 0;
    int64_t *tmp = (int64_t *)malloc((size_t)n * sizeof(int64_t));
    if (!tmp) return -2;
    for (int64_t i = 0; i < n; ++i) order[i] = i;
    int64_t *src = order, *dst = tmp;
    for (int64_t w = 1; w < n; w <<= 1) {
        for (int64_t lo = 0; lo < n; lo += 2 * w) {
            int64_t mid = lo + w < n ? lo + w : n;
            int64_t hi = lo + 2 * w < n ? lo + 2 * w : n;
            int64_t i = lo, j = mid, k = lo;
            while (i < mid && j < hi)
                dst[k++] = (code[src[j]] < code[src[i]]) ? src[j++] : src[i++];
            while (i < mid) dst[k++] = src[i++];
            while (j < hi) dst[k++] = src[j++];
        }
        int64_t *t = src; src = dst; dst = t;
    }
    if (src != order) memcpy(order, src, (size_t)n * sizeof(int64_t));
    free(tmp);
    return 0;
}

/* model.py:120-126 : inverse[order[j]] = j. */
int oracle_inverse(const int64_t *order, int64_t n, int64_t *inverse)
{
    for (int64_t j = 0; j < n; ++j) {
        if (order[j] < 0 || order[j] >= n) return -1;
        inverse[order[j]] = j;
    }
    return 0;
}

/*
 * Inverse of oracle_encode for order 0 ("z") and 2 ("hilbert"), default.py:27-38.
 * grid: n x 3 int64, batch: n int64 (may be NULL).
 */
int oracle_decode(const int64_t *code, int64_t n, int depth, int order, int64_t *grid, int64_t *batch)
{
    if (depth < 1 || depth > 21 || (order != ORDER_Z && order != ORDER_HILBERT)) return -1;
    const uint64_t mask = (depth * 3 >= 64) ? ~0ull : ((1ull << (3 * depth)) - 1);
    for (int64_t i = 0; i < n; ++i) {
        uint64_t c = (uint64_t)code[i];
        if (batch) batch[i] = (int64_t)(c >> (3 * depth));         /* default.py:30 */
        c &= mask;                                                  /* default.py:31 */
        if (order == ORDER_HILBERT) c ^= c >> 1;                    /* hilbert.py:46-66 binary2gray */
        uint64_t X[3] = { 0, 0, 0 };
        for (int b = 0; b < depth; ++b) {                           /* z_order.py:52-60 */
            X[0] |= ((c >> (3 * b + 2)) & 1ull) << b;
            X[1] |= ((c >> (3 * b + 1)) & 1ull) << b;
            X[2] |= ((c >> (3 * b + 0)) & 1ull) << b;
        }
        if (order == ORDER_HILBERT) {
            for (int bit = depth - 1; bit >= 0; --bit) {            /* hilbert.py:262 */
                uint64_t Q = 1ull << (depth - 1 - bit);
                uint64_t P = Q - 1;
                for (int dim = 2; dim >= 0; --dim) {                /* hilbert.py:264 */
                    if (X[dim] & Q) {
                        X[0] ^= P;
                    } else {
                        uint64_t t = (X[0] ^ X[dim]) & P;
                        X[0] ^= t;
                        X[dim] ^= t;
                    }
                }
            }
        }
        grid[3 * i + 0] = (int64_t)X[0];
        grid[3 * i + 1] = (int64_t)X[1];
        grid[3 * i + 2] = (int64_t)X[2];
    }
    return 0;
}
