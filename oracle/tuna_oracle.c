/*
 * CPU oracle (plain C) for the FP16 x 4-bit(codebook) GEMM path of
 * TryForefront/tuna.  TEST INFRASTRUCTURE ONLY: an independent second
 * restatement beside oracle/tuna_oracle.py, used by the tests, the smoke check
 * and the benchmark's CPU-baseline leg.  The shipped library never links it.
 *
 * Parity status: the reference has no golden vectors of its own; this file is
 * pinned against fixtures produced by the reference's CUDA kernels on a B200
 * (tests/golden/) and against the numpy restatement.
 *
 * Names follow the reference: m = output features, n = tokens, k = reduction.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>

typedef _Float16 f16;

static inline uint16_t f32_to_f16_bits(float v)
{
    f16 h = (f16)v; /* round-to-nearest-even, as the device's (half) cast */
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}

static inline float f16_bits_to_f32(uint16_t b)
{
    f16 h;
    memcpy(&h, &b, 2);
    return (float)h;
}

/* Offset of the byte that holds W[r][c] in the packed tensor [m/8][k/8][32]
 * (test.py:58-65; strides 4k / 32 / 1 as in kernel.cu:3171). *hi is set when
 * the code sits in the high nibble (even column of the pair). */
static inline size_t packed_offset(int r, int c, int k, int *hi)
{
    int mt = r >> 3, kt = c >> 3, rr = r & 7, cc = c & 7;
    *hi = (cc & 1) == 0;
    return (size_t)mt * 4 * (size_t)k + (size_t)kt * 32 + (size_t)(rr * 4 + (cc >> 1));
}

void oracle_pack(const uint8_t *codes, uint8_t *q, int m, int k)
{
    memset(q, 0, (size_t)m * k / 2);
    for (int r = 0; r < m; ++r)
        for (int c = 0; c < k; ++c) {
            int hi;
            size_t off = packed_offset(r, c, k, &hi);
            uint8_t v = codes[(size_t)r * k + c] & 15;
            q[off] |= hi ? (uint8_t)(v << 4) : v;
        }
}

void oracle_unpack(const uint8_t *q, uint8_t *codes, int m, int k)
{
    for (int r = 0; r < m; ++r)
        for (int c = 0; c < k; ++c) {
            int hi;
            size_t off = packed_offset(r, c, k, &hi);
            codes[(size_t)r * k + c] = hi ? (q[off] >> 4) : (q[off] & 15);
        }
}

/* The dequant op, kernel.cu:3218-3229: fp32(code) * fp32(absmax) -> fp16 RN.
 * out is [m][k] fp16 bit patterns.  Parallel over 8-row groups. */
void oracle_dequant(const uint8_t *q, const float *absmax, const float *code,
                    uint16_t *out, int m, int k)
{
#pragma omp parallel for schedule(static)
    for (int mt = 0; mt < m / 8; ++mt) {
        uint16_t lut[8][16];
        for (int rr = 0; rr < 8; ++rr)
            for (int j = 0; j < 16; ++j)
                lut[rr][j] = f32_to_f16_bits(code[j] * absmax[mt * 8 + rr]);
        const uint8_t *tile = q + (size_t)mt * 4 * (size_t)k;
        for (int kt = 0; kt < k / 8; ++kt, tile += 32)
            for (int j = 0; j < 32; ++j) {
                int rr = j >> 2, cc = (j & 3) * 2;
                uint16_t *dst = out + (size_t)(mt * 8 + rr) * k + kt * 8 + cc;
                dst[0] = lut[rr][tile[j] >> 4];
                dst[1] = lut[rr][tile[j] & 15];
            }
    }
}

/* The matmul op restated as dequantize-then-matmul: fp16 operands, fp32
 * accumulation in ascending k (kernel.cu:54-55 fixes fp32 accumulators), one
 * fp16 rounding at the end (kernel.cu:2719).  o is [n][m]. */
void oracle_matmul(const uint16_t *x, const uint8_t *q, const float *code,
                   const float *absmax, uint16_t *o, int m, int n, int k)
{
#pragma omp parallel for schedule(static)
    for (int mt = 0; mt < m / 8; ++mt) {
        for (int rr = 0; rr < 8; ++rr) {
            int r = mt * 8 + rr;
            float lut[16];
            for (int j = 0; j < 16; ++j)
                lut[j] = f16_bits_to_f32(f32_to_f16_bits(code[j] * absmax[r]));
            for (int t = 0; t < n; ++t) {
                const uint16_t *xr = x + (size_t)t * k;
                float acc = 0.f;
                const uint8_t *tile = q + (size_t)mt * 4 * (size_t)k + rr * 4;
                for (int kt = 0; kt < k / 8; ++kt, tile += 32)
                    for (int b = 0; b < 4; ++b) {
                        acc += f16_bits_to_f32(xr[kt * 8 + 2 * b]) * lut[tile[b] >> 4];
                        acc += f16_bits_to_f32(xr[kt * 8 + 2 * b + 1]) * lut[tile[b] & 15];
                    }
                o[(size_t)t * m + r] = f32_to_f16_bits(acc);
            }
        }
    }
}

int oracle_abi_version(void) { return 1; }
