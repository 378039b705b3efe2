/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement (plain C) of the reference project's repack of
 * GGUF quantized tensors into its affine layout:
 *   qref_gguf_repack   extract_q4_0_data / extract_q4_1_data / extract_q8_0_data and
 *                      unpack_32_4          mlx/io/gguf_quants.cpp:11-102
 *
 * Parity status: the nibble order of the 4-bit blocks is PINNED to the reference's own
 * unpack_32_4, compiled from the reference checkout with the third-party gguflib header replaced
 * by declarations (oracle/ref_gguf_driver.cpp, oracle/stub/gguflib.h): golden vectors in
 * tests/golden/gguf_unpack_golden.npz plus a live comparison where the binary exists.  The loops
 * around it (scale / bias in float16, sign flip of Q8_0) take the reference's array objects, whose
 * runtime cannot be linked here; they are restated and checked against the format definition
 * (value = d * (q - 8) for Q4_0, d * q + m for Q4_1, d * q for Q8_0), which fixes them up to the
 * float16 rounding of the bias (exact for Q4_0 and Q8_0: -8 d and -128 d are exact).
 *
 * Block layouts (32 weights per block):
 *   Q4_0  | f16 d | 16 bytes: byte j = weight j (low nibble), weight j + 16 (high nibble) |   18 B
 *   Q4_1  | f16 d | f16 m | 16 bytes as Q4_0 |                                               20 B
 *   Q8_0  | f16 d | 32 x int8 |                                                              34 B
 * Output: 4-bit (Q4_*) or 8-bit (Q8_0) fields in the affine layout (group size 32, LSB-first),
 * scales = d, biases = -8 d (Q4_0), m (Q4_1), -128 d (Q8_0, fields stored with the sign bit
 * flipped), all float16 with the reference's float16 arithmetic (product rounded to nearest even).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static float h2f(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FF, u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400));
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7F800000u | (man << 13);
  } else {
    u = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static uint16_t f2h(float f) {  /* round to nearest even */
  uint32_t u;
  memcpy(&u, &f, 4);
  const uint16_t sign = (uint16_t)((u >> 16) & 0x8000);
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a >= 0x7F800000u) return (uint16_t)(sign | 0x7C00 | ((a > 0x7F800000u) ? 0x200 : 0));
  if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00);               /* overflows to inf */
  if (a < 0x33000001u) return sign;                                      /* rounds to zero */
  int exp = (int)(a >> 23) - 127 + 15;
  uint32_t man = (a & 0x7FFFFFu) | 0x800000u;
  int shift = 13;
  if (exp <= 0) { shift += 1 - exp; exp = 0; }
  uint32_t half = man >> shift;
  const uint32_t rem = man & ((1u << shift) - 1u), mid = 1u << (shift - 1);
  if (rem > mid || (rem == mid && (half & 1))) ++half;
  if (exp == 0) return (uint16_t)(sign | half);                          /* subnormal (may carry into exp 1) */
  half &= 0x7FFFFFFFu;
  uint32_t out = ((uint32_t)exp << 10) + (half - 0x400u);                /* carry propagates into the exponent */
  return (uint16_t)(sign | out);
}

/* type: 2 = Q4_0, 3 = Q4_1, 8 = Q8_0 (the GGUF type ids).  Returns 0, or -1 for another type. */
int qref_gguf_repack(const uint8_t* blocks, int type, size_t n_blocks, uint8_t* wq, uint16_t* scales, uint16_t* biases) {
  for (size_t i = 0; i < n_blocks; ++i) {
    if (type == 2 || type == 3) {
      const size_t bytes = type == 2 ? 18 : 20;
      const uint8_t* blk = blocks + i * bytes;
      uint16_t d;
      memcpy(&d, blk, 2);
      scales[i] = d;
      const uint8_t* q;
      if (type == 2) {
        biases[i] = f2h(-8.0f * h2f(d));
        q = blk + 2;
      } else {
        memcpy(&biases[i], blk + 2, 2);
        q = blk + 4;
      }
      uint8_t* dst = wq + i * 16;
      memset(dst, 0, 16);
      for (int j = 0; j < 16; ++j) {          /* first 16 weights: low nibbles */
        uint8_t x = q[j] & 0x0F;
        if (j % 2) x <<= 4;
        dst[j / 2] += x;
      }
      for (int j = 0; j < 16; ++j) {          /* last 16 weights: high nibbles */
        uint8_t x = q[j] >> 4;
        if (j % 2) x <<= 4;
        dst[8 + j / 2] += x;
      }
    } else if (type == 8) {
      const uint8_t* blk = blocks + i * 34;
      uint16_t d;
      memcpy(&d, blk, 2);
      scales[i] = d;
      biases[i] = f2h(-128.0f * h2f(d));
      for (int j = 0; j < 32; ++j) wq[i * 32 + j] = blk[2 + j] ^ 0x80;
    } else {
      return -1;
    }
  }
  return 0;
}
