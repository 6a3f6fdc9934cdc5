/*
 * CPU oracle for the quantized-GEMM path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic that the reference project
 * defines for the path: the fp32 GEMM loop, the narrow-format decoders, the
 * packing rules and the tensor-parallel sharding.  It is the checker for the
 * CUDA kernels and the timed CPU baseline; nothing shipped calls it.
 *
 * Parity pins: every decoder, packing rule and known-answer value below is
 * checked against the constants held by the reference's own tests
 * (tests/test_oracle_pins.py) and the GEMM loop is compared bit-for-bit with the
 * reference's compiled gemm_mma_cpu (oracle/_ref).  The encoders, SwiGLU and the
 * W4A16 / per-channel dequantisation rules have no counterpart in the reference;
 * they follow the format definitions and are cross-checked against the CUDA
 * toolkit's host conversions (oracle/check_cuda_codecs.cu).
 *
 * Each function cites the reference file:line it follows (paths inside the
 * reference project).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ GEMM */

/* C[M,N] = A[M,K] * B[N,K]^T, strictly sequential fp32 accumulation over K.
 * Follows op/cpu/cpu_ops.cpp:95-114 (gemm_mma_cpu): same loop nest (i, j, p),
 * same single fp32 accumulator, K innermost. */
void oracle_gemm_f32(const float* A, const float* B, float* C, int M, int N, int K)
{
    for (int i = 0; i < M; ++i) {
        const float* a = A + (size_t)i * K;
        for (int j = 0; j < N; ++j) {
            const float* b = B + (size_t)j * K;
            float acc = 0.0f;
            for (int p = 0; p < K; ++p) acc += a[p] * b[p];
            C[(size_t)i * N + j] = acc;
        }
    }
}

/* Same contraction with a double accumulator: a diagnosis twin that removes the
 * fp32 summation-order noise from the comparison.  No reference counterpart. */
void oracle_gemm_f64acc(const float* A, const float* B, double* C, int M, int N, int K)
{
    for (int i = 0; i < M; ++i) {
        const float* a = A + (size_t)i * K;
        for (int j = 0; j < N; ++j) {
            const float* b = B + (size_t)j * K;
            double acc = 0.0;
            for (int p = 0; p < K; ++p) acc += (double)a[p] * (double)b[p];
            C[(size_t)i * N + j] = acc;
        }
    }
}

/* D = A*B^T + C0 in fp32 (the form the one-instruction known-answer tests use:
 * op/test/arch_primitives/ptx_mma_sparse.cu:416-434, ptx_mma_fp4.cu:311-324). */
void oracle_gemm_f32_addc(const float* A, const float* B, const float* C0, float* D,
                          int M, int N, int K)
{
    for (int i = 0; i < M; ++i)
        for (int j = 0; j < N; ++j) {
            float acc = C0[(size_t)i * N + j];
            for (int p = 0; p < K; ++p) acc += A[(size_t)i * K + p] * B[(size_t)j * K + p];
            D[(size_t)i * N + j] = acc;
        }
}

/* --------------------------------------------------------------- decoders */

/* E2M1: magnitudes {0,.5,1,1.5,2,3,4,6}, bit 3 = sign.
 * Follows op/test/arch_primitives/ptx_mma_fp4.cu:285-291. */
float oracle_decode_e2m1(uint8_t bits)
{
    static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float m = mag[bits & 7u];
    return (bits & 8u) ? -m : m;
}

/* UE4M3 block scale: bias 7, subnormals m/8 * 2^-6, 0x7F = NaN.
 * Follows op/test/arch_primitives/ptx_mma_fp4.cu:293-309. */
float oracle_decode_ue4m3(uint8_t bits)
{
    int e = (bits >> 3) & 0x0F, m = bits & 7;
    if (bits == 0x7Fu) return NAN;
    if (e == 0) return ldexpf((float)m / 8.0f, -6);
    return ldexpf(1.0f + (float)m / 8.0f, e - 7);
}

/* E4M3 (finite-only variant): sign + UE4M3 magnitude; 1.0 = 0x38
 * (op/test/arch_primitives/ptx_mma_fp8.cu:54-59). */
float oracle_decode_e4m3(uint8_t bits)
{
    float m = oracle_decode_ue4m3(bits & 0x7Fu);
    return (bits & 0x80u) ? -m : m;
}

/* UE8M0: 2^(bits-127), 0xFF = NaN (op/test/arch_primitives/ptx_mma_fp6.cu:344-351). */
float oracle_decode_ue8m0(uint8_t bits)
{
    if (bits == 0xFFu) return NAN;
    return ldexpf(1.0f, (int)bits - 127);
}

static float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

float oracle_decode_bf16(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

float oracle_decode_f16(uint16_t h)
{
    uint32_t s = (uint32_t)(h >> 15) << 31;
    int e = (h >> 10) & 0x1F, m = h & 0x3FF;
    float v;
    if (e == 0) v = ldexpf((float)m, -24);
    else if (e == 31) v = m ? NAN : INFINITY;
    else v = ldexpf(1.0f + (float)m / 1024.0f, e - 15);
    return (s ? -v : v);
}

/* --------------------------------------------------------------- encoders */
/* No reference counterpart: round-to-nearest-even, saturate-to-finite, as the
 * format definitions state; cross-checked against cuda_fp8.h / cuda_fp4.h. */

/* fp32 -> bf16, RN-even (the final output cast: the reference casts the fp32
 * accumulator with round-to-nearest-even at the very end,
 * op/test/arch_primitives/ptx_mma_fp4.cu:277-282). */
uint16_t oracle_encode_bf16(float f)
{
    uint32_t u = f32_to_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

uint16_t oracle_encode_f16(float f)
{
    uint32_t u = f32_to_bits(f);
    uint16_t s = (uint16_t)((u >> 16) & 0x8000u);
    float a = fabsf(f);
    if (isnan(f)) return (uint16_t)(s | 0x7E00u);
    if (a >= 65520.0f) return (uint16_t)(s | 0x7C00u);
    if (a < ldexpf(1.0f, -14)) {
        int q = (int)rintf(ldexpf(a, 24));
        return (uint16_t)(s | q);
    }
    int e; float m = frexpf(a, &e); /* a = m * 2^e, m in [0.5,1) */
    int q = (int)rintf((m * 2.0f - 1.0f) * 1024.0f); e -= 1;
    if (q == 1024) { q = 0; e += 1; }
    return (uint16_t)(s | ((e + 15) << 10) | q);
}

static uint8_t encode_ue4m3_mag(float a)
{
    if (isnan(a)) return 0x7F;
    if (a < ldexpf(1.0f, -6)) return (uint8_t)rintf(ldexpf(a, 9)); /* 8 -> 0x08 = 2^-6 */
    if (a > 448.0f) return 0x7E;
    int e; float m = frexpf(a, &e);
    int q = (int)rintf((m * 2.0f - 1.0f) * 8.0f); e -= 1;
    if (q == 8) { q = 0; e += 1; }
    if (e > 8 || (e == 8 && q > 6)) return 0x7E;
    return (uint8_t)(((e + 7) << 3) | q);
}

uint8_t oracle_encode_e4m3(float f)
{
    uint8_t s = (f32_to_bits(f) >> 31) ? 0x80u : 0;
    if (isnan(f)) return 0x7F;
    return (uint8_t)(s | encode_ue4m3_mag(fabsf(f)));
}

uint8_t oracle_encode_ue4m3(float f)
{
    if (isnan(f)) return 0x7F;
    if (f <= 0.0f) return 0;
    return encode_ue4m3_mag(f);
}

uint8_t oracle_encode_e2m1(float f)
{
    uint8_t s = (f32_to_bits(f) >> 31) ? 8u : 0;
    float a = fabsf(f);
    uint8_t c;
    if (isnan(f)) return 7; /* no NaN in E2M1: saturate */
    /* ties go to the even code (codes are monotone and the code LSB is the mantissa LSB) */
    if (a <= 0.25f) c = 0; else if (a < 0.75f) c = 1; else if (a <= 1.25f) c = 2;
    else if (a < 1.75f) c = 3; else if (a <= 2.5f) c = 4; else if (a < 3.5f) c = 5;
    else if (a <= 5.0f) c = 6; else c = 7;
    return (uint8_t)(s | c);
}

/* ---------------------------------------------------------------- packing */

/* Signed INT4: two's-complement nibble, element i of a word at bits [4i+3:4i], so
 * inside a byte the low nibble is the lower K index.
 * Follows op/test/arch_primitives/ptx_mma_integer.cu:93-108. */
void oracle_pack_s4(const int8_t* v, uint8_t* out, size_t n /* even */)
{
    for (size_t i = 0; i < n; i += 2)
        out[i / 2] = (uint8_t)(((uint8_t)v[i] & 0xF) | (((uint8_t)v[i + 1] & 0xF) << 4));
}
void oracle_unpack_s4(const uint8_t* in, int8_t* v, size_t n /* even */)
{
    for (size_t i = 0; i < n; i += 2) {
        v[i]     = (int8_t)((int8_t)(in[i / 2] << 4) >> 4);
        v[i + 1] = (int8_t)((int8_t)(in[i / 2] & 0xF0) >> 4);
    }
}

/* E2M1 packs the same way: 8 nibbles per 32-bit word, element i at bits [4i+3:4i]
 * (op/test/arch_primitives/ptx_mma_fp4.cu:120-130). */
void oracle_pack_u4(const uint8_t* v, uint8_t* out, size_t n)
{
    for (size_t i = 0; i < n; i += 2) out[i / 2] = (uint8_t)((v[i] & 0xF) | ((v[i + 1] & 0xF) << 4));
}
void oracle_unpack_u4(const uint8_t* in, uint8_t* v, size_t n)
{
    for (size_t i = 0; i < n; i += 2) { v[i] = in[i / 2] & 0xF; v[i + 1] = in[i / 2] >> 4; }
}

/* 2:4 structured sparsity, byte-sized elements.
 * dense[M,K] -> comp[M,K/2] keeps the two retained values of every group of four
 * in order; meta holds one nibble per group = two ascending 2-bit positions, the
 * lower position in bits [1:0]; nibbles pack LSB-first, two groups per byte.
 * Legal nibbles: 0x4 {0,1}, 0x8 {0,2}, 0x9 {1,2}, 0xC {0,3}, 0xD {1,3}, 0xE {2,3}.
 * Follows op/test/arch_primitives/ptx_mma_sparse.cu:53-64 (encoding) and
 * :163-184 (compressed layout).  A group with fewer than two non-zeros keeps the
 * lowest free positions so the pair stays ascending.  Returns 0, or -1 if a group
 * holds more than two non-zeros (the validator at :206-244 rejects those). */
int oracle_sp24_compress_u8(const uint8_t* dense, uint8_t* comp, uint8_t* meta, int M, int K)
{
    for (int i = 0; i < M; ++i)
        for (int g = 0; g < K / 4; ++g) {
            const uint8_t* d = dense + (size_t)i * K + 4 * g;
            int pos[2], n = 0;
            for (int t = 0; t < 4; ++t)
                if ((d[t] & 0x7F) != 0) { if (n == 2) return -1; pos[n++] = t; }
            /* pad with unused positions, keeping ascending order */
            if (n == 0) { pos[0] = 0; pos[1] = 1; }
            else if (n == 1) {
                if (pos[0] == 3) { pos[1] = 3; pos[0] = 2; }
                else pos[1] = pos[0] + 1;
            }
            comp[(size_t)i * (K / 2) + 2 * g]     = d[pos[0]];
            comp[(size_t)i * (K / 2) + 2 * g + 1] = d[pos[1]];
            uint8_t nib = (uint8_t)(pos[0] | (pos[1] << 2));
            size_t mi = (size_t)i * (K / 8) + g / 2;
            if (g & 1) meta[mi] = (uint8_t)((meta[mi] & 0x0F) | (nib << 4));
            else       meta[mi] = (uint8_t)((meta[mi] & 0xF0) | nib);
        }
    return 0;
}

/* Inverse: the dense matrix the reference multiplies as ground truth
 * (op/test/arch_primitives/ptx_mma_sparse.cu:416-434 uses dense_a). */
int oracle_sp24_expand_u8(const uint8_t* comp, const uint8_t* meta, uint8_t* dense, int M, int K)
{
    for (int i = 0; i < M; ++i)
        for (int g = 0; g < K / 4; ++g) {
            uint8_t b = meta[(size_t)i * (K / 8) + g / 2];
            uint8_t nib = (g & 1) ? (b >> 4) : (b & 0xF);
            int p0 = nib & 3, p1 = nib >> 2;
            if (p0 >= p1) return -1;
            uint8_t* d = dense + (size_t)i * K + 4 * g;
            d[0] = d[1] = d[2] = d[3] = 0;
            d[p0] = comp[(size_t)i * (K / 2) + 2 * g];
            d[p1] = comp[(size_t)i * (K / 2) + 2 * g + 1];
        }
    return 0;
}

/* ------------------------------------------------- bulk convert / quantise */

void oracle_decode_e4m3_n(const uint8_t* in, float* out, size_t n, float scale)
{
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = oracle_decode_e4m3((uint8_t)i);
    for (size_t i = 0; i < n; ++i) out[i] = lut[in[i]] * scale;
}
void oracle_encode_e4m3_n(const float* in, uint8_t* out, size_t n, float inv_scale_is_div /*scale*/)
{
    /* q = e4m3_rn(x / scale): a true division, as the kernels do */
    for (size_t i = 0; i < n; ++i) out[i] = oracle_encode_e4m3(in[i] / inv_scale_is_div);
}
void oracle_decode_bf16_n(const uint16_t* in, float* out, size_t n)
{
    for (size_t i = 0; i < n; ++i) out[i] = oracle_decode_bf16(in[i]);
}
void oracle_encode_bf16_n(const float* in, uint16_t* out, size_t n)
{
    for (size_t i = 0; i < n; ++i) out[i] = oracle_encode_bf16(in[i]);
}
void oracle_decode_f16_n(const uint16_t* in, float* out, size_t n)
{
    for (size_t i = 0; i < n; ++i) out[i] = oracle_decode_f16(in[i]);
}
void oracle_encode_f16_n(const float* in, uint16_t* out, size_t n)
{
    for (size_t i = 0; i < n; ++i) out[i] = oracle_encode_f16(in[i]);
}

/* Per-row (per-token) E4M3 quantisation: s[r] = max(max|x[r,:]| / 448, 2^-126) (1.0 for
 * an all-zero row; the floor keeps 1 / s finite for rows of subnormal magnitudes, which
 * would otherwise turn their zeros into NaN), q = e4m3_rn(x * (1 / s[r])): one fp32 reciprocal per row, one fp32
 * product per element (both round-to-nearest), then the E4M3 rounding.  No reference
 * counterpart; the rule is stated here and the kernel reproduces it bit for bit. */
void oracle_quant_rows_e4m3(const float* x, uint8_t* q, float* s, int rows, int cols)
{
    for (int r = 0; r < rows; ++r) {
        const float* xr = x + (size_t)r * cols;
        float mx = 0.0f;
        for (int c = 0; c < cols; ++c) mx = fmaxf(mx, fabsf(xr[c]));
        float sc = mx > 0.0f ? fmaxf(mx / 448.0f, 1.17549435e-38f) : 1.0f;
        volatile float inv = 1.0f / sc;       /* volatile: keep the two roundings separate */
        s[r] = sc;
        for (int c = 0; c < cols; ++c) {
            volatile float y = xr[c] * inv;
            q[(size_t)r * cols + c] = oracle_encode_e4m3(y);
        }
    }
}

/* NVFP4 quantisation of x[rows, cols] with a given global scale g:
 * per 16 contiguous K: sf = ue4m3_rn((max|blk| / 6) / g), d = sf_decoded * g, q = e2m1_rn(x * (1 / d)) — one fp32
 * reciprocal per block and one fp32 product per element, each rounded to nearest, then the E2M1 rounding (ties to
 * the even code); a block whose d is below the smallest normal float (all zeros, or a vanishing g) is all zeros.
 * Two E2M1 per byte, low nibble first; sf laid out row-major [rows, cols/16].
 * Scale rule: one UE4M3 per 16 consecutive K (op/test/arch_primitives/ptx_mma_fp4.cu:55-65); the reference has no
 * quantiser, the rule is stated here and the GPU quantiser reproduces it bit for bit. */
void oracle_quant_nvfp4(const float* x, uint8_t* q, uint8_t* sf, int rows, int cols, float g)
{
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < cols / 16; ++b) {
            const float* xb = x + (size_t)r * cols + 16 * b;
            float mx = 0.0f;
            for (int t = 0; t < 16; ++t) mx = fmaxf(mx, fabsf(xb[t]));
            volatile float t6 = mx / 6.0f;
            volatile float tg = t6 / g;
            uint8_t s8 = oracle_encode_ue4m3(tg);
            sf[(size_t)r * (cols / 16) + b] = s8;
            volatile float d = oracle_decode_ue4m3(s8) * g;
            const int live = d >= 1.17549435e-38f;
            volatile float inv = live ? 1.0f / d : 0.0f;
            uint8_t nib[16];
            for (int t = 0; t < 16; ++t) {
                volatile float y = xb[t] * inv;
                nib[t] = live ? oracle_encode_e2m1(y) : 0;
            }
            oracle_pack_u4(nib, q + ((size_t)r * cols + 16 * b) / 2, 16);
        }
}

/* NVFP4 -> fp32: value = e2m1 * ue4m3(block) * g. */
void oracle_dequant_nvfp4(const uint8_t* q, const uint8_t* sf, float* out, int rows, int cols, float g)
{
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c) {
            uint8_t b = q[((size_t)r * cols + c) / 2];
            uint8_t nib = (c & 1) ? (b >> 4) : (b & 0xF);
            float s = oracle_decode_ue4m3(sf[(size_t)r * (cols / 16) + c / 16]);
            out[(size_t)r * cols + c] = oracle_decode_e2m1(nib) * s * g;
        }
}

/* MXFP8 quantisation of x[rows, cols]: per 32 contiguous K one UE8M0 scale 2^(e - 127) with
 * e - 127 = floor(log2(max|blk|)) - 8 (8 = exponent of the largest E4M3 binade, so the block maximum lands
 * in [256, 512) and saturates to 448 at most), q = e4m3_rn_satfinite(x / scale); an all-zero block gets scale
 * byte 127 (1.0).  The format (E4M3 data, one UE8M0 per 32 K) is that of the reference's
 * kind::mxf8f6f4.block_scale.scale_vec::1X test (op/test/arch_primitives/ptx_mma_fp8.cu:126-178); the rule for
 * choosing the exponent is the usual microscaling one, the reference has none. */
void oracle_quant_mxfp8(const float* x, uint8_t* q, uint8_t* sf, int rows, int cols)
{
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < cols / 32; ++b) {
            const float* xb = x + (size_t)r * cols + 32 * b;
            float mx = 0.0f;
            for (int t = 0; t < 32; ++t) mx = fmaxf(mx, fabsf(xb[t]));
            int e = 127;
            if (mx > 0.0f) {
                int ex; frexpf(mx, &ex);                 /* mx = f * 2^ex, f in [0.5, 1): floor(log2 mx) = ex - 1 */
                e = (ex - 1) - 8 + 127;
                if (e < 0) e = 0;
                if (e > 254) e = 254;
            }
            sf[(size_t)r * (cols / 32) + b] = (uint8_t)e;
            const float inv = ldexpf(1.0f, 127 - e);     /* exact power of two */
            for (int t = 0; t < 32; ++t) q[(size_t)r * cols + 32 * b + t] = oracle_encode_e4m3(xb[t] * inv);
        }
}

/* MXFP8 -> fp32: value = e4m3 * 2^(sf - 127), one scale per 32 K
 * (decoder: op/test/arch_primitives/ptx_mma_fp6.cu:344-351). */
void oracle_dequant_mxfp8(const uint8_t* q, const uint8_t* sf, float* out, int rows, int cols)
{
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c)
            out[(size_t)r * cols + c] = oracle_decode_e4m3(q[(size_t)r * cols + c]) * oracle_decode_ue8m0(sf[(size_t)r * (cols / 32) + c / 32]);
}

/* W4A16 weights -> fp32: w[n,k] = q[n,k] * fp16 scale[n, k/group]; no zero point. */
void oracle_dequant_w4(const uint8_t* wq, const uint16_t* s, float* out, int N, int K, int group)
{
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k) {
            uint8_t b = wq[((size_t)n * K + k) / 2];
            int v = (k & 1) ? ((int8_t)(b & 0xF0) >> 4) : ((int8_t)(b << 4) >> 4);
            out[(size_t)n * K + k] = (float)v * oracle_decode_f16(s[(size_t)n * (K / group) + k / group]);
        }
}

/* SwiGLU, fp32: h = silu(g) * u = g / (1 + exp(-g)) * u.  No reference counterpart
 * (the reference MLP uses an exact-erf GELU, op/nccl/nccl_mlp_test.cu:92-103). */
void oracle_swiglu(const float* g, const float* u, float* h, size_t n)
{
    for (size_t i = 0; i < n; ++i) h[i] = g[i] / (1.0f + expf(-g[i])) * u[i];
}

/* C[m,n] *= row_scale[m] * col_scale[n] (either may be NULL). */
void oracle_scale_rows_cols(float* C, const float* rs, const float* cs, int M, int N)
{
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            float v = C[(size_t)m * N + n];
            if (rs && cs) v = v * (rs[m] * cs[n]);
            else if (rs) v *= rs[m];
            else if (cs) v *= cs[n];
            C[(size_t)m * N + n] = v;
        }
}

/* ------------------------------------------------------- tensor parallel */

/* Column-parallel shard of a weight stored [in, out] row-major: rank r keeps
 * output columns [r*out/R, (r+1)*out/R).  Follows op/nccl/nccl_mlp_test.cu:321-340. */
void oracle_shard_cols(const uint8_t* w, uint8_t* shard, size_t rows, size_t cols,
                       size_t elt, int rank, int world)
{
    size_t local = cols / world;
    for (size_t r = 0; r < rows; ++r)
        memcpy(shard + r * local * elt, w + (r * cols + (size_t)rank * local) * elt, local * elt);
}
/* Row-parallel shard: a contiguous slab of rows.  Follows op/nccl/nccl_mlp_test.cu:342-352. */
void oracle_shard_rows(const uint8_t* w, uint8_t* shard, size_t rows, size_t cols,
                       size_t elt, int rank, int world)
{
    size_t local = rows / world;
    memcpy(shard, w + (size_t)rank * local * cols * elt, local * cols * elt);
}

/* max-abs / max-rel error, denominator floored at 1e-6.
 * Follows op/nccl/nccl_mlp_test.cu:444-458. */
void oracle_compare(const float* actual, const float* expected, size_t n, float* max_abs, float* max_rel)
{
    float ma = 0.0f, mr = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float a = fabsf(actual[i] - expected[i]);
        float d = fmaxf(fabsf(expected[i]), 1.0e-6f);
        ma = fmaxf(ma, a); mr = fmaxf(mr, a / d);
    }
    *max_abs = ma; *max_rel = mr;
}
