// Host-only cross-check (test infrastructure): the oracle's fp32 -> E4M3 / E2M1 /
// bf16 / fp16 encoders against the CUDA toolkit's own host conversions, over a
// dense sweep of float bit patterns.  Prints the mismatch count; exit 0 iff zero.
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <cmath>
extern "C" {
uint8_t oracle_encode_e4m3(float); uint8_t oracle_encode_e2m1(float);
uint16_t oracle_encode_bf16(float); uint16_t oracle_encode_f16(float);
float oracle_decode_e4m3(uint8_t); float oracle_decode_e2m1(uint8_t);
}
int main()
{
    long bad = 0, n = 0;
    // every 2^9-th float bit pattern in the finite range, plus exact ties
    for (uint64_t u = 0; u < 0x100000000ull; u += 509) {
        uint32_t b = (uint32_t)u; float f; memcpy(&f, &b, 4);
        if (std::isnan(f) || std::isinf(f)) continue;
        ++n;
        uint8_t a8 = oracle_encode_e4m3(f);
        uint8_t c8 = (uint8_t)__nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E4M3);
        if (a8 != c8 && !((a8 & 0x7F) == 0 && (c8 & 0x7F) == 0)) { if (bad < 10) printf("e4m3 %a: %02x vs %02x\n", f, a8, c8); ++bad; }
        uint8_t a4 = oracle_encode_e2m1(f);
        uint8_t c4 = (uint8_t)__nv_cvt_float_to_fp4(f, __NV_E2M1, cudaRoundNearest) & 0xF;
        if (a4 != c4 && !((a4 & 7) == 0 && (c4 & 7) == 0)) { if (bad < 10) printf("e2m1 %a: %x vs %x\n", f, a4, c4); ++bad; }
        __nv_bfloat16 hb = __float2bfloat16_rn(f); uint16_t cb; memcpy(&cb, &hb, 2);
        if (oracle_encode_bf16(f) != cb) { if (bad < 10) printf("bf16 %a\n", f); ++bad; }
        __half hh = __float2half_rn(f); uint16_t ch; memcpy(&ch, &hh, 2);
        if (oracle_encode_f16(f) != ch) { if (bad < 10) printf("f16 %a: %04x vs %04x\n", f, oracle_encode_f16(f), ch); ++bad; }
    }
    // exact representable values and midpoints of both small formats
    for (int i = 0; i < 256; ++i) for (int j = 0; j < 256; ++j) {
        float x = oracle_decode_e4m3((uint8_t)i), y = oracle_decode_e4m3((uint8_t)j);
        if (std::isnan(x) || std::isnan(y)) continue;
        float f = 0.5f * (x + y); ++n;
        uint8_t a8 = oracle_encode_e4m3(f);
        uint8_t c8 = (uint8_t)__nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E4M3);
        if (a8 != c8 && !((a8 & 0x7F) == 0 && (c8 & 0x7F) == 0)) { if (bad < 10) printf("e4m3 mid %a: %02x vs %02x\n", f, a8, c8); ++bad; }
    }
    for (int i = 0; i < 16; ++i) for (int j = 0; j < 16; ++j) {
        float f = 0.5f * (oracle_decode_e2m1((uint8_t)i) + oracle_decode_e2m1((uint8_t)j)); ++n;
        uint8_t a4 = oracle_encode_e2m1(f);
        uint8_t c4 = (uint8_t)__nv_cvt_float_to_fp4(f, __NV_E2M1, cudaRoundNearest) & 0xF;
        if (a4 != c4 && !((a4 & 7) == 0 && (c4 & 7) == 0)) { if (bad < 10) printf("e2m1 mid %a: %x vs %x\n", f, a4, c4); ++bad; }
    }
    printf("checked %ld values, %ld mismatches\n", n, bad);
    return bad ? 1 : 0;
}
