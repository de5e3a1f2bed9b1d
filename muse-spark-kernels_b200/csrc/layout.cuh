// Packed NVFP4 tile layout and the in-register decode that goes with it.
//
// One tile = 128 weight rows x 256 K (one K stage):
//   bytes [0, 16384)      codes: 16-byte chunk c (0..7) of row r at (c*128 + r)*16; a chunk
//                         holds K [32c, 32c+32) of the stage as four 32-bit words, word i =
//                         eight codes k = 32c + 8i + (0..7), bit-permuted (below);
//   bytes [16384, 18432)  scales: row r's sixteen E4M3 bytes at 16384 + r*16, byte j = block j.
// Thread r of a 128-thread group owns row r, so every 16-byte shared-memory read of a
// quarter-warp is 128 contiguous bytes.
//
// Bit permutation of one word (eight 4-bit codes c0..c7, code bits b0=m, b1=e0, b2=e1, b3=s):
// output register j (codes 2j, 2j+1) must end as BF16x2 bit patterns
//     lo half: s->15, e1->8, e0->7, m->6      hi half: the same +16,
// i.e. e2m1 * 2^-126 (BF16 subnormal trick; the meaning of the code bits is the one of
// muse_moe_w4a16/cuda/moe.cu:293-310). The stored word places those eight bits so that
//     r0 =  q            & 0x81C081C0
//     r1 =  rotl(q, 6)   & 0x81C081C0
//     r2 =  rotl(q, 12)  & 0x81C081C0
//     r3 = (rotl(q, 2)   & 0x00400040) | (rotl(q, 10) & 0x81808180)
// (rotation set found by exhaustive search over rotation pairs; 8 integer ops per 8 codes).
// Each register is then multiplied (mul.bf16x2, exact) by the block scale as BF16
// e4m3 * 2^64, giving e2m1*e4m3 * 2^-62; the epilogue multiplies the FP32 accumulator by
// gs * 2^62 (global scale on the accumulator, as muse_moe_w4a16/cuda/moe.cu:771-773).
#pragma once
#include <cstdint>
#include <cuda_bf16.h>

namespace msk {

constexpr int KS = 256;                                   // K elements per stage
constexpr int TILE_ROWS = 128;                            // weight rows per tile (= MMA M)
constexpr int TILE_CODE_BYTES = TILE_ROWS * KS / 2;       // 16384
constexpr int TILE_SF_BYTES = TILE_ROWS * KS / 16;        // 2048
constexpr int TILE_BYTES = TILE_CODE_BYTES + TILE_SF_BYTES;  // 18432
constexpr float TWO_POW_62 = 4611686018427387904.0f;

// Source bit of the stored word for (output register j, half h, code bit b).
__host__ __device__ constexpr int stored_bit(int j, int h, int b) {
  const int o = (b == 0 ? 6 : b == 1 ? 7 : b == 2 ? 8 : 15) + 16 * h;
  const int rot = j == 0 ? 0 : j == 1 ? 6 : j == 2 ? 12 : (b == 0 ? 2 : 10);
  return (o - rot + 32) & 31;
}

// Eight natural-order codes (code c in bits [4c, 4c+4)) -> stored word.
__host__ __device__ inline uint32_t pack_word(uint32_t nat) {
  uint32_t q = 0;
  for (int c = 0; c < 8; ++c) {
    const uint32_t code = (nat >> (4 * c)) & 0xFu;
    for (int b = 0; b < 4; ++b) q |= ((code >> b) & 1u) << stored_bit(c >> 1, c & 1, b);
  }
  return q;
}
__host__ __device__ inline uint32_t unpack_word(uint32_t q) {
  uint32_t nat = 0;
  for (int c = 0; c < 8; ++c)
    for (int b = 0; b < 4; ++b) nat |= ((q >> stored_bit(c >> 1, c & 1, b)) & 1u) << (4 * c + b);
  return nat;
}

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t hmul2_bf16(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Stored word -> four BF16x2 registers holding e2m1 * 2^-126 (codes 2j, 2j+1 in register j).
__device__ __forceinline__ void decode_codes(uint32_t q, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  constexpr uint32_t M = 0x81C081C0u;
  r0 = q & M;
  r1 = __funnelshift_l(q, q, 6) & M;
  r2 = __funnelshift_l(q, q, 12) & M;
  r3 = (__funnelshift_l(q, q, 2) & 0x00400040u) | (__funnelshift_l(q, q, 10) & 0x81808180u);
}

// E4M3 byte -> BF16 bit pattern of value * 2^64, replicated in both halves (0x7F/0xFF -> NaN).
// Formula of the reference's table (muse_moe_w4a16/cuda/moe.cu:2450-2461): exponent field 0 is
// mt * 2^-9, otherwise (1 + mt/8) * 2^(ex-7).
__device__ __forceinline__ uint32_t e4m3_scale_bf16x2(uint32_t byte) {
  const uint32_t ex = (byte >> 3) & 15u, mt = byte & 7u;
  uint32_t bits;
  if ((byte & 0x7Fu) == 0x7Fu) {
    bits = 0x7FFFu;
  } else if (ex != 0u) {
    bits = ((byte & 0x7Fu) << 4) + 0x5C00u;  // (ex + 184) << 7 | mt << 4
  } else {
    const float v = static_cast<float>(mt) * 36028797018963968.0f;  // mt * 2^-9 * 2^64 = mt * 2^55
    bits = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(v)));
  }
  bits |= (byte & 0x80u) << 8;
  return bits | (bits << 16);
}
#endif

}  // namespace msk
