// Packed NVFP4 tile layout and the in-register decode that goes with it.
//
// One tile = 128 weight rows x 256 K (one K stage):
//   bytes [0, 16384)      codes: 16-byte chunk c (0..7) of row r at (c*128 + r)*16; a chunk
//                         holds K [32c, 32c+32) of the stage, two E2M1 codes per byte in the
//                         source order (low nibble = even k);
//   bytes [16384, 18432)  scales: row r's sixteen E4M3 bytes at 16384 + r*16, byte j = block j.
// Thread r of a 128-thread group owns row r, so every 16-byte shared-memory read of a
// quarter-warp is 128 contiguous bytes. The repack is a pure byte permutation.
//
// Decode (per 16-byte chunk: 32 codes, two scale blocks): the hardware converts
//   cvt.rn.f16x2.e2m1x2  one byte  -> two F16 code values {0, .5, 1, 1.5, 2, 3, 4, 6} (signed)
//   cvt.rn.f16x2.e4m3x2  two bytes -> two F16 scales (zero, subnormal and NaN bytes included)
// and one mul.f16x2 per code pair gives e2m1 * e4m3, exact in F16 (at most 6 significant bits,
// magnitudes 2^-10 .. 2688). Measured on B200, each of these retires one warp instruction per
// two cycles per scheduler, and a chunk costs 16 converts + 16 multiplies + 3 for the scales;
// the bit-trick decode to BF16 (subnormal placement + mul.bf16x2) needed about twice the ALU
// work and made the whole kernel ALU-pipe bound. The MMA therefore runs F16 x F16 -> FP32: the
// activation operand is converted BF16 -> F16 on the way in (exact for 2^-17 <= |x| <= 65504,
// the range the reference's decode layer also assumes when it feeds its expert kernel "exact
// fp16" activations, muse_decode_layer/py/04_triton_kernels.py:557), the global scale is
// applied to the FP32 accumulator (muse_moe_w4a16/cuda/moe.cu:771-773).
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace msk {

constexpr int KS = 256;                                   // K elements per stage
constexpr int TILE_ROWS = 128;                            // weight rows per tile (= MMA M)
constexpr int TILE_CODE_BYTES = TILE_ROWS * KS / 2;       // 16384
constexpr int TILE_SF_BYTES = TILE_ROWS * KS / 16;        // 2048
constexpr int TILE_BYTES = TILE_CODE_BYTES + TILE_SF_BYTES;  // 18432

#ifdef __CUDACC__
// One chunk: four words (32 codes) and the low 16 bits of `sf2` (the scale bytes of its two
// blocks) -> sixteen F16x2 registers, register 4w+j = codes (8w+2j, 8w+2j+1) of the chunk.
__device__ __forceinline__ void decode_chunk(const uint32_t (&q)[4], uint32_t sf2, uint32_t (&o)[16]) {
  const uint32_t s01 = cvt_e4m3x2_f16(static_cast<uint16_t>(sf2 & 0xFFFFu));
  const uint32_t s0 = prmt(s01, s01, 0x1010u), s1 = prmt(s01, s01, 0x3232u);
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    uint32_t h0, h1, h2, h3;
    cvt_e2m1x8_f16(q[w], h0, h1, h2, h3);
    const uint32_t s = w < 2 ? s0 : s1;
    o[4 * w + 0] = hmul2_f16(h0, s);
    o[4 * w + 1] = hmul2_f16(h1, s);
    o[4 * w + 2] = hmul2_f16(h2, s);
    o[4 * w + 3] = hmul2_f16(h3, s);
  }
}

// BF16 -> F16 of a register pair, saturating at the F16 range (values beyond it cannot be
// represented; they do not occur for normalised activations): each half widened to FP32 (exact), then
// one saturating convert for the pair (three instructions per pair; the clamps spelled out with
// fminf / fmaxf were nine, and the sorted row copy of an 8192-token step converts 270 M values).
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
  uint32_t d;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;"
      : "=r"(d)
      : "f"(__uint_as_float(v & 0xFFFF0000u)), "f"(__uint_as_float(v << 16)));
  return d;
}
#endif

}  // namespace msk
