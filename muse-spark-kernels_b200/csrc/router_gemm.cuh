// Router logits as a tcgen05 GEMM with the FP32 router weight held as an exact-sum pair of BF16
// matrices: logits[t, e] = sum_h x[t, h] * (hi[e, h] + lo[e, h]), hi = bf16(w), lo = bf16(w - hi),
// BF16 x BF16 products (exact in FP32), FP32 accumulation in TMEM. This is how the reference's layers
// feed their routing (muse_decode_layer/py/05_tune.py:279-286, muse_prefill_layer/py/00_layer.py:369-374:
// the two halves stacked as one [2E, H] weight of their dense BF16 GEMM); its FP32 matvec
// (muse_decode_layer/cuda/router_fp32.cu:4-40) is the few-token form, msk_moe_router_logits here.
//
// One CTA per (128 experts, N tokens): D[128 experts, N tokens] in TMEM, both halves accumulated into
// the same accumulator (per 16-wide K step first the hi product, then the lo product: a fixed order).
//   warp 0   producer: 2-D TMA loads (128-byte swizzle) of the hi tile, the lo tile and the token tile
//            of every 64-wide K step into a ring;
//   warp 1   MMA issuer (tcgen05.mma kind::f16, both operands from shared memory), owns the TMEM allocation;
//   warps 2-5 epilogue: TMEM -> logits (FP32 [T, E]); a warp writes 32 consecutive experts of one token.
// All waits are bounded (ptx.cuh); a wait that gives up sets the status word and the CTA leaves.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "ptx.cuh"

namespace msk {

constexpr int RG_THREADS = 192;
constexpr int RG_STAGES = 4;
constexpr int RG_KSTEP = 64;                        // K elements per stage: one 128-byte swizzle row
constexpr int RG_A_BYTES = 128 * RG_KSTEP * 2;      // one 128-expert tile of a stage

struct RouterGemmCtrl {
  uint64_t full[RG_STAGES], empty[RG_STAGES], d_full;
  uint32_t tmem_base;
  int abort_word;
};

template <int N>
__global__ void __launch_bounds__(RG_THREADS, 1)
    router_hilo_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                       float* __restrict__ logits, int32_t* status, int T, int E, int H) {
  constexpr int B_BYTES = N * RG_KSTEP * 2;
  constexpr int STAGE_BYTES = 2 * RG_A_BYTES + B_BYTES;
  constexpr uint32_t TCOLS = N < 32 ? 32 : N;       // TMEM columns: a power of two, at least 32
  extern __shared__ __align__(1024) uint8_t rg_smem[];
  uint8_t* ring = rg_smem;
  RouterGemmCtrl& ctl = *reinterpret_cast<RouterGemmCtrl*>(rg_smem + RG_STAGES * STAGE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e0 = blockIdx.x * 128, t0 = blockIdx.y * N;
  const int n_steps = H / RG_KSTEP;

  if (tid == 0) {
    for (int i = 0; i < RG_STAGES; ++i) {
      mbar_init(&ctl.full[i], 1);
      mbar_init(&ctl.empty[i], 1);
    }
    mbar_init(&ctl.d_full, 1);
    ctl.abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl.tmem_base, TCOLS);
    tmem_relinquish();
  }
  pdl_wait();   // x may come from the kernel before
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl.tmem_base;
  volatile int* abortw = &ctl.abort_word;

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t keep = policy_evict_last();   // both operands are re-read by the other CTAs of the grid
      for (int ks = 0; ks < n_steps; ++ks) {
        const uint32_t slot = ks % RG_STAGES, par = (ks / RG_STAGES) & 1u;
        if (!mbar_wait(&ctl.empty[slot], par ^ 1u, abortw)) break;
        uint8_t* dst = ring + slot * STAGE_BYTES;
        mbar_arrive_expect_tx(&ctl.full[slot], STAGE_BYTES);
        tma_load_2d(dst, &tmap_w, ks * RG_KSTEP, e0, &ctl.full[slot], keep);                    // hi rows e0 .. e0+127
        tma_load_2d(dst + RG_A_BYTES, &tmap_w, ks * RG_KSTEP, E + e0, &ctl.full[slot], keep);   // lo rows
        tma_load_2d(dst + 2 * RG_A_BYTES, &tmap_x, ks * RG_KSTEP, t0, &ctl.full[slot], keep);   // tokens t0 .. (rows past T read as zero)
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = idesc_f16(FMT_BF16, FMT_BF16, 128, N);
    bool ok = true;
    for (int ks = 0; ks < n_steps && ok; ++ks) {
      const uint32_t slot = ks % RG_STAGES, par = (ks / RG_STAGES) & 1u;
      if (!mbar_wait(&ctl.full[slot], par, abortw)) { ok = false; break; }
      tc_fence_after();
      if (elect_one()) {
        const uint32_t a_hi = smem_u32(ring + slot * STAGE_BYTES), a_lo = a_hi + RG_A_BYTES, b = a_hi + 2 * RG_A_BYTES;
#pragma unroll
        for (int kk = 0; kk < RG_KSTEP / 16; ++kk) {
          const uint64_t bd = smem_desc_kmajor_sw128(b + kk * 32);
          mma_ss(tmem, smem_desc_kmajor_sw128(a_hi + kk * 32), bd, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
          mma_ss(tmem, smem_desc_kmajor_sw128(a_lo + kk * 32), bd, idesc, 1u);
        }
        tc_commit(&ctl.empty[slot]);
      }
      __syncwarp();
    }
    if (ok && elect_one()) tc_commit(&ctl.d_full);
    __syncwarp();
  } else {
    // epilogue: this warp's TMEM lane quarter holds 32 experts; column c is token t0 + c
    if (mbar_wait(&ctl.d_full, 0u, abortw)) {
      tc_fence_after();
      const int q = warp & 3;
      const int e = e0 + q * 32 + lane;
      const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < N; c0 += 16) {
        if (t0 + c0 >= T) break;
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        tmem_wait_ld();
        if (e < E) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (t0 + c0 + j < T) logits[static_cast<size_t>(t0 + c0 + j) * E + e] = __uint_as_float(r[j]);
        }
      }
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (ctl.abort_word != 0) {
    const uint64_t w0 = globaltimer_ns();
    while (globaltimer_ns() - w0 < 2000000ull) __nanosleep(1000);   // let copies in flight land before smem is released
    if (tid == 0 && status != nullptr) atomicExch(status, 1);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TCOLS);
  }
}

}  // namespace msk
