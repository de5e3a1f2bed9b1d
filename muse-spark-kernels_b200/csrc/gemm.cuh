// Persistent grouped GEMM for the routed experts on sm_100a.
//
// D[128 weight rows, N tokens] = W_tile[128, K] * X_tile[N, K]^T, weights on the MMA M side.
// Per CTA (384 threads, one CTA per SM):
//   warp 0      weight producer: 1-D bulk async copies (TMA engine) of packed NVFP4 tiles,
//               two tiles (a "pair") per K stage, into a shared-memory ring;
//   warp 1      MMA issuer: tcgen05.mma kind::f16, A from TMEM, B from shared memory,
//               FP32 accumulators in TMEM; owns the TMEM allocation;
//   warps 2-3   activation gather: cp.async of the token rows of the tile (through the
//               permutation for the gate/up GEMM) into the K-major core-matrix layout;
//   warps 4-7   dequant group 0 / warps 8-11 dequant group 1: thread r owns weight row r
//               of its tile: shared-memory codes -> BF16 (layout.cuh) -> tcgen05.st into the
//               TMEM A operand; afterwards the same threads run the epilogue.
// A pair is (gate tile j, up tile j) for PHASE 0, so SwiGLU pairs sit in the same TMEM lane,
// and (row tile 2j, row tile 2j+1) for PHASE 1. Both tiles of a pair share the B operand.
//
// A work unit is (token tile, pair, K split). Units are dealt round-robin to CTAs. With
// more than one K split every unit stores its raw FP32 accumulators to a partial buffer
// and takes a ticket; the unit that draws the last ticket sums the partials in split
// order 0..S-1 (so the sum order never depends on arrival order) and runs the epilogue.
//
// Numerics: operands are e2m1*e4m3*2^-62 (exact in BF16) and BF16 activations, FP32
// accumulation, accumulator * (gs * 2^62) in the epilogue; PHASE 0 writes
// bf16(silu(g) * u), PHASE 1 writes FP32 rows times (1 + post_norm_w) when given
// (muse_moe_w4a16/cuda/moe.cu:440-478).
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "layout.cuh"
#include "ptx.cuh"

namespace msk {

constexpr int GEMM_THREADS = 384;
constexpr int TMEM_COLS = 512;
constexpr int TMEM_A_BASE = 256;   // columns [256, 512): A operand, 128 columns per dequant group
constexpr int B_SBO = 4096;        // bytes between 8-token groups of the B tile (32 core matrices)
constexpr int B_LBO = 128;         // bytes between K-adjacent core matrices

enum : int {
  MSK_DEV_ERR_TIMEOUT = 1,  // a bounded wait inside a GEMM kernel gave up
};

template <int N>
struct GemmCfg {
  static constexpr int B_STAGE_BYTES = N * KS * 2;
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES + B_STAGE_BYTES;
  static constexpr int NST = N <= 16 ? 5 : (N <= 32 ? 4 : (N <= 64 ? 3 : 2));
  static constexpr int LUT_BYTES = 1024;
  static constexpr int CTRL_BYTES = 1024;  // barriers, TMEM base, abort word, tile table header
  static constexpr int SMEM_BYTES = NST * STAGE_BYTES + LUT_BYTES + CTRL_BYTES + (MAX_LOCAL_EXPERTS + 1) * 4 + 1024;
};

struct GemmParams {
  const uint8_t* w;          // packed tiles of this GEMM
  const float* gs;           // [local_count] global scales
  const void* act;           // PHASE 0: x bf16 [T, H]; PHASE 1: inter bf16 [R, I]
  void* outp;                // PHASE 0: inter bf16 [R, I]; PHASE 1: y fp32 [R, H]
  const __nv_bfloat16* post_norm_w;  // PHASE 1 only, nullable
  const int32_t* cnt;        // [local_count]
  const int32_t* off;        // [local_count + 1]
  const int32_t* perm;       // [R]
  float* partial;            // split-K partials
  int32_t* tickets;          // one per (token tile, pair)
  int32_t* status;           // workspace word 0
  int K;                     // reduction length (H for PHASE 0, I for PHASE 1)
  int out_ld;                // I for PHASE 0, H for PHASE 1
  int n_pairs;               // pairs per expert
  int nloc;
  int top_k;
  int splits;
  int evict_first;
};

struct GemmCtrl {
  uint64_t raw_full[6], raw_empty[6], b_full[6], b_empty[6];
  uint64_t a_full[2][2], a_empty[2];
  uint64_t d_full, d_empty;
  uint64_t epi_bar;  // the 256 dequant/epilogue threads, for the split-K ticket
  uint32_t tmem_base;
  int abort_word;
  int n_tiles;
  int last_flag;
};
static_assert(sizeof(GemmCtrl) <= 1024, "control block too large");

struct UnitInfo {
  int expert, row0, rows, pair, split, tile;
};

// unit index -> (token tile, pair, split); the token tile is located in the per-expert
// exclusive prefix of tile counts by binary search.
__device__ __forceinline__ UnitInfo decode_unit(int u, const int* tile_start, const GemmParams& p, int N) {
  UnitInfo ui;
  ui.split = u % p.splits;
  const int v = u / p.splits;
  ui.pair = v % p.n_pairs;
  ui.tile = v / p.n_pairs;
  int lo = 0, hi = p.nloc;  // largest e with tile_start[e] <= tile
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_start[mid] <= ui.tile) lo = mid; else hi = mid;
  }
  ui.expert = lo;
  const int local_tile = ui.tile - tile_start[lo];
  const int c = p.cnt[lo];
  ui.row0 = p.off[lo] + local_tile * N;
  ui.rows = min(N, c - local_tile * N);
  return ui;
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

template <int N, int PHASE>
__global__ void __launch_bounds__(GEMM_THREADS, 1) moe_gemm_kernel(const GemmParams p) {
  using C = GemmCfg<N>;
  constexpr int NST = C::NST;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* ring = smem;                                        // NST x [tile g0 | tile g1 | B]
  uint32_t* lut = reinterpret_cast<uint32_t*>(smem + NST * C::STAGE_BYTES);
  GemmCtrl& ctl = *reinterpret_cast<GemmCtrl*>(smem + NST * C::STAGE_BYTES + C::LUT_BYTES);
  int* tile_start = reinterpret_cast<int*>(smem + NST * C::STAGE_BYTES + C::LUT_BYTES + C::CTRL_BYTES);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nst_total = p.K / KS;                      // K stages of the whole reduction
  const int per_split = (nst_total + p.splits - 1) / p.splits;

  // ---------------------------------------------------------------- set-up
  if (tid == 0) {
    for (int i = 0; i < NST; ++i) {
      mbar_init(&ctl.raw_full[i], 1);
      mbar_init(&ctl.raw_empty[i], 8);
      mbar_init(&ctl.b_full[i], 2);
      mbar_init(&ctl.b_empty[i], 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&ctl.a_full[g][0], 4);
      mbar_init(&ctl.a_full[g][1], 4);
      mbar_init(&ctl.a_empty[g], 1);
    }
    mbar_init(&ctl.d_full, 1);
    mbar_init(&ctl.d_empty, 8);
    mbar_init(&ctl.epi_bar, 256);
    ctl.abort_word = 0;
    ctl.last_flag = 0;
    fence_mbar_init();
  }
  if (tid < 256) lut[tid] = e4m3_scale_bf16x2(static_cast<uint32_t>(tid));
  if (warp == 1) {
    tmem_alloc(&ctl.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 2) {  // exclusive prefix of per-expert tile counts
    int carry = 0;
    for (int base = 0; base < p.nloc; base += 32) {
      const int e = base + lane;
      const int c = e < p.nloc ? (p.cnt[e] + N - 1) / N : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (e < p.nloc) tile_start[e] = carry + incl - c;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      tile_start[p.nloc] = carry;
      ctl.n_tiles = carry;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem = ctl.tmem_base;
  const int n_units = ctl.n_tiles * p.n_pairs * p.splits;
  volatile int* abortw = &ctl.abort_word;

  if (warp == 0) {
    // ------------------------------------------------------ weight producer
    if (lane == 0) {
      const uint64_t pol = p.evict_first ? policy_evict_first() : policy_evict_last();
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
        const UnitInfo ui = decode_unit(u, tile_start, p, N);
        const int ks0 = ui.split * per_split, ks1 = min(nst_total, ks0 + per_split);
        const size_t tile0 =
            (static_cast<size_t>(ui.expert) * (2 * p.n_pairs) + 2 * ui.pair) * static_cast<size_t>(nst_total);
        const uint8_t* g0 = p.w + tile0 * TILE_BYTES;
        const uint8_t* g1 = g0 + static_cast<size_t>(nst_total) * TILE_BYTES;
        for (int ks = ks0; ks < ks1; ++ks, ++it) {
          const uint32_t slot = it % NST, par = (it / NST) & 1u;
          if (!mbar_wait(&ctl.raw_empty[slot], par ^ 1u, abortw)) { ok = false; break; }
          uint8_t* dst = ring + slot * C::STAGE_BYTES;
          mbar_arrive_expect_tx(&ctl.raw_full[slot], 2 * TILE_BYTES);
          bulk_g2s(dst, g0 + static_cast<size_t>(ks) * TILE_BYTES, TILE_BYTES, &ctl.raw_full[slot], pol);
          bulk_g2s(dst + TILE_BYTES, g1 + static_cast<size_t>(ks) * TILE_BYTES, TILE_BYTES, &ctl.raw_full[slot], pol);
        }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc = idesc_f16(FMT_BF16, FMT_BF16, 128, N);
    uint32_t it = 0, unit_i = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++unit_i) {
      const UnitInfo ui = decode_unit(u, tile_start, p, N);
      const int ks0 = ui.split * per_split, ks1 = min(nst_total, ks0 + per_split);
      if (!mbar_wait(&ctl.d_empty, (unit_i & 1u) ^ 1u, abortw)) { ok = false; break; }
      tc_fence_after();
      for (int ks = ks0; ks < ks1 && ok; ++ks, ++it) {
        const uint32_t slot = it % NST, par = (it / NST) & 1u;
        if (!mbar_wait(&ctl.b_full[slot], par, abortw)) { ok = false; break; }
        const uint32_t b_addr = smem_u32(ring + slot * C::STAGE_BYTES + 2 * TILE_BYTES);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (!mbar_wait(&ctl.a_full[0][h], it & 1u, abortw) || !mbar_wait(&ctl.a_full[1][h], it & 1u, abortw)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (lane == 0) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const int k16 = h * 8 + kk;
              const uint64_t bdesc = smem_desc_kmajor_noswz(b_addr + k16 * 256, B_LBO, B_SBO);
              const uint32_t acc = (ks > ks0 || k16 > 0) ? 1u : 0u;
              mma_ts(tmem + 0, tmem + TMEM_A_BASE + k16 * 8, bdesc, idesc, acc);
              mma_ts(tmem + N, tmem + TMEM_A_BASE + 128 + k16 * 8, bdesc, idesc, acc);
            }
            tc_commit(&ctl.a_empty[h]);
          }
          __syncwarp();
        }
        if (!ok) break;
        if (lane == 0) tc_commit(&ctl.b_empty[slot]);
        __syncwarp();
      }
      if (ok && lane == 0) tc_commit(&ctl.d_full);
      __syncwarp();
    }
  } else if (warp < 4) {
    // ----------------------------------------------------- activation gather
    const int gt = tid - 64;             // 0..63
    const int n_sub = gt & 7, c_sub = gt >> 3;  // token within an 8-group, chunk within an 8-chunk group
    const int gl = lane;
    uint32_t it = 0;
    bool ok = true;
    bool pending = false;  // a committed cp.async group whose barrier has not been signalled
    uint32_t pending_slot = 0;
    const size_t act_ld = static_cast<size_t>(p.K);
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
      const UnitInfo ui = decode_unit(u, tile_start, p, N);
      const int ks0 = ui.split * per_split, ks1 = min(nst_total, ks0 + per_split);
      // source row of token n = ng*8 + n_sub, for every 8-group ng
      const __nv_bfloat16* src[N / 8];
#pragma unroll
      for (int ng = 0; ng < N / 8; ++ng) {
        const int n = ng * 8 + n_sub;
        src[ng] = nullptr;
        if (n < ui.rows) {
          const int r = ui.row0 + n;
          const size_t row = PHASE == 0 ? static_cast<size_t>(p.perm[r] / p.top_k) : static_cast<size_t>(r);
          src[ng] = static_cast<const __nv_bfloat16*>(p.act) + row * act_ld;
        }
      }
      for (int ks = ks0; ks < ks1; ++ks, ++it) {
        const uint32_t slot = it % NST, par = (it / NST) & 1u;
        if (!mbar_wait(&ctl.b_empty[slot], par ^ 1u, abortw)) { ok = false; break; }
        uint8_t* dstB = ring + slot * C::STAGE_BYTES + 2 * TILE_BYTES;
#pragma unroll
        for (int ng = 0; ng < N / 8; ++ng) {
          const bool valid = src[ng] != nullptr;
          const __nv_bfloat16* s = valid ? src[ng] + static_cast<size_t>(ks) * KS : static_cast<const __nv_bfloat16*>(p.act);
#pragma unroll
          for (int cg = 0; cg < 4; ++cg) {
            const int chunk = cg * 8 + c_sub;
            cp_async16(dstB + ng * B_SBO + chunk * B_LBO + n_sub * 16, s + chunk * 8, valid);
          }
        }
        cp_async_commit();
        if (pending) {
          cp_async_wait<1>();
          fence_proxy_async_smem();
          __syncwarp();
          if (gl == 0) mbar_arrive(&ctl.b_full[pending_slot]);
        }
        pending = true;
        pending_slot = slot;
      }
    }
    if (pending) {
      cp_async_wait<0>();
      fence_proxy_async_smem();
      __syncwarp();
      if (gl == 0) mbar_arrive(&ctl.b_full[pending_slot]);
    }
  } else {
    // ------------------------------------------------- dequant + epilogue
    const int g = (warp - 4) >> 2;            // dequant group = tile of the pair
    const int row = (warp & 3) * 32 + lane;   // weight row inside the tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t a_tmem = tmem + lane_base + TMEM_A_BASE + g * 128;
    uint32_t it = 0, unit_i = 0, epi_par = 0;
    bool ok = true;
    // bounded barrier over the 256 dequant threads (a plain bar.sync could not time out)
    auto epi_sync = [&]() -> bool {
      mbar_arrive(&ctl.epi_bar);
      const bool r = mbar_wait(&ctl.epi_bar, epi_par, abortw);
      epi_par ^= 1u;
      return r;
    };
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++unit_i) {
      const UnitInfo ui = decode_unit(u, tile_start, p, N);
      const int ks0 = ui.split * per_split, ks1 = min(nst_total, ks0 + per_split);
      for (int ks = ks0; ks < ks1 && ok; ++ks, ++it) {
        const uint32_t slot = it % NST, par = (it / NST) & 1u;
        if (!mbar_wait(&ctl.raw_full[slot], par, abortw)) { ok = false; break; }
        const uint8_t* tile = ring + slot * C::STAGE_BYTES + g * TILE_BYTES;
        const uint4 sfw = *reinterpret_cast<const uint4*>(tile + TILE_CODE_BYTES + row * 16);
        const uint32_t sfa[4] = {sfw.x, sfw.y, sfw.z, sfw.w};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (!mbar_wait(&ctl.a_empty[h], (it & 1u) ^ 1u, abortw)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int chunk = h * 4 + c;  // 32 K per chunk = two scale blocks
            const uint4 q = *reinterpret_cast<const uint4*>(tile + (chunk * 128 + row) * 16);
            const uint32_t sw = sfa[chunk >> 1] >> ((chunk & 1) * 16);
            const uint32_t s0 = lut[sw & 0xFFu], s1 = lut[(sw >> 8) & 0xFFu];
            uint32_t o[16], r0, r1, r2, r3;
            decode_codes(q.x, r0, r1, r2, r3);
            o[0] = hmul2_bf16(r0, s0); o[1] = hmul2_bf16(r1, s0); o[2] = hmul2_bf16(r2, s0); o[3] = hmul2_bf16(r3, s0);
            decode_codes(q.y, r0, r1, r2, r3);
            o[4] = hmul2_bf16(r0, s0); o[5] = hmul2_bf16(r1, s0); o[6] = hmul2_bf16(r2, s0); o[7] = hmul2_bf16(r3, s0);
            decode_codes(q.z, r0, r1, r2, r3);
            o[8] = hmul2_bf16(r0, s1); o[9] = hmul2_bf16(r1, s1); o[10] = hmul2_bf16(r2, s1); o[11] = hmul2_bf16(r3, s1);
            decode_codes(q.w, r0, r1, r2, r3);
            o[12] = hmul2_bf16(r0, s1); o[13] = hmul2_bf16(r1, s1); o[14] = hmul2_bf16(r2, s1); o[15] = hmul2_bf16(r3, s1);
            tmem_st16(a_tmem + chunk * 16, o);
          }
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl.a_full[g][h]);
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.raw_empty[slot]);
      }
      if (!ok) break;
      // ------------------------------------------------------- epilogue
      if (!mbar_wait(&ctl.d_full, unit_i & 1u, abortw)) { ok = false; break; }
      tc_fence_after();
      const float gsc = p.gs[ui.expert] * TWO_POW_62;
      const int base_unit = ui.tile * p.n_pairs + ui.pair;
      bool finish = true;   // this unit runs the final epilogue
      if (p.splits > 1) {
        // raw accumulators of both tiles -> partial[base_unit][split][tile][row][N]
        float* part = p.partial + ((static_cast<size_t>(base_unit) * p.splits + ui.split) * 2) * (128 * N);
#pragma unroll
        for (int t2 = 0; t2 < 2; ++t2) {
          // group g stores tile g
          if (t2 != g) continue;
          float* dst = part + (static_cast<size_t>(t2) * 128 + row) * N;
#pragma unroll
          for (int c0 = 0; c0 < N; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(tmem + lane_base + t2 * N + c0, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; j += 4)
              *reinterpret_cast<uint4*>(dst + c0 + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
          }
        }
        tc_fence_before();
        __threadfence();
        // all 256 epilogue threads have stored; one of them takes the ticket
        if (!epi_sync()) { ok = false; break; }
        if (warp == 4 && lane == 0) {
          const int old = atomicAdd(&p.tickets[base_unit], 1);
          const int last = (old == p.splits - 1) ? 1 : 0;
          if (last) p.tickets[base_unit] = 0;  // leave the workspace launch-ready
          __threadfence();
          ctl.last_flag = last;
        }
        if (!epi_sync()) { ok = false; break; }
        finish = ctl.last_flag != 0;
        // d_empty can be released now: the accumulators are in memory
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.d_empty);
        if (!epi_sync()) { ok = false; break; }  // last_flag is rewritten by the next unit
      }
      if (finish) {
        if (PHASE == 0) {
          // columns split between the groups; each thread needs gate and up of its row
          constexpr int CPG = N >= 32 ? N / 2 : 16;
          const int c_beg = g * CPG, c_end = min(N, c_beg + CPG);
          __nv_bfloat16* outp = static_cast<__nv_bfloat16*>(p.outp);
          const int col = ui.pair * 128 + row;
          for (int c0 = c_beg; c0 < c_end; c0 += 16) {
            float ga[16], up[16];
            if (p.splits > 1) {
#pragma unroll
              for (int j = 0; j < 16; ++j) { ga[j] = 0.f; up[j] = 0.f; }
              for (int s = 0; s < p.splits; ++s) {
                const float* part = p.partial + ((static_cast<size_t>(base_unit) * p.splits + s) * 2) * (128 * N);
                const float4* pg = reinterpret_cast<const float4*>(part + static_cast<size_t>(row) * N + c0);
                const float4* pu = reinterpret_cast<const float4*>(part + (128 + static_cast<size_t>(row)) * N + c0);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float4 a = __ldcg(pg + j), b = __ldcg(pu + j);
                  ga[4 * j] += a.x; ga[4 * j + 1] += a.y; ga[4 * j + 2] += a.z; ga[4 * j + 3] += a.w;
                  up[4 * j] += b.x; up[4 * j + 1] += b.y; up[4 * j + 2] += b.z; up[4 * j + 3] += b.w;
                }
              }
            } else {
              uint32_t r0[16], r1[16];
              tmem_ld16(tmem + lane_base + 0 + c0, r0);
              tmem_ld16(tmem + lane_base + N + c0, r1);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 16; ++j) { ga[j] = __uint_as_float(r0[j]); up[j] = __uint_as_float(r1[j]); }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int n = c0 + j;
              if (n < ui.rows) {
                const float v = silu_f(ga[j] * gsc) * (up[j] * gsc);
                outp[static_cast<size_t>(ui.row0 + n) * p.out_ld + col] = __float2bfloat16_rn(v);
              }
            }
          }
        } else {
          float* outp = static_cast<float*>(p.outp);
          const int col = (2 * ui.pair + g) * 128 + row;
          float osc = gsc;
          if (p.post_norm_w != nullptr) osc *= 1.0f + __bfloat162float(p.post_norm_w[col]);
          for (int c0 = 0; c0 < N; c0 += 16) {
            float acc[16];
            if (p.splits > 1) {
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[j] = 0.f;
              for (int s = 0; s < p.splits; ++s) {
                const float* part = p.partial + ((static_cast<size_t>(base_unit) * p.splits + s) * 2) * (128 * N);
                const float4* pp = reinterpret_cast<const float4*>(part + (static_cast<size_t>(g) * 128 + row) * N + c0);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float4 a = __ldcg(pp + j);
                  acc[4 * j] += a.x; acc[4 * j + 1] += a.y; acc[4 * j + 2] += a.z; acc[4 * j + 3] += a.w;
                }
              }
            } else {
              uint32_t r[16];
              tmem_ld16(tmem + lane_base + g * N + c0, r);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[j] = __uint_as_float(r[j]);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int n = c0 + j;
              if (n < ui.rows) outp[static_cast<size_t>(ui.row0 + n) * p.out_ld + col] = acc[j] * osc;
            }
          }
        }
      }
      if (p.splits == 1) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.d_empty);
      }
    }
  }

  // -------------------------------------------------------------- teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (ctl.abort_word != 0) {
    // give copies still in flight time to land before shared memory and TMEM are released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    if (tid == 0) atomicExch(p.status, MSK_DEV_ERR_TIMEOUT);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace msk
