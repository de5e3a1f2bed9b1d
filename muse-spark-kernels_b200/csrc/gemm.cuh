// Persistent grouped GEMM for the routed experts on sm_100a.
//
// D[128 weight rows, N tokens] = W_tile[128, K] * X_tile[N, K]^T, weights on the MMA M side.
// Per CTA (768 threads, one CTA per SM):
//   warp 0       weight producer: 1-D bulk async copies (TMA engine) of packed NVFP4 tiles,
//                two tiles (a "pair") per K stage, into a shared-memory ring;
//   warps 1, 3   MMA issuers (one per tile of the pair): tcgen05.mma kind::f16, A from TMEM,
//                B from shared memory, FP32 accumulators in TMEM; warp 1 owns the TMEM allocation;
//   warp 2       activation gather: cp.async of the token rows of the tile (through the
//                permutation for the gate/up GEMM) into the K-major core-matrix layout;
//   warps 4-7    epilogue (gemm_epilogue.inl): TMEM accumulators -> SwiGLU / scale -> global,
//                or split-K partials (token tiles up to 64; for 128 the accumulators are single-
//                buffered and the sixteen dequant warps, idle by then, share the epilogue);
//   warps 8-23   dequant (gemm_dequant.inl): 2 tiles x 4 lane quarters x 2 K halves. A thread
//                owns one weight row of its tile: shared-memory codes -> BF16 (layout.cuh) ->
//                tcgen05.st into a ring of TMEM A slots (128 K each) the MMA warp consumes.
// Measured on B200: tcgen05.mma M=128 N=16 K=16 with A in TMEM retires every ~9 cycles, with
// A in shared memory every ~39; the decode ALU work (~2 instructions per weight) is what has
// to be spread over all four schedulers, hence sixteen dequant warps.
// A pair is (gate tile j, up tile j) for PHASE 0, so SwiGLU pairs sit in the same TMEM lane,
// and (row tile 2j, row tile 2j+1) for PHASE 1. Both tiles of a pair share the B operand.
//
// A work unit is (token tile, pair, K split), dealt round-robin to CTAs. Accumulators are
// double-buffered in TMEM (N <= 64) so the epilogue of a unit overlaps the main loop of the
// next. With more than one K split every unit stores raw FP32 accumulators to a partial
// buffer and takes a ticket; the unit that draws the last ticket sums the partials in
// split order 0..S-1 (the order never depends on arrival) and runs the epilogue.
//
// Numerics: operands are e2m1*e4m3 (exact in F16) and the BF16 activations held as F16 (exact
// in the F16 range), FP32 accumulation, accumulator * gs in the epilogue; PHASE 0 writes
// bf16(silu(g) * u) (stored as F16), PHASE 1 writes FP32 rows times (1 + post_norm_w) when
// given (muse_moe_w4a16/cuda/moe.cu:440-478).
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda.h>
#include <cuda_runtime.h>

#include "layout.cuh"
#include "ptx.cuh"

namespace msk {

constexpr int GEMM_THREADS = 768;
constexpr int TMEM_COLS = 512;
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
  // TMEM: NDBUF accumulator buffers of 2N columns (tile 0 | tile 1) from column 0; above them
  // the A ring: two groups (tiles) of NSLOT slots, 64 columns (128 K = half a stage) each.
  static constexpr int NDBUF = N <= 64 ? 2 : 1;
  static constexpr int A_BASE = N <= 32 ? 128 : 256;
  static constexpr int NSLOT = N <= 32 ? 3 : 2;
  static constexpr int SLOT_COLS = 64;
  static constexpr int A_GROUP_COLS = NSLOT * SLOT_COLS;
  // Token tiles of 64 and more fetch the activation operand with TMA (2-D boxes of 64 K x N rows,
  // 128-byte swizzle) from rows that are contiguous in sorted order; narrower tiles gather rows
  // through the permutation with cp.async (gemm_gather.inl).
  static constexpr bool TMA_B = N >= 64;
  static constexpr int LUT_BYTES = 0;
  static constexpr int CTRL_BYTES = 1024;  // barriers, TMEM base, abort word, tile table header
  static constexpr int TABLE_INTS = MAX_LOCAL_EXPERTS + 4;  // per table: tile_start, cnt, off copies
  static constexpr int TABLE_BYTES = 3 * TABLE_INTS * 4;
  static constexpr int SMEM_BYTES = NST * STAGE_BYTES + LUT_BYTES + CTRL_BYTES + TABLE_BYTES + 1024;
  static_assert(NDBUF * 2 * N <= A_BASE && A_BASE + 2 * A_GROUP_COLS <= TMEM_COLS, "TMEM budget");
};

struct GemmParams {
  CUtensorMap tmap_act;      // TMA_B only: [rows, K] bf16, box 64 x N, 128-byte swizzle (64-byte aligned: first member)
  const uint8_t* w;          // packed tiles of this GEMM
  const float* gs;           // [local_count] global scales
  const void* act;           // PHASE 0: x as f16 [T, H] (or sorted rows [R, H] with TMA_B); PHASE 1: inter f16 [R, I]
  void* outp;                // PHASE 0: inter f16 [R, I]; PHASE 1: y fp32 [R, H]
  const __nv_bfloat16* post_norm_w;  // PHASE 1 only, nullable
  const int32_t* cnt;        // [local_count]
  const int32_t* off;        // [local_count + 1]
  const int32_t* perm;       // [R]
  float* partial;            // split-K partials
  int32_t* tickets;          // one per (token tile, pair)
  int32_t* status;           // workspace word 0
  unsigned long long* trace; // nullable: 16 %globaltimer stamps per CTA (see TR_* below)
  int K;                     // reduction length (H for PHASE 0, I for PHASE 1)
  int out_ld;                // I for PHASE 0, H for PHASE 1
  int n_pairs;               // pairs per expert
  int nloc;
  int top_k;
  int splits;
  int evict_first;
  int y_bf16;                // PHASE 1 without K splits: y rows as BF16 instead of FP32
};

// Trace slots (per CTA, nanoseconds): the counterpart of the reference's DBG(k) stamps
// (muse_moe_w4a16/cuda/moe.cu:279-284).
enum : int { TR_START = 0, TR_SETUP, TR_FIRST_BULK, TR_FIRST_RAW, TR_FIRST_AFULL, TR_FIRST_MMA, TR_FIRST_DFULL,
              TR_FIRST_EPI_DONE, TR_LAST_DFULL, TR_END, TR_UNITS, TR_STAGES };
#define MSK_TR(slot) do { if (p.trace != nullptr) p.trace[blockIdx.x * 16 + (slot)] = globaltimer_ns(); } while (0)
// Detailed event list of CTA 0: role r (0 first dequant thread, 1 MMA issuer, 2 weight producer)
// appends up to 256 stamps, each tagged with a small code in the low 8 bits, after the
// 256 x 16 per-CTA stamps.
#ifdef MSK_TRACE_DETAIL
#define MSK_TRD(role, idx, code) do { if (p.trace != nullptr && blockIdx.x == 0 && (idx) < 256) { \
  p.trace[256 * 16 + (role) * 256 + (idx)] = (globaltimer_ns() << 8) | (code); ++(idx); } } while (0)
#else
#define MSK_TRD(role, idx, code) do { (void)(idx); } while (0)
#endif

struct GemmCtrl {
  uint64_t raw_full[6], raw_empty[6], b_full[6], b_empty[6];
  uint64_t a_full[2][6], a_empty[2][6];
  uint64_t d_full[2], d_empty[2];
  uint64_t epi_bar;  // the 128 epilogue threads, for the split-K ticket
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
  // tile_start is followed in shared memory by copies of cnt[] and off[] (GemmCfg::TABLE_INTS apart)
  const int* cnt_s = tile_start + (MAX_LOCAL_EXPERTS + 4);
  const int* off_s = cnt_s + (MAX_LOCAL_EXPERTS + 4);
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
  const int c = cnt_s[lo];
  ui.row0 = off_s[lo] + local_tile * N;
  ui.rows = min(N, c - local_tile * N);
  return ui;
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

// The SwiGLU value as the down GEMM reads it: rounded to BF16 (the reference's one rounding of
// `inter`, muse_prefill_layer/py/07_selftest.py:70), then held as F16 (exact inside the F16 range).
__device__ __forceinline__ __half inter_value(float v) {
  const float r = __bfloat162float(__float2bfloat16_rn(v));
  return __float2half_rn(fminf(fmaxf(r, -65504.f), 65504.f));
}

// Epilogue of a unit without K splits for the thread that owns TMEM lane `row`: columns
// [c_beg, c_end) of the accumulators at d_tmem (lane base included). PHASE 0 reads gate (tile 0)
// and up (tile 1) and writes bf16(silu(g) * u) into inter; PHASE 1 writes the rows of `tile`
// scaled by gs (and 1 + post_norm_w) into y.
template <int N, int PHASE>
__device__ __forceinline__ void epilogue_columns(const GemmParams& p, const UnitInfo& ui, uint32_t d_tmem, int row,
                                                 int c_beg, int c_end, int tile) {
  const float gsc = p.gs[ui.expert];
  if (PHASE == 0) {
    __half* outp = static_cast<__half*>(p.outp) + static_cast<size_t>(ui.row0) * p.out_ld + ui.pair * 128 + row;
    for (int c0 = c_beg; c0 < c_end; c0 += 16) {
      if (c0 >= ui.rows) break;
      uint32_t r0[16], r1[16];
      tmem_ld16(d_tmem + c0, r0);
      tmem_ld16(d_tmem + N + c0, r1);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (c0 + j < ui.rows) {
          const float v = silu_f(__uint_as_float(r0[j]) * gsc) * (__uint_as_float(r1[j]) * gsc);
          outp[static_cast<size_t>(c0 + j) * p.out_ld] = inter_value(v);
        }
      }
    }
  } else {
    const int col = (2 * ui.pair + tile) * 128 + row;
    float osc = gsc;
    if (p.post_norm_w != nullptr) osc *= 1.0f + __bfloat162float(p.post_norm_w[col]);
    float* outp = static_cast<float*>(p.outp) + static_cast<size_t>(ui.row0) * p.out_ld + col;
    __nv_bfloat16* outb = static_cast<__nv_bfloat16*>(p.outp) + static_cast<size_t>(ui.row0) * p.out_ld + col;
    for (int c0 = c_beg; c0 < c_end; c0 += 32) {
      if (c0 >= ui.rows) break;
      uint32_t r[32];
      tmem_ld32(d_tmem + tile * N + c0, r);
      tmem_wait_ld();
      if (p.y_bf16) {   // wide token tiles: y rows in BF16, as the reference's wide-tile build keeps them
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c0 + j < ui.rows) outb[static_cast<size_t>(c0 + j) * p.out_ld] = __float2bfloat16_rn(__uint_as_float(r[j]) * osc);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c0 + j < ui.rows) outp[static_cast<size_t>(c0 + j) * p.out_ld] = __uint_as_float(r[j]) * osc;
      }
    }
  }
}

template <int N, int PHASE>
__global__ void __launch_bounds__(GEMM_THREADS, 1) moe_gemm_kernel(const __grid_constant__ GemmParams p) {
  using C = GemmCfg<N>;
  constexpr int NST = C::NST;
  constexpr int NSLOT = C::NSLOT;
  constexpr int NDBUF = C::NDBUF;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* ring = smem;                                        // NST x [tile g0 | tile g1 | B]
  GemmCtrl& ctl = *reinterpret_cast<GemmCtrl*>(smem + NST * C::STAGE_BYTES + C::LUT_BYTES);
  int* tile_start = reinterpret_cast<int*>(smem + NST * C::STAGE_BYTES + C::LUT_BYTES + C::CTRL_BYTES);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nst_total = p.K / KS;                      // K stages of the whole reduction
  const int per_split = (nst_total + p.splits - 1) / p.splits;

  // ---------------------------------------------------------------- set-up
  if (tid == 0) {
    MSK_TR(TR_START);
    for (int i = 0; i < NST; ++i) {
      mbar_init(&ctl.raw_full[i], 1);
      mbar_init(&ctl.raw_empty[i], 16);
      mbar_init(&ctl.b_full[i], 1);
      mbar_init(&ctl.b_empty[i], 2);  // one commit per MMA issuer
    }
    for (int i = 0; i < NSLOT; ++i) {
      mbar_init(&ctl.a_full[0][i], 4);
      mbar_init(&ctl.a_full[1][i], 4);
      mbar_init(&ctl.a_empty[0][i], 1);
      mbar_init(&ctl.a_empty[1][i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl.d_full[i], 2);  // one commit per MMA issuer
      mbar_init(&ctl.d_empty[i], C::NDBUF == 1 ? 16 : 4);  // single buffer: the dequant warps run the epilogue
    }
    mbar_init(&ctl.epi_bar, 128);
    ctl.abort_word = 0;
    ctl.last_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  // Programmatic dependent launch: everything above ran while the previous kernel was still
  // draining. PHASE 0 reads the sort tables next, so it waits here. PHASE 1 is launched behind
  // PHASE 0, which itself only passed this point after the sort had completed, so the tables
  // are already final: only the activation gather (inter rows) waits, and the weight stream,
  // dequant and TMEM ring of the down GEMM fill up during the tail of the gate/up GEMM.
  if (PHASE == 0) pdl_wait();
  pdl_launch_dependents();
  if (warp == 2) {  // exclusive prefix of per-expert tile counts
    int carry = 0;
    for (int base = 0; base < p.nloc; base += 32) {
      const int e = base + lane;
      const int cn = e < p.nloc ? p.cnt[e] : 0;
      if (e < p.nloc) tile_start[C::TABLE_INTS + e] = cn;
      const int c = (cn + N - 1) / N;
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
  if (warp == 3) {  // off[] copy, in parallel with the scan above
    for (int e = lane; e <= p.nloc; e += 32) tile_start[2 * C::TABLE_INTS + e] = p.off[e];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem = ctl.tmem_base;
  if (tid == 0) MSK_TR(TR_SETUP);
  const int n_units = ctl.n_tiles * p.n_pairs * p.splits;
  volatile int* abortw = &ctl.abort_word;

  if (warp == 0) {
#include "gemm_producer.inl"
  } else if (warp == 1 || warp == 3) {
#include "gemm_mma.inl"
  } else if (warp == 2) {
#include "gemm_gather.inl"
  } else if (warp >= 8) {
#include "gemm_dequant.inl"
  } else {
#include "gemm_epilogue.inl"
  }

  // -------------------------------------------------------------- teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (tid == 0) MSK_TR(TR_END);
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
