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
// A pair is (gate tile j, up tile j) for the gate/up GEMM (phase 0), so SwiGLU pairs sit in the same
// TMEM lane, and (row tile 2j, row tile 2j+1) for the down GEMM (phase 1). Both tiles of a pair
// share the B operand.
//
// One kernel template, three modes: MODE 0 runs phase 0, MODE 1 phase 1 (two launches chained by
// programmatic dependent launch, any token count), MODE 2 both phases in one launch for a few tokens:
// the weight stream, the dequant ring and the MMA pipeline run on from the last gate/up stage into
// the first down stage without draining; only the activation gather of phase 1 waits, per token tile,
// until the gate/up units of that tile have all written their columns of `inter` (the reference's single
// persistent kernel hands over per job in the same way, with no barrier between its phases:
// muse_moe_w4a16/cuda/moe.cu:690,1895,2020). MODE 2 also routes, sorts and
// converts the token rows itself and ends with the folded combine: the step is one launch.
//
// Work. A base unit is (token tile, pair); its reduction runs over K / 256 stages. The base units
// are laid out as one flat list ordered (token tile, pair) and dealt to the CTAs in one of two ways
// (PieceIter below):
//   whole units, round-robin (unit u to CTA u % gridDim.x);
//   flat shares (few routed rows, token tiles up to 64): full rounds of whole units as above, then
//          the last full round together with the units left over as a list of (base unit, K stage)
//          items cut into gridDim.x equal contiguous shares, so every SM streams the same number of
//          weight bytes (with fewer units than CTAs nothing is cut). A unit cut between CTAs is
//          accumulated as "pieces": every piece stores its raw FP32 accumulators to a slot of the
//          partial buffer and takes a ticket, the piece that draws the last ticket sums the pieces in
//          ascending K order (the order never depends on arrival) and runs the epilogue. Cut points
//          depend on the shapes, the number of token tiles and the grid size given by the host, not
//          on the device.
// Accumulators are double-buffered in TMEM (N <= 64) so the epilogue of a piece overlaps the main
// loop of the next.
//
// Numerics: operands are e2m1*e4m3 (exact in F16) and the BF16 activations held as F16 (exact
// in the F16 range), FP32 accumulation, accumulator * gs in the epilogue; phase 0 writes
// bf16(silu(g) * u) (stored as F16), phase 1 writes FP32 rows times (1 + post_norm_w) when
// given (muse_moe_w4a16/cuda/moe.cu:440-478).
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda.h>
#include <cuda_runtime.h>

#include "layout.cuh"
#include "ptx.cuh"
#include "route_sort.cuh"

namespace msk {

constexpr int GEMM_THREADS = 768;
static_assert(GEMM_THREADS / 32 == SMALL_ROUTE_WARPS, "one routing scratch row per warp");
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
  // 128-byte swizzle) from rows that are contiguous in sorted order (the sorted F16 copy of the token
  // rows for the gate/up GEMM, `inter` for the down GEMM); narrower tiles gather rows through the
  // permutation with cp.async (gemm_gather.inl). Gathering the wide tiles' rows with cp.async as well
  // (four warps, straight from the unsorted F16 rows, no sorted copy) was built and measured: the
  // 16-byte requests load L2 so much less efficiently than TMA's full lines that the gate/up GEMM of
  // the 8192-token step took 3.08 ms instead of 1.48 ms, far more than the 0.22 ms the copy costs.
  // Fetching them by index with TMA itself (tile::gather4 from the unsorted rows, a one-row box, every
  // lane of the producer warp issuing the four copies of its four rows per stage: 128 copies of 512
  // bytes where four tiled copies of 16 KB do) gave the same bits and was slower still: 4.07 ms for that
  // GEMM, 0.54 against 0.19 ms at 256 tokens. The copy engine's rate per request, not the bytes, bounds it.
  static constexpr bool TMA_B = N >= 64;
  static constexpr int LUT_BYTES = 0;
  static constexpr int CTRL_BYTES = 1024;  // barriers, TMEM base, abort word, tile table header
  static constexpr int TABLE_INTS = MAX_LOCAL_EXPERTS + 4;  // per table: tile_start, cnt, off copies
  static constexpr int TABLE_BYTES = 3 * TABLE_INTS * 4;
  static constexpr int SMEM_BYTES = NST * STAGE_BYTES + LUT_BYTES + CTRL_BYTES + TABLE_BYTES + 1024;
  static_assert(NDBUF * 2 * N <= A_BASE && A_BASE + 2 * A_GROUP_COLS <= TMEM_COLS, "TMEM budget");
};

struct PhaseParams {
  const uint8_t* w;          // packed tiles of this GEMM
  const float* gs;           // [local_count] global scales
  const void* act;           // phase 0: x as f16 [T, H] (or sorted rows [R, H] with TMA_B); phase 1: inter f16 [R, I]
  void* outp;                // phase 0: inter f16 [R, I]; phase 1: y fp32 [R, H]
  float* partial;            // pieces of cut units: 2 * gridDim.x slots of 2 * 128 * N floats
  int32_t* tickets;          // one per base unit, zero between launches
  int K;                     // reduction length (H for phase 0, I for phase 1)
  int out_ld;                // I for phase 0, H for phase 1
  int n_pairs;               // pairs per expert
  int pad_;
};

struct GemmParams {
  CUtensorMap tmap_act[2];   // TMA_B only, per phase: [rows, K] f16, box 64 x N, 128-byte swizzle (64-byte aligned: first member)
  PhaseParams ph[2];         // [0] gate/up, [1] down; a single-phase launch uses its own entry only
  const __nv_bfloat16* post_norm_w;  // phase 1, nullable
  int32_t* cnt;              // [local_count]      sort tables in global memory: read here, or written by CTA 0
  int32_t* off;              // [local_count + 1]  when this kernel routes and sorts itself (route != 0)
  int32_t* perm;             // [R]
  int32_t* inv;              // [T * top_k]
  int32_t* status;           // workspace word 0
  unsigned long long* trace; // nullable: 16 %globaltimer stamps per CTA (see TR_* below)
  int nloc;
  int top_k;
  int flat;                  // 1: equal shares of the flat (base unit, K stage) list; 0: whole units
  int evict_first;
  int handover;              // two launches: gate/up units count per token tile (tile_done), down units wait for their
                             // tile's count instead of for the whole gate/up grid (see gemm_gather.inl)
  int y_bf16;                // phase 1, token tile 128: y rows as BF16 instead of FP32
  // Phase 0 with route != 0 (at most 256 entries): every CTA derives the sort tables in its prologue.
  // route 1: top-k of `logits` first (CTA 0 writes ids_out / tw_out); route 2: ids_in given.
  int route;
  const float* logits;       // [T, E]
  const float* bias;         // [E], nullable
  const int32_t* ids_in;     // [T, top_k]
  int32_t* ids_out;
  float* tw_out;
  int T, E, lo, mode;
  float route_scale;
  // Phase 1 with fold != 0 (at most 32 tokens): the combine is done by the CTAs that complete a
  // token's last contributions, so no combine launch follows. fold 1 (post-expert norm): per token, at
  // the end of the kernel; fold 2 (no norm): per (token, pair of 256 output columns), in the epilogue.
  int fold;
  const float* tw;           // [T, top_k] routing weights
  __nv_bfloat16* out;        // [T, H]
  int32_t* tok_tickets;      // [T] (fold 1) or [T][pairs of phase 1] (fold 2), zero between launches
  float eps;                 // post-expert norm
  // MODE 2: the token rows as given (BF16), converted to F16 into ph[0].act by all CTAs together; the
  // grid-wide counters grid_bar[0] (CTAs whose slice of the F16 rows is written) and grid_bar[1]
  // (exits); and per token tile the number of finished gate/up units (tile_done) and of down units
  // that have seen them all (tile_seen), which hand `inter` from phase 0 to phase 1 tile by tile.
  const __nv_bfloat16* x_bf16;
  unsigned int* grid_bar;
  unsigned int* tile_done;
  unsigned int* tile_seen;
};

// Trace slots (per CTA, nanoseconds): the counterpart of the reference's DBG(k) stamps
// (muse_moe_w4a16/cuda/moe.cu:279-284).
enum : int { TR_START = 0, TR_SETUP, TR_FIRST_BULK, TR_FIRST_RAW, TR_FIRST_AFULL, TR_FIRST_MMA, TR_FIRST_DFULL,
              TR_FIRST_EPI_DONE, TR_LAST_DFULL, TR_END, TR_ROUTED, TR_FOLD_END, TR_CONVERTED, TR_TOPK };
#define MSK_TR(slot) do { if (p.trace != nullptr) p.trace[blockIdx.x * 16 + (slot)] = globaltimer_ns(); } while (0)
// Detailed event list of CTA 0: role r (0 first dequant thread, 1 MMA issuer, 2 weight producer, 3 first
// epilogue thread, 4 gather warp)
// appends up to 128 stamps, each tagged with a small code in the low 8 bits, after the
// 256 x 16 per-CTA stamps.
#ifdef MSK_TRACE_DETAIL
#define MSK_TRD(role, idx, code) do { if (p.trace != nullptr && blockIdx.x == MSK_TRACE_DETAIL && (idx) < 128) { \
  p.trace[256 * 16 + (role) * 128 + (idx)] = (globaltimer_ns() << 8) | (code); ++(idx); } } while (0)
#else
#define MSK_TRD(role, idx, code) do { (void)(idx); } while (0)
#endif

constexpr int FOLD_MAX_TOKENS = 32;

struct GemmCtrl {
  uint64_t raw_full[6], raw_empty[6], b_full[6], b_empty[6];
  uint64_t a_full[2][6], a_empty[2][6];
  uint64_t d_full[2], d_empty[2];
  uint64_t epi_bar;  // the 128 epilogue threads, for the tickets
  uint32_t tmem_base;
  int abort_word;
  int n_tiles;
  int last_flag[2];
  int fin_n;                           // fold: tokens this CTA has to combine when its units are done
  uint8_t fin_tok[FOLD_MAX_TOKENS];
  uint8_t klocal[FOLD_MAX_TOKENS];     // fold: local routes of each token
  uint8_t perm8[SMALL_SORT_MAX_ENTRIES];  // route / fold: entry index of each sorted row
};
static_assert(sizeof(GemmCtrl) <= 1024, "control block too large");

struct UnitInfo {
  int expert, row0, rows, pair, tile;
};

// base unit index -> (token tile, pair); the token tile is located in the per-expert exclusive
// prefix of tile counts by binary search.
__device__ __noinline__ UnitInfo decode_unit(int base, const int* tile_start, int n_pairs, int nloc, int N) {
  // tile_start is followed in shared memory by copies of cnt[] and off[] (GemmCfg::TABLE_INTS apart)
  const int* cnt_s = tile_start + (MAX_LOCAL_EXPERTS + 4);
  const int* off_s = cnt_s + (MAX_LOCAL_EXPERTS + 4);
  UnitInfo ui;
  ui.pair = base % n_pairs;
  ui.tile = base / n_pairs;
  int lo = 0, hi = nloc;  // largest e with tile_start[e] <= tile
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

// ---- work distribution (see the header comment). Positions are indices into the flat list of
// (base unit, K stage) items: pos = base * nst + ks. 32-bit arithmetic throughout (the host only
// plans flat shares while items * shares fits; a 64-bit divide is a subroutine call, and on a
// one-token step every cold instruction line counts).
__host__ __device__ inline int share_begin(int items, int shares, int c) {
  return static_cast<int>(static_cast<unsigned>(items) * static_cast<unsigned>(c) / static_cast<unsigned>(shares));
}
// The share that holds item x: the largest c with share_begin(c) <= x.
__host__ __device__ inline int share_owner(int items, int shares, int x) {
  return static_cast<int>((static_cast<unsigned>(x + 1) * static_cast<unsigned>(shares) - 1u) / static_cast<unsigned>(items));
}
// Slot of the partial buffer for the piece of a cut unit that share c holds: a share holds at most
// one piece that starts inside a unit (at the head of its range, slot 2c) and at most one that starts
// a unit but does not finish it (at the tail of its range, slot 2c + 1).
__host__ __device__ inline int piece_slot(int c, bool starts_unit) { return 2 * c + (starts_unit ? 1 : 0); }
constexpr long long FLAT_MAX_PRODUCT = 1ll << 31;   // items * shares must stay below this for flat shares

// Whole units first, round-robin (unit u to CTA u % shares, the order in which the weights lie in
// memory: at any time the CTAs stream neighbouring units), as long as full rounds can be dealt; with
// flat shares the units that are left over (fewer than there are CTAs) are then cut into equal
// contiguous shares of (unit, stage) items. Measured on B200: dealing all units as contiguous
// per-CTA ranges instead streams about 6 % slower than round-robin.
struct PieceIter {
  int a_pos, a_end, a_step;     // whole units, first round-robin sequence (see make_piece_iter)
  int rr_pos, rr_end, rr_step;  // whole units, round-robin over all CTAs
  int pos, end;                 // flat positions inside the tail: (base - tail_base) * nst + ks
  int nst, tail_base;
  __host__ __device__ bool next(int& base, int& ks0, int& ks1) {
    if (a_pos < a_end) {
      base = a_pos;
      ks0 = 0;
      ks1 = nst;
      a_pos += a_step;
      return true;
    }
    if (rr_pos < rr_end) {
      base = rr_pos;
      ks0 = 0;
      ks1 = nst;
      rr_pos += rr_step;
      return true;
    }
    if (pos >= end) return false;
    const int b = pos / nst;
    base = tail_base + b;
    ks0 = pos - b * nst;
    const int left = end - pos;
    const int len = left < nst - ks0 ? left : nst - ks0;
    ks1 = ks0 + len;
    pos += len;
    return true;
  }
};

// First unit of the flat tail: the units before it are dealt whole. The tail is the last full round
// plus the left-over units, so that a share holds at least one unit's worth of stages and a unit is cut
// into two or three pieces at most. With fewer units than CTAs nothing is cut: a cut unit pays for its
// pieces' round trips through L2 (store, fence, ticket, reload: several microseconds, about seven K
// stages of streaming), more than the idle CTAs of a single round cost.
__host__ __device__ inline int tail_begin(int flat, int n_base, int shares) {
  if (!flat || n_base < shares) return n_base;
  return (n_base / shares - 1) * shares;
}

// heavy / skip (one launch for both phases, phase 1 only): the first `heavy` CTAs hold one more unit
// of phase 0 than the others, so the first `skip` rounds of phase 1 are dealt to the other CTAs only;
// skip is that extra unit's cost in units of phase 1. With heavy == 0 every unit u goes to CTA u % shares.
__host__ __device__ inline PieceIter make_piece_iter(int flat, int n_base, int nst, int c, int shares, int heavy = 0,
                                                     int skip = 0) {
  PieceIter it;
  it.nst = nst;
  it.tail_base = tail_begin(flat, n_base, shares);
  const int light = shares - heavy;
  int n_a = (heavy > 0 && !flat) ? skip * light : 0;
  if (n_a > n_base) n_a = n_base;
  it.a_pos = c >= heavy ? c - heavy : n_a;
  it.a_end = n_a;
  it.a_step = light;
  it.rr_pos = n_a + c;
  it.rr_end = it.tail_base;
  it.rr_step = shares;
  const int items = (n_base - it.tail_base) * nst;
  it.pos = share_begin(items, shares, c);
  it.end = share_begin(items, shares, c + 1);
  return it;
}

// The (heavy, skip) pair of phase 1 in the one-launch kernel, from the unit count and stage count of phase 0.
__host__ __device__ inline void phase1_skew(int n_base0, int nst0, int nst1, int shares, int& heavy, int& skip) {
  // With less than one full round of phase 0 nothing is skewed: every tile then completes at the same
  // time, the CTAs without a gate/up unit cannot start phase 1 any earlier, and plain round-robin
  // spreads it best.
  heavy = n_base0 >= shares ? n_base0 % shares : 0;
  skip = heavy > 0 ? (nst0 + nst1 / 2) / nst1 : 0;
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

// The SwiGLU value as the down GEMM reads it: rounded to BF16 (the reference's one rounding of
// `inter`, muse_prefill_layer/py/07_selftest.py:70), then held as F16 (exact inside the F16 range).
__device__ __forceinline__ __half inter_value(float v) {
  const float r = __bfloat162float(__float2bfloat16_rn(v));
  return __float2half_rn(fminf(fmaxf(r, -65504.f), 65504.f));
}

// Epilogue of a whole unit for the thread that owns TMEM lane `row`: columns [c_beg, c_end) of the
// accumulators at d_tmem (lane base included). Phase 0 reads gate (tile 0) and up (tile 1) and
// writes bf16(silu(g) * u) into inter; phase 1 writes the rows of `tile` scaled by gs (and
// 1 + post_norm_w) into y. (Used by the wide token tile, whose dequant warps share the epilogue.)
template <int N>
__device__ __forceinline__ void epilogue_columns(const GemmParams& p, const PhaseParams& pp, int phase,
                                                 const UnitInfo& ui, uint32_t d_tmem, int row, int c_beg, int c_end,
                                                 int tile) {
  const float gsc = pp.gs[ui.expert];
  if (phase == 0) {
    __half* outp = static_cast<__half*>(pp.outp) + static_cast<size_t>(ui.row0) * pp.out_ld + ui.pair * 128 + row;
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
          outp[static_cast<size_t>(c0 + j) * pp.out_ld] = inter_value(v);
        }
      }
    }
  } else {
    const int col = (2 * ui.pair + tile) * 128 + row;
    float osc = gsc;
    if (p.post_norm_w != nullptr) osc *= 1.0f + __bfloat162float(p.post_norm_w[col]);
    float* outp = static_cast<float*>(pp.outp) + static_cast<size_t>(ui.row0) * pp.out_ld + col;
    __nv_bfloat16* outb = static_cast<__nv_bfloat16*>(pp.outp) + static_cast<size_t>(ui.row0) * pp.out_ld + col;
    for (int c0 = c_beg; c0 < c_end; c0 += 32) {
      if (c0 >= ui.rows) break;
      uint32_t r[32];
      tmem_ld32(d_tmem + tile * N + c0, r);
      tmem_wait_ld();
      if (p.y_bf16) {   // wide token tiles: y rows in BF16, as the reference's wide-tile build keeps them
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c0 + j < ui.rows) outb[static_cast<size_t>(c0 + j) * pp.out_ld] = __float2bfloat16_rn(__uint_as_float(r[j]) * osc);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c0 + j < ui.rows) outp[static_cast<size_t>(c0 + j) * pp.out_ld] = __uint_as_float(r[j]) * osc;
      }
    }
  }
}

// Folded combine (phase 1, fold): out[t] = bf16( sum over the token's local slots, in slot order, of
// w[t,s] * norm_s * y[inv[t,s]] ), norm_s = rsqrt(mean(y^2) + eps) with the post-expert norm, else 1
// (muse_moe_w4a16/cuda/moe.cu:2604-2766). Run by all threads of the CTA that retired the token's
// last base unit, after its own units are done. The rows come from other CTAs: they are read with
// L2 loads after the ticket that ordered them. Sums of squares: per-thread partials in a fixed column
// order, a fixed shuffle tree, then the warp partials in warp order. Plain loops on purpose (compact
// code: this runs once, from a cold instruction cache, at the very end of a one-token step).
struct FoldScratch {
  float red[GEMM_THREADS / 32][MAX_TOP_K];
  float wgt[MAX_TOP_K];
  int q[MAX_TOP_K];
  int nv;
};

__device__ __noinline__ void fold_combine_token(const GemmParams& p, int t, FoldScratch& fs) {
  constexpr int NW = GEMM_THREADS / 32;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = p.ph[1].out_ld, k = p.top_k, n4 = H / 4;
  const float* y = static_cast<const float*>(p.ph[1].outp);
  if (warp == 0) {   // lane s takes slot s; a ballot squeezes out the slots without a local expert, keeping their order
    const int qq = lane < k ? __ldcg(p.inv + t * k + lane) : -1;
    const float w = lane < k ? __ldcg(p.tw + t * k + lane) : 0.f;
    const unsigned have = __ballot_sync(0xffffffffu, qq >= 0);
    if (qq >= 0) {
      const int at = __popc(have & ((1u << lane) - 1u));
      fs.q[at] = qq;
      fs.wgt[at] = w;
    }
    if (lane == 0) fs.nv = __popc(have);
  }
  __syncthreads();
  const int nv = fs.nv;
  if (p.post_norm_w != nullptr) {
#pragma unroll 1
    for (int s = 0; s < nv; ++s) {
      const float4* row = reinterpret_cast<const float4*>(y + static_cast<size_t>(fs.q[s]) * H);
      float ss = 0.f;
#pragma unroll 1
      for (int i = tid; i < n4; i += GEMM_THREADS) {
        const float4 f = __ldcg(row + i);
        ss += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) fs.red[warp][s] = ss;
    }
    __syncthreads();
    if (tid < nv) {
      float tot = 0.f;
#pragma unroll 1
      for (int w = 0; w < NW; ++w) tot += fs.red[w][tid];  // fixed order
      fs.wgt[tid] *= rsqrtf(tot / static_cast<float>(H) + p.eps);
    }
    __syncthreads();
  }
#pragma unroll 1
  for (int i = tid; i < n4; i += GEMM_THREADS) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int s = 0; s < nv; ++s) {  // slot order
      const float4 f = __ldcg(reinterpret_cast<const float4*>(y + static_cast<size_t>(fs.q[s]) * H) + i);
      const float w = fs.wgt[s];
      acc.x += f.x * w; acc.y += f.y * w; acc.z += f.z * w; acc.w += f.w * w;
    }
    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p.out + static_cast<size_t>(t) * H + static_cast<size_t>(i) * 4) = pk;
  }
  __syncthreads();  // the scratch is reused by the next token
}

// Bounded wait until a grid-wide counter has reached `target` (MODE 2). Called by one lane.
__device__ __forceinline__ bool grid_counter_wait(const unsigned int* ctr, unsigned int target, volatile int* abort_word) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t polls = 0;
  while (true) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    if (v >= target) return true;
    __nanosleep(64);
    if ((++polls & 15u) == 0u) {
      if (*abort_word != 0) return false;
      if (globaltimer_ns() - t0 > MSK_WAIT_LIMIT_NS) {
        *abort_word = 1;
        return false;
      }
    }
  }
}

template <int N, int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1) moe_gemm_kernel(const __grid_constant__ GemmParams p) {
  using C = GemmCfg<N>;
  constexpr int NST = C::NST;
  constexpr int NSLOT = C::NSLOT;
  constexpr int NDBUF = C::NDBUF;
  constexpr int PH_FIRST = MODE == 1 ? 1 : 0, PH_LAST = MODE == 0 ? 0 : 1;
  constexpr bool FUSED = MODE == 2;
  constexpr bool TMA_B = C::TMA_B;
  static_assert(!(FUSED && (TMA_B || NDBUF == 1)), "the one-launch mode is built for the narrow token tiles");
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* ring = smem;                                        // NST x [tile g0 | tile g1 | B]
  GemmCtrl& ctl = *reinterpret_cast<GemmCtrl*>(smem + NST * C::STAGE_BYTES + C::LUT_BYTES);
  int* tile_start = reinterpret_cast<int*>(smem + NST * C::STAGE_BYTES + C::LUT_BYTES + C::CTRL_BYTES);
  int* cnt_s = tile_start + C::TABLE_INTS;
  int* off_s = cnt_s + C::TABLE_INTS;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool routed_here = PH_FIRST == 0 && p.route != 0;
  const bool fold = PH_LAST == 1 && p.fold != 0;
  const unsigned int n_ctas = gridDim.x;

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
    ctl.last_flag[0] = ctl.last_flag[1] = 0;
    ctl.fin_n = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  // Programmatic dependent launch: everything above ran while the previous kernel was still
  // draining. What a launch may read before the previous grid has completed:
  //  * MODE 0 behind a sort kernel (route == 0) reads that kernel's tables next, so it waits here.
  //  * MODE 0 that routes itself (route != 0) is launched behind the kernel that makes the F16 copy
  //    of the token rows. That kernel triggers its dependents only after its own wait, so whatever
  //    precedes it (the producer of logits / ids) has completed: routing starts at once, and only
  //    the activation gather waits (for the F16 rows).
  //  * MODE 1 is launched behind MODE 0, which triggers its dependents only once the tables are
  //    final (written by its CTA 0, or by the sort kernel it waited for): only the activation gather
  //    (inter rows) and the epilogue wait, and the weight stream, dequant and TMEM ring of the down
  //    GEMM fill up during the tail of the gate/up GEMM.
  //  * MODE 2 is the whole step: it reads its inputs next, so it waits here.
  if ((MODE == 0 && p.route == 0) || FUSED) pdl_wait();
  if (FUSED) {
    // F16 copy of the token rows, a slice per CTA; the gather warps wait for all slices (stage 1 of
    // the grid counter) before their first read
    const int n8 = p.T * (p.ph[0].K / 8);
    const uint4* src = reinterpret_cast<const uint4*>(p.x_bf16);
    uint4* dst = reinterpret_cast<uint4*>(const_cast<void*>(p.ph[0].act));
    for (int i = static_cast<int>(blockIdx.x) * GEMM_THREADS + tid; i < n8; i += static_cast<int>(n_ctas) * GEMM_THREADS) {
      const uint4 v = src[i];
      dst[i] = make_uint4(bf16x2_to_f16x2(v.x), bf16x2_to_f16x2(v.y), bf16x2_to_f16x2(v.z), bf16x2_to_f16x2(v.w));
    }
    __threadfence();
    if (tid == 0) MSK_TR(TR_CONVERTED);
  }
  if (routed_here) {
    // top-k (route 1) or the given ids (route 2), then the stable sort, redundantly in every CTA; the
    // scratch lives in the ring, which nothing has written yet
    SmallSortScratch& sc = *reinterpret_cast<SmallSortScratch*>(ring);
    const int n_entries = p.T * p.top_k;
    if (p.route == 1 && p.T * p.E <= SMALL_RANK_MAX_PAIRS && p.T * p.E * p.E <= SMALL_RANK_MAX_COMPARES) {
      route_by_rank_cta(sc, p.logits, p.bias, p.T, p.E, p.top_k, p.mode, p.route_scale);
    } else if (p.route == 1) {
      for (int t = warp; t < p.T; t += GEMM_THREADS / 32)
        route_token_compact(p.logits + static_cast<size_t>(t) * p.E, p.bias, sc.key[warp], sc.raw[warp],
                            sc.ids + t * p.top_k, sc.tw + t * p.top_k, p.E, p.top_k, p.mode, p.route_scale, lane);
    } else {
      for (int i = tid; i < n_entries; i += GEMM_THREADS) sc.ids[i] = p.ids_in[i];
    }
    __syncthreads();
    if (tid == 0) MSK_TR(TR_TOPK);
    const bool writer = blockIdx.x == 0;
    if (writer && p.route == 1) {
      for (int i = tid; i < n_entries; i += GEMM_THREADS) {
        p.ids_out[i] = sc.ids[i];
        p.tw_out[i] = sc.tw[i];
      }
    }
    sort_small_cta(sc, n_entries, p.lo, p.nloc, cnt_s, off_s, ctl.perm8, writer || FUSED, p.cnt, p.off, p.perm, p.inv);
    if (writer) __threadfence();  // the tables are in global memory before the dependent grid is let go
    fence_proxy_async_smem();     // the ring is handed to the bulk copies
    __syncthreads();
    if (tid == 0) MSK_TR(TR_ROUTED);
  }
  pdl_launch_dependents();
  if (warp == 2) {  // exclusive prefix of per-expert tile counts
    int carry = 0;
    for (int base = 0; base < p.nloc; base += 32) {
      const int e = base + lane;
      int cn = 0;
      if (e < p.nloc) {
        cn = routed_here ? cnt_s[e] : __ldcg(p.cnt + e);
        if (!routed_here) cnt_s[e] = cn;
      }
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
  if (warp == 3 && !routed_here) {  // off[] copy, in parallel with the scan above
    for (int e = lane; e <= p.nloc; e += 32) off_s[e] = __ldcg(p.off + e);
  }
  if (fold && warp >= 4 && warp < 4 + SMALL_SORT_WARPS) {
    // the entry index of every sorted row and each token's number of local routes. In MODE 2 this CTA
    // has just sorted: inv is its own write to global memory; in MODE 1 it is the previous grid's.
    const int i = (warp - 4) * 32 + lane;
    const int n_entries = p.T * p.top_k;
    if (!FUSED) {
      const int qq = i < n_entries ? __ldcg(p.inv + i) : -1;
      if (qq >= 0) ctl.perm8[qq] = static_cast<uint8_t>(i);
    }
    if (i < p.T) {
      int kl = 0;
      if (FUSED) {   // the ids this CTA has just sorted are still in the scratch (nothing has written the ring yet)
        const SmallSortScratch& sc = *reinterpret_cast<const SmallSortScratch*>(ring);
        for (int s = 0; s < p.top_k; ++s) kl += local_expert(sc.ids[i * p.top_k + s], p.lo, p.nloc) >= 0 ? 1 : 0;
      } else {
        for (int s = 0; s < p.top_k; ++s) kl += __ldcg(p.inv + i * p.top_k + s) >= 0 ? 1 : 0;
      }
      ctl.klocal[i] = static_cast<uint8_t>(kl);
      // a token without any local route is nobody's to finish: its output row is zero
      if (kl == 0 && static_cast<int>(blockIdx.x) == i % static_cast<int>(n_ctas)) {
        uint4* orow = reinterpret_cast<uint4*>(p.out + static_cast<size_t>(i) * p.ph[1].out_ld);
        for (int j = 0; j < p.ph[1].out_ld / 8; ++j) orow[j] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (FUSED && tid == 0) atomicAdd(p.grid_bar, 1u);  // this CTA's slice of the F16 rows is in memory

  const uint32_t tmem = ctl.tmem_base;
  if (tid == 0) MSK_TR(TR_SETUP);
  const int iter_mode = (N < 128 && p.flat) ? 1 : 0;
  // Down launch behind a gate/up launch with the per-tile hand-over: its CTAs start as the gate/up CTAs
  // leave, in block order, so the last blocks start on the SMs whose gate/up CTA held one unit more than
  // the others. They are dealt fewer down units, the way the one-launch kernel deals its second phase
  // (phase1_skew), with the block order reversed so that "heavy" means "started last". Only the balance
  // depends on that order, not the result.
  const bool chained_skew = MODE == 1 && p.handover != 0;
  const int deal_index = chained_skew ? static_cast<int>(n_ctas) - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
  volatile int* abortw = &ctl.abort_word;
#define MSK_WAIT(bar, par, ab) (N >= 64 ? mbar_wait_inline((bar), (par), (ab)) : mbar_wait((bar), (par), (ab)))
#define MSK_PHASES for (int phase = PH_FIRST; phase <= PH_LAST; ++phase)
#define MSK_PHASE_SETUP                                                                                           \
  const PhaseParams& pp = p.ph[phase];                                                                            \
  const int nst_total = pp.K / KS;                                                                                \
  const int n_base = ctl.n_tiles * pp.n_pairs;                                                                    \
  int heavy_ = 0, skip_ = 0;                                                                                     \
  if ((FUSED || chained_skew) && phase == 1) phase1_skew(ctl.n_tiles * p.ph[0].n_pairs, p.ph[0].K / KS, nst_total, static_cast<int>(n_ctas), heavy_, skip_); \
  PieceIter pieces = make_piece_iter(iter_mode, n_base, nst_total, deal_index, static_cast<int>(n_ctas), heavy_, skip_); \
  const int tail_base = pieces.tail_base;                                                                         \
  (void)tail_base;                                                                                                \
  int base, ks0, ks1;                                                                                             \
  (void)n_base

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
#undef MSK_PHASES
#undef MSK_WAIT
#undef MSK_PHASE_SETUP

  // -------------------------------------------------------------- teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  // With the per-tile hand-over nothing in this kernel has waited for the gate/up grid as a whole (all of
  // its units are done, or the tiles would not have been released; its CTAs may still be leaving). Waiting
  // here, where it costs nothing, keeps "this grid has completed" implying "the one before has" for
  // whatever follows in the stream.
  if (MODE == 1 && p.handover) pdl_wait();
  if (fold && p.fold == 1 && ctl.abort_word == 0) {
    // the tokens whose last base unit this CTA retired (the ring is free by now: scratch for the sums)
    FoldScratch& fs = *reinterpret_cast<FoldScratch*>(ring);
    const int nf = ctl.fin_n;
#pragma unroll 1
    for (int j = 0; j < nf; ++j) fold_combine_token(p, ctl.fin_tok[j], fs);
    if (tid == 0) MSK_TR(TR_FOLD_END);
  }
  if (tid == 0) MSK_TR(TR_END);
  if (FUSED && tid == 0 && ctl.abort_word == 0) {
    // the last CTA to leave puts the grid counters back to zero for the next launch
    const unsigned int old = atomicAdd(p.grid_bar + 1, 1u);
    if (old == n_ctas - 1u) {
      atomicExch(p.grid_bar, 0u);
      atomicExch(p.grid_bar + 1, 0u);
    }
  }
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
