// The whole routed-expert step for up to 8 tokens in ONE cooperative launch.
//
// With so few tokens the step is a pure weight stream (a token touches top_k experts, 18.9 MB
// each at H4096/I1536) and the chain of launches of the general path costs more than the
// stream itself. Here one persistent grid (one CTA per SM) does
//   phase 0  routing (optional) and the stable sort by expert, redundantly in every CTA, as the
//            reference does (muse_moe_w4a16/cuda/moe.cu:315-433);
//   phase 1  gate/up products: the packed tiles of the touched experts form one flat list of
//            "stage tiles" (128 weight rows x 256 K, 18 KB, contiguous in memory); CTA c streams
//            the c-th equal share of the list, so every SM reads the same number of bytes;
//   phase 2  SwiGLU of the summed pieces, then the down products the same way;
//   phase 3  scale, post-expert norm and the top-k weighted sum in slot order.
// Phases are separated by a grid barrier (bounded wait). A CTA's share cuts through K, so what
// it produces are partial sums ("pieces"); the consumer adds the pieces of an output element in
// a fixed order that depends only on the shapes and the grid, never on timing.
//
// Data flow: warp 16 is the producer: one lane copies this CTA's stage tiles, in order, into a
// ring of shared-memory slots (one 18 KB bulk copy per tile, completing on an mbarrier; the
// second stream's first tiles are already landing while the grid barrier between the streams is
// crossed). The 16 consumer warps work in two groups of 8; group i takes every second stage tile
// and its 8 warps take 16 weight rows each.
//
// Math: lane (g, q) (g = lane / 4, q = lane % 4) of a consumer warp fetches with ldmatrix, for each
// of the tile's 8 chunks, the 8 codes K = 32 c + 8 q .. + 7 of rows g and g + 8 (a matrix = 8
// rows x one 16-byte chunk = 128 contiguous bytes of the packed layout: no bank conflicts),
// decodes them with the hardware converts (layout.cuh) straight into the A fragments of
// mma.sync.m16n8k16 (F16 x F16 -> FP32, the same exact products and FP32 accumulation as the
// tcgen05 path); the up to 8 token rows of the expert are the B fragment's 8 columns. The K
// order inside an MMA is whatever the lanes hold, so the activations are laid out in shared
// memory in the matching permuted order and a lane reads its B fragment with one conflict-free
// 8-byte load.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "layout.cuh"
#include "ptx.cuh"
#include "route_sort.cuh"

namespace msk {

#ifndef MSK_ST_GROUPS
#define MSK_ST_GROUPS 2
#endif
constexpr int ST_GROUPS = MSK_ST_GROUPS;      // groups of 8 consumer warps; group i takes every ST_GROUPS-th stage tile
constexpr int ST_WARPS = 8 * ST_GROUPS;       // consumer warps; one more warp feeds the weight ring
constexpr int ST_MAX_TOKENS = 8;   // columns of one MMA: rows per expert never exceed the tokens
constexpr int ST_MAX_ROWS = 64;    // routed rows (tokens x top_k)

struct SmallParams {
  const uint8_t* w13; const uint8_t* w2;
  const float* gs13; const float* gs2;
  const __nv_bfloat16* post_norm_w;
  const __nv_bfloat16* x;
  const int32_t* ids_in; const float* tw_in;      // given routing, or
  const float* logits; const float* bias;         // routing from logits (ids_out / tw_out receive it)
  int32_t* ids_out; float* tw_out;
  __nv_bfloat16* out;
  int32_t* cnt; int32_t* off; int32_t* perm; int32_t* inv;   // the general path's tables (CTA 0 writes them)
  __half* inter; float* y;                                    // [R, I] and [R, H], as the general path leaves them
  float* part1; float* part2;                                 // pieces: [R][P1][2 I] and [R][P2][H]
  float* row_w;                                               // [R] top-k weight x norm of a sorted row
  unsigned int* bar;                                          // grid barrier: arrivals, generation
  int32_t* tickets;                                           // per token: rows finished in phase 3
  int32_t* status;
  unsigned long long* trace;                                  // optional: 16 time stamps per CTA
  int H, I, E, lo, nloc, k, T, mode, P1, P2;
  int slots;                                                  // weight ring slots (a multiple of ST_GROUPS)
  float route_scale, eps;
};

struct SmallTables {
  int32_t ids[ST_MAX_ROWS];
  float tw[ST_MAX_ROWS];
  int32_t s_exp[ST_MAX_ROWS];   // local expert of sorted row p
  int32_t perm[ST_MAX_ROWS];    // entry (token * k + slot) of sorted row p
  int32_t inv[ST_MAX_ROWS];     // sorted row of entry i, -1 without a local expert
  int32_t u_exp[ST_MAX_ROWS];   // touched experts in ascending order
  int32_t u_off[ST_MAX_ROWS + 1];
  int U, R;
  int flag;
  float wsum[ST_WARPS];
};

__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t ldg_stream_u16(const void* p) {
  uint16_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}

// Share c of a list of L items cut into G <= L equal shares: [c L / G, (c + 1) L / G).
__device__ __forceinline__ long long share_begin(long long c, long long L, int G) { return c * L / G; }
// The share that holds item x.
__device__ __forceinline__ int share_of(long long x, long long L, int G) {
  return static_cast<int>(((x + 1) * G - 1) / L);
}

// Grid barrier with a generation word; self-resetting, so it needs no host work between launches.
// Returns false when the wait ran out (one second): the caller leaves the kernel.
__device__ __forceinline__ bool grid_barrier(unsigned int* bar, int32_t* status, SmallTables& tb) {
  asm volatile("bar.sync 1, %0;" ::"n"(32 * ST_WARPS) : "memory");   // the consumer threads; the producer warp streams on
  if (threadIdx.x == 0) {
    volatile unsigned int* gen = bar + 1;
    const unsigned int my_gen = *gen;   // cannot advance before this CTA has arrived
    __threadfence();
    const unsigned int old = atomicAdd(bar, 1u);
    int ok = 1;
    if (old == gridDim.x - 1) {
      atomicExch(bar, 0u);
      __threadfence();
      atomicAdd(bar + 1, 1u);
    } else {
      const uint64_t t0 = globaltimer_ns();
      uint32_t polls = 0;
      while (*gen == my_gen) {
        if ((++polls & 255u) == 0 && globaltimer_ns() - t0 > 1000000000ull) { ok = 0; break; }
      }
      if (!ok) atomicExch(status, 2);
    }
    __threadfence();
    tb.flag = ok;
  }
  asm volatile("bar.sync 1, %0;" ::"n"(32 * ST_WARPS) : "memory");
  return tb.flag != 0;
}

// Group `grp` takes the stage tiles whose distance from the share's begin is grp modulo ST_GROUPS;
// the first such tile at or after distance d is d + group_offset(grp, d).
__device__ __forceinline__ int group_offset(int grp, int d) { return ((grp - d) % ST_GROUPS + ST_GROUPS) % ST_GROUPS; }

// Which piece slots of flat tile TI hold data: slot ST_GROUPS (c - c0) + group for every share c that
// overlaps the tile's stages [TI nst, (TI + 1) nst) and every warp group that has a stage in the overlap. Bit i of the result = slot i.
__device__ __forceinline__ unsigned long long piece_mask(int TI, int nst, int L, int G) {
  const int s0 = TI * nst, s1 = s0 + nst;
  const int c0 = share_of(s0, L, G), c1 = share_of(s1 - 1, L, G);
  unsigned long long m = 0ull;
  for (int c = c0; c <= c1; ++c) {
    const int a = static_cast<int>(share_begin(c, L, G)), b = static_cast<int>(share_begin(c + 1, L, G));
    const int lo = max(a, s0), hi = min(b, s1);
    for (int grp = 0; grp < ST_GROUPS; ++grp) {
      const int first = lo + group_offset(grp, lo - a);
      if (first < hi) m |= 1ull << (ST_GROUPS * (c - c0) + grp);
    }
  }
  return m;
}

// Sum of the pieces of four neighbouring output elements (one tile, so one mask), in slot order.
// `p` points at slot 0 of the first element. The loads of eight slots are issued together; an
// absent slot adds an exact zero.
__device__ __forceinline__ float4 sum_pieces4(const float* p, int ld, unsigned long long mask) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  while (mask) {
    float4 v[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      v[s] = make_float4(0.f, 0.f, 0.f, 0.f);
      if ((mask >> s) & 1ull) v[s] = __ldcg(reinterpret_cast<const float4*>(p + static_cast<size_t>(s) * ld));
    }
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      acc.x += v[s].x; acc.y += v[s].y; acc.z += v[s].z; acc.w += v[s].w;
    }
    mask >>= 8;
    p += static_cast<size_t>(8) * ld;
  }
  return acc;
}

// ---- the weight ring in shared memory
// One slot holds one stage tile exactly as it lies in global memory (one bulk copy of 18 KB;
// nine 2 KB copies into a padded layout were measured at half the rate).
constexpr int ST_SLOT_BYTES = TILE_BYTES;
constexpr int ST_MAX_SLOTS = 8;
constexpr int ST_CONSUMERS = 32 * ST_WARPS;                         // the warp after them is the producer

struct SmallCtl {
  uint64_t full[ST_MAX_SLOTS];
  uint64_t empty[ST_MAX_SLOTS];
  int abort_word;
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(ST_CONSUMERS) : "memory"); }

__device__ __forceinline__ uint4 lds128(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
  return v;
}
// Four 8 x 16-byte matrices: lanes 8 i .. 8 i + 7 give the row addresses of matrix i; lane
// (g, q) receives bytes [4 q, 4 q + 4) of row g of each matrix.
__device__ __forceinline__ void ldmatrix_x4(const uint8_t* row_addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(row_addr)));
}

// What a lane holds of one stage tile (16 weight rows x 256 K of its warp): for each of the 8
// chunks, the 8 codes K = 32 c + 8 q .. + 7 of rows g and g + 8 (one word each, fetched with
// ldmatrix: a matrix = 8 rows x one chunk, 128 contiguous bytes, no bank conflict), and the
// rows' 16 scale bytes.
struct StageRegs {
  uint32_t w[4][4];   // [chunk pair][chunk 2 p row g, chunk 2 p row g + 8, chunk 2 p + 1 row g, chunk 2 p + 1 row g + 8]
  uint4 sf[2];        // scale bytes of rows g and g + 8
};

__device__ __forceinline__ void read_stage(StageRegs& s, const uint8_t* slot, int slab, int lane) {
  // lane l addresses row (l & 7) of matrix (l >> 3): matrix 0/1 = chunk 2 p, rows 0-7 / 8-15 of the
  // slab; matrix 2/3 = chunk 2 p + 1
  const int m = lane >> 3;
  const uint8_t* base = slot + (((m >> 1) * 128) + slab * 16 + (m & 1) * 8 + (lane & 7)) * 16;
#pragma unroll
  for (int pr = 0; pr < 4; ++pr) ldmatrix_x4(base + pr * (2 * 128 * 16), s.w[pr]);
  const int g = lane >> 2;
  const uint8_t* sf = slot + TILE_CODE_BYTES + (slab * 16 + g) * 16;
  s.sf[0] = lds128(sf);
  s.sf[1] = lds128(sf + 8 * 16);
}

// Position, inside one 256-K stage, of element k of an activation row in shared memory: MMA step
// (chunk c, half t) reads the 4 elements K = 32 c + 8 q + 4 t .. + 3 of lane q, the 4 lanes side
// by side.
__device__ __forceinline__ int b_pos(int k_in_stage) {
  const int c = k_in_stage >> 5, q = (k_in_stage >> 3) & 3, t = (k_in_stage >> 2) & 1, i = k_in_stage & 3;
  return (((c * 2 + t) * 4) + q) * 4 + i;
}

// 16 rows x 256 K of weights against the 8 activation rows at `brow` (this lane's row g of the
// stage, permuted order): 16 MMAs on two accumulation chains. sel0 / sel1: byte selectors that
// duplicate this lane's scale byte of an even / odd chunk (byte 2 c + q / 2 of the scale row).
__device__ __forceinline__ void consume_stage(const StageRegs& s, const uint8_t* brow, int q, uint32_t sel0,
                                              uint32_t sel1, float (&acc)[2][4]) {
  const uint32_t sfa[4] = {s.sf[0].x, s.sf[0].y, s.sf[0].z, s.sf[0].w};
  const uint32_t sfb[4] = {s.sf[1].x, s.sf[1].y, s.sf[1].z, s.sf[1].w};
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t sel = (c & 1) ? sel1 : sel0;
    const uint32_t sa = cvt_e4m3x2_f16(static_cast<uint16_t>(prmt(sfa[c >> 1], 0u, sel)));
    const uint32_t sb = cvt_e4m3x2_f16(static_cast<uint16_t>(prmt(sfb[c >> 1], 0u, sel)));
    uint32_t a[4], b[4];
    cvt_e2m1x8_f16(s.w[c >> 1][(c & 1) * 2], a[0], a[1], a[2], a[3]);
    cvt_e2m1x8_f16(s.w[c >> 1][(c & 1) * 2 + 1], b[0], b[1], b[2], b[3]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      a[i] = hmul2_f16(a[i], sa);
      b[i] = hmul2_f16(b[i], sb);
    }
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const uint2 x = *reinterpret_cast<const uint2*>(brow + ((c * 2 + t) * 4 + q) * 8);
      mma_m16n8k16(acc[t], a[2 * t], b[2 * t], a[2 * t + 1], b[2 * t + 1], x.x, x.y);
    }
  }
}

// Shapes of one GEMM phase. PHASE 0: weights w13, K = H, pieces to part1 (columns: gate [0, I),
// up [I, 2 I)). PHASE 1: weights w2, K = I, pieces to part2.
struct PhaseShape {
  int K, tiles, nst, per_exp, L, G, a, b;
};
__device__ __forceinline__ PhaseShape phase_shape(const SmallParams& p, int U, int phase) {
  PhaseShape s;
  s.K = phase == 0 ? p.H : p.I;
  s.tiles = phase == 0 ? 2 * p.I / 128 : p.H / 128;
  s.nst = s.K / KS;
  s.per_exp = s.tiles * s.nst;
  s.L = U * s.per_exp;
  s.G = min(static_cast<int>(gridDim.x), s.L);   // shares are never empty: CTAs past L idle
  const int cta = blockIdx.x;
  s.a = cta < s.G ? static_cast<int>(share_begin(cta, s.L, s.G)) : 0;
  s.b = cta < s.G ? static_cast<int>(share_begin(cta + 1, s.L, s.G)) : 0;
  return s;
}

// Producer (one lane): this CTA's share of both phases, in order, through the ring. `it` counts
// the stage tiles since the kernel began; slot = it % slots. The weights do not depend on the
// first phase's results, so the second phase's tiles are already landing while the grid barrier
// between the phases is being crossed.
__device__ void produce(const SmallParams& p, const SmallTables& tb, SmallCtl& ctl, uint8_t* ring, int slots) {
  const uint64_t pol = policy_evict_first();
  int it = 0;
  for (int phase = 0; phase < 2; ++phase) {
    const PhaseShape s = phase_shape(p, tb.U, phase);
    const uint8_t* w = phase == 0 ? p.w13 : p.w2;
    for (int idx = s.a; idx < s.b; ++idx, ++it) {
      const int slot = it % slots, pass = it / slots;
      if (!mbar_wait(&ctl.empty[slot], (pass & 1) ^ 1, &ctl.abort_word)) return;
      const int u = idx / s.per_exp;
      const uint8_t* tile = w + (static_cast<size_t>(tb.u_exp[u]) * s.per_exp + (idx - u * s.per_exp)) * TILE_BYTES;
      uint8_t* dst = ring + static_cast<size_t>(slot) * ST_SLOT_BYTES;
      mbar_arrive_expect_tx(&ctl.full[slot], TILE_BYTES);
      bulk_g2s(dst, tile, TILE_BYTES, &ctl.full[slot], pol);
    }
  }
}

// Consumers (16 warps): one GEMM phase of this CTA's share. `it0` is the ordinal of the share's
// first stage tile in the ring (the producer counts the same way). `bs` is the activation buffer:
// 8 rows of K F16 in permuted order, row stride K * 2 + 32 bytes. After a failed wait (`ok`
// false) the control flow goes on, so every thread still meets every barrier, but nothing is read.
template <int PHASE>
__device__ void consume_phase(const SmallParams& p, SmallTables& tb, SmallCtl& ctl, const uint8_t* ring, int slots,
                              uint8_t* bs, unsigned long long* masks, int& it0, bool& ok) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, q = lane & 3;
  const int grp = warp >> 3, slab = warp & 7;
  const int cta = blockIdx.x;
  const PhaseShape s = phase_shape(p, tb.U, PHASE);
  const int K = s.K, nst = s.nst;
  const int P = PHASE == 0 ? p.P1 : p.P2;
  const int ld = PHASE == 0 ? 2 * p.I : p.H;
  float* part = PHASE == 0 ? p.part1 : p.part2;
  const int rs = K * 2 + 32;   // activation row stride in bytes
  const uint32_t sel0 = static_cast<uint32_t>(q >> 1) * 0x11u, sel1 = static_cast<uint32_t>(2 + (q >> 1)) * 0x11u;
  for (int sa = s.a; sa < s.b;) {
    const int u = sa / s.per_exp;
    const int sb = min(s.b, (u + 1) * s.per_exp);
    const int e = tb.u_exp[u], row0 = tb.u_off[u], cnt = tb.u_off[u + 1] - row0;
    consumer_sync();   // the previous segment's readers are done with the activation buffer
    if (PHASE == 0) {
      // token rows of this expert, BF16 -> F16, permuted; rows past cnt are zero
      const int groups = K / 8;
      for (int i = tid; i < ST_MAX_TOKENS * groups; i += ST_CONSUMERS) {
        const int n = i / groups, k8 = (i - n * groups) * 8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (n < cnt) {
          const int token = tb.perm[row0 + n] / p.k;
          v = *reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(token) * K + k8);
        }
        const int st = k8 / KS, kin = k8 - st * KS;
        uint8_t* dst = bs + n * rs + st * (KS * 2);
        *reinterpret_cast<uint2*>(dst + b_pos(kin) * 2) = make_uint2(bf16x2_to_f16x2(v.x), bf16x2_to_f16x2(v.y));
        *reinterpret_cast<uint2*>(dst + b_pos(kin + 4) * 2) = make_uint2(bf16x2_to_f16x2(v.z), bf16x2_to_f16x2(v.w));
      }
    } else {
      // inter = bf16(silu(gate) * up) of this expert's rows from the part1 pieces
      const int tiles1 = 2 * p.I / 128, nst1 = p.H / KS;
      const int L1 = tb.U * tiles1 * nst1;
      const int G1 = min(static_cast<int>(gridDim.x), L1);
      for (int i = tid; i < tiles1; i += ST_CONSUMERS) masks[i] = piece_mask(u * tiles1 + i, nst1, L1, G1);
      consumer_sync();
      const float gsc = p.gs13[e];
      const bool writer = sa == u * s.per_exp;   // the CTA that starts this expert also stores inter
      for (int i = tid; i < ST_MAX_TOKENS * (K / 4); i += ST_CONSUMERS) {
        const int n = i / (K / 4), col = (i - n * (K / 4)) * 4;
        float4 ga = make_float4(0.f, 0.f, 0.f, 0.f), up = ga;
        if (n < cnt) {
          const float* pr = p.part1 + static_cast<size_t>(row0 + n) * p.P1 * (2 * p.I);
          const int jt = col >> 7;
          ga = sum_pieces4(pr + col, 2 * p.I, masks[2 * jt]);
          up = sum_pieces4(pr + p.I + col, 2 * p.I, masks[2 * jt + 1]);
        }
        __half h[4];
        h[0] = inter_value(silu_f(ga.x * gsc) * (up.x * gsc));
        h[1] = inter_value(silu_f(ga.y * gsc) * (up.y * gsc));
        h[2] = inter_value(silu_f(ga.z * gsc) * (up.z * gsc));
        h[3] = inter_value(silu_f(ga.w * gsc) * (up.w * gsc));
        const int st = col / KS, kin = col - st * KS;
        const uint2 pk = *reinterpret_cast<const uint2*>(h);
        *reinterpret_cast<uint2*>(bs + n * rs + st * (KS * 2) + b_pos(kin) * 2) = pk;
        if (writer && n < cnt) *reinterpret_cast<uint2*>(p.inter + static_cast<size_t>(row0 + n) * K + col) = pk;
      }
    }
    consumer_sync();
    const uint8_t* brow = bs + g * rs;
    const int first = sa + group_offset(grp, sa - s.a);
    int TI = first / nst, st = first - TI * nst;
    const int ord0 = it0 + (first - s.a);
    int slot = ord0 % slots, pass = ord0 / slots;
    int cur_tile = -1;
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    auto flush = [&](int tile) {
      const int piece = ST_GROUPS * (cta - share_of(tile * nst, s.L, s.G)) + grp;
      const int tt = tile - u * s.tiles;
      const int col = (PHASE == 0 ? ((tt & 1) * p.I + (tt >> 1) * 128) : tt * 128) + slab * 16 + g;
      const int n0 = 2 * q, n1 = 2 * q + 1;
      if (n0 < cnt) {
        float* d = part + (static_cast<size_t>(row0 + n0) * P + piece) * ld + col;
        d[0] = acc[0][0] + acc[1][0];
        d[8] = acc[0][2] + acc[1][2];
      }
      if (n1 < cnt) {
        float* d = part + (static_cast<size_t>(row0 + n1) * P + piece) * ld + col;
        d[0] = acc[0][1] + acc[1][1];
        d[8] = acc[0][3] + acc[1][3];
      }
    };
    for (int idx = first; idx < sb; idx += ST_GROUPS) {
      if (TI != cur_tile) {
        if (cur_tile >= 0 && ok) flush(cur_tile);
        cur_tile = TI;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[0][i] = acc[1][i] = 0.f;
      }
      StageRegs r;
      if (ok) ok = mbar_wait(&ctl.full[slot], pass & 1, &ctl.abort_word);
      if (ok) read_stage(r, ring + static_cast<size_t>(slot) * ST_SLOT_BYTES, slab, lane);
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.empty[slot]);   // the slot's bytes are in registers
      if (ok) consume_stage(r, brow + st * (KS * 2), q, sel0, sel1, acc);
      st += ST_GROUPS;
      while (st >= nst) { st -= nst; ++TI; }
      slot += ST_GROUPS;
      if (slot >= slots) { slot -= slots; ++pass; }
    }
    if (cur_tile >= 0 && ok) flush(cur_tile);
    sa = sb;
  }
  it0 += s.b - s.a;
}

// Shared memory: tables | masks | ring control | activation buffer | weight ring.
constexpr int ST_OFF_MASKS = 2048;
constexpr int ST_OFF_CTL = ST_OFF_MASKS + 512;
constexpr int ST_OFF_ACT = ST_OFF_CTL + 256;
constexpr int ST_THREADS_ALL = ST_CONSUMERS + 32;

__global__ void __launch_bounds__(ST_THREADS_ALL, 1) moe_small_kernel(const __grid_constant__ SmallParams p) {
  extern __shared__ __align__(128) uint8_t st_smem[];
  SmallTables& tb = *reinterpret_cast<SmallTables*>(st_smem);
  unsigned long long* masks = reinterpret_cast<unsigned long long*>(st_smem + ST_OFF_MASKS);   // 64 entries
  SmallCtl& ctl = *reinterpret_cast<SmallCtl*>(st_smem + ST_OFF_CTL);
  uint8_t* bs = st_smem + ST_OFF_ACT;
  uint8_t* ring = bs + ST_MAX_TOKENS * (max(p.H, p.I) * 2 + 32);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  const int n_entries = p.T * p.k;
  auto stamp = [&](int i) {
    if (p.trace != nullptr && tid == 0) p.trace[static_cast<size_t>(cta) * 16 + i] = globaltimer_ns();
  };
  stamp(0);
  if (tid == 0) {
    for (int i = 0; i < p.slots; ++i) {
      mbar_init(&ctl.full[i], 1);
      mbar_init(&ctl.empty[i], 8);   // the eight consumer warps of a stage tile
    }
    ctl.abort_word = 0;
    fence_mbar_init();
  }

  // ---- phase 0: routing and the stable sort by local expert, the same in every CTA
  if (p.logits != nullptr) {
    if (warp < p.T)
      route_token_dispatch(p.logits + static_cast<size_t>(warp) * p.E, p.bias, tb.ids + warp * p.k, tb.tw + warp * p.k,
                           p.E, p.k, p.mode, p.route_scale, lane);
  } else if (tid < n_entries) {
    tb.ids[tid] = p.ids_in[tid];
    tb.tw[tid] = p.tw_in[tid];
  }
  __syncthreads();
  if (tid < n_entries) {
    const int e = local_expert(tb.ids[tid], p.lo, p.nloc);
    int pos = -1;
    if (e >= 0) {
      pos = 0;
      for (int j = 0; j < n_entries; ++j) {
        const int ej = local_expert(tb.ids[j], p.lo, p.nloc);
        if (ej >= 0 && (ej < e || (ej == e && j < tid))) ++pos;
      }
      tb.perm[pos] = tid;
      tb.s_exp[pos] = e;
    }
    tb.inv[tid] = pos;
  }
  __syncthreads();
  if (tid == 0) {
    int R = 0;
    for (int i = 0; i < n_entries; ++i) R += tb.inv[i] >= 0 ? 1 : 0;
    int U = 0;
    for (int r = 0; r < R; ++r) {
      if (r == 0 || tb.s_exp[r] != tb.s_exp[r - 1]) {
        tb.u_exp[U] = tb.s_exp[r];
        tb.u_off[U] = r;
        ++U;
      }
    }
    tb.u_off[U] = R;
    tb.U = U;
    tb.R = R;
  }
  __syncthreads();   // the last barrier the producer warp takes part in
  if (warp == ST_CONSUMERS / 32) {
    if (lane == 0) produce(p, tb, ctl, ring, p.slots);
    return;
  }
  const int R = tb.R;
  if (cta == 0) {   // the tables as the general path leaves them, and the routing result
    for (int e = tid; e <= p.nloc; e += ST_CONSUMERS) {
      int below = 0, same = 0;
      for (int r = 0; r < R; ++r) {
        below += tb.s_exp[r] < e ? 1 : 0;
        same += tb.s_exp[r] == e ? 1 : 0;
      }
      p.off[e] = below;
      if (e < p.nloc) p.cnt[e] = same;
    }
    if (tid < n_entries) {
      p.inv[tid] = tb.inv[tid];
      if (tid < R) p.perm[tid] = tb.perm[tid];
      if (p.logits != nullptr) {
        p.ids_out[tid] = tb.ids[tid];
        p.tw_out[tid] = tb.tw[tid];
      }
    }
  }

  // ---- phase 1 and 2: the two weight streams
  int it0 = 0;
  bool ok = true;
  stamp(1);
  consume_phase<0>(p, tb, ctl, ring, p.slots, bs, masks, it0, ok);
  stamp(2);
  if (!grid_barrier(p.bar, p.status, tb)) return;
  stamp(3);
  consume_phase<1>(p, tb, ctl, ring, p.slots, bs, masks, it0, ok);
  stamp(4);
  if (!grid_barrier(p.bar, p.status, tb)) return;
  stamp(5);
  if (ctl.abort_word != 0) {   // a wait on the weight ring ran out somewhere in this CTA
    if (tid == 0) atomicExch(p.status, 1);
    return;
  }

  // ---- phase 3: one CTA per routed row finishes y; the last one of a token sums its slots
  const int tiles2 = p.H / 128, nst2 = p.I / KS;
  const int L2 = tb.U * tiles2 * nst2;
  const int G2 = min(G, L2);
  for (int r = cta; r < R + p.T; r += G) {
    consumer_sync();   // tb.flag, tb.wsum and masks of the previous round are free
    if (r >= R) {      // a token without any local expert gets a zero row
      const int t = r - R;
      bool any = false;
      for (int s = 0; s < p.k; ++s) any |= tb.inv[t * p.k + s] >= 0;
      if (!any)
        for (int i = tid; i < p.H / 8; i += ST_CONSUMERS)
          *reinterpret_cast<uint4*>(p.out + static_cast<size_t>(t) * p.H + i * 8) = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const int entry = tb.perm[r], t = entry / p.k;
    const int e = tb.s_exp[r];
    int u = 0;
    while (tb.u_exp[u] != e) ++u;
    for (int i = tid; i < tiles2; i += ST_CONSUMERS) masks[i] = piece_mask(u * tiles2 + i, nst2, L2, G2);
    consumer_sync();
    const float gsc = p.gs2[e];
    const float* pr = p.part2 + static_cast<size_t>(r) * p.P2 * p.H;
    float ss = 0.f;
    for (int col = tid * 4; col < p.H; col += ST_CONSUMERS * 4) {
      float4 v = sum_pieces4(pr + col, p.H, masks[col >> 7]);
      float o0 = gsc, o1 = gsc, o2 = gsc, o3 = gsc;
      if (p.post_norm_w != nullptr) {
        const uint2 pw = *reinterpret_cast<const uint2*>(p.post_norm_w + col);
        o0 *= 1.0f + __uint_as_float(pw.x << 16); o1 *= 1.0f + __uint_as_float(pw.x & 0xFFFF0000u);
        o2 *= 1.0f + __uint_as_float(pw.y << 16); o3 *= 1.0f + __uint_as_float(pw.y & 0xFFFF0000u);
      }
      v.x *= o0; v.y *= o1; v.z *= o2; v.w *= o3;
      *reinterpret_cast<float4*>(p.y + static_cast<size_t>(r) * p.H + col) = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    float wgt = tb.tw[entry];
    if (p.post_norm_w != nullptr) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) tb.wsum[warp] = ss;
      consumer_sync();
      float tot = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < ST_WARPS; ++w2) tot += tb.wsum[w2];   // fixed order
      wgt *= rsqrtf(tot / static_cast<float>(p.H) + p.eps);
    }
    __threadfence();   // this row of y is visible before the ticket
    consumer_sync();
    if (tid == 0) {
      p.row_w[r] = wgt;
      int target = 0;
      for (int s = 0; s < p.k; ++s) target += tb.inv[t * p.k + s] >= 0 ? 1 : 0;
      __threadfence();
      const int old = atomicAdd(&p.tickets[t], 1);
      const int last = old == target - 1 ? 1 : 0;
      if (last) p.tickets[t] = 0;   // launch-ready again
      __threadfence();
      tb.flag = last;
    }
    consumer_sync();
    if (tb.flag) {
      // out[t] = bf16(sum over the token's slots, in slot order, of y * (weight * norm))
      for (int c4 = tid; c4 < p.H / 4; c4 += ST_CONSUMERS) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < p.k; ++s) {
          const int rr = tb.inv[t * p.k + s];
          if (rr < 0) continue;
          const float ws = __ldcg(p.row_w + rr);
          const float4 v = __ldcg(reinterpret_cast<const float4*>(p.y + static_cast<size_t>(rr) * p.H) + c4);
          acc.x += v.x * ws; acc.y += v.y * ws; acc.z += v.z * ws; acc.w += v.w * ws;
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&lo);
        pk.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p.out + static_cast<size_t>(t) * p.H + c4 * 4) = pk;
      }
    }
  }
  stamp(6);
}

}  // namespace msk
