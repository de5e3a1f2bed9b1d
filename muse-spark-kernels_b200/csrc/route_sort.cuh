// Routing kernels: FP32 router logits, top-k with its two score functions, and the
// stable counting sort of (token, slot) entries by local expert.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "layout.cuh"

namespace msk {

constexpr int SORT_THREADS = 1024;
constexpr int SORT_WARPS = SORT_THREADS / 32;
constexpr int MAX_LOCAL_EXPERTS = 256;
constexpr int MAX_EXPERTS = 512;
constexpr int MAX_TOP_K = 16;

// ------------------------------------------------------------------ router
// One block per (token, 8 experts): each warp owns one expert row and walks H with a
// fixed lane stride; the lane partials are combined by a fixed shuffle tree, so the
// sum order depends on H only (precedent: muse_decode_layer/cuda/router_fp32.cu:4-40).
__global__ void __launch_bounds__(256) router_logits_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const float* __restrict__ w, float* __restrict__ logits,
                                                            int H, int E) {
  const int t = blockIdx.x;
  const int e = blockIdx.y * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (e >= E) return;
  const __nv_bfloat16* xr = x + static_cast<size_t>(t) * H;
  const float* wr = w + static_cast<size_t>(e) * H;
  float acc = 0.f;
  for (int h = lane; h < H; h += 32) acc = fmaf(__bfloat162float(xr[h]), wr[h], acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) logits[static_cast<size_t>(t) * E + e] = acc;
}

// ------------------------------------------------------------------- top-k
// Monotone map float -> u32 (flip the sign bit of non-negatives, all bits of negatives),
// the transform the reference uses for its packed arg-max keys
// (muse_prefill_layer/cuda/prefill.cu:1655-1658, muse_decode_layer/py/07_link_chain.py:101-112).
__device__ __forceinline__ uint32_t orderable_u32(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One warp per token. key = orderable(score) << 32 | (0xFFFFFFFF - e): the largest key is the
// highest score, lowest index on ties. k rounds of warp arg-max, the winner is retired.
// mode 0: score = logit, weights = softmax over the k selected logits.
// mode 1: s = sigmoid(logit * scale), score = s + bias, weights = s / (sum s + 1e-15)
//         (muse_decode_layer/py/04_triton_kernels.py:541-552).
template <int PER>
__device__ __forceinline__ void route_one_token(const float* __restrict__ row, const float* __restrict__ bias,
                                                int32_t* __restrict__ ids_row, float* __restrict__ wts_row, int E, int k,
                                                int mode, float scale, int lane) {
  uint64_t key[PER];
  float raw[PER];  // the value the weight is formed from (logit or sigmoid score)
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = i * 32 + lane;
    key[i] = 0ull;
    raw[i] = 0.f;
    if (e < E) {
      const float l = row[e];
      float sel = l, r = l;
      if (mode == 1) {
        r = 1.0f / (1.0f + expf(-l * scale));
        sel = r + (bias ? bias[e] : 0.f);
      }
      raw[i] = r;
      key[i] = (static_cast<uint64_t>(orderable_u32(sel)) << 32) | static_cast<uint64_t>(0xFFFFFFFFu - e);
    }
  }
  float my_val = 0.f;  // lane s keeps the value of slot s
  int my_id = 0;
  for (int s = 0; s < k; ++s) {
    uint64_t best = 0ull;
#pragma unroll
    for (int i = 0; i < PER; ++i) best = key[i] > best ? key[i] : best;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const uint64_t other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    const int e = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(best & 0xFFFFFFFFull));
    float v = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      if (i * 32 + lane == e) {
        v = raw[i];
        key[i] = 0ull;
      }
    }
    v = __shfl_sync(0xffffffffu, v, e & 31);
    if (lane == s) {
      my_val = v;
      my_id = e;
    }
  }
  float w;
  if (mode == 0) {
    float m = lane < k ? my_val : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float ex = lane < k ? expf(my_val - m) : 0.f;
    float sum = ex;  // fixed butterfly: same order on every run
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    w = ex / sum;
  } else {
    float sum = lane < k ? my_val : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    w = my_val / (sum + 1e-15f);
  }
  if (lane < k) {
    ids_row[lane] = my_id;
    wts_row[lane] = w;
  }
}

__device__ __forceinline__ void route_token_dispatch(const float* row, const float* bias, int32_t* ids_row,
                                                     float* wts_row, int E, int k, int mode, float scale, int lane) {
  if (E <= 128) route_one_token<4>(row, bias, ids_row, wts_row, E, k, mode, scale, lane);
  else if (E <= 256) route_one_token<8>(row, bias, ids_row, wts_row, E, k, mode, scale, lane);
  else route_one_token<MAX_EXPERTS / 32>(row, bias, ids_row, wts_row, E, k, mode, scale, lane);
}

__global__ void __launch_bounds__(256) route_topk_kernel(const float* __restrict__ logits,
                                                         const float* __restrict__ bias, int32_t* __restrict__ ids,
                                                         float* __restrict__ wts, int T, int E, int k, int mode,
                                                         float scale) {
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  route_token_dispatch(logits + static_cast<size_t>(t) * E, bias, ids + static_cast<size_t>(t) * k,
                       wts + static_cast<size_t>(t) * k, E, k, mode, scale, lane);
}

// -------------------------------------------------------------------- sort
// Stable counting sort by local expert in one CTA (what every CTA of the reference
// kernel does redundantly in muse_moe_w4a16/cuda/moe.cu:315-433; here it runs once and
// writes global tables). Warp w owns the contiguous entry range [w*chunk, (w+1)*chunk);
// pass 1 counts per (warp, expert); a scan turns the counts into per-warp bases; pass 2
// ranks each entry inside its 32-entry step with match_any/popc, so equal experts keep
// ascending entry order.
struct SortSmem {
  int wcnt[SORT_WARPS][MAX_LOCAL_EXPERTS];
  int tot[MAX_LOCAL_EXPERTS];
  int wsum[MAX_LOCAL_EXPERTS / 32];
};

__device__ __forceinline__ int local_expert(int id, int lo, int nloc) {
  const int l = id - lo;
  return (id >= 0 && l >= 0 && l < nloc) ? l : -1;
}

// `ids` is deliberately not __restrict__: the fused kernel writes the ids in the same launch, so
// the loads must stay ordinary coherent loads.
__device__ void sort_entries_block(SortSmem& sm, const int32_t* ids, int n, int lo, int nloc,
                                   int32_t* __restrict__ cnt, int32_t* __restrict__ off, int32_t* __restrict__ perm,
                                   int32_t* __restrict__ inv) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk = ((n + SORT_WARPS - 1) / SORT_WARPS + 31) & ~31;
  const int beg = warp * chunk, end = min(n, beg + chunk);
  for (int i = tid; i < SORT_WARPS * MAX_LOCAL_EXPERTS; i += SORT_THREADS) (&sm.wcnt[0][0])[i] = 0;
  __syncthreads();
  for (int base = beg; base < end; base += 32) {
    const int i = base + lane;
    const int l = i < end ? local_expert(ids[i], lo, nloc) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, l);
    if (l >= 0 && (peers & ((1u << lane) - 1u)) == 0u) sm.wcnt[warp][l] += __popc(peers);
    __syncwarp();
  }
  __syncthreads();
  // per expert: exclusive scan over warps; thread e owns expert e
  if (tid < MAX_LOCAL_EXPERTS) {
    int acc = 0;
    if (tid < nloc) {
      for (int w = 0; w < SORT_WARPS; ++w) {
        const int c = sm.wcnt[w][tid];
        sm.wcnt[w][tid] = acc;
        acc += c;
      }
      cnt[tid] = acc;
    }
    // exclusive scan of the totals over experts (8 warps x 32)
    int incl = acc;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) sm.wsum[warp] = incl;
    sm.tot[tid] = incl - acc;  // exclusive within the warp
  }
  __syncthreads();
  if (tid < MAX_LOCAL_EXPERTS) {
    int wbase = 0;
    for (int w = 0; w < warp; ++w) wbase += sm.wsum[w];
    const int ex = sm.tot[tid] + wbase;
    __syncwarp();
    sm.tot[tid] = ex;
    if (tid < nloc) off[tid] = ex;
    if (tid == nloc - 1) off[nloc] = ex + cnt[tid];
  }
  __syncthreads();
  for (int base = beg; base < end; base += 32) {
    const int i = base + lane;
    const int l = i < end ? local_expert(ids[i], lo, nloc) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, l);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int q = -1;
    if (l >= 0) q = sm.tot[l] + sm.wcnt[warp][l] + rank;
    __syncwarp();
    if (l >= 0 && rank == 0) sm.wcnt[warp][l] += __popc(peers);
    __syncwarp();
    if (i < end) {
      inv[i] = q;
      if (q >= 0) perm[q] = i;
    }
  }
}

// F16 copy of the token rows by the sorting CTA (small token counts only: saves a launch in the
// decode chain). xh may be null.
__device__ __forceinline__ void convert_rows_block(const __nv_bfloat16* __restrict__ x, __half* __restrict__ xh,
                                                   int T, int H, const __nv_bfloat16* __restrict__ pre_w, float pre_eps) {
  if (xh == nullptr) return;
  if (pre_w != nullptr) {
    // with the pre-expert RMS norm (x * rsqrt(mean(x^2) + eps) * (1 + pre_w), one BF16 rounding): a warp
    // per row, the sum of squares by a fixed shuffle tree, the row read a second time from L1/L2
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint4* g = reinterpret_cast<const uint4*>(pre_w);
    for (int t = warp; t < T; t += SORT_WARPS) {
      const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H);
      uint4* dst = reinterpret_cast<uint4*>(xh + static_cast<size_t>(t) * H);
      float ss = 0.f;
      for (int i = lane; i < H / 8; i += 32) {
        const uint4 v = src[i];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float lo = __uint_as_float(w[c] << 16), hi = __uint_as_float(w[c] & 0xFFFF0000u);
          ss += lo * lo + hi * hi;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rs = rsqrtf(ss / static_cast<float>(H) + pre_eps);
      for (int i = lane; i < H / 8; i += 32) {
        const uint4 v = src[i], gv = g[i];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
        uint32_t o4[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float lo = __uint_as_float(w[c] << 16) * rs * (1.0f + __uint_as_float(gw[c] << 16));
          const float hi = __uint_as_float(w[c] & 0xFFFF0000u) * rs * (1.0f + __uint_as_float(gw[c] & 0xFFFF0000u));
          const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
          o4[c] = bf16x2_to_f16x2(*reinterpret_cast<const uint32_t*>(&b));
        }
        dst[i] = make_uint4(o4[0], o4[1], o4[2], o4[3]);
      }
    }
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x);
  uint4* dst = reinterpret_cast<uint4*>(xh);
  const int n = T * (H / 8);
  for (int i = threadIdx.x; i < n; i += SORT_THREADS) {
    const uint4 v = src[i];
    dst[i] = make_uint4(bf16x2_to_f16x2(v.x), bf16x2_to_f16x2(v.y), bf16x2_to_f16x2(v.z), bf16x2_to_f16x2(v.w));
  }
}

__global__ void __launch_bounds__(SORT_THREADS) sort_kernel(const int32_t* __restrict__ ids, int n, int lo, int nloc,
                                                            int32_t* __restrict__ cnt, int32_t* __restrict__ off,
                                                            int32_t* __restrict__ perm, int32_t* __restrict__ inv,
                                                            const __nv_bfloat16* __restrict__ x,
                                                            __half* __restrict__ xh, int T, int H,
                                                            const __nv_bfloat16* __restrict__ pre_w, float pre_eps) {
  extern __shared__ __align__(16) unsigned char sort_smem_raw[];
  SortSmem& sm = *reinterpret_cast<SortSmem*>(sort_smem_raw);
  asm volatile("griddepcontrol.wait;" ::: "memory");               // topk_ids may come from the kernel before
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // let the GEMM kernel set itself up meanwhile
  convert_rows_block(x, xh, T, H, pre_w, pre_eps);
  sort_entries_block(sm, ids, n, lo, nloc, cnt, off, perm, inv);
}

// ---- the same stable sort on several CTAs, for many entries (prefill, expert-parallel chunks)
// CTA b owns the contiguous entry range [b chunk, (b + 1) chunk). Three launches:
//   count    per-CTA per-expert counts                                   -> blk[b][e]
//   scan     one CTA: exclusive prefix over (expert, CTA) in that order  -> cnt, off, blk[b][e] = first
//            sorted position of CTA b's entries of expert e
//   scatter  each CTA ranks its entries as the single-CTA sort does (warps own ascending
//            sub-ranges, in-warp rank by match/popc) on top of its bases
// Entries of one expert keep ascending entry order across CTAs, warps and lanes: the same
// permutation as the single-CTA sort, bit for bit.
constexpr int SORT_MULTI_MIN = 16384;    // entries from which several CTAs sort
constexpr int SORT_MULTI_BLOCKS = 64;

// Pass 1 of a CTA over its range: sm.wcnt[w][e] = entries of expert e in warp w's sub-range.
__device__ __forceinline__ void sort_count_range(SortSmem& sm, const int32_t* ids, int beg, int end, int lo, int nloc,
                                                 int& wbeg, int& wend) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = max(end - beg, 0);
  const int chunk = ((n + SORT_WARPS - 1) / SORT_WARPS + 31) & ~31;
  wbeg = beg + warp * chunk;
  wend = min(end, wbeg + chunk);
  for (int i = tid; i < SORT_WARPS * MAX_LOCAL_EXPERTS; i += SORT_THREADS) (&sm.wcnt[0][0])[i] = 0;
  __syncthreads();
  for (int base = wbeg; base < wend; base += 32) {
    const int i = base + lane;
    const int l = i < wend ? local_expert(ids[i], lo, nloc) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, l);
    if (l >= 0 && (peers & ((1u << lane) - 1u)) == 0u) sm.wcnt[warp][l] += __popc(peers);
    __syncwarp();
  }
  __syncthreads();
}

__global__ void __launch_bounds__(SORT_THREADS) sort_multi_count_kernel(const int32_t* __restrict__ ids, int n, int lo,
                                                                        int nloc, int32_t* __restrict__ blk) {
  extern __shared__ __align__(16) unsigned char sort_smem_raw[];
  SortSmem& sm = *reinterpret_cast<SortSmem*>(sort_smem_raw);
  const int per = (n + gridDim.x - 1) / gridDim.x;
  const int beg = min(n, static_cast<int>(blockIdx.x) * per), end = min(n, beg + per);
  int wbeg, wend;
  sort_count_range(sm, ids, beg, end, lo, nloc, wbeg, wend);
  const int tid = threadIdx.x;
  if (tid < nloc) {
    int acc = 0;
    for (int w = 0; w < SORT_WARPS; ++w) acc += sm.wcnt[w][tid];
    blk[blockIdx.x * MAX_LOCAL_EXPERTS + tid] = acc;
  }
}

__global__ void __launch_bounds__(MAX_LOCAL_EXPERTS) sort_multi_scan_kernel(int32_t* __restrict__ blk, int n_blocks,
                                                                            int nloc, int32_t* __restrict__ cnt,
                                                                            int32_t* __restrict__ off) {
  __shared__ int wsum[MAX_LOCAL_EXPERTS / 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int total = 0;
  if (tid < nloc) {
    for (int b = 0; b < n_blocks; ++b) {
      const int c = blk[b * MAX_LOCAL_EXPERTS + tid];
      blk[b * MAX_LOCAL_EXPERTS + tid] = total;
      total += c;
    }
    cnt[tid] = total;
  }
  int incl = total;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  int ex = incl - total;
  for (int w = 0; w < warp; ++w) ex += wsum[w];
  if (tid < nloc) {
    off[tid] = ex;
    if (tid == nloc - 1) off[nloc] = ex + total;
    for (int b = 0; b < n_blocks; ++b) blk[b * MAX_LOCAL_EXPERTS + tid] += ex;
  }
}

__global__ void __launch_bounds__(SORT_THREADS) sort_multi_scatter_kernel(const int32_t* __restrict__ ids, int n, int lo,
                                                                          int nloc, const int32_t* __restrict__ blk,
                                                                          int32_t* __restrict__ perm,
                                                                          int32_t* __restrict__ inv) {
  extern __shared__ __align__(16) unsigned char sort_smem_raw[];
  SortSmem& sm = *reinterpret_cast<SortSmem*>(sort_smem_raw);
  const int per = (n + gridDim.x - 1) / gridDim.x;
  const int beg = min(n, static_cast<int>(blockIdx.x) * per), end = min(n, beg + per);
  int wbeg, wend;
  sort_count_range(sm, ids, beg, end, lo, nloc, wbeg, wend);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < nloc) {   // exclusive prefix over the warps, and this CTA's base of the expert
    int acc = 0;
    for (int w = 0; w < SORT_WARPS; ++w) {
      const int c = sm.wcnt[w][tid];
      sm.wcnt[w][tid] = acc;
      acc += c;
    }
    sm.tot[tid] = blk[blockIdx.x * MAX_LOCAL_EXPERTS + tid];
  }
  __syncthreads();
  for (int base = wbeg; base < wend; base += 32) {
    const int i = base + lane;
    const int l = i < wend ? local_expert(ids[i], lo, nloc) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, l);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int q = -1;
    if (l >= 0) q = sm.tot[l] + sm.wcnt[warp][l] + rank;
    __syncwarp();
    if (l >= 0 && rank == 0) sm.wcnt[warp][l] += __popc(peers);
    __syncwarp();
    if (i < wend) {
      inv[i] = q;
      if (q >= 0) perm[q] = i;
    }
  }
}

// Routing and sort in one launch for small token counts: every warp routes the tokens
// t = warp, warp + 32, ...; after a block barrier the same CTA sorts the entries it just wrote.
__global__ void __launch_bounds__(SORT_THREADS) route_sort_kernel(const float* __restrict__ logits,
                                                                  const float* __restrict__ bias,
                                                                  int32_t* __restrict__ ids, float* __restrict__ wts,
                                                                  int T, int E, int k, int mode, float scale, int lo,
                                                                  int nloc, int32_t* __restrict__ cnt,
                                                                  int32_t* __restrict__ off, int32_t* __restrict__ perm,
                                                                  int32_t* __restrict__ inv,
                                                                  const __nv_bfloat16* __restrict__ x,
                                                                  __half* __restrict__ xh, int H,
                                                                  const __nv_bfloat16* __restrict__ pre_w,
                                                                  float pre_eps) {
  extern __shared__ __align__(16) unsigned char sort_smem_raw[];
  SortSmem& sm = *reinterpret_cast<SortSmem*>(sort_smem_raw);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  convert_rows_block(x, xh, T, H, pre_w, pre_eps);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int t = warp; t < T; t += SORT_WARPS)
    route_token_dispatch(logits + static_cast<size_t>(t) * E, bias, ids + static_cast<size_t>(t) * k,
                         wts + static_cast<size_t>(t) * k, E, k, mode, scale, lane);
  __syncthreads();  // the ids written above are read back below by other threads of this CTA
  sort_entries_block(sm, ids, T * k, lo, nloc, cnt, off, perm, inv);
}

// Top-k of one token by one warp with the scores in shared memory: the same keys, the same k rounds of
// arg-max and the same weight arithmetic as route_one_token (so the same ids and weights, bit for
// bit), written as plain loops. Compact code matters where it runs: in the prologue of the GEMM kernel
// of a one-token step every instruction-cache line that has to come from memory is on the critical
// path. key_s / raw_s: this warp's E words each.
__device__ __noinline__ void route_token_compact(const float* __restrict__ row, const float* __restrict__ bias,
                                                 uint32_t* key_s, float* raw_s, int32_t* ids_row, float* wts_row, int E,
                                                 int k, int mode, float scale, int lane) {
#pragma unroll 1
  for (int e = lane; e < E; e += 32) {
    const float l = row[e];
    float sel = l, r = l;
    if (mode == 1) {
      r = 1.0f / (1.0f + expf(-l * scale));
      sel = r + (bias ? bias[e] : 0.f);
    }
    raw_s[e] = r;
    key_s[e] = orderable_u32(sel);
  }
  __syncwarp();
  float my_val = 0.f;  // lane s keeps the value of slot s
  int my_id = 0;
#pragma unroll 1
  for (int s = 0; s < k; ++s) {
    uint64_t best = 0ull;
#pragma unroll 1
    for (int e = lane; e < E; e += 32) {
      const uint32_t hi = key_s[e];
      // an expert already taken has its key word cleared and so loses to every remaining one
      const uint64_t key = hi == 0u ? 0ull : ((static_cast<uint64_t>(hi) << 32) | static_cast<uint64_t>(0xFFFFFFFFu - e));
      best = key > best ? key : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const uint64_t other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    const int e = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(best & 0xFFFFFFFFull));
    const float v = raw_s[e];
    __syncwarp();
    if (lane == 0) key_s[e] = 0u;
    __syncwarp();
    if (lane == s) {
      my_val = v;
      my_id = e;
    }
  }
  float w;
  if (mode == 0) {
    float m = lane < k ? my_val : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float ex = lane < k ? expf(my_val - m) : 0.f;
    float sum = ex;  // fixed butterfly: same order on every run
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    w = ex / sum;
  } else {
    float sum = lane < k ? my_val : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    w = my_val / (sum + 1e-15f);
  }
  if (lane < k) {
    ids_row[lane] = my_id;
    wts_row[lane] = w;
  }
  __syncwarp();  // key_s / raw_s may be refilled for the warp's next token
}

// ---- routing + stable sort of a few entries inside another kernel's prologue
// For up to 256 (token, slot) entries every CTA of the gate/up GEMM kernel derives the tables itself,
// as every CTA of the reference kernel does (muse_moe_w4a16/cuda/moe.cu:313-433), so the step needs no
// separate routing / sorting launch. Same algorithm as sort_entries_block with one 32-entry step per
// warp: warps 0-7 own entries [32 w, 32 w + 32), equal experts keep ascending entry order.
constexpr int SMALL_SORT_MAX_ENTRIES = 256;
constexpr int SMALL_SORT_WARPS = SMALL_SORT_MAX_ENTRIES / 32;

constexpr int SMALL_ROUTE_WARPS = 24;   // warps that route (one token each per turn)
constexpr int SMALL_RANK_MAX_PAIRS = 4096;   // (token, expert) pairs up to which the top-k is taken by rank
constexpr int SMALL_RANK_MAX_COMPARES = 1 << 20;
struct SmallSortScratch {
  int wcnt[SMALL_SORT_WARPS][MAX_LOCAL_EXPERTS];
  int wsum[SMALL_SORT_WARPS];
  int32_t ids[SMALL_SORT_MAX_ENTRIES];
  float tw[SMALL_SORT_MAX_ENTRIES];
  uint32_t key[SMALL_ROUTE_WARPS][MAX_EXPERTS];   // routing: orderable scores of the token a warp works on
  float raw[SMALL_ROUTE_WARPS][MAX_EXPERTS];      //          and the values the weights are formed from
  // routing by rank (few tokens x experts): one packed key and one raw value per (token, expert)
  unsigned long long key64[SMALL_RANK_MAX_PAIRS];
  float raw_all[SMALL_RANK_MAX_PAIRS];
};

// Top-k of a few tokens by rank, all threads of the CTA at once: the packed key of (token, expert) is
// the one route_one_token uses (orderable score << 32 | ~expert), keys of a token are distinct, so the
// number of larger keys of the same token is the expert's position in the descending order, and the
// experts of rank < k are the top-k in slot order: the same ids as k rounds of arg-max, with no
// dependent rounds. The weights are then formed by one warp per token with route_one_token's
// arithmetic (same butterflies, same padding). Called by every thread; n_threads = blockDim.x.
__device__ __noinline__ void route_by_rank_cta(SmallSortScratch& sc, const float* __restrict__ logits,
                                               const float* __restrict__ bias, int T, int E, int k, int mode,
                                               float scale) {
  const int tid = threadIdx.x, n_threads = blockDim.x, warp = tid >> 5, lane = tid & 31;
  const int n_pairs = T * E;
#pragma unroll 1
  for (int i = tid; i < n_pairs; i += n_threads) {
    const int e = i % E;
    const float l = logits[i];
    float sel = l, r = l;
    if (mode == 1) {
      r = 1.0f / (1.0f + expf(-l * scale));
      sel = r + (bias ? bias[e] : 0.f);
    }
    sc.raw_all[i] = r;
    sc.key64[i] = (static_cast<unsigned long long>(orderable_u32(sel)) << 32) |
                  static_cast<unsigned long long>(0xFFFFFFFFu - static_cast<uint32_t>(e));
  }
  __syncthreads();
#pragma unroll 1
  for (int i = tid; i < n_pairs; i += n_threads) {
    const int t = i / E, e = i - t * E;
    const unsigned long long mine = sc.key64[i];
    const unsigned long long* row = sc.key64 + t * E;
    int rank = 0;
#pragma unroll 4
    for (int j = 0; j < E; ++j) rank += row[j] > mine ? 1 : 0;
    if (rank < k) {
      sc.ids[t * k + rank] = e;
      sc.tw[t * k + rank] = sc.raw_all[i];
    }
  }
  __syncthreads();
#pragma unroll 1
  for (int t = warp; t < T; t += n_threads / 32) {
    const float my_val = lane < k ? sc.tw[t * k + lane] : 0.f;
    float w;
    if (mode == 0) {
      float m = lane < k ? my_val : -INFINITY;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      const float ex = lane < k ? expf(my_val - m) : 0.f;
      float sum = ex;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      w = ex / sum;
    } else {
      float sum = lane < k ? my_val : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      w = my_val / (sum + 1e-15f);
    }
    __syncwarp();
    if (lane < k) sc.tw[t * k + lane] = w;
  }
}

// Called by every thread of the CTA (block size a multiple of 32, at least 256). ids_s: the entries
// in shared memory. Results: cnt_s[nloc], off_s[nloc + 1], perm8_s[q] = entry index (fits a byte) in
// shared memory; when `global` the calling CTA also writes cnt, off, perm, inv to global memory.
__device__ __noinline__ void sort_small_cta(SmallSortScratch& sc, int n, int lo, int nloc, int* cnt_s, int* off_s,
                                               uint8_t* perm8_s, bool global, int32_t* cnt_g, int32_t* off_g,
                                               int32_t* perm_g, int32_t* inv_g) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nthreads = blockDim.x;
  for (int i = tid; i < SMALL_SORT_WARPS * MAX_LOCAL_EXPERTS; i += nthreads) (&sc.wcnt[0][0])[i] = 0;
  __syncthreads();
  int l = -1, rank = 0;
  if (warp < SMALL_SORT_WARPS) {
    const int i = warp * 32 + lane;
    l = i < n ? local_expert(sc.ids[i], lo, nloc) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, l);
    rank = __popc(peers & ((1u << lane) - 1u));
    if (l >= 0 && rank == 0) sc.wcnt[warp][l] = __popc(peers);
  }
  __syncthreads();
  int tot = 0, excl = 0;
  if (tid < MAX_LOCAL_EXPERTS) {   // thread e: exclusive scan of expert e over the warps, then over the experts
    if (tid < nloc) {
#pragma unroll
      for (int w = 0; w < SMALL_SORT_WARPS; ++w) {
        const int c = sc.wcnt[w][tid];
        sc.wcnt[w][tid] = tot;
        tot += c;
      }
      cnt_s[tid] = tot;
    }
    int incl = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) sc.wsum[warp] = incl;
    excl = incl - tot;
  }
  __syncthreads();
  if (tid < MAX_LOCAL_EXPERTS) {
    for (int w = 0; w < warp; ++w) excl += sc.wsum[w];
    if (tid < nloc) off_s[tid] = excl;
    if (tid == nloc - 1) off_s[nloc] = excl + tot;
  }
  __syncthreads();
  if (warp < SMALL_SORT_WARPS) {
    const int i = warp * 32 + lane;
    if (i < n) {
      const int q = l >= 0 ? off_s[l] + sc.wcnt[warp][l] + rank : -1;
      if (q >= 0) perm8_s[q] = static_cast<uint8_t>(i);
      if (global) {
        inv_g[i] = q;
        if (q >= 0) perm_g[q] = i;
      }
    }
  }
  if (global) {
    if (tid < nloc) cnt_g[tid] = cnt_s[tid];
    if (tid <= nloc) off_g[tid] = off_s[tid];
  }
  __syncthreads();
}

}  // namespace msk
