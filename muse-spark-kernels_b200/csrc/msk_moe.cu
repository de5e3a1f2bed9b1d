// C ABI of the routed-expert step (declarations and contracts: include/msk_moe.h).
// Host side: argument validation, workspace carving, plan choice and launches; no torch
// headers, no allocation, no synchronisation except msk_moe_read_status.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/msk_moe.h"
#include "route_sort.cuh"
#include "gemm.cuh"
#include "router_gemm.cuh"

namespace msk {

// ------------------------------------------------------------ repack kernels
// Tile order inside a packed buffer: ((expert * tiles_per_expert) + row_tile') * n_stages + ks,
// where for w13 row_tile' = 2*j + (0 gate | 1 up) and the source rows are gu*I + j*128 + r;
// for w2 row_tile' = row tile and the source rows are row_tile*128 + r.
struct RepackGeom {
  int rows_total;       // source rows per expert (2I or H)
  int K;                // source K
  int tiles_per_expert; // rows_total / 128
  int n_stages;         // K / 256
  int interleave_I;     // I for w13 (gate/up interleave), 0 for w2
};

__device__ __forceinline__ int source_row(const RepackGeom& g, int tile_in_expert, int r) {
  if (g.interleave_I > 0) {
    const int j = tile_in_expert >> 1, gu = tile_in_expert & 1;
    return gu * g.interleave_I + j * 128 + r;
  }
  return tile_in_expert * 128 + r;
}

// One thread per 16 output bytes (a code chunk or a row's scale bytes).
template <bool INVERSE>
__global__ void __launch_bounds__(256) repack_kernel(uint8_t* codes, uint8_t* sf, uint8_t* packed, RepackGeom g,
                                                     long long n_tiles) {
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long per_tile = 128 * 9;  // 8 code chunks + 1 scale chunk per row
  if (gid >= n_tiles * per_tile) return;
  const long long tile = gid / per_tile;
  const int rem = static_cast<int>(gid % per_tile);
  const int part = rem / 128, r = rem % 128;  // part 0..7 = code chunk, 8 = scales
  const int ks = static_cast<int>(tile % g.n_stages);
  const long long t2 = tile / g.n_stages;
  const int tile_in_expert = static_cast<int>(t2 % g.tiles_per_expert);
  const long long e = t2 / g.tiles_per_expert;
  const long long srow = e * g.rows_total + source_row(g, tile_in_expert, r);
  uint8_t* ptile = packed + tile * TILE_BYTES;
  if (part < 8) {
    uint4* src = reinterpret_cast<uint4*>(codes + srow * (g.K / 2) + ks * (KS / 2) + part * 16);
    uint4* dst = reinterpret_cast<uint4*>(ptile + (part * 128 + r) * 16);
    if (!INVERSE) *dst = *src; else *src = *dst;
  } else {
    uint4* src = reinterpret_cast<uint4*>(sf + srow * (g.K / 16) + ks * (KS / 16));
    uint4* dst = reinterpret_cast<uint4*>(ptile + TILE_CODE_BYTES + r * 16);
    if (!INVERSE) *dst = *src; else *src = *dst;
  }
}

// Packed tiles -> BF16 e2m1*e4m3 matrices, through the decode routine of the GEMM kernel (the
// F16 products are exact and convert to BF16 without rounding).
__global__ void __launch_bounds__(128) dequant_packed_kernel(const uint8_t* packed, __nv_bfloat16* out, RepackGeom g,
                                                             long long n_tiles) {
  const long long tile = blockIdx.x;
  if (tile >= n_tiles) return;
  const int r = threadIdx.x;
  const int ks = static_cast<int>(tile % g.n_stages);
  const long long t2 = tile / g.n_stages;
  const int tile_in_expert = static_cast<int>(t2 % g.tiles_per_expert);
  const long long e = t2 / g.tiles_per_expert;
  const long long srow = e * g.rows_total + source_row(g, tile_in_expert, r);
  const uint8_t* ptile = packed + tile * TILE_BYTES;
  const uint4 sfw = *reinterpret_cast<const uint4*>(ptile + TILE_CODE_BYTES + r * 16);
  const uint32_t sfa[4] = {sfw.x, sfw.y, sfw.z, sfw.w};
  __nv_bfloat16* orow = out + srow * g.K + ks * KS;
  for (int chunk = 0; chunk < 8; ++chunk) {
    const uint4 qv = *reinterpret_cast<const uint4*>(ptile + (chunk * 128 + r) * 16);
    const uint32_t q[4] = {qv.x, qv.y, qv.z, qv.w};
    const uint32_t sw = sfa[chunk >> 1] >> ((chunk & 1) * 16);
    uint32_t o[16];
    decode_chunk(q, sw, o);
    for (int j = 0; j < 16; ++j) {
      const __half2 h = *reinterpret_cast<const __half2*>(&o[j]);
      orow[chunk * 32 + 2 * j] = __float2bfloat16_rn(__low2float(h));
      orow[chunk * 32 + 2 * j + 1] = __float2bfloat16_rn(__high2float(h));
    }
  }
}

// ------------------------------------------------------------- row gather
// xs[q, :] = x[perm[q] / top_k, :] for the routed rows q < off[nloc]: token rows in sorted
// (expert-major) order, so that wide token tiles can be fetched as plain 2-D TMA boxes. The
// reference's prefill path gathers rows into per-expert tiles the same way
// (muse_prefill_layer/cuda/prefill.cu:1446-1608), there fused with its pre-expert norm.
// The copy also converts BF16 -> F16, the operand type of the MMA (layout.cuh).
// gather != 0: xs[q] = f16(x[perm[q] / top_k]) for q < off[nloc] (grid = T * top_k blocks);
// gather == 0: xs[t] = f16(x[t]) (grid = T blocks), for the narrow token tiles that gather rows
// through the permutation themselves.
// With pre_w the pre-expert RMS norm of the layer callers is applied on the way:
// x' = bf16( x * rsqrt(mean(x^2) + eps) * (1 + pre_w) ), FP32 arithmetic on the row the block holds in
// registers (muse_decode_layer/py/04_triton_kernels.py:556-568: the reference's routing kernel does the
// same before it stores the expert input). The sum of squares is a fixed shuffle tree followed by a
// fixed-order sum of the eight warp partials.
__global__ void __launch_bounds__(256) gather_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const int32_t* __restrict__ perm,
                                                          const int32_t* __restrict__ off, int nloc, int top_k, int H,
                                                          int gather, __half* __restrict__ xs,
                                                          const __nv_bfloat16* __restrict__ pre_w, float pre_eps) {
  __shared__ float wsum[8];
  pdl_wait();
  pdl_launch_dependents();
  const int q = blockIdx.x;
  if (gather && q >= off[nloc]) return;
  const size_t row = gather ? static_cast<size_t>(perm[q] / top_k) : static_cast<size_t>(q);
  const uint4* src = reinterpret_cast<const uint4*>(x + row * H);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(q) * H);
  if (pre_w == nullptr) {
    for (int i = threadIdx.x; i < H / 8; i += 256) {
      const uint4 v = src[i];
      dst[i] = make_uint4(bf16x2_to_f16x2(v.x), bf16x2_to_f16x2(v.y), bf16x2_to_f16x2(v.z), bf16x2_to_f16x2(v.w));
    }
    return;
  }
  constexpr int MAXV = 4;   // 8 values per uint4, 256 threads: H <= 8192
  uint4 v[MAXV];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = j * 256 + threadIdx.x;
    v[j] = make_uint4(0u, 0u, 0u, 0u);
    if (i < H / 8) v[j] = src[i];
    const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float lo = __uint_as_float(w[c] << 16), hi = __uint_as_float(w[c] & 0xFFFF0000u);
      ss += lo * lo + hi * hi;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w8 = 0; w8 < 8; ++w8) tot += wsum[w8];
  const float rs = rsqrtf(tot / static_cast<float>(H) + pre_eps);
  const uint4* gsrc = reinterpret_cast<const uint4*>(pre_w);
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = j * 256 + threadIdx.x;
    if (i >= H / 8) continue;
    const uint4 gv = gsrc[i];
    const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
    uint32_t o4[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float lo = __uint_as_float(w[c] << 16) * rs * (1.0f + __uint_as_float(gw[c] << 16));
      const float hi = __uint_as_float(w[c] & 0xFFFF0000u) * rs * (1.0f + __uint_as_float(gw[c] & 0xFFFF0000u));
      const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);   // the expert input is BF16
      o4[c] = bf16x2_to_f16x2(*reinterpret_cast<const uint32_t*>(&b));
    }
    dst[i] = make_uint4(o4[0], o4[1], o4[2], o4[3]);
  }
}

// The sorted copy without the pre-expert norm, as a persistent kernel: a warp per routed row, eight
// 16-byte loads in flight per lane, the next row's permutation entry fetched while the current row
// moves. (One block per row, as gather_rows_kernel works, spends most of its time on the two dependent
// loads every block starts with: 65,536 rows took 0.22 ms against 0.1 ms of memory time.)
__global__ void __launch_bounds__(256) gather_rows_sorted_kernel(const __nv_bfloat16* __restrict__ x,
                                                                 const int32_t* __restrict__ perm,
                                                                 const int32_t* __restrict__ off, int nloc, int top_k,
                                                                 int H, __half* __restrict__ xs) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (blockDim.x >> 5);
  const int n_rows = off[nloc];
  const int n16 = H / 8;   // 16-byte chunks per row
  int q = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int entry = q < n_rows ? perm[q] : 0;
  while (q < n_rows) {
    const int qn = q + warps;
    const int entry_next = qn < n_rows ? perm[qn] : 0;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(entry / top_k) * H);
    uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(q) * H);
    for (int i0 = 0; i0 < n16; i0 += 256) {
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = i0 + j * 32 + lane;
        if (i < n16) v[j] = __ldg(src + i);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = i0 + j * 32 + lane;
        if (i < n16)
          __stcs(dst + i, make_uint4(bf16x2_to_f16x2(v[j].x), bf16x2_to_f16x2(v[j].y), bf16x2_to_f16x2(v[j].z),
                                     bf16x2_to_f16x2(v[j].w)));
      }
    }
    q = qn;
    entry = entry_next;
  }
}

// xh = f16(x), one 16-byte chunk per thread, in small blocks: the row copy in front of a gate/up
// kernel that routes itself (few tokens). It waits for whatever precedes the step, then lets its
// dependents start: the gate/up kernel's prologue (routing, sort) overlaps this copy and only its
// activation gather waits for it.
__global__ void __launch_bounds__(64) convert_rows_kernel(const __nv_bfloat16* __restrict__ x, __half* __restrict__ xh,
                                                          int n_chunks) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * 64 + threadIdx.x;
  if (i >= n_chunks) return;
  const uint4 v = reinterpret_cast<const uint4*>(x)[i];
  reinterpret_cast<uint4*>(xh)[i] =
      make_uint4(bf16x2_to_f16x2(v.x), bf16x2_to_f16x2(v.y), bf16x2_to_f16x2(v.z), bf16x2_to_f16x2(v.w));
}

// ---------------------------------------------------------------- combine
// One block per token: out[t] = bf16( sum over slots in index order of
// w[t,s] * norm_s * y[inv[t,s]] ), norm_s = rsqrt(mean(y^2) + eps) when the post-expert
// norm is on (y already carries 1 + post_norm_w), else 1
// (muse_moe_w4a16/cuda/moe.cu:2604-2766; muse_decode_layer/py/04_triton_kernels.py:616-632).
// The block sum of squares is a fixed shuffle tree followed by a fixed-order sum of the
// eight warp partials, so the result does not depend on scheduling.
constexpr int COMBINE_THREADS = 512;
constexpr int COMBINE_MAX_F4 = 4;   // float4 per thread per row: H <= 8192
constexpr int COMBINE_WIDE_TOKENS = 512;  // from here on two blocks per SM, two slots per group

// G = slots whose rows are loaded together (one memory latency per group instead of one per
// slot; the sums still run in slot order). G = 4 for few tokens (latency), G = 2 with two blocks
// per SM for many (one block's loads overlap the other's reduction and stores); BF16 rows need
// half the registers while in flight, so they get G = 4 and two blocks per SM. Slots without a
// local route (inv < 0) are squeezed out first, keeping their order, so an expert-parallel rank
// that owns one or two of a token's eight routes pays for one group, and a token without any
// local route only writes zeros.
// Four consecutive y values of a row as they sit in registers while their group is in flight:
// FP32 (16 bytes) or BF16 (8 bytes, for the wide token tile), expanded when used.
template <bool YB> struct YQuad;
template <> struct YQuad<false> {
  float4 v;
  __device__ __forceinline__ void zero() { v = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ void load(const float* y, size_t row_elems, int j) {
    v = __ldcs(reinterpret_cast<const float4*>(y + row_elems) + j);
  }
  __device__ __forceinline__ float4 get() const { return v; }
};
template <> struct YQuad<true> {
  uint2 b;
  __device__ __forceinline__ void zero() { b = make_uint2(0u, 0u); }
  __device__ __forceinline__ void load(const float* y, size_t row_elems, int j) {
    b = __ldcs(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(y) + row_elems) + j);
  }
  __device__ __forceinline__ float4 get() const {
    return make_float4(__uint_as_float(b.x << 16), __uint_as_float(b.x & 0xFFFF0000u), __uint_as_float(b.y << 16),
                       __uint_as_float(b.y & 0xFFFF0000u));
  }
};

// NF4 = float4 slots per thread per row that the kernel is built for: 4 (H <= 8192) or 2 (H <= 4096, half
// the registers per row in flight, which is what lets all eight rows of a token be loaded at once).
template <int G, bool YB, int MINB, int NF4 = COMBINE_MAX_F4>
__global__ void __launch_bounds__(COMBINE_THREADS, MINB)
    combine_kernel(const float* __restrict__ y, const int32_t* __restrict__ inv, const float* __restrict__ tw,
                   __nv_bfloat16* __restrict__ out, int H, int k, int post_norm, float eps) {
  __shared__ float wsum[G][COMBINE_THREADS / 32];
  __shared__ int s_q[MAX_TOP_K];
  __shared__ float s_w[MAX_TOP_K];
  __shared__ int s_n;
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();  // y and inv come from the kernels before this one
  if (warp == 0) {  // lane s takes slot s (k <= 16); a ballot keeps the order
    const int q = lane < k ? inv[static_cast<size_t>(t) * k + lane] : -1;
    const float w = lane < k ? tw[static_cast<size_t>(t) * k + lane] : 0.f;
    const unsigned have = __ballot_sync(0xffffffffu, q >= 0);
    if (q >= 0) {
      const int at = __popc(have & ((1u << lane) - 1u));
      s_q[at] = q;
      s_w[at] = w;
    }
    if (lane == 0) s_n = __popc(have);
  }
  __syncthreads();
  const int nv = s_n;
  const int n4 = H / 4;  // float4 per row; thread tid owns indices i*512 + tid
  float4 acc[NF4];
#pragma unroll
  for (int i = 0; i < NF4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < nv; s0 += G) {
    int q[G];
    float wgt[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const bool in = s0 + g < nv;
      q[g] = in ? s_q[s0 + g] : -1;
      wgt[g] = in ? s_w[s0 + g] : 0.f;
    }
    YQuad<YB> v[G][NF4];
    float ss[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      ss[g] = 0.f;
      const size_t r = static_cast<size_t>(q[g] < 0 ? 0 : q[g]) * H;
#pragma unroll
      for (int i = 0; i < NF4; ++i) {
        v[g][i].zero();
        if (q[g] >= 0 && i * COMBINE_THREADS + tid < n4) v[g][i].load(y, r, i * COMBINE_THREADS + tid);
      }
    }
    if (post_norm) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int i = 0; i < NF4; ++i) {
          const float4 f = v[g][i].get();
          ss[g] += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss[g] += __shfl_xor_sync(0xffffffffu, ss[g], o);
      }
      __syncthreads();  // wsum of the previous group fully read
      if (lane == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) wsum[g][warp] = ss[g];
      }
      __syncthreads();
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < COMBINE_THREADS / 32; ++w) tot += wsum[g][w];  // fixed order
        wgt[g] *= rsqrtf(tot / static_cast<float>(H) + eps);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {  // slot order within the group
      if (q[g] < 0) continue;
#pragma unroll
      for (int i = 0; i < NF4; ++i) {
        const float4 f = v[g][i].get();
        acc[i].x += f.x * wgt[g]; acc[i].y += f.y * wgt[g];
        acc[i].z += f.z * wgt[g]; acc[i].w += f.w * wgt[g];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NF4; ++i) {
    if (i * COMBINE_THREADS + tid < n4) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc[i].x, acc[i].y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(acc[i].z, acc[i].w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(out + static_cast<size_t>(t) * H + (i * COMBINE_THREADS + tid) * 4) = pk;
    }
  }
}

// ------------------------------------------------------------- EP combine
// Expert-parallel combine at the token's home rank: out[t] = bf16( sum over ranks d, in rank
// order, of the partial row rank d returned for token t ), FP32 accumulation. Rank d contributes
// only when one of the token's top-k ids lies in d's expert range, so rows of ranks without a
// route are never read. back is [n, T, H] in rank order; the home rank's own partial may live
// elsewhere (self_rows).
__global__ void __launch_bounds__(256) ep_combine_kernel(const __nv_bfloat16* __restrict__ back,
                                                         const __nv_bfloat16* __restrict__ self_rows, int self_rank,
                                                         const int32_t* __restrict__ ids, int top_k, int per_rank,
                                                         __nv_bfloat16* __restrict__ out, int n, int T, int H) {
  __shared__ unsigned long long present;
  const int t = blockIdx.x;
  if (threadIdx.x == 0) present = 0ull;
  __syncthreads();
  if (threadIdx.x < top_k) {
    const int id = ids[static_cast<size_t>(t) * top_k + threadIdx.x];
    if (id >= 0 && id / per_rank < n) atomicOr(&present, 1ull << (id / per_rank));
  }
  __syncthreads();
  const unsigned long long have = present;
  const int n8 = H / 8;
  for (int i = threadIdx.x; i < n8; i += 256) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int d = 0; d < n; ++d) {
      if (!((have >> d) & 1ull)) continue;
      const __nv_bfloat16* rows = (d == self_rank && self_rows != nullptr)
                                      ? self_rows
                                      : back + static_cast<size_t>(d) * T * static_cast<size_t>(H);
      const uint4 v = *reinterpret_cast<const uint4*>(rows + static_cast<size_t>(t) * H + static_cast<size_t>(i) * 8);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __uint_as_float(w[j] << 16);
        acc[2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
      }
    }
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      ow[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + static_cast<size_t>(i) * 8) = o;
  }
}

// Stream memory operations (executed by the stream's front end, no SM): the cross-rank flags of
// the expert-parallel step. Looked up through the runtime, like the tensor-map encoder.
typedef CUresult (*StreamValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

static int stream_value32(const char* name, void* addr, uint32_t value, unsigned int flags, void* stream) {
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  const cudaError_t e = cudaGetDriverEntryPoint(name, &ptr, cudaEnableDefault, &qres);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (qres != cudaDriverEntryPointSuccess || ptr == nullptr) return static_cast<int>(cudaErrorNotSupported);
  const CUresult r = reinterpret_cast<StreamValue32Fn>(ptr)(static_cast<CUstream>(stream),
                                                            reinterpret_cast<CUdeviceptr>(addr), value, flags);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(cudaErrorInvalidValue);
}

// --------------------------------------------------------------- bw probe
// Every CTA streams its contiguous share of the buffer through a ring of bulk async
// copies, one elected thread issuing, one warp consuming (twin of the reference's
// muse_moe_w4a16/cuda/moe_bw.cu tma_kernel).
__global__ void __launch_bounds__(64) bw_probe_kernel(const uint8_t* src, unsigned long long bytes, int stages,
                                                      int stage_bytes, uint32_t* sink, int skip_release) {
  extern __shared__ __align__(1024) uint8_t psm[];
  __shared__ uint64_t full[8], empty[8];
  __shared__ int abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    abort_word = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const unsigned long long n_chunks = bytes / stage_bytes;
  const unsigned long long per = (n_chunks + gridDim.x - 1) / gridDim.x;
  const unsigned long long c0 = per * blockIdx.x, c1 = min(n_chunks, c0 + per);
  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol = policy_evict_first();
      uint32_t it = 0;
      for (unsigned long long c = c0; c < c1; ++c, ++it) {
        const uint32_t slot = it % stages, par = (it / stages) & 1u;
        if (!mbar_wait(&empty[slot], par ^ 1u, &abort_word)) break;
        mbar_arrive_expect_tx(&full[slot], stage_bytes);
        bulk_g2s(psm + static_cast<size_t>(slot) * stage_bytes, src + c * stage_bytes, stage_bytes, &full[slot], pol);
      }
    }
  } else {
    uint32_t it = 0, sum = 0;
    for (unsigned long long c = c0; c < c1; ++c, ++it) {
      const uint32_t slot = it % stages, par = (it / stages) & 1u;
      if (!mbar_wait(&full[slot], par, &abort_word)) break;
      sum += *reinterpret_cast<const uint32_t*>(psm + static_cast<size_t>(slot) * stage_bytes + lane * 16);
      __syncwarp();
      // skip_release (test hook): chunk number skip_release of every CTA is never handed back, so the
      // producer's bounded wait for that slot runs out and the kernel leaves through its time-out path
      if (lane == 0 && !(skip_release > 0 && it + 1 == static_cast<uint32_t>(skip_release))) mbar_arrive(&empty[slot]);
    }
    if (sum == 0x9E3779B9u) atomicAdd(sink, sum);  // keeps the reads alive
  }
  __syncthreads();
  if (abort_word != 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    if (threadIdx.x == 0) atomicExch(reinterpret_cast<int*>(sink) + 1, MSK_DEV_ERR_TIMEOUT);
  }
}

// ------------------------------------------------------------ host helpers
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static int check_cfg(const MskMoeCfg* c) {
  if (c == nullptr) return MSK_ERR_NULL;
  if (c->hidden <= 0 || c->inter <= 0 || c->hidden % 256 != 0 || c->inter % 256 != 0) return MSK_ERR_SHAPE;
  if (c->hidden > COMBINE_THREADS * COMBINE_MAX_F4 * 4) return MSK_ERR_SHAPE;  // combine keeps a row in registers
  if (c->max_tokens < 0) return MSK_ERR_SHAPE;
  if (c->top_k < 1 || c->top_k > MAX_TOP_K) return MSK_ERR_SHAPE;
  if (c->local_count < 1 || c->local_count > MAX_LOCAL_EXPERTS) return MSK_ERR_SHAPE;
  if (c->n_experts < 1 || c->n_experts > MAX_EXPERTS) return MSK_ERR_SHAPE;
  if (c->local_start < 0 || c->local_start + c->local_count > c->n_experts) return MSK_ERR_RANGE;
  if (c->token_tile != 0 && c->token_tile != 16 && c->token_tile != 32 && c->token_tile != 64 && c->token_tile != 128)
    return MSK_ERR_SHAPE;
  if (c->decode_path < 0 || c->decode_path > 4) return MSK_ERR_SHAPE;
  return MSK_OK;
}

static int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Persistent grid when the caller names none: the SM count of a B200. A constant, so that the
// shares of the weight stream (and with them the order in which a cut unit's pieces are summed)
// depend on the configuration, not on the device the library happens to run on.
constexpr int DEFAULT_CTAS = 148;
// MSK_NO_HANDOVER=1 switches the per-tile hand-over between the two GEMM launches off (measurements).
static bool handover_env_off() {
  static const bool v = [] {
    const char* e = std::getenv("MSK_NO_HANDOVER");
    return e != nullptr && e[0] == '1';
  }();
  return v;
}
constexpr int MAX_CTAS = 512;
constexpr int FLAT_MAX_ROWS = SMALL_SORT_MAX_ENTRIES;  // up to here the weight stream may be cut into equal shares
constexpr int ONE_LAUNCH_MAX_TOKENS = 8;               // up to here the step is one launch by default
constexpr int BOTH_GEMMS_MIN_TOKENS = 9;               // from here on (narrow tiles) both GEMMs share one launch by default

struct Plan {
  int N;         // token tile
  int path;      // 0 one launch, 1 chain of launches, 2 row copy + routing gate/up kernel + combining down kernel
  int flat;      // equal shares of the flat (base unit, K stage) list
  int grid;
};

static Plan make_plan(const MskMoeCfg* c, int T) {
  Plan p;
  p.grid = c->num_ctas > 0 ? std::min(c->num_ctas, MAX_CTAS) : DEFAULT_CTAS;
  p.path = 1;
  p.flat = 0;
  if (c->token_tile > 0) {
    p.N = c->token_tile;
  } else {
    const double rpe = static_cast<double>(T) * c->top_k / c->n_experts;  // mean tokens per expert
    // measured at H4096 I1536 E128 (us a step with 16 / 32 / 64-token tiles; the narrow ones with both GEMMs
    // in one launch): T = 160 (rpe 10): 281 / 313 / 307; T = 192 (rpe 12): 301 / 321 / 311; T = 256 (rpe 16):
    // 381 / 334 / 317; T = 384: 526 / 372 / 338; T = 512 (rpe 32): 648 / 510 / 352. The 16-token tile is the
    // fastest per K stage and wins while most experts fit one tile; past that the 64-token tile does; the
    // 32-token tile never wins at these shapes (it stays selectable with cfg.token_tile)
    p.N = rpe <= 12 ? 16 : rpe <= 32 ? 64 : 128;
  }
  const long long rows = static_cast<long long>(T) * c->top_k;
  // Flat shares are an option, off by default: measured on B200 a cut unit's pieces cost about 6 us of
  // round trips through L2 at the end of each GEMM (store, fence, ticket, reload from a cold instruction
  // cache), as much as the idle CTAs of the last round of whole units cost at these sizes.
  p.flat = (c->flat_shares != 0 && rows <= FLAT_MAX_ROWS && p.N <= 64) ? 1 : 0;
  {
    // the kernels do the share arithmetic in 32 bits: items * shares has to fit
    const long long pairs = std::max(c->inter / 128, c->hidden / 256), nst = std::max(c->hidden, c->inter) / KS;
    if ((rows + 1) * pairs * nst * p.grid >= FLAT_MAX_PRODUCT) p.flat = 0;
  }
  // few tokens: the kernels route, sort and combine themselves
  const bool few = rows <= SMALL_SORT_MAX_ENTRIES && T <= FOLD_MAX_TOKENS && p.N <= 32 && c->stop_after == 0;
  if (few) {
    // measured (H4096 I1536 E128 top-8, cold L2): one launch 47 / 64 / 89 / 136 us at 1 / 2 / 4 / 8 tokens
    // against 57 / 72 / 94 / 135 for the chain; at 16 and 32 tokens 195 / 268 against 197 / 249
    switch (c->decode_path) {
      case 1: p.path = 1; break;
      case 4: p.path = 1; break;   // becomes 4 below
      case 2: p.path = 2; break;
      case 3: p.path = 0; break;
      default: p.path = T <= ONE_LAUNCH_MAX_TOKENS ? 0 : 1; break;
    }
    if (p.path == 0 && p.grid > sm_count()) p.path = 2;  // the one-launch kernel needs every CTA resident
    if (p.path == 0) p.flat = 0;  // its phases hand over per token tile, which counts whole units
  }
  // Beyond a few tokens, narrow token tiles: the sort launches, then both GEMMs in one cooperative launch
  // (path 4: the weight stream, the dequant ring and the MMA pipeline run on from the gate/up units into the
  // down units, tile by tile, and the kernel makes its own F16 copy of the token rows), then the combine.
  // Measured at H4096 I1536 E128 (stamped runs): 16 / 32 / 64 / 128 tokens 176 / 227 / 253 / 268 us against
  // 186 / 240 / 258 / 270 for two GEMM launches with the per-tile hand-over between them. Same bits.
  if (p.path == 1 && p.N <= 32 && p.flat == 0 && c->stop_after == 0 && p.grid <= sm_count() &&
      (c->decode_path == 4 || (c->decode_path == 0 && T >= BOTH_GEMMS_MIN_TOKENS)))
    p.path = 4;
  return p;
}

// Workspace carving. Everything is sized for max_tokens with the worst plan.
struct Carve {
  size_t status, trace, cnt, off, perm, inv, tickets, few_ctl, sort_blk, tile_ctr, inter, y, partial, xs, total;
};
constexpr size_t TRACE_CTAS = 256;
constexpr size_t TRACE_WORDS = TRACE_CTAS * 16 + 3 * 256;

static size_t max_tiles(const MskMoeCfg* c, int T) {
  // ceil(cnt/16) summed over experts <= R/16 + (experts that can hold a row)
  const size_t R = static_cast<size_t>(T) * c->top_k;
  return R / 16 + std::min(static_cast<size_t>(c->local_count), R);
}

// Pieces of cut units (flat shares): two slots per CTA of the largest grid, each the two accumulator
// tiles of the widest token tile that is ever cut (64).
static size_t partial_floats(const MskMoeCfg* c) {
  const size_t grid = c->num_ctas > 0 ? static_cast<size_t>(std::min(c->num_ctas, MAX_CTAS)) : DEFAULT_CTAS;
  return 2 * grid * 2 * 128 * 64;
}

static size_t ticket_ints(const MskMoeCfg* c, int T) {
  return max_tiles(c, T) * static_cast<size_t>(std::max(c->inter / 128, c->hidden / 256));
}

static Carve carve(const MskMoeCfg* c, int T) {
  Carve k;
  const size_t R = static_cast<size_t>(T) * c->top_k;
  size_t o = 0;
  k.status = o; o += 256;
  k.trace = o; o += 2 * TRACE_WORDS * 8;  // two GEMM launches x (CTAs x 16 stamps + 3 x 256 events of CTA 0)
  k.cnt = o; o += round_up(static_cast<size_t>(c->local_count) * 4, 256);
  k.off = o; o += round_up(static_cast<size_t>(c->local_count + 1) * 4, 256);
  k.perm = o; o += round_up(R * 4, 256);
  k.inv = o; o += round_up(R * 4, 256);
  k.tickets = o; o += 2 * round_up(ticket_ints(c, T) * 4, 256);  // one region per GEMM
  k.few_ctl = o; o += 8192;    // few-token paths of the GEMM kernel: tickets [32 tokens][up to 32 pairs] at +0, grid counters [2] at
                               // +4096, per-tile counters [2][up to 384 tiles] at +4352
  k.sort_blk = o; o += static_cast<size_t>(SORT_MULTI_BLOCKS) * MAX_LOCAL_EXPERTS * 4;  // per-CTA counts of the multi-CTA sort
  // tile hand-over between the gate/up and the down launch: per token tile the finished gate/up units and
  // the down units that have seen them all (two counters per tile, zero between steps)
  k.tile_ctr = o; o += round_up(2 * max_tiles(c, T) * 4, 256);
  // everything above is control state: msk_moe_workspace_init zeroes [0, inter)
  k.inter = o; o += round_up(R * c->inter * 2, 256);
  k.y = o; o += round_up(R * c->hidden * 4, 256);
  k.partial = o; o += 2 * round_up(partial_floats(c) * 4, 256);  // one region per GEMM
  k.xs = o; o += round_up(R * c->hidden * 2, 256);  // F16 copy of the token rows ([T, H], or sorted [R, H] for wide token tiles)
  k.total = o;
  return k;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link against libcuda).
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int encode_act_map(CUtensorMap* map, const void* base, size_t rows, int K, int box_rows,
                          CUtensorMapDataType dtype = CU_TENSOR_MAP_DATA_TYPE_FLOAT16) {
  static TensorMapEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (qres != cudaDriverEntryPointSuccess || ptr == nullptr) return static_cast<int>(cudaErrorNotSupported);
    fn = reinterpret_cast<TensorMapEncodeFn>(ptr);
  }
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
  const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(cudaErrorInvalidValue);
}

// Experiment switch (environment variable MSK_FUSED_PLAIN): launch the one-launch kernel without the
// cooperative attribute. Its grid never exceeds the SM count and it holds an SM per CTA, so its CTAs
// are resident together in practice, and its waits are bounded either way.
static bool fused_plain_launch() {
  static int v = -1;
  if (v < 0) v = std::getenv("MSK_FUSED_PLAIN") != nullptr ? 1 : 0;
  return v == 1;
}

// MODE 2 (one launch for the step) waits on a grid-wide counter, so it is launched cooperatively:
// either every CTA is resident or the launch fails. The other modes are chained with programmatic
// dependent launch (unless pdl == 0).
template <int N, int MODE>
static int launch_gemm(const GemmParams& p, int grid, cudaStream_t st, int pdl) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(moe_gemm_kernel<N, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GemmCfg<N>::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3(static_cast<unsigned>(grid));
  lc.blockDim = dim3(GEMM_THREADS);
  lc.dynamicSmemBytes = GemmCfg<N>::SMEM_BYTES;
  lc.stream = st;
  cudaLaunchAttribute at[1];
  if (MODE == 2 && !fused_plain_launch()) {
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
  } else {
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start while its predecessor drains
    at[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  }
  lc.attrs = at;
  lc.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&lc, moe_gemm_kernel<N, MODE>, p));
}

template <int MODE>
static int launch_gemm_n(int N, const GemmParams& p, int grid, cudaStream_t st, int pdl) {
  switch (N) {
    case 16: return launch_gemm<16, MODE>(p, grid, st, pdl);
    case 32: return launch_gemm<32, MODE>(p, grid, st, pdl);
    case 64: return launch_gemm<64, MODE>(p, grid, st, pdl);
    case 128: return launch_gemm<128, MODE>(p, grid, st, pdl);
    default: return MSK_ERR_SHAPE;
  }
}

static int launch_gemm_fused(int N, const GemmParams& p, int grid, cudaStream_t st) {
  switch (N) {
    case 16: return launch_gemm<16, 2>(p, grid, st, 0);
    case 32: return launch_gemm<32, 2>(p, grid, st, 0);
    default: return MSK_ERR_SHAPE;
  }
}

static RepackGeom geom13(const MskMoeCfg* c) {
  return RepackGeom{2 * c->inter, c->hidden, 2 * c->inter / 128, c->hidden / KS, c->inter};
}
static RepackGeom geom2(const MskMoeCfg* c) {
  return RepackGeom{c->hidden, c->inter, c->hidden / 128, c->inter / KS, 0};
}
static long long n_tiles_of(const MskMoeCfg* c, const RepackGeom& g) {
  return static_cast<long long>(c->local_count) * g.tiles_per_expert * g.n_stages;
}

template <int N>
static int launch_router_hilo(const CUtensorMap& mw, const CUtensorMap& mx, float* logits, int32_t* status, int T, int E,
                              int H, cudaStream_t st) {
  const int smem = RG_STAGES * (2 * RG_A_BYTES + N * RG_KSTEP * 2) + static_cast<int>(sizeof(RouterGemmCtrl));
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(router_hilo_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3(static_cast<unsigned>((E + 127) / 128), static_cast<unsigned>((T + N - 1) / N));
  lc.blockDim = dim3(RG_THREADS);
  lc.dynamicSmemBytes = smem;
  lc.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&lc, router_hilo_kernel<N>, mw, mx, logits, status, T, E, H));
}

}  // namespace msk

using namespace msk;

extern "C" {

int msk_moe_packed_bytes(const MskMoeCfg* cfg, size_t* host_w13_bytes, size_t* host_w2_bytes) {
  const int rc = check_cfg(cfg);
  if (rc != MSK_OK) return rc;
  if (host_w13_bytes == nullptr || host_w2_bytes == nullptr) return MSK_ERR_NULL;
  *host_w13_bytes = static_cast<size_t>(n_tiles_of(cfg, geom13(cfg))) * TILE_BYTES;
  *host_w2_bytes = static_cast<size_t>(n_tiles_of(cfg, geom2(cfg))) * TILE_BYTES;
  return MSK_OK;
}

static int repack_common(const MskMoeCfg* cfg, void* w13, void* w13_sf, void* w2, void* w2_sf, void* packed13,
                         void* packed2, void* stream, bool inverse) {
  const int rc = check_cfg(cfg);
  if (rc != MSK_OK) return rc;
  if (!w13 || !w13_sf || !w2 || !w2_sf || !packed13 || !packed2) return MSK_ERR_NULL;
  if (!aligned16(w13) || !aligned16(w13_sf) || !aligned16(w2) || !aligned16(w2_sf) || !aligned16(packed13) ||
      !aligned16(packed2))
    return MSK_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const RepackGeom g13 = geom13(cfg), g2 = geom2(cfg);
  const long long n13 = n_tiles_of(cfg, g13), n2 = n_tiles_of(cfg, g2);
  const long long th13 = n13 * 128 * 9, th2 = n2 * 128 * 9;
  const unsigned b13 = static_cast<unsigned>((th13 + 255) / 256), b2 = static_cast<unsigned>((th2 + 255) / 256);
  if (!inverse) {
    repack_kernel<false><<<b13, 256, 0, st>>>(static_cast<uint8_t*>(w13), static_cast<uint8_t*>(w13_sf),
                                              static_cast<uint8_t*>(packed13), g13, n13);
    repack_kernel<false><<<b2, 256, 0, st>>>(static_cast<uint8_t*>(w2), static_cast<uint8_t*>(w2_sf),
                                             static_cast<uint8_t*>(packed2), g2, n2);
  } else {
    repack_kernel<true><<<b13, 256, 0, st>>>(static_cast<uint8_t*>(w13), static_cast<uint8_t*>(w13_sf),
                                             static_cast<uint8_t*>(packed13), g13, n13);
    repack_kernel<true><<<b2, 256, 0, st>>>(static_cast<uint8_t*>(w2), static_cast<uint8_t*>(w2_sf),
                                            static_cast<uint8_t*>(packed2), g2, n2);
  }
  return static_cast<int>(cudaGetLastError());
}

int msk_moe_repack(const MskMoeCfg* cfg, const void* w13, const void* w13_sf, const void* w2, const void* w2_sf,
                   void* packed13, void* packed2, void* stream) {
  return repack_common(cfg, const_cast<void*>(w13), const_cast<void*>(w13_sf), const_cast<void*>(w2),
                       const_cast<void*>(w2_sf), packed13, packed2, stream, false);
}

int msk_moe_unpack(const MskMoeCfg* cfg, const void* packed13, const void* packed2, void* w13, void* w13_sf,
                   void* w2, void* w2_sf, void* stream) {
  return repack_common(cfg, w13, w13_sf, w2, w2_sf, const_cast<void*>(packed13), const_cast<void*>(packed2), stream,
                       true);
}

int msk_moe_dequant_packed(const MskMoeCfg* cfg, const void* packed13, const void* packed2, void* dq13, void* dq2,
                           void* stream) {
  const int rc = check_cfg(cfg);
  if (rc != MSK_OK) return rc;
  if (!packed13 || !packed2 || !dq13 || !dq2) return MSK_ERR_NULL;
  if (!aligned16(packed13) || !aligned16(packed2) || !aligned16(dq13) || !aligned16(dq2)) return MSK_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const RepackGeom g13 = geom13(cfg), g2 = geom2(cfg);
  const long long n13 = n_tiles_of(cfg, g13), n2 = n_tiles_of(cfg, g2);
  dequant_packed_kernel<<<static_cast<unsigned>(n13), 128, 0, st>>>(static_cast<const uint8_t*>(packed13),
                                                                    static_cast<__nv_bfloat16*>(dq13), g13, n13);
  dequant_packed_kernel<<<static_cast<unsigned>(n2), 128, 0, st>>>(static_cast<const uint8_t*>(packed2),
                                                                   static_cast<__nv_bfloat16*>(dq2), g2, n2);
  return static_cast<int>(cudaGetLastError());
}

int msk_moe_router_logits(const MskMoeCfg* cfg, const void* x, const float* router_w, float* logits, int n_tokens,
                          void* stream) {
  const int rc = check_cfg(cfg);
  if (rc != MSK_OK) return rc;
  if (!x || !router_w || !logits) return MSK_ERR_NULL;
  if (n_tokens < 0) return MSK_ERR_SHAPE;
  if (n_tokens == 0) return MSK_OK;
  dim3 grid(static_cast<unsigned>(n_tokens), static_cast<unsigned>((cfg->n_experts + 7) / 8));
  router_logits_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), router_w, logits, cfg->hidden, cfg->n_experts);
  return static_cast<int>(cudaGetLastError());
}

int msk_moe_router_logits_hilo(const MskMoeCfg* cfg, const void* x, const void* router_hilo, float* logits,
                               int32_t* status_word, int n_tokens, void* stream) {
  const int rc = check_cfg(cfg);
  if (rc != MSK_OK) return rc;
  if (!x || !router_hilo || !logits) return MSK_ERR_NULL;
  if (!aligned16(x) || !aligned16(router_hilo) || !aligned16(logits)) return MSK_ERR_ALIGN;
  if (n_tokens < 0) return MSK_ERR_SHAPE;
  if (n_tokens == 0) return MSK_OK;
  if (n_tokens < 16) return MSK_ERR_SHAPE;   // fewer tokens than the narrowest MMA tile: use msk_moe_router_logits
  const int N = n_tokens >= 128 ? 128 : n_tokens >= 64 ? 64 : n_tokens >= 32 ? 32 : 16;
  CUtensorMap mw, mx;
  int e = encode_act_map(&mw, router_hilo, static_cast<size_t>(2) * cfg->n_experts, cfg->hidden, 128,
                         CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  if (e != 0) return e;
  e = encode_act_map(&mx, x, static_cast<size_t>(n_tokens), cfg->hidden, N, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  if (e != 0) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (N) {
    case 128: return launch_router_hilo<128>(mw, mx, logits, status_word, n_tokens, cfg->n_experts, cfg->hidden, st);
    case 64: return launch_router_hilo<64>(mw, mx, logits, status_word, n_tokens, cfg->n_experts, cfg->hidden, st);
    case 32: return launch_router_hilo<32>(mw, mx, logits, status_word, n_tokens, cfg->n_experts, cfg->hidden, st);
    default: return launch_router_hilo<16>(mw, mx, logits, status_word, n_tokens, cfg->n_experts, cfg->hidden, st);
  }
}

int msk_moe_route(const MskMoeCfg* cfg, const float* logits, const float* bias, int32_t* topk_ids,
                  float* topk_weights, int n_tokens, void* stream) {
  const int rc = check_cfg(cfg);
  if (rc != MSK_OK) return rc;
  if (!logits || !topk_ids || !topk_weights) return MSK_ERR_NULL;
  if (n_tokens < 0 || cfg->top_k > cfg->n_experts) return MSK_ERR_SHAPE;
  if (n_tokens == 0) return MSK_OK;
  route_topk_kernel<<<static_cast<unsigned>((n_tokens + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, bias, topk_ids, topk_weights, n_tokens, cfg->n_experts, cfg->top_k, cfg->routing_mode,
      cfg->route_scale);
  return static_cast<int>(cudaGetLastError());
}

static int launch_sort(const MskMoeCfg* cfg, const int32_t* ids, int n_tokens, int32_t* cnt, int32_t* off,
                       int32_t* perm, int32_t* inv, cudaStream_t st, const __nv_bfloat16* x = nullptr,
                       __half* xh = nullptr, int32_t* blk = nullptr, const void* pre_w = nullptr, float pre_eps = 0.f) {
  const int n_entries = n_tokens * cfg->top_k;
  if (blk != nullptr && xh == nullptr && n_entries >= SORT_MULTI_MIN) {
    // many entries: the same stable sort on several CTAs (count, scan, scatter)
    const int nb = SORT_MULTI_BLOCKS;
    sort_multi_count_kernel<<<nb, SORT_THREADS, sizeof(SortSmem), st>>>(ids, n_entries, cfg->local_start,
                                                                        cfg->local_count, blk);
    sort_multi_scan_kernel<<<1, MAX_LOCAL_EXPERTS, 0, st>>>(blk, nb, cfg->local_count, cnt, off);
    sort_multi_scatter_kernel<<<nb, SORT_THREADS, sizeof(SortSmem), st>>>(ids, n_entries, cfg->local_start,
                                                                          cfg->local_count, blk, perm, inv);
    return static_cast<int>(cudaGetLastError());
  }
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(sizeof(SortSmem)));
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3(1);
  lc.blockDim = dim3(SORT_THREADS);
  lc.dynamicSmemBytes = sizeof(SortSmem);
  lc.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&lc, sort_kernel, ids, static_cast<int>(n_tokens * cfg->top_k),
                                             static_cast<int>(cfg->local_start), static_cast<int>(cfg->local_count),
                                             cnt, off, perm, inv, x, xh, n_tokens, static_cast<int>(cfg->hidden),
                                             static_cast<const __nv_bfloat16*>(pre_w), pre_eps));
}

constexpr int FUSED_ROUTE_MAX_TOKENS = 32;  // up to here one CTA routes and sorts in a single launch

static int launch_route_sort(const MskMoeCfg* cfg, const float* logits, const float* bias, int32_t* ids, float* tw,
                             int n_tokens, int32_t* cnt, int32_t* off, int32_t* perm, int32_t* inv, cudaStream_t st,
                             const __nv_bfloat16* x, __half* xh, const void* pre_w = nullptr, float pre_eps = 0.f) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(route_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(sizeof(SortSmem)));
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3(1);
  lc.blockDim = dim3(SORT_THREADS);
  lc.dynamicSmemBytes = sizeof(SortSmem);
  lc.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&lc, route_sort_kernel, logits, bias, ids, tw, n_tokens,
                                             static_cast<int>(cfg->n_experts), static_cast<int>(cfg->top_k),
                                             static_cast<int>(cfg->routing_mode), cfg->route_scale,
                                             static_cast<int>(cfg->local_start), static_cast<int>(cfg->local_count),
                                             cnt, off, perm, inv, x, xh, static_cast<int>(cfg->hidden),
                                             static_cast<const __nv_bfloat16*>(pre_w), pre_eps));
}

int msk_moe_sort(const MskMoeCfg* cfg, const int32_t* topk_ids, int n_tokens, int32_t* cnt, int32_t* off,
                 int32_t* perm, int32_t* inv, void* stream) {
  const int rc = check_cfg(cfg);
  if (rc != MSK_OK) return rc;
  if (!cnt || !off || !perm || !inv) return MSK_ERR_NULL;
  if (n_tokens < 0) return MSK_ERR_SHAPE;
  if (n_tokens > 0 && !topk_ids) return MSK_ERR_NULL;
  return launch_sort(cfg, topk_ids, n_tokens, cnt, off, perm, inv, static_cast<cudaStream_t>(stream));
}

int msk_moe_workspace_bytes(const MskMoeCfg* cfg, size_t* host_bytes) {
  const int rc = check_cfg(cfg);
  if (rc != MSK_OK) return rc;
  if (!host_bytes) return MSK_ERR_NULL;
  if (cfg->max_tokens < 1) return MSK_ERR_SHAPE;
  *host_bytes = carve(cfg, cfg->max_tokens).total;
  return MSK_OK;
}

int msk_moe_workspace_init(const MskMoeCfg* cfg, void* workspace, size_t workspace_bytes, void* stream) {
  const int rc = check_cfg(cfg);
  if (rc != MSK_OK) return rc;
  if (!workspace) return MSK_ERR_NULL;
  if (cfg->max_tokens < 1) return MSK_ERR_SHAPE;
  const Carve k = carve(cfg, cfg->max_tokens);
  if (k.total > workspace_bytes) return MSK_ERR_WORKSPACE;
  // status word, tables and split-K tickets all sit below `inter`
  return static_cast<int>(cudaMemsetAsync(workspace, 0, k.inter, static_cast<cudaStream_t>(stream)));
}

int msk_moe_workspace_view(const MskMoeCfg* cfg, void* workspace, int which, void** host_ptr) {
  const int rc = check_cfg(cfg);
  if (rc != MSK_OK) return rc;
  if (!workspace || !host_ptr) return MSK_ERR_NULL;
  if (cfg->max_tokens < 1) return MSK_ERR_SHAPE;
  const Carve k = carve(cfg, cfg->max_tokens);
  uint8_t* b = static_cast<uint8_t*>(workspace);
  switch (which) {
    case 0: *host_ptr = b + k.cnt; break;
    case 1: *host_ptr = b + k.off; break;
    case 2: *host_ptr = b + k.perm; break;
    case 3: *host_ptr = b + k.inv; break;
    case 4: *host_ptr = b + k.inter; break;
    case 5: *host_ptr = b + k.y; break;
    case 6: *host_ptr = b + k.trace; break;
    case 7: *host_ptr = b + k.tickets; break;
    case 8: *host_ptr = b + k.few_ctl; break;
    case 9: *host_ptr = b + k.sort_blk; break;
    case 10: *host_ptr = b + k.tile_ctr; break;
    default: return MSK_ERR_SHAPE;
  }
  return MSK_OK;
}

// ev, when given, holds 6 events: [0] before the step, [1] after routing + sort, [5] after the row copy,
// [2] after the gate/up GEMM, [3] after the down GEMM, [4] after the combine.
static int forward_impl(const MskMoeCfg* cfg, const void* packed13, const void* packed2, const float* gs13,
                        const float* gs2, const void* post_norm_w, const void* x, const int32_t* topk_ids,
                        const float* topk_weights, void* out, void* workspace, size_t workspace_bytes, int n_tokens,
                        void* stream, cudaEvent_t* ev, const float* logits = nullptr, const float* bias = nullptr,
                        int32_t* ids_out = nullptr, float* tw_out = nullptr, const void* pre_norm_w = nullptr,
                        float pre_norm_eps = 1e-5f) {
  // with `logits` the routing runs here too: ids_out / tw_out receive it and feed the rest
  if (logits != nullptr) {
    if (!ids_out || !tw_out) return MSK_ERR_NULL;
    topk_ids = ids_out;
    topk_weights = tw_out;
  }
  const int rc = check_cfg(cfg);
  if (rc != MSK_OK) return rc;
  if (!packed13 || !packed2 || !gs13 || !gs2 || !workspace) return MSK_ERR_NULL;
  if (n_tokens < 0) return MSK_ERR_SHAPE;
  if (n_tokens == 0) return MSK_OK;
  if (!x || !topk_ids || !topk_weights || !out) return MSK_ERR_NULL;
  if (!aligned16(packed13) || !aligned16(packed2) || !aligned16(x) || !aligned16(out) || !aligned16(workspace))
    return MSK_ERR_ALIGN;
  if (n_tokens > cfg->max_tokens) return MSK_ERR_TOO_LARGE;
  // offsets depend on the capacity only, so control words keep their place from call to call
  const Carve k = carve(cfg, cfg->max_tokens);
  if (k.total > workspace_bytes) return MSK_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* b = static_cast<uint8_t*>(workspace);
  int32_t* status = reinterpret_cast<int32_t*>(b + k.status);
  int32_t* cnt = reinterpret_cast<int32_t*>(b + k.cnt);
  int32_t* off = reinterpret_cast<int32_t*>(b + k.off);
  int32_t* perm = reinterpret_cast<int32_t*>(b + k.perm);
  int32_t* inv = reinterpret_cast<int32_t*>(b + k.inv);
  int32_t* tickets = reinterpret_cast<int32_t*>(b + k.tickets);
  __half* inter = reinterpret_cast<__half*>(b + k.inter);
  float* y = reinterpret_cast<float*>(b + k.y);
  float* partial = reinterpret_cast<float*>(b + k.partial);
  __half* xs = reinterpret_cast<__half*>(b + k.xs);

  Plan plan = make_plan(cfg, n_tokens);
  if (plan.N != 16 && plan.N != 32 && plan.N != 64 && plan.N != 128) return MSK_ERR_SHAPE;
  if (plan.grid < 1 || plan.grid > MAX_CTAS) return MSK_ERR_SHAPE;
  const int pdl = cfg->no_pdl ? 0 : 1;
  const size_t r_max = static_cast<size_t>(cfg->max_tokens) * cfg->top_k;
  unsigned long long* trace = (cfg->trace != 0 && plan.grid <= static_cast<int>(TRACE_CTAS))
                                  ? reinterpret_cast<unsigned long long*>(b + k.trace) : nullptr;

  // what every launch of the two GEMMs shares
  GemmParams p{};
  p.cnt = cnt; p.off = off; p.perm = perm; p.inv = inv; p.status = status; p.trace = trace;
  p.nloc = cfg->local_count; p.top_k = cfg->top_k; p.flat = plan.flat;
  // weights stream through L2 once per token tile; the activation rows are what many CTAs re-read,
  // so the weights must not be the ones L2 keeps
  p.evict_first = 1;
  p.post_norm_w = static_cast<const __nv_bfloat16*>(post_norm_w);
  p.eps = cfg->post_norm_eps;
  PhaseParams& g13 = p.ph[0];
  PhaseParams& g2 = p.ph[1];
  g13.w = static_cast<const uint8_t*>(packed13); g13.gs = gs13; g13.act = xs; g13.outp = inter;
  g13.partial = partial; g13.tickets = tickets;
  g13.K = cfg->hidden; g13.out_ld = cfg->inter; g13.n_pairs = cfg->inter / 128;
  g2.w = static_cast<const uint8_t*>(packed2); g2.gs = gs2; g2.act = inter; g2.outp = y;
  g2.partial = partial + round_up(partial_floats(cfg) * 4, 256) / 4;
  g2.tickets = tickets + round_up(ticket_ints(cfg, cfg->max_tokens) * 4, 256) / 4;
  g2.K = cfg->inter; g2.out_ld = cfg->hidden; g2.n_pairs = cfg->hidden / 256;

  if (plan.path != 1 && plan.path != 4) {
    // ---- few tokens: the GEMM kernels route, sort and combine themselves
    p.route = logits != nullptr ? 1 : 2;
    p.logits = logits; p.bias = bias; p.ids_in = topk_ids; p.ids_out = ids_out; p.tw_out = tw_out;
    p.T = n_tokens; p.E = cfg->n_experts; p.lo = cfg->local_start; p.mode = cfg->routing_mode;
    p.route_scale = cfg->route_scale;
    p.fold = post_norm_w != nullptr ? 1 : 2; p.tw = topk_weights; p.out = static_cast<__nv_bfloat16*>(out);
    p.tok_tickets = reinterpret_cast<int32_t*>(b + k.few_ctl);
    p.grid_bar = reinterpret_cast<unsigned int*>(b + k.few_ctl + 4096);
    p.tile_done = reinterpret_cast<unsigned int*>(b + k.few_ctl + 4352);
    p.tile_seen = p.tile_done + 384;
    p.x_bf16 = static_cast<const __nv_bfloat16*>(x);
    if (ev) { cudaEventRecord(ev[0], st); cudaEventRecord(ev[1], st); }
    if (plan.path == 0 && pre_norm_w == nullptr) {
      if (ev) cudaEventRecord(ev[5], st);
      const int e1 = launch_gemm_fused(plan.N, p, plan.grid, st);
      if (ev) { cudaEventRecord(ev[2], st); cudaEventRecord(ev[3], st); cudaEventRecord(ev[4], st); }
      return e1;
    }
    // F16 copy of the token rows (with the pre-expert norm when asked for), small blocks so that the
    // gate/up kernel's CTAs fit beside them; it waits for what precedes the step and lets go of its
    // dependents after that wait
    int e = 0;
    {
      const bool pre = pre_norm_w != nullptr;
      cudaLaunchConfig_t lc{};
      lc.stream = st;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      at[0].val.programmaticStreamSerializationAllowed = pdl;
      lc.attrs = at;
      lc.numAttrs = 1;
      if (pre) {
        lc.gridDim = dim3(static_cast<unsigned>(n_tokens));
        lc.blockDim = dim3(256);
        e = static_cast<int>(cudaLaunchKernelEx(&lc, gather_rows_kernel, static_cast<const __nv_bfloat16*>(x),
                                                static_cast<const int32_t*>(perm), static_cast<const int32_t*>(off),
                                                static_cast<int>(cfg->local_count), static_cast<int>(cfg->top_k),
                                                static_cast<int>(cfg->hidden), 0, xs,
                                                static_cast<const __nv_bfloat16*>(pre_norm_w), pre_norm_eps));
      } else {
        const int n8 = n_tokens * (cfg->hidden / 8);
        lc.gridDim = dim3(static_cast<unsigned>((n8 + 63) / 64));
        lc.blockDim = dim3(64);
        e = static_cast<int>(cudaLaunchKernelEx(&lc, convert_rows_kernel, static_cast<const __nv_bfloat16*>(x), xs, n8));
      }
      if (e != 0) return e;
    }
    if (ev) cudaEventRecord(ev[5], st);
    e = launch_gemm_n<0>(plan.N, p, plan.grid, st, pdl);
    if (e != 0) return e;
    if (ev) cudaEventRecord(ev[2], st);
    if (trace) p.trace = trace + TRACE_WORDS;
    e = launch_gemm_n<1>(plan.N, p, plan.grid, st, pdl);
    if (ev) { cudaEventRecord(ev[3], st); cudaEventRecord(ev[4], st); }
    return e;
  }

  // ---- chain of launches: [top-k +] sort, [row copy,] gate/up GEMM, down GEMM, combine
  if (ev) cudaEventRecord(ev[0], st);
  int e = 0;
  // narrow token tiles read an F16 copy of x; for few tokens the sorting CTA makes it
  const bool tma_b = plan.N >= 64;  // GemmCfg<N>::TMA_B
  const bool both_gemms = plan.path == 4 && pre_norm_w == nullptr;   // the pre-expert norm needs the row-copy kernel
  const bool convert_in_sort = !tma_b && !both_gemms && n_tokens <= FUSED_ROUTE_MAX_TOKENS;
  const __nv_bfloat16* xin = convert_in_sort ? static_cast<const __nv_bfloat16*>(x) : nullptr;
  __half* xh_in_sort = convert_in_sort ? xs : nullptr;
  if (logits != nullptr && n_tokens <= FUSED_ROUTE_MAX_TOKENS) {
    e = launch_route_sort(cfg, logits, bias, ids_out, tw_out, n_tokens, cnt, off, perm, inv, st, xin, xh_in_sort,
                          pre_norm_w, pre_norm_eps);
  } else {
    if (logits != nullptr) {
      route_topk_kernel<<<static_cast<unsigned>((n_tokens + 7) / 8), 256, 0, st>>>(
          logits, bias, ids_out, tw_out, n_tokens, cfg->n_experts, cfg->top_k, cfg->routing_mode, cfg->route_scale);
      e = static_cast<int>(cudaGetLastError());
      if (e != 0) return e;
    }
    e = launch_sort(cfg, topk_ids, n_tokens, cnt, off, perm, inv, st, xin, xh_in_sort,
                    reinterpret_cast<int32_t*>(b + k.sort_blk), pre_norm_w, pre_norm_eps);
  }
  if (e != 0) return e;
  if (ev) cudaEventRecord(ev[1], st);
  if (cfg->stop_after == 1) return MSK_OK;

  if (both_gemms) {
    p.route = 0; p.fold = 0; p.flat = 0;
    p.x_bf16 = static_cast<const __nv_bfloat16*>(x);
    p.T = n_tokens;
    p.grid_bar = reinterpret_cast<unsigned int*>(b + k.few_ctl + 4096);
    p.tile_done = reinterpret_cast<unsigned int*>(b + k.tile_ctr);
    p.tile_seen = p.tile_done + max_tiles(cfg, cfg->max_tokens);
    if (ev) cudaEventRecord(ev[5], st);
    e = launch_gemm_fused(plan.N, p, plan.grid, st);
    if (e != 0) return e;
    if (ev) { cudaEventRecord(ev[2], st); cudaEventRecord(ev[3], st); }
  } else {
  if (!convert_in_sort) {
    // F16 copy of the token rows: sorted (expert-major) for the TMA tiles, plain [T, H] otherwise
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3(static_cast<unsigned>(tma_b ? n_tokens * cfg->top_k : n_tokens));
    lc.blockDim = dim3(256);
    lc.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl;
    lc.attrs = at;
    lc.numAttrs = 1;
    if (tma_b && pre_norm_w == nullptr) {
      lc.gridDim = dim3(static_cast<unsigned>(std::min<long long>((static_cast<long long>(n_tokens) * cfg->top_k + 7) / 8,
                                                                  8LL * sm_count())));
      e = static_cast<int>(cudaLaunchKernelEx(&lc, gather_rows_sorted_kernel, static_cast<const __nv_bfloat16*>(x),
                                              static_cast<const int32_t*>(perm), static_cast<const int32_t*>(off),
                                              static_cast<int>(cfg->local_count), static_cast<int>(cfg->top_k),
                                              static_cast<int>(cfg->hidden), xs));
    } else {
      e = static_cast<int>(cudaLaunchKernelEx(&lc, gather_rows_kernel, static_cast<const __nv_bfloat16*>(x),
                                              static_cast<const int32_t*>(perm), static_cast<const int32_t*>(off),
                                              static_cast<int>(cfg->local_count), static_cast<int>(cfg->top_k),
                                              static_cast<int>(cfg->hidden), tma_b ? 1 : 0, xs,
                                              static_cast<const __nv_bfloat16*>(pre_norm_w), pre_norm_eps));
    }
    if (e != 0) return e;
    if (tma_b) {
      e = encode_act_map(&p.tmap_act[0], xs, r_max, cfg->hidden, plan.N);
      if (e != 0) return e;
      e = encode_act_map(&p.tmap_act[1], inter, r_max, cfg->inter, plan.N);
      if (e != 0) return e;
    }
  }
  if (ev) cudaEventRecord(ev[5], st);
  p.y_bf16 = plan.N == 128 ? 1 : 0;  // the wide tile: half the y bytes written and read back
  // Tile hand-over: the down GEMM's CTAs start on the SMs the gate/up CTAs leave (programmatic launch) and
  // would then wait for that whole grid, whose last CTAs run a unit longer than the others (the units do not
  // divide evenly): a tenth of the gate/up time with every SM but a few idle. Instead each down unit waits
  // for the gate/up units of its own token tile, and the blocks that start last are dealt fewer down units.
  // Needs every gate/up CTA resident while down CTAs wait (grid within the SM count: a waiting CTA must not
  // keep a producing one off the machine), whole units (a cut unit would be counted once per piece) and
  // both launches of the step. Narrow token tiles only, where the gather warp does the waiting: measured at
  // H4096 I1536 E128, 16 / 32 / 64 / 128 tokens take 187 / 242 / 257 / 270 us with it against 190 / 248 /
  // 266 / 274 without. With the wide tiles, whose weight producer also fetches the activation tiles and so
  // would stand still at every new token tile, the same hand-over was slower (256 tokens 326 against 320 us,
  // 8192 tokens 2.62 against 2.58 ms) and is not built.
  p.handover = (pdl != 0 && !tma_b && plan.flat == 0 && plan.grid <= sm_count() && cfg->stop_after == 0) ? 1 : 0;
  if (handover_env_off()) p.handover = 0;
  p.tile_done = reinterpret_cast<unsigned int*>(b + k.tile_ctr);
  p.tile_seen = p.tile_done + max_tiles(cfg, cfg->max_tokens);
  e = launch_gemm_n<0>(plan.N, p, plan.grid, st, pdl);
  if (e != 0) return e;
  if (ev) cudaEventRecord(ev[2], st);
  if (cfg->stop_after == 2) return MSK_OK;

  if (trace) p.trace = trace + TRACE_WORDS;
  e = launch_gemm_n<1>(plan.N, p, plan.grid, st, pdl);
  if (e != 0) return e;
  if (ev) cudaEventRecord(ev[3], st);
  if (cfg->stop_after == 3) return MSK_OK;
  }

  {
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3(static_cast<unsigned>(n_tokens));
    lc.blockDim = dim3(COMBINE_THREADS);
    lc.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl;
    lc.attrs = at;
    lc.numAttrs = 1;
    const bool wide = n_tokens >= COMBINE_WIDE_TOKENS;
    const bool narrow_rows = cfg->hidden <= COMBINE_THREADS * 2 * 4;   // two float4 slots per thread hold a row
    auto* kern = p.y_bf16 ? (narrow_rows ? combine_kernel<8, true, 2, 2> : combine_kernel<4, true, 2>)
                          : (wide ? combine_kernel<2, false, 2> : combine_kernel<4, false, 1>);
    e = static_cast<int>(cudaLaunchKernelEx(&lc, kern, static_cast<const float*>(y),
                                            static_cast<const int32_t*>(inv), topk_weights,
                                            static_cast<__nv_bfloat16*>(out), static_cast<int>(cfg->hidden),
                                            static_cast<int>(cfg->top_k), post_norm_w != nullptr ? 1 : 0,
                                            cfg->post_norm_eps));
  }
  if (ev) cudaEventRecord(ev[4], st);
  return e;
}

int msk_moe_forward(const MskMoeCfg* cfg, const void* packed13, const void* packed2, const float* gs13,
                    const float* gs2, const void* post_norm_w, const void* x, const int32_t* topk_ids,
                    const float* topk_weights, void* out, void* workspace, size_t workspace_bytes, int n_tokens,
                    void* stream) {
  return forward_impl(cfg, packed13, packed2, gs13, gs2, post_norm_w, x, topk_ids, topk_weights, out, workspace,
                      workspace_bytes, n_tokens, stream, nullptr);
}

int msk_moe_forward_logits(const MskMoeCfg* cfg, const void* packed13, const void* packed2, const float* gs13,
                           const float* gs2, const void* post_norm_w, const void* x, const float* logits,
                           const float* bias, int32_t* topk_ids_out, float* topk_weights_out, void* out,
                           void* workspace, size_t workspace_bytes, int n_tokens, void* stream) {
  if (!logits) return MSK_ERR_NULL;
  if (cfg != nullptr && cfg->top_k > cfg->n_experts) return MSK_ERR_SHAPE;
  return forward_impl(cfg, packed13, packed2, gs13, gs2, post_norm_w, x, nullptr, nullptr, out, workspace,
                      workspace_bytes, n_tokens, stream, nullptr, logits, bias, topk_ids_out, topk_weights_out);
}

int msk_moe_forward_prenorm(const MskMoeCfg* cfg, const void* packed13, const void* packed2, const float* gs13,
                            const float* gs2, const void* post_norm_w, const void* pre_norm_w, float pre_norm_eps,
                            const void* x, const float* logits, const float* bias, int32_t* topk_ids,
                            float* topk_weights, void* out, void* workspace, size_t workspace_bytes, int n_tokens,
                            void* stream) {
  if (!pre_norm_w) return MSK_ERR_NULL;
  if (!aligned16(pre_norm_w)) return MSK_ERR_ALIGN;
  if (!(pre_norm_eps > 0.f)) return MSK_ERR_SHAPE;
  if (cfg != nullptr && cfg->hidden > 8192) return MSK_ERR_TOO_LARGE;   // a row is held in registers by 256 threads
  if (logits != nullptr) {
    if (cfg != nullptr && cfg->top_k > cfg->n_experts) return MSK_ERR_SHAPE;
    return forward_impl(cfg, packed13, packed2, gs13, gs2, post_norm_w, x, nullptr, nullptr, out, workspace,
                        workspace_bytes, n_tokens, stream, nullptr, logits, bias, topk_ids, topk_weights, pre_norm_w,
                        pre_norm_eps);
  }
  return forward_impl(cfg, packed13, packed2, gs13, gs2, post_norm_w, x, topk_ids, topk_weights, out, workspace,
                      workspace_bytes, n_tokens, stream, nullptr, nullptr, nullptr, nullptr, nullptr, pre_norm_w,
                      pre_norm_eps);
}

int msk_moe_forward_timed(const MskMoeCfg* cfg, const void* packed13, const void* packed2, const float* gs13,
                          const float* gs2, const void* post_norm_w, const void* x, const int32_t* topk_ids,
                          const float* topk_weights, void* out, void* workspace, size_t workspace_bytes,
                          int n_tokens, void* stream, float* host_ms) {
  if (!host_ms) return MSK_ERR_NULL;
  static cudaEvent_t ev[64][6];
  static bool made[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MSK_ERR_RANGE;
  if (!made[dev]) {
    for (int i = 0; i < 6; ++i) {
      cudaError_t ce = cudaEventCreate(&ev[dev][i]);
      if (ce != cudaSuccess) return static_cast<int>(ce);
    }
    made[dev] = true;
  }
  const int rc = forward_impl(cfg, packed13, packed2, gs13, gs2, post_norm_w, x, topk_ids, topk_weights, out,
                              workspace, workspace_bytes, n_tokens, stream, ev[dev]);
  if (rc != 0) return rc;
  cudaError_t ce = cudaEventSynchronize(ev[dev][4]);
  if (ce != cudaSuccess) return static_cast<int>(ce);
  const int from[5] = {0, 1, 5, 2, 3}, to[5] = {1, 5, 2, 3, 4};  // sort, row copy, gate/up, down, combine
  for (int i = 0; i < 5; ++i) {
    ce = cudaEventElapsedTime(&host_ms[i], ev[dev][from[i]], ev[dev][to[i]]);
    if (ce != cudaSuccess) return static_cast<int>(ce);
  }
  return MSK_OK;
}

// ------------------------------------------------------------------------------------------
// msk_moe_forward_static: the routed-expert step for callers that cannot allocate.
// Some hosts of this library run where no device allocation may happen on the calling path:
// a serving loop that has handed all device memory to its own pool, a plug-in called while the
// application's allocator is locked, a latency-critical thread that must not enter the driver's
// allocator.
// msk_moe_forward needs a caller-allocated workspace; this variant keeps its scratch (sort
// tables, the F16 copy of the token rows, the SwiGLU intermediate and the per-route expert outputs) in one file-scope device
// array instead. The array is part of the loaded library image: every GPU that loads the
// library holds MSK_STATIC_WS_BYTES of it until the process exits.
//  * Limits: n_tokens * top_k <= 128 routed rows, hidden <= 8192, inter <= 4096; anything
//    larger is refused with MSK_ERR_TOO_LARGE. The GEMMs run on whole units here (no cut units, no pieces).
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress,
//    with that device current). Make that first call outside stream capture.
//  * All calls on a device share the one array and it keeps what the last call left; the status
//    word is cleared on the stream at the start of every call, the tables are rewritten by the
//    sort. Two calls that overlap on the GPU (different streams) race on it: serialise them.
//  * No cudaMalloc, cudaFree or allocating library call is made.
constexpr size_t MSK_STATIC_WS_BYTES = 8u << 20;
constexpr int MSK_STATIC_MAX_ROWS = 128;
static __device__ __align__(256) unsigned char g_static_ws[MSK_STATIC_WS_BYTES];

// Device address of the array on the current device, looked up once per device (in host code the
// symbol's name is a host-side stand-in, not a device address).
static int static_ws_base(unsigned char** out) {
  static unsigned char* base_of[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MSK_ERR_RANGE;
  if (base_of[dev] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t ce = cudaGetSymbolAddress(&ptr, g_static_ws);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    base_of[dev] = static_cast<unsigned char*>(ptr);
  }
  *out = base_of[dev];
  return 0;
}

int msk_moe_static_status(int* host_status, void* stream) {
  if (!host_status) return MSK_ERR_NULL;
  unsigned char* b = nullptr;
  const int ar = static_ws_base(&b);
  if (ar != 0) return ar;
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemcpy(host_status, b, sizeof(int), cudaMemcpyDeviceToHost);
  return static_cast<int>(e);
}

int msk_moe_forward_static(const MskMoeCfg* cfg, const void* packed13, const void* packed2, const float* gs13,
                           const float* gs2, const void* post_norm_w, const void* x, const int32_t* topk_ids,
                           const float* topk_weights, void* out, int n_tokens, void* stream) {
  const int rc = check_cfg(cfg);
  if (rc != MSK_OK) return rc;
  if (!packed13 || !packed2 || !gs13 || !gs2) return MSK_ERR_NULL;
  if (n_tokens < 0) return MSK_ERR_SHAPE;
  if (n_tokens == 0) return MSK_OK;
  if (!x || !topk_ids || !topk_weights || !out) return MSK_ERR_NULL;
  if (!aligned16(packed13) || !aligned16(packed2) || !aligned16(x) || !aligned16(out)) return MSK_ERR_ALIGN;
  const size_t R = static_cast<size_t>(n_tokens) * cfg->top_k;
  if (R > static_cast<size_t>(MSK_STATIC_MAX_ROWS) || cfg->hidden > 8192 || cfg->inter > 4096) return MSK_ERR_TOO_LARGE;
  // carve: [status 256][cnt][off][perm][inv][inter f16 R x I][y fp32 R x H][x as f16 T x H]
  size_t o = 256;
  const size_t o_cnt = o; o += round_up(static_cast<size_t>(cfg->local_count) * 4, 256);
  const size_t o_off = o; o += round_up(static_cast<size_t>(cfg->local_count + 1) * 4, 256);
  const size_t o_perm = o; o += round_up(R * 4, 256);
  const size_t o_inv = o; o += round_up(R * 4, 256);
  const size_t o_inter = o; o += round_up(R * cfg->inter * 2, 256);
  const size_t o_y = o; o += round_up(R * cfg->hidden * 4, 256);
  const size_t o_xh = o; o += round_up(static_cast<size_t>(n_tokens) * cfg->hidden * 2, 256);
  if (o > MSK_STATIC_WS_BYTES) return MSK_ERR_TOO_LARGE;

  unsigned char* b = nullptr;
  const int ar = static_ws_base(&b);
  if (ar != 0) return ar;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t ce = cudaMemsetAsync(b, 0, 256, st);  // status word starts at zero
  if (ce != cudaSuccess) return static_cast<int>(ce);

  int32_t* cnt = reinterpret_cast<int32_t*>(b + o_cnt);
  int32_t* off = reinterpret_cast<int32_t*>(b + o_off);
  int32_t* perm = reinterpret_cast<int32_t*>(b + o_perm);
  int32_t* inv = reinterpret_cast<int32_t*>(b + o_inv);
  __half* inter = reinterpret_cast<__half*>(b + o_inter);
  float* y = reinterpret_cast<float*>(b + o_y);
  __half* xh = reinterpret_cast<__half*>(b + o_xh);

  int e = launch_sort(cfg, topk_ids, n_tokens, cnt, off, perm, inv, st);
  if (e != 0) return e;
  gather_rows_kernel<<<static_cast<unsigned>(n_tokens), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), perm, off, cfg->local_count, cfg->top_k, cfg->hidden, 0, xh, nullptr, 0.f);
  e = static_cast<int>(cudaGetLastError());
  if (e != 0) return e;
  GemmParams p{};
  p.cnt = cnt; p.off = off; p.perm = perm; p.inv = inv;
  p.status = reinterpret_cast<int32_t*>(b); p.trace = nullptr;
  p.nloc = cfg->local_count; p.top_k = cfg->top_k; p.evict_first = 1;
  p.flat = 0;  // whole units only: no pieces, so no partial buffer and no tickets
  p.post_norm_w = static_cast<const __nv_bfloat16*>(post_norm_w);
  const int grid = cfg->num_ctas > 0 ? std::min(cfg->num_ctas, MAX_CTAS) : DEFAULT_CTAS;
  p.ph[0].w = static_cast<const uint8_t*>(packed13); p.ph[0].gs = gs13; p.ph[0].act = xh; p.ph[0].outp = inter;
  p.ph[0].K = cfg->hidden; p.ph[0].out_ld = cfg->inter; p.ph[0].n_pairs = cfg->inter / 128;
  p.ph[1].w = static_cast<const uint8_t*>(packed2); p.ph[1].gs = gs2; p.ph[1].act = inter; p.ph[1].outp = y;
  p.ph[1].K = cfg->inter; p.ph[1].out_ld = cfg->hidden; p.ph[1].n_pairs = cfg->hidden / 256;
  e = launch_gemm_n<0>(16, p, grid, st, 1);
  if (e != 0) return e;
  e = launch_gemm_n<1>(16, p, grid, st, 1);
  if (e != 0) return e;
  combine_kernel<4, false, 1><<<static_cast<unsigned>(n_tokens), COMBINE_THREADS, 0, st>>>(
      y, inv, topk_weights, static_cast<__nv_bfloat16*>(out), cfg->hidden, cfg->top_k, post_norm_w != nullptr ? 1 : 0,
      cfg->post_norm_eps);
  return static_cast<int>(cudaGetLastError());
}

int msk_moe_share_pieces(int n_base, int n_stages, int shares, int flat, int cta, int heavy, int skip, int* host_out,
                         int capacity, int* host_count) {
  if (!host_out || !host_count) return MSK_ERR_NULL;
  if (n_base < 0 || n_stages < 1 || shares < 1 || cta < 0 || cta >= shares || capacity < 0 || heavy < 0 || heavy >= shares ||
      skip < 0)
    return MSK_ERR_SHAPE;
  if (static_cast<long long>(n_base) * n_stages * shares >= FLAT_MAX_PRODUCT) return MSK_ERR_TOO_LARGE;
  PieceIter it = make_piece_iter(flat, n_base, n_stages, cta, shares, heavy, skip);
  const int items = (n_base - it.tail_base) * n_stages;
  int n = 0, base, ks0, ks1;
  while (it.next(base, ks0, ks1)) {
    if (n < capacity) {
      int* o = host_out + 6 * n;
      const bool whole = ks0 == 0 && ks1 == n_stages;
      const int b0 = (base - it.tail_base) * n_stages;
      o[0] = base; o[1] = ks0; o[2] = ks1;
      o[3] = whole ? -1 : piece_slot(cta, ks0 == 0);
      o[4] = whole ? cta : share_owner(items, shares, b0);
      o[5] = whole ? cta : share_owner(items, shares, b0 + n_stages - 1);
    }
    ++n;
  }
  *host_count = n;
  return n <= capacity ? MSK_OK : MSK_ERR_TOO_LARGE;
}

// L2 sweep for cold-cache timing: every thread reads 16-byte words of the buffer with ordinary loads,
// so the lines land in L2 clean and displace what was there. (Zeroing a buffer also displaces it, but
// leaves L2 full of dirty lines whose write-back then competes with the kernel being timed; the
// reference sweeps by reading for the same reason, muse_decode_layer/py/05_tune.py:74-94.)
__global__ void __launch_bounds__(256) l2_sweep_kernel(const uint4* __restrict__ buf, size_t n16, uint32_t* sink) {
  uint32_t acc = 0;
  for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < n16; i += static_cast<size_t>(gridDim.x) * 256) {
    const uint4 v = buf[i];
    acc ^= v.x ^ v.y ^ v.z ^ v.w;
  }
  if (acc == 0x9E3779B9u) atomicAdd(sink, acc);  // keeps the loads alive
}

int msk_l2_sweep(const void* buf, size_t bytes, uint32_t* sink, void* stream) {
  if (!buf || !sink) return MSK_ERR_NULL;
  if (!aligned16(buf)) return MSK_ERR_ALIGN;
  if (bytes < 16) return MSK_OK;
  l2_sweep_kernel<<<1184, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(buf), bytes / 16, sink);
  return static_cast<int>(cudaGetLastError());
}

#ifndef MSK_BUILD_ID
#define MSK_BUILD_ID "unknown"
#endif
const char* msk_build_id(void) { return MSK_BUILD_ID; }

int msk_moe_plan(const MskMoeCfg* cfg, int n_tokens, int* host_out) {
  const int rc = check_cfg(cfg);
  if (rc != MSK_OK) return rc;
  if (!host_out) return MSK_ERR_NULL;
  if (n_tokens < 1) return MSK_ERR_SHAPE;
  const Plan plan = make_plan(cfg, n_tokens);
  host_out[0] = plan.N; host_out[1] = plan.path; host_out[2] = plan.flat; host_out[3] = plan.grid;
  return MSK_OK;
}

int msk_moe_read_status(const void* workspace, int* host_status, void* stream) {
  if (!workspace || !host_status) return MSK_ERR_NULL;
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemcpy(host_status, workspace, sizeof(int), cudaMemcpyDeviceToHost);
  return static_cast<int>(e);
}

int msk_moe_attrs(int which, int token_tile, int* host_out) {
  if (!host_out) return MSK_ERR_NULL;
  cudaFuncAttributes a{};
  cudaError_t e = cudaSuccess;
  switch (which) {
    case 0: e = cudaFuncGetAttributes(&a, sort_kernel); break;
    case 1: e = cudaFuncGetAttributes(&a, route_topk_kernel); break;
    case 2:
    case 3: {
      const bool ph1 = which == 3;
      switch (token_tile) {
        case 16: e = ph1 ? cudaFuncGetAttributes(&a, moe_gemm_kernel<16, 1>) : cudaFuncGetAttributes(&a, moe_gemm_kernel<16, 0>); break;
        case 32: e = ph1 ? cudaFuncGetAttributes(&a, moe_gemm_kernel<32, 1>) : cudaFuncGetAttributes(&a, moe_gemm_kernel<32, 0>); break;
        case 64: e = ph1 ? cudaFuncGetAttributes(&a, moe_gemm_kernel<64, 1>) : cudaFuncGetAttributes(&a, moe_gemm_kernel<64, 0>); break;
        case 128: e = ph1 ? cudaFuncGetAttributes(&a, moe_gemm_kernel<128, 1>) : cudaFuncGetAttributes(&a, moe_gemm_kernel<128, 0>); break;
        default: return MSK_ERR_SHAPE;
      }
      break;
    }
    case 4: e = cudaFuncGetAttributes(&a, combine_kernel<4, false, 1>); break;
    default: return MSK_ERR_SHAPE;
  }
  if (e != cudaSuccess) return static_cast<int>(e);
  host_out[0] = a.numRegs;
  host_out[1] = static_cast<int>(a.sharedSizeBytes);
  host_out[2] = a.maxDynamicSharedSizeBytes;
  host_out[3] = static_cast<int>(a.localSizeBytes);
  return MSK_OK;
}

int msk_ep_combine(const void* back, const void* self_rows, int self_rank, const int32_t* ids, int top_k,
                   int experts_per_rank, void* out, int n_ranks, int n_tokens, int hidden, void* stream) {
  if (!back || !ids || !out) return MSK_ERR_NULL;
  if (n_ranks < 1 || n_ranks > 64 || n_tokens < 0 || hidden < 8 || hidden % 8 != 0 || top_k < 1 ||
      top_k > MAX_TOP_K || experts_per_rank < 1)
    return MSK_ERR_SHAPE;
  if (!aligned16(back) || !aligned16(out) || (self_rows && !aligned16(self_rows))) return MSK_ERR_ALIGN;
  if (n_tokens == 0) return MSK_OK;
  ep_combine_kernel<<<static_cast<unsigned>(n_tokens), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(back), static_cast<const __nv_bfloat16*>(self_rows), self_rank, ids, top_k,
      experts_per_rank, static_cast<__nv_bfloat16*>(out), n_ranks, n_tokens, hidden);
  return static_cast<int>(cudaGetLastError());
}

int msk_ep_flag_write(void* addr, uint32_t value, void* stream) {
  if (!addr) return MSK_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(addr) % 4 != 0) return MSK_ERR_ALIGN;
  return stream_value32("cuStreamWriteValue32", addr, value, CU_STREAM_WRITE_VALUE_DEFAULT, stream);
}

int msk_ep_flag_wait(void* addr, uint32_t value, void* stream) {
  if (!addr) return MSK_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(addr) % 4 != 0) return MSK_ERR_ALIGN;
  return stream_value32("cuStreamWaitValue32", addr, value, CU_STREAM_WAIT_VALUE_GEQ, stream);
}

int msk_bw_probe(const void* src, size_t bytes, int stages, int stage_bytes, int num_ctas, uint32_t* sink,
                 int skip_release, void* stream) {
  if (!src || !sink) return MSK_ERR_NULL;
  if (!aligned16(src)) return MSK_ERR_ALIGN;
  if (stages < 1 || stages > 8 || stage_bytes < 16 || stage_bytes % 16 != 0) return MSK_ERR_SHAPE;
  const size_t smem = static_cast<size_t>(stages) * stage_bytes;
  if (smem > 220 * 1024) return MSK_ERR_TOO_LARGE;
  const int grid = num_ctas > 0 ? num_ctas : sm_count();
  cudaError_t e = cudaFuncSetAttribute(bw_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  bw_probe_kernel<<<grid, 64, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), static_cast<unsigned long long>(bytes), stages, stage_bytes, sink, skip_release);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
