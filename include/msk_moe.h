/*
 * msk_moe.h -- C ABI of the B200 (sm_100a) routed-expert step `muse_moe_w4a16`:
 * top-k routing, stable token permutation, NVFP4-weight x BF16-activation grouped
 * SwiGLU experts, deterministic top-k-weighted combine.
 *
 * This library is what the reference module's native binding would bind for this
 * path. The reference boundary it replaces is the pybind trio
 *     okc_run(w, scratch, x, ids, tw, out, lo, nloc, grid) / okc_set_pdl / okc_attrs
 * (muse_moe_w4a16/py/00_moe_w4a16.py:208-214, launcher muse_moe_w4a16/cuda/moe.cu:2796-2881),
 * restated with plain pointers and sizes: no torch types, no exceptions, no host
 * synchronisation (except where a function says so), every launch on the stream given.
 *
 * Conventions
 *  - every function returns an int status: 0 = ok, negative = rejected on the host
 *    before any launch (MSK_ERR_*), positive = cudaError_t of a failed launch;
 *  - all pointers are device pointers unless named host_*; `stream` is a cudaStream_t
 *    passed as void*;
 *  - device-side waits are bounded; a kernel that gives up writes a non-zero code to
 *    word 0 of the workspace (see msk_moe_read_status) and exits, it never traps.
 */
#ifndef MSK_MOE_H_
#define MSK_MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MSK_OK 0
#define MSK_ERR_NULL (-1)        /* a required pointer is NULL */
#define MSK_ERR_SHAPE (-2)       /* unsupported shape (see MskMoeCfg) */
#define MSK_ERR_ALIGN (-3)       /* pointer not 16-byte aligned */
#define MSK_ERR_WORKSPACE (-4)   /* workspace too small */
#define MSK_ERR_RANGE (-5)       /* local expert range outside [0, n_experts) */
#define MSK_ERR_TOO_LARGE (-6)   /* size beyond a stated maximum */

/* Routing score function (msk_moe_route). */
#define MSK_ROUTE_SOFTMAX_TOPK 0 /* select by logit, weights = softmax over the k selected logits */
#define MSK_ROUTE_SIGMOID_BIAS 1 /* s = sigmoid(logit * route_scale); select by s + bias; w = s / (sum s + 1e-15) */

/* Shapes and options. Mirrors the reference's `Config` dict (d_hidden, d_expert,
 * n_experts, local_start, local_count, top_k; muse_moe_w4a16/py/00_moe_w4a16.py:82-90),
 * which the reference bakes into its CUDA source (moe.cu:144); here they are run-time.
 * Constraints: hidden % 256 == 0, inter % 256 == 0, 1 <= top_k <= 16,
 * 1 <= local_count <= 256, n_experts <= 512. */
typedef struct MskMoeCfg {
  int32_t hidden;        /* H: d_hidden */
  int32_t inter;         /* I: d_expert */
  int32_t n_experts;     /* E: experts over all ranks (range of topk_ids) */
  int32_t local_start;   /* first expert owned by this rank */
  int32_t local_count;   /* experts owned by this rank */
  int32_t top_k;
  int32_t routing_mode;  /* MSK_ROUTE_* */
  float route_scale;     /* sigmoid mode: logit multiplier (reference: 1/sqrt(32)) */
  float post_norm_eps;   /* eps of the post-expert RMS norm (reference: 1e-8) */
  int32_t num_ctas;      /* persistent grid size (at most 512); 0 = 148, one CTA per SM of a B200. The shares of the
                            weight stream, and so the order in which a cut unit's partial sums are added, follow
                            this number and the shapes, never the device */
  int32_t decode_path;   /* steps of few tokens (n_tokens <= 32, n_tokens * top_k <= 256, token tile <= 32):
                            0 = chosen by token count (one launch up to 8 tokens, the chain beyond),
                            1 = the chain of launches used for many tokens,
                            2 = row copy, gate/up kernel that routes and sorts, down kernel that combines,
                            3 = one launch (routing, sort, both GEMMs and the combine in one kernel);
                            any token count with a token tile <= 32 (0 picks it from 9 tokens on):
                            4 = sort launch(es), both GEMMs in one cooperative launch, combine */
  int32_t no_pdl;        /* non-zero: launches are not chained with programmatic dependent launch (the reference's
                            okc_set_pdl(0), muse_moe_w4a16/cuda/moe.cu:2348,2565) */
  int32_t token_tile;    /* MMA N (tokens per tile): 16/32/64/128; 0 = chosen from the mean rows per expert
                            (up to 12: 16, up to 32: 64, beyond: 128) */
  int32_t max_tokens;    /* token capacity the workspace is sized for (msk_moe_forward rejects more) */
  int32_t trace;         /* non-zero: the GEMM kernels stamp %globaltimer per CTA into the workspace (view 6) */
  int32_t stop_after;    /* measuring aid: 0 = whole step; 1/2/3 = return after sort / gate-up GEMM / down GEMM */
  int32_t flat_shares;   /* non-zero (with n_tokens * top_k <= 256 and paths 1, 2): the last rounds of the weight stream
                            are cut into equal shares per CTA instead of whole units (see msk_moe_share_pieces) */
} MskMoeCfg;

/* ---- prepare-time repack (lossless; replaces the four layouts built by
 *      muse_moe_w4a16/py/01_build_pack.py:95-238 and py/02_prepare.py:24-57) ---- */

/* Bytes of the two packed weight buffers for local_count experts. */
int msk_moe_packed_bytes(const MskMoeCfg* cfg, size_t* host_w13_bytes, size_t* host_w2_bytes);

/* w13: uint8 [local_count, 2I, H/2] (two E2M1 codes per byte, low nibble = even k; rows
 * [gate 0..I-1; up I..2I-1]); w13_sf: E4M3 bytes [local_count, 2I, H/16];
 * w2: uint8 [local_count, H, I/2]; w2_sf: [local_count, H, I/16].
 * Output: tiles of 128 rows x 256 K, each 16 KiB of bit-permuted codes followed by
 * 2 KiB of scale bytes, ordered [expert][row tile][gate|up][k stage] for w13 and
 * [expert][row tile][k stage] for w2. Bit and byte permutation only. */
int msk_moe_repack(const MskMoeCfg* cfg, const void* w13, const void* w13_sf, const void* w2, const void* w2_sf,
                   void* packed13, void* packed2, void* stream);

/* Exact inverse of msk_moe_repack (for the losslessness test and state export). */
int msk_moe_unpack(const MskMoeCfg* cfg, const void* packed13, const void* packed2, void* w13, void* w13_sf,
                   void* w2, void* w2_sf, void* stream);

/* Dequantise packed tiles to BF16 matrices carrying e2m1*e4m3 (no global scale):
 * dq13 [local_count, 2I, H], dq2 [local_count, H, I]. Runs the same device decode
 * routine as the GEMM kernel; test hook for muse_moe_w4a16/cuda/moe.cu:293-310. */
int msk_moe_dequant_packed(const MskMoeCfg* cfg, const void* packed13, const void* packed2, void* dq13, void* dq2,
                           void* stream);

/* ---- routing (caller side of the reference: muse_decode_layer/py/04_triton_kernels.py:525-556,
 *      muse_prefill_layer/cuda/prefill.cu:1620-1705) ---- */

/* logits[t, e] = sum_h float(x[t, h]) * router_w[e, h], FP32, fixed summation order
 * (precedent: muse_decode_layer/cuda/router_fp32.cu:4-40). x: bf16 [T, H]; router_w: fp32 [E, H]. */
int msk_moe_router_logits(const MskMoeCfg* cfg, const void* x, const float* router_w, float* logits, int n_tokens,
                          void* stream);

/* The same logits as a tensor-core GEMM (tcgen05, FP32 accumulation) for 16 tokens and more, with the
 * FP32 router weight held the way the reference's layers hold it: an exact-sum pair of BF16 matrices
 * hi = bf16(w), lo = bf16(w - hi), stacked [hi; lo] as bf16 [2E, H]
 * (muse_decode_layer/py/05_tune.py:279-286, muse_prefill_layer/py/00_layer.py:369-374). Products are
 * exact; every logit is accumulated in one fixed order, so repeated calls give the same bits. The
 * logits differ from the FP32 product by what w - hi - lo drops (about 2^-17 of a weight), so a
 * top-k taken from them can differ from the FP32 one where two scores are closer than that.
 * status_word (nullable): receives 1 when a bounded wait in the kernel gave up. */
int msk_moe_router_logits_hilo(const MskMoeCfg* cfg, const void* x, const void* router_hilo, float* logits,
                               int32_t* status_word, int n_tokens, void* stream);

/* Top-k of fp32 logits [T, E]; ties go to the lowest expert index. bias may be NULL
 * (softmax mode ignores it). Writes ids int32 [T, k] (global ids, descending score) and
 * weights fp32 [T, k]. */
int msk_moe_route(const MskMoeCfg* cfg, const float* logits, const float* bias, int32_t* topk_ids,
                  float* topk_weights, int n_tokens, void* stream);

/* Stable counting sort of the (token, slot) entries by local expert
 * (muse_moe_w4a16/cuda/moe.cu:315-433). Entries whose id is outside
 * [local_start, local_start + local_count) or negative are dropped.
 *   cnt  int32 [local_count]       tokens per local expert
 *   off  int32 [local_count + 1]   exclusive prefix of cnt; off[local_count] = routed entries
 *   perm int32 [T * k]             perm[q] = entry index t*k+slot, ordered by (expert, entry)
 *   inv  int32 [T * k]             inv[entry] = q, or -1 when the entry is not local */
int msk_moe_sort(const MskMoeCfg* cfg, const int32_t* topk_ids, int n_tokens, int32_t* cnt, int32_t* off,
                 int32_t* perm, int32_t* inv, void* stream);

/* ---- the routed-expert step (replaces okc_run, muse_moe_w4a16/cuda/moe.cu:2796-2881) ---- */

/* Scratch needed by msk_moe_forward for up to cfg->max_tokens tokens. The carving depends
 * on cfg->max_tokens only, so every call must pass the cfg the workspace was sized with. */
int msk_moe_workspace_bytes(const MskMoeCfg* cfg, size_t* host_bytes);

/* Zero the control words of a workspace (status word, sort tables, unit and token tickets, grid and
 * tile counters). Once after allocation, and again after a step whose status word came back
 * non-zero: a kernel that gave up leaves tickets and counters half-way, and the status word itself
 * is sticky. */
int msk_moe_workspace_init(const MskMoeCfg* cfg, void* workspace, size_t workspace_bytes, void* stream);

/* out[t, :] = bf16( sum_{slot, local} w[t,slot] * post(y[t,slot]) ),
 *   y = (bf16(silu(x W13g^T gs13) * (x W13u^T gs13))) W2^T gs2,
 *   post(y) = y                                  when post_norm_w == NULL
 *           = y(1+w) * rsqrt(mean((y(1+w))^2)+eps)  otherwise
 * (muse_moe_w4a16/cuda/moe.cu:440-478, 2604-2766). x: bf16 [T, H], values within the F16 range
 * (|x| <= 65504; the MMA operands are F16, larger magnitudes saturate there, magnitudes below 2^-24
 * vanish; the reference's layers hand over RMS-normed rows, far inside it); topk_ids int32 [T, k]
 * (global ids); topk_weights fp32 [T, k]; gs13/gs2 fp32 [local_count]; post_norm_w bf16 [H]
 * or NULL; out bf16 [T, H], fully overwritten (zeros for tokens without a local route).
 * Launches: sort, [row copy,] gate/up GEMM, down GEMM, combine; a single launch for a few tokens
 * (see MskMoeCfg.decode_path). No host sync; capturable in a CUDA graph. */
int msk_moe_forward(const MskMoeCfg* cfg, const void* packed13, const void* packed2, const float* gs13,
                    const float* gs2, const void* post_norm_w, const void* x, const int32_t* topk_ids,
                    const float* topk_weights, void* out, void* workspace, size_t workspace_bytes, int n_tokens,
                    void* stream);

/* msk_moe_forward with the routing inside: top-k of `logits` (fp32 [T, E]; `bias` as in
 * msk_moe_route) is written to topk_ids_out / topk_weights_out and used for the step. Up to 32
 * tokens routing and sort share one launch. This is the call the layer callers' route-then-experts
 * sequence maps to (muse_decode_layer/py/06_kernel_fn.py:115-149). */
int msk_moe_forward_logits(const MskMoeCfg* cfg, const void* packed13, const void* packed2, const float* gs13,
                           const float* gs2, const void* post_norm_w, const void* x, const float* logits,
                           const float* bias, int32_t* topk_ids_out, float* topk_weights_out, void* out,
                           void* workspace, size_t workspace_bytes, int n_tokens, void* stream);

/* The step with the pre-expert RMS norm of the layer callers fused in front: the expert input is
 * bf16(x * rsqrt(mean(x^2) + pre_norm_eps) * (1 + pre_norm_w)), pre_norm_w bf16 [hidden], applied
 * by the kernel that makes the F16 copy of the token rows (the reference's routing kernels do it
 * before they store the expert input: muse_decode_layer/py/04_triton_kernels.py:556-568, eps 1e-5;
 * muse_prefill_layer's gather takes g_pre_expert_norm, py/04_moe_forward.py:35). Routing is not
 * affected: with `logits` (non-NULL) the routing runs here and topk_ids / topk_weights receive it;
 * with logits == NULL they are inputs. hidden <= 8192. Not available with token_tile = 8. */
int msk_moe_forward_prenorm(const MskMoeCfg* cfg, const void* packed13, const void* packed2, const float* gs13,
                            const float* gs2, const void* post_norm_w, const void* pre_norm_w, float pre_norm_eps,
                            const void* x, const float* logits, const float* bias, int32_t* topk_ids,
                            float* topk_weights, void* out, void* workspace, size_t workspace_bytes, int n_tokens,
                            void* stream);

/* msk_moe_forward with a CUDA event before and after each of its launches. Waits for the last one
 * and returns the elapsed milliseconds host_ms[5] = routing + sort, row copy, gate/up GEMM, down
 * GEMM, combine (a stage that a path does not launch reads 0; the one-launch path reports the whole
 * step under gate/up). A measuring entry point: it synchronises and creates its events on first use; the
 * counterpart of the reference's in-kernel %globaltimer trace (muse_moe_w4a16/cuda/moe.cu:279-284). */
int msk_moe_forward_timed(const MskMoeCfg* cfg, const void* packed13, const void* packed2, const float* gs13,
                          const float* gs2, const void* post_norm_w, const void* x, const int32_t* topk_ids,
                          const float* topk_weights, void* out, void* workspace, size_t workspace_bytes,
                          int n_tokens, void* stream, float* host_ms);

/* msk_moe_forward for callers that cannot allocate device memory on the calling path (all
 * memory handed to their own pool, allocator locked, a latency-critical thread that must not
 * enter the driver's allocator): the scratch lives in an 8 MiB file-scope device array inside the library, which every
 * GPU that loads the library holds until the process exits. No counterpart in the reference,
 * whose scratch is always allocated by prepare(). Limits: n_tokens * top_k <= 128,
 * hidden <= 8192, inter <= 4096, else MSK_ERR_TOO_LARGE. The first call on a device resolves
 * the array's address (make it outside stream capture). Every call shares the array, which
 * keeps the last call's contents; the status word is cleared at the start of each call; calls
 * that overlap on the GPU race on it. Calls no cudaMalloc/cudaFree or allocating routine. */
int msk_moe_forward_static(const MskMoeCfg* cfg, const void* packed13, const void* packed2, const float* gs13,
                           const float* gs2, const void* post_norm_w, const void* x, const int32_t* topk_ids,
                           const float* topk_weights, void* out, int n_tokens, void* stream);

/* Status word of msk_moe_forward_static's array on the current device, copied to *host_status after
 * synchronising `stream`: 0 = no device-side wait of the last static call gave up. The caller of
 * the static entry point holds no workspace pointer, so msk_moe_read_status cannot serve it.
 * Allocates nothing; not for the timed path. No counterpart in the reference. */
int msk_moe_static_status(int* host_status, void* stream);

/* The launch plan msk_moe_forward uses for n_tokens: host_out[4] = token tile N, path (as
 * MskMoeCfg.decode_path; 1 or 4 beyond a few tokens), 1 when the weight stream is cut into equal
 * shares (else whole units), persistent grid size. The reference picks its build by
 * token count the same way (muse_moe_w4a16/py/03_kernel_fn.py:33-40). */
int msk_moe_plan(const MskMoeCfg* cfg, int n_tokens, int* host_out);

/* How the GEMM kernels deal their work (host-side twin of the device code, a test hook): the pieces
 * that CTA `cta` of `shares` gets from n_base base units of n_stages K stages each. flat == 0: whole
 * units, round-robin; flat != 0: equal shares of the flat (unit, stage) list. host_out receives six
 * ints per piece: base unit, first stage, end stage, slot of the partial buffer (-1 for a whole
 * unit), first and last CTA that can hold a piece of the unit. heavy / skip (whole units only): the
 * first `heavy` CTAs are left out of the first `skip` rounds, which is how the one-launch kernel deals
 * its down-GEMM units when those CTAs hold one more gate/up unit. The reference's counterpart is its
 * cost-weighted range scheduler (muse_moe_w4a16/cuda/moe.cu:2245-2289). */
int msk_moe_share_pieces(int n_base, int n_stages, int shares, int flat, int cta, int heavy, int skip, int* host_out,
                         int capacity, int* host_count);

/* Views into the workspace after msk_moe_forward (device pointers, for parity tests):
 * which: 0 cnt, 1 off, 2 perm, 3 inv, 4 inter (fp16 [R, I], holding bf16-rounded values), 5 y (fp32 [R, H]; bf16 [R, H] when the plan's
 * token tile is 128),
 * 7 unit tickets, 8 control words of the few-token paths, 9 per-CTA counts of the multi-CTA sort, 10 the
 * per-tile counters that hand `inter` from the gate/up launch to the down launch tile by tile (all four
 * zeroed by msk_moe_workspace_init, like everything below view 4),
 * 6 trace (uint64 [2 launches][256 CTAs x 16 stamps, then 6 x 128 event words], ns; written when cfg->trace != 0). */
int msk_moe_workspace_view(const MskMoeCfg* cfg, void* workspace, int which, void** host_ptr);

/* Copies workspace word 0 to *host_status after synchronising `stream`. 0 = no device-side
 * wait gave up. Not for the timed path. */
int msk_moe_read_status(const void* workspace, int* host_status, void* stream);

/* Registers / static + dynamic shared memory / local memory per kernel, as the reference's
 * okc_attrs() reports (muse_moe_w4a16/cuda/moe.cu:2789-2794). which: 0 sort, 1 route,
 * 2 gate/up GEMM, 3 down GEMM, 4 combine. host_out: int[4] = regs, static smem, max dyn smem, local. */
int msk_moe_attrs(int which, int token_tile, int* host_out);

/* Expert-parallel combine at a token's home rank: out[t] = bf16(sum over ranks d, in rank order, of
 * the partial row rank d returned for token t), FP32 accumulation; rank d contributes only when one
 * of the token's ids lies in [d*experts_per_rank, (d+1)*experts_per_rank). back: bf16 [n_ranks,
 * n_tokens, hidden] in rank order; self_rows (may be NULL): the home rank's own partial rows,
 * read instead of back[self_rank]; ids: int32 [n_tokens, top_k] (global ids). n_ranks <= 64.
 * No counterpart in the reference, which stops at per-rank partial sums and leaves the exchange
 * to its caller (muse_moe_w4a16/cuda/moe.cu:347-350, 2604). */
int msk_ep_combine(const void* back, const void* self_rows, int self_rank, const int32_t* ids, int top_k,
                   int experts_per_rank, void* out, int n_ranks, int n_tokens, int hidden, void* stream);

/* Cross-rank flags of the expert-parallel step, as stream memory operations (no kernel, no SM):
 * write `value` to a 32-bit word (this GPU's or a peer-mapped one) once all earlier work of the
 * stream is done and visible; make the stream wait until a word of this GPU is >= value. The wait
 * is unbounded by design of the driver call: callers pair every wait with a write that a live
 * peer is certain to issue, and run under a host-side time-out. No counterpart in the reference. */
int msk_ep_flag_write(void* addr, uint32_t value, void* stream);
int msk_ep_flag_wait(void* addr, uint32_t value, void* stream);

/* Cold-cache timing aid: reads `bytes` of `buf` (more than the L2 capacity) with ordinary loads so that
 * L2 ends up holding clean lines of the buffer and nothing of the step to be timed; the reference's
 * read sweep (muse_decode_layer/py/05_tune.py:74-94, muse_moe_w4a16/py/04_diag.py:24-49). */
int msk_l2_sweep(const void* buf, size_t bytes, uint32_t* sink, void* stream);

/* Hash of the source files this library was built from (set by the build script); the Python
 * binding compares it with the sources beside it and refuses a stale binary. */
const char* msk_build_id(void);

/* HBM streaming probe: every CTA pulls its share of `bytes` from `src` through a ring of
 * bulk async copies, as the GEMM kernel's weight producer does, and adds a checksum to
 * sink[0] (twin of muse_moe_w4a16/cuda/moe_bw.cu). sink is two words; sink[1] receives the device
 * status (0, or 1 when a bounded wait gave up), like word 0 of a workspace. skip_release > 0 is a
 * test hook for that path: every CTA withholds the release of its chunk number skip_release, so
 * the producer's wait for the slot runs into its limit (MSK_WAIT_LIMIT_NS, one second), the kernel
 * unwinds and returns with sink[1] = 1. Nothing traps or spins for ever; the context stays usable
 * (the reference's counterpart is its SK2_DELAY_ESC knob, muse_decode_layer/py/01_moe.py:340). */
int msk_bw_probe(const void* src, size_t bytes, int stages, int stage_bytes, int num_ctas, uint32_t* sink,
                 int skip_release, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MSK_MOE_H_ */
